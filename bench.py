#!/usr/bin/env python
"""Benchmark of the packed W4A4 projection sweep (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload ("w4a4_projection_sweep"): the four Llama-3.2-1B projection shapes
(N x K: 2048x2048, 512x2048, 8192x2048, 2048x8192), weights N(0, 0.02^2)
Hadamard-rotated and NQRT4-encoded with the stateless dither, activations
seeded BF16 N(0,1) Hadamard-rotated with M in {1,8,16,64,128,512,2048,8192}
rows.  One step = on-the-fly A4 encode + packed projection for all 32 cells.
`value` is 2*M*N*K summed over the cells divided by the device time of a step,
inputs already resident in HBM; `e2e` is the same sweep through the
FusedNQRTLinear plugin call with pinned host inputs and outputs (copies timed).
With N > 1 GPUs (torchrun) every rank runs the same sweep on its own GPU: the
projections are independent, so there is no data-path collective.

`--impl reference` times the reference's own PyTorch-CPU path (installed
unmodified under oracle/_ref; the C restatement if it is not there) with all
host threads on a bounded sample of every cell of the same sweep.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPES = (("q_o", 2048, 2048), ("k_v", 512, 2048), ("gate_up", 8192, 2048), ("down", 2048, 8192))
TOKENS = (1, 8, 16, 64, 128, 512, 2048, 8192)
ACT_BETAS = tuple(v / 14 for v in (3.47, 4.74, 6.90, 18.11))
W_BETAS = tuple(v / 14 for v in (4.0, 5.5, 7.0, 18.0))
ENCODE_TRAFFIC_8192X8192 = 134_373_376 + 123_120_896  # dram__bytes_read.sum + dram__bytes_write.sum (ncu)
METRIC = "w4a4_e8_gemm_sweep_tflops"
UNIT = "TFLOP/s"


def sweep_flops() -> float:
    return float(sum(2 * m * n * k for _, n, k in SHAPES for m in TOKENS))


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]),
                "bf16_tflops_sustained": float(data.get("bf16_tflops_sustained", data["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.lines: list[str] = []
        self.proc = None
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self) -> None:
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- CPU arms
# Both CPU arms time every one of the sweep's 32 cells on a bounded sample and compose the time of the whole
# sweep from it: the A4 encode and the dequantisation of its output cost the same per row, so they are
# timed on the first CPU_ENCODE_ROWS rows of the cell and scaled to its M rows; the weight dequantisation is
# timed on CPU_WEIGHT_ROWS rows and scaled to N; the float32 product runs at the cell's full size.
CPU_ENCODE_ROWS = 32
CPU_WEIGHT_ROWS = 256


def sweep_config(world: int) -> dict:
    """The workload description both arms print (identical objects, so the two lines can be compared)."""
    return {"workload": "w4a4_projection_sweep", "shapes": [list(s) for s in SHAPES], "tokens": list(TOKENS),
            "q": 14, "betas": 4, "encode": "on the fly every call", "parallelism": f"replicas{world}",
            "l2": "one step touches > 1 GB of distinct operands, so inputs of a cell are evicted from the "
                  "126 MB L2 before the cell repeats"}


def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except (AttributeError, OSError):
        return max(1, os.cpu_count() or 1)


def _compose(per_shape_weight_s, per_cell_rows_s, per_cell_product_s) -> float:
    """Seconds of the whole sweep from the sampled pieces (see the note above)."""
    total = 0.0
    for si, (_, n, k) in enumerate(SHAPES):
        for m in TOKENS:
            total += per_shape_weight_s[si] * (n / min(n, CPU_WEIGHT_ROWS))
            total += per_cell_rows_s[(si, m)] * (m / min(m, CPU_ENCODE_ROWS))
            total += per_cell_product_s[(si, m)]
    return total


class ReferenceCpuArm:
    """The reference's own PyTorch-CPU path (nestquant.core, installed unmodified under oracle/_ref).

    quantize_rows (core/quantizer.py:214) + pack_nestquant_indices (core/packing.py:137) of the activation,
    QuantizedRows.dequantize (core/quantizer.py:39) of both operands, float32 product -- config 0's pipeline
    on config 1's shapes.  The weight is encoded once outside the timed region (it is offline work).
    """

    kind = "reference"

    def __init__(self, threads: int) -> None:
        from oracle.build_ref import build as build_ref, ref_path

        location = ref_path() or build_ref()
        if location is None:
            raise RuntimeError("oracle/_ref holds no installed reference and no reference source is present")
        if str(location) not in sys.path:
            sys.path.insert(0, str(location))
        import torch
        from nestquant.core.codec import generate_e8_dither_stateless
        from nestquant.core.packing import pack_nestquant_indices
        from nestquant.core.quantizer import quantize_rows
        from nestquant.core.rotation import hadamard

        torch.set_num_threads(threads)
        self.torch, self.threads = torch, torch.get_num_threads()
        self.quantize_rows, self.pack = quantize_rows, pack_nestquant_indices
        gen = torch.Generator().manual_seed(1000)
        self.weights, self.inputs, self.full = [], {}, {}
        for i, (_, n, k) in enumerate(SHAPES):
            rows = min(n, CPU_WEIGHT_ROWS)
            w = hadamard(0.02 * torch.randn(rows, k, generator=gen))
            dither = generate_e8_dither_stateless(rows * k // 8, seed=20261029 + i).reshape(rows, k // 8, 8)
            self.weights.append(quantize_rows(w, 14, W_BETAS, dither=dither))
            self.full[("w", i)] = torch.randn(n, k, generator=gen)
        for k in sorted({k for _, _, k in SHAPES}):
            for m in TOKENS:
                x = torch.randn(m, k, generator=torch.Generator().manual_seed(2000 + m)).bfloat16()
                self.inputs[(k, m)] = hadamard(x)[:min(m, CPU_ENCODE_ROWS)].float().contiguous()
                self.full[("a", k, m)] = torch.randn(m, k, generator=gen)

    def sample_step(self):
        torch, clock = self.torch, time.perf_counter
        weight_s, rows_s, product_s = {}, {}, {}
        with torch.no_grad():
            for si, (_, n, k) in enumerate(SHAPES):
                t0 = clock()
                self.weights[si].dequantize()
                weight_s[si] = clock() - t0
                for m in TOKENS:
                    t0 = clock()
                    qa = self.quantize_rows(self.inputs[(k, m)], 14, ACT_BETAS)
                    self.pack(qa.codes, qa.beta_indices, q=qa.q, beta_count=len(qa.betas))
                    qa.dequantize()
                    rows_s[(si, m)] = clock() - t0
                    t0 = clock()
                    torch.matmul(self.full[("a", k, m)], self.full[("w", si)].T)
                    product_s[(si, m)] = clock() - t0
        return weight_s, rows_s, product_s

    def describe(self) -> str:
        return ("all 32 cells; nestquant.core quantize_rows + pack_nestquant_indices + dequantize of the activation on "
                f"the first {CPU_ENCODE_ROWS} rows of each cell (scaled to M), QuantizedRows.dequantize of {CPU_WEIGHT_ROWS} "
                "weight rows with the dither held in memory (scaled to N), torch float32 product at full size")


class PortCpuArm:
    """The C restatement of the same pipeline (oracle/nq_oracle.c, OpenMP), sampled the same way."""

    kind = "port"

    def __init__(self, threads: int) -> None:
        import numpy as np

        from oracle import nq_oracle as oracle

        oracle.build()
        oracle.set_threads(threads)
        self.oracle, self.np, self.threads = oracle, np, oracle.thread_count()
        rng = np.random.default_rng(1000)
        self.weights, self.inputs, self.full = [], {}, {}
        for i, (_, n, k) in enumerate(SHAPES):
            rows = min(n, CPU_WEIGHT_ROWS)
            w = oracle.hadamard((0.02 * rng.standard_normal((rows, k))).astype(np.float32))
            seed = 20261029 + i
            self.weights.append((*oracle.encode_packed(w, W_BETAS, seed=seed), seed, rows))
            self.full[("w", i)] = rng.standard_normal((n, k)).astype(np.float32)
        for k in sorted({k for _, _, k in SHAPES}):
            for m in TOKENS:
                rows = min(m, CPU_ENCODE_ROWS)
                x = oracle.round_bf16(rng.standard_normal((rows, k)).astype(np.float32))
                self.inputs[(k, m)] = oracle.hadamard(x, round_bf16=True)
                self.full[("a", k, m)] = rng.standard_normal((m, k)).astype(np.float32)

    def sample_step(self):
        oracle, clock = self.oracle, time.perf_counter
        weight_s, rows_s, product_s = {}, {}, {}
        for si, (_, n, k) in enumerate(SHAPES):
            wc, wb, wn, seed, rows = self.weights[si]
            t0 = clock()
            oracle.dequantize_rows(wc, wb, wn, W_BETAS, rows, k, seed=seed)
            weight_s[si] = clock() - t0
            for m in TOKENS:
                x = self.inputs[(k, m)]
                t0 = clock()
                ac, ab, an = oracle.encode_packed(x, ACT_BETAS)
                oracle.dequantize_rows(ac, ab, an, ACT_BETAS, x.shape[0], k)
                rows_s[(si, m)] = clock() - t0
                t0 = clock()
                self.np.matmul(self.full[("a", k, m)], self.full[("w", si)].T)  # the host's BLAS, as torch uses one
                product_s[(si, m)] = clock() - t0
        return weight_s, rows_s, product_s

    def describe(self) -> str:
        return ("all 32 cells; C restatement: encode + pack + dequantise of the activation on the first "
                f"{CPU_ENCODE_ROWS} rows of each cell (scaled to M), dequantise of {CPU_WEIGHT_ROWS} weight rows with the "
                "dither regenerated (scaled to N), float32 product at full size through numpy's BLAS")


def cpu_arm(prefer_reference: bool = True):
    """The reference's own CPU path when it is installed under oracle/_ref, else the C restatement."""
    threads = host_threads()
    os.environ["OMP_NUM_THREADS"] = str(threads)  # a launcher may have exported 1 for its children
    os.environ["MKL_NUM_THREADS"] = str(threads)
    if prefer_reference:
        try:
            return ReferenceCpuArm(threads)
        except Exception as error:  # not installed on this machine: fall back to the restatement, and say so
            print(f"bench: reference CPU path unavailable ({type(error).__name__}: {error}); timing the C restatement",
                  file=sys.stderr)
    return PortCpuArm(threads)


def cpu_baseline(arm, repeats: int = 1, warmup: int = 0) -> dict:
    for _ in range(warmup):
        arm.sample_step()
    sample_seconds, composed = [], []
    for _ in range(repeats):
        start = time.perf_counter()
        pieces = arm.sample_step()
        sample_seconds.append(time.perf_counter() - start)
        composed.append(_compose(*pieces))
    composed.sort()
    sweep_seconds = composed[len(composed) // 2]
    return {"value": sweep_flops() / sweep_seconds / 1e12, "unit": UNIT, "cores": arm.threads, "kind": arm.kind,
            "sample": f"{arm.describe()}; {sum(sample_seconds) / len(sample_seconds):.2f} s of CPU work per step, "
                      f"{sweep_seconds:.1f} s for the whole sweep when composed",
            "seconds_per_sample_step": sum(sample_seconds) / len(sample_seconds),
            "sweep_seconds_composed": sweep_seconds}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    arm = cpu_arm()
    base = cpu_baseline(arm, repeats=max(1, args.steps), warmup=args.warmup)
    seconds = base.pop("seconds_per_sample_step")
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": sweep_config(world),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "ms_per_step is the wall time of one bounded sample step; value is the sweep's flops over the time "
                "of the whole sweep composed from the sampled pieces",
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def gpu_setup(torch, rt, device):
    from nestquant_aiinfra_b200.rotation import hadamard

    gen = torch.Generator(device="cpu").manual_seed(1000)
    weights, inputs = [], {}
    for i, (name, n, k) in enumerate(SHAPES):
        w = hadamard((0.02 * torch.randn(n, k, generator=gen)).to(device))
        weights.append(rt.quantize_weight_cuda(w, betas=W_BETAS, dither_seed=20261029 + i, tensor_name=name))
        del w
    for k in sorted({k for _, _, k in SHAPES}):
        for m in TOKENS:
            x = torch.randn(m, k, generator=torch.Generator().manual_seed(2000 + m)).bfloat16().to(device)
            inputs[(k, m)] = hadamard(x)
    beta_table = torch.tensor(ACT_BETAS, dtype=torch.float32, device=device)
    torch.cuda.synchronize(device)
    return weights, inputs, beta_table


def run_gpu(args) -> None:
    import torch

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist

        # NCCL's banner / debug lines must not land on stdout next to the JSON line
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")  # plain peer paths: the all-reduces are ~2 % of a TP step
        dist.init_process_group("nccl", device_id=device)
    import nestquant_aiinfra_b200.runtime as rt
    from nestquant_aiinfra_b200.fused_linear import FusedNQRTLinear

    weights, inputs, beta_table = gpu_setup(torch, rt, device)
    cells = [(si, m) for si in range(len(SHAPES)) for m in TOKENS]
    stream = torch.cuda.current_stream(device)

    def run_cell(si: int, m: int):
        x = inputs[(SHAPES[si][2], m)]
        act = rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS, beta_table=beta_table, keep_decoded=True)
        return rt.linear_packed_w4a4(act, weights[si])

    def step_one_stream() -> None:
        for si, m in cells:
            run_cell(si, m)

    # The 32 cells are independent calls.  A step issues them on `--streams` streams that fork from the timing
    # stream and join it again (parallel branches of the captured graph): most launches of the small cells and the
    # tails of the large ones leave SMs idle that another cell's kernels can use.  Cells are dealt longest first
    # to the least loaded stream, from one measurement of every cell alone during the warm-up.
    lanes: list[list[tuple[int, int]]] = [list(cells)]
    side_streams = [torch.cuda.Stream(device) for _ in range(max(args.streams, 1))]

    def step() -> None:
        if len(lanes) == 1:
            step_one_stream()
            return
        origin = torch.cuda.current_stream(device)  # the timing stream, or the capturing one
        fork = torch.cuda.Event()
        fork.record(origin)
        results = []  # outputs stay allocated until every stream has joined
        for lane, todo in zip(side_streams, lanes):
            lane.wait_event(fork)
            with torch.cuda.stream(lane):
                for si, m in todo:
                    results.append(run_cell(si, m))
                done = torch.cuda.Event()
                done.record(lane)
            origin.wait_event(done)

    def barrier() -> None:
        if distributed:
            dist.barrier()
        torch.cuda.synchronize(device)

    sampler = ClockSampler(local_rank)  # samples from the warm-up on, so the timed region is always covered
    sampler.start()
    step()  # loads the kernels
    if args.streams > 1:
        alone = {}
        for si, m in cells:
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record(stream)
            run_cell(si, m)
            t1.record(stream)
            torch.cuda.synchronize(device)
            alone[(si, m)] = t0.elapsed_time(t1)
        lanes = [[] for _ in range(args.streams)]
        load = [0.0] * args.streams
        for cell in sorted(cells, key=lambda c: -alone[c]):
            lightest = load.index(min(load))
            lanes[lightest].append(cell)
            load[lightest] += alone[cell]
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    # One sweep step is 112 launches, most of them a few microseconds long: issued call by call the host is the
    # slower side on the small cells (and more so with eight ranks sharing one host), so the step is captured
    # once as a CUDA graph and the timed region replays it, as the decode engine does with its step.
    graph, per_step = None, None
    try:
        counted = rt.launch_count()
        captured = torch.cuda.CUDAGraph()
        with torch.cuda.graph(captured):
            step()
        per_step = rt.launch_count() - counted
        captured.replay()
        torch.cuda.synchronize(device)
        graph = captured
    except Exception as error:  # keep measuring call by call if the capture is refused
        print(f"bench: sweep step not captured ({type(error).__name__}: {error}); timing eager calls", file=sys.stderr)
        torch.cuda.synchronize(device)
    launches0 = rt.launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record(stream)
    for _ in range(args.steps):
        if graph is not None:
            graph.replay()
        else:
            step()
    stop.record(stream)
    barrier()
    launches = per_step * args.steps if graph is not None else rt.launch_count() - launches0
    # The encoder's own time inside a step: the 32 encode launches of one step alone, as a CUDA graph on the same
    # stream (events around three replays; each replay re-reads 0.4 GB of inputs, more than the L2 holds).
    def encodes_only() -> None:
        for si, m in cells:
            x = inputs[(SHAPES[si][2], m)]
            rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS, beta_table=beta_table, keep_decoded=True)

    enc_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(enc_graph):
        encodes_only()
    enc_graph.replay()
    torch.cuda.synchronize(device)
    enc0, enc1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    enc0.record(stream)
    for _ in range(3):
        enc_graph.replay()
    enc1.record(stream)
    torch.cuda.synchronize(device)
    # the same step with the cells one after the other on one stream, for reference
    serial_ms = None
    if len(lanes) > 1:
        serial_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(serial_graph):
            step_one_stream()
        serial_graph.replay()
        torch.cuda.synchronize(device)
        ser0, ser1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ser0.record(stream)
        for _ in range(3):
            serial_graph.replay()
        ser1.record(stream)
        torch.cuda.synchronize(device)
        serial_ms = ser0.elapsed_time(ser1) / 3
    clocks = sampler.stop()
    enc_ms_per_step = enc0.elapsed_time(enc1) / 3
    elapsed_ms = start.elapsed_time(stop)
    if rt.read_status(device) != 0:
        raise SystemExit("device status word is non-zero: a bounded wait in the GEMM gave up")
    if distributed:
        t = torch.tensor([elapsed_ms, serial_ms or 0.0], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t[0].item())
        serial_ms = float(t[1].item()) or None
    ms_per_step = elapsed_ms / args.steps
    value = world * sweep_flops() / (ms_per_step * 1e-3) / 1e12

    # dominant kernel (by device time): the A4 encoder, HBM-bound by bytes
    pk = peaks()
    enc_bytes = sum(m * SHAPES[si][2] * 2 + m * (17 * SHAPES[si][2] // 32 + 4) for si, m in cells)
    enc_gbs = enc_bytes / (enc_ms_per_step * 1e-3) / 1e9
    roofline = {"kernel": "nq_encode_rows_kernel", "bound": "hbm", "achieved": enc_gbs, "peak": pk["hbm_gbs"],
                "unit": "GB/s", "frac": enc_gbs / pk["hbm_gbs"], "peak_source": pk["source"],
                # share of the device work of a step: against the step with its cells one after the other
                "share_of_step": enc_ms_per_step / (serial_ms or ms_per_step), "launches": len(cells),
                "us_per_step": round(enc_ms_per_step * 1e3, 1),
                # DRAM bytes of the largest encode launch (8192 x 8192 BF16) from the ncu capture summarised in
                # profiles/nq_encode_rows_kernel_8192x8192_bf16.md; its algorithmic bytes are 2MK + M(17K/32+4),
                # the rest is the optional BF16 reconstruction the projection consumes.
                "traffic": ENCODE_TRAFFIC_8192X8192, "traffic_launch": "M=8192 K=8192",
                "algorithmic_bytes_of_that_launch": 8192 * 8192 * 2 + 8192 * (17 * 8192 // 32 + 4)}

    # per-cell table and the tensor-bound kernel alone (outside the timed region)
    table, gemm = ([], None) if args.skip_extras else cell_table(torch, rt, weights, inputs, beta_table, device, pk)

    e2e = ({"ms": None, "h2d": 0, "d2h": 0} if args.skip_extras else
           run_e2e(torch, rt, FusedNQRTLinear, weights, device, max(3, min(args.steps, 10)), distributed))
    if distributed and e2e["ms"] is not None:
        t = torch.tensor([e2e["ms"]], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e["ms"] = float(t.item())
    e2e_value = None if e2e["ms"] is None else world * sweep_flops() / (e2e["ms"] * 1e-3) / 1e12

    extras = {}
    if not args.skip_extras:
        try:
            if rank == 0:
                extras["kv"] = kv_workload(torch, rt, device, pk)
        except Exception as error:  # keep the headline line even if an extra workload fails
            extras["kv"] = {"error": f"{type(error).__name__}: {error}"[:300]}
        torch.cuda.empty_cache()
        try:
            dec = decode_workload(torch, device)
            if distributed:  # independent replicas: total tokens over the slowest rank's time
                t = torch.tensor([dec["ms_per_step"]], device=device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                dec["ms_per_step"] = round(float(t.item()), 3)
                dec["decode_tok_s"] = round(world * dec["requests"] / (dec["ms_per_step"] * 1e-3), 1)
                dec["replicas"] = world
                cont = dec.get("continuous_batch", {})
                if "decode_tok_s" in cont:  # replicas: every rank runs the same request stream; N x the slowest rank
                    t = torch.tensor([cont["decode_tok_s"], cont["tok_s_including_prefill"]], device=device)
                    dist.all_reduce(t, op=dist.ReduceOp.MIN)
                    cont["decode_tok_s"] = round(world * float(t[0].item()), 1)
                    cont["tok_s_including_prefill"] = round(world * float(t[1].item()), 1)
                    cont["replicas"] = world
                resident = dec.get("resident_decoded_weights", {})
                for leg in (resident, resident.get("with_kv_lattice_shadow", {})):  # the opt-in legs the same way
                    if "ms_per_step" in leg:
                        t = torch.tensor([leg["ms_per_step"]], device=device)
                        dist.all_reduce(t, op=dist.ReduceOp.MAX)
                        leg["ms_per_step"] = round(float(t.item()), 3)
                        leg["decode_tok_s"] = round(world * dec["requests"] / (leg["ms_per_step"] * 1e-3), 1)
            extras["decode"] = dec
        except Exception as error:
            extras["decode"] = {"error": f"{type(error).__name__}: {error}"[:300]}
        torch.cuda.empty_cache()
        if distributed:
            # config 4: the tensor-parallel decode step over these ranks (the only workload here with a collective)
            try:
                extras["tp"] = tp_decode(torch, dist, device, rank, world, layers=args.tp_layers, batch=args.tp_batch,
                                         context=args.tp_context, steps=3, warmup=3, collective=args.tp_collective,
                                         decode_ahead=args.tp_decode_ahead == "on")
            except Exception as error:
                extras["tp"] = {"error": f"{type(error).__name__}: {error}"[:300]}
            torch.cuda.empty_cache()
    if rank == 0:
        base = port = None
        if world == 1 and not args.skip_extras:
            arm = cpu_arm()
            base = cpu_baseline(arm, repeats=2, warmup=1)
            if arm.kind == "reference":  # the C restatement beside it, as a second figure
                port = cpu_baseline(PortCpuArm(host_threads()), repeats=2, warmup=1)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": sweep_config(world),
            "launch": (("CUDA graph of one step, replayed" if graph is not None else "call by call")
                       + (f"; the 32 cells on {len(lanes)} streams, dealt longest first" if len(lanes) > 1 else "")),
            "one_stream": None if serial_ms is None else {
                "ms_per_step": serial_ms, "value": world * sweep_flops() / (serial_ms * 1e-3) / 1e12,
                "note": "the same step with its 32 cells one after the other on one stream (CUDA graph, 3 replays)"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                    "ms_per_step": e2e["ms"], "launch": e2e.get("launch"), "cell_order": e2e.get("cell_order"),
                    "numa": e2e.get("numa"),
                    "result_on_host": e2e.get("nonzero_result")},
            "gpu_launches": int(launches),
            "roofline": roofline,
            "roofline_gemm": gemm,
            "cpu_baseline": base,
            "cpu_baseline_port": port,
            "cells": table,
        }
        line.update(extras)
        print(json.dumps(line), flush=True)
    if distributed:
        _teardown(torch, dist, device)


def _time_graph(torch, fn, device, reps: int = 5) -> float:
    """Average device time of fn() in microseconds (CUDA-graph replay of `reps` calls).

    The events bracket one graph launch, whose fixed cost (~10-20 us) is shared by the calls inside: short
    calls are therefore timed again in a graph of 48, so that this share drops below half a microsecond.
    """
    def timed(count: int) -> float:
        side = torch.cuda.Stream(device)
        with torch.cuda.stream(side):
            fn()
            torch.cuda.synchronize(device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(count):
                    fn()
            graph.replay()
            torch.cuda.synchronize(device)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            graph.replay()
            e1.record(side)
            torch.cuda.synchronize(device)
        return e0.elapsed_time(e1) * 1e3 / count

    t = timed(reps)
    if t < 100.0 and reps < 48:
        t = timed(48)
    return t


def cell_table(torch, rt, weights, inputs, beta_table, device, pk):
    """Per-cell device times: encode, projection (decode + GEMM), GB/s of packed weights, TFLOP/s."""
    table, best = [], None
    for si, (name, n, k) in enumerate(SHAPES):
        w = weights[si]
        w_dec = rt.decode_packed_weight(w)
        w_bytes = n * k * 17 // 32 + 4 * n + 32
        for m in TOKENS:
            x = inputs[(k, m)]
            act = rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS, beta_table=beta_table, keep_decoded=True)
            t_enc = _time_graph(torch, lambda: rt.quantize_activation_cuda(x, q=14, betas=ACT_BETAS, beta_table=beta_table,
                                                                           keep_decoded=True), device)
            t_proj = _time_graph(torch, lambda: rt.linear_packed_w4a4(act, w), device)
            row = {"shape": name, "M": m, "encode_us": round(t_enc, 2), "proj_us": round(t_proj, 2),
                   "w_gbs": round((w_bytes + m * k * 2 + m * n * 2) / t_proj / 1e3, 1),
                   "tflops": round(2 * m * n * k / t_proj / 1e6, 2)}
            if m >= 8:  # the same projection as ONE launch that decodes the weight beside its own MMAs (not the default)
                from nestquant_aiinfra_b200.runtime import w4a4 as _w4a4

                t_fused = _time_graph(torch, lambda: _w4a4._run(act, w, torch.bfloat16, fused=True), device)
                row["fused_kernel_us"] = round(t_fused, 2)
            if m <= 128:
                w_res = rt.keep_decoded_weight(w) if m == TOKENS[0] else w_res
                t_res = _time_graph(torch, lambda: rt.linear_packed_w4a4(act, w_res), device)
                row["resident_us"] = round(t_res, 2)
                row["resident_bf16_gbs"] = round((n * k * 2 + m * k * 2 + m * n * 2) / t_res / 1e3, 1)
            if m >= 512:
                t_mma = _time_graph(torch, lambda: rt.gemm_bf16_tc(act.decoded, w_dec), device)
                row["mma_us"] = round(t_mma, 2)
                row["mma_tflops"] = round(2 * m * n * k / t_mma / 1e6, 1)
                if best is None or row["mma_tflops"] > best["achieved"]:
                    best = {"kernel": "nq_w4a4_tc_gemm_kernel", "bound": "tensor", "achieved": row["mma_tflops"],
                            "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": row["mma_tflops"] / pk["bf16_tflops"],
                            "cell": f"{name} M={m}", "peak_source": pk["source"]}
            table.append(row)
        del w_dec, w_res
    return table, best


def bind_to_gpu_numa_node(torch, device) -> dict:
    """Best effort: run this process (and first-touch its pinned buffers) on the CPUs of the GPU's NUMA node.

    Eight ranks on one host otherwise all sit on node 0 and push their copies through one memory controller.
    Only this process's CPU affinity changes; nothing on the GPU or the host outlives the process.
    """
    info: dict = {"bound": False}
    try:
        props = torch.cuda.get_device_properties(device)
        bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        node = int(Path(f"/sys/bus/pci/devices/{bdf}/numa_node").read_text().strip())
        info.update({"pci": bdf, "node": node})
        if node < 0:
            return info
        cpus: set[int] = set()
        for part in Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & set(os.sched_getaffinity(0))
        if allowed:
            os.sched_setaffinity(0, allowed)
            info.update({"bound": True, "cpus": len(allowed)})
    except Exception as error:  # no sysfs entry, no permission, old torch: leave the affinity as it is
        info["note"] = f"{type(error).__name__}: {error}"[:120]
    return info


def e2e_cell_order(torch, layers, device) -> list[tuple[int, int]]:
    """Order of the 32 cells inside one end-to-end step.

    A step is a three-stage flow shop -- copy in, module call, copy out, each stage serial on its own stream -- and
    the copy in is the longest stage, so the order decides how long the other two trail behind it.  Every cell is
    run once by itself (after a warm-up call) with CUDA events around its three stages; Johnson's rule on
    (copy in, module call + copy out) then puts the cells that take longer to drain than to feed first, by
    increasing copy-in time, and the others last, by decreasing drain time.  Nothing is skipped or merged: the
    timed step still copies every input in and every output out.
    """
    stream = torch.cuda.current_stream(device)
    measured = []
    for si, (_name, n, k) in enumerate(SHAPES):
        for m in TOKENS:
            host_x = torch.randn(m, k).bfloat16().pin_memory()
            host_y = torch.empty(m, n, dtype=torch.bfloat16).pin_memory()
            dev_x = torch.empty(m, k, dtype=torch.bfloat16, device=device)
            marks = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            with torch.no_grad():
                for attempt in range(2):  # the first pass loads kernels and sizes workspaces
                    marks[0].record(stream)
                    dev_x.copy_(host_x, non_blocking=True)
                    marks[1].record(stream)
                    y = layers[si](dev_x)
                    marks[2].record(stream)
                    host_y.copy_(y, non_blocking=True)
                    marks[3].record(stream)
                    torch.cuda.synchronize(device)
            feed = marks[0].elapsed_time(marks[1])
            drain = marks[1].elapsed_time(marks[3])
            measured.append(((si, m), feed, drain))
    first = sorted((c for c in measured if c[1] < c[2]), key=lambda c: c[1])
    last = sorted((c for c in measured if c[1] >= c[2]), key=lambda c: -c[2])
    return [c[0] for c in first + last]


def run_e2e(torch, rt, FusedNQRTLinear, weights, device, steps: int, distributed: bool) -> dict:
    """The sweep through the plugin call (FusedNQRTLinear.forward) with pinned host inputs and outputs.

    One pinned slab holds the inputs of all 32 cells and one the outputs (in the order ``e2e_cell_order`` derives
    from per-cell measurements).  A step copies every cell's input to the
    device, calls the module, and copies the result back; the three kinds of work run on three streams so that
    copies in both directions overlap the kernels.  The whole step -- 32 host-to-device copies, 32 module calls,
    32 device-to-host copies -- is captured once as a CUDA graph and the timed region replays it: every input
    still crosses PCIe inside the timed region and every output is back in pinned host memory before the stop
    event, but the host issues one launch per step instead of several hundred calls.
    """
    numa = bind_to_gpu_numa_node(torch, device)
    layers = [FusedNQRTLinear(w, input_hadamard=True, activation_betas=ACT_BETAS).to(device) for w in weights]
    cells = e2e_cell_order(torch, layers, device)
    in_elems = [m * SHAPES[si][2] for si, m in cells]
    out_elems = [m * SHAPES[si][1] for si, m in cells]
    host_in = torch.empty(sum(in_elems), dtype=torch.bfloat16).pin_memory()
    host_out = torch.empty(sum(out_elems), dtype=torch.bfloat16).pin_memory()
    dev_in = torch.empty(sum(in_elems), dtype=torch.bfloat16, device=device)
    gen = torch.Generator().manual_seed(3000)
    host_in.copy_(torch.randn(host_in.numel(), generator=gen).bfloat16())
    in_off = [0]
    for n in in_elems:
        in_off.append(in_off[-1] + n)
    out_off = [0]
    for n in out_elems:
        out_off.append(out_off[-1] + n)
    h2d, d2h = host_in.numel() * 2, host_out.numel() * 2
    compute = torch.cuda.Stream(device)
    copy_in, copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)

    keep: list = []  # results stay allocated while another stream still reads them (for the graph: for its lifetime)

    def step() -> None:  # issued on `compute`; the side streams fork from it and join it again
        keep.clear()
        with torch.no_grad():
            copy_in.wait_stream(compute)
            copy_out.wait_stream(compute)
            ready = []
            with torch.cuda.stream(copy_in):
                for i in range(len(cells)):
                    dev_in[in_off[i]:in_off[i + 1]].copy_(host_in[in_off[i]:in_off[i + 1]], non_blocking=True)
                    event = torch.cuda.Event()
                    event.record(copy_in)
                    ready.append(event)
            for i, (si, m) in enumerate(cells):
                compute.wait_event(ready[i])
                y = layers[si](dev_in[in_off[i]:in_off[i + 1]].view(m, SHAPES[si][2]))
                keep.append(y)
                done = torch.cuda.Event()
                done.record(compute)
                with torch.cuda.stream(copy_out):
                    copy_out.wait_event(done)
                    host_out[out_off[i]:out_off[i + 1]].view(m, SHAPES[si][1]).copy_(y, non_blocking=True)
            compute.wait_stream(copy_in)
            compute.wait_stream(copy_out)

    graph = None
    with torch.cuda.stream(compute):
        step()  # warm-up, call by call
        torch.cuda.synchronize(device)
        try:
            captured = torch.cuda.CUDAGraph()
            with torch.cuda.graph(captured, stream=compute):
                step()
            captured.replay()
            torch.cuda.synchronize(device)
            graph = captured
        except Exception as error:  # keep the call-by-call step if the capture is refused
            print(f"bench: end-to-end step not captured ({type(error).__name__}: {error})", file=sys.stderr)
            torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(compute)
        for _ in range(steps):
            if graph is not None:
                graph.replay()
            else:
                step()
        e1.record(compute)
        torch.cuda.synchronize(device)
    checksum = float(host_out[:out_elems[0]].float().abs().sum())  # the largest cell's result really is on the host
    return {"ms": e0.elapsed_time(e1) / steps, "h2d": h2d, "d2h": d2h, "numa": numa, "nonzero_result": checksum > 0,
            "launch": "CUDA graph of one step (copies and module calls), replayed" if graph is not None else "call by call",
            "cell_order": "Johnson's rule on the measured (copy in, call + copy out) of every cell; first "
                          + f"{SHAPES[cells[0][0]][0]} M={cells[0][1]}, last {SHAPES[cells[-1][0]][0]} M={cells[-1][1]}"}


def gemv_workload(torch, rt, device, pk, only: str | None = None) -> dict:
    """M = 1 projection of the four shapes: packed weight (decode in the kernel) and resident decoded weight.

    Each timed graph cycles over enough copies of the weight to exceed the 126 MB L2, so every launch streams
    its weight from HBM.
    """
    import dataclasses

    weights, inputs, beta_table = gpu_setup(torch, rt, device)
    rows = []
    for (name, n, k), w in zip(SHAPES, weights):
        if only and name != only:
            continue
        act = rt.quantize_activation_cuda(inputs[(k, 1)], q=14, betas=ACT_BETAS, beta_table=beta_table, keep_decoded=True)
        resident = rt.keep_decoded_weight(w)
        copies = max(2, (160 << 20) // (n * k * 2) + 1)
        clones = [dataclasses.replace(resident, decoded=resident.decoded.clone()) for _ in range(copies)]

        def run_resident():
            for clone in clones:
                rt.linear_packed_w4a4(act, clone)

        t_res = _time_graph(torch, run_resident, device, reps=2) / copies
        t_packed = _time_graph(torch, lambda: rt.linear_packed_w4a4(act, w), device)
        packed_bytes = n * k * 17 // 32 + 4 * n + 32
        rows.append({"shape": name, "n": n, "k": k, "packed_us": round(t_packed, 2),
                     "packed_gbs": round(packed_bytes / t_packed / 1e3, 1),
                     "resident_us": round(t_res, 2), "resident_bf16_gbs": round(n * k * 2 / t_res / 1e3, 1),
                     "resident_frac_of_hbm": round(n * k * 2 / t_res / 1e3 / pk["hbm_gbs"], 3),
                     "packed_bytes_over_resident_time_gbs": round(packed_bytes / t_res / 1e3, 1)})
        del clones, resident
    return {"m": 1, "cells": rows}


def kv_workload(torch, rt, device, pk) -> dict:
    """NQKV4 pack + quantized-KV decode attention (batch 32, 8 KV heads, ctx 4096 + 1 hot token, head_dim 64)."""
    from nestquant_aiinfra_b200.formats import KEY_BETAS, VALUE_BETAS
    from nestquant_aiinfra_b200.rotation import hadamard

    batch, heads, q_heads, dim, page, ctx = 32, 8, 32, 64, 16, 4096
    pages_per_seq = ctx // page
    capacity = batch * pages_per_seq
    pool = rt.NQKVPagePool(capacity=capacity, page_size=page, num_kv_heads=heads, head_dim=dim, key_betas=KEY_BETAS,
                           value_betas=VALUE_BETAS, device=device)
    cache = rt.NQKVHotColdCache(pool, max_sequences=batch, max_pages_per_sequence=pages_per_seq + 1)
    gen = torch.Generator().manual_seed(4096)
    perm = torch.randperm(capacity, generator=gen).to(device)
    rows = capacity * page * heads
    for which, (codes, betas, norms, table, tbl_vals) in enumerate((
            (pool.key_codes, pool.key_betas, pool.key_norms, pool.beta_table, KEY_BETAS),
            (pool.value_codes, pool.value_betas, pool.value_norms, pool.value_beta_table, VALUE_BETAS))):
        x = torch.randn(batch, ctx, heads, dim, generator=gen)
        flat = torch.randperm(heads * dim, generator=gen)[:6]
        x.view(batch, ctx, heads * dim)[:, :, flat] *= 8.0          # 1 % outlier channels
        x = x.to(device)
        x = hadamard(x) if which == 0 else x                        # keys are rotated per head, values are not
        act = rt.quantize_activation_cuda(x.bfloat16().reshape(rows, dim), q=14, betas=tbl_vals, beta_table=table,
                                          keep_decoded=False)
        codes[perm] = act.code_payload.view(capacity, -1)
        betas[perm] = act.beta_payload.view(capacity, -1)
        norms[perm] = act.row_norms.view(capacity, -1)
        del x, act
    for slot in range(batch):
        cache.register(slot)
    cache.page_indices[:, :pages_per_seq] = perm.view(batch, pages_per_seq).to(torch.int32)
    cache.page_counts.fill_(pages_per_seq)
    cache.last_page_len.fill_(page)
    cache.hot_lengths.fill_(1)
    cache.sequence_lengths.fill_(ctx + 1)
    cache.hot_keys[:, 0] = torch.randn(batch, heads, dim, generator=gen).bfloat16().to(device)
    cache.hot_values[:, 0] = torch.randn(batch, heads, dim, generator=gen).bfloat16().to(device)
    q = hadamard(torch.randn(batch, q_heads, dim, generator=gen).to(device)).bfloat16()
    slot_ids = torch.arange(batch, dtype=torch.int32, device=device)
    active = torch.ones(batch, dtype=torch.bool, device=device)
    ws = rt.BatchedNQKVAttentionWorkspace.create(cache, batch_size=batch, query_heads=q_heads)
    t_attn = _time_graph(torch, lambda: rt._launch_nqkv_decode_attention_batched_k1(
        q, cache, slot_ids=slot_ids, active_mask=active, attention_scale=0.125, workspace=ws), device)
    attn_bytes = batch * pages_per_seq * pool.page_payload_bytes + batch * 2 * heads * dim * 2 + 2 * batch * q_heads * dim * 2
    # page pack: all 32 hot tails full, packed into fresh pages of a second pool region (re-armed every launch)
    pack_pool = rt.NQKVPagePool(capacity=batch, page_size=page, num_kv_heads=heads, head_dim=dim, key_betas=KEY_BETAS,
                                value_betas=VALUE_BETAS, device=device)
    pack_cache = rt.NQKVHotColdCache(pack_pool, max_sequences=batch, max_pages_per_sequence=4)
    for slot in range(batch):
        pack_cache.register(slot)
    pack_cache.hot_keys.copy_(torch.randn(pack_cache.hot_keys.shape, generator=gen).bfloat16())
    pack_cache.hot_values.copy_(torch.randn(pack_cache.hot_values.shape, generator=gen).bfloat16())
    pack_cache.graph_target_page_ids.copy_(torch.arange(batch, dtype=torch.int32))

    def rearm():  # the publish step empties the hot tails and advances the page tables: put both back
        pack_cache.hot_lengths.fill_(page)
        pack_cache.page_counts.zero_()

    def pack_once():
        rearm()
        rt.launch_pack_full_hot_pages_graph_safe(pack_cache, boundary_mask=active)

    t_rearm = _time_graph(torch, rearm, device, reps=48)
    t_pack = max(_time_graph(torch, pack_once, device, reps=48) - t_rearm, 0.0)  # the pack + publish launches alone
    pack_bytes = batch * (2 * page * heads * dim * 2 + pack_pool.page_payload_bytes)
    # ragged prefill over the same pool: every sequence continues a cached context of U[0, 4032] tokens with a
    # chunk of U[1, 64] new tokens whose K/V are already appended (cold pages + hot tail); causal, pages read directly
    starts = torch.randint(0, 4033, (batch,), generator=gen)
    chunks = torch.randint(1, 65, (batch,), generator=gen)
    totals = starts + chunks
    pre_cache = rt.NQKVHotColdCache(pool, max_sequences=batch, max_pages_per_sequence=pages_per_seq + 1)
    for slot in range(batch):
        pre_cache.register(slot)
    pre_cache.page_indices[:, :pages_per_seq] = perm.view(batch, pages_per_seq).to(torch.int32)
    pre_cache.page_counts.copy_((totals // page).to(torch.int32))
    pre_cache.last_page_len.copy_(torch.where(totals >= page, page, 0).to(torch.int32))
    pre_cache.hot_lengths.copy_((totals % page).to(torch.int32))
    pre_cache.sequence_lengths.copy_(totals.to(torch.int32))
    pre_cache.hot_keys.copy_(torch.randn(pre_cache.hot_keys.shape, generator=gen).bfloat16())
    pre_cache.hot_values.copy_(torch.randn(pre_cache.hot_values.shape, generator=gen).bfloat16())
    t_max = int(chunks.max())
    pq = hadamard(torch.randn(batch, t_max, q_heads, dim, generator=gen).to(device)).bfloat16()
    q_lens = chunks.to(torch.int32).to(device)
    pws = rt.BatchedNQKVAttentionWorkspace.create(pre_cache, batch_size=batch, query_heads=q_heads, query_tokens=t_max)
    t_prefill = _time_graph(torch, lambda: rt.nqkv_prefill_attention(
        pq, pre_cache, slot_ids=slot_ids, query_lengths=q_lens, scale=0.125, workspace=pws), device)
    new_tokens = int(chunks.sum())
    # algorithmic bytes: every sequence's pages and hot tail once, its queries in and its outputs out
    prefill_bytes = int(((totals // page) * pool.page_payload_bytes + (totals % page) * 2 * heads * dim * 2).sum()) \
        + 2 * new_tokens * q_heads * dim * 2
    # opt-in decoded shadow of the pool: same attention call, coordinates read instead of searched
    before = ws.output.clone()
    shadow_bytes = pool.enable_lattice_shadow()
    t_shadow = _time_graph(torch, lambda: rt._launch_nqkv_decode_attention_batched_k1(
        q, cache, slot_ids=slot_ids, active_mask=active, attention_scale=0.125, workspace=ws), device)
    torch.cuda.synchronize(device)
    identical = bool(torch.equal(before, ws.output))
    lattice_read = batch * pages_per_seq * (2 * page * heads * dim + pool.page_payload_bytes - 2 * pool._code_bytes)
    return {
        "attention_decode": {"batch": batch, "ctx": ctx + 1, "q_heads": q_heads, "kv_heads": heads, "head_dim": dim,
                             "pages_per_seq": pages_per_seq, "us": round(t_attn, 2),
                             "gbs": round(attn_bytes / t_attn / 1e3, 1),
                             "frac_of_hbm": round(attn_bytes / t_attn / 1e3 / pk["hbm_gbs"], 4)},
        "attention_decode_lattice_shadow": {
            "note": "opt-in: int8 lattice coordinates kept beside the codes", "extra_bytes": int(shadow_bytes),
            "us": round(t_shadow, 2), "bytes_read": int(lattice_read),
            "gbs": round(lattice_read / t_shadow / 1e3, 1),
            "frac_of_hbm": round(lattice_read / t_shadow / 1e3 / pk["hbm_gbs"], 4),
            "output_identical_to_packed": identical},
        "page_pack_publish": {"pages": batch, "us": round(t_pack, 2), "us_per_page": round(t_pack / batch, 3),
                              "gbs": round(pack_bytes / t_pack / 1e3, 1),
                              "frac_of_hbm": round(pack_bytes / t_pack / 1e3 / pk["hbm_gbs"], 4),
                              "note": "pack + publish launches alone (the two fills that re-arm the cache, "
                                      f"{t_rearm:.2f} us, are timed separately and subtracted)"},
        "attention_prefill_ragged": {
            "batch": batch, "start_contexts": "U[0, 4032]", "chunk_lengths": "U[1, 64]", "new_tokens": new_tokens,
            "cached_tokens": int(totals.sum()), "q_heads": q_heads, "kv_heads": heads, "head_dim": dim,
            "us": round(t_prefill, 2), "new_tok_per_s": round(new_tokens / t_prefill * 1e6, 1),
            "gbs": round(prefill_bytes / t_prefill / 1e3, 1),
            "frac_of_hbm": round(prefill_bytes / t_prefill / 1e3 / pk["hbm_gbs"], 4),
            "bytes": "pages + hot tail of every sequence once, queries in, outputs out"},
    }


def continuous_batch(torch, runner, cache, device, *, total_requests: int = 96, new_tokens: int = 256,
                     prefill_group: int = 8, seed: int = 129) -> dict:
    """Config 3 as a continuous batch: more requests than slots, prompts U[128, 2048], `new_tokens` greedy tokens each.

    Requests are admitted `prefill_group` at a time into free slots (whole-prompt prefill, eager), every admitted
    request decodes one token per step of the ONE captured graph, a request that has its tokens releases its slot
    and the next waiting requests join.  Sampling stays on the device; the host only counts.
    """
    from collections import deque

    capacity = cache.capacity
    cache.release_slots(list(range(capacity)))
    gen = torch.Generator().manual_seed(seed)
    lengths = torch.randint(128, 2049, (total_requests,), generator=gen).tolist()
    prompts = [torch.randint(0, 128256, (n,), generator=gen) for n in lengths]
    waiting = deque(range(total_requests))
    owner = [None] * capacity   # request of a slot
    left = [0] * capacity       # decode tokens the slot's request still needs
    generated = prefilled = steps = active_rows = 0
    decode_events, prefill_s = [], 0.0
    torch.cuda.synchronize(device)
    wall0 = time.perf_counter()
    while waiting or any(left):
        free = [s for s in range(capacity) if owner[s] is None]
        running = capacity - len(free)
        if waiting and free and (len(free) >= prefill_group or running == 0 or len(waiting) <= len(free)):
            group = [waiting.popleft() for _ in range(min(prefill_group, len(free), len(waiting)))]
            slots = free[:len(group)]
            t0 = time.perf_counter()
            runner.prefill_slots(slots, [prompts[i] for i in group])   # also samples each request's first token
            torch.cuda.synchronize(device)
            prefill_s += time.perf_counter() - t0
            for slot, request in zip(slots, group):
                owner[slot], left[slot] = request, new_tokens - 1
                prefilled += lengths[request]
                generated += 1
            if runner.graph is None:
                runner.capture_decode_graph()
        if any(left):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            runner.decode()
            e1.record()
            decode_events.append((e0, e1))
            steps += 1
            done = []
            for slot in range(capacity):
                if left[slot]:
                    left[slot] -= 1
                    generated += 1
                    active_rows += 1
                    if left[slot] == 0:
                        done.append(slot)
            if done:
                cache.release_slots(done)
                for slot in done:
                    owner[slot] = None
    torch.cuda.synchronize(device)
    wall = time.perf_counter() - wall0
    decode_ms = sum(a.elapsed_time(b) for a, b in decode_events)
    return {"requests": total_requests, "slots": capacity, "new_tokens_each": new_tokens, "prompt_tokens": int(prefilled),
            "generated_tokens": generated, "decode_steps": steps, "mean_active_rows": round(active_rows / max(steps, 1), 1),
            "decode_ms_per_step": round(decode_ms / max(steps, 1), 3),
            "decode_tok_s": round(active_rows / (decode_ms * 1e-3), 1),
            "prefill_s": round(prefill_s, 2), "wall_s": round(wall, 2),
            "tok_s_including_prefill": round(generated / wall, 1), "cuda_graph": True,
            "note": "requests finish, release their slot and new ones join between replays of one decode graph"}


def decode_workload(torch, device, *, requests: int = 64, new_tokens: int = 256, kernel_mix: bool = False) -> dict:
    """Llama-3.2-1B architecture, random init, W4A4KV4: ragged prefill then graph decode of `requests` rows."""
    from nestquant_aiinfra_b200.engine import BatchedNQKVLlamaRunner, build_llama_w4a4kv4

    model, cache = build_llama_w4a4kv4(hidden_size=2048, intermediate_size=8192, num_layers=16, num_heads=32,
                                       num_kv_heads=8, head_dim=64, vocab_size=128256, capacity=requests,
                                       max_cache_len=2048 + new_tokens + 16 + 144, device=device, seed=0)
    runner = BatchedNQKVLlamaRunner(model, cache)
    gen = torch.Generator().manual_seed(128)
    lengths = torch.randint(128, 2049, (requests,), generator=gen).tolist()
    prompts = [torch.randint(0, 128256, (n,), generator=gen) for n in lengths]
    order = sorted(range(requests), key=lambda i: lengths[i])
    torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    for start in range(0, requests, 8):  # 8 prompts of similar length per prefill call
        group = order[start:start + 8]
        runner.prefill_slots(group, [prompts[i] for i in group])
    torch.cuda.synchronize(device)
    prefill_s = time.perf_counter() - t0
    runner.capture_decode_graph()
    for _ in range(3):
        runner.decode()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    steps = new_tokens - 3
    for _ in range(steps):
        runner.decode()
    e1.record()
    torch.cuda.synchronize(device)
    ms = e0.elapsed_time(e1)
    mix = None
    if kernel_mix:  # device time per kernel over a few more graph replays (CUPTI through torch.profiler)
        from torch.profiler import ProfilerActivity, profile

        replays = 5
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(replays):
                runner.decode()
            torch.cuda.synchronize(device)
        rows = []
        for event in prof.key_averages():
            total = getattr(event, "device_time_total", None) or getattr(event, "cuda_time_total", 0)
            if total > 0:
                rows.append((total / replays, event.count / replays, event.key))
        rows.sort(reverse=True)
        whole = sum(r[0] for r in rows)
        mix = [{"kernel": key[:80], "us_per_step": round(us, 1), "launches_per_step": round(count, 1),
                "share": round(us / whole, 4)} for us, count, key in rows[:16]]
        mix.append({"kernel": "all kernels", "us_per_step": round(whole, 1)})
    # config 3 proper: a continuous batch on the same model (96 requests over the 64 slots)
    try:
        continuous = continuous_batch(torch, runner, cache, device)
    except Exception as error:
        continuous = {"error": f"{type(error).__name__}: {error}"[:300]}
    # back to a full static batch for the opt-in legs below
    cache.release_slots(list(range(requests)))
    for start in range(0, requests, 8):
        group = order[start:start + 8]
        runner.prefill_slots(group, [prompts[i] for i in group])
    # opt-in mode: the decoded BF16 weights stay in HBM (4x the packed bytes), no per-call weight decode;
    # same graph-decode loop, 64 more steps on the contexts reached by then
    added = runner.keep_decoded_weights()  # captures the decode graph again
    for _ in range(3):
        runner.decode()
    torch.cuda.synchronize(device)
    r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    r0.record()
    resident_steps = 61
    for _ in range(resident_steps):
        runner.decode()
    r1.record()
    torch.cuda.synchronize(device)
    resident_ms = r0.elapsed_time(r1)
    resident = {"note": "opt-in: decoded BF16 weights kept in HBM, no per-call weight decode",
                "extra_weight_bytes": int(added), "decode_steps": resident_steps,
                "ms_per_step": round(resident_ms / resident_steps, 3),
                "decode_tok_s": round(requests * resident_steps / (resident_ms * 1e-3), 1)}
    # second opt-in on top: the decoded lattice coordinates of every KV page kept beside its codes (8 bits per
    # entry), attention reads them instead of searching E8 per block; outputs are bit-identical
    kv_added = runner.enable_lattice_shadow()  # captures the decode graph again
    for _ in range(3):
        runner.decode()
    torch.cuda.synchronize(device)
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(resident_steps):
        runner.decode()
    s1.record()
    torch.cuda.synchronize(device)
    shadow_ms = s0.elapsed_time(s1)
    resident["with_kv_lattice_shadow"] = {
        "note": "also opt-in: decoded lattice coordinates of the KV pages kept beside the codes",
        "extra_kv_bytes": int(kv_added), "decode_steps": resident_steps,
        "ms_per_step": round(shadow_ms / resident_steps, 3),
        "decode_tok_s": round(requests * resident_steps / (shadow_ms * 1e-3), 1)}
    return {**({"kernel_mix": mix} if mix else {}), "continuous_batch": continuous, "resident_decoded_weights": resident,
            "model": "llama-3.2-1b-arch random init, W4A4KV4, 112 NQRT4 projections", "requests": requests,
            "static_batch_note": "the top-level figures are a static batch: all requests prefilled, then lock-step decode",
            "prompt_tokens": int(sum(lengths)), "decode_steps": steps, "ms_per_step": round(ms / steps, 3),
            "decode_tok_s": round(requests * steps / (ms * 1e-3), 1), "prefill_s": round(prefill_s, 2),
            "prefill_tok_s": round(sum(lengths) / prefill_s, 1), "cuda_graph": True}


def tp_decode(torch, dist, device, rank: int, world: int, *, layers: int, batch: int, context: int, steps: int,
              warmup: int, resident: bool = False, collective: str = "peer", decode_ahead: bool = False) -> dict:
    """Config 4: Llama-3-70B architecture (one seeded model sharded over the ranks), W4A4KV4, graph decode.

    Returns the measurements (identical on every rank; the times are the maximum over the ranks).  The
    all-reduce share comes from one more step issued call by call with CUDA events around every collective.
    """
    from nestquant_aiinfra_b200.fused_linear import FusedNQRTLinear
    from nestquant_aiinfra_b200.tensor_parallel import RowParallelNQRTLinear
    from nestquant_aiinfra_b200.tp_engine import TensorParallelRunner, build_llama_tp_shard, fill_cache_synthetic

    def timed(runner) -> float:
        for _ in range(warmup):
            runner.decode()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            runner.decode()
        e1.record()
        torch.cuda.synchronize(device)
        ms = torch.tensor([e0.elapsed_time(e1) / steps], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    t0 = time.perf_counter()
    model, cache = build_llama_tp_shard(hidden_size=8192, intermediate_size=28672, num_layers=layers, num_heads=64,
                                        num_kv_heads=8, head_dim=128, vocab_size=128256, rank=rank, world=world,
                                        capacity=batch, max_cache_len=context + 4 * (steps + warmup) + 48, device=device)
    fill_cache_synthetic(cache, context)
    runner = TensorParallelRunner(model, cache, weight_decode_ahead=decode_ahead)
    runner.start_decode(context)
    torch.cuda.synchronize(device)
    build_s = time.perf_counter() - t0
    row_modules = [m for m in model.modules() if isinstance(m, RowParallelNQRTLinear)]

    def capture() -> object:
        if isinstance(runner.graph, torch.cuda.CUDAGraph):
            runner.graph.reset()
        runner.graph = None
        try:
            runner.capture_decode_graph()
            return True
        except Exception as error:  # collectives inside a capture are not available everywhere
            runner.graph = None
            runner.cache.set_decode_state()
            return f"eager ({type(error).__name__})"

    # The partial sums after o_proj / down_proj: NCCL, or this repository's own kernel over peer memory (one node).
    collective_note = "NCCL all_reduce(sum) of [batch, 8192] BF16 after o_proj and down_proj"
    reducer = None
    if world > 1 and collective == "peer":
        try:
            from nestquant_aiinfra_b200.tp_engine import attach_peer_all_reduce

            reducer = attach_peer_all_reduce(model, batch, device)
            collective_note = ("nq_tp_allreduce_bf16 (peer-memory loads over NVLink, float32 sum in rank order) of "
                               "[batch, 8192] BF16 after o_proj and down_proj")
        except Exception as error:
            reducer = None
            for module in row_modules:
                module.peer_all_reduce = None
            collective_note += f"; peer-memory collective unavailable ({type(error).__name__}: {error})"[:200]
    graph = capture()
    ms_step = timed(runner)
    if reducer is not None:
        # a bounded wait of the peer-memory collective that gave up on any rank voids the run: NCCL takes over
        broken = torch.tensor([reducer.status()], device=device)
        dist.all_reduce(broken, op=dist.ReduceOp.MAX)
        if int(broken.item()) != 0:
            collective_note = (f"NCCL all_reduce(sum) of [batch, 8192] BF16 (the peer-memory collective reported "
                               f"status {int(broken.item())} and was dropped)")
            reducer = None
            for module in row_modules:
                module.peer_all_reduce = None
            graph = capture()
            ms_step = timed(runner)
    tokens = runner.next_tokens.clone()
    same = torch.tensor([1], device=device)
    if world > 1:
        first = tokens.clone()
        dist.broadcast(first, src=0)
        same = torch.tensor([int(torch.equal(first, tokens))], device=device)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
    # all-reduce share: one eager step with events around every collective (2 per layer)
    collective_ms, collectives = 0.0, 0
    if world > 1:
        events: list = []
        for module in row_modules:
            module.collective_events = events
        runner.decode_eager()
        torch.cuda.synchronize(device)
        for module in row_modules:
            module.collective_events = None
        t = torch.tensor([sum(a.elapsed_time(b) for a, b in events)], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        collective_ms, collectives = float(t.item()), len(events)
    # the same step with the OTHER collective, for comparison (never the headline; any failure only drops the key)
    other = None
    if world > 1:
        try:
            if reducer is None:
                from nestquant_aiinfra_b200.tensor_parallel import PeerAllReduce

                trial = PeerAllReduce(batch * 8192, device)
                for module in row_modules:
                    module.peer_all_reduce = trial
                graph_other = capture()
                other_ms = timed(runner)
                broken = torch.tensor([trial.status()], device=device)
                dist.all_reduce(broken, op=dist.ReduceOp.MAX)
                other = {"collective": "nq_tp_allreduce_bf16 (this repository's kernel: peer-memory loads over NVLink)",
                         "ms_per_step": other_ms, "cuda_graph": graph_other, "status": int(broken.item())}
            else:
                for module in row_modules:
                    module.peer_all_reduce = None
                graph_other = capture()
                other = {"collective": "NCCL all_reduce", "ms_per_step": timed(runner), "cuda_graph": graph_other}
        except Exception as error:
            other = {"error": f"{type(error).__name__}: {error}"[:200]}
        for module in row_modules:
            module.peer_all_reduce = reducer
        graph = capture()  # back to the measured configuration for the opt-in legs below
    packed = sum(m.packed_device_bytes for m in model.modules() if isinstance(m, (FusedNQRTLinear, RowParallelNQRTLinear)))
    result = {
        "workload": "llama-3-70b-arch W4A4KV4 tensor-parallel decode (one seeded model sharded over the ranks)",
        "parallelism": f"tp{world}", "layers": layers, "batch": batch, "context": context, "steps": steps,
        "warmup": warmup, "ms_per_step": ms_step, "tok_s": batch / (ms_step * 1e-3),
        "ms_per_layer": ms_step / layers,
        "weight_decode_ahead": runner.cache.decode_ahead is not None,
        "all_reduce": {"collective": collective_note,
                       "per_step": collectives, "ms_per_step_eager": round(collective_ms, 3),
                       "share_of_step": round(collective_ms / ms_step, 4) if ms_step else None,
                       "other_collective": other},
        "cuda_graph": graph, "kv": "pages pre-filled by the page encoder with synthetic K/V",
        "packed_weight_bytes_per_rank": int(packed), "build_s": round(build_s, 1),
        "ranks_agree_on_tokens": bool(same.item()),
    }
    if layers != 80:
        result["ms_per_step_80_layers_extrapolated"] = ms_step / layers * 80
    if resident:
        # opt-in mode: every rank keeps the decoded BF16 weights of its shard; same graph-decode loop again
        from nestquant_aiinfra_b200.fused_linear import keep_decoded_weights_

        def recapture() -> None:
            if isinstance(runner.graph, torch.cuda.CUDAGraph):
                runner.graph.reset()
                runner.graph = None
            if graph is True:
                runner.capture_decode_graph()

        if isinstance(runner.graph, torch.cuda.CUDAGraph):
            runner.graph.reset()
            runner.graph = None
        added = keep_decoded_weights_(model)
        recapture()
        rms = timed(runner)
        result["resident_decoded_weights"] = {"note": "opt-in: decoded BF16 weights of the shard kept in HBM",
                                              "extra_weight_bytes_per_rank": int(added), "ms_per_step": rms,
                                              "tok_s": batch / (rms * 1e-3)}
        if isinstance(runner.graph, torch.cuda.CUDAGraph):
            runner.graph.reset()
            runner.graph = None
        kv_added = cache.enable_lattice_shadow()
        recapture()
        kms = timed(runner)
        result["resident_decoded_weights"]["with_kv_lattice_shadow"] = {
            "extra_kv_bytes_per_rank": int(kv_added), "ms_per_step": kms, "tok_s": batch / (kms * 1e-3)}
    # A live CUDA graph that captured NCCL kernels keeps the communicator busy: release it before any teardown.
    if isinstance(runner.graph, torch.cuda.CUDAGraph):
        runner.graph.reset()
    runner.graph = None
    del runner, model, cache
    torch.cuda.synchronize(device)
    torch.cuda.empty_cache()
    return result


def _teardown(torch, dist, device) -> None:
    """Leave the process group; bounded, so that a stuck finalize cannot hold the GPUs."""
    torch.cuda.synchronize(device)
    dist.barrier()
    torch.cuda.synchronize(device)
    sys.stdout.flush()
    watchdog = threading.Timer(45.0, lambda: os._exit(0))
    watchdog.daemon = True
    watchdog.start()
    dist.destroy_process_group()
    watchdog.cancel()


def run_tp70b(args) -> None:
    """Config 4 alone (run under torchrun, one process per GPU)."""
    import torch
    import torch.distributed as dist

    rank, local_rank = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    result = tp_decode(torch, dist, device, rank, world, layers=args.tp_layers, batch=args.tp_batch,
                       context=args.tp_context, steps=max(args.steps, 1), warmup=max(args.warmup, 3),
                       resident=args.tp_resident, collective=args.tp_collective,
                       decode_ahead=args.tp_decode_ahead == "on")
    if rank == 0:
        print(json.dumps({
            "metric": "w4a4kv4_tp_decode_tok_s", "value": result["tok_s"], "unit": "tok/s", "n_gpus": world,
            "steps": result["steps"], "warmup": result["warmup"], "ms_per_step": result["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "dtype": "bf16", "data": "synthetic",
            "config": {"workload": result["workload"], "layers": result["layers"], "batch": result["batch"],
                       "context": result["context"], "parallelism": result["parallelism"]},
            **{k: v for k, v in result.items() if k not in ("workload", "layers", "batch", "context", "parallelism",
                                                            "steps", "warmup", "ms_per_step")},
        }), flush=True)
    if world > 1:
        _teardown(torch, dist, device)


def run_single_extra(args) -> None:
    """One extra workload alone on GPU 0 (used for profiling captures)."""
    import torch

    import nestquant_aiinfra_b200.runtime as rt

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    if args.workload == "kv":
        result = kv_workload(torch, rt, device, peaks())
    elif args.workload == "gemv":
        result = gemv_workload(torch, rt, device, peaks(), args.shape)
    else:
        result = decode_workload(torch, device, kernel_mix=args.kernel_mix)
    print(json.dumps({"workload": args.workload, **result}), flush=True)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=5)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--streams", type=int, default=4,
                        help="streams the cells of one sweep step are issued on (1 = one after the other; the "
                             "one-stream time is measured and reported either way)")
    parser.add_argument("--impl", choices=("native", "reference"), default="native")
    parser.add_argument("--workload", choices=("all", "kv", "decode", "gemv", "tp70b"), default="all",
                        help="all = sweep (+ extras); kv / decode / gemv = only that extra workload, for profiling; "
                             "tp70b = Llama-3-70B-architecture tensor-parallel decode (run under torchrun)")
    parser.add_argument("--tp-layers", type=int, default=80, help="decoder layers of the tp70b workload")
    parser.add_argument("--tp-batch", type=int, default=128)
    parser.add_argument("--tp-context", type=int, default=4096)
    parser.add_argument("--shape", choices=[name for name, _, _ in SHAPES], default=None,
                        help="with --workload gemv: only this projection shape (short profiling runs)")
    parser.add_argument("--tp-collective", choices=("peer", "nccl"), default="peer",
                        help="tensor-parallel sum after o_proj / down_proj: this repository's peer-memory kernel "
                             "(falls back to NCCL when symmetric memory is unavailable or a wait gives up) or NCCL; "
                             "the other one is timed too and reported under all_reduce.other_collective")
    parser.add_argument("--tp-decode-ahead", choices=("on", "off"), default="on",
                        help="tensor-parallel decode: decode the shard's o / gate-up / down weights of a layer on a "
                             "second stream during the layer's attention (as the single-GPU runner does by default)")
    parser.add_argument("--tp-resident", action="store_true",
                        help="tp70b: also time the opt-in mode that keeps the decoded BF16 weights of the shard in HBM")
    parser.add_argument("--kernel-mix", action="store_true",
                        help="with --workload decode: add the device time per kernel of a decode step (torch.profiler)")
    parser.add_argument("--skip-extras", action="store_true",
                        help="timed sweep only: no per-cell table, no end-to-end pass, no CPU baseline (profiling runs)")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "tp70b":
        run_tp70b(args)
    elif args.workload != "all":
        run_single_extra(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
