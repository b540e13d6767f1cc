// Host build of the device codec header, so the CPU test-suite can compare the
// exact source the kernels use against the CPU checker.  Built by the test
// with: g++ -O2 -shared -fPIC -ffp-contract=off.
#include "nq_e8.cuh"

extern "C" {

void shim_nearest_e8(const float* x, float* out, long n) {
    for (long i = 0; i < n; ++i) nq_e8_nearest_exact(x + 8 * i, out + 8 * i);
}

void shim_dither(long first_block, long blocks, long seed, float* out) {
    for (long b = 0; b < blocks; ++b)
        nq_dither_block((uint32_t)((uint64_t)(first_block + b) * 8u + (uint64_t)seed), out + 8 * b);
}

void shim_decode(const uint32_t* words, long n, float* out) {
    for (long i = 0; i < n; ++i) nq_decode_codeword_exact(words[i], nullptr, out + 8 * i);
}

// x: normalised blocks [n,8]; seed < 0 -> no dither.
void shim_encode_blocks(const float* x, long n, const float* beta, long seed, long first_block,
                        uint32_t* words, int* beta_ids, float* recon) {
    for (long i = 0; i < n; ++i) {
        float d[8];
        const float* dp = nullptr;
        if (seed >= 0) {
            nq_dither_block((uint32_t)((uint64_t)(first_block + i) * 8u + (uint64_t)seed), d);
            dp = d;
        }
        words[i] = nq_encode_block(x + 8 * i, beta, dp, beta_ids[i], recon + 8 * i);
    }
}

float shim_bf16_round(float v) { return nq_bf16_round(v); }
}

extern "C" {
void shim_nearest_e8_guarded(const float* x, float* out, long n) {
    for (long i = 0; i < n; ++i) nq_e8_nearest_guarded(x + 8 * i, out + 8 * i);
}
void shim_nearest_e8_guarded_lean(const float* x, float* out, long n) {
    for (long i = 0; i < n; ++i) nq_e8_nearest_guarded<true>(x + 8 * i, out + 8 * i);
}

// Weight-path decode of packed codewords: r = t - d - 14 Q((t - d)/14).
void shim_decode_weight(const uint32_t* words, long n, long first_block, long seed, float* out) {
    for (long i = 0; i < n; ++i)
        nq_decode_weight_block(words[i], (uint32_t)((uint64_t)(first_block + i) * 8u + (uint64_t)seed), out + 8 * i);
}
}

extern "C" {
// Pruned undithered search; must equal shim_encode_blocks(seed < 0) on every input.
void shim_encode_blocks_pruned(const float* x, long n, const float* beta, uint32_t* words, int* beta_ids,
                               float* recon) {
    for (long i = 0; i < n; ++i) words[i] = nq_encode_block_pruned(x + 8 * i, beta, beta_ids[i], recon + 8 * i);
}

// The search as the encoder kernel runs it: cheap pass, boundary candidates evaluated from
// their lattice point, leftovers by the generic evaluation, everything merged by key.
// Must equal shim_encode_blocks(seed < 0) on every input.
void shim_encode_blocks_queued(const float* xs, long n, const float* beta, uint32_t* words, int* beta_ids,
                               float* recon, long* boundary_items) {
    long items = 0;
    for (long i = 0; i < n; ++i) {
        const float* x = xs + 8 * i;
        int best;
        float best_err, best_lam[8];
        unsigned pending;
        int qn = 0, qb[4];
        float qlam[4][8];
        nq_encode_block_fastpass_push(x, beta, best, best_err, best_lam, pending, [&](int b, const float* lam) {
            qb[qn] = b;
            for (int j = 0; j < 8; ++j) qlam[qn][j] = lam[j];
            ++qn;
        });
        unsigned long long key = ~0ull;
        uint32_t word = 0;
        float rec[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (best >= 0) {
            key = nq_candidate_key(best_err, best);
            word = nq_lattice_to_codeword(best_lam);
            for (int j = 0; j < 8; ++j) rec[j] = nq_mul(best_lam[j], beta[best]);
        }
        for (int q = 0; q < qn; ++q) {
            float r[8], err;
            const uint32_t w = nq_eval_candidate_from_lam(x, qlam[q], beta[qb[q]], r, err);
            const unsigned long long k2 = nq_candidate_key(err, qb[q]);
            if (k2 < key) { key = k2; word = w; for (int j = 0; j < 8; ++j) rec[j] = r[j]; }
        }
        for (int c = 0; c < 4; ++c) {
            if (!((pending >> c) & 1u)) continue;
            float r[8], err;
            const uint32_t w = nq_encode_candidate_exact(x, beta[c], nullptr, r, err);
            const unsigned long long k2 = nq_candidate_key(err, c);
            if (k2 < key) { key = k2; word = w; for (int j = 0; j < 8; ++j) rec[j] = r[j]; }
        }
        items += qn;
        words[i] = word;
        beta_ids[i] = (int)(key & 3u);
        for (int j = 0; j < 8; ++j) recon[8 * i + j] = rec[j];
    }
    if (boundary_items) *boundary_items = items;
}

void shim_cell_class(const float* lam, long n, int* out) {
    for (long i = 0; i < n; ++i) out[i] = nq_e8_cell_class(lam + 8 * i);
}

// Lean undithered decode against the exact one: every `stride`-th of the 14^8 codewords
// (offset varied with the high digits so that no digit pattern is left out); also decodes a
// caller-given list.  Returns the number of codewords whose eight values differ in any bit.
long shim_undithered_mismatches(long stride) {
    long bad = 0;
    const long half = 14L * 14 * 14 * 14;
    for (long hi = 0; hi < half; ++hi) {
        int c[8];
        long v = hi;
        for (int j = 4; j < 8; ++j) { c[j] = (int)(v % 14); v /= 14; }
        for (long lo = hi % stride; lo < half; lo += stride) {
            long u = lo;
            for (int j = 0; j < 4; ++j) { c[j] = (int)(u % 14); u /= 14; }
            uint32_t w = 0;
            for (int j = 0; j < 8; ++j) w |= (uint32_t)c[j] << (4 * j);
            float a[8], b[8], ta[8], tb[8];
            nq_decode_codeword_exact(w, nullptr, a);
            nq_decode_codeword_undithered(w, b);
            nq_generator_apply(c, ta);          // the generator matrix applied coordinate by coordinate
            nq_codeword_coset_packed(w, tb);    // the byte-parallel build the kernels use
            if (memcmp(a, b, sizeof a) || memcmp(ta, tb, sizeof ta)) ++bad;
        }
    }
    return bad;
}

void shim_decode_undithered(const uint32_t* words, long n, float* out) {
    for (long i = 0; i < n; ++i) nq_decode_codeword_undithered(words[i], out + 8 * i);
}

// 1 when the short division equals IEEE division for every half-integer coset coordinate.
int shim_div14_exact(void) {
    for (int twice = -80; twice <= 160; ++twice) {
        const float t = 0.5f * (float)twice;
        if (nq_div14_coset(t) != t / 14.0f) return 0;
    }
    return 1;
}
}

// Table-driven undithered decode (nq_decode_codeword_lut) against the exact decode.
namespace {
struct HostLut {
    uint32_t k[NQ_LUT_ENTRIES], o[NQ_LUT_ENTRIES];
    float q[NQ_LUT_ENTRIES][4];
    int bad_sub;
    HostLut() : bad_sub(0) {
        NqLutCoord all[NQ_LUT_ENTRIES];
        for (int i = 0; i < NQ_LUT_ENTRIES; ++i) nq_lut_coordinate(i - NQ_LUT_BIAS, all[i]);
        for (int i = 0; i < NQ_LUT_ENTRIES; ++i) {
            nq_lut_pack(all, i, k[i], o[i]);
            for (int c = 0; c < 4; ++c) q[i][c] = all[i].q[c];
            // the rank among entries of equal |R| must fit its three bits
            int sub0 = 0, sub1 = 0;
            for (int j = 0; j < NQ_LUT_ENTRIES; ++j) {
                sub0 += abs(all[j].r0_twice14) == abs(all[i].r0_twice14) && fabsf(all[j].e0) < fabsf(all[i].e0);
                sub1 += abs(all[j].r1_twice14) == abs(all[i].r1_twice14) && fabsf(all[j].e1) < fabsf(all[i].e1);
            }
            if (sub0 > 7 || sub1 > 7 || abs(all[i].r0_twice14) > 14 || abs(all[i].r1_twice14) > 14 ||
                abs(all[i].r0_twice14) + abs(all[i].r1_twice14) != 14)
                ++bad_sub;
        }
    }
};
const HostLut& host_lut() {
    static HostLut lut;
    return lut;
}
inline void decode_lut(uint32_t w, float* r) {
    const HostLut& lut = host_lut();
    nq_decode_codeword_lut(
        w,
        [&](uint32_t packed, int i, uint32_t& k, uint32_t& o) {
            const int idx = (packed >> (8 * i)) & 0xff;
            k = lut.k[idx];
            o = lut.o[idx];
        },
        [&](uint32_t packed, int i, float q[4]) {
            const int idx = (packed >> (8 * i)) & 0xff;
            for (int c = 0; c < 4; ++c) q[c] = lut.q[idx][c];
        },
        r);
}
}  // namespace

extern "C" {
// 0 when every table entry keeps its fields inside their bit widths.
int shim_lut_field_overflows(void) { return host_lut().bad_sub; }

// Codewords (every `stride`-th of the 14^8, upper half of the digits in [hi_begin, hi_end)) whose
// table-driven decode differs in any bit from the exact decode.
long shim_lut_mismatches(long stride, long hi_begin, long hi_end) {
    long bad = 0;
    const long half = 14L * 14 * 14 * 14;
    if (hi_end > half) hi_end = half;
    for (long hi = hi_begin; hi < hi_end; ++hi) {
        int c[8];
        long v = hi;
        for (int j = 4; j < 8; ++j) { c[j] = (int)(v % 14); v /= 14; }
        for (long lo = hi % stride; lo < half; lo += stride) {
            long u = lo;
            for (int j = 0; j < 4; ++j) { c[j] = (int)(u % 14); u /= 14; }
            uint32_t w = 0;
            for (int j = 0; j < 8; ++j) w |= (uint32_t)c[j] << (4 * j);
            float a[8], b[8];
            nq_decode_codeword_exact(w, nullptr, a);
            decode_lut(w, b);
            if (memcmp(a, b, sizeof a)) ++bad;
        }
    }
    return bad;
}

void shim_decode_lut(const uint32_t* words, long n, float* out) {
    for (long i = 0; i < n; ++i) decode_lut(words[i], out + 8 * i);
}
}
