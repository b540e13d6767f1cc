// Rotary position embedding of the query / key heads, optionally followed by the float32
// Hadamard rotation the KV backend applies to them, in one launch.
//
// Arithmetic of the tensor-op sequence it replaces, result for result:
//   rope      (x * cos) + (rotate_half(x) * sin), each product and the sum rounded to the tensor
//             dtype (Hugging Face's apply_rotary_pos_emb on BF16 tensors; rotate_half(x) =
//             (-x[D/2:], x[:D/2]))
//   rotation  hadamard(x.float()).to(dtype) as runtime/nqkv_batched_hf_backend.py:381,549 does for
//             keys and queries: float32 butterflies, IEEE division by sqrt(D), one final rounding.
// One thread owns 8 consecutive features of one (batch, head, token) vector.
#include <math.h>

#include "nq_common.cuh"
#include "nq_rotate_core.cuh"

namespace {

constexpr int kRopeThreads = 128;

struct RopeParams {
    const void* x;
    const void* cos;
    const void* sin;
    void* out;
    int64_t vectors;                       // batch * heads * tokens
    int heads, tokens, dim;
    int64_t stride_b, stride_h, stride_t;  // element strides of x
    int apply_hadamard;
    float root, inv_root;
};

// blockIdx.y selects the tensor: a launch takes the query heads and the key heads of a layer together
// (second.vectors = 0 for a launch with one tensor).
template <typename T>
__global__ void __launch_bounds__(kRopeThreads) nq_rope_kernel(const RopeParams first, const RopeParams second) {
    extern __shared__ __align__(16) float buf[];
    const RopeParams& p = blockIdx.y ? second : first;
    const int bpr = p.dim >> 3;                        // groups of 8 features per vector
    const int vectors_per_cta = kRopeThreads / bpr;
    const int64_t v0 = (int64_t)blockIdx.x * vectors_per_cta;
    if (v0 >= p.vectors) return;  // the grid is sized for the larger tensor
    const int nvec = (int)min((int64_t)vectors_per_cta, p.vectors - v0);
    const int total = nvec * p.dim;
    const T* x = reinterpret_cast<const T*>(p.x);
    const T* cs = reinterpret_cast<const T*>(p.cos);
    const T* sn = reinterpret_cast<const T*>(p.sin);
    T* out = reinterpret_cast<T*>(p.out);

    auto load = [&](int g, float v[8]) {
        const int64_t vec = v0 + g / bpr;
        const int grp = g % bpr;
        const int64_t t = vec % p.tokens, bh = vec / p.tokens, h = bh % p.heads, b = bh / p.heads;
        const T* base = x + b * p.stride_b + h * p.stride_h + t * p.stride_t;
        const int half = bpr >> 1;
        const bool low = grp < half;
        float a[8], partner[8], c[8], s[8];
        nq_load8<T>(base + grp * 8, a);
        nq_load8<T>(base + (low ? grp + half : grp - half) * 8, partner);
        nq_load8<T>(cs + (b * p.tokens + t) * p.dim + grp * 8, c);
        nq_load8<T>(sn + (b * p.tokens + t) * p.dim + grp * 8, s);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float rot = low ? -partner[j] : partner[j];
            const float first = nq_round_to<T>(nq_mul(a[j], c[j]));
            const float second = nq_round_to<T>(nq_mul(rot, s[j]));
            v[j] = nq_round_to<T>(nq_add(first, second));
        }
    };

    if (!p.apply_hadamard) {
        for (int g = threadIdx.x; g < (total >> 3); g += kRopeThreads) {
            float v[8];
            load(g, v);
            nq_store8<T>(out + v0 * p.dim + (int64_t)g * 8, v);
        }
        return;
    }
    nq_fwht_groups_to_smem<float>(load, buf, total, p.dim);  // float32 butterflies on the rounded rope result
    for (int g = threadIdx.x; g < (total >> 3); g += kRopeThreads) {
        const float4 lo = reinterpret_cast<const float4*>(buf + g * 8)[0];
        const float4 hi = reinterpret_cast<const float4*>(buf + g * 8)[1];
        float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = nq_div_by(v[j], p.root, p.inv_root);
        nq_store8<T>(out + v0 * p.dim + (int64_t)g * 8, v);
    }
}

template <typename T>
int launch_rope(const RopeParams& p, const RopeParams& second, cudaStream_t s) {
    const int vectors_per_cta = kRopeThreads / (p.dim >> 3);
    const int64_t most = p.vectors > second.vectors ? p.vectors : second.vectors;
    const int64_t grid = (most + vectors_per_cta - 1) / vectors_per_cta;
    const size_t smem = (size_t)vectors_per_cta * p.dim * sizeof(float);
    nq_rope_kernel<T><<<dim3((unsigned)grid, second.vectors > 0 ? 2u : 1u), kRopeThreads, smem, s>>>(p, second);
    NQ_CHECK_LAUNCH("nq_rope_hadamard");
    return NQ_OK;
}

int rope_params(RopeParams& p, const char* what, const void* x, int dtype, int64_t batch, int64_t heads, int64_t tokens,
                int64_t dim, int64_t stride_b, int64_t stride_h, int64_t stride_t, const void* cos, const void* sin,
                int apply_hadamard, void* out) {
    NQ_REQUIRE(x && cos && sin && out, NQ_ERR_ARG, "%s: null pointer", what);
    NQ_REQUIRE(batch >= 1 && heads >= 1 && tokens >= 1, NQ_ERR_ARG, "%s: empty tensor", what);
    NQ_REQUIRE(dim >= 16 && dim <= 1024 && (dim & (dim - 1)) == 0, NQ_ERR_ARG,
               "%s: dim=%lld must be a power of two in [16, 1024]", what, (long long)dim);
    NQ_REQUIRE(batch * heads * tokens <= ((int64_t)1 << 40), NQ_ERR_ARG, "%s: tensor too large", what);
    const int64_t esize = dtype == NQ_F32 ? 4 : 2;
    NQ_REQUIRE(nq_aligned16(x) && nq_aligned16(cos) && nq_aligned16(sin) && nq_aligned16(out) &&
                   (stride_b * esize) % 16 == 0 && (stride_h * esize) % 16 == 0 && (stride_t * esize) % 16 == 0,
               NQ_ERR_ALIGN, "%s: pointers and strides must be 16-byte aligned", what);
    p.x = x; p.cos = cos; p.sin = sin; p.out = out;
    p.vectors = batch * heads * tokens;
    p.heads = (int)heads; p.tokens = (int)tokens; p.dim = (int)dim;
    p.stride_b = stride_b; p.stride_h = stride_h; p.stride_t = stride_t;
    p.apply_hadamard = apply_hadamard;
    p.root = (float)sqrt((double)dim);
    p.inv_root = 1.0f / p.root;
    return NQ_OK;
}

int launch_rope_dtype(int dtype, const RopeParams& p, const RopeParams& second, cudaStream_t s) {
    switch (dtype) {
        case NQ_F32: return launch_rope<float>(p, second, s);
        case NQ_BF16: return launch_rope<__nv_bfloat16>(p, second, s);
        case NQ_F16: return launch_rope<__half>(p, second, s);
        default: nq_set_error("nq_rope_hadamard: unknown dtype %d", dtype); return NQ_ERR_ARG;
    }
}

}  // namespace

extern "C" int nq_rope_hadamard(const void* x, int dtype, int64_t batch, int64_t heads, int64_t tokens, int64_t dim,
                                int64_t stride_b, int64_t stride_h, int64_t stride_t, const void* cos,
                                const void* sin, int apply_hadamard, void* out, nq_stream_t stream) {
    NQ_RANGE("nq_rope_hadamard");
    RopeParams p, none = {};
    const int rc = rope_params(p, "nq_rope_hadamard", x, dtype, batch, heads, tokens, dim, stride_b, stride_h, stride_t,
                               cos, sin, apply_hadamard, out);
    if (rc) return rc;
    return launch_rope_dtype(dtype, p, none, reinterpret_cast<cudaStream_t>(stream));
}

// The query heads and the key heads of one attention layer in ONE launch (same cos / sin, same dtype, same
// batch, tokens and dim; each tensor with its own head count, strides and output).
extern "C" int nq_rope_hadamard_pair(const void* q, const void* k, int dtype, int64_t batch, int64_t q_heads,
                                     int64_t k_heads, int64_t tokens, int64_t dim, const int64_t* q_strides,
                                     const int64_t* k_strides, const void* cos, const void* sin, int apply_hadamard,
                                     void* q_out, void* k_out, nq_stream_t stream) {
    NQ_RANGE("nq_rope_hadamard_pair");
    NQ_REQUIRE(q_strides && k_strides, NQ_ERR_ARG, "nq_rope_hadamard_pair: null strides");
    RopeParams pq, pk;
    int rc = rope_params(pq, "nq_rope_hadamard_pair(q)", q, dtype, batch, q_heads, tokens, dim, q_strides[0], q_strides[1],
                         q_strides[2], cos, sin, apply_hadamard, q_out);
    if (rc) return rc;
    rc = rope_params(pk, "nq_rope_hadamard_pair(k)", k, dtype, batch, k_heads, tokens, dim, k_strides[0], k_strides[1],
                     k_strides[2], cos, sin, apply_hadamard, k_out);
    if (rc) return rc;
    return launch_rope_dtype(dtype, pq, pk, reinterpret_cast<cudaStream_t>(stream));
}
