// Nested-E8 codec arithmetic shared by every kernel of the W4A4KV4 path.
//
// The functions are written once for host and device: device builds use the
// IEEE round-to-nearest intrinsics (which the compiler never contracts into
// FMAs), host builds (g++ -ffp-contract=off) use plain operators.  The host
// build exists so the CPU test-suite can run exactly this source against the
// CPU checker before any GPU time is spent.
//
// "exact" functions reproduce the float32 operation ORDER of the reference's
// CPU path (nestquant/core/lattice.py:18-81, codec.py:53-142,
// quantizer.py:257-301): sequential 8-term error sums, strict "<" between the
// two E8 cosets, first-max / first-min tie rules.  They are used wherever the
// result must be bit-identical (the encoder, and every decode of an
// undithered stream, where exact Voronoi-boundary ties do occur).
#pragma once

#include <stdint.h>
#include <string.h>
#include <math.h>

#if defined(__CUDACC__)
#define NQ_HD __host__ __device__ __forceinline__
#else
#define NQ_HD inline
#endif

#define NQ_Q 14
#define NQ_MAGIC 12582912.0f /* 1.5 * 2^23: adding it rounds to nearest-even integer */

NQ_HD float nq_add(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fadd_rn(a, b);
#else
    return a + b;
#endif
}
NQ_HD float nq_sub(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fsub_rn(a, b);
#else
    return a - b;
#endif
}
NQ_HD float nq_mul(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fmul_rn(a, b);
#else
    return a * b;
#endif
}
NQ_HD float nq_div(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fdiv_rn(a, b);
#else
    return a / b;
#endif
}
NQ_HD float nq_rcp(float a) {
#if defined(__CUDA_ARCH__)
    return __frcp_rn(a);
#else
    return 1.0f / a;
#endif
}
NQ_HD float nq_sqrt(float a) {
#if defined(__CUDA_ARCH__)
    return __fsqrt_rn(a);
#else
    return sqrtf(a);
#endif
}
NQ_HD float nq_fma(float a, float b, float c) {
#if defined(__CUDA_ARCH__)
    return __fmaf_rn(a, b, c);
#else
    return fmaf(a, b, c);
#endif
}

// Correctly rounded a / b from the correctly rounded reciprocal rb = RN(1/b):
// two FMA residual corrections (Markstein).  Identical to IEEE division for
// normal-range operands (no overflow / underflow handling, which the
// normalised values of this codec never need); 5 instructions instead of the
// ~25 of the generic division.
NQ_HD float nq_div_by(float a, float b, float rb) {
    const float q0 = nq_mul(a, rb);
    const float r0 = nq_fma(-b, q0, a);
    const float q1 = nq_fma(r0, rb, q0);
    const float r1 = nq_fma(-b, q1, a);
    return nq_fma(r1, rb, q1);
}
#define NQ_RCP14 0.0714285746216774f /* RN(1/14) */

NQ_HD int nq_float_bits(float v) {
#if defined(__CUDA_ARCH__)
    return __float_as_int(v);
#else
    int b;
    memcpy(&b, &v, 4);
    return b;
#endif
}
NQ_HD float nq_bits_float(uint32_t b) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(b);
#else
    float v;
    memcpy(&v, &b, 4);
    return v;
#endif
}

// float32 -> bfloat16 (round to nearest even) -> float32, finite inputs only.
NQ_HD float nq_bf16_round(float v) {
    uint32_t u = (uint32_t)nq_float_bits(v);
    u += 0x7fffu + ((u >> 16) & 1u);
    return nq_bits_float(u & 0xffff0000u);
}
NQ_HD uint32_t nq_bf16_bits(float v) {
    uint32_t u = (uint32_t)nq_float_bits(v);
    u += 0x7fffu + ((u >> 16) & 1u);
    return u >> 16;
}

// ---------------------------------------------------------------- E8 ------

// Nearest point of D8 = {z in Z^8, sum even}; exact reference order.
// Rounding uses the magic-constant trick (valid for |y| < 2^22, far above
// any normalised value here); the low mantissa bit of the shifted value is
// the parity of the rounded integer, so no float->int conversion is needed.
NQ_HD void nq_d8_nearest_exact(const float y[8], float r[8]) {
    float e[8];
    int parity = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float t = nq_add(y[j], NQ_MAGIC);
        r[j] = nq_sub(t, NQ_MAGIC);
        parity ^= nq_float_bits(t);
        e[j] = nq_sub(y[j], r[j]);
    }
    float best = fabsf(e[0]);
    int jm = 0;
#pragma unroll
    for (int j = 1; j < 8; ++j) {
        const float a = fabsf(e[j]);
        if (a > best) { best = a; jm = j; }
    }
    if (parity & 1) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (j == jm) r[j] = nq_add(r[j], e[j] >= 0.0f ? 1.0f : -1.0f);
    }
}

NQ_HD float nq_sqdist8_seq(const float a[8], const float b[8]) {
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float d = nq_sub(a[j], b[j]);
        acc = nq_add(acc, nq_mul(d, d));
    }
    return acc;
}

// Nearest E8 point, half-integer coset wins ties (strict "<" for the integer
// coset) -- the "e8_upstream_half_coset_tie_v1" semantic.
NQ_HD void nq_e8_nearest_exact(const float x[8], float out[8]) {
    float p0[8], p1[8], y[8];
    nq_d8_nearest_exact(x, p0);
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = nq_sub(x[j], 0.5f);
    nq_d8_nearest_exact(y, p1);
#pragma unroll
    for (int j = 0; j < 8; ++j) p1[j] = nq_add(p1[j], 0.5f);
    const float e0 = nq_sqdist8_seq(x, p0);
    const float e1 = nq_sqdist8_seq(x, p1);
    const bool integer_coset = e0 < e1;
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = integer_coset ? p0[j] : p1[j];
}

// Nearest E8 point for continuous inputs (dithered weights): same roundings,
// parity rule and first-max rule as the exact function, but the two coset
// distances are formed from the rounding residuals with FMAs, and only the
// winning coset is repaired.  Whenever the distances are closer than 1e-4
// (summation-order effects are below 1e-6) the reference's comparison decides,
// evaluated from the roundings already at hand, so the result always equals
// nq_e8_nearest_exact.
// LEAN moves two pieces of work from the logic pipe to the FMA pipe: the parities of the two roundings come
// from the (exact) float sums of the rounded values instead of eight XORs of their bit patterns, and the
// rounded value of the winning coset is formed with an exact FMA instead of a select.  Same results; measured
// on B200 it shortens the encoder (four searches per block between other float work) by 0.7 % and lengthens the
// weight decode by 1 %, so only the encoder's searches use it.
template <bool LEAN = false>
NQ_HD void nq_e8_nearest_guarded(const float x[8], float out[8]) {
    float r0[8], e0[8], r1[8], e1[8];
    int par0 = 0, par1 = 0;
    float sum0 = 0.0f, sum1 = 0.0f;
    float s0 = 0.0f, s1 = 0.0f, m0 = 0.0f, m1 = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float t0 = nq_add(x[j], NQ_MAGIC);
        r0[j] = nq_sub(t0, NQ_MAGIC);
        if (LEAN) sum0 = nq_add(sum0, r0[j]);
        else par0 ^= nq_float_bits(t0);
        e0[j] = nq_sub(x[j], r0[j]);
        s0 = nq_fma(e0[j], e0[j], s0);
        m0 = fmaxf(m0, fabsf(e0[j]));
        const float y = nq_sub(x[j], 0.5f);
        const float t1 = nq_add(y, NQ_MAGIC);
        r1[j] = nq_sub(t1, NQ_MAGIC);
        if (LEAN) sum1 = nq_add(sum1, r1[j]);
        else par1 ^= nq_float_bits(t1);
        e1[j] = nq_sub(y, r1[j]);
        s1 = nq_fma(e1[j], e1[j], s1);
        m1 = fmaxf(m1, fabsf(e1[j]));
    }
    if (LEAN) {
        par0 = nq_float_bits(nq_add(sum0, NQ_MAGIC));
        par1 = nq_float_bits(nq_add(sum1, NQ_MAGIC));
    }
    const bool odd0 = (par0 & 1) != 0, odd1 = (par1 & 1) != 0;
    if (odd0) s0 += 1.0f - 2.0f * m0;
    if (odd1) s1 += 1.0f - 2.0f * m1;
    const float diff = s0 - s1;
    bool integer_coset = diff < 0.0f;
    if (fabsf(diff) < 1e-4f) {
        // too close to call from the residuals: the reference's own comparison, i.e. both repaired
        // points and their sequentially summed distances (same roundings as nq_e8_nearest_exact)
        float d0 = 0.0f, d1 = 0.0f;
        bool pend0 = odd0, pend1 = odd1;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const bool hit0 = pend0 && fabsf(e0[j]) == m0;
            const bool hit1 = pend1 && fabsf(e1[j]) == m1;
            pend0 = pend0 && !hit0;
            pend1 = pend1 && !hit1;
            const float p0 = hit0 ? nq_add(r0[j], e0[j] >= 0.0f ? 1.0f : -1.0f) : r0[j];
            const float q1 = hit1 ? nq_add(r1[j], e1[j] >= 0.0f ? 1.0f : -1.0f) : r1[j];
            const float p1 = nq_add(q1, 0.5f);
            const float a = nq_sub(x[j], p0), b = nq_sub(x[j], p1);
            d0 = nq_add(d0, nq_mul(a, a));
            d1 = nq_add(d1, nq_mul(b, b));
        }
        integer_coset = d0 < d1;
    }
    const bool odd = integer_coset ? odd0 : odd1;
    const float m = integer_coset ? m0 : m1;
    const float half = integer_coset ? 0.0f : 0.5f;
    const float half_coset = integer_coset ? 0.0f : 1.0f;
    bool pending = odd;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float e = integer_coset ? e0[j] : e1[j];
        float r;
        if (LEAN) {
            // r0 or r1 + 1/2 without a select: (r1 + 1/2) - r0 is +-1/2 exactly, so the FMA is exact
            r = nq_fma(half_coset, nq_sub(nq_add(r1[j], 0.5f), r0[j]), r0[j]);
        } else {
            r = integer_coset ? r0[j] : r1[j];
        }
        const bool hit = pending && fabsf(e) == m;  // first coordinate reaching the maximum
        r += hit ? (e >= 0.0f ? 1.0f : -1.0f) : 0.0f;
        pending = pending && !hit;
        out[j] = LEAN ? r : r + half;
    }
}

// Exact int -> float for |v| < 2^22 without the (slow) conversion unit: the
// integer is added into the mantissa of the magic constant.
NQ_HD float nq_small_int_to_float(int v) {
    return nq_sub(nq_bits_float(0x4B400000u + (uint32_t)v), NQ_MAGIC);
}

// coset representative G*c of integer coordinates c (codec.py:30-43).
NQ_HD void nq_generator_apply(const int c[8], float t[8]) {
    const float h = 0.5f * nq_small_int_to_float(c[7]);
    t[0] = nq_small_int_to_float(2 * c[0] - c[1]) + h;
#pragma unroll
    for (int j = 1; j < 6; ++j) t[j] = nq_small_int_to_float(c[j] - c[j + 1]) + h;
    t[6] = nq_small_int_to_float(c[6]) + h;
    t[7] = h;
}

// Coset representative G*c of a packed codeword with few integer instructions: the nibbles are
// split into even / odd bytes, the differences c_j - c_{j+1} are formed four at a time in one
// 32-bit subtraction (every byte biased by 16, so no borrow crosses a byte), and each byte is
// dropped into the mantissa of 1.5 * 2^23 to become a float without a conversion instruction.
NQ_HD float nq_mantissa_byte(uint32_t bytes, int index) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(__byte_perm(bytes, 0x4B400000u, 0x7650u | (uint32_t)index));
#else
    return nq_bits_float(0x4B400000u | ((bytes >> (8 * index)) & 0xffu));
#endif
}
NQ_HD void nq_codeword_coset_packed(uint32_t word, float t[8]) {
    const uint32_t even = word & 0x0F0F0F0Fu;          // c0 c2 c4 c6
    const uint32_t odd = (word >> 4) & 0x0F0F0F0Fu;    // c1 c3 c5 c7
    const uint32_t odd3 = odd & 0x00FFFFFFu;           // c1 c3 c5 0
    const uint32_t a = even + 0x10101010u - odd3;      // c0-c1, c2-c3, c4-c5, c6      (+16 each)
    const uint32_t b = odd3 + 0x00101010u - (even >> 8);  // c1-c2, c3-c4, c5-c6, 0    (+16 each)
    const float bias = NQ_MAGIC + 16.0f;
    const float h = 0.5f * nq_sub(nq_mantissa_byte(odd, 3), NQ_MAGIC);
    const float c0 = nq_sub(nq_mantissa_byte(even, 0), NQ_MAGIC);
    t[0] = nq_add(nq_add(nq_sub(nq_mantissa_byte(a, 0), bias), c0), h);
    t[1] = nq_add(nq_sub(nq_mantissa_byte(b, 0), bias), h);
    t[2] = nq_add(nq_sub(nq_mantissa_byte(a, 1), bias), h);
    t[3] = nq_add(nq_sub(nq_mantissa_byte(b, 1), bias), h);
    t[4] = nq_add(nq_sub(nq_mantissa_byte(a, 2), bias), h);
    t[5] = nq_add(nq_sub(nq_mantissa_byte(b, 2), bias), h);
    t[6] = nq_add(nq_sub(nq_mantissa_byte(a, 3), bias), h);
    t[7] = h;
}

// Same from a packed codeword (coordinate j in bits [4j, 4j+3]).
NQ_HD void nq_codeword_coset(uint32_t word, float t[8]) { nq_codeword_coset_packed(word, t); }

// Integer coordinates of a lattice point, reduced modulo q, as a codeword.
// All intermediate values are exact small integers in float32.
NQ_HD uint32_t nq_lattice_to_codeword(const float l[8]) {
    float c[8];
    c[7] = 2.0f * l[7];
    c[6] = l[6] - l[7];
    c[5] = l[5] + c[6] - l[7];
    c[4] = l[4] + c[5] - l[7];
    c[3] = l[3] + c[4] - l[7];
    c[2] = l[2] + c[3] - l[7];
    c[1] = l[1] + c[2] - l[7];
    c[0] = 0.5f * (l[0] + c[1] - l[7]);
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        // c is an exact integer with |c| < 2^22: it can be read back from the
        // mantissa of (c + magic) without a float->int conversion.
        const int v = (nq_float_bits(nq_add(c[j], NQ_MAGIC)) & 0x7fffff) - 0x400000;
        int m = v % NQ_Q;
        m += (m < 0) ? NQ_Q : 0;
        word |= (uint32_t)m << (4 * j);
    }
    return word;
}

// Minimum-energy representative of the coset of `word`:  t - q*Q(t/q), with
// the optional dither subtracted first (weights).  Exact reference order.
NQ_HD void nq_decode_codeword_exact(uint32_t word, const float* dither, float r[8]) {
    float t[8], s[8], n[8];
    nq_codeword_coset(word, t);
    if (dither) {
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = nq_sub(t[j], dither[j]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j] = nq_div_by(t[j], 14.0f, NQ_RCP14);
    nq_e8_nearest_guarded(s, n);  // same result as the exact search
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = nq_fma(-14.0f, n[j], t[j]);  // 14*n is exact, so one rounding either way
}

// t / 14 for the coset coordinates of an undithered codeword (half-integers in [-13, 32.5]):
// one residual correction of t * RN(1/14) already is the correctly rounded quotient for every
// such value (checked exhaustively by the host test-suite), 3 instructions instead of 5.
NQ_HD float nq_div14_coset(float t) {
    const float q0 = nq_mul(t, NQ_RCP14);
    return nq_fma(nq_fma(-14.0f, q0, t), NQ_RCP14, q0);
}

// Minimum-energy representative of an UNDITHERED codeword (activations, K/V pages): the same
// result as nq_decode_codeword_exact(word, nullptr, r) for every one of the 14^8 codewords
// (checked exhaustively on the host) with the packed coset build and the short exact division.
// About 2 % of real K/V blocks sit exactly between the two cosets (a true tie that the
// reference resolves through the rounding of its sequential sums), so the guarded search keeps
// its roundings at hand for that comparison rather than calling out of line: with 32 blocks
// per warp step nearly every other step meets one.
NQ_HD void nq_decode_codeword_undithered(uint32_t word, float r[8]) {
    float t[8], s[8], n[8];
    nq_codeword_coset_packed(word, t);
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j] = nq_div14_coset(t[j]);
    nq_e8_nearest_guarded(s, n);
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = nq_fma(-14.0f, n[j], t[j]);
}

// ------------------------------------------------- table-driven decode ------
//
// The decode of an UNDITHERED codeword only ever sees 92 different coordinate values: the
// doubled coset coordinates T = 2t are integers in [-26, 65].  Everything the search derives
// from one coordinate -- the two roundings, their residuals, the rounding parities -- is a
// function of T alone, so it is tabulated once and a block becomes eight table reads plus a
// few integer operations on packed fields:
//
//   R0 = T - 28*round(t/14), R1 = T - 14 - 28*round(t/14 - 1/2)   residuals in units of 1/28
//                                                                  (|R1| = 14 - |R0| always)
//   integer-coset distance minus half-coset distance, in units of 28/784:
//       delta = sum|R0| - 56 + odd0*(28 - 2*max|R0|) - odd1*(28 - 2*max|R1|)
//   delta != 0 decides the coset (the float32 sums of the reference differ by >= 0.0357 then);
//   delta == 0 is a true tie of the two cosets, which the reference resolves through the
//   rounding of its sequential float32 sums: those sums are reproduced from tabulated squares.
//
// The parity repair moves the FIRST coordinate with the largest |residual| in float32.  For
// different |R| that order is the order of |R|; coordinates with equal |R| but different T
// differ by rounding noise, so the table carries the rank of the float32 value among the
// entries of equal |R| ("sub").  Ordering key of coordinate j: |R| : sub : (7 - j).
//
// Entry (two 32-bit words):
//   k: [31:28] |R0|  [27:25] sub0  [24:22] 0 (7-j goes here)  [18] parity1  [17] parity0  [16] e0<0
//      [15:12] |R1|  [11: 9] sub1  [ 8: 6] 0 (7-j)            [0] e1<0
//   o: bf16(R0/2) << 16 | bf16(R1/2)        the decoded coordinate for either coset (exact)
// Tie entry: squares of (s - p) for {integer, integer repaired, half, half repaired}.
// The table spans T in [-30, 75], the range of ANY 32-bit word (nibbles up to 15), so that a
// stray word can never index outside it; codewords proper only reach [-26, 65].
#define NQ_LUT_ENTRIES 106
#define NQ_LUT_BIAS 30

struct NqLutCoord {
    float e0, e1;      // residuals of the two roundings as the reference computes them
    int r0_twice14;    // R0, R1
    int r1_twice14;
    int par0, par1;    // parity of the rounded values
    float q[4];        // squared distances: integer coset, repaired; half coset, repaired
};

NQ_HD void nq_lut_coordinate(int twice_t, NqLutCoord& c) {
    const float t = 0.5f * nq_small_int_to_float(twice_t);
    const float s = nq_div14_coset(t);
    const float t0 = nq_add(s, NQ_MAGIC);
    const float r0 = nq_sub(t0, NQ_MAGIC);
    c.par0 = nq_float_bits(t0) & 1;
    c.e0 = nq_sub(s, r0);
    const float y = nq_sub(s, 0.5f);
    const float t1 = nq_add(y, NQ_MAGIC);
    const float r1 = nq_sub(t1, NQ_MAGIC);
    c.par1 = nq_float_bits(t1) & 1;
    c.e1 = nq_sub(y, r1);
    const int ir0 = (nq_float_bits(t0) & 0x7fffff) - 0x400000, ir1 = (nq_float_bits(t1) & 0x7fffff) - 0x400000;
    c.r0_twice14 = twice_t - 28 * ir0;
    c.r1_twice14 = twice_t - 14 - 28 * ir1;
    const float d0 = nq_sub(s, r0);
    const float d0f = nq_sub(s, nq_add(r0, c.e0 >= 0.0f ? 1.0f : -1.0f));
    const float d1 = nq_sub(s, nq_add(r1, 0.5f));
    const float d1f = nq_sub(s, nq_add(nq_add(r1, c.e1 >= 0.0f ? 1.0f : -1.0f), 0.5f));
    c.q[0] = nq_mul(d0, d0);
    c.q[1] = nq_mul(d0f, d0f);
    c.q[2] = nq_mul(d1, d1);
    c.q[3] = nq_mul(d1f, d1f);
}

// Packs entry `index` from the coordinates of all entries (`all`, NQ_LUT_ENTRIES of them).
NQ_HD void nq_lut_pack(const NqLutCoord* all, int index, uint32_t& k, uint32_t& o) {
    const NqLutCoord& c = all[index];
    const int a0 = c.r0_twice14 < 0 ? -c.r0_twice14 : c.r0_twice14;
    const int a1 = c.r1_twice14 < 0 ? -c.r1_twice14 : c.r1_twice14;
    int sub0 = 0, sub1 = 0;
    for (int i = 0; i < NQ_LUT_ENTRIES; ++i) {
        const int b0 = all[i].r0_twice14 < 0 ? -all[i].r0_twice14 : all[i].r0_twice14;
        const int b1 = all[i].r1_twice14 < 0 ? -all[i].r1_twice14 : all[i].r1_twice14;
        sub0 += (b0 == a0 && fabsf(all[i].e0) < fabsf(c.e0)) ? 1 : 0;
        sub1 += (b1 == a1 && fabsf(all[i].e1) < fabsf(c.e1)) ? 1 : 0;
    }
    k = ((uint32_t)a0 << 28) | ((uint32_t)(sub0 & 7) << 25) | ((uint32_t)c.par1 << 18) | ((uint32_t)c.par0 << 17) |
        ((c.e0 < 0.0f ? 1u : 0u) << 16) | ((uint32_t)a1 << 12) | ((uint32_t)(sub1 & 7) << 9) | (c.e1 < 0.0f ? 1u : 0u);
    o = (nq_bf16_bits(0.5f * nq_small_int_to_float(c.r0_twice14)) << 16) |
        nq_bf16_bits(0.5f * nq_small_int_to_float(c.r1_twice14));
}

// Table indices (T + NQ_LUT_BIAS) of the eight coordinates of a codeword, four per word: `ia` holds
// coordinates 0, 2, 4, 6 and `ib` coordinates 1, 3, 5, 7 (byte i = coordinate 2i / 2i + 1).
NQ_HD void nq_lut_indices(uint32_t word, uint32_t& ia, uint32_t& ib) {
    const uint32_t even = word & 0x0F0F0F0Fu;              // c0 c2 c4 c6
    const uint32_t odd3 = (word >> 4) & 0x000F0F0Fu;       // c1 c3 c5 0
    const uint32_t a = even + 0x10101010u - odd3;          // c0-c1, c2-c3, c4-c5, c6     (+16 each)
    const uint32_t b = odd3 + 0x10101010u - (even >> 8);   // c1-c2, c3-c4, c5-c6, 0      (+16 each)
    const uint32_t x = (word >> 28) * 0x01010101u - 0x02020202u;  // c7 - 32 + 30 in every byte (no byte of a sum underflows)
    ia = 2u * a + x + 2u * (word & 0xFu);
    ib = 2u * b + x;
}

NQ_HD uint32_t nq_max_u16x2(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
    return __vmaxu2(a, b);
#else
    const uint32_t lo = (a & 0xffffu) > (b & 0xffffu) ? (a & 0xffffu) : (b & 0xffffu);
    const uint32_t hi = (a >> 16) > (b >> 16) ? (a >> 16) : (b >> 16);
    return (hi << 16) | lo;
#endif
}
NQ_HD uint32_t nq_max3_u16x2(uint32_t a, uint32_t b, uint32_t c) {
#if defined(__CUDA_ARCH__) && __CUDA_ARCH__ >= 900
    return __vimax3_u16x2(a, b, c);
#else
    return nq_max_u16x2(nq_max_u16x2(a, b), c);
#endif
}

// Decode of an undithered codeword from the table, in three phases so that a caller can interleave
// the straight-line parts of several blocks around the (rare, divergent) tie resolution:
//   nq_lut_begin        eight table reads, the integer decision;  blk.delta < 0: integer coset,
//                       > 0: half coset, == 0: the two cosets are equally far
//   nq_lut_resolve_tie  only for delta == 0: the reference's sequential float32 sums decide
//   nq_lut_finish       the eight decoded coordinates of the chosen coset, parity repair applied
// fetch(packed, i, k, o) reads the entry whose index is byte i of `packed`; tie(packed, i, q) reads
// the four squares of that entry.
struct NqLutBlock {
    uint32_t o[8];       // bf16 pair (integer coset, half coset) of every coordinate
    uint32_t m;          // largest ordering key of the integer coset (upper half) and of the half coset (lower half)
    uint32_t ia, ib;     // table indices, kept for the tie path
    int delta;
    uint32_t odd;        // bit 0: the integer coset needs the parity repair, bit 1: the half coset does
};

template <class Fetch>
NQ_HD void nq_lut_begin(uint32_t word, Fetch&& fetch, NqLutBlock& blk) {
    uint32_t k[8];
    nq_lut_indices(word, blk.ia, blk.ib);
#pragma unroll
    for (int j = 0; j < 8; ++j) fetch((j & 1) ? blk.ib : blk.ia, j >> 1, k[j], blk.o[j]);
    uint32_t asum = 0, x = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#if defined(__CUDA_ARCH__)
        asum = __umulhi(k[j], 16u) + asum;
#else
        asum += k[j] >> 28;
#endif
        x ^= k[j];
    }
    blk.odd = (x >> 17) & 3u;
    blk.m = nq_max3_u16x2(
        nq_max3_u16x2(k[0] | 0x01C001C0u, k[1] | 0x01800180u, k[2] | 0x01400140u),
        nq_max3_u16x2(k[3] | 0x01000100u, k[4] | 0x00C000C0u, k[5] | 0x00800080u),
        nq_max_u16x2(k[6] | 0x00400040u, k[7]));
    const int rmax0 = (int)(blk.m >> 28), rmax1 = (int)((blk.m >> 12) & 15u);
    blk.delta = (int)asum - 56 + ((blk.odd & 1u) ? 28 - 2 * rmax0 : 0) - ((blk.odd & 2u) ? 28 - 2 * rmax1 : 0);
}

template <class Tie>
NQ_HD bool nq_lut_resolve_tie(const NqLutBlock& blk, Tie&& tie) {
    const int fix0 = (blk.odd & 1u) ? 7 - (int)((blk.m >> 22) & 7u) : -1;
    const int fix1 = (blk.odd & 2u) ? 7 - (int)((blk.m >> 6) & 7u) : -1;
    float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float q[4];
        tie((j & 1) ? blk.ib : blk.ia, j >> 1, q);
        s0 = nq_add(s0, j == fix0 ? q[1] : q[0]);
        s1 = nq_add(s1, j == fix1 ? q[3] : q[2]);
    }
    return s0 < s1;
}

NQ_HD void nq_lut_finish(const NqLutBlock& blk, bool integer_coset, float r[8]) {
    const uint32_t key = integer_coset ? (blk.m >> 16) : (blk.m & 0xffffu);
    const bool odd = ((integer_coset ? blk.odd : (blk.odd >> 1)) & 1u) != 0;
#if defined(__CUDA_ARCH__)
    const uint32_t pick = integer_coset ? 0x3244u : 0x1044u;  // byte selector: the chosen bf16 into the upper half
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = __uint_as_float(__byte_perm(blk.o[j], 0u, pick));
#else
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = nq_bits_float(integer_coset ? (blk.o[j] & 0xffff0000u) : (blk.o[j] << 16));
#endif
    // parity repair; residual e < 0: the rounded value moves down by one, the decoded coordinate up by 14
    const int fix = odd ? 7 - (int)((key >> 6) & 7u) : -1;
    const float by = (key & 1u) ? 14.0f : -14.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = (j == fix) ? nq_add(r[j], by) : r[j];
}

// The three phases in one call: the same eight values as nq_decode_codeword_exact(word, nullptr, r)
// for every one of the 14^8 codewords (checked on the host).
template <class Fetch, class Tie>
NQ_HD void nq_decode_codeword_lut(uint32_t word, Fetch&& fetch, Tie&& tie, float r[8]) {
    NqLutBlock blk;
    nq_lut_begin(word, fetch, blk);
    bool integer_coset = blk.delta < 0;
    if (blk.delta == 0) integer_coset = nq_lut_resolve_tie(blk, tie);
    nq_lut_finish(blk, integer_coset, r);
}

// ------------------------------------------------------------ dither ------

// "lcg31_mix_v1" (codec.py:204-221): every stage reduced modulo 2^31.  Bit 31 of the intermediate
// values is left as garbage instead of being masked after every stage: a product's low 31 bits only
// depend on the low 31 bits of its factor, and the shifted copies are masked where they are folded
// in (one three-input logic operation), so bits 0..30 are those of the reference at every stage.
NQ_HD uint32_t nq_lcg31_mix(uint32_t counter_plus_seed) {
    uint32_t v = counter_plus_seed;
    v ^= (v >> 16) & 0x7fffu;
    v = v * 1103515245u + 12345u;
    v ^= (v >> 13) & 0x3ffffu;
    v = v * 134775813u + 1u;
    v ^= (v >> 16) & 0x7fffu;
    return v & 0x7fffffffu;
}

// Subtractive dither of one global block: u - Q(u), u uniform in [0,2)^8.
// `base` = (8*global_block + seed) mod 2^32 (only its low 31 bits matter).
NQ_HD void nq_dither_block(uint32_t base, float d[8]) {
    float u[8], n[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) u[j] = (float)nq_lcg31_mix(base + (uint32_t)j) * (2.0f / 2147483648.0f);
    nq_e8_nearest_exact(u, n);
#pragma unroll
    for (int j = 0; j < 8; ++j) d[j] = nq_sub(u[j], n[j]);
}

// Weight-path variants (continuous arguments): guarded nearest-point search.
NQ_HD void nq_dither_block_fast(uint32_t base, float d[8]) {
    float u[8], n[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) u[j] = (float)nq_lcg31_mix(base + (uint32_t)j) * (2.0f / 2147483648.0f);
    nq_e8_nearest_guarded(u, n);
#pragma unroll
    for (int j = 0; j < 8; ++j) d[j] = nq_sub(u[j], n[j]);
}

NQ_HD void nq_decode_weight_block(uint32_t word, uint32_t counter_base, float r[8]) {
    float d[8], t[8], s[8], n[8];
    nq_dither_block_fast(counter_base, d);
    nq_codeword_coset(word, t);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        t[j] = nq_sub(t[j], d[j]);
        s[j] = nq_div_by(t[j], 14.0f, NQ_RCP14);
    }
    nq_e8_nearest_guarded(s, n);
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = nq_fma(-14.0f, n[j], t[j]);  // 14*n is exact, so one rounding either way
}

// Position of a lattice point lam relative to the scaled Voronoi cell 14*V(E8):
// +1 strictly inside, -1 strictly outside, 0 on the boundary.  V(E8) is cut out
// by its 2400 relevant vectors (240 roots, 2160 vectors of norm 4); for each
// class the largest inner product with lam has a closed form in the sorted
// absolute coordinates.  All quantities are exact multiples of 1/4 in float32.
//   roots  (+-1,+-1,0^6)              a1+a2                      vs 14
//          (+-1/2)^8, even # minus    (S - [odd negatives]*2*amin)/2   vs 14
//   norm 4 (+-1)^4 on four coords     a1+a2+a3+a4                vs 28
//          (+-3/2,(+-1/2)^7), odd #   S/2 + a1 - [even negatives]*amin vs 28
//          (+-2,0^7)                  implied by the first row
// Strictly inside means t/14 reduces to lam itself with a margin of >= 0.0126 in
// distance, far above float32 rounding, so the re-decode can be skipped exactly.
NQ_HD int nq_e8_cell_class(const float lam[8]) {
    float a[8];
    float sum = 0.0f, amin = fabsf(lam[0]);
    int negatives = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        a[j] = fabsf(lam[j]);
        sum += a[j];
        amin = fminf(amin, a[j]);
        negatives ^= nq_float_bits(lam[j]) >> 31;  // sign bit; zeros force amin = 0, where parity is irrelevant
    }
    // four largest absolute values by partial selection
    float t1 = 0.0f, t2 = 0.0f, t3 = 0.0f, t4 = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float v = a[j];
        float hi = fmaxf(t1, v); v = fminf(t1, v); t1 = hi;
        hi = fmaxf(t2, v); v = fminf(t2, v); t2 = hi;
        hi = fmaxf(t3, v); v = fminf(t3, v); t3 = hi;
        t4 = fmaxf(t4, v);
    }
    const bool odd = (negatives & 1) != 0;
    const float c1 = t1 + t2;                                   // vs 14
    const float c2 = 0.5f * (sum - (odd ? 2.0f * amin : 0.0f)); // vs 14
    const float c3 = t1 + t2 + t3 + t4;                         // vs 28
    const float c4 = 0.5f * sum + t1 - (odd ? 0.0f : amin);     // vs 28
    const float m14 = fmaxf(c1, c2), m28 = fmaxf(c3, c4);
    if (m14 < 14.0f && m28 < 28.0f) return 1;
    if (m14 > 14.0f || m28 > 28.0f) return -1;
    return 0;
}

// One beta candidate evaluated exactly as the reference does (quantise,
// reduce modulo q, reconstruct, error).  Returns the codeword.
NQ_HD uint32_t nq_encode_candidate_exact(const float x[8], float beta, const float* dither, float r[8], float& err) {
    float y[8], lam[8];
    const float rbeta = nq_rcp(beta);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        y[j] = nq_div_by(x[j], beta, rbeta);
        if (dither) y[j] = nq_add(y[j], dither[j]);
    }
    nq_e8_nearest_exact(y, lam);
    const uint32_t word = nq_lattice_to_codeword(lam);
    nq_decode_codeword_exact(word, dither, r);
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = nq_mul(r[j], beta);
    err = nq_sqdist8_seq(r, x);
    return word;
}

// Undithered multi-beta search with exact pruning.  For every beta the
// lattice point lam and the error "as if lam were reproduced" are computed;
// then
//   * lam strictly inside 14*V: the reconstruction IS lam, the error is final;
//   * lam strictly outside: the reconstruction differs from lam by a vector of
//     14*E8 (norm >= 14*sqrt(2)), so its error is >= (14*sqrt(2)-1)^2 beta^2 >
//     353 beta^2 and it cannot beat a candidate whose error is below that;
//   * lam on the boundary, or nothing to prune against: full exact evaluation.
// The result (codeword, beta index, reconstruction) is identical to
// nq_encode_block for every input.
// First half of the pruned search: classifies the four candidates.  On return
// `best` (or -1) / best_err / best_lam describe the best candidate whose lattice
// point is strictly inside 14*V, and bit b of `pending` is set for every
// candidate that still needs the full evaluation (nq_encode_candidate_exact).
NQ_HD void nq_encode_block_fastpass(const float x[8], const float* beta, int& best, float& best_err,
                                    float best_lam[8], unsigned& pending) {
    best = -1;
    best_err = 0.0f;
    pending = 0;
    unsigned outside = 0;
    float asif[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const float bt = beta[b], rbeta = nq_rcp(bt);
        float y[8], lam[8], r[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = nq_div_by(x[j], bt, rbeta);
        nq_e8_nearest_guarded<true>(y, lam);
#pragma unroll
        for (int j = 0; j < 8; ++j) r[j] = nq_mul(lam[j], bt);
        asif[b] = nq_sqdist8_seq(r, x);
        // |lam|^2 <= 96 < (14/sqrt(2))^2 puts lam inside the inscribed ball of 14*V: no facet test needed
        float norm2 = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) norm2 = nq_fma(lam[j], lam[j], norm2);
        const int cls = norm2 <= 96.0f ? 1 : nq_e8_cell_class(lam);
        if (cls > 0) {
            if (best < 0 || asif[b] < best_err) {
                best = b;
                best_err = asif[b];
#pragma unroll
                for (int j = 0; j < 8; ++j) best_lam[j] = lam[j];
            }
        } else if (cls == 0) {
            pending |= 1u << b;
        } else {
            outside |= 1u << b;
        }
    }
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const float bt = beta[b];
        // an outside candidate's true error exceeds 353*beta^2; a boundary candidate's is >= its as-if error
        if ((outside >> b) & 1u) {
            if (!(best >= 0 && 353.0f * bt * bt > best_err)) pending |= 1u << b;
        } else if ((pending >> b) & 1u) {
            if (best >= 0 && asif[b] > best_err) pending &= ~(1u << b);
        }
    }
}

// Search key of a candidate: the rule "smallest error, first beta on ties" is the minimum of
// (error bits << 8 | beta index); errors are sums of squares, so their bit patterns order like the values.
NQ_HD unsigned long long nq_candidate_key(float err, int b) {
    return ((unsigned long long)(uint32_t)nq_float_bits(err) << 8) | (unsigned)b;
}

// Full evaluation of one candidate whose lattice point lam = Q(x / beta) is already known:
// codeword, reconstruction r (times beta) and error, bit-identical to nq_encode_candidate_exact.
// Used for lattice points on the boundary of 14*V(E8), where the reduction modulo 14*E8 meets
// exact ties -- the guarded search would fall back to the exact one anyway, so it is skipped.
NQ_HD uint32_t nq_eval_candidate_from_lam(const float x[8], const float lam[8], float beta, float r[8], float& err) {
    float t[8], s[8], n[8];
    const uint32_t word = nq_lattice_to_codeword(lam);
    nq_codeword_coset(word, t);
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j] = nq_div_by(t[j], 14.0f, NQ_RCP14);
    nq_e8_nearest_exact(s, n);
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = nq_mul(nq_fma(-14.0f, n[j], t[j]), beta);
    err = nq_sqdist8_seq(r, x);
    return word;
}

// Cheap exact classification of one candidate of the undithered search: the lattice point
// lam = Q(x / beta), the error "as if lam were reproduced" (the reference's sequential sum), and
// the position of lam relative to 14*V(E8): +1 strictly inside (the reconstruction IS lam and
// asif is the candidate's error), 0 on the boundary (error >= asif), -1 strictly outside
// (error > 353 beta^2).
NQ_HD int nq_classify_candidate(const float x[8], float bt, float lam[8], float& asif) {
    const float rbeta = nq_rcp(bt);
    float y[8], r[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = nq_div_by(x[j], bt, rbeta);
    nq_e8_nearest_guarded<true>(y, lam);
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = nq_mul(lam[j], bt);
    asif = nq_sqdist8_seq(r, x);
    // |lam|^2 <= 96 < (14/sqrt(2))^2 puts lam inside the inscribed ball of 14*V: no facet test needed
    float norm2 = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) norm2 = nq_fma(lam[j], lam[j], norm2);
    return norm2 <= 96.0f ? 1 : nq_e8_cell_class(lam);
}

// Variant of nq_encode_block_fastpass for a caller with a work queue: every candidate whose
// lattice point lies ON the boundary of 14*V(E8) is handed to on_boundary(b, lam) as soon as it
// is found (unless a better finished candidate already rules it out), the caller evaluates it
// with nq_eval_candidate_from_lam and merges by key.  `pending` only holds the rare candidates
// strictly outside the cell that no finished candidate rules out; those take the generic
// nq_encode_candidate_exact.  best / best_err / best_lam: best candidate strictly inside, or -1.
template <class OnBoundary>
NQ_HD void nq_encode_block_fastpass_push(const float x[8], const float* beta, int& best, float& best_err,
                                         float best_lam[8], unsigned& pending, OnBoundary&& on_boundary) {
    best = -1;
    best_err = 0.0f;
    pending = 0;
    unsigned outside = 0;
    // One copy of the candidate body (the loop is kept rolled): laid out four times the search
    // stalls on instruction fetch.
#pragma unroll 1
    for (int b = 0; b < 4; ++b) {
        float lam[8], asif;
        const int cls = nq_classify_candidate(x, beta[b], lam, asif);
        if (cls > 0) {
            if (best < 0 || asif < best_err) {
                best = b;
                best_err = asif;
#pragma unroll
                for (int j = 0; j < 8; ++j) best_lam[j] = lam[j];
            }
        } else if (cls == 0) {
            // its error is at least the as-if error: an earlier finished candidate below that wins anyway
            if (!(best >= 0 && asif > best_err)) on_boundary(b, lam);
        } else {
            outside |= 1u << b;
        }
    }
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const float bt = beta[b];
        // an outside candidate's true error exceeds 353*beta^2
        if (((outside >> b) & 1u) && !(best >= 0 && 353.0f * bt * bt > best_err)) pending |= 1u << b;
    }
}

// Merge rule of the search: smaller error wins, equal errors go to the smaller beta index.
NQ_HD bool nq_candidate_wins(int b, float err, int best, float best_err) {
    return best < 0 || err < best_err || (err == best_err && b < best);
}

NQ_HD uint32_t nq_encode_block_pruned(const float x[8], const float* beta, int& beta_id, float recon[8]) {
    float best_err, best_lam[8];
    int best;
    unsigned pending;
    nq_encode_block_fastpass(x, beta, best, best_err, best_lam, pending);
    uint32_t best_word = 0;
    bool have_word = false;
    if (pending) {
#pragma unroll 1
        for (int b = 0; b < 4; ++b) {
            if (!((pending >> b) & 1u)) continue;
            float r[8], err;
            const uint32_t word = nq_encode_candidate_exact(x, beta[b], nullptr, r, err);
            if (nq_candidate_wins(b, err, best, best_err)) {
                best = b;
                best_err = err;
                best_word = word;
                have_word = true;
#pragma unroll
                for (int j = 0; j < 8; ++j) recon[j] = r[j];
            }
        }
    }
    beta_id = best;
    if (!have_word) {
        best_word = nq_lattice_to_codeword(best_lam);
        const float bt = beta[best];
#pragma unroll
        for (int j = 0; j < 8; ++j) recon[j] = nq_mul(best_lam[j], bt);
    }
    return best_word;
}

// ----------------------------------------------------------- encoder ------

// Multi-beta search for one normalised block x (quantizer.py:275-283): for
// each beta in table order quantise x/beta (+dither), reconstruct, and keep
// the FIRST beta with the smallest sequentially-summed squared error.
// Returns the codeword; writes the beta index and the chosen reconstruction
// (normalised domain, already multiplied by beta).
NQ_HD uint32_t nq_encode_block(const float x[8], const float* beta, const float* dither,
                               int& beta_id, float recon[8]) {
    float best_err = 0.0f;
    uint32_t best_word = 0;
    beta_id = -1;
#pragma unroll 1
    for (int b = 0; b < 4; ++b) {
        float y[8], lam[8], r[8];
        const float rbeta = nq_rcp(beta[b]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            y[j] = nq_div_by(x[j], beta[b], rbeta);
            if (dither) y[j] = nq_add(y[j], dither[j]);
        }
        nq_e8_nearest_exact(y, lam);
        const uint32_t word = nq_lattice_to_codeword(lam);
        nq_decode_codeword_exact(word, dither, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) r[j] = nq_mul(r[j], beta[b]);
        const float err = nq_sqdist8_seq(r, x);
        if (beta_id < 0 || err < best_err) {
            best_err = err;
            best_word = word;
            beta_id = b;
#pragma unroll
            for (int j = 0; j < 8; ++j) recon[j] = r[j];
        }
    }
    return best_word;
}
