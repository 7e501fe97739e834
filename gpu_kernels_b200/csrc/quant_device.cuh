// Device-side pieces of the NVFP4 quantiser shared by the stand-alone quantise kernel and the
// fused SwiGLU + re-quantise kernel of the expert path: E4M3 scale rounding, the block routine
// (amax -> scale -> sixteen exact quotients -> E2M1 codes) and the scale-atom addressing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace nvfp4_b200 {

// Byte offset of the scale of (row, 16-wide K block) in the VEC16 layout
// (closed form pinned by the reference's tests/test_nvfp4.py:25-26).
__host__ __device__ __forceinline__ size_t scale_byte_offset(int row, int kblock, int K) {
    return (size_t(row / 128) * (K / 64) + kblock / 4) * 512 + (row % 32) * 16 + ((row % 128) / 32) * 4 + kblock % 4;
}

// E4M3 byte of t, t already clamped to [2^-9, 448]; nearest-even in both the
// normal range (3 mantissa bits) and the subnormal range (step 2^-9).
__device__ __forceinline__ uint32_t ue4m3_from_float(float t) {
    if (t < 0.015625f) return static_cast<uint32_t>(__float2int_rn(t * 512.0f));
    const uint32_t b = __float_as_uint(t);
    return ((b + 0x7FFFFu + ((b >> 20) & 1u)) >> 20) - (120u << 3);
}

__device__ __forceinline__ float ue4m3_to_float(uint32_t code) {
    if (code < 8u) return static_cast<float>(code) * 0.001953125f;
    return __uint_as_float((((code >> 3) + 120u) << 23) | ((code & 7u) << 20));
}

// Four bytes of packed E2M1 from eight non-negative quotients (element 0 in the low nibble of
// byte 0). The hardware conversion rounds to nearest with ties to the even code and saturates at
// 6, which is the reference's midpoint rule (reference/python/nvfp4.py:8-13); signs are added by
// the caller because the reference's sign bit is (q < 0), not the sign of the input.
// The conversion is slow (its pipe was the busiest unit when 16-bit inputs still came this way);
// it remains for FP32 inputs, which have twice the bytes per value to hide it behind.
__device__ __forceinline__ uint32_t e2m1x8_from_quotients(const float (&q)[8]) {
    uint32_t w;
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
        "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
        : "=r"(w)
        : "f"(q[0]), "f"(q[1]), "f"(q[2]), "f"(q[3]), "f"(q[4]), "f"(q[5]), "f"(q[6]), "f"(q[7]));
    return w;
}

// One 16-value block: returns the scale byte, writes the 8 packed bytes.
//
// The reference divides every value by the block scale with an IEEE division. Sixteen
// `__fdiv_rn` per block made this kernel compute-bound at a quarter of HBM speed, so the
// division is done as one correctly rounded reciprocal per block and, per value, a product plus
// one residual correction: q0 = x*r, e = fma(-q0, s, x), q = fma(e, r, q0). With r = RN(1/s) this
// is the correctly rounded quotient RN(x/s) for every value whose quotient is a normal number
// (Markstein's division theorem; s has a 4-bit significand, far from the one excluded divisor),
// i.e. the same bits as the division. Quotients so small that they
// leave the normal range encode as 0 whatever their last bit is; the only thing that depends on
// them is the sign bit of a negative value whose quotient rounds to zero, which needs |x| below
// 2^-141 and is sent through the real division (FP32 input only: no bf16 or fp16 value is that
// small).
template <bool TINY_POSSIBLE>
__device__ __forceinline__ uint32_t quantise_block(const float (&v)[16], uint2& packed) {
    uint32_t mx = 0;
    #pragma unroll
    for (int i = 0; i < 16; ++i) mx = max(mx, __float_as_uint(v[i]) & 0x7FFFFFFFu);
    if (mx > 0x7F800000u) {
        // A NaN poisons the block exactly as it does in the reference: NaN scale
        // byte, and every element compares above all midpoints with sign 0.
        packed = make_uint2(0x77777777u, 0x77777777u);
        return 0x7Fu;
    }
    const float amax = __uint_as_float(mx);
    const float t = fminf(fmaxf(__fdiv_rn(amax, 6.0f), 0.001953125f), 448.0f);
    const uint32_t sbyte = ue4m3_from_float(t);
    const float s = ue4m3_to_float(sbyte);
    const float r = __frcp_rn(s);
    // Magnitudes are clamped to 8 * s: everything above 5 * s encodes as 6 anyway, and the clamp
    // keeps the product finite when the scale saturated at 448 or sits in the E4M3 subnormals.
    const float limit = 8.0f * s;
    uint32_t words[2];
    #pragma unroll
    for (int h = 0; h < 2; ++h) {
        float q[8];
        uint32_t signs = 0;
        #pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float x = v[8 * h + i];
            const float ax = fminf(fabsf(x), limit);
            const float q0 = __fmul_rn(ax, r);
            const float e = __fmaf_rn(-q0, s, ax);
            q[i] = __fmaf_rn(e, r, q0);
            bool negative = x < 0.0f;
            if (TINY_POSSIBLE && ax < 1e-42f) negative = negative && __fdiv_rn(ax, s) != 0.0f;
            signs |= negative ? (8u << (4 * i)) : 0u;
        }
        words[h] = e2m1x8_from_quotients(q) | signs;
    }
    packed = make_uint2(words[0], words[1]);
    return sbyte;
}

// silu(x) = x / (1 + e^-x) with the hardware exponential and reciprocal (a few ulp of FP32). The
// result is multiplied and then rounded to bf16 (8 significant bits) before it is quantised, so the
// approximation almost never survives the rounding; the exact expf + IEEE division cost ten times the
// instructions and made the fused FC1 epilogue the bottleneck of compute-dense expert GEMMs.
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// ---- 16-bit inputs: two values per instruction, no division -----------------------------------
//
// For a bf16 or fp16 input the E2M1 code of x/s can be read off x itself: RN(x/s) lies above,
// on or below a midpoint m exactly when |x| lies above, on or below m*s, and m*s is an exact
// number with at most 7 significant bits (m has 3, an E4M3 scale 4), i.e. representable in the
// input's own 16-bit format. The code is the number of the seven midpoints (.25, .75, 1.25, 1.75,
// 2.5, 3.5, 5) that |x| passes, where a tie passes the midpoints whose even neighbour lies above
// (.75, 1.75, 3.5: compared with >=) and not the others (>): reference/python/nvfp4.py:8-13.
// Seven compares per pair made the integer/logic pipe the limit of the kernel (74 % busy at 41 % of
// the DRAM bandwidth), so the count is taken as a three-step binary search whose thresholds are
// selected arithmetically on the FMA pipe:
//   c3 = |x| >= 1.75 s                                        (code bit 2)
//   c2 = |x| >= .75 s + c3 * 2.75 s                           (.75 s or 3.5 s: both ties go up)
//   c1 = |x| >  (.25 s + c2 * s) + c3 * (2.25 s + c2 * 1.5 s) (.25, 1.25, 2.5 or 5 s: all ties go down)
// Every product and sum above is an exact number of at most 8 significant bits (the multipliers have
// at most 4, the scale 4), so each fused multiply-add returns the exact threshold, in bf16 as in
// fp16. The code 4 c3 + 2 c2 + c1 is accumulated on top of a constant whose ulp is 1 (128 in bf16,
// 1024 in fp16), so the low byte of the sum's bit pattern is the code; the sign bit (x < 0, false
// for -0.0 as in the reference, where q = -0.0 is not < 0) is added as 8.
// No value of these formats is small enough for a non-zero quotient to round to zero.
struct Bf16Pairs {
    using pair = __nv_bfloat162;
    static constexpr uint32_t INF_BITS = 0x7F80u;
    static __device__ __forceinline__ pair from_bits(uint32_t w) { return *reinterpret_cast<const pair*>(&w); }
    static __device__ __forceinline__ uint32_t bits(pair p) { return *reinterpret_cast<const uint32_t*>(&p); }
    static __device__ __forceinline__ pair both(float v) { return __float2bfloat162_rn(v); }
    static __device__ __forceinline__ float widen(uint32_t bits16) { return __uint_as_float(bits16 << 16); }
    static __device__ __forceinline__ float count_base() { return 128.0f; }
};
struct Fp16Pairs {
    using pair = __half2;
    static constexpr uint32_t INF_BITS = 0x7C00u;
    static __device__ __forceinline__ pair from_bits(uint32_t w) { return *reinterpret_cast<const pair*>(&w); }
    static __device__ __forceinline__ uint32_t bits(pair p) { return *reinterpret_cast<const uint32_t*>(&p); }
    static __device__ __forceinline__ pair both(float v) { return __float2half2_rn(v); }
    static __device__ __forceinline__ float widen(uint32_t bits16) { return __half2float(__ushort_as_half(static_cast<unsigned short>(bits16))); }
    static __device__ __forceinline__ float count_base() { return 1024.0f; }
};

// w[k] holds values 2k (low half) and 2k+1 (high half) of the block as raw 16-bit patterns.
template <typename F>
__device__ __forceinline__ uint32_t quantise_block_pairs(const uint32_t (&w)[8], uint2& packed) {
    using pair = typename F::pair;
    uint32_t a[8];
    #pragma unroll
    for (int k = 0; k < 8; ++k) a[k] = F::bits(__habs2(F::from_bits(w[k])));   // folds into the users' operand modifiers
    // magnitudes of these formats order like their bit patterns
    uint32_t m = __vimax3_u16x2(__vimax3_u16x2(a[0], a[1], a[2]), __vimax3_u16x2(a[3], a[4], a[5]), __vimax3_u16x2(a[6], a[7], a[7]));
    const uint32_t top = max(m & 0xFFFFu, m >> 16);
    if (top > F::INF_BITS) {
        packed = make_uint2(0x77777777u, 0x77777777u);       // NaN block, as quantise_block
        return 0x7Fu;
    }
    const float amax = F::widen(top);
    // amax / 6, correctly rounded, without the division: reciprocal constant plus one residual step
    const float sixth = 0.16666667163372039794921875f;       // RN(1/6)
    const float d0 = __fmul_rn(amax, sixth);
    const float de = __fmaf_rn(-d0, 6.0f, amax);
    const float t = fminf(fmaxf(__fmaf_rn(de, sixth, d0), 0.001953125f), 448.0f);
    const uint32_t sbyte = ue4m3_from_float(amax <= 3.0e38f ? t : 448.0f);
    const float s = ue4m3_to_float(sbyte);
    // one conversion of the scale, then exact 16-bit products (<= 7 significant bits each)
    const pair s2 = F::both(s);
    const pair t3 = __hmul2(s2, F::both(1.75f)), t1 = __hmul2(s2, F::both(0.75f)), d51 = __hmul2(s2, F::both(2.75f)),
               t0 = __hmul2(s2, F::both(0.25f)), d225 = __hmul2(s2, F::both(2.25f)), d150 = __hmul2(s2, F::both(1.5f));
    const pair base = F::both(F::count_base()), eight = F::both(8.0f), four = F::both(4.0f), two = F::both(2.0f),
               zero = F::both(0.0f);
    uint32_t n[8];
    #pragma unroll
    for (int k = 0; k < 8; ++k) {
        const pair mag = F::from_bits(a[k]);
        const pair c3 = __hge2(mag, t3);
        const pair c2 = __hge2(mag, __hfma2(c3, d51, t1));
        const pair c1 = __hgt2(mag, __hfma2(c3, __hfma2(c2, d150, d225), __hfma2(c2, s2, t0)));
        pair count = __hfma2(c3, four, base);
        count = __hfma2(c2, two, count);
        count = __hadd2(count, c1);
        count = __hfma2(__hlt2(F::from_bits(w[k]), zero), eight, count);
        n[k] = F::bits(count);                               // low byte of each half: the 4-bit code
    }
    // codes of values (2k, 2k+1) sit in bytes 0 and 2 of n[k]: gather four codes per word, fold the odd
    // ones into the high nibbles, gather the four finished bytes
    uint32_t out[2];
    #pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t x01 = __byte_perm(n[4 * h], n[4 * h + 1], 0x6420), x23 = __byte_perm(n[4 * h + 2], n[4 * h + 3], 0x6420);
        const uint32_t y01 = x01 | (x01 >> 4), y23 = x23 | (x23 >> 4);
        out[h] = __byte_perm(y01, y23, 0x6420);
    }
    packed = make_uint2(out[0], out[1]);
    return sbyte;
}

}  // namespace nvfp4_b200
