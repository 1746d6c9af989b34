// Integer scaling primitives shared by the RESCALE kernel, the fused convolution / matmul epilogues,
// the residual-add kernel and AVG_POOL2D.
#pragma once
#include <cstdint>

namespace tb200
{

// QuantUtil::apply_scale_32 (reference_model/src/quant_util.h:45-84).  `bad` is OR-ed with true when one of
// the reference's range checks (which it reports as REQUIRE failures) does not hold.
__host__ __device__ __forceinline__ int32_t apply_scale_32_dev(int32_t value, int32_t multiplier, int32_t shift,
                                                               bool double_round, bool& bad)
{
    bool b = (multiplier < 0) || (shift < 2) || (shift > 62);
    const int32_t s = shift < 2 ? 2 : (shift > 62 ? 62 : shift);    // keep the shifts below defined
    const int64_t half = (int64_t)1 << (s - 1);
    b |= ((int64_t)value < -half) || ((int64_t)value >= half);
    int64_t round = half;
    if (double_round && s > 31)
        round += (value >= 0) ? ((int64_t)1 << 30) : -((int64_t)1 << 30);
    int64_t result = (int64_t)value * (int64_t)multiplier + round;
    result >>= s;
    b |= (result < -((int64_t)1 << 31)) || (result >= ((int64_t)1 << 31));
    bad |= b;
    return (int32_t)result;
}

// QuantUtil::apply_scale_16 (reference_model/src/quant_util.h:86-108)
__host__ __device__ __forceinline__ int32_t apply_scale_16_dev(int64_t value, int16_t multiplier, int32_t shift,
                                                               bool& bad)
{
    bool b = (multiplier < 0) || (shift < 2) || (shift > 62);
    const int32_t s = shift < 2 ? 2 : (shift > 62 ? 62 : shift);
    const int64_t round = (int64_t)1 << (s - 1);
    int64_t result = value * (int64_t)multiplier + round;
    result >>= s;
    b |= (result < -((int64_t)1 << 31)) || (result >= ((int64_t)1 << 31));
    bad |= b;
    return (int32_t)result;
}

// QuantUtil::reciprocal_scale (reference_model/src/quant_util.h:32-43)
__host__ __device__ __forceinline__ void reciprocal_scale_dev(int32_t value, int32_t& multiplier, int32_t& shift)
{
    const uint32_t v = (uint32_t)value - 1u;
    int k = 0;
    while (k < 32 && (v >> k) != 0)
        k++;    // k = 32 - clz(value - 1)
    const int64_t numerator = (((int64_t)1 << 30) + 1) << k;
    multiplier = (int32_t)(numerator / value);
    shift      = 30 + k;
}

// value_extend64_impl (reference_model/src/ops/type_conversion.cpp:183-221) for 8/16/32-bit containers
__host__ __device__ __forceinline__ int64_t value_extend64_dev(int32_t val, int bits, bool is_unsigned)
{
    if (bits == 8)
        return is_unsigned ? (int64_t)(uint8_t)(val & 0xFF) : (int64_t)(int8_t)(val & 0xFF);
    if (bits == 16)
        return is_unsigned ? (int64_t)(uint16_t)(val & 0xFFFF) : (int64_t)(int16_t)(val & 0xFFFF);
    return is_unsigned ? (int64_t)(uint32_t)val : (int64_t)val;
}

// ---------------------------------------------------------------------------------------------------------------
// Lean form of apply_scale_32 + output zero point for the tensor-core epilogue (int8 outputs).
//
// QuantUtil::apply_scale_32 (reference_model/src/quant_util.h:45-84) computes (v * m + round) >> shift with
// round = 2^(shift-1), plus or minus 2^30 by the sign of v under double rounding when shift > 31.  Here every column
// gets one record, built once from its constants, so that the per-element work is two multiply-adds and two shifts:
//
//     s  = acc * pk + cpk          (32-bit; pk a power of two, cpk = correction * pk: the zero-point / bias term rides
//                                   on the pre-scale; wraps mod 2^32, the true value fits)
//     P  = s * m + R               (64-bit)
//     z  = (hi(P) + (FIX ? s >> 31 : 0)) >> sh          FIX = the RESCALE's double_round attribute, one per layer
//
//   shift >= 32: pk = 2, sh = shift - 31, R = 2^shift + DR * 2^31 + out_zp * 2^(shift+1): everything is doubled, which
//                makes the two rounding constants of double rounding differ by exactly 2^32, i.e. by one in the high
//                word and nothing in the low word, so the sign-dependent choice is the "+ (s >> 31)" above;
//   shift <= 31: pk = 2^(32-shift), sh = 0, R = 2^31 + out_zp * 2^32: the product is aligned to the high word.  No
//                double rounding exists below shift 32, but a layer with double_round applies the sign term to every
//                column (it is one instruction when unconditional, three when selected per column), so such a column
//                is kept non-negative instead: cpk carries an extra B = 2^30 and R an extra -B * m, which cancel in P
//                and make s > 0 whenever |t| * pk < 2^30.
// out_zp added before the shift by its full weight comes out as exactly out_zp after it.  z still has to be saturated
// to int8 (cvt.pack.sat does it).  The form is exact when t = acc + correction satisfies |t| < 2^30 for shift >= 32,
// |t| < 2^(shift-1) for shift <= 31 without double_round (apply_scale_32's own REQUIRE, so that can never fail either)
// and |t| < 2^(shift-2) for shift <= 31 with it; `vmax`, the largest magnitude t can take for this column given the
// layer's K and its bias, proves that statically or the record is marked unusable (word 7 = 0) and the block takes
// the general epilogue.
// Record words: {m, pk, cpk, sh, R low, R high, 0, usable}.
__host__ __device__ __forceinline__ void rescale_rec_build(int32_t m, int32_t shift, int double_round, int32_t out_zp,
                                                            int32_t correction, int64_t vmax, int32_t r8[8])
{
    bool ok = (m >= 0) && (shift >= 2) && (shift <= 53) && (out_zp >= -128) && (out_zp <= 127);
    const int32_t sc = shift < 2 ? 2 : (shift > 53 ? 53 : shift);
    int32_t pk, sh;
    uint32_t bias = 0;
    uint64_t R;
    if (sc <= 31)
    {
        pk  = (int32_t)1 << (32 - sc);
        sh  = 0;
        R   = ((uint64_t)1 << 31) + (uint64_t)((int64_t)out_zp * ((int64_t)1 << 32));
        if (double_round)
        {
            ok   = ok && vmax < ((int64_t)1 << (sc - 2));
            bias = (uint32_t)1 << 30;
            R -= (uint64_t)bias * (uint64_t)(uint32_t)m;
        }
        else
            ok = ok && vmax < ((int64_t)1 << (sc - 1));
    }
    else
    {
        ok  = ok && vmax < ((int64_t)1 << 30);
        pk  = 2;
        sh  = sc - 31;
        R   = ((uint64_t)1 << sc) + (double_round ? ((uint64_t)1 << 31) : 0) +
              (uint64_t)((int64_t)out_zp * ((int64_t)1 << (sc + 1)));
    }
    r8[0] = m;
    r8[1] = pk;
    r8[2] = (int32_t)((uint32_t)correction * (uint32_t)pk + bias);
    r8[3] = sh;
    r8[4] = (int32_t)(uint32_t)(R & 0xffffffffULL);
    r8[5] = (int32_t)(uint32_t)(R >> 32);
    r8[6] = 0;
    r8[7] = ok ? 1 : 0;
}

// One accumulator through the lean form; the result still needs saturation to int8.  `fix` is the layer's double_round.
__host__ __device__ __forceinline__ int32_t rescale_rec_apply(int32_t acc, int32_t m, int32_t pk, int32_t cpk, int32_t sh,
                                                               int32_t rlo, int32_t rhi, bool fix)
{
    const int32_t s  = (int32_t)((uint32_t)acc * (uint32_t)pk + (uint32_t)cpk);
    const int64_t P  = (int64_t)s * (int64_t)m + (int64_t)(((uint64_t)(uint32_t)rhi << 32) | (uint32_t)rlo);
    int32_t hi       = (int32_t)(P >> 32);
    if (fix)
        hi += s >> 31;
    return hi >> sh;
}

// ---------------------------------------------------------------------------------------------------------------
// Unsigned division by an invariant d >= 1 as a multiply-high and shifts, exact for every 32-bit dividend:
// l = ceil(log2 d), m = floor(2^32 (2^l - d) / d) + 1, q = (t + ((n - t) >> 1)) >> (l - 1) with t = high word of m * n;
// l = 0 (d = 1) stands for q = n.  The kernels decode tile numbers with it (three divisions per tile otherwise).
__host__ __device__ __forceinline__ void fastdiv_make(uint32_t d, uint32_t out[2])
{
    uint32_t l = 0;
    while ((1ull << l) < d)
        l++;
    out[0] = l == 0 ? 0u : (uint32_t)((((1ull << l) - d) << 32) / d + 1);
    out[1] = l;
}

__host__ __device__ __forceinline__ uint32_t fastdiv_apply(uint32_t n, const uint32_t (&md)[2])
{
    if (md[1] == 0)
        return n;
#ifdef __CUDA_ARCH__
    const uint32_t t = __umulhi(md[0], n);
#else
    const uint32_t t = (uint32_t)(((uint64_t)md[0] * n) >> 32);
#endif
    return (t + ((n - t) >> 1)) >> (md[1] - 1);
}

}    // namespace tb200
