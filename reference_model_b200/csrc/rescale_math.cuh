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

}    // namespace tb200
