// CUDA-core kernels: elementwise RESCALE / CLAMP / ADD / residual join, pooling, depthwise convolution,
// general direct CONV2D / MATMUL (any shape; also the on-device cross-check of the tensor-core path), and the
// small preparation kernels (zero-point row / column sums, per-tap weight sums).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <type_traits>

#include "common.h"
#include "rescale_math.cuh"

namespace tb200
{

// ------------------------------------------------------------------------------------------------ type helpers
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v)
{
    return v;
}
template <>
__device__ __forceinline__ float to_f32<__half>(__half v)
{
    return __half2float(v);
}
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v)
{
    return __bfloat162float(v);
}

// fp8 operands are exact in fp32 (OpMatMul's FP8 instantiations, reference_model/src/ops/tensor_ops.cpp:2263-2270)
template <>
__device__ __forceinline__ float to_f32<__nv_fp8_e4m3>(__nv_fp8_e4m3 v)
{
    return float(v);
}
template <>
__device__ __forceinline__ float to_f32<__nv_fp8_e5m2>(__nv_fp8_e5m2 v)
{
    return float(v);
}

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v)
{
    return v;
}
template <>
__device__ __forceinline__ __half from_f32<__half>(float v)
{
    return __float2half_rn(v);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v)
{
    return __float2bfloat16_rn(v);
}

// ------------------------------------------------------------------------------------------------ RESCALE
struct RescaleDev
{
    const void* mult;
    const int8_t* shift;
    int mult_is_i16, per_channel, scale32, rounding;
    int64_t in_zp_ext, out_zp_ext;
    int in_bits, out_bits;
    int in_unsigned, out_unsigned;
    int64_t qmin, qmax;
};

__device__ __forceinline__ int32_t rescale_elem(int32_t raw, int ch, const RescaleDev& r, bool& bad)
{
    const int64_t v64 = value_extend64_dev(raw, r.in_bits, r.in_unsigned != 0) - r.in_zp_ext;
    const int c       = r.per_channel ? ch : 0;
    const int32_t m   = r.mult_is_i16 ? (int32_t) reinterpret_cast<const int16_t*>(r.mult)[c]
                                      : reinterpret_cast<const int32_t*>(r.mult)[c];
    const int32_t s   = (int32_t)r.shift[c];
    int32_t scaled;
    bool b = false;
    if (r.rounding != TB200_INEXACT_ROUND)
    {
        if (r.scale32)
            scaled = apply_scale_32_dev((int32_t)v64, m, s, r.rounding == TB200_DOUBLE_ROUND, b);
        else
            scaled = apply_scale_16_dev(v64, (int16_t)m, s, b);
    }
    else
    {
        // INEXACT_ROUND in fp32 maths (reference_model/src/ops/type_conversion.cpp:318-323)
        const float res = __fmul_rn(__fmul_rn((float)v64, (float)m), exp2f((float)(-s)));
        scaled          = (int32_t)rintf(res);
    }
    int64_t z = (int64_t)scaled + r.out_zp_ext;
    b |= (z > 2147483647LL) || (z < -2147483648LL);
    z = z < r.qmin ? r.qmin : z;
    z = z > r.qmax ? r.qmax : z;
    bad |= b;
    return b ? 0 : (int32_t)z;
}

template <typename TIn, typename TOut, int VEC>
__global__ void rescale_kernel(const TIn* __restrict__ in, TOut* __restrict__ out, int64_t n, int C, RescaleDev r,
                               int* status)
{
    bool bad            = false;
    const int64_t nvec  = n / VEC;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += step)
    {
        TIn vi[VEC];
        TOut vo[VEC];
        if (VEC == 4)
        {
            if (sizeof(TIn) == 4)
                *reinterpret_cast<int4*>(vi) = reinterpret_cast<const int4*>(in)[i];
            else if (sizeof(TIn) == 2)
                *reinterpret_cast<int2*>(vi) = reinterpret_cast<const int2*>(in)[i];
            else
                *reinterpret_cast<int*>(vi) = reinterpret_cast<const int*>(in)[i];
        }
        else
            vi[0] = in[i];
        const int ch0 = (int)((i * VEC) % C);
#pragma unroll
        for (int j = 0; j < VEC; j++)
            vo[j] = (TOut)rescale_elem((int32_t)vi[j], ch0 + j, r, bad);
        if (VEC == 4)
        {
            if (sizeof(TOut) == 4)
                reinterpret_cast<int4*>(out)[i] = *reinterpret_cast<int4*>(vo);
            else if (sizeof(TOut) == 2)
                reinterpret_cast<int2*>(out)[i] = *reinterpret_cast<int2*>(vo);
            else
                reinterpret_cast<int*>(out)[i] = *reinterpret_cast<int*>(vo);
        }
        else
            out[i] = vo[0];
    }
    if (bad)
        atomicOr(status, TB200_DEV_UNPREDICTABLE);
}

// Residual join: out = clamp(rescale_o(rescale_a(a) + rescale_b(b))), 16 int8 values per thread.
struct ResidualDev
{
    RescaleDev ra, rb, ro;
    int has_clamp;
    int32_t clamp_min, clamp_max;
};

template <int VEC>
__global__ void residual_add_i8_kernel(const int8_t* __restrict__ a, const int8_t* __restrict__ b,
                                       int8_t* __restrict__ out, int64_t n, int C, ResidualDev r, int* status)
{
    bool bad           = false;
    const int64_t nvec = n / VEC;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += step)
    {
        int8_t va[VEC], vb[VEC], vo[VEC];
        if (VEC == 16)
        {
            *reinterpret_cast<int4*>(va) = reinterpret_cast<const int4*>(a)[i];
            *reinterpret_cast<int4*>(vb) = reinterpret_cast<const int4*>(b)[i];
        }
        else
        {
            va[0] = a[i];
            vb[0] = b[i];
        }
        const int ch0 = (int)((i * VEC) % C);
#pragma unroll
        for (int j = 0; j < VEC; j++)
        {
            const int32_t x = rescale_elem((int32_t)va[j], ch0 + j, r.ra, bad);
            const int32_t y = rescale_elem((int32_t)vb[j], ch0 + j, r.rb, bad);
            const int64_t s = (int64_t)x + (int64_t)y;
            bad |= (s > 2147483647LL) || (s < -2147483648LL);
            int32_t z = rescale_elem((int32_t)(uint32_t)((uint32_t)x + (uint32_t)y), ch0 + j, r.ro, bad);
            if (r.has_clamp)
            {
                z = z >= r.clamp_min ? z : r.clamp_min;
                z = z < r.clamp_max ? z : r.clamp_max;
            }
            vo[j] = (int8_t)z;
        }
        if (VEC == 16)
            reinterpret_cast<int4*>(out)[i] = *reinterpret_cast<int4*>(vo);
        else
            out[i] = vo[0];
    }
    if (bad)
        atomicOr(status, TB200_DEV_UNPREDICTABLE);
}

// Fast residual join for the common case: per-tensor scale32 RESCALEs whose int8 -> int32 legs cannot violate any
// REQUIRE (checked on the host from the operands' ranges).  16 int8 values per thread, 64-bit products split into
// words so every shift is a 32-bit operation.
struct Scale32Fast
{
    int32_t mult, shift;
    int32_t rpos_lo, rpos_hi, rneg_lo, rneg_hi;    // rounding constant for v >= 0 / v < 0
    int32_t zp_in, zp_out;
};

__device__ __forceinline__ int32_t scale32_fast(int32_t v, const Scale32Fast& c, bool& narrow_overflow)
{
    const int64_t rpos = ((int64_t)c.rpos_hi << 32) | (uint32_t)c.rpos_lo;
    const int64_t rneg = ((int64_t)c.rneg_hi << 32) | (uint32_t)c.rneg_lo;
    const int64_t prod = (int64_t)v * (int64_t)c.mult + (v >= 0 ? rpos : rneg);
    const uint32_t plo = (uint32_t)prod;
    const int32_t phi  = (int32_t)(prod >> 32);
    if (c.shift >= 32)
        return phi >> (c.shift - 32);
    const int32_t res = (int32_t)__funnelshift_r(plo, (uint32_t)phi, c.shift);
    narrow_overflow |= (phi >> c.shift) != (res >> 31);
    return res;
}

// per-tensor leg described by device pointers to its multiplier / shift (read once per thread)
struct ResidualLeg
{
    const int32_t* mult;
    const int8_t* shift;
    int32_t zp_in, zp_out, double_round;
};

struct ResidualFast
{
    ResidualLeg a, b, o;
    int32_t lo, hi;    // int8 clip folded with the CLAMP bounds
};

// Builds the constants of one leg; *vlim receives the largest |v| apply_scale_32 accepts (-1: invalid operands)
__device__ __forceinline__ Scale32Fast make_scale32_fast(const ResidualLeg& l, int32_t* vlim)
{
    Scale32Fast c;
    const int32_t m = __ldg(l.mult);
    const int32_t s = (int32_t)__ldg(l.shift);
    const bool valid = (m >= 0) && (s >= 2) && (s <= 62);
    c.mult  = m;
    c.shift = valid ? s : 2;
    const int64_t half = (int64_t)1 << (c.shift - 1);
    int64_t rpos = half, rneg = half;
    if (l.double_round && c.shift > 31)
    {
        rpos += (int64_t)1 << 30;
        rneg -= (int64_t)1 << 30;
    }
    c.rpos_lo = (int32_t)(uint32_t)(rpos & 0xffffffffLL);
    c.rpos_hi = (int32_t)(rpos >> 32);
    c.rneg_lo = (int32_t)(uint32_t)(rneg & 0xffffffffLL);
    c.rneg_hi = (int32_t)(rneg >> 32);
    c.zp_in   = l.zp_in;
    c.zp_out  = l.zp_out;
    *vlim     = !valid ? -1 : (c.shift - 1 >= 31 ? 2147483647 : (int32_t)(half - 1));
    return c;
}

__global__ void __launch_bounds__(256) residual_add_i8_fast_kernel(const int8_t* __restrict__ a, const int8_t* __restrict__ b,
                                                                   int8_t* __restrict__ out, int64_t n16, ResidualFast r,
                                                                   int* status)
{
    // The int8 -> int32 legs have only 256 possible inputs each: tabulate them once per block, with their REQUIRE
    // verdicts, and leave the per-element work to the INT32 ADD and the output leg.
    __shared__ int32_t lut[2][256];
    __shared__ int lut_bad[2];
    int32_t vlim_o;
    const Scale32Fast co = make_scale32_fast(r.o, &vlim_o);
    if (threadIdx.x < 2)
        lut_bad[threadIdx.x] = 0;
    __syncthreads();
    {
        int32_t vlim;
        for (int leg = 0; leg < 2; leg++)
        {
            const Scale32Fast c = make_scale32_fast(leg == 0 ? r.a : r.b, &vlim);
            const int32_t x     = (int32_t)(int8_t)(threadIdx.x ^ 0x80) - c.zp_in;    // table index = raw byte ^ 0x80
            bool ov             = (x > vlim) || (x < ~vlim);
            lut[leg][threadIdx.x] = scale32_fast(x, c, ov);
            if (ov)
                lut_bad[leg] = 1;
        }
    }
    __syncthreads();
    // with a bad entry in a table the legs are re-checked per element below (the entry may never be used)
    const bool recheck = lut_bad[0] || lut_bad[1];
    int32_t vlim_a = 0, vlim_b = 0;
    Scale32Fast ca = co, cb = co;
    if (recheck)
    {
        ca = make_scale32_fast(r.a, &vlim_a);
        cb = make_scale32_fast(r.b, &vlim_b);
    }
    bool bad = false;
    const int32_t zp_add_hi = co.zp_out > 0 ? 2147483647 - co.zp_out : 2147483647;
    const int32_t zp_add_lo = co.zp_out < 0 ? (int32_t)(-2147483647 - 1 - co.zp_out) : (-2147483647 - 1);
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += step)
    {
        const int4 va = __ldg(reinterpret_cast<const int4*>(a) + i);
        const int4 vb = __ldg(reinterpret_cast<const int4*>(b) + i);
        const uint32_t wa[4] = { (uint32_t)va.x ^ 0x80808080u, (uint32_t)va.y ^ 0x80808080u, (uint32_t)va.z ^ 0x80808080u,
                                 (uint32_t)va.w ^ 0x80808080u };
        const uint32_t wb[4] = { (uint32_t)vb.x ^ 0x80808080u, (uint32_t)vb.y ^ 0x80808080u, (uint32_t)vb.z ^ 0x80808080u,
                                 (uint32_t)vb.w ^ 0x80808080u };
        uint32_t wo[4];
#pragma unroll
        for (int q = 0; q < 4; q++)
        {
            uint32_t packed = 0;
#pragma unroll
            for (int j = 0; j < 4; j++)
            {
                const uint32_t ia = (wa[q] >> (8 * j)) & 0xffu, ib = (wb[q] >> (8 * j)) & 0xffu;
                const int32_t ya = lut[0][ia], yb = lut[1][ib];
                bool ov = false;
                if (recheck)
                {
                    const int32_t xa = (int32_t)(int8_t)(ia ^ 0x80) - ca.zp_in, xb = (int32_t)(int8_t)(ib ^ 0x80) - cb.zp_in;
                    ov = (xa > vlim_a) || (xa < ~vlim_a) || (xb > vlim_b) || (xb < ~vlim_b);
                    (void)scale32_fast(xa, ca, ov);
                    (void)scale32_fast(xb, cb, ov);
                }
                const int32_t sum = (int32_t)((uint32_t)ya + (uint32_t)yb);
                // INT32 ADD: the mathematical sum must fit (operand signs equal and result sign differs = overflow)
                ov |= ((ya ^ sum) & (yb ^ sum)) < 0;
                const int32_t res = scale32_fast(sum, co, ov);
                bad |= ov || (sum > vlim_o) || (sum < ~vlim_o) || (res > zp_add_hi) || (res < zp_add_lo);
                int32_t z = res + co.zp_out;
                z = max(z, r.lo);
                z = min(z, r.hi);
                packed |= (uint32_t)(z & 0xff) << (8 * j);
            }
            wo[q] = packed;
        }
        reinterpret_cast<uint4*>(out)[i] = make_uint4(wo[0], wo[1], wo[2], wo[3]);
    }
    if (bad)
        atomicOr(status, TB200_DEV_UNPREDICTABLE);
}

// Residual join through one table.  With per-tensor parameters the whole RESCALE, RESCALE, ADD, RESCALE, CLAMP chain is
// a function of the two input bytes alone.  residual_table_kernel evaluates it for all 65536 byte pairs (with every
// REQUIRE verdict as one bit per pair), and residual_add_i8_table_kernel keeps the table in shared memory and spends one
// byte lookup per element.  Row a of the table is stored with its b index XOR-ed by 4 * (a mod 32) so that equal b
// values next to different a values fall into different shared-memory banks.
constexpr int kJoinTableBytes = 65536;
constexpr int kJoinBadWords   = 2048;

__device__ __forceinline__ uint32_t join_table_slot(uint32_t ua, uint32_t ub)
{
    return (ua << 8) | (ub ^ ((ua & 31u) << 2));
}

__global__ void __launch_bounds__(256) residual_table_kernel(ResidualFast r, uint8_t* __restrict__ table,
                                                             uint32_t* __restrict__ bad_bits)
{
    int32_t vlim_a, vlim_b, vlim_o;
    const Scale32Fast ca = make_scale32_fast(r.a, &vlim_a);
    const Scale32Fast cb = make_scale32_fast(r.b, &vlim_b);
    const Scale32Fast co = make_scale32_fast(r.o, &vlim_o);
    // raw bytes of the two operands; thread t of block a fills slot (a << 8 | t)
    const uint32_t ua = blockIdx.x, ub = threadIdx.x ^ ((blockIdx.x & 31u) << 2);
    const int32_t xa  = (int32_t)(int8_t)ua - ca.zp_in;
    const int32_t xb  = (int32_t)(int8_t)ub - cb.zp_in;
    bool ov           = (xa > vlim_a) || (xa < ~vlim_a) || (xb > vlim_b) || (xb < ~vlim_b);
    const int32_t ya  = scale32_fast(xa, ca, ov);
    const int32_t yb  = scale32_fast(xb, cb, ov);
    const int32_t sum = (int32_t)((uint32_t)ya + (uint32_t)yb);
    // INT32 ADD: the mathematical sum must fit (operand signs equal and result sign differs = overflow)
    ov |= ((ya ^ sum) & (yb ^ sum)) < 0;
    const int32_t res       = scale32_fast(sum, co, ov);
    const int32_t zp_add_hi = co.zp_out > 0 ? 2147483647 - co.zp_out : 2147483647;
    const int32_t zp_add_lo = co.zp_out < 0 ? (int32_t)(-2147483647 - 1 - co.zp_out) : (-2147483647 - 1);
    ov |= (sum > vlim_o) || (sum < ~vlim_o) || (res > zp_add_hi) || (res < zp_add_lo);
    int32_t z = res + co.zp_out;
    z = max(z, r.lo);
    z = min(z, r.hi);
    const uint32_t slot = join_table_slot(ua, ub);    // == (ua << 8) | threadIdx.x
    table[slot]      = (uint8_t)(z & 0xff);
    const uint32_t m = __ballot_sync(0xffffffffu, ov);
    if ((threadIdx.x & 31) == 0)
        bad_bits[slot >> 5] = m;
}

__global__ void __launch_bounds__(512, 2) residual_add_i8_table_kernel(const int8_t* __restrict__ a, const int8_t* __restrict__ b,
                                                                       int8_t* __restrict__ out, int64_t n16,
                                                                       const uint8_t* __restrict__ table,
                                                                       const uint32_t* __restrict__ bad_bits, int* status)
{
    extern __shared__ __align__(16) uint8_t join_smem[];
    uint8_t* tab   = join_smem;
    uint32_t* bits = reinterpret_cast<uint32_t*>(join_smem + kJoinTableBytes);
    // Programmatic dependent launch: the successor may be scheduled from now on; the table and the REQUIRE bits are
    // constants of the join (a kernel that prepares them never lets its successor start early), so their copy to shared
    // memory runs while the predecessor still drains; the operands are its output and wait for it.
    if (threadIdx.x == 0)
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    for (int i = threadIdx.x; i < kJoinTableBytes / 16; i += blockDim.x)
        reinterpret_cast<int4*>(tab)[i] = __ldg(reinterpret_cast<const int4*>(table) + i);
    uint32_t any = 0;
    for (int i = threadIdx.x; i < kJoinBadWords; i += blockDim.x)
    {
        const uint32_t w = __ldg(bad_bits + i);
        bits[i] = w;
        any |= w;
    }
    // (also the barrier that publishes the table)
    const bool check = __syncthreads_or(any != 0) != 0;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    bool bad = false;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    auto lookup16 = [&](const int4& va, const int4& vb) -> uint4 {
        const uint32_t wa[4] = { (uint32_t)va.x, (uint32_t)va.y, (uint32_t)va.z, (uint32_t)va.w };
        const uint32_t wb[4] = { (uint32_t)vb.x, (uint32_t)vb.y, (uint32_t)vb.z, (uint32_t)vb.w };
        uint32_t wo[4];
#pragma unroll
        for (int q = 0; q < 4; q++)
        {
            // two 16-bit slots per word: (a byte << 8 | b byte), then the bank swizzle on both at once
            uint32_t p01 = __byte_perm(wa[q], wb[q], 0x1504);
            uint32_t p23 = __byte_perm(wa[q], wb[q], 0x3726);
            p01 ^= (p01 >> 6) & 0x007c007cu;
            p23 ^= (p23 >> 6) & 0x007c007cu;
            const uint32_t i0 = p01 & 0xffffu, i1 = p01 >> 16, i2 = p23 & 0xffffu, i3 = p23 >> 16;
            const uint32_t r0 = tab[i0], r1 = tab[i1], r2 = tab[i2], r3 = tab[i3];
            if (check)
                bad |= (((bits[i0 >> 5] >> (i0 & 31)) | (bits[i1 >> 5] >> (i1 & 31)) | (bits[i2 >> 5] >> (i2 & 31)) |
                         (bits[i3 >> 5] >> (i3 & 31))) & 1u) != 0;
            wo[q] = __byte_perm(__byte_perm(r0, r1, 0x0040), __byte_perm(r2, r3, 0x0040), 0x5410);
        }
        return make_uint4(wo[0], wo[1], wo[2], wo[3]);
    };
    // two vectors per pass: four 16-byte loads in flight per thread (the kernel waits on memory, not on arithmetic)
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + step < n16; i += 2 * step)
    {
        const int4 va0 = __ldg(reinterpret_cast<const int4*>(a) + i);
        const int4 vb0 = __ldg(reinterpret_cast<const int4*>(b) + i);
        const int4 va1 = __ldg(reinterpret_cast<const int4*>(a) + i + step);
        const int4 vb1 = __ldg(reinterpret_cast<const int4*>(b) + i + step);
        reinterpret_cast<uint4*>(out)[i]        = lookup16(va0, vb0);
        reinterpret_cast<uint4*>(out)[i + step] = lookup16(va1, vb1);
    }
    if (i < n16)
    {
        const int4 va = __ldg(reinterpret_cast<const int4*>(a) + i);
        const int4 vb = __ldg(reinterpret_cast<const int4*>(b) + i);
        reinterpret_cast<uint4*>(out)[i] = lookup16(va, vb);
    }
    if (bad)
        atomicOr(status, TB200_DEV_UNPREDICTABLE);
}

// ------------------------------------------------------------------------------------------------ CLAMP
template <typename T>
__global__ void clamp_int_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t n, int32_t lo, int32_t hi)
{
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    constexpr int VEC  = 16 / sizeof(T);
    const int64_t nvec = n / VEC;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += step)
    {
        T v[VEC];
        *reinterpret_cast<int4*>(v) = reinterpret_cast<const int4*>(in)[i];
#pragma unroll
        for (int j = 0; j < VEC; j++)
        {
            int32_t x = (int32_t)v[j];
            x         = x >= lo ? x : lo;
            x         = x < hi ? x : hi;
            v[j]      = (T)x;
        }
        reinterpret_cast<int4*>(out)[i] = *reinterpret_cast<int4*>(v);
    }
    for (int64_t i = nvec * VEC + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step)
    {
        int32_t x = (int32_t)in[i];
        x         = x >= lo ? x : lo;
        x         = x < hi ? x : hi;
        out[i]    = (T)x;
    }
}

// applyClip then fpTrunc (reference_model/src/ops/activation_funcs.cpp:105-111, src/arith_util.h:340-413)
template <typename T>
__device__ __forceinline__ T clamp_fp_elem(T raw, float lo, float hi, int nan_ignore)
{
    float v = to_f32<T>(raw);
    if (isnan(v))
        v = nan_ignore ? lo : v;
    else
        v = (v >= lo) ? v : lo;
    if (!isnan(v))
        v = (v < hi) ? v : hi;
    return from_f32<T>(v);
}

template <typename T>
__global__ void clamp_fp_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t n, float lo, float hi,
                                int nan_ignore)
{
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    constexpr int VEC  = 16 / sizeof(T);
    const int64_t nvec = n / VEC;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += step)
    {
        T v[VEC];
        *reinterpret_cast<int4*>(v) = reinterpret_cast<const int4*>(in)[i];
#pragma unroll
        for (int j = 0; j < VEC; j++)
            v[j] = clamp_fp_elem<T>(v[j], lo, hi, nan_ignore);
        reinterpret_cast<int4*>(out)[i] = *reinterpret_cast<int4*>(v);
    }
    for (int64_t i = nvec * VEC + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step)
        out[i] = clamp_fp_elem<T>(in[i], lo, hi, nan_ignore);
}

// ------------------------------------------------------------------------------------------------ ADD
struct BcastDev
{
    int rank;
    int oshape[6];
    int64_t astride[6], bstride[6];    // 0 where the operand broadcasts
    int same_shape;
};

template <typename T>
__device__ __forceinline__ T add_elem(T a, T b, bool& bad);
template <>
__device__ __forceinline__ int32_t add_elem<int32_t>(int32_t a, int32_t b, bool& bad)
{
    const int64_t s = (int64_t)a + (int64_t)b;
    bad |= (s > 2147483647LL) || (s < -2147483648LL);
    return (int32_t)((uint32_t)a + (uint32_t)b);
}
template <>
__device__ __forceinline__ float add_elem<float>(float a, float b, bool&)
{
    return a + b;
}
template <>
__device__ __forceinline__ __half add_elem<__half>(__half a, __half b, bool&)
{
    return __float2half_rn(__half2float(a) + __half2float(b));
}
template <>
__device__ __forceinline__ __nv_bfloat16 add_elem<__nv_bfloat16>(__nv_bfloat16 a, __nv_bfloat16 b, bool&)
{
    return __float2bfloat16_rn(__bfloat162float(a) + __bfloat162float(b));
}

template <typename T>
__global__ void add_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t n,
                           BcastDev bc, int* status)
{
    bool bad           = false;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    if (bc.same_shape)
    {
        constexpr int VEC  = 16 / sizeof(T);
        const int64_t nvec = n / VEC;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += step)
        {
            T va[VEC], vb[VEC];
            *reinterpret_cast<int4*>(va) = reinterpret_cast<const int4*>(a)[i];
            *reinterpret_cast<int4*>(vb) = reinterpret_cast<const int4*>(b)[i];
#pragma unroll
            for (int j = 0; j < VEC; j++)
                va[j] = add_elem<T>(va[j], vb[j], bad);
            reinterpret_cast<int4*>(out)[i] = *reinterpret_cast<int4*>(va);
        }
        for (int64_t i = nvec * VEC + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step)
            out[i] = add_elem<T>(a[i], b[i], bad);
    }
    else
    {
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step)
        {
            int64_t rem = i, ai = 0, bi = 0;
            for (int d = bc.rank - 1; d >= 0; d--)
            {
                const int64_t c = rem % bc.oshape[d];
                rem /= bc.oshape[d];
                ai += c * bc.astride[d];
                bi += c * bc.bstride[d];
            }
            out[i] = add_elem<T>(a[ai], b[bi], bad);
        }
    }
    if (bad)
        atomicOr(status, TB200_DEV_UNPREDICTABLE);
}

// ------------------------------------------------------------------------------------------------ pooling
struct PoolDev
{
    int N, IH, IW, C, OH, OW;
    int ky, kx, pad_t, pad_l, sy, sx;
};

// MAX_POOL2D on int8 NHWC, 16 channels per thread (C % 16 == 0)
__global__ void max_pool_i8x16_kernel(const int8_t* __restrict__ in, int8_t* __restrict__ out, PoolDev p)
{
    const int cv        = p.C / 16;
    const int64_t total = (int64_t)p.N * p.OH * p.OW * cv;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int c16 = (int)(i % cv);
        int64_t r     = i / cv;
        const int ox  = (int)(r % p.OW);
        r /= p.OW;
        const int oy = (int)(r % p.OH);
        const int n  = (int)(r / p.OH);
        uint32_t m[4] = { 0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u };    // four lanes of -128
        for (int ky = 0; ky < p.ky; ky++)
        {
            const int y = oy * p.sy - p.pad_t + ky;
            if (y < 0 || y >= p.IH)
                continue;
            for (int kx = 0; kx < p.kx; kx++)
            {
                const int x = ox * p.sx - p.pad_l + kx;
                if (x < 0 || x >= p.IW)
                    continue;
                const uint4 v =
                    *reinterpret_cast<const uint4*>(in + (((int64_t)n * p.IH + y) * p.IW + x) * p.C + c16 * 16);
                m[0] = __vmaxs4(m[0], v.x);
                m[1] = __vmaxs4(m[1], v.y);
                m[2] = __vmaxs4(m[2], v.z);
                m[3] = __vmaxs4(m[3], v.w);
            }
        }
        *reinterpret_cast<uint4*>(out + (((int64_t)n * p.OH + oy) * p.OW + ox) * p.C + c16 * 16) =
            make_uint4(m[0], m[1], m[2], m[3]);
    }
}

// The same for a 3 x 3 window (the pooling layer of ResNet-shaped graphs): all nine 16-byte loads are issued before the
// first comparison, so a thread waits for memory once instead of nine times (taps outside the image read the centre,
// which is always inside, and so do not change the maximum).
__global__ void max_pool3x3_i8x16_kernel(const int8_t* __restrict__ in, int8_t* __restrict__ out, PoolDev p)
{
    const int cv        = p.C / 16;
    const int64_t total = (int64_t)p.N * p.OH * p.OW * cv;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int c16 = (int)(i % cv);
        int64_t r     = i / cv;
        const int ox  = (int)(r % p.OW);
        r /= p.OW;
        const int oy = (int)(r % p.OH);
        const int n  = (int)(r / p.OH);
        const int y0 = oy * p.sy - p.pad_t, x0 = ox * p.sx - p.pad_l;
        // a tap that exists: the window always overlaps the image (checked on the host: pad < kernel)
        const int yc = min(max(y0 + 1, 0), p.IH - 1), xc = min(max(x0 + 1, 0), p.IW - 1);
        const int8_t* base = in + (int64_t)n * p.IH * p.IW * p.C + c16 * 16;
        uint4 v[9];
#pragma unroll
        for (int ky = 0; ky < 3; ky++)
        {
            const int y  = y0 + ky;
            const int yy = (y < 0 || y >= p.IH) ? yc : y;
#pragma unroll
            for (int kx = 0; kx < 3; kx++)
            {
                const int x  = x0 + kx;
                const int xx = (x < 0 || x >= p.IW) ? xc : x;
                v[ky * 3 + kx] = __ldg(reinterpret_cast<const uint4*>(base + ((int64_t)yy * p.IW + xx) * p.C));
            }
        }
        uint32_t m[4] = { v[0].x, v[0].y, v[0].z, v[0].w };
#pragma unroll
        for (int t = 1; t < 9; t++)
        {
            m[0] = __vmaxs4(m[0], v[t].x);
            m[1] = __vmaxs4(m[1], v[t].y);
            m[2] = __vmaxs4(m[2], v[t].z);
            m[3] = __vmaxs4(m[3], v[t].w);
        }
        *reinterpret_cast<uint4*>(out + (((int64_t)n * p.OH + oy) * p.OW + ox) * p.C + c16 * 16) =
            make_uint4(m[0], m[1], m[2], m[3]);
    }
}

// general MAX_POOL2D, one element per thread; `lowest` is the padding value of the dtype
template <typename T, typename TCmp>
__global__ void max_pool_kernel(const T* __restrict__ in, T* __restrict__ out, PoolDev p, TCmp lowest)
{
    const int64_t total = (int64_t)p.N * p.OH * p.OW * p.C;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int c  = (int)(i % p.C);
        int64_t r    = i / p.C;
        const int ox = (int)(r % p.OW);
        r /= p.OW;
        const int oy = (int)(r % p.OH);
        const int n  = (int)(r / p.OH);
        TCmp m       = lowest;
        bool nan     = false;
        for (int ky = 0; ky < p.ky; ky++)
            for (int kx = 0; kx < p.kx; kx++)
            {
                const int y = oy * p.sy - p.pad_t + ky;
                const int x = ox * p.sx - p.pad_l + kx;
                if (y < 0 || y >= p.IH || x < 0 || x >= p.IW)
                    continue;
                const TCmp v = (TCmp)in[(((int64_t)n * p.IH + y) * p.IW + x) * p.C + c];
                if constexpr (std::is_floating_point<TCmp>::value)
                {
                    if (isnan(v))
                        nan = true;
                }
                m = (m >= v) ? m : v;
            }
        if constexpr (std::is_floating_point<TCmp>::value)
        {
            if (nan)
                m = NAN;    // NaN-propagating mode
        }
        out[i] = (T)m;
    }
}

// AVG_POOL2D integer path (reference_model/src/ops/tensor_ops.cpp:604-653)
template <typename T>
__global__ void avg_pool_int_kernel(const T* __restrict__ in, T* __restrict__ out, PoolDev p, int32_t in_zp,
                                    int32_t out_zp, int32_t qmin, int32_t qmax, int* status)
{
    const int64_t total = (int64_t)p.N * p.OH * p.OW * p.C;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    bool bad            = false;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int c  = (int)(i % p.C);
        int64_t r    = i / p.C;
        const int ox = (int)(r % p.OW);
        r /= p.OW;
        const int oy = (int)(r % p.OH);
        const int n  = (int)(r / p.OH);
        int32_t acc  = 0;
        int count    = 0;
        for (int ky = 0; ky < p.ky; ky++)
            for (int kx = 0; kx < p.kx; kx++)
            {
                const int y = oy * p.sy - p.pad_t + ky;
                const int x = ox * p.sx - p.pad_l + kx;
                if (y < 0 || y >= p.IH || x < 0 || x >= p.IW)
                    continue;
                acc += (int32_t)in[(((int64_t)n * p.IH + y) * p.IW + x) * p.C + c] - in_zp;
                count++;
            }
        int32_t mult, shift;
        reciprocal_scale_dev(count, mult, shift);
        bool b    = false;
        int32_t v = apply_scale_32_dev(acc, mult, shift, false, b);
        if (b)
            v = 0;
        bad |= b;
        v = (int32_t)((uint32_t)v + (uint32_t)out_zp);
        v = v > qmin ? v : qmin;
        v = v < qmax ? v : qmax;
        out[i] = (T)v;
    }
    if (bad)
        atomicOr(status, TB200_DEV_UNPREDICTABLE);
}

// The int8 case with four channels per thread (one 32-bit load per tap and thread, 128 bytes per warp): the global
// average pool at the end of a ResNet-shaped graph reads 49 taps per output and was bound by one-byte loads.
__global__ void avg_pool_i8x4_kernel(const int8_t* __restrict__ in, int8_t* __restrict__ out, PoolDev p, int32_t in_zp,
                                     int32_t out_zp, int32_t qmin, int32_t qmax, int* status)
{
    const int cv        = p.C / 4;
    const int64_t total = (int64_t)p.N * p.OH * p.OW * cv;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    bool bad            = false;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int c4 = (int)(i % cv) * 4;
        int64_t r    = i / cv;
        const int ox = (int)(r % p.OW);
        r /= p.OW;
        const int oy = (int)(r % p.OH);
        const int n  = (int)(r / p.OH);
        int32_t acc[4] = { 0, 0, 0, 0 };
        int count      = 0;
        const int y0 = oy * p.sy - p.pad_t, x0 = ox * p.sx - p.pad_l;
        if (y0 >= 0 && y0 + p.ky <= p.IH && x0 >= 0 && x0 + p.kx <= p.IW)
        {
            // the whole window lies inside the image: eight loads are issued before the first of them is used (a 7 x 7
            // global pool took 49 memory latencies one after the other, 29 us whatever the batch)
            const int taps       = p.ky * p.kx;
            const int8_t* base   = in + (((int64_t)n * p.IH + y0) * p.IW + x0) * p.C + c4;
            for (int t0 = 0; t0 < taps; t0 += 8)
            {
                uint32_t w[8];
#pragma unroll
                for (int j = 0; j < 8; j++)
                {
                    const int t = min(t0 + j, taps - 1);
                    const int ky = t / p.kx, kx = t - ky * p.kx;
                    w[j] = __ldg(reinterpret_cast<const uint32_t*>(base + ((int64_t)ky * p.IW + kx) * p.C));
                }
#pragma unroll
                for (int j = 0; j < 8; j++)
                    if (t0 + j < taps)
                    {
                        acc[0] += (int32_t)(int8_t)(w[j] & 0xff) - in_zp;
                        acc[1] += (int32_t)(int8_t)((w[j] >> 8) & 0xff) - in_zp;
                        acc[2] += (int32_t)(int8_t)((w[j] >> 16) & 0xff) - in_zp;
                        acc[3] += (int32_t)(int8_t)(w[j] >> 24) - in_zp;
                    }
            }
            count = taps;
        }
        else
        for (int ky = 0; ky < p.ky; ky++)
        {
            const int y = y0 + ky;
            if (y < 0 || y >= p.IH)
                continue;
            for (int kx = 0; kx < p.kx; kx++)
            {
                const int x = x0 + kx;
                if (x < 0 || x >= p.IW)
                    continue;
                const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(in + (((int64_t)n * p.IH + y) * p.IW + x) * p.C + c4));
                acc[0] += (int32_t)(int8_t)(w & 0xff) - in_zp;
                acc[1] += (int32_t)(int8_t)((w >> 8) & 0xff) - in_zp;
                acc[2] += (int32_t)(int8_t)((w >> 16) & 0xff) - in_zp;
                acc[3] += (int32_t)(int8_t)(w >> 24) - in_zp;
                count++;
            }
        }
        int32_t mult, shift;
        reciprocal_scale_dev(count, mult, shift);
        uint32_t packed = 0;
#pragma unroll
        for (int j = 0; j < 4; j++)
        {
            bool b    = false;
            int32_t v = apply_scale_32_dev(acc[j], mult, shift, false, b);
            if (b)
                v = 0;
            bad |= b;
            v = (int32_t)((uint32_t)v + (uint32_t)out_zp);
            v = v > qmin ? v : qmin;
            v = v < qmax ? v : qmax;
            packed |= ((uint32_t)v & 0xffu) << (8 * j);
        }
        *reinterpret_cast<uint32_t*>(out + (((int64_t)n * p.OH + oy) * p.OW + ox) * p.C + c4) = packed;
    }
    if (bad)
        atomicOr(status, TB200_DEV_UNPREDICTABLE);
}

template <typename T>
__global__ void avg_pool_fp_kernel(const T* __restrict__ in, T* __restrict__ out, PoolDev p)
{
    const int64_t total = (int64_t)p.N * p.OH * p.OW * p.C;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int c  = (int)(i % p.C);
        int64_t r    = i / p.C;
        const int ox = (int)(r % p.OW);
        r /= p.OW;
        const int oy = (int)(r % p.OH);
        const int n  = (int)(r / p.OH);
        float acc    = 0.f;
        int count    = 0;
        for (int ky = 0; ky < p.ky; ky++)
            for (int kx = 0; kx < p.kx; kx++)
            {
                const int y = oy * p.sy - p.pad_t + ky;
                const int x = ox * p.sx - p.pad_l + kx;
                if (y < 0 || y >= p.IH || x < 0 || x >= p.IW)
                    continue;
                acc += to_f32<T>(in[(((int64_t)n * p.IH + y) * p.IW + x) * p.C + c]);
                count++;
            }
        out[i] = from_f32<T>(acc / (float)count);
    }
}

// ------------------------------------------------------------------------------------------------ direct conv
struct ConvDev
{
    int N, IH, IW, IC, OH, OW, OC, KH, KW, M;    // M: depthwise multiplier
    int pad_t, pad_l, sy, sx, dy, dx;
    int64_t in_sn, in_sh, in_sw;    // element strides of the input (a SLICE view keeps its parent's pitch)
    int32_t in_zp, w_zp;
    int bias_n;
    // optional fused epilogue
    int has_rescale;
    RescaleDev rs;
    int has_clamp;
    int32_t clamp_lo, clamp_hi;
    float clamp_lo_f, clamp_hi_f;
};

// One thread per output element, channel fastest.  Integer: int32 accumulation of (in - in_zp)(w - w_zp)
// over in-scope taps in ky, kx, ic order (reference_model/src/ops/tensor_ops.cpp:828-873).
template <typename TOut>
__global__ void conv2d_direct_i8_kernel(const int8_t* __restrict__ in, const int8_t* __restrict__ w,
                                        const int32_t* __restrict__ bias, TOut* __restrict__ out, ConvDev p,
                                        int* status)
{
    const int64_t total = (int64_t)p.N * p.OH * p.OW * p.OC;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    bool bad            = false;
    const bool vec4 = (p.IC % 4) == 0 && (p.in_sw % 4) == 0 && (p.in_sh % 4) == 0 && (p.in_sn % 4) == 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int oc = (int)(i % p.OC);
        int64_t r    = i / p.OC;
        const int ox = (int)(r % p.OW);
        r /= p.OW;
        const int oy = (int)(r % p.OH);
        const int n  = (int)(r / p.OH);
        int32_t acc  = 0;
        for (int ky = 0; ky < p.KH; ky++)
        {
            const int y = oy * p.sy + ky * p.dy - p.pad_t;
            if (y < 0 || y >= p.IH)
                continue;
            for (int kx = 0; kx < p.KW; kx++)
            {
                const int x = ox * p.sx + kx * p.dx - p.pad_l;
                if (x < 0 || x >= p.IW)
                    continue;
                const int8_t* ip = in + (int64_t)n * p.in_sn + (int64_t)y * p.in_sh + (int64_t)x * p.in_sw;
                const int8_t* wp = w + (((int64_t)oc * p.KH + ky) * p.KW + kx) * p.IC;
                if (vec4)
                {
                    // sum (a - za)(b - zb) = sum ab - zb sum a - za sum b + n za zb, four lanes at a time
                    int32_t sab = 0, sa = 0, sb = 0;
                    for (int ic = 0; ic < p.IC; ic += 4)
                    {
                        const int a4 = *reinterpret_cast<const int*>(ip + ic);
                        const int b4 = *reinterpret_cast<const int*>(wp + ic);
                        sab          = __dp4a(a4, b4, sab);
                        sa           = __dp4a(a4, 0x01010101, sa);
                        sb           = __dp4a(b4, 0x01010101, sb);
                    }
                    acc += sab - p.w_zp * sa - p.in_zp * sb + p.IC * p.in_zp * p.w_zp;
                }
                else
                {
                    for (int ic = 0; ic < p.IC; ic++)
                        acc += ((int32_t)ip[ic] - p.in_zp) * ((int32_t)wp[ic] - p.w_zp);
                }
            }
        }
        int32_t v = (int32_t)((uint32_t)bias[p.bias_n == 1 ? 0 : oc] + (uint32_t)acc);
        if (p.has_rescale)
        {
            v = rescale_elem(v, oc, p.rs, bad);
            if (p.has_clamp)
            {
                v = v >= p.clamp_lo ? v : p.clamp_lo;
                v = v < p.clamp_hi ? v : p.clamp_hi;
            }
        }
        out[i] = (TOut)v;
    }
    if (bad)
        atomicOr(status, TB200_DEV_UNPREDICTABLE);
}

// Floating types: sequential fp32 accumulation, result (plus optional CLAMP) rounded once to the storage type.
// TO: type of bias and output (the operand type, or FP16 for fp8 operands)
template <typename T, typename TO = T>
__global__ void conv2d_direct_fp_kernel(const T* __restrict__ in, const T* __restrict__ w, const TO* __restrict__ bias,
                                        TO* __restrict__ out, ConvDev p)
{
    const int64_t total = (int64_t)p.N * p.OH * p.OW * p.OC;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int oc = (int)(i % p.OC);
        int64_t r    = i / p.OC;
        const int ox = (int)(r % p.OW);
        r /= p.OW;
        const int oy = (int)(r % p.OH);
        const int n  = (int)(r / p.OH);
        float acc    = 0.f;
        for (int ky = 0; ky < p.KH; ky++)
        {
            const int y = oy * p.sy + ky * p.dy - p.pad_t;
            if (y < 0 || y >= p.IH)
                continue;
            for (int kx = 0; kx < p.KW; kx++)
            {
                const int x = ox * p.sx + kx * p.dx - p.pad_l;
                if (x < 0 || x >= p.IW)
                    continue;
                const T* ip = in + (int64_t)n * p.in_sn + (int64_t)y * p.in_sh + (int64_t)x * p.in_sw;
                const T* wp = w + (((int64_t)oc * p.KH + ky) * p.KW + kx) * p.IC;
                for (int ic = 0; ic < p.IC; ic++)
                    acc = fmaf(to_f32<T>(ip[ic]), to_f32<T>(wp[ic]), acc);
            }
        }
        float v = to_f32<TO>(bias[p.bias_n == 1 ? 0 : oc]) + acc;
        if (p.has_clamp)
        {
            v = (v < p.clamp_lo_f) ? p.clamp_lo_f : v;
            v = (v > p.clamp_hi_f) ? p.clamp_hi_f : v;
        }
        out[i] = from_f32<TO>(v);
    }
}

// CONV3D (reference_model/src/ops/tensor_ops.cpp:934-1120): input [N,ID,IH,IW,IC], weights [OC,KD,KH,KW,IC], one thread per
// output element, channel fastest; taps outside the input are skipped, order kd, ky, kx, ic.  `p` carries the height and
// width attributes, `z` the depth ones.
struct ConvDepthDev
{
    int ID, OD, KD, pad_d, sd, dd;
};

// CONV3D as a CONV2D: the depth taps of every output depth gathered beside the channels,
// out[n][od][pixel][kd][unit] = in[n][od * sd + kd * dd - pad_d][pixel][unit] (`fill` for a depth outside the input: the
// input zero point, so that the tap contributes nothing), `units` elements of type U per pixel; and the weights
// [OC][KD][KH][KW][units] re-ordered to [OC][KH][KW][KD][units].
template <typename U>
__global__ void conv3d_unfold_depth_kernel(const U* __restrict__ in, U* __restrict__ out, int N, int ID, int OD, int KD,
                                           int64_t pixels, int units, int sd, int dd, int pad_d, U fill)
{
    const int64_t total = (int64_t)N * OD * pixels * KD * units;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int u   = (int)(i % units);
        int64_t r     = i / units;
        const int kd  = (int)(r % KD);
        r /= KD;
        const int64_t px = r % pixels;
        r /= pixels;
        const int od = (int)(r % OD);
        const int n  = (int)(r / OD);
        const int d  = od * sd + kd * dd - pad_d;
        out[i]       = (d >= 0 && d < ID) ? in[(((int64_t)n * ID + d) * pixels + px) * units + u] : fill;
    }
}

template <typename U>
__global__ void conv3d_fold_weights_kernel(const U* __restrict__ w, U* __restrict__ out, int OC, int KD, int taps, int units)
{
    const int64_t total = (int64_t)OC * taps * KD * units;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int u  = (int)(i % units);
        int64_t r    = i / units;
        const int kd = (int)(r % KD);
        r /= KD;
        const int t  = (int)(r % taps);
        const int oc = (int)(r / taps);
        out[i]       = w[(((int64_t)oc * KD + kd) * taps + t) * units + u];
    }
}

template <typename TOut>
__global__ void conv3d_direct_i8_kernel(const int8_t* __restrict__ in, const int8_t* __restrict__ w,
                                        const int32_t* __restrict__ bias, TOut* __restrict__ out, ConvDev p, ConvDepthDev z,
                                        int* status)
{
    const int64_t total = (int64_t)p.N * z.OD * p.OH * p.OW * p.OC;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    bool bad            = false;
    const bool vec4     = (p.IC % 4) == 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int oc = (int)(i % p.OC);
        int64_t r    = i / p.OC;
        const int ox = (int)(r % p.OW);
        r /= p.OW;
        const int oy = (int)(r % p.OH);
        r /= p.OH;
        const int od = (int)(r % z.OD);
        const int n  = (int)(r / z.OD);
        int32_t acc  = 0;
        for (int kd = 0; kd < z.KD; kd++)
        {
            const int d = od * z.sd + kd * z.dd - z.pad_d;
            if (d < 0 || d >= z.ID)
                continue;
            for (int ky = 0; ky < p.KH; ky++)
            {
                const int y = oy * p.sy + ky * p.dy - p.pad_t;
                if (y < 0 || y >= p.IH)
                    continue;
                for (int kx = 0; kx < p.KW; kx++)
                {
                    const int x = ox * p.sx + kx * p.dx - p.pad_l;
                    if (x < 0 || x >= p.IW)
                        continue;
                    const int8_t* ip = in + ((((int64_t)n * z.ID + d) * p.IH + y) * p.IW + x) * p.IC;
                    const int8_t* wp = w + ((((int64_t)oc * z.KD + kd) * p.KH + ky) * p.KW + kx) * p.IC;
                    if (vec4)
                    {
                        // sum (a - za)(b - zb) = sum ab - zb sum a - za sum b + n za zb, four lanes at a time
                        int32_t sab = 0, sa = 0, sb = 0;
                        for (int ic = 0; ic < p.IC; ic += 4)
                        {
                            const int a4 = *reinterpret_cast<const int*>(ip + ic);
                            const int b4 = *reinterpret_cast<const int*>(wp + ic);
                            sab          = __dp4a(a4, b4, sab);
                            sa           = __dp4a(a4, 0x01010101, sa);
                            sb           = __dp4a(b4, 0x01010101, sb);
                        }
                        acc += sab - p.w_zp * sa - p.in_zp * sb + p.IC * p.in_zp * p.w_zp;
                    }
                    else
                    {
                        for (int ic = 0; ic < p.IC; ic++)
                            acc += ((int32_t)ip[ic] - p.in_zp) * ((int32_t)wp[ic] - p.w_zp);
                    }
                }
            }
        }
        int32_t v = (int32_t)((uint32_t)bias[p.bias_n == 1 ? 0 : oc] + (uint32_t)acc);
        if (p.has_rescale)
        {
            v = rescale_elem(v, oc, p.rs, bad);
            if (p.has_clamp)
            {
                v = v >= p.clamp_lo ? v : p.clamp_lo;
                v = v < p.clamp_hi ? v : p.clamp_hi;
            }
        }
        out[i] = (TOut)v;
    }
    if (bad)
        atomicOr(status, TB200_DEV_UNPREDICTABLE);
}

template <typename T>
__global__ void conv3d_direct_fp_kernel(const T* __restrict__ in, const T* __restrict__ w, const T* __restrict__ bias,
                                        T* __restrict__ out, ConvDev p, ConvDepthDev z)
{
    const int64_t total = (int64_t)p.N * z.OD * p.OH * p.OW * p.OC;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int oc = (int)(i % p.OC);
        int64_t r    = i / p.OC;
        const int ox = (int)(r % p.OW);
        r /= p.OW;
        const int oy = (int)(r % p.OH);
        r /= p.OH;
        const int od = (int)(r % z.OD);
        const int n  = (int)(r / z.OD);
        float acc    = 0.f;
        for (int kd = 0; kd < z.KD; kd++)
        {
            const int d = od * z.sd + kd * z.dd - z.pad_d;
            if (d < 0 || d >= z.ID)
                continue;
            for (int ky = 0; ky < p.KH; ky++)
            {
                const int y = oy * p.sy + ky * p.dy - p.pad_t;
                if (y < 0 || y >= p.IH)
                    continue;
                for (int kx = 0; kx < p.KW; kx++)
                {
                    const int x = ox * p.sx + kx * p.dx - p.pad_l;
                    if (x < 0 || x >= p.IW)
                        continue;
                    const T* ip = in + ((((int64_t)n * z.ID + d) * p.IH + y) * p.IW + x) * p.IC;
                    const T* wp = w + ((((int64_t)oc * z.KD + kd) * p.KH + ky) * p.KW + kx) * p.IC;
                    for (int ic = 0; ic < p.IC; ic++)
                        acc = fmaf(to_f32<T>(ip[ic]), to_f32<T>(wp[ic]), acc);
                }
            }
        }
        float v = to_f32<T>(bias[p.bias_n == 1 ? 0 : oc]) + acc;
        if (p.has_clamp)
        {
            v = (v < p.clamp_lo_f) ? p.clamp_lo_f : v;
            v = (v > p.clamp_hi_f) ? p.clamp_hi_f : v;
        }
        out[i] = from_f32<T>(v);
    }
}

// DEPTHWISE_CONV2D, weights [KH,KW,C,M], output channel c*M+m (reference_model/src/ops/tensor_ops.cpp:1283-1325)
template <typename TOut>
__global__ void depthwise_direct_i8_kernel(const int8_t* __restrict__ in, const int8_t* __restrict__ w,
                                           const int32_t* __restrict__ bias, TOut* __restrict__ out, ConvDev p,
                                           int* status)
{
    const int OC        = p.IC * p.M;
    const int64_t total = (int64_t)p.N * p.OH * p.OW * OC;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    bool bad            = false;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int oc = (int)(i % OC);
        int64_t r    = i / OC;
        const int ox = (int)(r % p.OW);
        r /= p.OW;
        const int oy = (int)(r % p.OH);
        const int n  = (int)(r / p.OH);
        const int c = oc / p.M, m = oc % p.M;
        int32_t acc = 0;
        for (int ky = 0; ky < p.KH; ky++)
        {
            const int y = oy * p.sy + ky * p.dy - p.pad_t;
            if (y < 0 || y >= p.IH)
                continue;
            for (int kx = 0; kx < p.KW; kx++)
            {
                const int x = ox * p.sx + kx * p.dx - p.pad_l;
                if (x < 0 || x >= p.IW)
                    continue;
                acc += ((int32_t)in[(((int64_t)n * p.IH + y) * p.IW + x) * p.IC + c] - p.in_zp) *
                       ((int32_t)w[(((int64_t)ky * p.KW + kx) * p.IC + c) * p.M + m] - p.w_zp);
            }
        }
        int32_t v = (int32_t)((uint32_t)bias[p.bias_n == 1 ? 0 : oc] + (uint32_t)acc);
        if (p.has_rescale)
        {
            v = rescale_elem(v, oc, p.rs, bad);
            if (p.has_clamp)
            {
                v = v >= p.clamp_lo ? v : p.clamp_lo;
                v = v < p.clamp_hi ? v : p.clamp_hi;
            }
        }
        out[i] = (TOut)v;
    }
    if (bad)
        atomicOr(status, TB200_DEV_UNPREDICTABLE);
}

template <typename T, typename TO = T>
__global__ void depthwise_direct_fp_kernel(const T* __restrict__ in, const T* __restrict__ w,
                                           const TO* __restrict__ bias, TO* __restrict__ out, ConvDev p)
{
    const int OC        = p.IC * p.M;
    const int64_t total = (int64_t)p.N * p.OH * p.OW * OC;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int oc = (int)(i % OC);
        int64_t r    = i / OC;
        const int ox = (int)(r % p.OW);
        r /= p.OW;
        const int oy = (int)(r % p.OH);
        const int n  = (int)(r / p.OH);
        const int c = oc / p.M, m = oc % p.M;
        float acc = 0.f;
        for (int ky = 0; ky < p.KH; ky++)
        {
            const int y = oy * p.sy + ky * p.dy - p.pad_t;
            if (y < 0 || y >= p.IH)
                continue;
            for (int kx = 0; kx < p.KW; kx++)
            {
                const int x = ox * p.sx + kx * p.dx - p.pad_l;
                if (x < 0 || x >= p.IW)
                    continue;
                acc = fmaf(to_f32<T>(in[(((int64_t)n * p.IH + y) * p.IW + x) * p.IC + c]),
                           to_f32<T>(w[(((int64_t)ky * p.KW + kx) * p.IC + c) * p.M + m]), acc);
            }
        }
        float v = to_f32<TO>(bias[p.bias_n == 1 ? 0 : oc]) + acc;
        if (p.has_clamp)
        {
            v = (v < p.clamp_lo_f) ? p.clamp_lo_f : v;
            v = (v > p.clamp_hi_f) ? p.clamp_hi_f : v;
        }
        out[i] = from_f32<TO>(v);
    }
}

// int8 DEPTHWISE_CONV2D with a 3 x 3 window, multiplier 1, no dilation: sixteen channels (one 128-bit load) per thread.
// sum (x - zx)(w - zw) over the in-scope taps = sum x w - zw sum x - zx sum w + taps zx zw, each sum per channel: a dp4a
// whose second operand has one live byte picks one channel out of a 32-bit word (the weight word masked to that byte
// for x w, the constant 1 in that byte for the plain sums).  Same accumulator, bias and fused RESCALE / CLAMP as
// depthwise_direct_i8_kernel (the one-thread-per-output form measured 1.27 ms on 64 x 112 x 112 x 192 with stride 2).
template <typename TOut>
__global__ void depthwise3x3_i8x16_kernel(const int8_t* __restrict__ in, const int8_t* __restrict__ w,
                                          const int32_t* __restrict__ bias, TOut* __restrict__ out, ConvDev p, int* status)
{
    const int cv        = p.IC / 16;
    const int64_t total = (int64_t)p.N * p.OH * p.OW * cv;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    bool bad            = false;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int c16 = (int)(i % cv) * 16;
        int64_t r     = i / cv;
        const int ox  = (int)(r % p.OW);
        r /= p.OW;
        const int oy = (int)(r % p.OH);
        const int n  = (int)(r / p.OH);
        const int y0 = oy * p.sy - p.pad_t, x0 = ox * p.sx - p.pad_l;
        int32_t sxw[16], sx[16], sw[16];
#pragma unroll
        for (int j = 0; j < 16; j++)
            sxw[j] = sx[j] = sw[j] = 0;
        int taps = 0;
#pragma unroll
        for (int ky = 0; ky < 3; ky++)
#pragma unroll
            for (int kx = 0; kx < 3; kx++)
            {
                const int y = y0 + ky, x = x0 + kx;
                if (y < 0 || y >= p.IH || x < 0 || x >= p.IW)
                    continue;    // the reference skips taps outside the image
                const int4 xv = __ldg(reinterpret_cast<const int4*>(in + (((int64_t)n * p.IH + y) * p.IW + x) * p.IC + c16));
                const int4 wv = __ldg(reinterpret_cast<const int4*>(w + (int64_t)(ky * 3 + kx) * p.IC + c16));
                const int xw[4] = { xv.x, xv.y, xv.z, xv.w };
                const int ww[4] = { wv.x, wv.y, wv.z, wv.w };
                taps++;
#pragma unroll
                for (int q = 0; q < 4; q++)
#pragma unroll
                    for (int b = 0; b < 4; b++)
                    {
                        const int sel    = 0xff << (8 * b);
                        sxw[4 * q + b]   = __dp4a(xw[q], ww[q] & sel, sxw[4 * q + b]);
                        if (p.in_zp != 0)
                            sw[4 * q + b] = __dp4a(ww[q], 0x01 << (8 * b), sw[4 * q + b]);
                        if (p.w_zp != 0)
                            sx[4 * q + b] = __dp4a(xw[q], 0x01 << (8 * b), sx[4 * q + b]);
                    }
            }
        int32_t v[16];
#pragma unroll
        for (int j = 0; j < 16; j++)
        {
            // int32 arithmetic wraps, like the reference's accumulator
            const uint32_t acc = (uint32_t)sxw[j] - (uint32_t)p.w_zp * (uint32_t)sx[j] - (uint32_t)p.in_zp * (uint32_t)sw[j] +
                                 (uint32_t)taps * (uint32_t)(p.in_zp * p.w_zp);
            int32_t o = (int32_t)((uint32_t)bias[p.bias_n == 1 ? 0 : c16 + j] + acc);
            if (p.has_rescale)
            {
                o = rescale_elem(o, c16 + j, p.rs, bad);
                if (p.has_clamp)
                {
                    o = o >= p.clamp_lo ? o : p.clamp_lo;
                    o = o < p.clamp_hi ? o : p.clamp_hi;
                }
            }
            v[j] = o;
        }
        TOut* op = out + (((int64_t)n * p.OH + oy) * p.OW + ox) * p.IC + c16;
        if (sizeof(TOut) == 1)
        {
            uint32_t pk[4];
#pragma unroll
            for (int q = 0; q < 4; q++)
                pk[q] = ((uint32_t)v[4 * q] & 0xffu) | (((uint32_t)v[4 * q + 1] & 0xffu) << 8) | (((uint32_t)v[4 * q + 2] & 0xffu) << 16) |
                        (((uint32_t)v[4 * q + 3] & 0xffu) << 24);
            *reinterpret_cast<uint4*>(op) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
        else
        {
#pragma unroll
            for (int j = 0; j < 16; j++)
                op[j] = (TOut)v[j];
        }
    }
    if (bad)
        atomicOr(status, TB200_DEV_UNPREDICTABLE);
}

// Depthwise, multiplier 1, 8 channels (one 128-bit load) per thread, fp16 / bf16 storage, fp32 accumulation.
template <typename T>
__global__ void depthwise_fp_x8_kernel(const T* __restrict__ in, const T* __restrict__ w, const T* __restrict__ bias,
                                       T* __restrict__ out, ConvDev p)
{
    const int cv        = p.IC / 8;
    const int64_t total = (int64_t)p.N * p.OH * p.OW * cv;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int c8 = (int)(i % cv) * 8;
        int64_t r    = i / cv;
        const int ox = (int)(r % p.OW);
        r /= p.OW;
        const int oy = (int)(r % p.OH);
        const int n  = (int)(r / p.OH);
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; j++)
            acc[j] = 0.f;
        for (int ky = 0; ky < p.KH; ky++)
        {
            const int y = oy * p.sy + ky * p.dy - p.pad_t;
            if (y < 0 || y >= p.IH)
                continue;
            for (int kx = 0; kx < p.KW; kx++)
            {
                const int x = ox * p.sx + kx * p.dx - p.pad_l;
                if (x < 0 || x >= p.IW)
                    continue;
                T vi[8], vw[8];
                *reinterpret_cast<int4*>(vi) =
                    *reinterpret_cast<const int4*>(in + (((int64_t)n * p.IH + y) * p.IW + x) * p.IC + c8);
                *reinterpret_cast<int4*>(vw) =
                    *reinterpret_cast<const int4*>(w + ((int64_t)ky * p.KW + kx) * p.IC + c8);
#pragma unroll
                for (int j = 0; j < 8; j++)
                    acc[j] = fmaf(to_f32<T>(vi[j]), to_f32<T>(vw[j]), acc[j]);
            }
        }
        T vo[8];
#pragma unroll
        for (int j = 0; j < 8; j++)
        {
            float v = to_f32<T>(bias[p.bias_n == 1 ? 0 : c8 + j]) + acc[j];
            if (p.has_clamp)
            {
                v = (v < p.clamp_lo_f) ? p.clamp_lo_f : v;
                v = (v > p.clamp_hi_f) ? p.clamp_hi_f : v;
            }
            vo[j] = from_f32<T>(v);
        }
        *reinterpret_cast<int4*>(out + (((int64_t)n * p.OH + oy) * p.OW + ox) * p.IC + c8) =
            *reinterpret_cast<int4*>(vo);
    }
}

// The same for a 3 x 3 window without dilation: the nine input loads are issued before the first multiply-add (taps
// outside the image load nothing and contribute a zero vector, added in its place so the accumulation order is the
// reference's), so a thread waits for memory once.
template <typename T>
__global__ void depthwise3x3_fp_x8_kernel(const T* __restrict__ in, const T* __restrict__ w, const T* __restrict__ bias,
                                          T* __restrict__ out, ConvDev p)
{
    const int cv        = p.IC / 8;
    const int64_t total = (int64_t)p.N * p.OH * p.OW * cv;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int c8 = (int)(i % cv) * 8;
        int64_t r    = i / cv;
        const int ox = (int)(r % p.OW);
        r /= p.OW;
        const int oy = (int)(r % p.OH);
        const int n  = (int)(r / p.OH);
        const int y0 = oy * p.sy - p.pad_t, x0 = ox * p.sx - p.pad_l;
        int4 vin[9];
        bool ok[9];
#pragma unroll
        for (int ky = 0; ky < 3; ky++)
#pragma unroll
            for (int kx = 0; kx < 3; kx++)
            {
                const int y = y0 + ky, x = x0 + kx;
                const int t = ky * 3 + kx;
                ok[t]       = y >= 0 && y < p.IH && x >= 0 && x < p.IW;
                vin[t]      = make_int4(0, 0, 0, 0);
                if (ok[t])
                    vin[t] = __ldg(reinterpret_cast<const int4*>(in + (((int64_t)n * p.IH + y) * p.IW + x) * p.IC + c8));
            }
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; j++)
            acc[j] = 0.f;
#pragma unroll
        for (int t = 0; t < 9; t++)
        {
            if (!ok[t])
                continue;    // the reference skips taps outside the image: nothing is added for them
            T vi[8], vw[8];
            *reinterpret_cast<int4*>(vi) = vin[t];
            *reinterpret_cast<int4*>(vw) = __ldg(reinterpret_cast<const int4*>(w + (int64_t)t * p.IC + c8));
#pragma unroll
            for (int j = 0; j < 8; j++)
                acc[j] = fmaf(to_f32<T>(vi[j]), to_f32<T>(vw[j]), acc[j]);
        }
        T vo[8];
#pragma unroll
        for (int j = 0; j < 8; j++)
        {
            float v = to_f32<T>(bias[p.bias_n == 1 ? 0 : c8 + j]) + acc[j];
            if (p.has_clamp)
            {
                v = (v < p.clamp_lo_f) ? p.clamp_lo_f : v;
                v = (v > p.clamp_hi_f) ? p.clamp_hi_f : v;
            }
            vo[j] = from_f32<T>(v);
        }
        *reinterpret_cast<int4*>(out + (((int64_t)n * p.OH + oy) * p.OW + ox) * p.IC + c8) =
            *reinterpret_cast<int4*>(vo);
    }
}

// ------------------------------------------------------------------------------------------------ direct matmul
__global__ void matmul_direct_i8_kernel(const int8_t* __restrict__ a, const int8_t* __restrict__ b,
                                        int32_t* __restrict__ out, int N, int H, int C, int W, int32_t a_zp,
                                        int32_t b_zp)
{
    const int64_t total = (int64_t)N * H * W;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int wc = (int)(i % W);
        int64_t r    = i / W;
        const int h  = (int)(r % H);
        const int n  = (int)(r / H);
        const int8_t* ap = a + ((int64_t)n * H + h) * C;
        const int8_t* bp = b + (int64_t)n * C * W + wc;
        int32_t acc = 0;
        for (int c = 0; c < C; c++)
            acc += ((int32_t)ap[c] - a_zp) * ((int32_t)bp[(int64_t)c * W] - b_zp);
        out[i] = acc;
    }
}

template <typename T, typename TOut, typename TB = T>
__global__ void matmul_direct_fp_kernel(const T* __restrict__ a, const TB* __restrict__ b, TOut* __restrict__ out,
                                        int N, int H, int C, int W)
{
    const int64_t total = (int64_t)N * H * W;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int wc = (int)(i % W);
        int64_t r    = i / W;
        const int h  = (int)(r % H);
        const int n  = (int)(r / H);
        const T* ap  = a + ((int64_t)n * H + h) * C;
        const TB* bp = b + (int64_t)n * C * W + wc;
        float acc    = 0.f;
        for (int c = 0; c < C; c++)
            acc = fmaf(to_f32<T>(ap[c]), to_f32<TB>(bp[(int64_t)c * W]), acc);
        out[i] = from_f32<TOut>(acc);
    }
}

// ------------------------------------------------------------------------------------------------ preparation
// MATMUL zero points: sum (a - za)(b - zb) = sum ab - zb rowsum(a) - za colsum(b) + C za zb.
// row_corr[n*H + h] = -zb * rowsum(A[n,h,:]) + C za zb ; one warp per row.
__global__ void matmul_row_corr_kernel(const int8_t* __restrict__ a, int32_t* __restrict__ row_corr, int64_t rows,
                                       int C, int32_t a_zp, int32_t b_zp)
{
    const int lane     = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nw   = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = warp; r < rows; r += nw)
    {
        const int8_t* ap = a + r * C;
        int32_t s        = 0;
        if ((C & 15) == 0)
        {
            for (int c = lane * 16; c < C; c += 32 * 16)
            {
                const int4 v = *reinterpret_cast<const int4*>(ap + c);
                s = __dp4a(v.x, 0x01010101, s);
                s = __dp4a(v.y, 0x01010101, s);
                s = __dp4a(v.z, 0x01010101, s);
                s = __dp4a(v.w, 0x01010101, s);
            }
        }
        else
        {
            for (int c = lane; c < C; c += 32)
                s += ap[c];
        }
        for (int o = 16; o > 0; o >>= 1)
            s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0)
            row_corr[r] = -b_zp * s + C * a_zp * b_zp;
    }
}

// col_corr[n*Wpad + w] += -za * sum over this block's K range of B[n,k,w].  The destination (stride Wpad, zeroed by
// the caller) receives one atomic add per K split.  Block = 8 warps; a warp row covers 512 columns (16 per lane,
// one 128-bit load); warps interleave over the K range.
__global__ void __launch_bounds__(256) matmul_col_corr_kernel(const int8_t* __restrict__ b, int32_t* __restrict__ col_corr,
                                                              int C, int W, int Wpad, int k_per_block, int32_t a_zp)
{
    __shared__ int32_t part[8][512];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n    = blockIdx.z;
    const int col0 = blockIdx.x * 512 + lane * 16;
    const int k0   = blockIdx.y * k_per_block;
    const int k1   = min(C, k0 + k_per_block);
    const int8_t* bp = b + (int64_t)n * C * W;
    int32_t s[16];
#pragma unroll
    for (int j = 0; j < 16; j++)
        s[j] = 0;
    if ((W & 15) == 0)
    {
        if (col0 < W)
        {
            // four rows per pass, all four loads issued before the arithmetic (memory-level parallelism)
            const int8_t* rp = bp + (int64_t)(k0 + warp) * W + col0;
            const int64_t rstep = (int64_t)8 * W;
            int k = k0 + warp;
            for (; k + 24 < k1; k += 32, rp += 4 * rstep)
            {
                int4 v[4];
#pragma unroll
                for (int u = 0; u < 4; u++)
                    v[u] = __ldg(reinterpret_cast<const int4*>(rp + u * rstep));
#pragma unroll
                for (int u = 0; u < 4; u++)
                {
                    const int w4[4] = { v[u].x, v[u].y, v[u].z, v[u].w };
#pragma unroll
                    for (int q = 0; q < 4; q++)
                    {
                        s[4 * q + 0] = __dp4a(w4[q], 0x00000001, s[4 * q + 0]);
                        s[4 * q + 1] = __dp4a(w4[q], 0x00000100, s[4 * q + 1]);
                        s[4 * q + 2] = __dp4a(w4[q], 0x00010000, s[4 * q + 2]);
                        s[4 * q + 3] = __dp4a(w4[q], 0x01000000, s[4 * q + 3]);
                    }
                }
            }
            for (; k < k1; k += 8, rp += rstep)
            {
                const int4 v = __ldg(reinterpret_cast<const int4*>(rp));
                const int w4[4] = { v.x, v.y, v.z, v.w };
#pragma unroll
                for (int q = 0; q < 4; q++)
                {
                    s[4 * q + 0] = __dp4a(w4[q], 0x00000001, s[4 * q + 0]);
                    s[4 * q + 1] = __dp4a(w4[q], 0x00000100, s[4 * q + 1]);
                    s[4 * q + 2] = __dp4a(w4[q], 0x00010000, s[4 * q + 2]);
                    s[4 * q + 3] = __dp4a(w4[q], 0x01000000, s[4 * q + 3]);
                }
            }
        }
    }
    else
    {
        for (int k = k0 + warp; k < k1; k += 8)
#pragma unroll
            for (int j = 0; j < 16; j++)
                if (col0 + j < W)
                    s[j] += bp[(int64_t)k * W + col0 + j];
    }
#pragma unroll
    for (int j = 0; j < 16; j++)
        part[warp][lane * 16 + j] = s[j];
    __syncthreads();
    for (int c = threadIdx.x; c < 512; c += 256)
    {
        int32_t t = 0;
#pragma unroll
        for (int g = 0; g < 8; g++)
            t += part[g][c];
        const int col = blockIdx.x * 512 + c;
        if (col < W && t != 0)
            atomicAdd(&col_corr[(int64_t)n * Wpad + col], -a_zp * t);
    }
}

// CONV2D epilogue constants for int8 weights OHWI with weight_zp == 0, one warp per padded output channel:
//   prefix[OC][(KH+1)(KW+1)]  scratch: inclusive 2-D prefix sums over taps of sum_ic w[oc,ky,kx,ic]
//   corr[classes][OCpad]      bias[oc] - in_zp * (sum of the weights of the in-scope taps).  With `classes` the table
//                             has (KH+1)^2 (KW+1)^2 rows indexed ((ky_lo*(KH+1)+ky_hi)*(KW+1)+kx_lo)*(KW+1)+kx_hi;
//                             otherwise a single row for the full filter
//   mult_pad / shift_pad      RESCALE operands expanded per channel (per_channel == 0 repeats element 0), zero padded
// Also writes, when `rec` is given, one record per column for the tensor-core epilogue's lean RESCALE form (see
// rescale_rec_build) and, for padded layers with an input zero point, `delta`: per class of clipped tap rectangle the
// difference between that class's correction row and the interior one (all taps in scope), which border pixels add
// to their accumulators before the common arithmetic.  `all_ok`, preset to non-zero by the caller, is cleared when some
// column's record is unusable.
__global__ void conv_epilogue_tables_kernel(const int8_t* __restrict__ w, const int32_t* __restrict__ bias, int bias_n,
                                            int OC, int OCpad, int KH, int KW, int IC, int32_t in_zp, int classes,
                                            const int32_t* __restrict__ mult, const int8_t* __restrict__ shift,
                                            int per_channel, int32_t* __restrict__ prefix, int32_t* __restrict__ corr,
                                            int32_t* __restrict__ mult_pad, int8_t* __restrict__ shift_pad,
                                            int32_t* __restrict__ rec = nullptr, int32_t* __restrict__ delta = nullptr,
                                            int double_round = 0, int32_t out_zp = 0, int* __restrict__ all_ok = nullptr)
{
    // One warp per output channel: lanes split the channel run of each tap (128-bit loads), the warp-reduced tap
    // sums become 2-D prefix sums kept in registers by lane 0 .. and mirrored to `prefix` for the class loop, which
    // the lanes split again.
    const int lane = threadIdx.x & 31;
    const int oc   = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (oc >= OCpad)
        return;
    const int W1 = KW + 1, H1 = KH + 1;
    const int ncls = classes ? H1 * H1 * W1 * W1 : 1;
    if (oc >= OC)
    {
        for (int c = lane; c < ncls; c += 32)
        {
            corr[(int64_t)c * OCpad + oc] = 0;
            if (delta)
                delta[(int64_t)c * OCpad + oc] = 0;
        }
        if (mult_pad && lane == 0)
        {
            mult_pad[oc]  = 0;
            shift_pad[oc] = 2;
        }
        if (rec && lane < 8)
            rec[(int64_t)oc * 8 + lane] = lane == 7 ? 1 : 0;    // a padding column never disqualifies its block
        return;
    }
    int32_t* P = prefix + (int64_t)oc * H1 * W1;    // this channel's (KH+1) x (KW+1) prefix sums
    for (int ky = 0; ky <= KH; ky++)
        for (int kx = 0; kx <= KW; kx++)
        {
            int32_t v = 0;
            if (ky > 0 && kx > 0)
            {
                const int8_t* wp = w + (((int64_t)oc * KH + (ky - 1)) * KW + (kx - 1)) * IC;
                int32_t s        = 0;
                if ((IC & 15) == 0)
                {
                    for (int ic = lane * 16; ic < IC; ic += 512)
                    {
                        const int4 q = __ldg(reinterpret_cast<const int4*>(wp + ic));
                        s = __dp4a(q.x, 0x01010101, s);
                        s = __dp4a(q.y, 0x01010101, s);
                        s = __dp4a(q.z, 0x01010101, s);
                        s = __dp4a(q.w, 0x01010101, s);
                    }
                }
                else
                {
                    for (int ic = lane; ic < IC; ic += 32)
                        s += wp[ic];
                }
                for (int o = 16; o > 0; o >>= 1)
                    s += __shfl_xor_sync(0xffffffffu, s, o);
                v = s;
            }
            if (lane == 0)
            {
                if (ky > 0 && kx > 0)
                    v += P[(ky - 1) * W1 + kx] + P[ky * W1 + kx - 1] - P[(ky - 1) * W1 + kx - 1];
                P[ky * W1 + kx] = v;
            }
        }
    __syncwarp();
    const int32_t b = bias[bias_n == 1 ? 0 : oc];
    const int32_t corr_interior = b - in_zp * P[KH * W1 + KW];    // every tap in scope
    if (!classes)
    {
        if (lane == 0)
            corr[oc] = corr_interior;
    }
    else
    {
        for (int c = lane; c < ncls; c += 32)
        {
            const int xh = c % W1, xl = (c / W1) % W1, yh = (c / (W1 * W1)) % H1, yl = c / (W1 * W1 * H1);
            int32_t rs = 0;
            if (yh > yl && xh > xl)
                rs = P[yh * W1 + xh] - P[yl * W1 + xh] - P[yh * W1 + xl] + P[yl * W1 + xl];
            corr[(int64_t)c * OCpad + oc] = b - in_zp * rs;
            if (delta)
                delta[(int64_t)c * OCpad + oc] = (b - in_zp * rs) - corr_interior;
        }
    }
    if (mult_pad && lane == 0)
    {
        mult_pad[oc]  = mult[per_channel ? oc : 0];
        shift_pad[oc] = shift[per_channel ? oc : 0];
    }
    if (rec && lane == 0)
    {
        // largest magnitude bias + accumulator can reach: every tap at full scale |x - zp| <= 255, |w| <= 128
        const int64_t vmax = (int64_t)KH * KW * IC * 255 * 128 + (b < 0 ? -(int64_t)b : (int64_t)b);
        int32_t r8[8];
        rescale_rec_build(mult[per_channel ? oc : 0], (int32_t)shift[per_channel ? oc : 0], double_round, out_zp,
                          corr_interior, vmax, r8);
#pragma unroll
        for (int i = 0; i < 8; i++)
            rec[(int64_t)oc * 8 + i] = r8[i];
        // one word for the host (preset to non-zero): does every column of the layer have a usable record?
        if (all_ok != nullptr && r8[7] == 0)
            *all_ok = 0;
    }
}

// TRANSPOSE_CONV2D as a convolution: the input is spread out with (stride - 1) fill pixels between neighbours
// (fill = the input zero point, which the convolution subtracts to 0) and the kernel is mirrored in both spatial
// axes; a stride-1 CONV2D over that pair gives OpTransposeConv2d::eval's sums term by term
// (reference_model/src/ops/tensor_ops.cpp:2148-2171: tap (ky, kx) of output y reads input (y - out_pad - ky) / stride
// when that division is exact).  U is the copy unit: 16 bytes when a pixel's channel run allows it, else one element.
template <typename U>
__global__ void spread_pixels_kernel(const U* __restrict__ in, U* __restrict__ out, int N, int IH, int IW, int units,
                                     int DH, int DW, int sy, int sx, U fill)
{
    const int64_t total = (int64_t)N * DH * DW * units;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int u  = (int)(i % units);
        int64_t r    = i / units;
        const int dx = (int)(r % DW);
        r /= DW;
        const int dy = (int)(r % DH);
        const int n  = (int)(r / DH);
        U v          = fill;
        if ((dy % sy) == 0 && (dx % sx) == 0)
            v = in[(((int64_t)n * IH + dy / sy) * IW + dx / sx) * units + u];
        out[i] = v;
    }
}

// OHWI weights, every (sy, sx)-th tap starting at (ky0, kx0), mirrored:
// out[oc][ty][tx][:] = in[oc][ky0 + sy*(Ty-1-ty)][kx0 + sx*(Tx-1-tx)][:].  (0, 1, KH, 0, 1, KW) mirrors the whole kernel;
// a phase of a strided TRANSPOSE_CONV2D uses the taps congruent to its offset.
template <typename U>
__global__ void mirror_weights_kernel(const U* __restrict__ in, U* __restrict__ out, int OC, int KH, int KW, int units,
                                      int ky0, int sy, int Ty, int kx0, int sx, int Tx)
{
    const int64_t total = (int64_t)OC * Ty * Tx * units;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int u  = (int)(i % units);
        int64_t r    = i / units;
        const int tx = (int)(r % Tx);
        r /= Tx;
        const int ty = (int)(r % Ty);
        const int oc = (int)(r / Ty);
        const int ky = ky0 + sy * (Ty - 1 - ty), kx = kx0 + sx * (Tx - 1 - tx);
        out[i]       = in[(((int64_t)oc * KH + ky) * KW + kx) * units + u];
    }
}

// The sub-kernels of every phase of a strided TRANSPOSE_CONV2D in one launch: phase i owns the work items
// [first[i], first[i+1]) and writes its mirrored taps at out + out_off[i] (both in copy units).
struct PhaseWeights
{
    enum { kMax = 64 };
    int count;
    int ky0[kMax], Ty[kMax], kx0[kMax], Tx[kMax];
    long long out_off[kMax], first[kMax + 1];
};

template <typename U>
__global__ void mirror_phase_weights_kernel(const U* __restrict__ in, U* __restrict__ out, int OC, int KH, int KW, int units,
                                            int sy, int sx, const __grid_constant__ PhaseWeights ph)
{
    const int64_t total = ph.first[ph.count];
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += step)
    {
        int p = 0;
        while (p + 1 < ph.count && g >= ph.first[p + 1])
            p++;
        int64_t i    = g - ph.first[p];
        const int Ty = ph.Ty[p], Tx = ph.Tx[p];
        const int u  = (int)(i % units);
        int64_t r    = i / units;
        const int tx = (int)(r % Tx);
        r /= Tx;
        const int ty = (int)(r % Ty);
        const int oc = (int)(r / Ty);
        const int ky = ph.ky0[p] + sy * (Ty - 1 - ty), kx = ph.kx0[p] + sx * (Tx - 1 - tx);
        out[ph.out_off[p] + i] = in[(((int64_t)oc * KH + ky) * KW + kx) * units + u];
    }
}

// TRANSPOSE_CONV2D as ONE stride-1 convolution whose output columns are (py, px, oc): phase (py, px) of the output
// (rows py mod sy, columns px mod sx) reads, for macro-pixel (j, i), the input rows j + c_py - t with tap
// k0_py + sy*t.  Over all phases these rows lie in one window of U rows ending at j + cmax, so every phase's taps are
// embedded (mirrored, zero elsewhere) in a U_y x U_x kernel and the phases become column blocks of one GEMM.  One
// launch prepares its operands: the embedded weights [(py*sx + px)*OC + oc][U_y][U_x][IC] and the per-channel vectors
// (bias, RESCALE multiplier and shift; null = absent) repeated per block, copied as raw 1-, 2- or 4-byte words.
struct PhaseEmbed
{
    enum { kMax = 8 };               // phases per axis
    int sy, sx, Uy, Ux;
    int k0y[kMax], Ty[kMax], shy[kMax];    // first tap, tap count, window shift (cmax - c) of every y phase
    int k0x[kMax], Tx[kMax], shx[kMax];
};

template <typename U>
__global__ void embed_phase_operands_kernel(const U* __restrict__ w, U* __restrict__ w_out, int OC, int KH, int KW, int units,
                                            const __grid_constant__ PhaseEmbed e, const void* __restrict__ bias,
                                            void* __restrict__ bias_out, int bias_es, const void* __restrict__ mult,
                                            void* __restrict__ mult_out, int mult_es, const uint8_t* __restrict__ shift,
                                            uint8_t* __restrict__ shift_out)
{
    const int blocks    = e.sy * e.sx;
    const int64_t total = (int64_t)blocks * OC * e.Uy * e.Ux * units;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    const int64_t first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (int64_t i = first; i < total; i += step)
    {
        const int u  = (int)(i % units);
        int64_t r    = i / units;
        const int ux = e.Ux - 1 - (int)(r % e.Ux);    // stored mirrored: the convolution walks the window forwards
        r /= e.Ux;
        const int uy = e.Uy - 1 - (int)(r % e.Uy);
        r /= e.Uy;
        const int oc = (int)(r % OC);
        const int b  = (int)(r / OC);
        const int py = b / e.sx, px = b - py * e.sx;
        const int ty = uy - e.shy[py], tx = ux - e.shx[px];
        U v;
        memset(&v, 0, sizeof(U));
        if (ty >= 0 && ty < e.Ty[py] && tx >= 0 && tx < e.Tx[px])
            v = w[(((int64_t)oc * KH + e.k0y[py] + e.sy * ty) * KW + e.k0x[px] + e.sx * tx) * units + u];
        w_out[i] = v;
    }
    auto copy_word = [](const void* src, void* dst, int es, int from, int to) {
        if (es == 4)
            reinterpret_cast<uint32_t*>(dst)[to] = reinterpret_cast<const uint32_t*>(src)[from];
        else if (es == 2)
            reinterpret_cast<uint16_t*>(dst)[to] = reinterpret_cast<const uint16_t*>(src)[from];
        else
            reinterpret_cast<uint8_t*>(dst)[to] = reinterpret_cast<const uint8_t*>(src)[from];
    };
    for (int64_t c = first; c < (int64_t)OC * blocks; c += step)
    {
        const int oc = (int)(c % OC);
        if (bias != nullptr)
            copy_word(bias, bias_out, bias_es, oc, (int)c);
        if (mult != nullptr)
            copy_word(mult, mult_out, mult_es, oc, (int)c);
        if (shift != nullptr)
            shift_out[c] = shift[oc];
    }
}

// Few-channel convolutions (an RGB stem) on the tensor cores.  The image is copied once into a border-padded,
// channel-padded buffer  xp[N][Hp][Wp][Cp]  (border and slack filled with the input zero point, pad channels with
// anything: their weights are zero).  With Cp * stride_x a multiple of 16 bytes, the KW taps of one filter row are
// one contiguous window of `win` bytes per output pixel, so the convolution becomes a KH-tap implicit GEMM whose
// "channel" run is that window.
__global__ void pad_expand_i8_kernel(const int8_t* __restrict__ in, int8_t* __restrict__ xp, int N, int IH, int IW, int IC,
                                     int Hp, int Wp, int Cp, int pad_t, int pad_l, int32_t zp)
{
    const int64_t total = (int64_t)N * Hp * Wp;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int xpix = (int)(i % Wp);
        int64_t r      = i / Wp;
        const int ypix = (int)(r % Hp);
        const int n    = (int)(r / Hp);
        const int y = ypix - pad_t, x = xpix - pad_l;
        const bool inside = (y >= 0) && (y < IH) && (x >= 0) && (x < IW);
        const int8_t* src = in + (((int64_t)n * IH + y) * IW + x) * IC;
        int8_t v[16];
#pragma unroll
        for (int c = 0; c < 16; c++)
            v[c] = (int8_t)zp;
        if (inside)
            for (int c = 0; c < IC; c++)
                v[c] = src[c];
        int8_t* dst = xp + i * Cp;
        if (Cp == 8)
            *reinterpret_cast<int2*>(dst) = *reinterpret_cast<int2*>(v);
        else
            *reinterpret_cast<int4*>(dst) = *reinterpret_cast<int4*>(v);
    }
}

// Few-channel input for a stride-2 window, four bytes per pixel, one copy per parity of the output column:
// xq[n][p][y][xi] (4 bytes) = padded pixel (y, xi + 2 p), the input zero point outside the image.  The KW <= 8 taps of
// output column 2 ox' + p then start at byte 16 ox' of row y of copy p, which is the 16-byte pitch a TMA row needs;
// with one copy and eight bytes per pixel the same window is 64 bytes, twice the MMAs.  Four pixels per thread.
__global__ void pad_expand_parity_i8_kernel(const int8_t* __restrict__ in, int8_t* __restrict__ xq, int N, int IH, int IW, int IC,
                                            int Hp, int Wq, int pad_t, int pad_l, int32_t zp)
{
    const int wq4       = Wq / 4;
    const int64_t total = (int64_t)N * 2 * Hp * wq4;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    const uint32_t zp4  = (uint32_t)(zp & 0xff) * 0x01010101u;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int g    = (int)(i % wq4);
        int64_t r      = i / wq4;
        const int ypix = (int)(r % Hp);
        r /= Hp;
        const int par = (int)(r & 1);
        const int n   = (int)(r >> 1);
        const int y   = ypix - pad_t;
        uint32_t v[4];
#pragma unroll
        for (int j = 0; j < 4; j++)
        {
            const int x = g * 4 + j + 2 * par - pad_l;
            uint32_t w  = zp4;
            if (y >= 0 && y < IH && x >= 0 && x < IW)
            {
                const int8_t* src = in + (((int64_t)n * IH + y) * IW + x) * IC;
                for (int c = 0; c < IC; c++)
                    w = (w & ~(0xffu << (8 * c))) | ((uint32_t)(uint8_t)src[c] << (8 * c));
            }
            v[j] = w;
        }
        *reinterpret_cast<uint4*>(xq + i * 16) = make_uint4(v[0], v[1], v[2], v[3]);
    }
}

// weights OHWI [OC][KH][KW][IC] -> [OC][KH][win] with win >= KW*Cp, element (kx*Cp + c) = w[oc][ky][kx][c], rest 0
__global__ void repack_weights_smallc_kernel(const int8_t* __restrict__ w, int8_t* __restrict__ wr, int OC, int KH, int KW,
                                             int IC, int Cp, int win)
{
    const int64_t total = (int64_t)OC * KH * win;
    const int64_t i     = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total)
        return;
    const int k  = (int)(i % win);
    const int64_t r = i / win;
    const int ky = (int)(r % KH);
    const int oc = (int)(r / KH);
    const int kx = k / Cp, c = k % Cp;
    int8_t v = 0;
    if (kx < KW && c < IC)
        v = w[(((int64_t)oc * KH + ky) * KW + kx) * IC + c];
    wr[i] = v;
}

// fp bias widened to fp32 and zero padded for the tensor-core epilogue (bias_n == 1 broadcasts)
template <typename T>
__global__ void bias_to_f32_kernel(const T* __restrict__ bias, int bias_n, int OC, float* __restrict__ out, int OCpad)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < OCpad)
        out[i] = i < OC ? to_f32<T>(bias[bias_n == 1 ? 0 : i]) : 0.f;
}

}    // namespace tb200
