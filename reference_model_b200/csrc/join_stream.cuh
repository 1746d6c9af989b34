// Residual join of a quantized graph (RESCALE x2, ADD, RESCALE, CLAMP with per-tensor parameters) as a byte-pair table
// lookup, streaming form: the two operands come into shared memory through a ring of bulk copies issued by one thread,
// so that the bytes in flight per SM do not depend on registers or occupancy (the plain kernel keeps four 16-byte loads
// per thread in flight and waits for memory: 4.7 of 6.5 TB/s); the other warps read the operands from shared memory,
// look the result bytes up and store them.  Equivalent to the five reference nodes evaluated one after another
// (reference_model/src/ops/type_conversion.cpp:223-422, reference_model/src/ops/ewise_binary.cpp:144-173,
// reference_model/src/ops/activation_funcs.cpp:27-128): the table holds their result for every pair of input bytes.
// Included by api.cu after kernels_cc.cuh (table layout, bank swizzle and REQUIRE bits are those of
// residual_add_i8_table_kernel).
#pragma once

#include "ptx_sm100.cuh"

namespace tb200
{

constexpr int kJoinStreamStages     = 6;
constexpr int kJoinStreamChunkVecs  = 512;                              // 16-byte vectors of each operand per stage
constexpr int kJoinStreamChunkBytes = kJoinStreamChunkVecs * 16;        // 8 KB
constexpr int kJoinStreamConsumers  = kJoinStreamChunkVecs;             // one vector per consumer thread and stage
constexpr int kJoinStreamThreads    = kJoinStreamConsumers + 32;        // + the producer warp
constexpr size_t kJoinStreamSmem    = (size_t)kJoinTableBytes + kJoinBadWords * sizeof(uint32_t) +
                                   (size_t)kJoinStreamStages * 2 * kJoinStreamChunkBytes + 1024;

__device__ __forceinline__ void join_bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

// a, b, out: n16 vectors of 16 int8 each, 16-byte aligned.  One CTA per SM; chunk j of the tensor (512 vectors) belongs
// to CTA j % gridDim.x.  wait_limit bounds every wait on the ring (SM cycles); a wait that gives up sets
// TB200_DEV_TIMEOUT and the CTA leaves after the copies in flight have landed.
__global__ void __launch_bounds__(kJoinStreamThreads, 1)
    residual_add_i8_stream_kernel(const int8_t* __restrict__ a, const int8_t* __restrict__ b, int8_t* __restrict__ out, int64_t n16,
                                  const uint8_t* __restrict__ table, const uint32_t* __restrict__ bad_bits, int* status,
                                  long long wait_limit)
{
    extern __shared__ __align__(16) uint8_t join_stream_smem[];
    __shared__ __align__(8) uint64_t bar_full[kJoinStreamStages];
    __shared__ __align__(8) uint64_t bar_empty[kJoinStreamStages];
    __shared__ int abort_flag;
    const uint32_t smem0 = (ptx::smem_u32(join_stream_smem) + 127u) & ~127u;
    uint8_t* const base  = join_stream_smem + (smem0 - ptx::smem_u32(join_stream_smem));
    uint8_t* tab         = base;
    uint32_t* bits       = reinterpret_cast<uint32_t*>(base + kJoinTableBytes);
    const uint32_t ring  = smem0 + (uint32_t)kJoinTableBytes + (uint32_t)(kJoinBadWords * sizeof(uint32_t));
    uint8_t* const ring_g = base + kJoinTableBytes + kJoinBadWords * sizeof(uint32_t);

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < kJoinStreamStages; s++)
        {
            ptx::mbar_init(ptx::smem_u32(&bar_full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&bar_empty[s]), kJoinStreamConsumers / 32);    // one arrival per consumer warp
        }
        abort_flag = 0;
        ptx::fence_barrier_init();
        // the successor kernel may be scheduled from here on
        ptx::dep_launch_trigger();
    }
    // table and REQUIRE bits are constants of the join: copied while the predecessor may still be running
    for (int i = threadIdx.x; i < kJoinTableBytes / 16; i += blockDim.x)
        reinterpret_cast<int4*>(tab)[i] = __ldg(reinterpret_cast<const int4*>(table) + i);
    uint32_t any = 0;
    for (int i = threadIdx.x; i < kJoinBadWords; i += blockDim.x)
    {
        const uint32_t w = __ldg(bad_bits + i);
        bits[i] = w;
        any |= w;
    }
    const bool check = __syncthreads_or(any != 0) != 0;    // (also publishes the table and the barriers)
    ptx::dep_launch_wait();                                // the operands are the predecessor's output

    const int64_t nchunks  = (n16 + kJoinStreamChunkVecs - 1) / kJoinStreamChunkVecs;
    const int64_t my_first = blockIdx.x;
    const int warp         = threadIdx.x >> 5;

    if (warp == kJoinStreamConsumers / 32)
    {
        // ---------------------------------------------------------------- producer (one thread)
        if ((threadIdx.x & 31) == 0)
        {
            int stage      = 0;
            uint32_t phase = 0;
            bool ok        = true;
            for (int64_t j = my_first; j < nchunks && ok; j += gridDim.x)
            {
                if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bar_empty[stage]), phase ^ 1u, wait_limit))
                {
                    ok = false;
                    break;
                }
                const int64_t v0   = j * kJoinStreamChunkVecs;
                const uint32_t nb  = (uint32_t)(min((int64_t)kJoinStreamChunkVecs, n16 - v0) * 16);
                const uint32_t bar = ptx::smem_u32(&bar_full[stage]);
                const uint32_t dst = ring + (uint32_t)(stage * 2 * kJoinStreamChunkBytes);
                ptx::mbar_arrive_expect_tx(bar, 2 * nb);
                join_bulk_load(dst, a + v0 * 16, nb, bar);
                join_bulk_load(dst + kJoinStreamChunkBytes, b + v0 * 16, nb, bar);
                if (++stage == kJoinStreamStages)
                {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            if (!ok)
            {
                atomicOr(status, TB200_DEV_TIMEOUT);
                atomicExch(&abort_flag, 1);
            }
        }
    }
    else
    {
        // ---------------------------------------------------------------- consumers: one vector per thread and chunk
        bool bad       = false;
        bool ok        = true;
        int stage      = 0;
        uint32_t phase = 0;
        for (int64_t j = my_first; j < nchunks; j += gridDim.x)
        {
            ok = ptx::mbar_wait_bounded(ptx::smem_u32(&bar_full[stage]), phase, wait_limit);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            const int64_t v = j * kJoinStreamChunkVecs + threadIdx.x;
            const uint8_t* sp = ring_g + (size_t)stage * 2 * kJoinStreamChunkBytes + (size_t)threadIdx.x * 16;
            const int4 va = *reinterpret_cast<const int4*>(sp);
            const int4 vb = *reinterpret_cast<const int4*>(sp + kJoinStreamChunkBytes);
            // the operands are in registers: the slot can be refilled while the lookups run
            __syncwarp();
            if ((threadIdx.x & 31) == 0)
                ptx::mbar_arrive(ptx::smem_u32(&bar_empty[stage]));
            if (v < n16)
            {
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
                reinterpret_cast<uint4*>(out)[v] = make_uint4(wo[0], wo[1], wo[2], wo[3]);
            }
            if (++stage == kJoinStreamStages)
            {
                stage = 0;
                phase ^= 1u;
            }
        }
        if (bad)
            atomicOr(status, TB200_DEV_UNPREDICTABLE);
        if (!ok && (threadIdx.x & 31) == 0)
        {
            atomicOr(status, TB200_DEV_TIMEOUT);
            atomicExch(&abort_flag, 1);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag)
    {
        // a role gave up: let copies that may still be in flight land before the shared memory is released
        for (int s = 0; s < kJoinStreamStages; s++)
        {
            ptx::mbar_wait_bounded(ptx::smem_u32(&bar_full[s]), 0u, 2000000LL);
            ptx::mbar_wait_bounded(ptx::smem_u32(&bar_full[s]), 1u, 2000000LL);
        }
    }
}

}    // namespace tb200
