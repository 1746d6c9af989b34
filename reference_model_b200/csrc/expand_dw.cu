// CONV2D 1x1 (+ CLAMP) followed by DEPTHWISE_CONV2D 3x3 (+ CLAMP) in fp16 / bf16 as ONE kernel: the first half of an
// inverted-residual block, whose expanded tensor (six times the input for 32 -> 192 channels) is the largest tensor of
// the block and has exactly one consumer.  Here it lives in shared memory only: a work item is one image, one group of
// 64 expanded channels and a band of output rows; for every input row the band needs, the tensor cores multiply the row's
// pixels ([<=128 pixels] x [IC]) by the group's weights ([IC] x [64]) into tensor memory, eight worker warps add the
// bias, clamp, round to the storage type (the rounding the reference's CONV2D output has) and put the row into a ring
// of three rows in shared memory; after the rows an output row needs are there, the same warps run the 3x3 window over
// the ring with fp32 accumulation in the reference's tap order, add the depthwise bias, clamp, round and store.
// Equivalent to OpConv2d::eval followed by OpClamp, OpDepthwiseConv2d::eval and OpClamp
// (reference_model/src/ops/tensor_ops.cpp:723-882 and :1172-1334, reference_model/src/ops/activation_funcs.cpp:27-128).
//
// Roles: warps 0..7 workers (warp w reads the tensor-memory lane quarter w % 4, i.e. pixels 32 (w % 4) .. + 31, and the
// 32-channel half w / 4 of the group; in the window pass warp w takes the output pixels w, w + 8, ... and lane l the
// channel pair 2 l, 2 l + 1), warp 8 lane 0 TMA producer, warp 9 lane 0 MMA issuer (warp 9 owns tensor memory).
// Every wait is bounded (p.wait_limit SM cycles); a wait that gives up sets TB200_DEV_TIMEOUT, the roles leave their
// loops together, copies and MMAs in flight are waited for and tensor memory is freed.
//
// What measurement said about this kernel (64 x 112 x 112 x 32 -> 192 channels, stride 2):
//   * the worker warps' instruction issue is the bound, not memory (the tensors that reach device memory are 128 MB, 20 us
//     at the copy rate; the tensor pipe is 2 % busy): every instruction per expanded or output value counts.  CLAMP runs on
//     the rounded, packed pairs (two instructions per pair); bias and accumulator are added two channels per instruction;
//     the window pass multiplies the 16-bit values directly (fma.rn.f32.f16 / .bf16: exact product, one fp32 rounding, the
//     result fmaf gives on the converted values) instead of converting them first;
//   * a ring row is stored as eight channel planes, so that the three taps of a window row are immediate offsets of one
//     address and neither side needs swizzle arithmetic (see the worker code);
//   * one tcgen05.commit per input row kept the tensor pipe idle most of the time (the MMAs of a row take about 200 cycles,
//     a commit several hundred): two rows share a commit, which both publishes their accumulators and frees their stages;
//   * more input-row stages, three CTAs per SM instead of two, or two output pixels per thread at once changed nothing.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <mutex>

#include "common.h"
#include "ptx_sm100.cuh"

namespace tb200
{
namespace
{

constexpr int kXdWorkerWarps = 8;
constexpr int kXdWorkers     = 32 * kXdWorkerWarps;
constexpr int kXdThreads     = kXdWorkers + 64;
constexpr int kXdGroup       = 64;    // expanded channels per work item = columns of one accumulator buffer
constexpr int kXdBatchRows   = 2;     // input rows whose MMAs share one tcgen05.commit (a commit idles the tensor pipe for hundreds of cycles)
constexpr int kXdAccBufs     = 2;     // accumulator buffers, each of kXdBatchRows rows x kXdGroup columns
constexpr int kXdStages      = kXdAccBufs * kXdBatchRows;    // input-row stages: one per accumulator row
constexpr int kXdTmemCols    = kXdAccBufs * kXdBatchRows * kXdGroup;
constexpr int kXdRing        = 3;     // expanded rows kept: a 3-row window moving down by one or two rows
constexpr int kXdMinCtas     = 2;     // CTAs the compiler leaves register room for on one SM (two CTAs of 256 tensor-memory columns fill its 512)

struct XdParams
{
    CUtensorMap tmA;    // input as [N*IH*IW][IC], box = (IC, a_box_rows)
    CUtensorMap tmB;    // CONV2D weights as [C][IC], box = (IC, 64)
    const void* b1;     // CONV2D bias [C] or [1]
    const void* wd;     // depthwise weights [3][3][C][1]
    const void* bd;     // depthwise bias [C] or [1]
    void* out;          // [N][OH][OW][C]
    int b1_n, bd_n;
    int N, IH, IW, IC, C, OH, OW;
    int pad_t, pad_l, sy, sx;
    int clamp1, clamp2;
    float lo1, hi1, lo2, hi2;
    int groups, bands, band_rows, items;
    int a_stage_bytes, a_tx_bytes, b_group_bytes;
    int b_off, a_off, ring_off, bias_off;    // from the 1024-byte aligned start of dynamic shared memory
    int ring_row_bytes, plane_bytes;    // a ring row is eight planes (8 channels each) of plane_bytes
    int mmas;    // MMAs (16 channels of K each) per input row
    uint32_t idesc;
    uint64_t desc_hi;
    long long wait_limit;
    int* status;
};

template <typename T>
struct XdType;
template <>
struct XdType<__half>
{
    static __device__ __forceinline__ float2 up2(uint32_t w)
    {
        return __half22float2(*reinterpret_cast<const __half2*>(&w));
    }
    static __device__ __forceinline__ uint32_t down2(float2 v)
    {
        const __half2 h = __floats2half2_rn(v.x, v.y);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
    // CLAMP of two rounded values; a NaN stays a NaN
    static __device__ __forceinline__ uint32_t clamp2(uint32_t w, uint32_t lo, uint32_t hi)
    {
        const __half2 h = __hmin2_nan(__hmax2_nan(*reinterpret_cast<const __half2*>(&w), *reinterpret_cast<const __half2*>(&lo)),
                                      *reinterpret_cast<const __half2*>(&hi));
        return *reinterpret_cast<const uint32_t*>(&h);
    }
    static __device__ __forceinline__ float up(const void* p, int i)
    {
        return __half2float(reinterpret_cast<const __half*>(p)[i]);
    }
    // acc.x = fma(low(a), low(b), acc.x), acc.y = fma(high(a), high(b), acc.y): the 16-bit operands widened exactly, the
    // product exact, one rounding to fp32 (what fmaf on the converted values gives), without a conversion instruction
    static __device__ __forceinline__ void fma2(float2& acc, uint32_t a, uint32_t b)
    {
        asm("{\n"
            ".reg .b16 al, ah, bl, bh;\n"
            "mov.b32 {al, ah}, %2;\n"
            "mov.b32 {bl, bh}, %3;\n"
            "fma.rn.f32.f16 %0, al, bl, %0;\n"
            "fma.rn.f32.f16 %1, ah, bh, %1;\n"
            "}\n"
            : "+f"(acc.x), "+f"(acc.y)
            : "r"(a), "r"(b));
    }
};
template <>
struct XdType<__nv_bfloat16>
{
    static __device__ __forceinline__ float2 up2(uint32_t w)
    {
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    }
    static __device__ __forceinline__ uint32_t down2(float2 v)
    {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v.x, v.y);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
    static __device__ __forceinline__ uint32_t clamp2(uint32_t w, uint32_t lo, uint32_t hi)
    {
        const __nv_bfloat162 h =
            __hmin2_nan(__hmax2_nan(*reinterpret_cast<const __nv_bfloat162*>(&w), *reinterpret_cast<const __nv_bfloat162*>(&lo)),
                        *reinterpret_cast<const __nv_bfloat162*>(&hi));
        return *reinterpret_cast<const uint32_t*>(&h);
    }
    static __device__ __forceinline__ float up(const void* p, int i)
    {
        return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    }
    static __device__ __forceinline__ void fma2(float2& acc, uint32_t a, uint32_t b)
    {
        asm("{\n"
            ".reg .b16 al, ah, bl, bh;\n"
            "mov.b32 {al, ah}, %2;\n"
            "mov.b32 {bl, bh}, %3;\n"
            "fma.rn.f32.bf16 %0, al, bl, %0;\n"
            "fma.rn.f32.bf16 %1, ah, bh, %1;\n"
            "}\n"
            : "+f"(acc.x), "+f"(acc.y)
            : "r"(a), "r"(b));
    }
};

// CLAMP runs on the rounded, packed values: rounding is monotonic, so clamping the rounded value to the rounded bounds
// gives what rounding the clamped fp32 value gives, at one instruction per bound for two values.

template <int OFF>
__device__ __forceinline__ uint32_t xd_lds32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
    return v;
}

struct XdItem
{
    int n, g, oy0, oy1, r_lo, r_hi;    // image, channel group, output rows [oy0, oy1), input rows [r_lo, r_hi]
};

// Items are numbered (image, band, group) with the group fastest: the CTAs that work on the three groups of a band at
// the same time read the same input rows.
__device__ __forceinline__ XdItem xd_decode(const XdParams& p, int item)
{
    XdItem t;
    t.g         = item % p.groups;
    const int r = item / p.groups;
    const int b = r % p.bands;
    t.n         = r / p.bands;
    t.oy0       = b * p.band_rows;
    t.oy1       = min(p.OH, t.oy0 + p.band_rows);
    t.r_lo      = max(0, t.oy0 * p.sy - p.pad_t);
    t.r_hi      = min(p.IH - 1, (t.oy1 - 1) * p.sy - p.pad_t + 2);
    return t;
}

template <typename T>
__global__ void __launch_bounds__(kXdThreads, kXdMinCtas) expand_dw_kernel(const __grid_constant__ XdParams p)
{
    extern __shared__ uint8_t xd_smem_raw[];
    __shared__ __align__(8) uint64_t bar_a_full[kXdStages];        // TMA -> MMA: the input row has landed
    __shared__ __align__(8) uint64_t bar_acc_full[kXdAccBufs];     // MMA -> workers: a batch of expanded rows is in tensor memory
                                                                   // (and -> TMA: the batch's input-row stages are free)
    __shared__ __align__(8) uint64_t bar_acc_empty[kXdAccBufs];    // workers -> MMA: accumulator buffer drained
    __shared__ __align__(8) uint64_t bar_b;                        // the CONV2D weights have landed
    __shared__ __align__(8) uint64_t bar_drain;                    // teardown after a wait gave up
    __shared__ uint32_t tmem_base_holder;
    __shared__ int abort_flag;

    const int warp           = threadIdx.x >> 5;
    const int lane           = threadIdx.x & 31;
    const uint32_t smem_base = (ptx::smem_u32(xd_smem_raw) + 1023u) & ~1023u;
    uint8_t* const smem_al   = xd_smem_raw + (smem_base - ptx::smem_u32(xd_smem_raw));
    const uint32_t s_b       = smem_base + (uint32_t)p.b_off;
    const uint32_t s_a       = smem_base + (uint32_t)p.a_off;
    float* const s_bias      = reinterpret_cast<float*>(smem_al + p.bias_off);

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < kXdStages; s++)
            ptx::mbar_init(ptx::smem_u32(&bar_a_full[s]), 1);
        for (int a = 0; a < kXdAccBufs; a++)
        {
            ptx::mbar_init(ptx::smem_u32(&bar_acc_full[a]), 1);
            ptx::mbar_init(ptx::smem_u32(&bar_acc_empty[a]), kXdWorkerWarps);    // one arrival per worker warp
        }
        ptx::mbar_init(ptx::smem_u32(&bar_b), 1);
        ptx::mbar_init(ptx::smem_u32(&bar_drain), 1);
        abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tmap(&p.tmA);
        ptx::prefetch_tmap(&p.tmB);
    }
    if (warp == kXdWorkerWarps + 1)
    {
        ptx::tmem_alloc(ptx::smem_u32(&tmem_base_holder), (uint32_t)kXdTmemCols);
        ptx::tmem_relinquish();
    }
    // the CONV2D bias of every channel as fp32 (added to the fp32 accumulator, as the reference adds it before rounding)
    for (int c = threadIdx.x; c < p.C; c += blockDim.x)
        s_bias[c] = XdType<T>::up(p.b1, p.b1_n == 1 ? 0 : c);
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_holder;
    const int my_items       = (p.items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

    if (warp == kXdWorkerWarps)
    {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0)
        {
            // the weights of all channel groups, once
            ptx::mbar_arrive_expect_tx(ptx::smem_u32(&bar_b), (uint32_t)(p.groups * p.b_group_bytes));
            for (int g = 0; g < p.groups; g++)
                ptx::tma_load_2d(s_b + (uint32_t)(g * p.b_group_bytes), &p.tmB, ptx::smem_u32(&bar_b), 0, g * kXdGroup);
            bool ok     = true;
            uint32_t bi = 0;    // batches issued so far: batch bi uses accumulator buffer bi & 1 and that buffer's row stages
            for (int i = 0; i < my_items && ok; i++)
            {
                const XdItem t = xd_decode(p, (int)blockIdx.x + i * (int)gridDim.x);
                for (int r = t.r_lo; r <= t.r_hi; r += kXdBatchRows, bi++)
                {
                    // the stages are free once the MMAs of the batch that used them last (bi - 2) have completed: the commit
                    // that published that batch's accumulators says so
                    const uint32_t buf = bi & 1u;
                    if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bar_acc_full[buf]), ((bi >> 1) & 1u) ^ 1u, p.wait_limit))
                    {
                        ok = false;
                        break;
                    }
                    const int nb = min(kXdBatchRows, t.r_hi - r + 1);
                    for (int rr = 0; rr < nb; rr++)
                    {
                        const uint32_t stage = buf * kXdBatchRows + rr;
                        const uint32_t full  = ptx::smem_u32(&bar_a_full[stage]);
                        ptx::mbar_arrive_expect_tx(full, (uint32_t)p.a_tx_bytes);
                        ptx::tma_load_2d(s_a + stage * (uint32_t)p.a_stage_bytes, &p.tmA, full, 0, (t.n * p.IH + r + rr) * p.IW);
                    }
                    // a short last batch of an item: complete the unused stages' phase too, so that every stage barrier
                    // advances once per batch of its buffer and one parity serves them all
                    for (int rr = nb; rr < kXdBatchRows; rr++)
                        ptx::mbar_arrive(ptx::smem_u32(&bar_a_full[buf * kXdBatchRows + rr]));
                }
            }
            if (!ok)
            {
                atomicOr(p.status, TB200_DEV_TIMEOUT);
                atomicExch(&abort_flag, 1);
            }
        }
    }
    else if (warp == kXdWorkerWarps + 1)
    {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0)
        {
            bool ok = ptx::mbar_wait_bounded(ptx::smem_u32(&bar_b), 0u, p.wait_limit);
            ptx::tc_fence_after_sync();
            uint32_t bi = 0;    // batches issued so far
            for (int i = 0; i < my_items && ok; i++)
            {
                const XdItem t    = xd_decode(p, (int)blockIdx.x + i * (int)gridDim.x);
                const uint64_t bd = ptx::smem_desc(p.desc_hi, s_b + (uint32_t)(t.g * p.b_group_bytes));
                for (int r = t.r_lo; r <= t.r_hi && ok; r += kXdBatchRows, bi++)
                {
                    const uint32_t buf    = bi & 1u;
                    const uint32_t parity = (bi >> 1) & 1u;
                    if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bar_acc_empty[buf]), parity ^ 1u, p.wait_limit))
                    {
                        ok = false;
                        break;
                    }
                    const int nb = min(kXdBatchRows, t.r_hi - r + 1);
                    for (int rr = 0; rr < kXdBatchRows; rr++)
                    {
                        const uint32_t stage = buf * kXdBatchRows + rr;
                        if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bar_a_full[stage]), parity, p.wait_limit))
                        {
                            ok = false;
                            break;
                        }
                        if (rr >= nb)
                            continue;    // unused stage of a short batch: only its phase is consumed
                        ptx::tc_fence_after_sync();
                        const uint64_t ad     = ptx::smem_desc(p.desc_hi, s_a + stage * (uint32_t)p.a_stage_bytes);
                        const uint32_t d_tmem = tmem_base + stage * (uint32_t)kXdGroup;
                        for (int m = 0; m < p.mmas; m++)    // 16 channels (32 bytes) of K per MMA
                            ptx::mma_f16_ss(d_tmem, ad + (uint64_t)(2 * m), bd + (uint64_t)(2 * m), p.idesc, m > 0 ? 1u : 0u);
                    }
                    // one commit per batch: it publishes the rows and frees their stages (MMAs issued before a wait that
                    // gave up are covered by the teardown's commit)
                    if (ok)
                        ptx::mma_commit(ptx::smem_u32(&bar_acc_full[buf]));
                }
            }
            if (!ok)
            {
                atomicOr(p.status, TB200_DEV_TIMEOUT);
                atomicExch(&abort_flag, 1);
            }
        }
    }
    else
    {
        // ------------------------------------------------------------------ workers
        const int quarter         = warp & 3;     // tensor-memory lane quarter this warp may read
        const int half            = warp >> 2;    // which 32 of the group's 64 channels it expands
        const int px              = quarter * 32 + lane;    // its pixel of an input row
        uint8_t* const ring       = smem_al + p.ring_off;
        const uint32_t ring_s     = smem_base + (uint32_t)p.ring_off;
        // A ring row is eight planes of 8 channels: plane j holds, pixel after pixel, the 16 bytes of channels 8 j .. 8 j + 7.
        // Expanding, a warp's lanes are neighbouring pixels and write neighbouring 16-byte slots of a plane.  In the window
        // pass lane l reads the channel pair 2 l, 2 l + 1 = word l & 3 of plane l >> 2; the plane stride is 16 bytes more
        // than a multiple of 128, so the 32 lanes hit 32 different banks, and the three taps of a window row are 16 bytes
        // apart: immediate offsets of one address.
        const uint32_t lane_off = ((uint32_t)lane >> 2) * (uint32_t)p.plane_bytes + (((uint32_t)lane & 3u) << 2);
        const int base_ix       = warp * p.sx - p.pad_l;               // first tap column of the warp's first output pixel
        const int jstep         = kXdWorkerWarps * p.sx * 16;          // bytes between a warp's consecutive output pixels
        const int nj            = warp < p.OW ? (p.OW - warp + kXdWorkerWarps - 1) / kXdWorkerWarps : 0;    // its output pixels per row
        // its pixels whose three tap columns all lie inside the image: [jf0, jf1)
        const int xstep = kXdWorkerWarps * p.sx;
        int jf0         = base_ix >= 0 ? 0 : (-base_ix + xstep - 1) / xstep;
        int jf1         = p.IW - 3 - base_ix >= 0 ? (p.IW - 3 - base_ix) / xstep + 1 : 0;
        jf0             = min(jf0, nj);
        jf1             = max(jf0, min(jf1, nj));
        const uint32_t lo1 = XdType<T>::down2(make_float2(p.lo1, p.lo1)), hi1 = XdType<T>::down2(make_float2(p.hi1, p.hi1));
        const uint32_t lo2 = XdType<T>::down2(make_float2(p.lo2, p.lo2)), hi2 = XdType<T>::down2(make_float2(p.hi2, p.hi2));
        bool ok      = true;
        uint32_t bi  = 0;    // batches drained so far
        int loaded_g = -1;
        uint32_t wgt[9];    // the lane's two channels of every tap, as stored
        float2 dbias;
        for (int i = 0; i < my_items && ok; i++)
        {
            const XdItem t = xd_decode(p, (int)blockIdx.x + i * (int)gridDim.x);
            if (t.g != loaded_g)
            {
                const int c = t.g * kXdGroup + 2 * lane;
#pragma unroll
                for (int tap = 0; tap < 9; tap++)
                    wgt[tap] = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const T*>(p.wd) + tap * p.C + c);
                dbias    = make_float2(XdType<T>::up(p.bd, p.bd_n == 1 ? 0 : c), XdType<T>::up(p.bd, p.bd_n == 1 ? 0 : c + 1));
                loaded_g = t.g;
            }
            const float* const bb = s_bias + t.g * kXdGroup + half * 32;
            int next_row          = t.r_lo;
            int in_batch          = 0;    // rows of the current batch already drained
            for (int oy = t.oy0; oy < t.oy1; oy++)
            {
                const int iy0  = oy * p.sy - p.pad_t;
                const int last = min(p.IH - 1, iy0 + 2);
                // ---- expand the input rows this output row needs and the ring does not hold yet
                for (; next_row <= last; next_row++)
                {
                    const uint32_t buf  = bi & 1u;
                    const int batch_len = min(kXdBatchRows, t.r_hi - (next_row - in_batch) + 1);    // rows of the current batch
                    const int row_slot  = (int)buf * kXdBatchRows + in_batch;                        // its accumulator row
                    const bool first    = in_batch == 0;
                    const bool lastrow  = ++in_batch == batch_len;
                    const uint32_t par  = (bi >> 1) & 1u;
                    if (lastrow)
                    {
                        in_batch = 0;
                        bi++;
                    }
                    if (!ok)
                        continue;    // after a wait gave up: only keep the counters in step with the other warps
                    if (first)
                    {
                        ok = ptx::mbar_wait_bounded(ptx::smem_u32(&bar_acc_full[buf]), par, p.wait_limit);
                        ok = __all_sync(0xffffffffu, ok);    // the whole warp agrees before the warp-collective loads
                        if (!ok)
                            continue;
                    }
                    ptx::tc_fence_after_sync();
                    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(row_slot * kXdGroup + half * 32);
                    uint8_t* const dst   = ring + (next_row % kXdRing) * p.ring_row_bytes + px * 16 + (half * 4) * p.plane_bytes;
#pragma unroll
                    for (int hh = 0; hh < 2; hh++)
                    {
                        uint32_t v[16];
                        ptx::tmem_ld_32x32b_x16(taddr + (uint32_t)(hh * 16), v);
                        ptx::tmem_ld_wait();
                        uint32_t w[8];
#pragma unroll
                        for (int q = 0; q < 4; q++)
                        {
                            const float4 b4 = *reinterpret_cast<const float4*>(bb + hh * 16 + 4 * q);
                            // accumulator + bias in fp32, two channels per instruction, then one rounding
                            w[2 * q] = XdType<T>::down2(__fadd2_rn(make_float2(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1])),
                                                                   make_float2(b4.x, b4.y)));
                            w[2 * q + 1] = XdType<T>::down2(__fadd2_rn(make_float2(__uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3])),
                                                                       make_float2(b4.z, b4.w)));
                            if (p.clamp1)
                            {
                                w[2 * q]     = XdType<T>::clamp2(w[2 * q], lo1, hi1);
                                w[2 * q + 1] = XdType<T>::clamp2(w[2 * q + 1], lo1, hi1);
                            }
                        }
                        if (px < p.IW)
                        {
                            *reinterpret_cast<uint4*>(dst + (hh * 2) * p.plane_bytes)     = make_uint4(w[0], w[1], w[2], w[3]);
                            *reinterpret_cast<uint4*>(dst + (hh * 2 + 1) * p.plane_bytes) = make_uint4(w[4], w[5], w[6], w[7]);
                        }
                    }
                    if (lastrow)
                    {
                        // this warp has read its part of every row of the batch
                        ptx::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0)
                            ptx::mbar_arrive(ptx::smem_u32(&bar_acc_empty[buf]));
                    }
                }
                // the rows are in the ring for every warp (and every warp learns of a wait that gave up)
                ok = ptx::named_barrier_and(1, kXdWorkers, ok);
                if (!ok)
                    break;
                // ---- the 3x3 window over the ring: warp = output pixel (stride 8), lane = channel pair
                bool yv[3];
                uint32_t rrow[3];    // shared-memory address of the lane's word of the warp's first tap column, per window row
#pragma unroll
                for (int ky = 0; ky < 3; ky++)
                {
                    const int iy = iy0 + ky;
                    yv[ky]       = iy >= 0 && iy < p.IH;
                    rrow[ky]     = ring_s + (uint32_t)((yv[ky] ? iy % kXdRing : 0) * p.ring_row_bytes) + lane_off + (uint32_t)(base_ix * 16);
                }
                const bool rows_in = yv[0] && yv[1] && yv[2];
                uint32_t* const orow =
                    reinterpret_cast<uint32_t*>(reinterpret_cast<T*>(p.out) + ((int64_t)(t.n * p.OH + oy) * p.OW + warp) * p.C + t.g * kXdGroup) + lane;
                const int ostep = kXdWorkerWarps * (p.C / 2);    // 32-bit words between a warp's consecutive output pixels
                auto finish = [&](int j, float2 acc) {
                    uint32_t o = XdType<T>::down2(__fadd2_rn(dbias, acc));
                    if (p.clamp2)
                        o = XdType<T>::clamp2(o, lo2, hi2);
                    orow[(int64_t)j * ostep] = o;
                };
                // taps outside the image are skipped, as the reference skips them
                auto edge = [&](int j) {
                    const int ix0      = base_ix + j * xstep;
                    const uint32_t off = (uint32_t)(j * jstep);
                    float2 acc         = make_float2(0.f, 0.f);
#pragma unroll
                    for (int ky = 0; ky < 3; ky++)
                    {
                        if (!yv[ky])
                            continue;
                        if (ix0 >= 0 && ix0 < p.IW)
                            XdType<T>::fma2(acc, xd_lds32<0>(rrow[ky] + off), wgt[ky * 3 + 0]);
                        if (ix0 + 1 >= 0 && ix0 + 1 < p.IW)
                            XdType<T>::fma2(acc, xd_lds32<16>(rrow[ky] + off), wgt[ky * 3 + 1]);
                        if (ix0 + 2 >= 0 && ix0 + 2 < p.IW)
                            XdType<T>::fma2(acc, xd_lds32<32>(rrow[ky] + off), wgt[ky * 3 + 2]);
                    }
                    finish(j, acc);
                };
                const int f0 = rows_in ? jf0 : nj, f1 = rows_in ? jf1 : nj;
                for (int j = 0; j < f0; j++)
                    edge(j);
#pragma unroll 1
                for (int j = f0; j < f1; j++)
                {
                    const uint32_t off = (uint32_t)(j * jstep);
                    uint32_t win[9];
#pragma unroll
                    for (int ky = 0; ky < 3; ky++)
                    {
                        win[ky * 3 + 0] = xd_lds32<0>(rrow[ky] + off);
                        win[ky * 3 + 1] = xd_lds32<16>(rrow[ky] + off);
                        win[ky * 3 + 2] = xd_lds32<32>(rrow[ky] + off);
                    }
                    float2 acc = make_float2(0.f, 0.f);
#pragma unroll
                    for (int tap = 0; tap < 9; tap++)
                        XdType<T>::fma2(acc, win[tap], wgt[tap]);
                    finish(j, acc);
                }
                for (int j = f1; j < nj; j++)
                    edge(j);
                // the next row's expansion overwrites ring rows this pass has read
                asm volatile("bar.sync 1, %0;" ::"n"(kXdWorkers) : "memory");
            }
        }
        if (!ok && lane == 0)
        {
            atomicOr(p.status, TB200_DEV_TIMEOUT);
            atomicExch(&abort_flag, 1);
        }
    }

    // ---------------------------------------------------------------------- teardown
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag)
    {
        // a role gave up: let copies that may still be in flight land before the CTA's shared memory is released
        for (int s = 0; s < kXdStages; s++)
        {
            ptx::mbar_wait_bounded(ptx::smem_u32(&bar_a_full[s]), 0u, 2000000LL);
            ptx::mbar_wait_bounded(ptx::smem_u32(&bar_a_full[s]), 1u, 2000000LL);
        }
        ptx::mbar_wait_bounded(ptx::smem_u32(&bar_b), 0u, 2000000LL);
    }
    if (warp == kXdWorkerWarps + 1 && lane == 0 && abort_flag)
    {
        // ... and let the tensor-core work already issued retire before its accumulators' tensor memory is freed
        ptx::mma_commit(ptx::smem_u32(&bar_drain));
        ptx::mbar_wait_bounded(ptx::smem_u32(&bar_drain), 0u, 40000000LL);
    }
    __syncthreads();
    if (warp == kXdWorkerWarps + 1)
    {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, (uint32_t)kXdTmemCols);
    }
}

typedef CUresult (*PFN_xdEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                      const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

PFN_xdEncodeTiled xd_encode_fn()
{
    static PFN_xdEncodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_xdEncodeTiled>(sym);
    });
    return fn;
}

struct XdLayout
{
    int stages, smem_bytes, b_off, a_off, ring_off, bias_off, a_stage_bytes, b_group_bytes, ring_row_bytes, plane_bytes;
};

// Shared memory of one CTA with `stages` input-row stages: weights of all groups, the stages, the ring, the fp32 bias.
XdLayout xd_layout(const ExpandDwProblem& q, int stages)
{
    XdLayout l;
    const int row_bytes = q.IC * 2;
    l.stages            = stages;
    l.b_group_bytes     = std::max(1024, kXdGroup * row_bytes);
    l.a_stage_bytes     = 128 * row_bytes;    // the MMA reads 128 rows whatever the image width
    l.plane_bytes       = ((q.IW * 16 + 127) & ~127) + 16;    // 16 bytes past a multiple of 128: see the window pass
    l.ring_row_bytes    = (kXdGroup / 8) * l.plane_bytes;
    l.b_off             = 0;
    l.a_off             = l.b_off + (q.C / kXdGroup) * l.b_group_bytes;
    l.ring_off          = l.a_off + stages * l.a_stage_bytes;
    l.bias_off          = l.ring_off + kXdRing * l.ring_row_bytes;
    l.smem_bytes        = l.bias_off + q.C * 4 + 1024;    // + room to align the start to 1024 bytes
    return l;
}

}    // namespace

bool expand_dw_supported(const tb200_ctx* ctx, const ExpandDwProblem& q, std::string* why)
{
    auto no = [&](const char* m) {
        if (why)
            *why = m;
        return false;
    };
    if (q.dtype != TB200_FP16 && q.dtype != TB200_BF16)
        return no("fp16 and bf16 only");
    if (q.IC != 16 && q.IC != 32 && q.IC != 64)
        return no("input channels must be 16, 32 or 64 (one swizzled row of K per pixel)");
    if (q.C % kXdGroup != 0 || q.C <= 0)
        return no("expanded channels must be a multiple of 64");
    if (q.IW > 128 || q.IW < 1)
        return no("input rows wider than one 128-pixel MMA tile");
    if (q.sy < 1 || q.sy > 2 || q.sx < 1 || q.sx > 2)
        return no("strides other than 1 and 2");
    if (q.pad_t < 0 || q.pad_l < 0)
        return no("negative padding");
    if ((int64_t)q.N * q.IH * q.IW >= (int64_t)1 << 31 || (int64_t)q.N * q.OH * q.OW * q.C >= (int64_t)1 << 40)
        return no("tensor too large for 32-bit pixel coordinates");
    if ((reinterpret_cast<uintptr_t>(q.in) | reinterpret_cast<uintptr_t>(q.w1)) & 15)
        return no("input and weights must be 16-byte aligned");
    if ((reinterpret_cast<uintptr_t>(q.out) | reinterpret_cast<uintptr_t>(q.wd)) & 3)
        return no("output and depthwise weights must be 4-byte aligned");
    const int limit = ctx && ctx->max_smem_optin > 0 ? ctx->max_smem_optin : 227 * 1024;
    if (xd_layout(q, kXdStages).smem_bytes > limit)
        return no("weights and ring do not fit in shared memory");
    return true;
}

tb200_status expand_dw_launch(tb200_ctx* ctx, const ExpandDwProblem& q)
{
    std::string why;
    if (!expand_dw_supported(ctx, q, &why))
        return fail(ctx, TB200_ERROR, "fused CONV2D + DEPTHWISE_CONV2D not applicable: %s", why.c_str());
    PFN_xdEncodeTiled enc = xd_encode_fn();
    if (!enc)
        return fail(ctx, TB200_INTERNAL, "cuTensorMapEncodeTiled is not available from the driver");
    const bool bf16 = q.dtype == TB200_BF16;
    const void* kernel = bf16 ? reinterpret_cast<const void*>(&expand_dw_kernel<__nv_bfloat16>)
                              : reinterpret_cast<const void*>(&expand_dw_kernel<__half>);
    const XdLayout lay = xd_layout(q, kXdStages);
    const int attr_bit = bf16 ? 13 : 12;
    if (!(ctx->smem_attr_set & (1u << attr_bit)))    // several CTAs of this size per SM need the largest shared-memory carve-out
        TB200_CUDA_CHECK(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    tb200_status st = raise_smem_limit(ctx, attr_bit, kernel, lay.smem_bytes);
    if (st != TB200_OK)
        return st;
    // CTAs one SM holds: registers, shared memory (each block also pays the driver's reserve), threads, tensor memory
    // (512 columns per SM).  Only the grid size and the band height depend on it: a wrong figure costs time, not results.
    cudaFuncAttributes fa;
    TB200_CUDA_CHECK(ctx, cudaFuncGetAttributes(&fa, kernel));
    int sm_regs = 0, sm_smem = 0, blk_reserve = 0;
    TB200_CUDA_CHECK(ctx, cudaDeviceGetAttribute(&sm_regs, cudaDevAttrMaxRegistersPerMultiprocessor, ctx->device));
    TB200_CUDA_CHECK(ctx, cudaDeviceGetAttribute(&sm_smem, cudaDevAttrMaxSharedMemoryPerMultiprocessor, ctx->device));
    TB200_CUDA_CHECK(ctx, cudaDeviceGetAttribute(&blk_reserve, cudaDevAttrReservedSharedMemoryPerBlock, ctx->device));
    const int regs_per_cta = ((fa.numRegs * 32 + 511) / 512 * 512) * (kXdThreads / 32);
    int resident = std::min(sm_regs / std::max(1, regs_per_cta), sm_smem / (lay.smem_bytes + (int)fa.sharedSizeBytes + blk_reserve));
    resident     = std::min(resident, std::min(2048 / kXdThreads, 512 / kXdTmemCols));
    if (resident < 1)
        return fail(ctx, TB200_INTERNAL, "fused CONV2D + DEPTHWISE_CONV2D kernel does not fit on an SM");

    XdParams k;
    memset(&k, 0, sizeof(k));
    const int row_bytes = q.IC * 2;
    const CUtensorMapSwizzle swz =
        row_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
    const CUtensorMapDataType dt = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const int a_box_rows         = std::min(128, (q.IW + 7) & ~7);    // rows past the image row feed accumulator rows nobody reads
    {
        const cuuint64_t dims[2]    = { (cuuint64_t)q.IC, (cuuint64_t)q.N * q.IH * q.IW };
        const cuuint64_t strides[1] = { (cuuint64_t)row_bytes };
        const cuuint32_t box[2]     = { (cuuint32_t)q.IC, (cuuint32_t)a_box_rows };
        const cuuint32_t estr[2]    = { 1, 1 };
        CUresult r = enc(&k.tmA, dt, 2, const_cast<void*>(q.in), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return fail(ctx, TB200_INTERNAL, "tensor map for the input rejected (CUresult %d)", (int)r);
    }
    {
        const cuuint64_t dims[2]    = { (cuuint64_t)q.IC, (cuuint64_t)q.C };
        const cuuint64_t strides[1] = { (cuuint64_t)row_bytes };
        const cuuint32_t box[2]     = { (cuuint32_t)q.IC, (cuuint32_t)kXdGroup };
        const cuuint32_t estr[2]    = { 1, 1 };
        CUresult r = enc(&k.tmB, dt, 2, const_cast<void*>(q.w1), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return fail(ctx, TB200_INTERNAL, "tensor map for the weights rejected (CUresult %d)", (int)r);
    }
    k.b1 = q.b1; k.wd = q.wd; k.bd = q.bd; k.out = q.out;
    k.b1_n = q.b1_n; k.bd_n = q.bd_n;
    k.N = q.N; k.IH = q.IH; k.IW = q.IW; k.IC = q.IC; k.C = q.C; k.OH = q.OH; k.OW = q.OW;
    k.pad_t = q.pad_t; k.pad_l = q.pad_l; k.sy = q.sy; k.sx = q.sx;
    k.clamp1 = q.clamp1; k.lo1 = q.lo1; k.hi1 = q.hi1;
    k.clamp2 = q.clamp2; k.lo2 = q.lo2; k.hi2 = q.hi2;
    k.groups = q.C / kXdGroup;
    k.a_stage_bytes = lay.a_stage_bytes; k.b_group_bytes = lay.b_group_bytes;
    k.a_tx_bytes     = a_box_rows * row_bytes;
    k.b_off = lay.b_off; k.a_off = lay.a_off; k.ring_off = lay.ring_off; k.bias_off = lay.bias_off;
    k.ring_row_bytes = lay.ring_row_bytes;
    k.plane_bytes    = lay.plane_bytes;
    k.mmas           = q.IC / 16;
    k.idesc          = ptx::make_idesc(1u, bf16 ? 1u : 0u, bf16 ? 1u : 0u, 0u, 0u, 128u, (uint32_t)kXdGroup);
    k.desc_hi        = ptx::make_smem_desc_hi(16, 8 * row_bytes, row_bytes == 32 ? 6u : row_bytes == 64 ? 4u : 2u);
    k.wait_limit     = ctx->wait_limit_cycles;
    k.status         = ctx->d_status;

    // Band height: a band of R output rows expands R * sy + 2 input rows (two of them again in the next band).  Few rows per
    // band waste expansions; many leave SMs with unequal shares (the CTAs resident on one SM share its issue slots, so
    // what counts is the number of items the fullest SM gets) or fewer CTAs than the SMs can hold.  Costs in instructions
    // per thread: about three per expanded value, twenty-two per output value.
    const int slots  = ctx->num_sms * resident;
    double best_cost = 0;
    int best_rows    = 0;
    for (int pass = 0; pass < 2 && best_rows == 0; pass++)    // first only band heights that fill every resident slot
        for (int rows = 1; rows <= q.OH; rows++)
        {
            const int bands     = (q.OH + rows - 1) / rows;
            const int64_t items = (int64_t)q.N * bands * k.groups;
            if (pass == 0 && items < slots)
                continue;
            const int64_t per_sm = (items + ctx->num_sms - 1) / ctx->num_sms;
            const double item    = 3.0 * (rows * q.sy + 2) * q.IW + 22.0 * rows * q.OW;
            const double cost    = (double)per_sm * item;
            if (best_rows == 0 || cost <= best_cost)
            {
                best_cost = cost;
                best_rows = rows;
            }
        }
    k.band_rows = best_rows;
    k.bands     = (q.OH + best_rows - 1) / best_rows;
    const int64_t items = (int64_t)q.N * k.bands * k.groups;
    if (items >= (int64_t)1 << 31)
        return fail(ctx, TB200_ERROR, "fused CONV2D + DEPTHWISE_CONV2D: too many work items");
    k.items        = (int)items;
    const int grid = (int)std::min<int64_t>(items, slots);

    timer_begin(ctx);
    if (bf16)
        expand_dw_kernel<__nv_bfloat16><<<grid, kXdThreads, lay.smem_bytes, ctx->stream>>>(k);
    else
        expand_dw_kernel<__half><<<grid, kXdThreads, lay.smem_bytes, ctx->stream>>>(k);
    timer_end(ctx);
    return post_launch(ctx, bf16 ? "expand_dw_bf16" : "expand_dw_f16");
}

}    // namespace tb200
