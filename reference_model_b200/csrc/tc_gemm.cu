// Tensor-core GEMM / implicit-GEMM convolution for sm_100a.
//
// One persistent, warp-specialised kernel serves MATMUL and CONV2D:
//   warp 0     : issues TMA tile loads (activation patches per filter tap, weight tiles) into a multi-stage
//                shared-memory ring; zero fill outside the tensor implements the convolution padding
//   warp 1     : owns tensor memory (TMEM) and issues tcgen05.mma (kind::i8 with s32 accumulators, or kind::f16
//                with f32 accumulators); two accumulator buffers alternate so the epilogue of one output tile
//                overlaps the MMAs of the next (one buffer, and two CTAs per SM, for short-K 256-column layers)
//   warps 2..9 : epilogue; two warps per TMEM lane quarter, each thread owns one output row (pixel), reads its
//                accumulators from TMEM and applies zero-point corrections / bias / RESCALE / CLAMP before the store
// (Large int8 MATMULs with int32 output go to the CTA-pair kernel in tc_gemm_pair.cu instead.)
// Every wait on an mbarrier is bounded; a wait that gives up sets TB200_DEV_TIMEOUT in the context's status word
// and the kernel drains and exits.
#include <algorithm>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <mutex>

#include "common.h"
#include "ptx_sm100.cuh"
#include "rescale_math.cuh"

namespace tb200
{

namespace
{

#ifdef TB200_DIAG
#define TB200_TRACE(p, slot)                                                                              \
    do                                                                                                    \
    {                                                                                                     \
        if ((p).trace)                                                                                    \
        {                                                                                                 \
            unsigned long long gt__;                                                                      \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt__));                                      \
            (p).trace[(size_t)blockIdx.x * 16 + (slot)] = (long long)gt__;                                \
        }                                                                                                 \
    } while (0)
#else
#define TB200_TRACE(p, slot)                                                                              \
    do                                                                                                    \
    {                                                                                                     \
    } while (0)
#endif

constexpr int kMaxStages   = 8;
constexpr int kTileM       = 128;
constexpr int kNumThreads  = 320;    // TMA warp, MMA warp, 8 epilogue warps
constexpr int kEpiThreads  = 256;

struct TcKernelParams
{
    CUtensorMap tmA;
    CUtensorMap tmB;
    // tile grid
    int tiles_x, tiles_y, tiles_n, tiles_col, num_tiles;
    int tile_begin, tile_end;    // range of tiles this launch covers
    int BW, BH, BN;
    int N, OH, OW, OC;
    int IH, IW;
    int block_n;
    // K loop
    int KH, KW, chunks_per_tap, total_chunks, ksub, num_kstages, chunk_elems;
    int pad_t, pad_l, stride_y, stride_x, dil_y, dil_x;
    int b_mn_major, b_nbox, b_box_n, b_box_bytes;
    // shared memory ring
    int a_chunk_bytes, b_chunk_bytes, stage_bytes, num_stages, tx_bytes_per_chunk;
    int commit_group;    // stages released per tcgen05.commit (each commit costs tensor-pipe idle time)
    // MMA
    uint64_t a_desc_hi, b_desc_hi;
    int b_kstep_bytes, mmas_per_chunk;
    uint32_t idesc;
    int is_f16_kind;    // 0: kind::i8, 1: kind::f16, 2: kind::f8f6f4
    int tmem_cols;
    int acc_bufs;    // TMEM accumulator buffers: 2 overlaps a tile's epilogue with the next tile's MMAs, 1 halves TMEM use
    // epilogue
    void* out;
    int out_es;
    int out_is_bf16;
    const int32_t* row_corr;       // [rows] int32 added to every column of a row (MATMUL b_zp term) or null
    const int32_t* corr;           // [classes][corr_stride] per-column additive constants or null
    int corr_stride;               // padded column count (multiple of the tile width)
    int corr_ystride;              // MATMUL: elements to advance per batch; 0 otherwise
    int corr_classes;              // 1: rows select a table row by their rectangle of in-scope filter taps
    int out_OH, out_OW, out_sy, out_sx, out_y0, out_x0;    // output pixel (oy, ox) -> (oy*out_sy + out_y0, ox*out_sx + out_x0)
    int flat_iw, flat_ih;  // != 0: OW is N*flat_ih*flat_iw flattened pixels of a strided output view
    int d2s_oc, d2s_kw;    // != 0: column c is channel c % d2s_oc of the pixel (c / d2s_oc / d2s_kw, c / d2s_oc % d2s_kw) further on
    const float* bias_f_pad;       // TC_EPI_FLOAT: padded fp32 bias or null
    const int32_t* mult_pad;       // TC_EPI_RESCALE: padded per-column multipliers and shifts
    const int8_t* shift_pad;
    // TC_EPI_RESCALE, optional: one prepared record of 8 words per column for the lean RESCALE form (rescale_rec_build),
    // and for layers with border classes the per-class difference to the interior correction row ([classes][corr_stride])
    const int32_t* rec;
    const int32_t* delta;
    int cls_interior;
    // tc_conv_lean_kernel only: shared-memory offsets from the 1024-byte aligned base (resident weights, stage ring,
    // the four epilogue groups' record copies), whether the weights are resident, stages per tile
    int lean_b_off, lean_ring_off, lean_rec_off, lean_b_resident, lean_stages_per_tile;
    int lean_rec_stride;           // bytes between the epilogue groups' copies of the records (0: one copy, single column block)
    uint32_t fd_m[2], fd_x[2], fd_y[2];    // division by tiles_m, tiles_x, tiles_y as multiply-high + shift (fastdiv_make)
    int lean_xpar, lean_ow_real;   // batch index = 2 image + parity of the output column; true output width
    int lean_halo, lean_halo_wp;   // halo mode: one box per channel chunk and tile; wp = OW + KW - 1 accumulator rows per output row
    int double_round;
    int32_t out_zp, clamp_lo, clamp_hi;
    float clamp_lo_f, clamp_hi_f;
    int has_clamp;
    int debug;    // diagnostic bit mask, read only by builds with TB200_DIAG: 1 skip epilogue memory work, 2 skip MMA issue, 4 skip loads; lean kernel: 32 skip stores, 64 skip tensor-memory loads, 128 skip arithmetic, 256 one record for all columns
    long long wait_limit;    // SM cycles after which a pipeline wait gives up (TB200_DEV_TIMEOUT)
#ifdef TB200_DIAG
    long long* trace;        // diagnostic builds: [CTA][16] globaltimer stamps (ns) of the roles' milestones, or null
#endif
    int* status;
};

struct TileCoord
{
    int x0, y0, n0, col0;
};

__device__ __forceinline__ TileCoord decode_tile(const TcKernelParams& p, int tile)
{
    TileCoord t;
    int c  = tile % p.tiles_col;
    int r  = tile / p.tiles_col;
    t.col0 = c * p.block_n;
    t.x0   = (r % p.tiles_x) * p.BW;
    r /= p.tiles_x;
    t.y0 = (r % p.tiles_y) * p.BH;
    t.n0 = (r / p.tiles_y) * p.BN;
    return t;
}

// 16 consecutive int8 results
__device__ __forceinline__ uint32_t pack4_i8(int a, int b, int c, int d)
{
    return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) |
           ((uint32_t)(d & 0xff) << 24);
}

// four int32 values saturated to int8 and packed, first value in the low byte
__device__ __forceinline__ uint32_t pack4_sat_i8(int a, int b, int c, int d)
{
    uint32_t hi, r;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(d), "r"(c), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(b), "r"(a), "r"(hi));
    return r;
}

// Column-block properties found while the RESCALE constants are built
enum : int
{
    EPI_COLS_GENERIC  = 1,    // some column has operands outside what the high-word form below handles
    EPI_COLS_PRESHIFT = 2,    // some shift is below 32: values are pre-scaled, and apply_scale_32's range check applies
    EPI_COLS_NOT_LEAN = 4,    // some column's prepared record is marked unusable: the lean form is off for this block
};

// apply_scale_32 + output zero point + int8 saturation and packing of four accumulators, for column blocks whose
// shifts are all at most 54.  The result is always taken as the high word of a 64-bit sum:
//   shift >= 32: result + out_zp = high word of (v * multiplier + R) >> (shift - 32); every int32 value is accepted;
//   shift <  32: with k = 32 - shift, ((v << k) * multiplier + (round << k)) >> 32 equals (v * multiplier + round)
//                >> shift, and v << k fits int32 for every v inside the range apply_scale_32 accepts (checked by the
//                caller for such blocks);
// and adding out_zp * 2^(shift + k) to the rounding constant before the arithmetic shift adds exactly out_zp after it
// (|sum| < 2^62 + 2^61 + 2^54).
//   cols[i] = {multiplier, max(shift, 32) - 32, R(v >= 0) lo, hi, R(v < 0) lo, hi, largest |v| accepted, k}
// (the two constants differ only under double rounding).  Measured on this part, one 64-bit multiply-add with a
// selected addend is cheaper than a high and a low multiply with the carry worked out by hand.
template <bool PRESHIFT>
__device__ __forceinline__ uint32_t rescale32_high_x4(const uint32_t* v, const int32_t (*cols)[8])
{
    int32_t z[4];
#pragma unroll
    for (int i = 0; i < 4; i++)
    {
        const int4 c0 = *reinterpret_cast<const int4*>(&cols[i][0]);
        const int4 c1 = *reinterpret_cast<const int4*>(&cols[i][4]);
        int32_t a     = (int32_t)v[i];
        // (without double rounding the two constants are equal and the selection is a no-op: one code path for both)
        const int64_t r = a >= 0 ? (((int64_t)c0.w << 32) | (uint32_t)c0.z) : (((int64_t)c1.y << 32) | (uint32_t)c1.x);
        if (PRESHIFT)
            a = (int32_t)((uint32_t)a << c1.w);
        const int64_t prod = (int64_t)a * (int64_t)c0.x + r;
        z[i]               = (int32_t)(prod >> 32) >> c0.y;
    }
    return pack4_sat_i8(z[0], z[1], z[2], z[3]);
}

#include "tc_conv_lean.cuh"

template <int EPI>
__global__ void __launch_bounds__(kNumThreads, 2) tc_gemm_kernel(const __grid_constant__ TcKernelParams p)
{
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[kMaxStages];
    __shared__ __align__(8) uint64_t bar_empty[kMaxStages];
    __shared__ __align__(8) uint64_t bar_tmem_full[2];
    __shared__ __align__(8) uint64_t bar_tmem_empty[2];
    __shared__ __align__(8) uint64_t bar_drain;    // teardown after a wait gave up: "every MMA issued so far has retired"
    __shared__ uint32_t tmem_base_holder;
    __shared__ int abort_flag;
    // TC_EPI_RESCALE: per-column scaling constants of the current column block, written once per block by the
    // epilogue threads: {multiplier, shift, round(v >= 0) lo/hi, round(v < 0) lo/hi, largest |v| allowed, 0}
    __shared__ __align__(16) int32_t epi_cols[EPI == TC_EPI_RESCALE ? 256 : 1][8];
    __shared__ int32_t epi_vlim_min;    // smallest per-column value limit of the current column block
    __shared__ int epi_flags;           // EPI_COLS_* of the current column block

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0)
        TB200_TRACE(p, 0);

    // ring buffer base, 1024-byte aligned (swizzle atoms repeat every 1024 bytes)
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < p.num_stages; s++)
        {
            ptx::mbar_init(ptx::smem_u32(&bar_full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&bar_empty[s]), 1);
        }
        for (int a = 0; a < 2; a++)
        {
            ptx::mbar_init(ptx::smem_u32(&bar_tmem_full[a]), 1);
            ptx::mbar_init(ptx::smem_u32(&bar_tmem_empty[a]), kEpiThreads);
        }
        ptx::mbar_init(ptx::smem_u32(&bar_drain), 1);
        abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tmap(&p.tmA);
        ptx::prefetch_tmap(&p.tmB);
    }
    if (warp == 1)
    {
        ptx::tmem_alloc(ptx::smem_u32(&tmem_base_holder), (uint32_t)p.tmem_cols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_holder;
    if (threadIdx.x == 0)
        TB200_TRACE(p, 1);

    if (warp == 0)
    {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0)
        {
            // All loop-carried quantities are running counters: this single thread sits on the critical path of the
            // pipeline, so it avoids divisions and recomputed addresses.
            int stage = 0, group_pos = 0;
            uint32_t phase = 0;
            bool ok = true;
            const int ksub = p.ksub, num_stages = p.num_stages, group = p.commit_group;
            const int a_chunk_bytes = p.a_chunk_bytes, b_chunk_bytes = p.b_chunk_bytes, chunk_elems = p.chunk_elems;
            const uint32_t tx_per_chunk = (uint32_t)p.tx_bytes_per_chunk;
            uint32_t sA_stage = smem_base;
            for (int tile = p.tile_begin + blockIdx.x; tile < p.tile_end && ok; tile += gridDim.x)
            {
                const TileCoord t = decode_tile(p, tile);
                const int ax0 = t.x0 * p.stride_x - p.pad_l;
                const int ay0 = t.y0 * p.stride_y - p.pad_t;
                int chunk_k = 0, cc = 0, ky = 0, kx = 0;    // K offset of the running chunk, its (tap, channel block)
                int chunks_left = p.total_chunks;
                while (chunks_left > 0)
                {
                    // stages are released in groups of `commit_group` (one tcgen05.commit per group): the first stage
                    // of a group waits for the group's last barrier, the others are free by then
                    if (group_pos == 0 &&
                        !ptx::mbar_wait_bounded(ptx::smem_u32(&bar_empty[stage + group - 1]), phase ^ 1u, p.wait_limit))
                    {
                        ok = false;
                        break;
                    }
                    const int nchunks   = min(ksub, chunks_left);
                    chunks_left -= nchunks;
                    const uint32_t full = ptx::smem_u32(&bar_full[stage]);
                    uint32_t sA         = sA_stage;
                    uint32_t sB         = sA_stage + ksub * a_chunk_bytes;
                    if (TB200_DIAG_BIT(p.debug, 4))
                    {
                        ptx::mbar_arrive(full);
                    }
                    else
                    {
                        ptx::mbar_arrive_expect_tx(full, (uint32_t)nchunks * tx_per_chunk);
                        for (int j = 0; j < nchunks; j++)
                        {
                            ptx::tma_load_4d(sA, &p.tmA, full, cc * chunk_elems, ax0 + kx * p.dil_x, ay0 + ky * p.dil_y,
                                             t.n0);
                            if (!p.b_mn_major)
                            {
                                ptx::tma_load_3d(sB, &p.tmB, full, chunk_k, t.col0, 0);
                            }
                            else
                            {
                                for (int bx = 0; bx < p.b_nbox; bx++)
                                    ptx::tma_load_3d(sB + bx * p.b_box_bytes, &p.tmB, full, t.col0 + bx * p.b_box_n, chunk_k,
                                                     t.y0);
                            }
                            sA += a_chunk_bytes;
                            sB += b_chunk_bytes;
                            chunk_k += chunk_elems;
                            if (++cc == p.chunks_per_tap)
                            {
                                cc = 0;
                                if (++kx == p.KW)
                                {
                                    kx = 0;
                                    ky++;
                                }
                            }
                        }
                    }
                    if (++group_pos == group)
                        group_pos = 0;
                    sA_stage += p.stage_bytes;
                    if (++stage == num_stages)
                    {
                        stage    = 0;
                        sA_stage = smem_base;
                        phase ^= 1u;
                    }
                }
                if (tile == p.tile_begin + (int)blockIdx.x)
                    TB200_TRACE(p, 2);
            }
            TB200_TRACE(p, 3);
            if (!ok)
            {
                atomicOr(p.status, TB200_DEV_TIMEOUT);
                atomicExch(&abort_flag, 1);
            }
        }
    }
    else if (warp == 1)
    {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0)
        {
            // Same discipline as the producer: running counters and descriptor words only.  The two descriptors
            // differ between MMAs only in their 14-bit start-address field (16-byte units), so they are advanced by
            // adding to the low word.
            int stage = 0, group_pos = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            const int ksub = p.ksub, num_stages = p.num_stages, group = p.commit_group, mmas = p.mmas_per_chunk;
            const uint32_t idesc = p.idesc;
            const uint64_t a_chunk16 = (uint64_t)(p.a_chunk_bytes >> 4), b_chunk16 = (uint64_t)(p.b_chunk_bytes >> 4);
            const uint64_t b_kstep16 = (uint64_t)(p.b_kstep_bytes >> 4), stage16 = (uint64_t)(p.stage_bytes >> 4);
            const uint64_t ad_ring0 = ptx::smem_desc(p.a_desc_hi, smem_base);
            const uint64_t bd_ring0 = ptx::smem_desc(p.b_desc_hi, smem_base + ksub * p.a_chunk_bytes);
            uint64_t ad_stage = ad_ring0, bd_stage = bd_ring0;
            const bool issue = !TB200_DIAG_BIT(p.debug, 2);
            for (int tile = p.tile_begin + blockIdx.x; tile < p.tile_end && ok; tile += gridDim.x)
            {
                if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bar_tmem_empty[acc]), acc_phase ^ 1u, p.wait_limit))
                {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * p.block_n);
                uint32_t accum  = 0;    // the first MMA of a tile overwrites the accumulator
                int chunks_left = p.total_chunks;
                while (chunks_left > 0)
                {
                    if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bar_full[stage]), phase, p.wait_limit))
                    {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    if (tile == p.tile_begin + (int)blockIdx.x && chunks_left == p.total_chunks)
                        TB200_TRACE(p, 4);
                    const int nchunks = min(ksub, chunks_left);
                    chunks_left -= nchunks;
                    if (issue)
                    {
                        uint64_t ad_chunk = ad_stage, bd_chunk = bd_stage;
                        for (int j = 0; j < nchunks; j++)
                        {
                            uint64_t ad = ad_chunk, bd = bd_chunk;
                            for (int m = 0; m < mmas; m++)
                            {
                                if (EPI == TC_EPI_FLOAT)
                                {
                                    if (p.is_f16_kind == 2)
                                        ptx::mma_f8_ss(d_tmem, ad, bd, idesc, accum);
                                    else
                                        ptx::mma_f16_ss(d_tmem, ad, bd, idesc, accum);
                                }
                                else
                                    ptx::mma_i8_ss(d_tmem, ad, bd, idesc, accum);
                                accum = 1;
                                ad += 2;    // 32 bytes of K
                                bd += b_kstep16;
                            }
                            ad_chunk += a_chunk16;
                            bd_chunk += b_chunk16;
                        }
                    }
                    if (++group_pos == group)
                    {
                        ptx::mma_commit(ptx::smem_u32(&bar_empty[stage]));
                        group_pos = 0;
                    }
                    ad_stage += stage16;
                    bd_stage += stage16;
                    if (++stage == num_stages)
                    {
                        stage    = 0;
                        ad_stage = ad_ring0;
                        bd_stage = bd_ring0;
                        phase ^= 1u;
                    }
                }
                if (!ok)
                    break;
                ptx::mma_commit(ptx::smem_u32(&bar_tmem_full[acc]));
                if (tile == p.tile_begin + (int)blockIdx.x)
                    TB200_TRACE(p, 5);
                if (++acc == p.acc_bufs)
                {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
            TB200_TRACE(p, 6);
            if (!ok)
            {
                atomicOr(p.status, TB200_DEV_TIMEOUT);
                atomicExch(&abort_flag, 1);
            }
        }
    }
    else
    {
        // ------------------------------------------------------------------ epilogue warps
        const int quarter = warp & 3;    // TMEM lane quarter this warp may read
        const int half    = (warp - 2) >> 2;    // two warps share a quarter: even / odd 32-column chunks
        const int row     = quarter * 32 + lane;
        const int xx      = row % p.BW;
        const int yy      = (row / p.BW) % p.BH;
        const int nn      = row / (p.BW * p.BH);
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        int dev_flags = 0;
        int cols_loaded_for = -1;
        bool lean_block = false;    // the current column block runs the lean RESCALE form (same in every epilogue thread)
        for (int tile = p.tile_begin + blockIdx.x; tile < p.tile_end; tile += gridDim.x)
        {
            const TileCoord t = decode_tile(p, tile);
            if (EPI == TC_EPI_RESCALE && cols_loaded_for != t.col0)
            {
                // (re)build the per-column constants; the named barrier keeps the 128 epilogue threads in step
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (threadIdx.x == 64)
                {
                    epi_vlim_min = 2147483647;
                    // the short form packs to int8 with saturation and stores whole 32-column chunks
                    const bool shortable = p.out_es == 1 && (p.OC & 31) == 0 && p.clamp_lo >= -128 &&
                                           p.clamp_hi <= 127 && p.clamp_lo <= p.clamp_hi && p.out_zp >= -128 &&
                                           p.out_zp <= 127 && !TB200_DIAG_BIT(p.debug, 8);
                    epi_flags = shortable ? 0 : EPI_COLS_GENERIC;
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");
                // Lean form first: the records were prepared with the layer's other tables; one unusable column (its
                // value range could not be proven small enough) sends the whole block to the forms below.
                lean_block = false;
                if (p.rec != nullptr && !(epi_flags & EPI_COLS_GENERIC))
                {
                    for (int c = (int)threadIdx.x - 64; c < p.block_n; c += kEpiThreads)
                    {
                        const int4* rp = reinterpret_cast<const int4*>(p.rec + (int64_t)(t.col0 + c) * 8);
                        const int4 r0 = __ldg(rp), r1 = __ldg(rp + 1);
                        if (r1.w == 0)
                            atomicOr(&epi_flags, EPI_COLS_NOT_LEAN);
                        *reinterpret_cast<int4*>(&epi_cols[c][0]) = r0;
                        *reinterpret_cast<int4*>(&epi_cols[c][4]) = r1;
                    }
                    asm volatile("bar.sync 1, 256;" ::: "memory");
                    lean_block = !(epi_flags & EPI_COLS_NOT_LEAN);
                    if (lean_block)
                    {
                        cols_loaded_for = t.col0;
                        goto cols_ready;
                    }
                    // (the general construction below overwrites epi_cols: every thread has read the flag by now)
                    asm volatile("bar.sync 1, 256;" ::: "memory");
                }
                for (int c = (int)threadIdx.x - 64; c < p.block_n; c += kEpiThreads)
                {
                    if (t.col0 + c >= p.OC)
                        continue;
                    const int32_t m = __ldg(p.mult_pad + t.col0 + c);
                    const int32_t s = (int32_t)__ldg(p.shift_pad + t.col0 + c);
                    int f = 0;
                    // high-word form: out_zp * 2^shift clear of the int64 range
                    if (m < 0 || s < 2 || s > 54)
                        f |= EPI_COLS_GENERIC;
                    if (s < 32)
                        f |= EPI_COLS_PRESHIFT;
                    if (f & ~epi_flags)
                        atomicOr(&epi_flags, f);
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");
                const bool high_form = !(epi_flags & EPI_COLS_GENERIC);
                for (int c = (int)threadIdx.x - 64; c < p.block_n; c += kEpiThreads)
                {
                    const int32_t m = __ldg(p.mult_pad + t.col0 + c);
                    const int32_t s = (int32_t)__ldg(p.shift_pad + t.col0 + c);
                    const bool valid  = (m >= 0) && (s >= 2) && (s <= 62);
                    const int32_t sc  = valid ? s : 2;
                    const int64_t half = (int64_t)1 << (sc - 1);
                    int64_t rpos = half, rneg = half;
                    const bool dr = p.double_round && sc > 31;
                    if (dr)
                    {
                        rpos += (int64_t)1 << 30;
                        rneg -= (int64_t)1 << 30;
                    }
                    // apply_scale_32 requires -2^(shift-1) <= v < 2^(shift-1); invalid operands fail every value
                    const int32_t vlim = !valid ? -1 : (sc - 1 >= 31 ? 2147483647 : (int32_t)(half - 1));
                    int4 lo4, hi4;
                    if (high_form && t.col0 + c < p.OC)
                    {
                        const int k       = sc < 32 ? 32 - sc : 0;
                        const int64_t z64 = (int64_t)p.out_zp * ((int64_t)1 << (sc + k));
                        rpos = rpos * ((int64_t)1 << k) + z64;
                        rneg = rneg * ((int64_t)1 << k) + z64;
                        lo4 = make_int4(m, sc + k - 32, (int32_t)(uint32_t)(rpos & 0xffffffffLL), (int32_t)(rpos >> 32));
                        hi4 = make_int4((int32_t)(uint32_t)(rneg & 0xffffffffLL), (int32_t)(rneg >> 32), vlim, k);
                    }
                    else
                    {
                        lo4 = make_int4(m, sc, (int32_t)(uint32_t)(rpos & 0xffffffffLL), (int32_t)(rpos >> 32));
                        hi4 = make_int4((int32_t)(uint32_t)(rneg & 0xffffffffLL), (int32_t)(rneg >> 32), vlim, 0);
                    }
                    if (t.col0 + c < p.OC)
                        atomicMin(&epi_vlim_min, vlim);
                    *reinterpret_cast<int4*>(&epi_cols[c][0]) = lo4;
                    *reinterpret_cast<int4*>(&epi_cols[c][4]) = hi4;
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");
                cols_loaded_for = t.col0;
            }
        cols_ready:
            // After a wait has given up this warp only keeps visiting the named barrier above (the other epilogue
            // warps may still be running and would otherwise block on it); it does no further work.
            if (!ok)
                continue;
            ok = ptx::mbar_wait_bounded(ptx::smem_u32(&bar_tmem_full[acc]), acc_phase, p.wait_limit);
            // the whole warp must agree before the warp-collective TMEM loads
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                continue;
            ptx::tc_fence_after_sync();
            if (threadIdx.x == 64 && tile == p.tile_begin + (int)blockIdx.x)
                TB200_TRACE(p, 7);

            const int ox = t.x0 + xx, oy = t.y0 + yy, on = t.n0 + nn;
            const bool row_valid = (nn < p.BN) && (ox < p.OW) && (oy < p.OH) && (on < p.N);
            // index of this row's pixel in the output tensor (a dense grid, or one phase of a strided one)
            int pn = on, py = oy, px = ox;
            if (p.flat_iw != 0)
            {
                // the pixel grid was flattened to one row of N*IH*IW pixels: recover the coordinates for the strided store
                px          = ox % p.flat_iw;
                const int t = ox / p.flat_iw;
                py          = t % p.flat_ih;
                pn          = t / p.flat_ih;
            }
            const int64_t pix = ((int64_t)pn * p.out_OH + py * p.out_sy + p.out_y0) * p.out_OW + px * p.out_sx + p.out_x0;
            // the neighbouring lane's row (lane ^ 1), for stores that fill whole 32-byte sectors between two lanes
            const int64_t pix_pair     = __shfl_xor_sync(0xffffffffu, pix, 1);
            const bool row_valid_pair  = __shfl_xor_sync(0xffffffffu, (int)row_valid, 1) != 0;

            // Additive per-column constants of this row (bias and zero-point terms).  For a padded convolution with a
            // non-zero input zero point the constant depends on which filter taps fall inside the image, so the table
            // has one row per (ky_lo, ky_hi, kx_lo, kx_hi) rectangle of in-scope taps; interior pixels share one row.
            const int32_t* corr_row  = nullptr;
            const int32_t* delta_row = nullptr;    // lean form: what a border pixel adds to reach its own correction row
            if (EPI != TC_EPI_FLOAT && p.corr != nullptr)
            {
                int cls = 0;
                if (p.corr_classes)
                {
                    int ky_lo = 0, ky_hi = p.KH, kx_lo = 0, kx_hi = p.KW;
                    if (row_valid)
                    {
                        const int iy0 = oy * p.stride_y - p.pad_t;
                        const int ix0 = ox * p.stride_x - p.pad_l;
                        if (iy0 < 0)
                            ky_lo = (-iy0 + p.dil_y - 1) / p.dil_y;
                        if (ix0 < 0)
                            kx_lo = (-ix0 + p.dil_x - 1) / p.dil_x;
                        if (iy0 + (p.KH - 1) * p.dil_y >= p.IH)
                            ky_hi = iy0 >= p.IH ? 0 : (p.IH - 1 - iy0) / p.dil_y + 1;
                        if (ix0 + (p.KW - 1) * p.dil_x >= p.IW)
                            kx_hi = ix0 >= p.IW ? 0 : (p.IW - 1 - ix0) / p.dil_x + 1;
                        ky_lo = min(ky_lo, p.KH);
                        kx_lo = min(kx_lo, p.KW);
                        ky_hi = max(ky_hi, ky_lo);
                        kx_hi = max(kx_hi, kx_lo);
                    }
                    cls = ((ky_lo * (p.KH + 1) + ky_hi) * (p.KW + 1) + kx_lo) * (p.KW + 1) + kx_hi;
                }
                corr_row = p.corr + (int64_t)cls * p.corr_stride +
                           (int64_t)((p.corr_ystride && row_valid) ? oy : 0) * p.corr_ystride;
                if (EPI == TC_EPI_RESCALE && p.corr_classes && p.delta != nullptr && cls != p.cls_interior)
                    delta_row = p.delta + (int64_t)cls * p.corr_stride;
            }
            int32_t rc = 0;
            if (EPI == TC_EPI_I32 && p.row_corr != nullptr && row_valid)
                rc = p.row_corr[((int64_t)on * p.OH + oy) * p.OW + ox];

            const uint32_t taddr_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * p.block_n);
            const int ncol_chunks = p.block_n / 32;
            for (int c = half; c < ncol_chunks; c += 2)
            {
                uint32_t v[32];
                ptx::tmem_ld_32x32b_x32(taddr_row + (uint32_t)(c * 32), v);
                ptx::tmem_ld_wait();
                const int col = t.col0 + c * 32;
                if (col >= p.OC || TB200_DIAG_BIT(p.debug, 1))
                    continue;
                const int nvalid = min(32, p.OC - col);
                // element offset of (this row, col) in the output, and of the neighbouring lane's row
                int64_t ooff = pix * p.OC + col, ooff_pair = pix_pair * p.OC + col;
                bool rv = row_valid, rv_pair = row_valid_pair;    // validity of this row's (and the neighbour lane's) store
                if (p.d2s_oc != 0)
                {
                    // columns are (ky, kx, oc): a block of d2s_oc channels per output pixel of the stamp
                    const int ph = col / p.d2s_oc, ky = ph / p.d2s_kw, kx = ph - ky * p.d2s_kw;
                    const int64_t within = ((int64_t)ky * p.out_OW + kx) * p.d2s_oc + (col - ph * p.d2s_oc);
                    ooff      = pix * p.d2s_oc + within;
                    ooff_pair = pix_pair * p.d2s_oc + within;
                    // the last macro-pixel of a row or column may reach past the output (odd sizes, cropping out_pad)
                    const bool inside = (py * p.out_sy + ky < p.out_OH) && (px * p.out_sx + kx < p.out_OW);
                    rv            = rv && inside;
                    rv_pair       = false;    // such outputs are 32-byte aligned: the paired-lane store form is never taken
                }

                if (EPI == TC_EPI_RESCALE && lean_block)
                {
                    // the interior correction is part of the records; border pixels add their difference to it
                    if (delta_row != nullptr)
                    {
                        const int4* dp = reinterpret_cast<const int4*>(delta_row + col);
#pragma unroll
                        for (int q = 0; q < 8; q++)
                        {
                            const int4 dv = __ldg(dp + q);
                            v[4 * q + 0] += (uint32_t)dv.x;
                            v[4 * q + 1] += (uint32_t)dv.y;
                            v[4 * q + 2] += (uint32_t)dv.z;
                            v[4 * q + 3] += (uint32_t)dv.w;
                        }
                    }
                }
                else if (EPI != TC_EPI_FLOAT && corr_row != nullptr && !TB200_DIAG_BIT(p.debug, 16))
                {
                    // every per-column array is padded to a multiple of the tile width: unconditional 128-bit loads
                    const int4* cp = reinterpret_cast<const int4*>(corr_row + col);
#pragma unroll
                    for (int q = 0; q < 8; q++)
                    {
                        const int4 cv = __ldg(cp + q);
                        v[4 * q + 0] += (uint32_t)cv.x;
                        v[4 * q + 1] += (uint32_t)cv.y;
                        v[4 * q + 2] += (uint32_t)cv.z;
                        v[4 * q + 3] += (uint32_t)cv.w;
                    }
                }

                if (EPI == TC_EPI_I32)
                {
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        v[i] += (uint32_t)rc;
                    if (rv)
                    {
                        int32_t* o = reinterpret_cast<int32_t*>(p.out) + ooff;
                        if (nvalid == 32 && ((p.OC & 7) == 0) && (reinterpret_cast<uintptr_t>(p.out) & 31) == 0)
                        {
#pragma unroll
                            for (int i = 0; i < 32; i += 8)
                                ptx::st_global_v8(o + i, v[i], v[i + 1], v[i + 2], v[i + 3], v[i + 4], v[i + 5], v[i + 6], v[i + 7]);
                        }
                        else if (nvalid == 32 && ((p.OC & 3) == 0))
                        {
#pragma unroll
                            for (int i = 0; i < 32; i += 4)
                                *reinterpret_cast<int4*>(o + i) =
                                    make_int4((int)v[i], (int)v[i + 1], (int)v[i + 2], (int)v[i + 3]);
                        }
                        else
                        {
#pragma unroll
                            for (int i = 0; i < 32; i++)
                                if (i < nvalid)
                                    o[i] = (int32_t)v[i];
                        }
                    }
                }
                else if (EPI == TC_EPI_RESCALE)
                {
                    // REQUIRE checks of apply_scale_32.  With multiplier < 2^31, a value inside the accepted range
                    // -2^(shift-1) <= v < 2^(shift-1) always scales to |result| <= 2^30 + 1, so the "fits int32" checks
                    // (before and after adding the small output zero point) follow from the range check.  The range
                    // check itself is done on the largest magnitude of the 32 values against the smallest limit of
                    // the column block; only when that fails are the columns compared one by one.
                    const int cflags = epi_flags;
                    if (!(cflags & EPI_COLS_GENERIC))
                    {
                        bool bad = false;
                        uint32_t w[8];
                        if (lean_block)
                        {
                            // no REQUIRE can fail here: the records exist only for columns whose value range was proven
#pragma unroll
                            for (int q = 0; q < 8; q++)
                            {
                                int32_t z[4];
#pragma unroll
                                for (int j = 0; j < 4; j++)
                                {
                                    const int32_t(*rcol)[8] = &epi_cols[c * 32 + 4 * q + j];
                                    const int4 r0 = *reinterpret_cast<const int4*>(&(*rcol)[0]);
                                    const int2 r1 = *reinterpret_cast<const int2*>(&(*rcol)[4]);
                                    z[j] = rescale_rec_apply((int32_t)v[4 * q + j], r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, p.double_round != 0);
                                }
                                w[q] = pack4_sat_i8(z[0], z[1], z[2], z[3]);
                            }
                        }
                        else if (cflags & EPI_COLS_PRESHIFT)
                        {
                            // some shift of the block is below 32: the range check of apply_scale_32 can fail there
                            int32_t vmax = -2147483647 - 1, vmin = 2147483647;
#pragma unroll
                            for (int i = 0; i < 32; i++)
                            {
                                vmax = max(vmax, (int32_t)v[i]);
                                vmin = min(vmin, (int32_t)v[i]);
                            }
                            const int32_t lim = epi_vlim_min;
                            if (vmax > lim || vmin < ~lim)
                            {
                                for (int i = 0; i < 32; i++)
                                {
                                    const int32_t vl = epi_cols[c * 32 + i][6];
                                    int32_t a = 0;
#pragma unroll
                                    for (int j = 0; j < 32; j++)
                                        a = (j == i) ? (int32_t)v[j] : a;
                                    bad |= (a > vl) || (a < ~vl);
                                }
                            }
#pragma unroll
                            for (int q = 0; q < 8; q++)
                                w[q] = rescale32_high_x4<true>(&v[4 * q], &epi_cols[c * 32 + 4 * q]);
                        }
                        else
                        {
                            // every shift of the block is at least 32: apply_scale_32 accepts all of int32
#pragma unroll
                            for (int q = 0; q < 8; q++)
                                w[q] = rescale32_high_x4<false>(&v[4 * q], &epi_cols[c * 32 + 4 * q]);
                        }
                        if (bad && rv)
                            dev_flags |= TB200_DEV_UNPREDICTABLE;
                        // a CLAMP narrower than int8 (rare) works on the packed bytes
                        if (p.clamp_lo > -128 || p.clamp_hi < 127)
                        {
                            const uint32_t lo4 = (uint32_t)(p.clamp_lo & 0xff) * 0x01010101u;
                            const uint32_t hi4 = (uint32_t)(p.clamp_hi & 0xff) * 0x01010101u;
#pragma unroll
                            for (int q = 0; q < 8; q++)
                                w[q] = __vmins4(__vmaxs4(w[q], lo4), hi4);
                        }
                        // Each lane holds the 32 output bytes of its own row: one 32-byte store hands the memory system a
                        // complete sector (two 16-byte stores would deliver two half-filled ones).  Outputs that are not
                        // 32-byte aligned (views) swap halves between the two lanes of a pair instead, so that one store
                        // instruction writes the even lane's row and the next one the odd lane's row.
                        const bool skip = TB200_DIAG_BIT(p.debug, 32) && w[0] != 0x12345678u;
                        if ((reinterpret_cast<uintptr_t>(p.out) & 31) == 0)
                        {
                            if (rv && !skip)
                                ptx::st_global_v8(reinterpret_cast<int8_t*>(p.out) + ooff, w[0], w[1], w[2], w[3],
                                                  w[4], w[5], w[6], w[7]);
                        }
                        else
                        {
                            const bool odd = (lane & 1) != 0;
                            uint32_t other[4];
#pragma unroll
                            for (int k = 0; k < 4; k++)
                                other[k] = __shfl_xor_sync(0xffffffffu, odd ? w[k] : w[4 + k], 1);
                            int8_t* o_own  = reinterpret_cast<int8_t*>(p.out) + ooff + (odd ? 16 : 0);
                            int8_t* o_pair = reinterpret_cast<int8_t*>(p.out) + ooff_pair + (odd ? 16 : 0);
                            const uint4 mine   = odd ? make_uint4(w[4], w[5], w[6], w[7]) : make_uint4(w[0], w[1], w[2], w[3]);
                            const uint4 theirs = make_uint4(other[0], other[1], other[2], other[3]);
                            if ((odd ? rv_pair : rv) && !skip)
                                *reinterpret_cast<uint4*>(odd ? o_pair : o_own) = odd ? theirs : mine;
                            if ((odd ? rv : rv_pair) && !skip)
                                *reinterpret_cast<uint4*>(odd ? o_own : o_pair) = odd ? mine : theirs;
                        }
                        continue;
                    }
                    bool bad = false;
                    {
                        int32_t vmax = -2147483647 - 1, vmin = 2147483647;
                #pragma unroll
                        for (int i = 0; i < 32; i++)
                        {
                            vmax = max(vmax, (int32_t)v[i]);
                            vmin = min(vmin, (int32_t)v[i]);
                        }
                        const int32_t lim = epi_vlim_min;
                        if (vmax > lim || vmin < ~lim)
                        {
                            for (int i = 0; i < nvalid; i++)
                            {
                                const int32_t vl = epi_cols[c * 32 + i][6];
                                int32_t a = 0;
                #pragma unroll
                                for (int j = 0; j < 32; j++)
                                    a = (j == i) ? (int32_t)v[j] : a;
                                bad |= (a > vl) || (a < ~vl);
                            }
                        }
                    }
                #pragma unroll
                    for (int i = 0; i < 32; i++)
                    {
                        // QuantUtil::apply_scale_32 with the per-column constants prepared above; the 64-bit product
                        // is kept as two words so that the shift is one 32-bit operation either way
                        const int4 c0 = *reinterpret_cast<const int4*>(&epi_cols[c * 32 + i][0]);
                        const int2 c1 = *reinterpret_cast<const int2*>(&epi_cols[c * 32 + i][4]);
                        const int32_t a = (int32_t)v[i];
                        const int64_t rpos = ((int64_t)c0.w << 32) | (uint32_t)c0.z;
                        const int64_t rneg = ((int64_t)c1.y << 32) | (uint32_t)c1.x;
                        const int64_t prod = (int64_t)a * (int64_t)c0.x + (a >= 0 ? rpos : rneg);
                        const uint32_t plo = (uint32_t)prod;
                        const int32_t phi  = (int32_t)(prod >> 32);
                        const int32_t sh   = c0.y;
                        const int32_t res  = sh >= 32 ? (phi >> (sh - 32)) : (int32_t)__funnelshift_r(plo, (uint32_t)phi, sh);
                        int32_t z = res + p.out_zp;
                        z = max(z, p.clamp_lo);
                        z = min(z, p.clamp_hi);
                        v[i] = (uint32_t)z;
                    }

                    if (rv)
                    {
                        if (p.out_es == 1)
                        {
                            int8_t* o = reinterpret_cast<int8_t*>(p.out) + ooff;
                            if (nvalid == 32 && ((p.OC & 15) == 0))
                            {
                                uint4 w0 = make_uint4(pack4_i8(v[0], v[1], v[2], v[3]), pack4_i8(v[4], v[5], v[6], v[7]),
                                                      pack4_i8(v[8], v[9], v[10], v[11]), pack4_i8(v[12], v[13], v[14], v[15]));
                                uint4 w1 = make_uint4(pack4_i8(v[16], v[17], v[18], v[19]), pack4_i8(v[20], v[21], v[22], v[23]),
                                                      pack4_i8(v[24], v[25], v[26], v[27]), pack4_i8(v[28], v[29], v[30], v[31]));
                                *reinterpret_cast<uint4*>(o)      = w0;
                                *reinterpret_cast<uint4*>(o + 16) = w1;
                            }
                            else
                            {
                #pragma unroll
                                for (int i = 0; i < 32; i++)
                                    if (i < nvalid)
                                        o[i] = (int8_t)(int32_t)v[i];
                            }
                        }
                        else if (p.out_es == 2)
                        {
                            int16_t* o = reinterpret_cast<int16_t*>(p.out) + ooff;
                #pragma unroll
                            for (int i = 0; i < 32; i++)
                                if (i < nvalid)
                                    o[i] = (int16_t)(int32_t)v[i];
                        }
                        else
                        {
                            int32_t* o = reinterpret_cast<int32_t*>(p.out) + ooff;
                #pragma unroll
                            for (int i = 0; i < 32; i++)
                                if (i < nvalid)
                                    o[i] = (int32_t)v[i];
                        }
                    }

                    if (bad && rv)
                        dev_flags |= TB200_DEV_UNPREDICTABLE;
                }
                else
                {
                    float f[32];
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        f[i] = __uint_as_float(v[i]);
                    if (p.bias_f_pad != nullptr)
                    {
                        const float4* bp = reinterpret_cast<const float4*>(p.bias_f_pad + col);
#pragma unroll
                        for (int q = 0; q < 8; q++)
                        {
                            const float4 b4 = __ldg(bp + q);
                            f[4 * q + 0] += b4.x;
                            f[4 * q + 1] += b4.y;
                            f[4 * q + 2] += b4.z;
                            f[4 * q + 3] += b4.w;
                        }
                    }
                    if (p.has_clamp)
                    {
#pragma unroll
                        for (int i = 0; i < 32; i++)
                        {
                            // NaN propagates: comparisons with NaN are false on both sides
                            f[i] = (f[i] < p.clamp_lo_f) ? p.clamp_lo_f : f[i];
                            f[i] = (f[i] > p.clamp_hi_f) ? p.clamp_hi_f : f[i];
                        }
                    }
                    if (!rv)
                        continue;
                    if (p.out_es == 4)
                    {
                        float* o = reinterpret_cast<float*>(p.out) + ooff;
                        if (nvalid == 32 && ((p.OC & 7) == 0) && (reinterpret_cast<uintptr_t>(p.out) & 31) == 0)
                        {
                            // 32 bytes per store: whole sectors (see the int32 epilogue)
#pragma unroll
                            for (int i = 0; i < 32; i += 8)
                                ptx::st_global_v8(o + i, __float_as_uint(f[i]), __float_as_uint(f[i + 1]), __float_as_uint(f[i + 2]),
                                                  __float_as_uint(f[i + 3]), __float_as_uint(f[i + 4]), __float_as_uint(f[i + 5]),
                                                  __float_as_uint(f[i + 6]), __float_as_uint(f[i + 7]));
                        }
                        else if (nvalid == 32 && ((p.OC & 3) == 0))
                        {
#pragma unroll
                            for (int i = 0; i < 32; i += 4)
                                *reinterpret_cast<float4*>(o + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
                        }
                        else
                        {
#pragma unroll
                            for (int i = 0; i < 32; i++)
                                if (i < nvalid)
                                    o[i] = f[i];
                        }
                    }
                    else
                    {
                        uint16_t h[32];
#pragma unroll
                        for (int i = 0; i < 32; i++)
                        {
                            if (p.out_is_bf16)
                                h[i] = __bfloat16_as_ushort(__float2bfloat16_rn(f[i]));
                            else
                                h[i] = __half_as_ushort(__float2half_rn(f[i]));
                        }
                        uint16_t* o = reinterpret_cast<uint16_t*>(p.out) + ooff;
                        if (nvalid == 32 && ((p.OC & 15) == 0) && (reinterpret_cast<uintptr_t>(p.out) & 31) == 0)
                        {
#pragma unroll
                            for (int i = 0; i < 32; i += 16)
                                ptx::st_global_v8(o + i, (uint32_t)h[i] | ((uint32_t)h[i + 1] << 16),
                                                  (uint32_t)h[i + 2] | ((uint32_t)h[i + 3] << 16),
                                                  (uint32_t)h[i + 4] | ((uint32_t)h[i + 5] << 16),
                                                  (uint32_t)h[i + 6] | ((uint32_t)h[i + 7] << 16),
                                                  (uint32_t)h[i + 8] | ((uint32_t)h[i + 9] << 16),
                                                  (uint32_t)h[i + 10] | ((uint32_t)h[i + 11] << 16),
                                                  (uint32_t)h[i + 12] | ((uint32_t)h[i + 13] << 16),
                                                  (uint32_t)h[i + 14] | ((uint32_t)h[i + 15] << 16));
                        }
                        else if (nvalid == 32 && ((p.OC & 7) == 0))
                        {
#pragma unroll
                            for (int i = 0; i < 32; i += 8)
                            {
                                uint4 w = make_uint4((uint32_t)h[i] | ((uint32_t)h[i + 1] << 16),
                                                     (uint32_t)h[i + 2] | ((uint32_t)h[i + 3] << 16),
                                                     (uint32_t)h[i + 4] | ((uint32_t)h[i + 5] << 16),
                                                     (uint32_t)h[i + 6] | ((uint32_t)h[i + 7] << 16));
                                *reinterpret_cast<uint4*>(o + i) = w;
                            }
                        }
                        else
                        {
#pragma unroll
                            for (int i = 0; i < 32; i++)
                                if (i < nvalid)
                                    o[i] = h[i];
                        }
                    }
                }
            }
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(ptx::smem_u32(&bar_tmem_empty[acc]));
            if (threadIdx.x == 64 && tile == p.tile_begin + (int)blockIdx.x)
                TB200_TRACE(p, 8);
            if (++acc == p.acc_bufs)
            {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
        if (threadIdx.x == 64)
            TB200_TRACE(p, 9);
        if (!ok && lane == 0)
        {
            atomicOr(p.status, TB200_DEV_TIMEOUT);
            atomicExch(&abort_flag, 1);
        }
        if (dev_flags)
            atomicOr(p.status, dev_flags);
    }

    // ---------------------------------------------------------------------- teardown
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag)
    {
        // a role gave up: let copies that may still be in flight land before the CTA's shared memory is released
        for (int s = 0; s < p.num_stages; s++)
        {
            ptx::mbar_wait_bounded(ptx::smem_u32(&bar_full[s]), 0u, 2000000LL);
            ptx::mbar_wait_bounded(ptx::smem_u32(&bar_full[s]), 1u, 2000000LL);
        }
    }
    if (warp == 1 && lane == 0 && abort_flag)
    {
        // ... and let the tensor-core work already issued retire before its accumulators' tensor memory is freed: the
        // role that normally waits for it (the epilogue) may be the one that gave up
        ptx::mma_commit(ptx::smem_u32(&bar_drain));
        ptx::mbar_wait_bounded(ptx::smem_u32(&bar_drain), 0u, 40000000LL);
    }
    __syncthreads();
    if (warp == 1)
    {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
    }
    if (threadIdx.x == 0)
        TB200_TRACE(p, 10);
}

// ------------------------------------------------------------------------------------------------ host side

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

PFN_encodeTiled get_encode_fn()
{
    static PFN_encodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_encodeTiled>(sym);
    });
    return fn;
}

struct TcPlan
{
    TcKernelParams kp;
    int smem_bytes;
    int grid;
    int ctas_per_sm;
    // tensor map recipes (filled by plan, encoded at launch)
    cuuint64_t a_dims[4], a_strides[3];
    cuuint32_t a_box[4], a_estr[4];
    cuuint64_t b_dims[3], b_strides[2];
    cuuint32_t b_box[3];
    CUtensorMapDataType dt;
    CUtensorMapSwizzle a_swz, b_swz;
    bool lean;    // launch tc_conv_lean_kernel
};

bool make_plan(const TcProblem& q, int num_sms, TcPlan* plan, std::string* why)
{
    auto no = [&](const char* m) {
        if (why)
            *why = m;
        return false;
    };
    const int es = (int)dtype_size(q.in_dtype);
    if (!(q.in_dtype == TB200_INT8 || q.in_dtype == TB200_FP16 || q.in_dtype == TB200_BF16 || dtype_is_fp8(q.in_dtype)))
        return no("element type has no tensor-core path");
    if (dtype_is_fp8(q.in_dtype) && q.epi != TC_EPI_FLOAT)
        return no("fp8 operands need the floating epilogue");
    if ((reinterpret_cast<uintptr_t>(q.a) & 15) || (reinterpret_cast<uintptr_t>(q.b) & 15))
        return no("operand base not 16-byte aligned");
    const int row_bytes = q.IC * es;    // contiguous K bytes of one tap
    if (row_bytes % 32 != 0)
        return no("channel run is not a multiple of 32 bytes");
    const int swz = (row_bytes % 128 == 0) ? 128 : (row_bytes % 64 == 0) ? 64 : 32;

    TcKernelParams& k = plan->kp;
    memset(&k, 0, sizeof(k));
    // A view.  A stride-1, pad-0 1x1 convolution (and MATMUL) is a plain GEMM over flattened pixels.
    int N = q.N, IH = q.IH, IW = q.IW, OH = q.OH, OW = q.OW;
    const int64_t sw = q.a_stride_w ? q.a_stride_w : (int64_t)q.IC;
    const int64_t sh = q.a_stride_h ? q.a_stride_h : sw * q.IW;
    const int64_t sn = q.a_stride_n ? q.a_stride_n : sh * q.IH;
    const bool dense = sw == q.IC && sh == sw * q.IW && sn == sh * q.IH;
    const bool pure_gemm = q.KH == 1 && q.KW == 1 && q.stride_y == 1 && q.stride_x == 1 && q.pad_t == 0 &&
                           q.pad_l == 0 && OH == IH && OW == IW && !q.b_mn_major && dense;
    const int view_iw = q.IW, view_ih = q.IH;
    if (pure_gemm)
    {
        int64_t pixels = (int64_t)N * IH * IW;
        if (pixels >= (1LL << 31))
            return no("too many pixels");
        IW = OW = (int)pixels;
        IH = OH = 1;
        N  = 1;
    }
    if (q.stride_x > 2 || q.stride_y > 256)
        return no("stride too large for the tile loader");
    int BW, BH = 1, BN = 1;
    if (OW >= kTileM)
        BW = kTileM;
    else
    {
        BW = OW;
        BH = std::min(OH, kTileM / BW);
        // prefer a row count that divides OH when it costs little
        for (int cand = BH; cand >= std::max(1, BH - 2); cand--)
            if (OH % cand == 0)
            {
                BH = cand;
                break;
            }
        if (BH == OH)
            BN = std::min(N, kTileM / (BW * BH));
    }
    if (q.b_mn_major)
    {
        BH = 1;
        BN = 1;
    }
    if (BW * q.stride_x > 256 || BH * q.stride_y > 256)
        return no("tile span exceeds the TMA box limit");

    k.BW = BW;
    k.BH = BH;
    k.BN = BN;
    k.N  = N;
    k.OH = OH;
    k.OW = OW;
    k.OC = q.OC;
    k.IH = IH;
    k.IW = IW;
    k.flat_iw = (q.out_sy && pure_gemm) ? view_iw : 0;
    k.flat_ih = (q.out_sy && pure_gemm) ? view_ih : 0;
    k.out_OH = q.out_sy ? q.out_OH : OH;
    k.out_OW = q.out_sy ? q.out_OW : OW;
    k.out_sy = q.out_sy ? q.out_sy : 1;
    k.out_sx = q.out_sy ? q.out_sx : 1;
    k.out_y0 = q.out_sy ? q.out_y0 : 0;
    k.out_x0 = q.out_sy ? q.out_x0 : 0;
    k.d2s_oc = q.out_sy ? q.d2s_oc : 0;
    k.d2s_kw = q.d2s_kw;
    if (k.d2s_oc != 0 && (k.d2s_oc % 32 != 0 || q.OC % k.d2s_oc != 0))
        return no("depth-to-space output needs channel blocks that are multiples of 32");
    k.tiles_x = (OW + BW - 1) / BW;
    k.tiles_y = (OH + BH - 1) / BH;
    k.tiles_n = (N + BN - 1) / BN;

    int block_n = diag_env_int("TB200_TC_BLOCK_N", 0);
    // one column block that covers all channels when there are at most 256 of them (no half-empty second block);
    // the epilogue works in 32-column chunks
    if (block_n == 0)
    {
        block_n = q.OC >= 256 ? 256 : q.OC > 128 ? (q.OC + 31) / 32 * 32 : q.OC > 64 ? 128 : q.OC > 32 ? 64 : 32;
        // A small layer (a shard of a batch, the last stages of a network) has fewer tiles than the GPU has SMs, and
        // each tile is a serial chain of load, MMAs and epilogue: narrower column blocks give every SM a tile and
        // shorten the chain.  Only for the fused int8 convolution, whose column blocks are independent.
        // Which width: the one with the smallest (rounds of CTAs) x (time of one tile), a tile costing its MMAs (about 190
        // cycles each at 256 columns, 125 below, commits included) plus its epilogue (about 25 cycles per column).  Halving
        // until every SM has a tile, as an earlier version did, went one step too far where the halved blocks needed a
        // second round (3x3 256 -> 256 on 32 x 14 x 14: 196 tiles of 64 columns, 21 us, against 98 tiles of 128).
        if (q.epi == TC_EPI_RESCALE && !q.b_mn_major && (block_n == 256 || block_n == 128) && q.OC % block_n == 0)
        {
            const int64_t tiles_m = (int64_t)k.tiles_x * k.tiles_y * k.tiles_n;
            if (tiles_m * (q.OC / block_n) < (int64_t)num_sms)    // only layers that cannot give every SM a tile at the default width
            {
                const int64_t kmmas = ((int64_t)q.KH * q.KW * q.IC * es + 31) / 32;
                int64_t best_cost   = 0;
                int best            = block_n;
                for (int bn = block_n; bn >= 64 && q.OC % bn == 0; bn /= 2)
                {
                    const int64_t rounds = (tiles_m * (q.OC / bn) + num_sms - 1) / num_sms;
                    const int64_t cost   = rounds * (kmmas * (bn == 256 ? 190 : 125) + 25 * bn);
                    if (bn == block_n || cost * 100 < best_cost * 97)    // a narrower block has to win by 3 %
                    {
                        best_cost = cost;
                        best      = bn;
                    }
                }
                block_n = best;
            }
        }
    }
    if (q.b_mn_major && (block_n * es) % 128 != 0)
        block_n = 128 / es * ((block_n * es + 127) / 128);
    if (block_n > 256 || block_n % 32 != 0)
        return no("bad block_n");
    k.block_n   = block_n;
    k.tiles_col = (q.OC + block_n - 1) / block_n;
    int64_t nt  = (int64_t)k.tiles_x * k.tiles_y * k.tiles_n * k.tiles_col;
    if (nt >= (1LL << 31))
        return no("too many tiles");
    k.num_tiles = (int)nt;

    k.KH = q.KH;
    k.KW = q.KW;
    k.chunk_elems    = swz / es;
    k.chunks_per_tap = row_bytes / swz;
    k.total_chunks   = q.KH * q.KW * k.chunks_per_tap;
    k.ksub           = std::min(std::max(1, diag_env_int("TB200_TC_KSUB", 128 / swz)), k.total_chunks);
    k.num_kstages    = (k.total_chunks + k.ksub - 1) / k.ksub;
    k.pad_t = q.pad_t;
    k.pad_l = q.pad_l;
    k.stride_y = q.stride_y;
    k.stride_x = q.stride_x;
    k.dil_y = q.dil_y;
    k.dil_x = q.dil_x;
    k.mmas_per_chunk = swz / 32;

    const uint32_t layout = swz == 128 ? 2u : swz == 64 ? 4u : 6u;
    k.a_chunk_bytes = ((kTileM * swz) + 1023) & ~1023;
    k.a_desc_hi     = ptx::make_smem_desc_hi(16, 8 * swz, layout);
    k.b_mn_major    = q.b_mn_major;
    int a_tx        = BW * BH * BN * swz;
    int b_tx;
    if (!q.b_mn_major)
    {
        if (((int64_t)q.KH * q.KW * q.IC * es) % 16 != 0)
            return no("weight row stride not 16-byte aligned");
        k.b_chunk_bytes = ((block_n * swz) + 1023) & ~1023;
        k.b_desc_hi     = ptx::make_smem_desc_hi(16, 8 * swz, layout);
        k.b_kstep_bytes = 32;
        b_tx            = block_n * swz;
    }
    else
    {
        if (swz != 128)
            return no("MN-major B needs 128-byte K chunks of A");
        if (((q.b_ld ? q.b_ld : (int64_t)q.OC) * es) % 16 != 0)
            return no("B row stride not 16-byte aligned");
        k.b_box_n       = 128 / es;
        k.b_nbox        = block_n / k.b_box_n;
        k.b_box_bytes   = k.chunk_elems * 128;
        k.b_chunk_bytes = k.b_nbox * k.b_box_bytes;
        const int lbo   = diag_env_int("TB200_TC_MN_LBO", k.b_box_bytes);
        const int sbo   = diag_env_int("TB200_TC_MN_SBO", 1024);
        k.b_desc_hi     = ptx::make_smem_desc_hi(lbo, sbo, 2u);
        k.b_kstep_bytes = diag_env_int("TB200_TC_MN_KSTEP", (32 / es) * 128);
        b_tx            = k.b_chunk_bytes;
    }
    k.tx_bytes_per_chunk = a_tx + b_tx;
    k.stage_bytes        = k.ksub * (k.a_chunk_bytes + k.b_chunk_bytes);
    // Small column blocks leave most of a tile's time in fixed per-tile synchronisation; two co-resident CTAs per SM
    // (half the shared-memory budget each, 2 x TMEM columns <= 512) overlap one CTA's bubbles with the other's work.
    // Layers whose tiles carry little MMA work (short K) spend their time in the epilogue.  With a 256-column block
    // a single accumulator buffer (256 TMEM columns) lets two CTAs share an SM there, which doubles the epilogue warps
    // in flight; the lost MMA / epilogue overlap inside one CTA is made up by the neighbour CTA.
    const int mmas_per_tile = k.total_chunks * k.mmas_per_chunk;
    k.acc_bufs = diag_env_int("TB200_TC_ACC_BUFS", (block_n > 128 && mmas_per_tile <= 16) ? 1 : 2);
    if (k.acc_bufs != 1)
        k.acc_bufs = 2;
    const bool pair_small = block_n <= 128 && 4 * k.stage_bytes <= 100 * 1024;
    const bool pair_short = k.acc_bufs == 1 && 2 * k.stage_bytes <= 100 * 1024;
    plan->ctas_per_sm     = diag_env_int("TB200_TC_CTAS_PER_SM", (pair_small || pair_short) ? 2 : 1);
    plan->ctas_per_sm = std::max(1, std::min(plan->ctas_per_sm, 512 / std::max(32, k.acc_bufs * block_n)));
    const int smem_budget = (plan->ctas_per_sm > 1 ? 208 / plan->ctas_per_sm : 200) * 1024;
    k.num_stages = std::min(kMaxStages, smem_budget / k.stage_bytes);
    k.num_stages = std::min(k.num_stages, std::max(2, k.num_kstages * 2));
    const int forced = diag_env_int("TB200_TC_STAGES", 0);
    if (forced > 0)
        k.num_stages = std::min(forced, kMaxStages);
    if (k.num_stages < 2)
        return no("stage does not fit in shared memory");
    k.commit_group = diag_env_int("TB200_TC_COMMIT_GROUP", 1);
    if (k.commit_group < 1 || k.num_stages % k.commit_group != 0 || k.num_stages / k.commit_group < 2)
        k.commit_group = 1;
    plan->smem_bytes = k.num_stages * k.stage_bytes + 1024;

    const bool is_f8  = dtype_is_fp8(q.in_dtype);
    const bool is_f16 = q.in_dtype != TB200_INT8 && !is_f8;
    k.is_f16_kind     = is_f8 ? 2 : is_f16 ? 1 : 0;
    if (is_f8)
    {
        // kind::f8f6f4 operand formats: 0 = E4M3, 1 = E5M2, chosen per operand; fp32 accumulators
        const tb200_dtype bdt = q.b_fp8_dtype ? (tb200_dtype)q.b_fp8_dtype : q.in_dtype;
        k.idesc = ptx::make_idesc(1u, q.in_dtype == TB200_FP8E5M2 ? 1u : 0u, bdt == TB200_FP8E5M2 ? 1u : 0u, 0u,
                                  q.b_mn_major ? 1u : 0u, kTileM, (uint32_t)block_n);
    }
    else
    {
        const uint32_t ab_fmt = is_f16 ? (q.in_dtype == TB200_BF16 ? 1u : 0u) : (uint32_t)diag_env_int("TB200_TC_I8_FMT", 1);
        k.idesc = ptx::make_idesc(is_f16 ? 1u : 2u, ab_fmt, ab_fmt, 0u, q.b_mn_major ? 1u : 0u, kTileM, (uint32_t)block_n);
    }
    int cols = 32;
    while (cols < k.acc_bufs * block_n)
        cols *= 2;
    k.tmem_cols = cols;

    // tensor maps
    plan->dt    = (q.in_dtype == TB200_INT8 || is_f8) ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                  : q.in_dtype == TB200_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                             : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    plan->a_swz = swz == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : swz == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
    plan->a_dims[0] = (cuuint64_t)q.IC;
    plan->a_dims[1] = (cuuint64_t)IW;
    plan->a_dims[2] = (cuuint64_t)IH;
    plan->a_dims[3] = (cuuint64_t)N;
    if (pure_gemm)
    {
        plan->a_strides[0] = (cuuint64_t)q.IC * es;
        plan->a_strides[1] = plan->a_strides[0] * IW;
        plan->a_strides[2] = plan->a_strides[1] * IH;
    }
    else
    {
        plan->a_strides[0] = (cuuint64_t)sw * es;
        plan->a_strides[1] = (cuuint64_t)sh * es;
        plan->a_strides[2] = (cuuint64_t)sn * es;
    }
    plan->a_box[0]  = (cuuint32_t)k.chunk_elems;
    plan->a_box[1]  = (cuuint32_t)(BW * q.stride_x);
    plan->a_box[2]  = (cuuint32_t)(BH * q.stride_y);
    plan->a_box[3]  = (cuuint32_t)BN;
    plan->a_estr[0] = 1;
    plan->a_estr[1] = (cuuint32_t)q.stride_x;
    plan->a_estr[2] = (cuuint32_t)q.stride_y;
    plan->a_estr[3] = 1;
    if (!q.b_mn_major)
    {
        const cuuint64_t ktot = (cuuint64_t)q.KH * q.KW * q.IC;
        plan->b_swz        = plan->a_swz;
        plan->b_dims[0]    = ktot;
        plan->b_dims[1]    = (cuuint64_t)q.OC;
        plan->b_dims[2]    = 1;
        plan->b_strides[0] = ktot * es;
        plan->b_strides[1] = ktot * es * q.OC;
        plan->b_box[0]     = (cuuint32_t)k.chunk_elems;
        plan->b_box[1]     = (cuuint32_t)block_n;
        plan->b_box[2]     = 1;
    }
    else
    {
        plan->b_swz        = CU_TENSOR_MAP_SWIZZLE_128B;
        plan->b_dims[0]    = (cuuint64_t)q.OC;
        plan->b_dims[1]    = (cuuint64_t)q.IC;
        plan->b_dims[2]    = (cuuint64_t)q.OH;    // batches
        plan->b_strides[0] = (cuuint64_t)(q.b_ld ? q.b_ld : (int64_t)q.OC) * es;
        plan->b_strides[1] = plan->b_strides[0] * q.IC;
        plan->b_box[0]     = (cuuint32_t)k.b_box_n;
        plan->b_box[1]     = (cuuint32_t)k.chunk_elems;
        plan->b_box[2]     = 1;
    }
    for (int i = 0; i < 3; i++)
        if (plan->a_strides[i] % 16 != 0 || plan->a_strides[i] >= (1ULL << 40))
            return no("activation stride not usable by TMA");
    k.tile_begin = 0;
    k.tile_end   = k.num_tiles;
    if (q.tile_end > q.tile_begin)
    {
        k.tile_begin = std::max(0, q.tile_begin);
        k.tile_end   = std::min(k.num_tiles, q.tile_end);
    }
    plan->grid = std::max(1, std::min(k.tile_end - k.tile_begin, num_sms * plan->ctas_per_sm));
    return true;
}


void lean_fastdiv_set(TcKernelParams& k)
{
    fastdiv_make((uint32_t)(k.tiles_x * k.tiles_y * k.tiles_n), k.fd_m);
    fastdiv_make((uint32_t)k.tiles_x, k.fd_x);
    fastdiv_make((uint32_t)k.tiles_y, k.fd_y);
}

// Re-plans a problem make_plan has laid out for tc_conv_lean_kernel: one CTA per SM, the fewest stages per tile that
// fit (one when a tile's operands fit twice into shared memory), weights resident when there is a single column block.
bool make_lean_plan(const TcProblem& q, int num_sms, int max_smem_optin, TcPlan* plan)
{
    if (diag_env_int("TB200_TC_LEAN", 1) == 0)
        return false;
    if (q.epi != TC_EPI_RESCALE || !q.lean_ok || q.rec == nullptr || q.b_mn_major || q.in_dtype != TB200_INT8 ||
        q.out_dtype != TB200_INT8 || q.out_sy != 0 || q.tile_begin != 0 || q.tile_end != 0)
        return false;
    if ((q.OC % 32) != 0 || (reinterpret_cast<uintptr_t>(q.out) & 31) != 0)
        return false;
    if (q.clamp_lo < -128 || q.clamp_hi > 127 || q.clamp_lo > q.clamp_hi || q.out_zp < -128 || q.out_zp > 127)
        return false;
    if (q.corr_classes && q.delta == nullptr)
        return false;
    if (!make_plan(q, num_sms, plan, nullptr))
        return false;
    TcKernelParams& k = plan->kp;
    k.lean_xpar    = q.xpar;
    k.lean_ow_real = q.out_ow_real;
    const int budget     = (max_smem_optin > 0 ? max_smem_optin : 232448) - 1024 /* alignment */ - 2048 /* static + margin */;
    const int rec_bytes  = 4 * k.block_n * 32;
    const int b_tx       = k.block_n * k.chunk_elems;
    const int a_tx       = k.tx_bytes_per_chunk - b_tx;
    const int b_total    = k.total_chunks * k.b_chunk_bytes;
    k.lean_rec_stride    = k.block_n * 32;
    k.lean_halo          = 0;
    k.lean_halo_wp       = 0;

    // ---- halo mode: stride-1 window, one column block, weights resident (see tc_conv_lean_kernel).  Not for column
    // blocks of 64: those layers are bound by the issue rate of their N = 64 MMAs (about 170 cycles each with the commit),
    // which the halo form does not change, and measured 20 % slower with it (3x3 64 -> 64 at 56 x 56: 136 against 111 us at
    // batch 256; 3x3 128 -> 128 at 28 x 28: 57 against 74 us).
    {
        const int swz = k.chunk_elems;    // int8: bytes of one pixel row of a chunk
        const int wp  = q.OW + q.KW - 1;
        if (diag_env_int("TB200_LEAN_HALO", 1) != 0 && !q.xpar && q.KH * q.KW > 1 && q.stride_x == 1 && q.stride_y == 1 && q.dil_x == 1 &&
            q.dil_y == 1 && k.tiles_col == 1 && wp <= kTileM && wp <= 256 && k.block_n >= diag_env_int("TB200_LEAN_HALO_MIN_N", 128))
        {
            int bh = std::min(q.OH, kTileM / wp);
            for (int cand = bh; cand >= std::max(1, bh - 2); cand--)
                if (q.OH % cand == 0)
                {
                    bh = cand;
                    break;
                }
            const int hb        = bh + q.KH - 1;
            const int alloc_pos = std::max(wp * hb, kTileM + (q.KH - 1) * wp + q.KW - 1);
            const int a_chunk   = (alloc_pos * swz + 1023) & ~1023;
            const int stage     = k.chunks_per_tap * a_chunk;
            const int rec_one   = k.block_n * 32;
            int nacc            = k.block_n <= 128 ? 4 : 2;
            if (b_total + rec_one + nacc * stage > budget)
                nacc = 2;
            // at least three quarters of the accumulator rows must be output pixels, or the tensor pipe works on halo
            if (bh * wp >= 96 && hb <= 256 && b_total + rec_one + nacc * stage <= budget)
            {
                k.lean_halo     = 1;
                k.lean_halo_wp  = wp;
                k.BW            = q.OW;
                k.BH            = bh;
                k.BN            = 1;
                k.tiles_x       = 1;
                k.tiles_y       = (q.OH + bh - 1) / bh;
                k.tiles_n       = q.N;
                k.num_tiles     = k.tiles_y * k.tiles_n;
                k.tile_begin    = 0;
                k.tile_end      = k.num_tiles;
                k.a_chunk_bytes = a_chunk;
                plan->a_box[0]  = (cuuint32_t)k.chunk_elems;
                plan->a_box[1]  = (cuuint32_t)wp;
                plan->a_box[2]  = (cuuint32_t)hb;
                plan->a_box[3]  = 1;
                k.ksub                 = k.total_chunks;
                k.num_kstages          = 1;
                k.lean_stages_per_tile = 1;
                k.num_stages           = nacc;
                k.stage_bytes          = stage;
                k.tx_bytes_per_chunk   = wp * hb * swz;    // bytes of one box
                k.lean_b_resident      = 1;
                k.lean_b_off           = 0;
                k.lean_ring_off        = b_total;
                k.lean_rec_off         = b_total + nacc * stage;
                k.lean_rec_stride      = 0;
                k.acc_bufs             = nacc;
                int cols = 32;
                while (cols < nacc * k.block_n)
                    cols *= 2;
                k.tmem_cols       = cols;
                plan->smem_bytes  = k.lean_rec_off + rec_one + 1024;
                plan->ctas_per_sm = 1;
                plan->grid        = std::max(1, std::min(k.num_tiles, num_sms));
                plan->lean        = true;
                lean_fastdiv_set(k);
                return true;
            }
        }
    }
    const bool b_res     = k.tiles_col == 1 && b_total <= 96 * 1024;
    const int avail      = budget - rec_bytes - (b_res ? b_total : 0);
    const int per_chunk  = k.a_chunk_bytes + (b_res ? 0 : k.b_chunk_bytes);
    int ksub, spt, stages;
    if (2 * k.total_chunks * per_chunk <= avail)
    {
        ksub   = k.total_chunks;
        spt    = 1;
        stages = kLeanAccBufs;    // a slot per accumulator buffer: one commit releases both
        // (a deeper ring of such tiles with barriers of its own was measured: no faster, the loads are not what a
        // short-K layer waits for)
        // Column blocks of at most 128: four accumulator buffers fit tensor memory, one per epilogue group, so that all
        // four groups work (with two buffers and two 32-column chunks per tile, half of them wait); taken when four
        // one-tile stages fit as well.
        if (k.block_n <= 128 && kLeanMaxAccBufs * k.total_chunks * per_chunk <= avail &&
            diag_env_int("TB200_LEAN_ACC4", 1) != 0)
            stages = kLeanMaxAccBufs;
    }
    else
    {
        const int target = diag_env_int("TB200_LEAN_STAGE_KB", 48) * 1024;
        ksub = std::max(1, std::min(k.total_chunks, target / per_chunk));
        spt  = (k.total_chunks + ksub - 1) / ksub;
        if (spt < 2)
            spt = 2;
        ksub   = (k.total_chunks + spt - 1) / spt;
        spt    = (k.total_chunks + ksub - 1) / ksub;
        stages = std::min(kMaxStages, avail / (ksub * per_chunk));
        if (stages < 2 || spt < 2)
            return false;
    }
    k.ksub                 = ksub;
    k.num_kstages          = spt;
    k.lean_stages_per_tile = spt;
    k.num_stages           = stages;
    k.stage_bytes          = ksub * per_chunk;
    k.tx_bytes_per_chunk   = a_tx + (b_res ? 0 : b_tx);
    k.lean_b_resident      = b_res ? 1 : 0;
    k.lean_b_off           = 0;
    k.lean_ring_off        = b_res ? b_total : 0;
    k.lean_rec_off         = k.lean_ring_off + stages * k.stage_bytes;
    k.acc_bufs             = (spt == 1) ? stages : kLeanAccBufs;
    int cols = 32;
    while (cols < k.acc_bufs * k.block_n)
        cols *= 2;
    k.tmem_cols      = cols;
    plan->smem_bytes = k.lean_rec_off + rec_bytes + 1024;
    plan->ctas_per_sm = 1;
    plan->grid        = std::max(1, std::min(k.num_tiles, num_sms));
    plan->lean        = true;
    lean_fastdiv_set(k);
    return plan->smem_bytes <= budget + 1024;
}

}    // namespace

bool tc_gemm_supported(const TcProblem& p, std::string* why)
{
    TcPlan plan;
    return make_plan(p, 148, &plan, why);
}

bool tc_gemm_lean_supported(const tb200_ctx* ctx, const TcProblem& p)
{
    TcPlan plan;
    plan.lean = false;
    return !tc_gemm_pair_supported(p, ctx->num_sms) && make_lean_plan(p, ctx->num_sms, ctx->max_smem_optin, &plan);
}

bool tc_gemm_tile_counts(const TcProblem& p, int* num_tiles, int* tiles_per_row_block)
{
    TcPlan plan;
    if (!make_plan(p, 148, &plan, nullptr))
        return false;
    *num_tiles           = plan.kp.num_tiles;
    *tiles_per_row_block = plan.kp.tiles_x * plan.kp.tiles_col;
    return true;
}

tb200_status tc_gemm_launch(tb200_ctx* ctx, const TcProblem& q)
{
    if (tc_gemm_pair_supported(q, ctx->num_sms))
        return tc_gemm_pair_launch(ctx, q);
    TcPlan plan;
    plan.lean = false;
    std::string why;
    if (!make_lean_plan(q, ctx->num_sms, ctx->max_smem_optin, &plan))
    {
        plan.lean = false;
        if (q.xpar)
            return fail(ctx, TB200_INTERNAL, "a parity-split problem needs the lean convolution kernel");
        if (!make_plan(q, ctx->num_sms, &plan, &why))
            return fail(ctx, TB200_ERROR, "tensor-core path not applicable: %s", why.c_str());
    }
    PFN_encodeTiled enc = get_encode_fn();
    if (!enc)
        return fail(ctx, TB200_INTERNAL, "cuTensorMapEncodeTiled is not available from the driver");
    TcKernelParams& k = plan.kp;
    CUresult r = enc(&k.tmA, plan.dt, 4, const_cast<void*>(q.a), plan.a_dims, plan.a_strides, plan.a_box, plan.a_estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, plan.a_swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(ctx, TB200_INTERNAL, "tensor map for A rejected (CUresult %d)", (int)r);
    cuuint32_t b_estr[3] = { 1, 1, 1 };
    r = enc(&k.tmB, plan.dt, 3, const_cast<void*>(q.b), plan.b_dims, plan.b_strides, plan.b_box, b_estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, plan.b_swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(ctx, TB200_INTERNAL, "tensor map for B rejected (CUresult %d)", (int)r);

    k.out              = q.out;
    k.out_es           = (int)dtype_size(q.out_dtype);
    k.out_is_bf16      = q.out_dtype == TB200_BF16;
    k.row_corr     = q.row_corr;
    k.corr         = q.corr;
    k.corr_stride  = q.corr_stride;
    k.corr_ystride = q.corr_ystride;
    k.corr_classes = q.corr_classes;
    k.bias_f_pad   = q.bias_f_pad;
    k.mult_pad     = q.mult_pad;
    k.shift_pad    = q.shift_pad;
    k.rec          = q.rec;
    k.delta        = q.delta;
    k.cls_interior = ((0 * (q.KH + 1) + q.KH) * (q.KW + 1) + 0) * (q.KW + 1) + q.KW;
    k.double_round = q.double_round;
    k.out_zp       = q.out_zp;
    k.clamp_lo     = q.clamp_lo;
    k.clamp_hi     = q.clamp_hi;
    k.clamp_lo_f   = q.clamp_lo_f;
    k.clamp_hi_f   = q.clamp_hi_f;
    k.has_clamp    = q.has_clamp;
    k.status       = ctx->d_status;
    k.debug        = diag_env_int("TB200_TC_DEBUG", 0);
#ifdef TB200_DIAG
    {
        // TB200_TC_TRACE=<device address>: room for 16 stamps per CTA (a tool allocates and reads it)
        const char* tr = getenv("TB200_TC_TRACE");
        k.trace        = tr ? reinterpret_cast<long long*>(strtoull(tr, nullptr, 0)) : nullptr;
    }
#endif
    k.wait_limit   = ctx->wait_limit_cycles;

    if (plan.lean)
    {
        void (*lean)(const TcKernelParams) =
            k.corr_classes ? (k.double_round ? tc_conv_lean_kernel<true, true> : tc_conv_lean_kernel<true, false>)
                           : (k.double_round ? tc_conv_lean_kernel<false, true> : tc_conv_lean_kernel<false, false>);
        const tb200_status ast = raise_smem_limit(ctx, 4 + (k.corr_classes ? 1 : 0) + (k.double_round ? 2 : 0), reinterpret_cast<const void*>(lean),
                                                  plan.smem_bytes);
        if (ast != TB200_OK)
            return ast;
        timer_begin(ctx);
        {
            // programmatic stream serialization: the kernel may be scheduled while its predecessor drains; it waits
            // (griddepcontrol.wait) before it touches anything the predecessor may write or still read
            cudaLaunchConfig_t cfg;
            memset(&cfg, 0, sizeof(cfg));
            cfg.gridDim          = dim3((unsigned)plan.grid);
            cfg.blockDim         = dim3((unsigned)kLeanThreads);
            cfg.dynamicSmemBytes = (size_t)plan.smem_bytes;
            cfg.stream           = ctx->stream;
            cudaLaunchAttribute at[1];
            at[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
            at[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs    = at;
            cfg.numAttrs = ctx->launch_overlap ? 1 : 0;
            cudaLaunchKernelEx(&cfg, lean, k);
        }
        timer_end(ctx);
        const tb200_status lst = post_launch(ctx, "tc_conv_lean_i8");
        if (lst != TB200_OK)
        {
            // say what the launch asked for: the usual cause is a build whose register or shared-memory use grew
            cudaFuncAttributes fa;
            if (cudaFuncGetAttributes(&fa, reinterpret_cast<const void*>(lean)) == cudaSuccess)
                ctx->err += " (" + std::to_string(kLeanThreads) + " threads x " + std::to_string(fa.numRegs) + " registers, " +
                            std::to_string(plan.smem_bytes) + " + " + std::to_string((int)fa.sharedSizeBytes) +
                            " bytes of shared memory, limit " + std::to_string(fa.maxDynamicSharedSizeBytes) + ")";
        }
        return lst;
    }
    void (*kern)(const TcKernelParams) = nullptr;
    const char* name                   = "";
    switch (q.epi)
    {
        case TC_EPI_I32:
            kern = tc_gemm_kernel<TC_EPI_I32>;
            name = "tc_gemm_i8_i32";
            break;
        case TC_EPI_RESCALE:
            kern = tc_gemm_kernel<TC_EPI_RESCALE>;
            name = "tc_gemm_i8_rescale";
            break;
        default:
            kern = tc_gemm_kernel<TC_EPI_FLOAT>;
            name = dtype_is_fp8(q.in_dtype) ? "tc_gemm_f8" : "tc_gemm_f16";
            break;
    }
    {
        const tb200_status ast = raise_smem_limit(ctx, q.epi, reinterpret_cast<const void*>(kern), plan.smem_bytes);
        if (ast != TB200_OK)
            return ast;
    }
    timer_begin(ctx);
    kern<<<plan.grid, kNumThreads, plan.smem_bytes, ctx->stream>>>(k);
    timer_end(ctx);
    return post_launch(ctx, name);
}

}    // namespace tb200
