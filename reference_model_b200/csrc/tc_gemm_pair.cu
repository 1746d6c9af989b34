// int8 MATMUL on CTA pairs (tcgen05 cta_group::2) for sm_100a.
//
// OpMatMul with int8 operands and int32 output (reference_model/src/ops/tensor_ops.cpp:1423-1492), for shapes large
// enough to fill 256 x 256 output tiles.  The kernel is launched as clusters of two CTAs on neighbouring SMs; a pair
// owns one 256 x 256 tile at a time:
//   * each CTA loads its own 128 rows of A and its own 128 columns of B per 128-byte K chunk (TMA, no multi-destination
//     copies); the tensor cores of both SMs read B from both shared memories, so a pair moves 2/3 of the bytes two
//     independent 128 x 256 tiles would, which is what bounds the single-CTA kernel at this size (L2 -> SM traffic)
//   * one thread of the pair's first CTA issues tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 32 bytes); measured
//     at 128 SM cycles per instruction (8192 MAC per cycle and SM) against 171 for the single-CTA form
//   * accumulators live in both CTAs' TMEM (128 rows x 256 columns each, two buffers); each CTA's eight epilogue warps
//     add the zero-point terms and store their own rows
// Tiles are handed out in rounds of one tile per pair; the pair that takes position k of a round moves to position k+1
// in the next one (all roles compute the same walk).  With a fixed assignment and an even number of pairs the same
// pairs would get every tile that carries zero-point sums; the rotation spreads that extra work evenly.
// Completion signals cross the pair: TMA byte counts of both CTAs land on the first CTA's "full" barrier,
// tcgen05.commit arrives on the "empty" / "accumulator ready" barriers of both, and every epilogue warp arrives on the
// first CTA's "accumulator free" barrier.  Every wait is bounded; a wait that gives up sets TB200_DEV_TIMEOUT and all
// roles drain to the common exit.
#include <algorithm>
#include <cuda.h>
#include <cstring>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <mutex>

#include "common.h"
#include "ptx_sm100.cuh"

namespace tb200
{

namespace
{

constexpr int kPairEpiWarps   = 8;        // two per TMEM lane quarter, each taking every second 32-column chunk
constexpr int kPairSumWarps   = 4;        // row sums of A straight from the shared-memory ring (b_zp term of MATMUL)
constexpr int kPairThreads    = 64 + 32 * (kPairEpiWarps + kPairSumWarps);    // TMA warp, MMA warp, epilogue, sums
constexpr int kPairMaxStages  = 8;
constexpr int kPairChunkBytes = 16384;    // 128 rows x 128 bytes (A: rows x K, B: K rows x columns), 128-byte swizzle
constexpr int kPairTmemCols   = 512;      // two accumulator buffers of 256 columns

struct PairParams
{
    CUtensorMap tmA;    // (C, H, batch), box 128 x 128 x 1
    CUtensorMap tmB;    // (W, C, batch), box 128 x 128 x 1
    int NB, H, C, W;
    int tiles_m, tiles_w, num_tiles;    // 256 x 256 tiles, numbered batch-major, columns fastest
    int total_chunks;                   // 128-byte K chunks
    int ksub, num_stages, stage_bytes;  // K chunks per stage (one tcgen05.commit per stage), ring depth
    uint64_t a_desc_hi, b_desc_hi;
    uint32_t idesc;
    int32_t* out;
    int out_kind;               // 0: int8 operands, int32 output with the corrections below; floating operands (fp32
                                // accumulators, no corrections): 1 = fp32 output, 2 = fp16 output, 3 = bf16 output
    int mma_kind;               // 0: kind::i8, 1: kind::f8f6f4, 2: kind::f16 (fp16 / bf16 operands)
    // Geometry of a 128-byte K chunk.  8-bit operands: 128 K elements, each CTA's half of B is one box of 128 columns.
    // 16-bit operands: 64 K elements, the half is two boxes of 64 columns (one 128-byte swizzle atom each).
    int chunk_elems, b_boxes, b_box_cols, b_box_bytes;
    uint32_t b_kstep16;         // descriptor advance per MMA: its K rows x 128 bytes, in 16-byte units
    const int32_t* row_corr;    // [batch * H] or null
    // Zero-point sums inside the kernel (sum warps read the tiles as they pass through shared memory):
    //   1: every tile sums the rows of its own A tile and hands them to its epilogue through shared memory; the term
    //      of an output row is -b_zp * sum_k A[row, k] + C * a_zp * b_zp (row_corr is then null, corr as usual)
    //   2: sums are shared between tiles through global memory.  The tile in column-tile 0 of a row of tiles sums the
    //      rows of A (into row_corr, raw sums), the tile in row-tile 0 of a column of tiles sums the columns of B (into
    //      corr, raw sums), each publishes an epoch number in `flags` when its 128 rows / columns are written, and
    //      every epilogue waits for the flags of its rows and columns.  Producers always have smaller tile numbers than
    //      their consumers and every pair walks its tiles in increasing order, so the waits cannot form a cycle.
    int fuse_row_sums;
    int32_t a_zp, b_zp;
    uint32_t* flags;    // mode 2: [batch * tiles_m * 2] row flags, then [batch * tiles_w * 2] column flags
    uint32_t epoch;     // mode 2: value a flag takes in this launch
    const int32_t* corr;        // [batch][corr_stride] or null; corr_stride a multiple of 256 that covers W
    int corr_stride;
    int debug;                  // diagnostic bit mask, read only by builds with TB200_DIAG: 1 skip epilogue memory work, 2 skip MMA issue, 4 skip loads
    long long wait_limit;       // SM cycles after which a pipeline or flag wait gives up (TB200_DEV_TIMEOUT)
    int* status;
};

struct PairTile
{
    int n, m0, w0;
};

__device__ __forceinline__ PairTile decode_pair_tile(const PairParams& p, int tile)
{
    PairTile t;
    t.w0  = (tile % p.tiles_w) * 256;
    int r = tile / p.tiles_w;
    t.m0  = (r % p.tiles_m) * 256;
    t.n   = r / p.tiles_m;
    return t;
}

// KIND selects the operand type at compile time, so that each instantiation carries only its own MMA, tile geometry
// and epilogue: 0 = int8 (kind::i8, int32 output with zero-point corrections), 1 = fp8 (kind::f8f6f4), 2 = fp16 / bf16
// (kind::f16); the floating kinds store fp32 accumulators as fp32, fp16 or bf16 (p.out_kind).
template <int KIND>
__global__ void __launch_bounds__(kPairThreads, 1) tc_gemm_pair_kernel(const __grid_constant__ PairParams p)
{
    extern __shared__ uint8_t smem_raw[];
    // identical layout in both CTAs of a pair: remote signals address a barrier by its offset
    __shared__ __align__(8) uint64_t bar_full[kPairMaxStages];     // used in the first CTA: bytes of both CTAs
    __shared__ __align__(8) uint64_t bar_empty[kPairMaxStages];    // per CTA: stage consumed by the MMAs
    __shared__ __align__(8) uint64_t bar_tmem_full[2];          // per CTA: accumulator buffer complete
    __shared__ __align__(8) uint64_t bar_tmem_empty[2];         // first CTA: buffer drained by both CTAs' epilogues
    __shared__ __align__(8) uint64_t bar_go[kPairMaxStages];    // second CTA: "stage full" relayed by the first CTA
    __shared__ __align__(8) uint64_t bar_rs_full[2];            // per CTA: row sums of an accumulator buffer's tile ready
    __shared__ __align__(8) uint64_t bar_rs_empty[2];           // per CTA: epilogue has read them
    __shared__ int32_t row_sums[2][128];
    __shared__ int32_t col_red[16][128];    // mode 2: partial column sums of the 16 row groups of a B tile
    __shared__ uint32_t tmem_base_holder;

    const int warp          = threadIdx.x >> 5;
    const int lane          = threadIdx.x & 31;
    const uint32_t rank     = ptx::cluster_ctarank();
    const int cluster_id    = blockIdx.x >> 1;
    const int num_clusters  = gridDim.x >> 1;
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < p.num_stages; s++)
        {
            ptx::mbar_init(ptx::smem_u32(&bar_full[s]), 1);
            // a stage is free when the MMAs have read it and, with fused row sums, the sum warps have too
            ptx::mbar_init(ptx::smem_u32(&bar_empty[s]), 1 + (p.fuse_row_sums ? kPairSumWarps : 0));
            ptx::mbar_init(ptx::smem_u32(&bar_go[s]), 1);
        }
        for (int a = 0; a < 2; a++)
        {
            ptx::mbar_init(ptx::smem_u32(&bar_tmem_full[a]), 1);
            ptx::mbar_init(ptx::smem_u32(&bar_tmem_empty[a]), 2 * kPairEpiWarps);
            ptx::mbar_init(ptx::smem_u32(&bar_rs_full[a]), kPairSumWarps);
            ptx::mbar_init(ptx::smem_u32(&bar_rs_empty[a]), kPairEpiWarps);
        }
        ptx::fence_barrier_init();
        ptx::prefetch_tmap(&p.tmA);
        ptx::prefetch_tmap(&p.tmB);
    }
    if (warp == 1)
    {
        ptx::tmem_alloc_pair(ptx::smem_u32(&tmem_base_holder), kPairTmemCols);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    // no signal may reach the other CTA before its barriers exist
    ptx::cluster_sync();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_holder;

    if (warp == 0)
    {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0)
        {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int round = 0, base = 0; base < p.num_tiles && ok; round++, base += num_clusters)
            {
                const int tile = base + (cluster_id + round) % num_clusters;
                if (tile >= p.num_tiles)
                    continue;
                const PairTile t = decode_pair_tile(p, tile);
                const int m0 = t.m0 + (int)rank * 128;
                const int w0 = t.w0 + (int)rank * 128;
                int chunks_left = p.total_chunks;
                int k = 0;
                while (chunks_left > 0)
                {
                    if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bar_empty[stage]), phase ^ 1u, p.wait_limit))
                    {
                        ok = false;
                        break;
                    }
                    const int nch = min(p.ksub, chunks_left);
                    chunks_left -= nch;
                    const uint32_t full_local = ptx::smem_u32(&bar_full[stage]);
                    if (TB200_DIAG_BIT(p.debug, 4))
                    {
                        if (rank == 0)
                            ptx::mbar_arrive(full_local);
                    }
                    else
                    {
                        // the first CTA arms the barrier with the bytes of both CTAs; each CTA's copies report there
                        if (rank == 0)
                            ptx::mbar_arrive_expect_tx(full_local, (uint32_t)(nch * 4 * kPairChunkBytes));
                        const uint32_t full_first = ptx::map_to_cta(full_local, 0);
                        const uint32_t sA = smem_base + (uint32_t)(stage * p.stage_bytes);
                        const uint32_t sB = sA + (uint32_t)(p.ksub * kPairChunkBytes);
                        for (int j = 0; j < nch; j++)
                        {
                            ptx::tma_load_3d_pair(sA + (uint32_t)(j * kPairChunkBytes), &p.tmA, full_first, k, m0, t.n);
                            if (KIND == 2)
                            {
                                // halves: the CTA's 128 columns are two 64-column swizzle atoms of 64 K rows each
                                ptx::tma_load_3d_pair(sB + (uint32_t)(j * kPairChunkBytes), &p.tmB, full_first, w0, k, t.n);
                                ptx::tma_load_3d_pair(sB + (uint32_t)(j * kPairChunkBytes + 8192), &p.tmB, full_first, w0 + 64, k,
                                                      t.n);
                                k += 64;
                            }
                            else
                            {
                                ptx::tma_load_3d_pair(sB + (uint32_t)(j * kPairChunkBytes), &p.tmB, full_first, w0, k, t.n);
                                k += 128;
                            }
                        }
                    }
                    if (++stage == p.num_stages)
                    {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok)
                atomicOr(p.status, TB200_DEV_TIMEOUT);
        }
    }
    else if (warp == 1)
    {
        // ------------------------------------------------------------------ MMA issuer (first CTA of the pair)
        if (lane == 0 && rank == 0)
        {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            const bool issue = !TB200_DIAG_BIT(p.debug, 2);
            for (int round = 0, base = 0; base < p.num_tiles && ok; round++, base += num_clusters)
            {
                const int tile = base + (cluster_id + round) % num_clusters;
                if (tile >= p.num_tiles)
                    continue;
                if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bar_tmem_empty[acc]), acc_phase ^ 1u, p.wait_limit))
                {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * 256);
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
                    // The second CTA's sum warps cannot watch this barrier: tell them their A tile has landed.  (A
                    // relaxed arrival: the tile was written by the TMA unit, whose completion this thread has just
                    // observed; a release at cluster scope here was measured at about a microsecond per stage.)
                    if (p.fuse_row_sums)
                        ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&bar_go[stage]), 1));
                    const int nch = min(p.ksub, chunks_left);
                    chunks_left -= nch;
                    if (issue)
                    {
                        const uint32_t sA = smem_base + (uint32_t)(stage * p.stage_bytes);
                        const uint32_t sB = sA + (uint32_t)(p.ksub * kPairChunkBytes);
                        for (int j = 0; j < nch; j++)
                        {
                            uint64_t ad = ptx::smem_desc(p.a_desc_hi, sA + (uint32_t)(j * kPairChunkBytes));
                            uint64_t bd = ptx::smem_desc(p.b_desc_hi, sB + (uint32_t)(j * kPairChunkBytes));
#pragma unroll
                            for (int m = 0; m < 4; m++)
                            {
                                if (KIND == 2)
                                    ptx::mma_f16_ss_pair(d_tmem, ad, bd, p.idesc, accum);
                                else if (KIND == 1)
                                    ptx::mma_f8_ss_pair(d_tmem, ad, bd, p.idesc, accum);
                                else
                                    ptx::mma_i8_ss_pair(d_tmem, ad, bd, p.idesc, accum);
                                accum = 1;
                                ad += 2;                         // 32 bytes of K inside the swizzled row
                                bd += (KIND == 2) ? 128 : 256;    // the MMA's K rows of 128 bytes: 16 rows of halves, 32 of bytes
                            }
                        }
                    }
                    // frees the stage in both CTAs once the MMAs above have read it
                    ptx::mma_commit_pair(ptx::smem_u32(&bar_empty[stage]), 3);
                    if (++stage == p.num_stages)
                    {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok)
                    break;
                ptx::mma_commit_pair(ptx::smem_u32(&bar_tmem_full[acc]), 3);
                acc ^= 1;
                if (acc == 0)
                    acc_phase ^= 1u;
            }
            if (!ok)
                atomicOr(p.status, TB200_DEV_TIMEOUT);
        }
    }
    else if (warp >= 2 + kPairEpiWarps)
    {
        // ------------------------------------------------------------------ row-sum warps (both CTAs)
        // 128 threads, eight per row of the A tile (one 16-byte piece each; the 128-byte swizzle only permutes pieces
        // inside a row), sixteen rows per pass.  A thread keeps the sums of its eight rows over the whole K loop.
        if (p.fuse_row_sums == 2)
        {
            // 128 threads.  A tile: eight threads per row (one 16-byte piece each), 16 rows per pass.  B tile (128 K rows
            // of 128 column bytes, pieces XOR-swizzled by the row number): thread (piece, group) reads logical piece
            // `piece` of the eight rows of its group and keeps sixteen column sums.
            const int ts    = (int)threadIdx.x - 32 * (2 + kPairEpiWarps);
            const int piece = ts & 7, grp = ts >> 3;
            uint32_t* flags_col = p.flags + (size_t)p.NB * p.tiles_m * 2;
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int round = 0, base = 0; base < p.num_tiles; round++, base += num_clusters)
            {
                const int tile = base + (cluster_id + round) % num_clusters;
                if (tile >= p.num_tiles)
                    continue;
                const PairTile t   = decode_pair_tile(p, tile);
                const bool do_rows = p.row_corr != nullptr && t.w0 == 0;
                const bool do_cols = p.corr != nullptr && t.m0 == 0;
                int32_t s[8], cs[16];
#pragma unroll
                for (int i = 0; i < 8; i++)
                    s[i] = 0;
#pragma unroll
                for (int i = 0; i < 16; i++)
                    cs[i] = 0;
                int chunks_left = p.total_chunks;
                while (chunks_left > 0 && ok)
                {
                    const uint32_t ready = ptx::smem_u32(rank == 0 ? &bar_full[stage] : &bar_go[stage]);
                    if (!ptx::mbar_wait_bounded(ready, phase, p.wait_limit))
                    {
                        ok = false;
                        break;
                    }
                    const int nch = min(p.ksub, chunks_left);
                    chunks_left -= nch;
                    const uint8_t* sA = smem_raw + (smem_base - ptx::smem_u32(smem_raw)) + stage * p.stage_bytes;
                    const uint8_t* sB = sA + p.ksub * kPairChunkBytes;
                    if (do_rows)
                    {
                        for (int j = 0; j < nch; j++)
                        {
                            const uint8_t* base = sA + j * kPairChunkBytes + grp * 128 + piece * 16;
#pragma unroll
                            for (int i = 0; i < 8; i++)
                            {
                                const int4 v = *reinterpret_cast<const int4*>(base + i * 16 * 128);
                                s[i] = __dp4a(v.x, 0x01010101, s[i]);
                                s[i] = __dp4a(v.y, 0x01010101, s[i]);
                                s[i] = __dp4a(v.z, 0x01010101, s[i]);
                                s[i] = __dp4a(v.w, 0x01010101, s[i]);
                            }
                        }
                    }
                    if (do_cols)
                    {
                        for (int j = 0; j < nch; j++)
                        {
                            const uint8_t* base = sB + j * kPairChunkBytes + grp * 8 * 128;
#pragma unroll
                            for (int i = 0; i < 8; i++)
                            {
                                const int4 v    = *reinterpret_cast<const int4*>(base + i * 128 + ((piece ^ i) << 4));
                                const int w4[4] = { v.x, v.y, v.z, v.w };
#pragma unroll
                                for (int q = 0; q < 4; q++)
                                {
                                    cs[4 * q + 0] = __dp4a(w4[q], 0x00000001, cs[4 * q + 0]);
                                    cs[4 * q + 1] = __dp4a(w4[q], 0x00000100, cs[4 * q + 1]);
                                    cs[4 * q + 2] = __dp4a(w4[q], 0x00010000, cs[4 * q + 2]);
                                    cs[4 * q + 3] = __dp4a(w4[q], 0x01000000, cs[4 * q + 3]);
                                }
                            }
                        }
                    }
                    // this warp is done with the stage
                    __syncwarp();
                    if (lane == 0)
                        ptx::mbar_arrive(ptx::smem_u32(&bar_empty[stage]));
                    if (++stage == p.num_stages)
                    {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                // The four sum warps leave the loop together: a warp whose wait gave up must not leave the others at the
                // named barriers below.
                ok = ptx::named_barrier_and(2, 32 * kPairSumWarps, ok);
                if (!ok)
                    break;
                if (do_rows)
                {
                    const int m_base = t.m0 + (int)rank * 128;
#pragma unroll
                    for (int i = 0; i < 8; i++)
                    {
                        s[i] += __shfl_xor_sync(0xffffffffu, s[i], 1);
                        s[i] += __shfl_xor_sync(0xffffffffu, s[i], 2);
                        s[i] += __shfl_xor_sync(0xffffffffu, s[i], 4);
                        const int m = m_base + grp + 16 * i;
                        if (piece == 0 && m < p.H)
                            const_cast<int32_t*>(p.row_corr)[(int64_t)t.n * p.H + m] = s[i];
                    }
                }
                if (do_cols)
                {
#pragma unroll
                    for (int i = 0; i < 16; i++)
                        col_red[grp][piece * 16 + i] = cs[i];
                    asm volatile("bar.sync 2, 128;" ::: "memory");
                    int32_t tsum = 0;
#pragma unroll
                    for (int g = 0; g < 16; g++)
                        tsum += col_red[g][ts];
                    const_cast<int32_t*>(p.corr)[(int64_t)t.n * p.corr_stride + t.w0 + (int)rank * 128 + ts] = tsum;
                }
                if (do_rows || do_cols)
                {
                    // publish: every writer fences its own stores, then one thread raises the flags
                    __threadfence();
                    asm volatile("bar.sync 2, 128;" ::: "memory");
                    if (ts == 0)
                    {
                        if (do_rows)
                            ptx::st_release_gpu(p.flags + ((size_t)t.n * p.tiles_m + t.m0 / 256) * 2 + rank, p.epoch);
                        if (do_cols)
                            ptx::st_release_gpu(flags_col + ((size_t)t.n * p.tiles_w + t.w0 / 256) * 2 + rank, p.epoch);
                    }
                }
            }
            if (!ok && lane == 0)
                atomicOr(p.status, TB200_DEV_TIMEOUT);
        }
        else if (p.fuse_row_sums)
        {
            const int ts    = (int)threadIdx.x - 32 * (2 + kPairEpiWarps);
            const int piece = ts & 7, row0 = ts >> 3;
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int round = 0, base = 0; base < p.num_tiles && ok; round++, base += num_clusters)
            {
                const int tile = base + (cluster_id + round) % num_clusters;
                if (tile >= p.num_tiles)
                    continue;
                ok = ptx::mbar_wait_bounded(ptx::smem_u32(&bar_rs_empty[acc]), acc_phase ^ 1u, p.wait_limit);
                int32_t s[8];
#pragma unroll
                for (int i = 0; i < 8; i++)
                    s[i] = 0;
                int chunks_left = p.total_chunks;
                while (chunks_left > 0 && ok)
                {
                    const uint32_t ready = ptx::smem_u32(rank == 0 ? &bar_full[stage] : &bar_go[stage]);
                    if (!ptx::mbar_wait_bounded(ready, phase, p.wait_limit))
                    {
                        ok = false;
                        break;
                    }
                    const int nch = min(p.ksub, chunks_left);
                    chunks_left -= nch;
                    const uint8_t* sA = smem_raw + (smem_base - ptx::smem_u32(smem_raw)) + stage * p.stage_bytes;
                    for (int j = 0; j < nch; j++)
                    {
                        const uint8_t* base = sA + j * kPairChunkBytes + row0 * 128 + piece * 16;
#pragma unroll
                        for (int i = 0; i < 8; i++)
                        {
                            const int4 v = *reinterpret_cast<const int4*>(base + i * 16 * 128);
                            s[i] = __dp4a(v.x, 0x01010101, s[i]);
                            s[i] = __dp4a(v.y, 0x01010101, s[i]);
                            s[i] = __dp4a(v.z, 0x01010101, s[i]);
                            s[i] = __dp4a(v.w, 0x01010101, s[i]);
                        }
                    }
                    // this warp is done with the stage
                    __syncwarp();
                    if (lane == 0)
                        ptx::mbar_arrive(ptx::smem_u32(&bar_empty[stage]));
                    if (++stage == p.num_stages)
                    {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok)
                    break;
#pragma unroll
                for (int i = 0; i < 8; i++)
                {
                    s[i] += __shfl_xor_sync(0xffffffffu, s[i], 1);
                    s[i] += __shfl_xor_sync(0xffffffffu, s[i], 2);
                    s[i] += __shfl_xor_sync(0xffffffffu, s[i], 4);
                    if (piece == 0)
                        row_sums[acc][row0 + 16 * i] = s[i];
                }
                __syncwarp();
                if (lane == 0)
                    ptx::mbar_arrive(ptx::smem_u32(&bar_rs_full[acc]));
                acc ^= 1;
                if (acc == 0)
                    acc_phase ^= 1u;
            }
            if (!ok && lane == 0)
                atomicOr(p.status, TB200_DEV_TIMEOUT);
        }
    }
    else
    {
        // ------------------------------------------------------------------ epilogue warps (both CTAs)
        const int quarter = warp & 3;           // TMEM lane quarter this warp may read
        const int slot    = (warp - 2) >> 2;    // the warps of a quarter take the 32-column chunks round robin
        const int32_t rc_const = p.fuse_row_sums ? p.C * p.a_zp * p.b_zp : 0;
        const int row     = quarter * 32 + lane;
        const uint32_t empty_first[2] = { ptx::map_to_cta(ptx::smem_u32(&bar_tmem_empty[0]), 0),
                                          ptx::map_to_cta(ptx::smem_u32(&bar_tmem_empty[1]), 0) };
        const bool wide_ok = (reinterpret_cast<uintptr_t>(p.out) & 31) == 0 && !TB200_DIAG_BIT(p.debug, 8);
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int round = 0, base = 0; base < p.num_tiles; round++, base += num_clusters)
        {
            const int tile = base + (cluster_id + round) % num_clusters;
            if (tile >= p.num_tiles)
                continue;
            const PairTile t = decode_pair_tile(p, tile);
            ok = ptx::mbar_wait_bounded(ptx::smem_u32(&bar_tmem_full[acc]), acc_phase, p.wait_limit);
            // the whole warp must agree before the warp-collective TMEM loads
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            ptx::tc_fence_after_sync();

            const int m          = t.m0 + (int)rank * 128 + row;
            const bool row_valid = m < p.H;
            const int64_t orow   = (int64_t)t.n * p.H + m;
            int32_t rc = 0;
            if (p.row_corr != nullptr && row_valid && p.fuse_row_sums != 2)
                rc = __ldg(p.row_corr + orow);
            int32_t col_scale = 1;    // mode 2 keeps raw column sums: corr = -a_zp * sum
            if (p.fuse_row_sums == 2)
            {
                // wait for the tiles that publish this tile's row sums (own half) and column sums (both halves)
                if (lane == 0)
                {
                    const uint32_t* fcol = p.flags + (size_t)p.NB * p.tiles_m * 2 + ((size_t)t.n * p.tiles_w + t.w0 / 256) * 2;
                    const uint32_t* frow = p.flags + ((size_t)t.n * p.tiles_m + t.m0 / 256) * 2 + rank;
                    const long long t0 = clock64();
                    while ((p.row_corr != nullptr && ptx::ld_acquire_gpu(frow) != p.epoch) ||
                           (p.corr != nullptr && (ptx::ld_acquire_gpu(fcol) != p.epoch || ptx::ld_acquire_gpu(fcol + 1) != p.epoch)))
                    {
                        if (clock64() - t0 > p.wait_limit)
                        {
                            ok = false;
                            break;
                        }
                    }
                }
                ok = __all_sync(0xffffffffu, ok);
                if (!ok)
                    break;
                rc = p.C * p.a_zp * p.b_zp;
                if (p.row_corr != nullptr && row_valid)
                    rc -= p.b_zp * __ldcg(p.row_corr + orow);
                col_scale = -p.a_zp;
            }
            else if (p.fuse_row_sums)
            {
                ok = ptx::mbar_wait_bounded(ptx::smem_u32(&bar_rs_full[acc]), acc_phase, p.wait_limit);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok)
                    break;
                rc = rc_const - p.b_zp * row_sums[acc][row];
                // every lane has its value: the sum warps may reuse the buffer
                __syncwarp();
                if (lane == 0)
                    ptx::mbar_arrive(ptx::smem_u32(&bar_rs_empty[acc]));
            }
            const int32_t* corr_row = p.corr != nullptr ? p.corr + (int64_t)t.n * p.corr_stride : nullptr;
            int32_t* out_row        = p.out + orow * p.W;
            const uint32_t taddr_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * 256);
            for (int c = slot; c < 8; c += kPairEpiWarps / 4)
            {
                uint32_t v[32];
                ptx::tmem_ld_32x32b_x32(taddr_row + (uint32_t)(c * 32), v);
                ptx::tmem_ld_wait();
                const int col = t.w0 + c * 32;
                if (col >= p.W || TB200_DIAG_BIT(p.debug, 1))
                    continue;
                if (KIND != 0)
                {
                    // fp32 accumulators of floating operands: stored as they are, or rounded once to fp16 / bf16
                    if (!row_valid)
                        continue;
                    const int nvalid = min(32, p.W - col);
                    if (p.out_kind == 1)
                    {
                        uint32_t* o = reinterpret_cast<uint32_t*>(p.out) + orow * p.W + col;
                        if (nvalid == 32 && (p.W & 7) == 0 && wide_ok)
                        {
#pragma unroll
                            for (int i = 0; i < 32; i += 8)
                                ptx::st_global_v8(o + i, v[i], v[i + 1], v[i + 2], v[i + 3], v[i + 4], v[i + 5], v[i + 6], v[i + 7]);
                        }
                        else
                        {
#pragma unroll
                            for (int i = 0; i < 32; i++)
                                if (i < nvalid)
                                    o[i] = v[i];
                        }
                    }
                    else
                    {
                        uint32_t h[16];
                        if (p.out_kind == 2)
                        {
#pragma unroll
                            for (int i = 0; i < 16; i++)
                            {
                                const __half2 pr = __floats2half2_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                                h[i]             = *reinterpret_cast<const uint32_t*>(&pr);
                            }
                        }
                        else
                        {
#pragma unroll
                            for (int i = 0; i < 16; i++)
                            {
                                const __nv_bfloat162 pr =
                                    __floats2bfloat162_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                                h[i] = *reinterpret_cast<const uint32_t*>(&pr);
                            }
                        }
                        uint16_t* o = reinterpret_cast<uint16_t*>(p.out) + orow * p.W + col;
                        if (nvalid == 32 && (p.W & 15) == 0 && wide_ok)
                        {
                            ptx::st_global_v8(o, h[0], h[1], h[2], h[3], h[4], h[5], h[6], h[7]);
                            ptx::st_global_v8(o + 16, h[8], h[9], h[10], h[11], h[12], h[13], h[14], h[15]);
                        }
                        else if (nvalid == 32 && (p.W & 7) == 0)
                        {
#pragma unroll
                            for (int i = 0; i < 16; i += 4)
                                *reinterpret_cast<uint4*>(o + 2 * i) = make_uint4(h[i], h[i + 1], h[i + 2], h[i + 3]);
                        }
                        else
                        {
#pragma unroll
                            for (int i = 0; i < 32; i++)
                                if (i < nvalid)
                                    o[i] = (uint16_t)((i & 1) ? (h[i >> 1] >> 16) : (h[i >> 1] & 0xffffu));
                        }
                    }
                    continue;
                }
                if (corr_row != nullptr)
                {
                    // the table is padded to a multiple of 256 columns: unconditional 128-bit loads
                    const int4* cp = reinterpret_cast<const int4*>(corr_row + col);
#pragma unroll
                    for (int q = 0; q < 8; q++)
                    {
                        // (L2 loads: in mode 2 the table was written by other SMs during this launch)
                        const int4 cv = __ldcg(cp + q);
                        v[4 * q + 0] += (uint32_t)(cv.x * col_scale) + (uint32_t)rc;
                        v[4 * q + 1] += (uint32_t)(cv.y * col_scale) + (uint32_t)rc;
                        v[4 * q + 2] += (uint32_t)(cv.z * col_scale) + (uint32_t)rc;
                        v[4 * q + 3] += (uint32_t)(cv.w * col_scale) + (uint32_t)rc;
                    }
                }
                else
                {
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        v[i] += (uint32_t)rc;
                }
                if (!row_valid)
                    continue;
                int32_t* o = out_row + col;
                if (col + 32 <= p.W && (p.W & 7) == 0 && wide_ok)
                {
#pragma unroll
                    for (int i = 0; i < 32; i += 8)
                        ptx::st_global_v8(o + i, v[i], v[i + 1], v[i + 2], v[i + 3], v[i + 4], v[i + 5], v[i + 6], v[i + 7]);
                }
                else if (col + 32 <= p.W && (p.W & 3) == 0)
                {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<int4*>(o + i) = make_int4((int)v[i], (int)v[i + 1], (int)v[i + 2], (int)v[i + 3]);
                }
                else
                {
                    const int nvalid = min(32, p.W - col);
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        if (i < nvalid)
                            o[i] = (int32_t)v[i];
                }
            }
            // this warp has read its part of the buffer: one arrival per warp on the first CTA's barrier
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                ptx::mbar_arrive_cluster(empty_first[acc]);
            acc ^= 1;
            if (acc == 0)
                acc_phase ^= 1u;
        }
        if (!ok && lane == 0)
            atomicOr(p.status, TB200_DEV_TIMEOUT);
    }

    // ---------------------------------------------------------------------- teardown
    // Neither CTA may leave (or free its TMEM) while the other can still signal it or read its shared memory.
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync();
    if (warp == 1)
    {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc_pair(tmem_base, kPairTmemCols);
    }
}

typedef CUresult (*PFN_encodeTiledPair)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                        const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                        CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

PFN_encodeTiledPair pair_encode_fn()
{
    static PFN_encodeTiledPair fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_encodeTiledPair>(sym);
    });
    return fn;
}

}    // namespace

// MATMUL problems as api.cu describes them: A [1][batch][H][C], B MN-major [batch][C][W], int32 output.
bool tc_gemm_pair_supported(const TcProblem& q, int num_sms)
{
    if (diag_env_int("TB200_TC_PAIR", 1) == 0)
        return false;
    const bool i8 = q.in_dtype == TB200_INT8 && q.epi == TC_EPI_I32 && q.out_dtype == TB200_INT32;
    const bool fl = q.epi == TC_EPI_FLOAT && !q.has_clamp && q.bias_f_pad == nullptr;
    const bool f8 = fl && dtype_is_fp8(q.in_dtype) && (q.out_dtype == TB200_FP16 || q.out_dtype == TB200_FP32) &&
                    diag_env_int("TB200_TC_PAIR_F8", 1) != 0;
    const bool f16 = fl && (q.in_dtype == TB200_FP16 || q.in_dtype == TB200_BF16) &&
                     (q.out_dtype == q.in_dtype || q.out_dtype == TB200_FP32) && diag_env_int("TB200_TC_PAIR_F16", 1) != 0;
    if ((!i8 && !f8 && !f16) || !q.b_mn_major)
        return false;
    if ((f8 || f16) && (q.corr != nullptr || q.row_corr != nullptr || q.fuse_row_sums != 0))
        return false;
    const int es = f16 ? 2 : 1;
    if (q.N != 1 || q.KH != 1 || q.KW != 1 || q.stride_x != 1 || q.stride_y != 1 || q.pad_t || q.pad_l)
        return false;
    if (q.a_stride_w || q.a_stride_h || q.a_stride_n || q.corr_classes || q.tile_begin || q.tile_end)
        return false;
    if (q.corr != nullptr && (q.corr_stride % 256 != 0 || q.corr_stride < q.OC || q.corr_ystride != q.corr_stride))
        return false;
    const int64_t ldb = q.b_ld ? q.b_ld : q.OC;
    // whole 256 x 256 tiles must dominate, and TMA wants 16-byte row pitches
    if (q.IW < 256 || q.OC < 256 || q.IC * es < 128 || (q.IC * es) % 16 != 0 || (ldb * es) % 16 != 0)
        return false;
    if ((reinterpret_cast<uintptr_t>(q.a) | reinterpret_cast<uintptr_t>(q.b) | reinterpret_cast<uintptr_t>(q.out)) & 15)
        return false;
    // fewer tiles than half the pairs: the single-CTA kernel spreads such a problem over more SMs
    const int64_t tiles = (int64_t)q.IH * ((q.IW + 255) / 256) * ((q.OC + 255) / 256);
    return tiles >= num_sms / 4 && tiles < (1LL << 30);
}

tb200_status tc_gemm_pair_launch(tb200_ctx* ctx, const TcProblem& q)
{
    PFN_encodeTiledPair enc = pair_encode_fn();
    if (!enc)
        return fail(ctx, TB200_INTERNAL, "cuTensorMapEncodeTiled is not available from the driver");
    PairParams k;
    memset(&k, 0, sizeof(k));
    k.NB = q.IH;
    k.H  = q.IW;
    k.C  = q.IC;
    k.W  = q.OC;
    const int64_t ldb = q.b_ld ? q.b_ld : q.OC;
    k.tiles_m      = (k.H + 255) / 256;
    k.tiles_w      = (k.W + 255) / 256;
    k.num_tiles    = k.NB * k.tiles_m * k.tiles_w;
    const bool f8  = dtype_is_fp8(q.in_dtype);
    const bool f16 = q.in_dtype == TB200_FP16 || q.in_dtype == TB200_BF16;
    const int es   = f16 ? 2 : 1;
    k.chunk_elems  = 128 / es;
    k.total_chunks = (k.C + k.chunk_elems - 1) / k.chunk_elems;
    // A: K-major rows of 128 bytes, 8-row groups 1024 bytes apart.  B: MN-major, 128-byte atoms of columns (128 columns
    // of bytes: one atom per CTA; 64 columns of halves: two atoms per CTA, a box of chunk_elems K rows apart), K rows
    // 128 bytes apart, 8-row groups 1024 bytes apart; an MMA's K rows (32 of bytes, 16 of halves) span 4096 / 2048 bytes.
    k.b_box_cols  = 128 / es;
    k.b_boxes     = 128 / k.b_box_cols;
    k.b_box_bytes = k.chunk_elems * 128;
    k.b_kstep16   = (uint32_t)((32 / es) * 128) >> 4;
    k.a_desc_hi = ptx::make_smem_desc_hi(16, 1024, 2);
    k.b_desc_hi = ptx::make_smem_desc_hi(k.b_box_bytes, 1024, 2);
    k.mma_kind  = f16 ? 2 : f8 ? 1 : 0;
    if (f16)
    {
        const uint32_t fmt = q.in_dtype == TB200_BF16 ? 1u : 0u;
        k.idesc    = ptx::make_idesc(1u, fmt, fmt, 0u, 1u, 256u, 256u);
        k.out_kind = q.out_dtype == TB200_FP32 ? 1 : q.out_dtype == TB200_BF16 ? 3 : 2;
    }
    else if (f8)
    {
        // kind::f8f6f4: operand formats 0 = E4M3, 1 = E5M2, chosen per operand; fp32 accumulators
        const tb200_dtype bdt = q.b_fp8_dtype ? (tb200_dtype)q.b_fp8_dtype : q.in_dtype;
        k.idesc    = ptx::make_idesc(1u, q.in_dtype == TB200_FP8E5M2 ? 1u : 0u, bdt == TB200_FP8E5M2 ? 1u : 0u, 0u, 1u, 256u, 256u);
        k.out_kind = q.out_dtype == TB200_FP32 ? 1 : 2;
    }
    else
        k.idesc = ptx::make_idesc(2u, 1u, 1u, 0u, 1u, 256u, 256u);
    k.out         = reinterpret_cast<int32_t*>(q.out);
    k.row_corr    = q.row_corr;
    k.fuse_row_sums = q.fuse_row_sums;
    k.flags         = q.sum_flags;
    k.epoch         = q.sum_epoch;
    k.a_zp          = q.a_zp;
    k.b_zp          = q.b_zp;
    k.corr        = q.corr;
    k.corr_stride = q.corr_stride;
    k.debug       = diag_env_int("TB200_TC_DEBUG", 0);
    k.wait_limit  = ctx->wait_limit_cycles;
    k.status      = ctx->d_status;

    cuuint64_t a_dims[3]    = { (cuuint64_t)k.C, (cuuint64_t)k.H, (cuuint64_t)k.NB };
    cuuint64_t a_strides[2] = { (cuuint64_t)k.C * es, (cuuint64_t)k.C * (cuuint64_t)k.H * es };
    cuuint64_t b_dims[3]    = { (cuuint64_t)k.W, (cuuint64_t)k.C, (cuuint64_t)k.NB };
    cuuint64_t b_strides[2] = { (cuuint64_t)ldb * es, (cuuint64_t)ldb * (cuuint64_t)k.C * es };
    cuuint32_t box[3]       = { (cuuint32_t)k.chunk_elems, 128, 1 };                        // A: K elements x rows
    cuuint32_t box_b[3]     = { (cuuint32_t)k.b_box_cols, (cuuint32_t)k.chunk_elems, 1 };   // B: columns x K rows
    cuuint32_t estr[3]      = { 1, 1, 1 };
    const CUtensorMapDataType tdt = !f16                        ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                    : q.in_dtype == TB200_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                               : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    CUresult r = enc(&k.tmA, tdt, 3, const_cast<void*>(q.a), a_dims, a_strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(ctx, TB200_INTERNAL, "tensor map for A rejected (CUresult %d)", (int)r);
    r = enc(&k.tmB, tdt, 3, const_cast<void*>(q.b), b_dims, b_strides, box_b, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(ctx, TB200_INTERNAL, "tensor map for B rejected (CUresult %d)", (int)r);

    // The ring holds what is in flight from L2: the kernel is bound by latency x bytes in flight, so it takes all the
    // shared memory there is.  One commit per stage; 4 MMAs (one chunk) per commit costs tensor-pipe time, 8 do not.
    k.ksub        = std::max(1, std::min(4, diag_env_int("TB200_PAIR_KSUB", 2)));
    k.stage_bytes = 2 * k.ksub * kPairChunkBytes;
    k.num_stages  = std::min(kPairMaxStages, std::max(2, diag_env_int("TB200_PAIR_STAGES", (224 * 1024) / k.stage_bytes)));
    const int smem_bytes = k.num_stages * k.stage_bytes + 1024;
    void (*kern)(const PairParams) = f16 ? tc_gemm_pair_kernel<2> : f8 ? tc_gemm_pair_kernel<1> : tc_gemm_pair_kernel<0>;
    {
        const tb200_status ast = raise_smem_limit(ctx, 8 + k.mma_kind, reinterpret_cast<const void*>(kern), smem_bytes);
        if (ast != TB200_OK)
            return ast;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim         = dim3(kPairThreads);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cfg.stream           = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id               = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs    = attr;
    cfg.numAttrs = 1;
    // Tiles wait for sums that other pairs publish, so every pair of the grid has to be resident at once: never more
    // pairs than the device can hold of this kernel (asked once per context, i.e. per device; one CTA per SM because
    // of its shared memory).
    int& max_pairs = ctx->max_pairs[k.mma_kind];
    if (max_pairs == 0)
    {
        cfg.gridDim = dim3((unsigned)(2 * (ctx->num_sms / 2)));
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0)
        {
            cudaGetLastError();
            n = ctx->num_sms / 2;
        }
        max_pairs = n;
    }
    const int clusters = std::max(1, std::min(k.num_tiles, std::min(max_pairs, ctx->num_sms / 2)));
    cfg.gridDim        = dim3((unsigned)(2 * clusters));
    timer_begin(ctx);
    const cudaError_t le = cudaLaunchKernelEx(&cfg, kern, k);
    timer_end(ctx);
    if (le != cudaSuccess)
        return fail(ctx, TB200_INTERNAL, "launch of the CTA-pair MATMUL kernel failed: %s", cudaGetErrorString(le));
    return post_launch(ctx, f16 ? "tc_gemm_pair_f16" : f8 ? "tc_gemm_pair_f8" : "tc_gemm_pair_i8_i32");
}

}    // namespace tb200
