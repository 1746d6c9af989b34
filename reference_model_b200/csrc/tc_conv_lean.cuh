// int8 CONV2D + RESCALE (+ CLAMP) to int8 on tcgen05, the form the quantized graphs spend their time in.
// Included by tc_gemm.cu inside its anonymous namespace (it shares TcKernelParams, the tile geometry and the tensor
// maps with the general kernel); the host chooses it when every column's lean RESCALE record is usable
// (rescale_rec_build), the output is a dense, 32-byte aligned int8 tensor and the channel count is a multiple of 32.
//
// What measurement on this part said, and what this kernel does about it:
//   * every tcgen05.commit idles the tensor pipe for 300-700 cycles (a 128 x 64 x 32 MMA takes 104): a tile whose
//     operands fit one shared-memory slot is ONE stage, and its single commit both frees the slot and publishes the
//     accumulator; larger K is cut into the fewest stages that fit;
//   * for N <= 128 the MMA rate does not depend on N, so small layers are bound by bytes and commits, not by math: the
//     weights of a layer with one column block are loaded once per CTA and stay (a third of the traffic of a 3x3
//     64 -> 64 layer);
//   * the fused epilogue is bound by integer issue and by latency: sixteen epilogue warps (four per scheduler) on one
//     CTA per SM, the lean RESCALE form (two multiply-adds and two shifts per output, constants from shared memory,
//     no range check left to do), accumulators fetched sixteen columns at a time (a 32-column tcgen05.ld
//     costs five times two 16-column ones, and sixteen live values keep the loop out of local memory);
//   * two accumulator buffers: warps 2..9 drain one tile while the MMAs fill the other and warps 10..17 wait for it.
// Roles: warp 0 lane 0 TMA producer, warp 1 lane 0 MMA issuer, warps 2..17 epilogue in four groups of four warps
// (a warp reads the TMEM lane quarter `warp % 4`); groups 0, 1 share accumulator buffer 0 (even / odd 32-column
// chunks), groups 2, 3 buffer 1.  Every wait is bounded (p.wait_limit); a wait that gives up sets TB200_DEV_TIMEOUT,
// the roles leave their loops, copies and MMAs in flight are waited for, TMEM is freed.

constexpr int kLeanEpiWarps  = 16;
constexpr int kLeanThreads   = 64 + 32 * kLeanEpiWarps;
constexpr int kLeanAccBufs   = 2;    // accumulator buffers of a 256-column block
constexpr int kLeanMaxAccBufs = 4;   // column blocks of at most 128 get four (one per epilogue group)

// Tiles are numbered column block major here (tile = column block * tiles_m + ((image block * tiles_y + y block) * tiles_x
// + x block)): a CTA stays in one column block as long as it can.
__device__ __forceinline__ TileCoord lean_decode_tile(const TcKernelParams& p, int tile)
{
    TileCoord t;
    const int tiles_m = p.tiles_x * p.tiles_y * p.tiles_n;
    const int cb      = (int)fastdiv_apply((uint32_t)tile, p.fd_m);
    int r             = tile - cb * tiles_m;
    t.col0            = cb * p.block_n;
    const int ry      = (int)fastdiv_apply((uint32_t)r, p.fd_x);
    t.x0              = (r - ry * p.tiles_x) * p.BW;
    const int rn      = (int)fastdiv_apply((uint32_t)ry, p.fd_y);
    t.y0              = (ry - rn * p.tiles_y) * p.BH;
    t.n0              = rn * p.BN;
    return t;
}

// The walk over them without a division per tile: a role visits tiles first, first + step, first + 2 step, ...; the four
// digits of the tile number (x block, y block, image block, column block) advance by the digits of `step` with carries.
// (The producer is a single thread that shares its scheduler with busy epilogue warps: three integer divisions per tile
// were a measurable part of its time per tile.)
struct LeanTileWalk
{
    int xi, yi, ni, cb;        // digits of the current tile
    int dx, dy, dn, dcb;       // digits of the step
    __device__ __forceinline__ void start(const TcKernelParams& p, int first, int step)
    {
        const int tiles_m = p.tiles_x * p.tiles_y * p.tiles_n;
        cb    = first / tiles_m;
        int r = first - cb * tiles_m;
        xi    = r % p.tiles_x;
        r /= p.tiles_x;
        yi = r % p.tiles_y;
        ni = r / p.tiles_y;
        dcb = step / tiles_m;
        r   = step - dcb * tiles_m;
        dx  = r % p.tiles_x;
        r /= p.tiles_x;
        dy = r % p.tiles_y;
        dn = r / p.tiles_y;
    }
    __device__ __forceinline__ TileCoord coord(const TcKernelParams& p) const
    {
        TileCoord t;
        t.col0 = cb * p.block_n;
        t.x0   = xi * p.BW;
        t.y0   = yi * p.BH;
        t.n0   = ni * p.BN;
        return t;
    }
    __device__ __forceinline__ void advance(const TcKernelParams& p)
    {
        xi += dx;
        int c = xi >= p.tiles_x ? 1 : 0;
        xi -= c * p.tiles_x;
        yi += dy + c;
        c = yi >= p.tiles_y ? 1 : 0;
        yi -= c * p.tiles_y;
        ni += dn + c;
        c = ni >= p.tiles_n ? 1 : 0;
        ni -= c * p.tiles_n;
        cb += dcb + c;
    }
};

// Sixteen accumulators of one row through the lean RESCALE form, saturated and packed to sixteen int8.  `delta`, for a
// border pixel, points at what its class of clipped tap rectangle adds to the interior correction (added four columns
// at a time, right before they are used, to keep few values alive).
template <bool FIX>
__device__ __forceinline__ void lean_rescale_x16(const uint32_t (&v)[16], const int32_t (*rec)[8], const int32_t* delta,
                                                 uint32_t (&w)[4])
{
#pragma unroll
    for (int q = 0; q < 4; q++)
    {
        int4 d = make_int4(0, 0, 0, 0);
        if (delta != nullptr)
            d = __ldg(reinterpret_cast<const int4*>(delta) + q);
        const int32_t dv[4] = { d.x, d.y, d.z, d.w };
        int32_t z[4];
#pragma unroll
        for (int j = 0; j < 4; j++)
        {
            const int4 r0 = *reinterpret_cast<const int4*>(&rec[4 * q + j][0]);
            const int2 r1 = *reinterpret_cast<const int2*>(&rec[4 * q + j][4]);
            z[j] = rescale_rec_apply((int32_t)(v[4 * q + j] + (uint32_t)dv[j]), r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, FIX);
        }
        w[q] = pack4_sat_i8(z[0], z[1], z[2], z[3]);
    }
}

// (18 warps: the register file is four partitions of 16 K registers, one per scheduler, and the fullest partition holds
// five of these warps, so a thread gets 96 registers, not the 112 that 65536 / 576 would suggest)
// CLASSES: the layer has border classes (padding with a non-zero input zero point); the instantiation without them
// carries no trace of the border path, which keeps its epilogue loop free of register spills.  FIX: the layer's RESCALE
// has double_round (the sign term of rescale_rec_apply, applied to every column).
template <bool CLASSES, bool FIX>
__global__ void __launch_bounds__(kLeanThreads, 1) tc_conv_lean_kernel(const __grid_constant__ TcKernelParams p)
{
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[kMaxStages];     // TMA -> MMA: the stage's bytes have landed
    __shared__ __align__(8) uint64_t bar_empty[kMaxStages];    // MMA -> TMA (several stages per tile only): stage consumed
    __shared__ __align__(8) uint64_t bar_acc_full[kLeanMaxAccBufs];     // MMA -> epilogue (and -> TMA when a tile is one stage)
    __shared__ __align__(8) uint64_t bar_acc_empty[kLeanMaxAccBufs];    // epilogue -> MMA: accumulator buffer drained
    __shared__ __align__(8) uint64_t bar_b;        // resident weights have landed
    __shared__ __align__(8) uint64_t bar_drain;    // teardown after a wait gave up
    __shared__ uint32_t tmem_base_holder;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* const smem_al   = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
    const uint32_t s_b       = smem_base + (uint32_t)p.lean_b_off;       // resident weights (when p.lean_b_resident)
    const uint32_t s_ring    = smem_base + (uint32_t)p.lean_ring_off;    // stages: ksub A chunks, then ksub B chunks if streamed
    const int acc_bufs       = p.acc_bufs;                  // 2, or 4 when four buffers of block_n columns fit tensor memory
    const int acc_shift      = acc_bufs == 4 ? 2 : 1;       // log2(acc_bufs): tile counters are split with shifts, not divisions
    const int groups_per_buf = 4 >> acc_shift;              // epilogue groups that share one accumulator buffer
    const bool one_stage     = p.lean_stages_per_tile == 1;
    // Halo mode (stride-1 convolutions with a window, weights resident): a tile is BH whole output rows, and ONE box
    // per channel chunk brings the BH + KH - 1 input rows it needs, halo columns included (zero filled outside the
    // image, which is the padding), as rows of `wp` = OW + KW - 1 pixels.  Accumulator row q stands for position
    // (q / wp, q % wp) of that padded grid, and tap (ky, kx) reads the same shared-memory rows shifted by
    // ky * wp + kx pixels: the shift goes into the start address of the operand descriptor (the swizzle is a function
    // of the shared-memory address, so any row offset is a valid start).  Positions with q % wp >= OW compute garbage
    // that is never stored.  Against one box per tap this is KH * KW times fewer bytes and copies per tile.
    const bool halo          = p.lean_halo != 0;
    if (threadIdx.x == 0)
        TB200_TRACE(p, 0);

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < p.num_stages; s++)
        {
            ptx::mbar_init(ptx::smem_u32(&bar_full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&bar_empty[s]), 1);
        }
        for (int a = 0; a < acc_bufs; a++)
        {
            ptx::mbar_init(ptx::smem_u32(&bar_acc_full[a]), 1);
            ptx::mbar_init(ptx::smem_u32(&bar_acc_empty[a]), 4 * groups_per_buf);    // one arrival per epilogue warp
        }
        ptx::mbar_init(ptx::smem_u32(&bar_b), 1);
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
    const int my_tiles = (p.tile_end - p.tile_begin - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    if (threadIdx.x == 0)
        TB200_TRACE(p, 1);
    // the successor kernel may be scheduled from here on: its CTAs take an SM as soon as this grid's leave it
    if (threadIdx.x == 0)
        ptx::dep_launch_trigger();

    if (warp == 0)
    {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0)
        {
            bool ok = true;
            if (p.lean_b_resident)
            {
                // the whole K extent of the (only) column block, once
                ptx::mbar_arrive_expect_tx(ptx::smem_u32(&bar_b), (uint32_t)(p.total_chunks * p.block_n * (p.chunk_elems)));
                for (int ch = 0; ch < p.total_chunks; ch++)
                    ptx::tma_load_3d(s_b + (uint32_t)(ch * p.b_chunk_bytes), &p.tmB, ptx::smem_u32(&bar_b), ch * p.chunk_elems, 0, 0);
            }
            // Weights and epilogue tables are constants (anything written since they were prepared puts a preparing
            // kernel, which never lets its successor start early, between the writer and this launch); activations are
            // the predecessor's output: wait for it.
            ptx::dep_launch_wait();
            int stage = 0;
            uint32_t phase = 0;
            const int a_chunk_bytes = p.a_chunk_bytes, b_chunk_bytes = p.b_chunk_bytes, chunk_elems = p.chunk_elems;
            const uint32_t tx_per_chunk = (uint32_t)p.tx_bytes_per_chunk;
            LeanTileWalk walk;
            walk.start(p, p.tile_begin + (int)blockIdx.x, (int)gridDim.x);
            for (int i = 0; i < my_tiles && ok; i++, walk.advance(p))
            {
                const TileCoord t = walk.coord(p);
                const int ax0 = t.x0 * p.stride_x - p.pad_l;
                const int ay0 = t.y0 * p.stride_y - p.pad_t;
                int chunk_k = 0, cc = 0, ky = 0, kx = 0;
                int chunks_left = p.total_chunks;
                while (chunks_left > 0)
                {
                    // a one-stage tile's slot is released by the commit that publishes its accumulator
                    const uint32_t free_bar = one_stage ? ptx::smem_u32(&bar_acc_full[stage]) : ptx::smem_u32(&bar_empty[stage]);
                    if (!ptx::mbar_wait_bounded(free_bar, phase ^ 1u, p.wait_limit))
                    {
                        ok = false;
                        break;
                    }
                    const int nchunks = min(p.ksub, chunks_left);
                    chunks_left -= nchunks;
                    const uint32_t full = ptx::smem_u32(&bar_full[stage]);
                    uint32_t sA = s_ring + (uint32_t)(stage * p.stage_bytes);
                    uint32_t sB = sA + (uint32_t)(p.ksub * a_chunk_bytes);
                    if (halo)
                    {
                        // one box per channel chunk: every input row the tile's taps touch, halo columns included
                        ptx::mbar_arrive_expect_tx(full, (uint32_t)p.chunks_per_tap * tx_per_chunk);
                        for (int c2 = 0; c2 < p.chunks_per_tap; c2++)
                            ptx::tma_load_4d(sA + (uint32_t)(c2 * a_chunk_bytes), &p.tmA, full, c2 * chunk_elems, -p.pad_l, ay0, t.n0);
                        chunks_left = 0;
                    }
                    else
                    {
                    ptx::mbar_arrive_expect_tx(full, (uint32_t)nchunks * tx_per_chunk);
                    for (int j = 0; j < nchunks; j++)
                    {
                        ptx::tma_load_4d(sA, &p.tmA, full, cc * chunk_elems, ax0 + kx * p.dil_x, ay0 + ky * p.dil_y, t.n0);
                        if (!p.lean_b_resident)
                        {
                            ptx::tma_load_3d(sB, &p.tmB, full, chunk_k, t.col0, 0);
                            sB += b_chunk_bytes;
                        }
                        sA += a_chunk_bytes;
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
                    if (++stage == p.num_stages)
                    {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (i == 0)
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
            bool ok = true;
            if (p.lean_b_resident)
            {
                ok = ptx::mbar_wait_bounded(ptx::smem_u32(&bar_b), 0u, p.wait_limit);
                ptx::tc_fence_after_sync();
            }
            int stage = 0;
            uint32_t phase = 0;
            const int mmas = p.mmas_per_chunk;
            const uint32_t idesc = p.idesc;
            const uint64_t a_chunk16 = (uint64_t)(p.a_chunk_bytes >> 4), b_chunk16 = (uint64_t)(p.b_chunk_bytes >> 4);
            for (int i = 0; i < my_tiles && ok; i++)
            {
                const int acc            = i & (acc_bufs - 1);
                const uint32_t acc_phase = (uint32_t)(i >> acc_shift) & 1u;
                if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bar_acc_empty[acc]), acc_phase ^ 1u, p.wait_limit))
                {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * p.block_n);
                uint32_t accum  = 0;
                int chunk_index = 0;
                int chunks_left = p.total_chunks;
                while (chunks_left > 0)
                {
                    if (!ptx::mbar_wait_bounded(ptx::smem_u32(&bar_full[stage]), phase, p.wait_limit))
                    {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    if (i == 0 && chunks_left == p.total_chunks)
                        TB200_TRACE(p, 4);
                    const int nchunks = min(p.ksub, chunks_left);
                    chunks_left -= nchunks;
                    const uint32_t sA = s_ring + (uint32_t)(stage * p.stage_bytes);
                    uint64_t ad_chunk = ptx::smem_desc(p.a_desc_hi, sA);
                    uint64_t bd_chunk = p.lean_b_resident
                                            ? ptx::smem_desc(p.b_desc_hi, s_b + (uint32_t)(chunk_index * p.b_chunk_bytes))
                                            : ptx::smem_desc(p.b_desc_hi, sA + (uint32_t)(p.ksub * p.a_chunk_bytes));
                    if (halo)
                    {
                        // the stage holds chunks_per_tap boxes; tap (ky, kx) starts ky * wp + kx pixel rows into each
                        const uint64_t row16 = (uint64_t)(p.chunk_elems >> 4);    // one pixel row of a chunk, in 16-byte units
                        uint64_t tap_row = ad_chunk;
                        for (int ky = 0; ky < p.KH; ky++, tap_row += (uint64_t)p.lean_halo_wp * row16)
                        {
                            uint64_t tap = tap_row;
                            for (int kx = 0; kx < p.KW; kx++, tap += row16)
                            {
                                uint64_t ac = tap;
                                for (int c2 = 0; c2 < p.chunks_per_tap; c2++)
                                {
                                    ptx::mma_i8_ss_chunk(d_tmem, ac, bd_chunk, idesc, accum, mmas);
                                    accum = 1;
                                    ac += a_chunk16;
                                    bd_chunk += b_chunk16;
                                }
                            }
                        }
                    }
                    else
                    for (int j = 0; j < nchunks; j++)
                    {
                        ptx::mma_i8_ss_chunk(d_tmem, ad_chunk, bd_chunk, idesc, accum, mmas);    // 32 bytes of K per MMA
                        accum = 1;
                        ad_chunk += a_chunk16;
                        bd_chunk += b_chunk16;
                    }
                    chunk_index += nchunks;
                    if (!one_stage)
                        ptx::mma_commit(ptx::smem_u32(&bar_empty[stage]));
                    if (++stage == p.num_stages)
                    {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok)
                    break;
                ptx::mma_commit(ptx::smem_u32(&bar_acc_full[acc]));
                if (i == 0)
                    TB200_TRACE(p, 5);
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
        // ------------------------------------------------------------------ epilogue: 4 groups of 4 warps
        const int quarter = warp & 3;                  // TMEM lane quarter this warp may read
        const int group   = (warp - 2) >> 2;           // 0..3
        const int acc     = group / groups_per_buf;    // accumulator buffer of this group
        const int sub     = group % groups_per_buf;    // which 32-column chunks of a tile it takes
        const int gtid    = (int)threadIdx.x - 64 - group * 128;    // 0..127 inside the group
        int32_t(*rec)[8]  = reinterpret_cast<int32_t(*)[8]>(smem_al + p.lean_rec_off + (size_t)group * p.lean_rec_stride);
        const int row     = quarter * 32 + lane;
        const int row_w   = halo ? p.lean_halo_wp : p.BW;    // accumulator rows per output row (halo: with the halo columns)
        const int xx      = row % row_w;
        const int yy      = (row / row_w) % p.BH;
        const int nn      = row / (row_w * p.BH);
        const bool narrow_clamp = p.clamp_lo > -128 || p.clamp_hi < 127;
        const uint32_t lo4 = (uint32_t)(p.clamp_lo & 0xff) * 0x01010101u;
        const uint32_t hi4 = (uint32_t)(p.clamp_hi & 0xff) * 0x01010101u;
        const int nchunks32 = p.block_n / 32;
        int loaded_col0 = -1;
        bool ok = true;
        bool dep_waited = false;
        for (int i = acc; i < my_tiles; i += acc_bufs)
        {
            // (the epilogue decodes with divisions: the eight registers of a LeanTileWalk cost it more in spills under the
            // 96-register cap than the divisions cost, 1x1 64 -> 256 measured 139 against 130 us)
            const TileCoord t = lean_decode_tile(p, p.tile_begin + (int)blockIdx.x + i * (int)gridDim.x);
            if (loaded_col0 != t.col0)
            {
                // this group's copy of the column block's records (the barrier also keeps the copy from overtaking the
                // group's last reads of the previous block)
                asm volatile("bar.sync %0, 128;" ::"r"(2 + group) : "memory");
                for (int c = gtid; c < p.block_n; c += 128)
                {
                    const int4* rp = reinterpret_cast<const int4*>(p.rec + (int64_t)(t.col0 + c) * 8);
                    *reinterpret_cast<int4*>(&rec[c][0]) = __ldg(rp);
                    *reinterpret_cast<int4*>(&rec[c][4]) = __ldg(rp + 1);
                }
                asm volatile("bar.sync %0, 128;" ::"r"(2 + group) : "memory");
                loaded_col0 = t.col0;
            }
            // the records are constants; the border deltas are too, but the output may still be read by the predecessor
            if (!dep_waited)
            {
                ptx::dep_launch_wait();
                dep_waited = true;
            }
            // After a wait has given up, this warp keeps walking its tiles only to meet its group at the barrier above
            // (the other three warps may still be working); it does no further work.
            if (!ok)
                continue;
            ok = ptx::mbar_wait_bounded(ptx::smem_u32(&bar_acc_full[acc]), (uint32_t)(i >> acc_shift) & 1u, p.wait_limit);
            ok = __all_sync(0xffffffffu, ok);    // the whole warp agrees before the warp-collective TMEM loads
            if (!ok)
                continue;
            ptx::tc_fence_after_sync();
            if (threadIdx.x == 64 && i == 0)
                TB200_TRACE(p, 7);

            const int ox = t.x0 + xx, oy = t.y0 + yy, on = t.n0 + nn;
            bool row_valid = (nn < p.BN) && (ox < p.OW) && (oy < p.OH) && (on < p.N);
            // parity-split problems: batch index 2 n + parity holds the output columns 2 ox + parity of image n
            const int on_r = p.lean_xpar ? (on >> 1) : on;
            const int ox_r = p.lean_xpar ? 2 * ox + (on & 1) : ox;
            const int ow_r = p.lean_xpar ? p.lean_ow_real : p.OW;
            row_valid      = row_valid && ox_r < ow_r;
            int8_t* out_row = reinterpret_cast<int8_t*>(p.out) + (((int64_t)on_r * p.OH + oy) * ow_r + ox_r) * p.OC;
            const int32_t* delta_row = nullptr;
            if (CLASSES && row_valid)
            {
                int ky_lo = 0, ky_hi = p.KH, kx_lo = 0, kx_hi = p.KW;
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
                const int cls = ((ky_lo * (p.KH + 1) + ky_hi) * (p.KW + 1) + kx_lo) * (p.KW + 1) + kx_hi;
                if (cls != p.cls_interior)
                    delta_row = p.delta + (int64_t)cls * p.corr_stride + t.col0;
            }

            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * p.block_n);
            // chunks past the last channel exist only in a last, partly filled column block (OC is a multiple of 32)
            const int chunks_here = min(nchunks32, (p.OC - t.col0) / 32);
            for (int c = sub; c < chunks_here; c += groups_per_buf)
            {
                uint32_t w[8];
#pragma unroll
                for (int h = 0; h < 2; h++)
                {
                    uint32_t v[16];
                    if (TB200_DIAG_BIT(p.debug, 64))
                    {
                        // diagnostic: no tensor-memory load
#pragma unroll
                        for (int e = 0; e < 16; e++)
                            v[e] = (uint32_t)(row + e + c);
                    }
                    else
                    {
                        ptx::tmem_ld_32x32b_x16(taddr + (uint32_t)(c * 32 + h * 16), v);
                        ptx::tmem_ld_wait();
                    }
                    uint32_t w4[4];
                    if (TB200_DIAG_BIT(p.debug, 128))
                    {
                        // diagnostic: no arithmetic, no record reads
#pragma unroll
                        for (int e = 0; e < 4; e++)
                            w4[e] = v[4 * e] ^ v[4 * e + 1] ^ v[4 * e + 2] ^ v[4 * e + 3];
                    }
                    else if (TB200_DIAG_BIT(p.debug, 256))
                    {
                        // diagnostic: the arithmetic with one record for all columns (a single shared-memory read)
                        const int4 r0 = *reinterpret_cast<const int4*>(&rec[0][0]);
                        const int2 r1 = *reinterpret_cast<const int2*>(&rec[0][4]);
#pragma unroll
                        for (int e = 0; e < 4; e++)
                        {
                            int32_t z[4];
#pragma unroll
                            for (int j = 0; j < 4; j++)
                                z[j] = rescale_rec_apply((int32_t)v[4 * e + j], r0.x, r0.y + j, r0.z + e, r0.w, r1.x, r1.y, FIX);
                            w4[e] = pack4_sat_i8(z[0], z[1], z[2], z[3]);
                        }
                    }
                    else
                        lean_rescale_x16<FIX>(v, &rec[c * 32 + h * 16],
                                              (CLASSES && delta_row != nullptr) ? delta_row + c * 32 + h * 16 : nullptr, w4);
                    w[4 * h + 0] = w4[0]; w[4 * h + 1] = w4[1]; w[4 * h + 2] = w4[2]; w[4 * h + 3] = w4[3];
                }
                if (narrow_clamp)
                {
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        w[q] = __vmins4(__vmaxs4(w[q], lo4), hi4);
                }
                if (row_valid && !(TB200_DIAG_BIT(p.debug, 32) && w[0] != 0x12345678u))
                    ptx::st_global_v8(out_row + t.col0 + c * 32, w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);
            }
            // this warp has read its part of the buffer
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
                ptx::mbar_arrive(ptx::smem_u32(&bar_acc_empty[acc]));
            if (threadIdx.x == 64 && i == 0)
                TB200_TRACE(p, 8);
        }
        if (threadIdx.x == 64)
            TB200_TRACE(p, 9);
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
        for (int s = 0; s < p.num_stages; s++)
        {
            ptx::mbar_wait_bounded(ptx::smem_u32(&bar_full[s]), 0u, 2000000LL);
            ptx::mbar_wait_bounded(ptx::smem_u32(&bar_full[s]), 1u, 2000000LL);
        }
        if (p.lean_b_resident)
            ptx::mbar_wait_bounded(ptx::smem_u32(&bar_b), 0u, 2000000LL);
    }
    if (warp == 1 && lane == 0 && abort_flag)
    {
        // ... and let the tensor-core work already issued retire before its accumulators' tensor memory is freed
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
