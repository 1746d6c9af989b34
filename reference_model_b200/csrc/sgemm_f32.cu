// fp32 batched MATMUL on CUDA cores: FFMA only, no TF32, so every product and sum is an IEEE fp32 operation
// and the result stays inside the reference's dot-product error bound.
//
// 128 x 128 output tile per 256-thread block, K stepped 16 at a time through double-buffered shared memory,
// 8 x 8 accumulators per thread arranged as 2 x 2 groups of 4 x 4 so that shared-memory reads are 128-bit
// and conflict-free, held as pairs of neighbouring columns for the packed multiply-add.  A [N,H,C] is read along C (transposed into shared memory), B [N,C,W] along W.
#include <cuda_runtime.h>

#include "common.h"

namespace tb200
{
namespace
{

constexpr int BM = 128, BN = 128, BK = 16;

template <bool VEC>
__global__ void __launch_bounds__(256, 2)
    sgemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ Cout, int H, int C,
                     int W, int tiles_w)
{
    __shared__ __align__(16) float As[2][BK][BM];
    __shared__ __align__(16) float Bs[2][BK][BN];

    const int batch = blockIdx.y;
    const int tm    = blockIdx.x / tiles_w;
    const int tn    = blockIdx.x % tiles_w;
    const int m0 = tm * BM, n0 = tn * BN;
    const float* Ab = A + (int64_t)batch * H * C;
    const float* Bb = B + (int64_t)batch * C * W;
    float* Cb       = Cout + (int64_t)batch * H * W;

    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    // global -> shared assignment: A tile 128 rows x 16 k (two float4 along k per thread: k halves 0-7 and 8-15),
    // B tile 16 k x 128 cols (two float4 along n per thread: k rows b_k and b_k + 8)
    const int a_row = tid / 2, a_k = (tid % 2) * 4;
    const int b_k = tid / 32, b_col = (tid % 32) * 4;

    // accumulators as pairs of neighbouring columns: one packed multiply-add (fma.rn.f32x2, two IEEE fp32 operations,
    // the results fmaf gives) per pair
    float2 acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
            acc[i][j] = make_float2(0.f, 0.f);

    float4 ra[2], rb[2];
    auto load_tiles = [&](int k0, int nbuf) {
#pragma unroll
        for (int h = 0; h < 2; h++)
        {
            const int gm = m0 + a_row, gk = k0 + a_k + 8 * h;
            if (VEC)
            {
                ra[h] = (gm < H && gk < C) ? *reinterpret_cast<const float4*>(Ab + (int64_t)gm * C + gk)
                                           : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            else
            {
                float t[4];
#pragma unroll
                for (int j = 0; j < 4; j++)
                    t[j] = (gm < H && gk + j < C) ? Ab[(int64_t)gm * C + gk + j] : 0.f;
                ra[h] = make_float4(t[0], t[1], t[2], t[3]);
            }
            const int bk = k0 + b_k + 8 * h, bn = n0 + b_col;
            if (VEC)
            {
                // B needs no transposition: an asynchronous 16-byte copy straight into the other shared-memory buffer
                // (zero-filled outside the matrix), no staging registers
                const bool inside = bk < C && bn < W;
                const float* src  = inside ? Bb + (int64_t)bk * W + bn : Bb;
                const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(&Bs[nbuf][b_k + 8 * h][b_col]));
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(inside ? 16 : 0)
                             : "memory");
            }
            else
            {
                float t[4];
#pragma unroll
                for (int j = 0; j < 4; j++)
                    t[j] = (bk < C && bn + j < W) ? Bb[(int64_t)bk * W + bn + j] : 0.f;
                rb[h] = make_float4(t[0], t[1], t[2], t[3]);
            }
        }
    };
    auto store_tiles = [&](int buf) {
#pragma unroll
        for (int h = 0; h < 2; h++)
        {
            As[buf][a_k + 8 * h + 0][a_row] = ra[h].x;
            As[buf][a_k + 8 * h + 1][a_row] = ra[h].y;
            As[buf][a_k + 8 * h + 2][a_row] = ra[h].z;
            As[buf][a_k + 8 * h + 3][a_row] = ra[h].w;
            if (!VEC)
                *reinterpret_cast<float4*>(&Bs[buf][b_k + 8 * h][b_col]) = rb[h];
        }
        if (VEC)
            asm volatile("cp.async.wait_all;" ::: "memory");
    };

    const int nk = (C + BK - 1) / BK;
    load_tiles(0, 0);
    store_tiles(0);
    __syncthreads();
    for (int kt = 0; kt < nk; kt++)
    {
        const int buf = kt & 1;
        if (kt + 1 < nk)
            load_tiles((kt + 1) * BK, buf ^ 1);
#pragma unroll
        for (int k = 0; k < BK; k++)
        {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4 + 64]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4 + 64]);
            const float av[8]  = { a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w };
            const float2 bv[4] = { make_float2(b0.x, b0.y), make_float2(b0.z, b0.w), make_float2(b1.x, b1.y), make_float2(b1.z, b1.w) };
#pragma unroll
            for (int i = 0; i < 8; i++)
            {
                const float2 a2 = make_float2(av[i], av[i]);
#pragma unroll
                for (int j = 0; j < 4; j++)
                    acc[i][j] = __ffma2_rn(a2, bv[j], acc[i][j]);
            }
        }
        if (kt + 1 < nk)
        {
            store_tiles(buf ^ 1);
            __syncthreads();
        }
    }

#pragma unroll
    for (int i = 0; i < 8; i++)
    {
        const int gm = m0 + ty * 4 + (i & 3) + (i >> 2) * 64;
        if (gm >= H)
            continue;
#pragma unroll
        for (int jh = 0; jh < 2; jh++)
        {
            const int gn = n0 + tx * 4 + jh * 64;
            float* o     = Cb + (int64_t)gm * W + gn;
            if (VEC && gn + 3 < W)
                *reinterpret_cast<float4*>(o) = make_float4(acc[i][jh * 2].x, acc[i][jh * 2].y, acc[i][jh * 2 + 1].x, acc[i][jh * 2 + 1].y);
            else
            {
                const float v[4] = { acc[i][jh * 2].x, acc[i][jh * 2].y, acc[i][jh * 2 + 1].x, acc[i][jh * 2 + 1].y };
                for (int j = 0; j < 4; j++)
                    if (gn + j < W)
                        o[j] = v[j];
            }
        }
    }
}

}    // namespace

tb200_status sgemm_f32_launch(tb200_ctx* ctx, const float* a, const float* b, float* out, int N, int H, int C, int W)
{
    const int tiles_h = (H + BM - 1) / BM, tiles_w = (W + BN - 1) / BN;
    dim3 grid(tiles_h * tiles_w, N);
    const bool vec = (C % 4 == 0) && (W % 4 == 0) &&
                     ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    timer_begin(ctx);
    if (vec)
        sgemm_f32_kernel<true><<<grid, 256, 0, ctx->stream>>>(a, b, out, H, C, W, tiles_w);
    else
        sgemm_f32_kernel<false><<<grid, 256, 0, ctx->stream>>>(a, b, out, H, C, W, tiles_w);
    timer_end(ctx);
    return post_launch(ctx, "sgemm_f32");
}

}    // namespace tb200
