// Shared host-side definitions of the tb200 library: context, tensor handle, status helpers.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <cuda_runtime.h>
#include <string>
#include <utility>
#include <vector>

#include "../../include/tb200.h"

struct tb200_tensor
{
    tb200_dtype dtype;
    int rank;
    int32_t shape[6];
    void* data;
    size_t bytes;
    bool owns;
    // element strides per dimension; a view made by tb200_tensor_slice shares its parent's memory and pitch
    int64_t stride[6];
    bool contiguous;
};

// Bits of the device status word (one int32 per context, OR-ed into by kernels).
enum : int
{
    TB200_DEV_UNPREDICTABLE = 1,    // a REQUIRE condition of the reference failed for some element
    TB200_DEV_TIMEOUT       = 2,    // a bounded pipeline wait gave up (internal error)
};

struct tb200_graph
{
    cudaGraph_t graph    = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint64_t launches    = 0;    // kernels recorded
};

struct tb200_ctx
{
    int device           = 0;
    cudaStream_t stream  = nullptr;
    bool owns_stream     = false;
    int* d_status        = nullptr;    // device status word
    int* h_status        = nullptr;    // pinned mirror
    void* scratch        = nullptr;    // grow-on-demand device scratch (zero-point sums, weight tables)
    size_t scratch_bytes = 0;
    uint32_t* pair_flags = nullptr;    // flags of the CTA-pair MATMUL's in-kernel zero-point sums, zeroed when allocated
    size_t pair_flag_words = 0;
    uint32_t pair_epoch  = 0;          // bumped per launch; a flag equal to it means "written in this launch"
    void* stage          = nullptr;    // grow-on-demand staging of TRANSPOSE_CONV2D (spread input, mirrored weights)
    size_t stage_bytes   = 0;
    void* io_pinned      = nullptr;    // 64 MiB pinned host buffer of the .npy loader / writer, allocated on first use
    void* join_table     = nullptr;    // 64 KiB result table + 8 KiB REQUIRE bits of the per-tensor residual join
    uint64_t launches    = 0;
    int policy           = 0;
    int num_sms          = 148;
    bool capturing       = false;    // between tb200_capture_begin / tb200_capture_end
    const char* last_kernel = "none";
    std::string err;
    // host-buffer pipeline of tb200_matmul_host: copy streams, events and two sets of device staging buffers
    struct HostPipe
    {
        cudaStream_t h2d = nullptr, d2h = nullptr;
        cudaEvent_t up[2] = {}, done[2] = {}, down[2] = {};
        void* buf[2]      = {};
        size_t cap        = 0;
        bool ready        = false;
    } pipe;
    // optional CUDA-event brackets around the main kernels (tb200_timer_enable)
    bool timing = false;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> timed;
};

namespace tb200
{

inline size_t dtype_size(tb200_dtype d)
{
    switch (d)
    {
        case TB200_INT8:
        case TB200_UINT8:
        case TB200_FP8E4M3:
        case TB200_FP8E5M2:
            return 1;
        case TB200_BF16:
        case TB200_FP16:
        case TB200_INT16:
        case TB200_UINT16:
            return 2;
        case TB200_FP32:
        case TB200_INT32:
            return 4;
    }
    return 0;
}

inline bool dtype_is_float(tb200_dtype d)
{
    return d == TB200_FP16 || d == TB200_BF16 || d == TB200_FP32;
}

inline bool dtype_is_fp8(tb200_dtype d)
{
    return d == TB200_FP8E4M3 || d == TB200_FP8E5M2;
}

inline int64_t numel(const tb200_tensor* t)
{
    int64_t n = 1;
    for (int i = 0; i < t->rank; i++)
        n *= t->shape[i];
    return n;
}

inline tb200_status fail(tb200_ctx* ctx, tb200_status st, const char* fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (ctx)
        ctx->err = buf;
    return st;
}

#define TB200_CUDA_CHECK(ctx, expr)                                                                        \
    do                                                                                                     \
    {                                                                                                      \
        cudaError_t e__ = (expr);                                                                          \
        if (e__ != cudaSuccess)                                                                            \
            return tb200::fail((ctx), TB200_INTERNAL, "%s failed: %s", #expr, cudaGetErrorString(e__));    \
    } while (0)

// The reference's ERROR_IF: a violated graph rule ends evaluation with TOSA_ERROR
// (reference_model/include/func_debug.h:112-178).
#define TB200_ERROR_IF(ctx, cond, ...)                                                                     \
    do                                                                                                     \
    {                                                                                                      \
        if (cond)                                                                                          \
            return tb200::fail((ctx), TB200_ERROR, __VA_ARGS__);                                           \
    } while (0)

tb200_status ensure_scratch(tb200_ctx* ctx, size_t bytes);
tb200_status post_launch(tb200_ctx* ctx, const char* kernel_name, int n_launches = 1);
// Event brackets for tb200_timer_*: call timer_begin before and timer_end after the main kernel's launch.
void timer_begin(tb200_ctx* ctx);
void timer_end(tb200_ctx* ctx);

// ----------------------------------------------------------------------------------------------
// Tensor-core GEMM / implicit-GEMM convolution (tc_gemm.cu)
// ----------------------------------------------------------------------------------------------
enum TcEpilogue : int
{
    TC_EPI_I32     = 0,    // int32 out = acc + row_corr[row] + col_corr[col]
    TC_EPI_RESCALE = 1,    // int8/int16/int32 out = clamp(rescale(acc + col_corr[col]) + out_zp)
    TC_EPI_FLOAT   = 2,    // fp16/bf16/fp32 out = clamp(acc + bias[col])
};

struct TcProblem
{
    // element type of A and B: TB200_INT8, TB200_FP16, TB200_BF16, or an fp8 format (then B may be the other fp8 format:
    // b_fp8_dtype, 0 = same as A)
    tb200_dtype in_dtype;
    int b_fp8_dtype;
    // A: activation tensor viewed as [N][IH][IW][IC] (matmul: [1][batch][M][K])
    const void* a;
    int N, IH, IW, IC;
    int64_t a_stride_w, a_stride_h, a_stride_n;    // element strides of A (0 = contiguous NHWC)
    // output pixel grid [N][OH][OW] and columns OC (matmul: [1][batch][M] x Ncols)
    int OH, OW, OC;
    int KH, KW;
    int pad_t, pad_l, stride_y, stride_x, dil_y, dil_x;
    // B: K-major weights [OC][KH*KW*IC] (b_mn_major == 0) or MN-major [batch][K][OC] (b_mn_major == 1, matmul)
    const void* b;
    int b_mn_major;
    int64_t b_ld;    // MN-major B: elements between consecutive K rows (0 = OC)
    // epilogue
    int epi;
    tb200_dtype out_dtype;
    void* out;
    // out_sy != 0: the output pixel grid is a strided view of a dense [N][out_OH][out_OW][OC] tensor, pixel (oy, ox)
    // landing at (oy * out_sy + out_y0, ox * out_sx + out_x0) (one phase of a TRANSPOSE_CONV2D); 0: dense [N][OH][OW]
    int out_OH, out_OW, out_sy, out_sx, out_y0, out_x0;
    // d2s_oc != 0 (with out_sy != 0): the OC columns are (ky, kx, oc) blocks of d2s_oc channels; block (ky, kx) of
    // pixel (oy, ox) is output pixel (oy * out_sy + ky, ox * out_sx + kx) of a [N][out_OH][out_OW][d2s_oc] tensor
    // (a TRANSPOSE_CONV2D whose kernel equals its stride: one GEMM, stamps do not overlap); d2s_kw = kernel width
    int d2s_oc, d2s_kw;
    const int32_t* row_corr;    // [N*OH*OW] added to every column of a row, or null
    // MATMUL on the CTA-pair kernel: derive the row term from A inside the kernel instead (row_corr null):
    // row term = -b_zp * sum_k A[row, k] + IC * a_zp * b_zp
    // 2: both zero-point sums inside the kernel, shared between tiles through global memory: row_corr / corr then point
    // at buffers for the raw row sums of A / column sums of B (null where the other zero point is 0), sum_flags at
    // [batch * tiles_m * 2 + batch * tiles_w * 2] words that persist between launches, sum_epoch at a value no flag holds
    int fuse_row_sums;
    int32_t a_zp, b_zp;
    uint32_t* sum_flags;
    uint32_t sum_epoch;
    // per-column additive constants, padded: [classes][corr_stride]; corr_stride must be a multiple of 256 and cover
    // OC.  corr_classes != 0: the table has (KH+1)^2 (KW+1)^2 rows indexed by the rectangle of in-scope filter taps
    // ((ky_lo*(KH+1)+ky_hi)*(KW+1)+kx_lo)*(KW+1)+kx_hi.  corr_ystride: MATMUL, elements to advance per batch.
    const int32_t* corr;
    int corr_stride, corr_ystride, corr_classes;
    const float* bias_f_pad;     // TC_EPI_FLOAT: fp32 bias padded to corr_stride, or null
    const int32_t* mult_pad;     // TC_EPI_RESCALE: multipliers / shifts expanded per column and padded to corr_stride
    const int8_t* shift_pad;
    int double_round;
    int32_t out_zp;
    int32_t clamp_lo, clamp_hi;    // also the dtype range
    float clamp_lo_f, clamp_hi_f;
    int has_clamp;
    // optional: launch only tiles [tile_begin, tile_end) of the problem (both 0 = all tiles)
    int tile_begin, tile_end;
};

// Returns TB200_OK and launches, or TB200_ERROR with ctx->err set when the shape does not qualify
// (the caller then uses the CUDA-core kernels).
bool tc_gemm_supported(const TcProblem& p, std::string* why);
tb200_status tc_gemm_launch(tb200_ctx* ctx, const TcProblem& p);
// Total tile count of a problem and the tiles per row block (per batch for MATMUL); tiles are numbered batch-major.
bool tc_gemm_tile_counts(const TcProblem& p, int* num_tiles, int* tiles_per_row_block);

// int8 MATMUL on CTA pairs (tc_gemm_pair.cu): large MN-major-B problems with int32 output; tc_gemm_launch routes to it
bool tc_gemm_pair_supported(const TcProblem& p, int num_sms);
tb200_status tc_gemm_pair_launch(tb200_ctx* ctx, const TcProblem& p);

// fp32 SGEMM on CUDA cores (sgemm_f32.cu): out[n] = a[n] x b[n], a [N,H,C], b [N,C,W]
tb200_status sgemm_f32_launch(tb200_ctx* ctx, const float* a, const float* b, float* out, int N, int H, int C, int W);

}    // namespace tb200
