// Shared host-side definitions of the tb200 library: context, tensor handle, status helpers.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <cuda_runtime.h>
#include <cstdlib>
#include <functional>
#include <memory>
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

namespace tb200
{
// What an operator derives from its constant operands alone: for a convolution the zero-point correction rows, the
// per-column RESCALE records and padded multiplier / shift arrays, the fp32 bias, and for few-channel layers the
// re-packed weights; for a residual join the table of all byte pairs.  Built on first use into a device block of its
// own and reused by every later call with the same operands and attributes (the reference decodes constants once per
// graph, reference_model/src/subgraph_traverser.cpp:617-781).
struct Prepared
{
    std::string key;    // kind, operand addresses and every attribute the block's contents depend on
    std::vector<std::pair<const char*, size_t>> operands;    // device ranges the contents were derived from
    void* block   = nullptr;
    size_t bytes  = 0;
    bool valid    = false;    // the block holds what the operands' current contents give
    bool unstable = false;    // an operator wrote into an operand: rebuild before every use
    int host_flag = -1;       // a verdict the builder left in the block and the host has read back (-1: not read yet)
    uint64_t last_use = 0;
    // enqueues, on the context's stream, the kernels that fill `block` from the operands
    std::function<tb200_status(tb200_ctx*, void* block)> rebuild;
};
}    // namespace tb200

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
    int max_smem_optin   = 0;    // largest dynamic shared memory a block may opt into on this device (0 = unknown)
    bool capturing       = false;    // between tb200_capture_begin / tb200_capture_end
    // Captured graphs hold raw addresses of the blocks above: while any is alive a block that would have to move is
    // refused (TB200_ERROR) and blocks of dropped cache entries are parked in `retired` instead of being freed.
    int live_graphs      = 0;
    std::vector<void*> retired;
    // every bounded device-side wait gives up after this many SM clock cycles (about two seconds by default)
    long long wait_limit_cycles = 4000000000LL;
    // 1: other work may hold SMs of this GPU, so no kernel may wait for another CTA of its own grid (the CTA-pair
    // MATMUL then takes its zero-point sums from separate kernels instead of exchanging them through flags)
    int shared_gpu       = 0;
    int join_stream      = 1;    // large table joins through the bulk-copy ring kernel (join_stream.cuh)
    int launch_overlap   = 1;    // launch the kernels that support it with programmatic stream serialization
    int max_pairs[3]     = { 0, 0, 0 };    // resident CTA pairs of the three CTA-pair kernels on this device, 0 = not asked yet
    uint32_t smem_attr_set = 0;            // bit per kernel whose dynamic shared-memory limit has been raised on this device
    // output gather across GPUs (dist.cu): an NCCL communicator created by tb200_comm_init or handed in by the host
    void* comm           = nullptr;
    bool comm_owned      = false;
    int comm_rank        = 0;
    int comm_nranks      = 1;
    bool const_cache_on  = true;
    uint64_t cache_clock = 0;
    std::vector<std::unique_ptr<tb200::Prepared>> prepared;
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

// Entry points run on the context's device whatever device the calling thread had current (a worker thread starts on
// device 0; a host may hold contexts on several GPUs): the thread is switched to the context's device and stays there.
#define TB200_ENTER(ctx)                                                                                   \
    do                                                                                                     \
    {                                                                                                      \
        int dev__ = -1;                                                                                    \
        if (cudaGetDevice(&dev__) != cudaSuccess || dev__ != (ctx)->device)                                \
            TB200_CUDA_CHECK((ctx), cudaSetDevice((ctx)->device));                                         \
    } while (0)

// The reference's ERROR_IF: a violated graph rule ends evaluation with TOSA_ERROR
// (reference_model/include/func_debug.h:112-178).
#define TB200_ERROR_IF(ctx, cond, ...)                                                                     \
    do                                                                                                     \
    {                                                                                                      \
        if (cond)                                                                                          \
            return tb200::fail((ctx), TB200_ERROR, __VA_ARGS__);                                           \
    } while (0)

// Experiment switches.  The default build has none: these helpers return their default and TB200_DIAG_BIT is a
// constant false, so no environment variable and no mask can change what the library computes.  A build with
// -DTB200_DIAG reads TB200_* environment variables at launch and compiles the kernels' diagnostic skip masks in.
#ifdef TB200_DIAG
inline int diag_env_int(const char* name, int dflt)
{
    const char* v = getenv(name);
    return v ? atoi(v) : dflt;
}
#define TB200_DIAG_BIT(mask, bit) (((mask) & (bit)) != 0)
#else
inline int diag_env_int(const char*, int dflt)
{
    return dflt;
}
#define TB200_DIAG_BIT(mask, bit) false
#endif

tb200_status ensure_scratch(tb200_ctx* ctx, size_t bytes);
// ---- cache of blocks derived from constant operands (const_cache.cu)
// Appends a value's bytes to a cache key.
template <typename T>
inline void key_add(std::string* key, const T& v)
{
    key->append(reinterpret_cast<const char*>(&v), sizeof(T));
}
// Entry with this key, or null.
Prepared* cache_find(tb200_ctx* ctx, const std::string& key);
// New entry with a device block of `bytes` (contents not built yet); null when the cache is off, while capturing
// (nothing may allocate then) or when the allocation fails: the caller then works from context scratch as if there
// were no cache.
Prepared* cache_insert(tb200_ctx* ctx, const std::string& key, std::vector<std::pair<const char*, size_t>> operands,
                       size_t bytes, std::function<tb200_status(tb200_ctx*, void*)> rebuild);
// Makes the entry's block current (runs `rebuild` when it is not, or always for an unstable entry).
tb200_status cache_use(tb200_ctx* ctx, Prepared* e);
// An operator is about to write [ptr, ptr + bytes): entries derived from that memory stop being trusted.
void cache_note_write(tb200_ctx* ctx, const void* ptr, size_t bytes);
// New contents were copied into [ptr, ptr + bytes) from outside (upload, file load): entries derived from it are
// rebuilt at once on the stream, behind the copy, so that captured graphs that hold their blocks stay right.
tb200_status cache_note_upload(tb200_ctx* ctx, const void* ptr, size_t bytes);
// [ptr, ptr + bytes) is being released: entries derived from it are dropped.
void cache_note_free(tb200_ctx* ctx, const void* ptr, size_t bytes);
void cache_clear(tb200_ctx* ctx);
// Frees a device block now, or parks it until the context goes while a captured graph may still hold its address.
void release_block(tb200_ctx* ctx, void* block);

// Raises a kernel's dynamic shared-memory limit once per context (bit = a small id per kernel instantiation).
tb200_status raise_smem_limit(tb200_ctx* ctx, int bit, const void* kernel, int bytes);
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
    const int32_t* rec;          // optional: [corr_stride][8] prepared records of the lean RESCALE form (rescale_rec_build)
    const int32_t* delta;        // optional, with corr_classes: [classes][corr_stride] class row minus interior row
    int lean_ok;                 // the host knows every column's record is usable: tc_conv_lean_kernel may run
    // tc_conv_lean_kernel only: the batch dimension is (image, parity of the output column): batch index 2 n + p holds
    // the output columns 2 ox' + p of image n; out_ow_real is the true output width (OW is the per-parity width)
    int xpar, out_ow_real;
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
// true when tc_gemm_launch would run the problem on tc_conv_lean_kernel (the only kernel that understands p.xpar)
bool tc_gemm_lean_supported(const tb200_ctx* ctx, const TcProblem& p);
tb200_status tc_gemm_launch(tb200_ctx* ctx, const TcProblem& p);
// Total tile count of a problem and the tiles per row block (per batch for MATMUL); tiles are numbered batch-major.
bool tc_gemm_tile_counts(const TcProblem& p, int* num_tiles, int* tiles_per_row_block);

// int8 MATMUL on CTA pairs (tc_gemm_pair.cu): large MN-major-B problems with int32 output; tc_gemm_launch routes to it
bool tc_gemm_pair_supported(const TcProblem& p, int num_sms);
tb200_status tc_gemm_pair_launch(tb200_ctx* ctx, const TcProblem& p);

// CONV2D 1x1 (+ CLAMP) -> DEPTHWISE_CONV2D 3x3 (+ CLAMP) as one kernel, fp16 / bf16 (expand_dw.cu): the expanded tensor
// between the two operators stays in shared memory.
struct ExpandDwProblem
{
    tb200_dtype dtype;    // TB200_FP16 or TB200_BF16: every operand and the output
    const void* in;       // [N][IH][IW][IC]
    const void* w1;       // CONV2D weights [C][1][1][IC]
    const void* b1;       // CONV2D bias [C] or [1]
    const void* wd;       // depthwise weights [3][3][C][1]
    const void* bd;       // depthwise bias [C] or [1]
    void* out;            // [N][OH][OW][C]
    int b1_n, bd_n;
    int N, IH, IW, IC, C, OH, OW;
    int pad_t, pad_l, sy, sx;    // of the depthwise operator
    int clamp1, clamp2;          // CLAMP after the CONV2D / after the depthwise operator
    float lo1, hi1, lo2, hi2;
};
bool expand_dw_supported(const tb200_ctx* ctx, const ExpandDwProblem& q, std::string* why);
tb200_status expand_dw_launch(tb200_ctx* ctx, const ExpandDwProblem& q);

// fp32 SGEMM on CUDA cores (sgemm_f32.cu): out[n] = a[n] x b[n], a [N,H,C], b [N,C,W]
tb200_status sgemm_f32_launch(tb200_ctx* ctx, const float* a, const float* b, float* out, int N, int H, int C, int W);

}    // namespace tb200
