// int8 MATMUL entry point that performs no device allocation.
//
// tb200_matmul keeps its zero-point row / column sums in scratch memory that the context allocates with
// cudaMalloc on first use.  Some hosts cannot do that: an embedding application may hand the adapter a fixed
// set of device buffers and forbid any further allocation (all device memory belongs to its own pool), and a
// latency-sensitive evaluation loop cannot afford cudaMalloc / cudaFree, which synchronise the whole device.
// For those callers the same computation is offered here with its scratch in a fixed-size array that is part
// of the library image: every GPU that loads libtb200.so holds kNoAllocScratchBytes for the life of the
// process, and nothing is allocated or freed at call time.
#include <mutex>

#include <algorithm>

#include "common.h"

namespace
{

// Zero-point sums of this variant (same arithmetic as the context path's preparation kernels):
//   row_corr[n*H + h] = -b_zp * sum_c A[n,h,c] + C * a_zp * b_zp      (one warp per row)
//   col_corr[n*Wpad + w] = -a_zp * sum_c B[n,c,w]                      (one thread per column, after the rows)
__global__ void noalloc_zp_sums_kernel(const int8_t* __restrict__ a, const int8_t* __restrict__ b,
                                       int32_t* __restrict__ row_corr, int32_t* __restrict__ col_corr, int N, int H,
                                       int C, int W, int Wpad, int32_t a_zp, int32_t b_zp)
{
    const int lane      = threadIdx.x & 31;
    const int64_t gtid  = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nthr  = (int64_t)gridDim.x * blockDim.x;
    const int64_t rows  = (int64_t)N * H;
    for (int64_t r = gtid >> 5; r < rows; r += nthr >> 5)
    {
        const int8_t* ap = a + r * C;
        int32_t s        = 0;
        for (int c = lane; c < C; c += 32)
            s += ap[c];
        for (int o = 16; o > 0; o >>= 1)
            s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0)
            row_corr[r] = -b_zp * s + C * a_zp * b_zp;
    }
    // column sums are stored with a row stride padded to a multiple of 256 (the GEMM reads them 128 bits at a time)
    const int64_t cols = (int64_t)N * Wpad;
    for (int64_t j = gtid; j < cols; j += nthr)
    {
        const int n = (int)(j / Wpad);
        const int w = (int)(j - (int64_t)n * Wpad);
        int32_t s   = 0;
        if (w < W)
        {
            const int8_t* bp = b + (int64_t)n * C * W + w;
            for (int c = 0; c < C; c++)
                s += bp[(int64_t)c * W];
        }
        col_corr[j] = -a_zp * s;
    }
}

// shapes the tensor-core kernel does not take: one thread per output, no scratch needed
__global__ void noalloc_matmul_direct_kernel(const int8_t* __restrict__ a, const int8_t* __restrict__ b,
                                             int32_t* __restrict__ out, int N, int H, int C, int W, int32_t a_zp,
                                             int32_t b_zp)
{
    const int64_t total = (int64_t)N * H * W;
    const int64_t step  = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    {
        const int wc     = (int)(i % W);
        int64_t r        = i / W;
        const int h      = (int)(r % H);
        const int n      = (int)(r / H);
        const int8_t* ap = a + ((int64_t)n * H + h) * C;
        const int8_t* bp = b + (int64_t)n * C * W + wc;
        int32_t acc      = 0;
        for (int c = 0; c < C; c++)
            acc += ((int32_t)ap[c] - a_zp) * ((int32_t)bp[(int64_t)c * W] - b_zp);
        out[i] = acc;
    }
}

// scratch layout: [0] status word (first 256 bytes reserved), then row sums, then column sums
constexpr int kMaxSumEntries           = TB200_NOALLOC_MAX_SUMS;
constexpr size_t kStatusBytes          = 256;
constexpr size_t kNoAllocScratchBytes  = kStatusBytes + sizeof(int32_t) * (size_t)kMaxSumEntries;

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {};    // device address of g_noalloc_scratch, per device
int g_num_sms[kMaxDevices]       = {};

void set_err(char* err, size_t err_len, const char* msg)
{
    if (err && err_len)
        snprintf(err, err_len, "%s", msg);
}

}    // namespace

extern "C" tb200_status tb200_matmul_i8_noalloc(void* stream, const int8_t* a, const int8_t* b, int32_t* out, int32_t N,
                                                int32_t H, int32_t C, int32_t W, int32_t a_zp, int32_t b_zp,
                                                int32_t synchronize, char* err, size_t err_len)
{
    using namespace tb200;
    if (!a || !b || !out)
    {
        set_err(err, err_len, "tb200_matmul_i8_noalloc: null operand");
        return TB200_ERROR;
    }
    if (N <= 0 || H <= 0 || C <= 0 || W <= 0)
    {
        set_err(err, err_len, "tb200_matmul_i8_noalloc: dimensions must be positive");
        return TB200_ERROR;
    }
    if (a_zp < -128 || a_zp > 127 || b_zp < -128 || b_zp > 127)
    {
        set_err(err, err_len, "tb200_matmul_i8_noalloc: zero point outside the int8 range");
        return TB200_ERROR;
    }
    if ((int64_t)N * H * C > 2147483647LL || (int64_t)N * C * W > 2147483647LL || (int64_t)N * H * W > 2147483647LL)
    {
        set_err(err, err_len, "tb200_matmul_i8_noalloc: tensor exceeds 2^31-1 elements");
        return TB200_ERROR;
    }
    const int Wpad     = (W + 255) / 256 * 256;
    const int64_t rows = ((int64_t)N * H + 3) & ~(int64_t)3, cols = (int64_t)N * Wpad;
    if (rows + cols > kMaxSumEntries)
    {
        char msg[200];
        snprintf(msg, sizeof(msg),
                 "tb200_matmul_i8_noalloc: roundup(N*H,4) + N*roundup(W,256) = %lld exceeds the built-in scratch of %d entries; use tb200_matmul",
                 (long long)(rows + cols), kMaxSumEntries);
        set_err(err, err_len, msg);
        return TB200_ERROR;
    }
    if (((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15) != 0)
    {
        set_err(err, err_len, "tb200_matmul_i8_noalloc: device pointers must be 16-byte aligned");
        return TB200_ERROR;
    }

    if (synchronize)
    {
        // a synchronisation inside a stream capture would invalidate the capture
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(reinterpret_cast<cudaStream_t>(stream), &cap) == cudaSuccess &&
            cap != cudaStreamCaptureStatusNone)
        {
            set_err(err, err_len, "tb200_matmul_i8_noalloc: synchronize != 0 is not possible while the stream is being captured");
            return TB200_ERROR;
        }
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    {
        set_err(err, err_len, "tb200_matmul_i8_noalloc: no current CUDA device");
        return TB200_INTERNAL;
    }
    {
        // One-time set-up per device, with that device current: in host code the array's name is only a handle,
        // the address kernels can use comes from cudaGetSymbolAddress.
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (!g_scratch_ptr[dev])
        {
            void* p       = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess || !p)
            {
                set_err(err, err_len, cudaGetErrorString(e));
                return TB200_INTERNAL;
            }
            int sms = 0;
            if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            {
                set_err(err, err_len, "tb200_matmul_i8_noalloc: cannot read the SM count");
                return TB200_INTERNAL;
            }
            g_num_sms[dev]     = sms;
            g_scratch_ptr[dev] = p;
        }
    }
    unsigned char* base = reinterpret_cast<unsigned char*>(g_scratch_ptr[dev]);
    int* d_status       = reinterpret_cast<int*>(base);
    int32_t* row_corr   = reinterpret_cast<int32_t*>(base + kStatusBytes);
    int32_t* col_corr   = row_corr + rows;

    // a context object on the stack: plain host bookkeeping for the shared launch code, owns nothing
    tb200_ctx local;
    local.device   = dev;
    local.stream   = reinterpret_cast<cudaStream_t>(stream);
    local.d_status = d_status;
    local.num_sms  = g_num_sms[dev];
    tb200_ctx* ctx = &local;

    // the status word is shared by every call and keeps the last call's value: clear it first
    cudaError_t e = cudaMemsetAsync(d_status, 0, sizeof(int), local.stream);
    if (e != cudaSuccess)
    {
        set_err(err, err_len, cudaGetErrorString(e));
        return TB200_INTERNAL;
    }

    TcProblem q;
    memset(&q, 0, sizeof(q));
    q.in_dtype = TB200_INT8;
    q.a        = a;
    q.N = 1; q.IH = N; q.IW = H; q.IC = C;
    q.OH = N; q.OW = H; q.OC = W;
    q.KH = 1; q.KW = 1;
    q.stride_y = q.stride_x = q.dil_y = q.dil_x = 1;
    q.b          = b;
    q.b_mn_major = 1;
    q.out        = out;
    q.out_dtype  = TB200_INT32;
    q.epi        = TC_EPI_I32;
    tb200_status st = TB200_OK;
    std::string why;
    // the same choice of kernels as tb200_matmul: the CTA-pair kernel takes some shapes (K tails) the single-CTA one
    // does not
    if (tc_gemm_pair_supported(q, local.num_sms) || tc_gemm_supported(q, &why))
    {
        if (a_zp != 0 || b_zp != 0)
        {
            const int block     = 256;
            const int64_t items = std::max(rows * 32, cols);
            const int grid      = (int)std::max<int64_t>(1, std::min<int64_t>((items + block - 1) / block, (int64_t)local.num_sms * 16));
            noalloc_zp_sums_kernel<<<grid, block, 0, local.stream>>>(a, b, row_corr, col_corr, N, H, C, W, Wpad, a_zp, b_zp);
            q.row_corr     = row_corr;
            q.corr         = col_corr;
            q.corr_stride  = Wpad;
            q.corr_ystride = Wpad;
        }
        st = tc_gemm_launch(ctx, q);
    }
    else
    {
        const int block     = 256;
        const int64_t total = (int64_t)N * H * W;
        const int grid      = (int)std::max<int64_t>(1, std::min<int64_t>((total + block - 1) / block, (int64_t)local.num_sms * 16));
        noalloc_matmul_direct_kernel<<<grid, block, 0, local.stream>>>(a, b, out, N, H, C, W, a_zp, b_zp);
        st = post_launch(ctx, "matmul_direct");
    }
    if (st != TB200_OK)
    {
        set_err(err, err_len, local.err.c_str());
        return st;
    }
    if (synchronize)
    {
        int host_status = 0;
        e = cudaMemcpyAsync(&host_status, d_status, sizeof(int), cudaMemcpyDeviceToHost, local.stream);
        if (e == cudaSuccess)
            e = cudaStreamSynchronize(local.stream);
        if (e != cudaSuccess)
        {
            set_err(err, err_len, cudaGetErrorString(e));
            return TB200_INTERNAL;
        }
        if (host_status & TB200_DEV_TIMEOUT)
        {
            set_err(err, err_len, "tb200_matmul_i8_noalloc: the kernel gave up waiting on its pipeline");
            return TB200_INTERNAL;
        }
    }
    return TB200_OK;
}
