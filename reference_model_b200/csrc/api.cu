// C-ABI entry points of libtb200: context and tensor management, host-side validation that mirrors the
// reference's checkTensorAttributes / ERROR_IF rules, and dispatch to the kernels.
#include <algorithm>
#include <climits>
#include <cmath>
#include <cstdlib>
#include <new>

#include "common.h"
#include "kernels_cc.cuh"
#include "join_stream.cuh"

using namespace tb200;

namespace tb200
{

tb200_status raise_smem_limit(tb200_ctx* ctx, int bit, const void* kernel, int bytes)
{
    if (ctx->smem_attr_set & (1u << bit))
        return TB200_OK;
    // a context that knows its device's limit raises the kernel to it once; a bare one (the allocation-free entry
    // point's stack object) asks for what this launch needs, every time
    int want = bytes;
    if (ctx->max_smem_optin > 0)
    {
        // the device's opt-in limit covers static and dynamic shared memory together
        cudaFuncAttributes fa;
        TB200_CUDA_CHECK(ctx, cudaFuncGetAttributes(&fa, kernel));
        want = std::max(bytes, ctx->max_smem_optin - (int)fa.sharedSizeBytes);
    }
    TB200_CUDA_CHECK(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, want));
    if (ctx->max_smem_optin > 0)
        ctx->smem_attr_set |= 1u << bit;
    return TB200_OK;
}

tb200_status ensure_scratch(tb200_ctx* ctx, size_t bytes)
{
    if (bytes <= ctx->scratch_bytes)
        return TB200_OK;
    if (ctx->capturing)
        return fail(ctx, TB200_ERROR, "scratch memory would have to grow during capture; evaluate once eagerly first");
    // the old block may still be in use by kernels queued on the stream, or by a captured graph that recorded its
    // address: release_block waits for the former and parks the block while any graph is alive
    release_block(ctx, ctx->scratch);
    ctx->scratch       = nullptr;
    ctx->scratch_bytes = 0;
    size_t want        = std::max(bytes, (size_t)1 << 20);
    TB200_CUDA_CHECK(ctx, cudaMalloc(&ctx->scratch, want));
    ctx->scratch_bytes = want;
    return TB200_OK;
}

tb200_status post_launch(tb200_ctx* ctx, const char* kernel_name, int n_launches)
{
    ctx->launches += (uint64_t)n_launches;
    ctx->last_kernel = kernel_name;
    cudaError_t e    = cudaGetLastError();
    if (e != cudaSuccess)
        return fail(ctx, TB200_INTERNAL, "launch of %s failed: %s", kernel_name, cudaGetErrorString(e));
    return TB200_OK;
}

void timer_begin(tb200_ctx* ctx)
{
    if (!ctx->timing)
        return;
    cudaEvent_t a = nullptr, b = nullptr;
    if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess)
        return;
    cudaEventRecord(a, ctx->stream);
    ctx->timed.emplace_back(a, b);
}

void timer_end(tb200_ctx* ctx)
{
    if (!ctx->timing || ctx->timed.empty())
        return;
    cudaEventRecord(ctx->timed.back().second, ctx->stream);
}

static int grid_for(tb200_ctx* ctx, int64_t work_items, int block)
{
    int64_t blocks = (work_items + block - 1) / block;
    int64_t cap    = (int64_t)ctx->num_sms * 16;
    return (int)std::max<int64_t>(1, std::min(blocks, cap));
}

static bool all_contiguous(std::initializer_list<const tb200_tensor*> ts)
{
    for (const tb200_tensor* t : ts)
        if (t && !t->contiguous)
            return false;
    return true;
}

static bool same_shape(const tb200_tensor* a, const tb200_tensor* b)
{
    if (a->rank != b->rank)
        return false;
    for (int i = 0; i < a->rank; i++)
        if (a->shape[i] != b->shape[i])
            return false;
    return true;
}

static int dtype_bits(tb200_dtype d)
{
    return (int)dtype_size(d) * 8;
}

static bool is_int_dtype(tb200_dtype d)
{
    return d == TB200_INT8 || d == TB200_INT16 || d == TB200_INT32 || d == TB200_UINT8 || d == TB200_UINT16;
}

// Validates a RESCALE attribute the way OpRescale::checkTensorAttributes / eval do
// (reference_model/src/ops/type_conversion.cpp:71-154, :242-255) and fills the device descriptor.
static tb200_status make_rescale_dev(tb200_ctx* ctx, const tb200_rescale_attr* a, tb200_dtype in_dt, tb200_dtype out_dt,
                                     int channels, RescaleDev* r)
{
    TB200_ERROR_IF(ctx, !a || !a->multiplier || !a->shift, "OpRescale: missing multiplier / shift operand");
    TB200_ERROR_IF(ctx, !a->multiplier->contiguous || !a->shift->contiguous, "OpRescale: multiplier / shift must be contiguous");
    TB200_ERROR_IF(ctx, !is_int_dtype(in_dt) || !is_int_dtype(out_dt), "OpRescale: integer tensors only");
    TB200_ERROR_IF(ctx, a->rounding_mode < TB200_SINGLE_ROUND || a->rounding_mode > TB200_INEXACT_ROUND,
                   "OpRescale: only SINGLE_ROUND, DOUBLE_ROUND and INEXACT_ROUND are supported");
    TB200_ERROR_IF(ctx, !a->scale32 && a->rounding_mode == TB200_DOUBLE_ROUND,
                   "OpRescale: Scale set to false but double round set to true");
    TB200_ERROR_IF(ctx, a->input_unsigned && a->output_unsigned, "OpRescale: input and output cannot both be unsigned");
    const int in_bits = dtype_bits(in_dt), out_bits = dtype_bits(out_dt);
    TB200_ERROR_IF(ctx, (in_bits == 32 && a->input_unsigned) || (out_bits == 32 && a->output_unsigned),
                   "OpRescale: unsigned is not allowed with int32 tensors");
    TB200_ERROR_IF(ctx, a->multiplier->dtype != (a->scale32 ? TB200_INT32 : TB200_INT16),
                   "OpRescale: multiplier must be INT32 when scale32 else INT16");
    TB200_ERROR_IF(ctx, a->shift->dtype != TB200_INT8, "OpRescale: shift must be INT8");
    TB200_ERROR_IF(ctx, a->multiplier->rank != 1 || a->shift->rank != 1, "OpRescale: multiplier and shift must be rank 1");
    const int need = a->per_channel ? channels : 1;
    TB200_ERROR_IF(ctx, a->multiplier->shape[0] != need,
                   "OpRescale: multiplier size %d does not match %s (%d)", a->multiplier->shape[0],
                   a->per_channel ? "the channel count" : "per_channel=false", need);
    TB200_ERROR_IF(ctx, a->shift->shape[0] != need, "OpRescale: shift size %d does not match %s (%d)",
                   a->shift->shape[0], a->per_channel ? "the channel count" : "per_channel=false", need);
    const int64_t in_zp  = value_extend64_dev(a->input_zp, in_bits, a->input_unsigned != 0);
    const int64_t out_zp = value_extend64_dev(a->output_zp, out_bits, a->output_unsigned != 0);
    TB200_ERROR_IF(ctx, in_bits != 8 && !(in_bits == 16 && a->input_unsigned) && in_zp != 0,
                   "OpRescale: Input TOSA_REF_TYPE not INT8/UINT8/UINT16 and zero point not 0");
    TB200_ERROR_IF(ctx, out_bits != 8 && !(out_bits == 16 && a->output_unsigned) && out_zp != 0,
                   "OpRescale: Output TOSA_REF_TYPE not INT8/UINT8/UINT16 and zero point not 0");
    TB200_ERROR_IF(ctx, in_bits == 16 && a->input_unsigned && in_zp != 0 && in_zp != 32768,
                   "OpRescale: Input unsigned int16 and zero point not 0 or 32768");
    TB200_ERROR_IF(ctx, out_bits == 16 && a->output_unsigned && out_zp != 0 && out_zp != 32768,
                   "OpRescale: Output unsigned int16 and zero point not 0 or 32768");
    r->mult         = a->multiplier->data;
    r->shift        = reinterpret_cast<const int8_t*>(a->shift->data);
    r->mult_is_i16  = !a->scale32;
    r->per_channel  = a->per_channel;
    r->scale32      = a->scale32;
    r->rounding     = a->rounding_mode;
    r->in_zp_ext    = in_zp;
    r->out_zp_ext   = out_zp;
    r->in_bits      = in_bits;
    r->out_bits     = out_bits;
    r->in_unsigned  = a->input_unsigned;
    r->out_unsigned = a->output_unsigned;
    if (a->output_unsigned)
    {
        r->qmin = 0;
        r->qmax = out_bits == 8 ? 255 : 65535;
    }
    else
    {
        r->qmin = -((int64_t)1 << (out_bits - 1));
        r->qmax = ((int64_t)1 << (out_bits - 1)) - 1;
    }
    return TB200_OK;
}

// check_conv_attribute (reference_model/src/ops/tensor_ops.cpp:120-226)
static tb200_status check_conv_attr(tb200_ctx* ctx, const char* op, int IH, int IW, int OH, int OW, int KH, int KW,
                                    const int32_t* pad, const int32_t* stride, const int32_t* dilation)
{
    for (int i = 0; i < 4; i++)
        TB200_ERROR_IF(ctx, pad[i] < 0, "%s: At least one pad is smaller than zero", op);
    for (int i = 0; i < 2; i++)
        TB200_ERROR_IF(ctx, stride[i] < 1, "%s: At least one stride dimension is smaller than one", op);
    for (int i = 0; i < 2; i++)
        TB200_ERROR_IF(ctx, dilation[i] < 1, "%s: At least one dilation dimension is smaller than one", op);
    const int full_H = IH - 1 + pad[0] + pad[1] - (KH - 1) * dilation[0];
    const int full_W = IW - 1 + pad[2] + pad[3] - (KW - 1) * dilation[1];
    TB200_ERROR_IF(ctx, (full_H % stride[0] != 0) || (full_W % stride[1] != 0),
                   "%s: Parameters must yield exact integer output dimensions", op);
    TB200_ERROR_IF(ctx, (OH != full_H / stride[0] + 1) || (OW != full_W / stride[1] + 1),
                   "%s: Mismatch between output shape provided and expected output shape (%d,%d)", op,
                   full_H / stride[0] + 1, full_W / stride[1] + 1);
    return TB200_OK;
}

// check_pool2d_attribute (reference_model/src/ops/tensor_ops.cpp:28-117)
static tb200_status check_pool_attr(tb200_ctx* ctx, const char* op, int IH, int IW, int OH, int OW, const int32_t* kernel,
                                    const int32_t* pad, const int32_t* stride)
{
    for (int i = 0; i < 4; i++)
        TB200_ERROR_IF(ctx, pad[i] < 0, "%s: At least one pad is smaller than zero", op);
    for (int i = 0; i < 2; i++)
        TB200_ERROR_IF(ctx, kernel[i] < 1, "%s: At least one kernel dimension is smaller than one", op);
    for (int i = 0; i < 2; i++)
        TB200_ERROR_IF(ctx, stride[i] < 1, "%s: At least one stride dimension is smaller than one", op);
    TB200_ERROR_IF(ctx, pad[0] >= kernel[0] || pad[1] >= kernel[0] || pad[2] >= kernel[1] || pad[3] >= kernel[1],
                   "%s: At least one pad is >= kernel dimension", op);
    const int full_H = IH + pad[0] + pad[1] - kernel[0];
    const int full_W = IW + pad[2] + pad[3] - kernel[1];
    TB200_ERROR_IF(ctx, (full_H % stride[0] != 0) || (full_W % stride[1] != 0),
                   "%s: Parameters must yield exact integer output dimensions", op);
    TB200_ERROR_IF(ctx, (OH != full_H / stride[0] + 1) || (OW != full_W / stride[1] + 1),
                   "%s: Mismatch between output shape provided and expected output shape (%d,%d)", op,
                   full_H / stride[0] + 1, full_W / stride[1] + 1);
    return TB200_OK;
}

struct EpiInfo
{
    bool has_rescale = false;
    bool has_clamp   = false;
    RescaleDev rs;
    int32_t clamp_lo = 0, clamp_hi = 0;
    float clamp_lo_f = 0.f, clamp_hi_f = 0.f;
};

static tb200_status parse_epilogue(tb200_ctx* ctx, const char* op, const tb200_epilogue* e, bool int_path, int channels,
                                   tb200_dtype out_dt, EpiInfo* info)
{
    memset(&info->rs, 0, sizeof(info->rs));
    if (!e)
    {
        TB200_ERROR_IF(ctx, int_path && out_dt != TB200_INT32, "%s: integer accumulator output must be INT32", op);
        return TB200_OK;
    }
    if (e->has_rescale)
    {
        TB200_ERROR_IF(ctx, !int_path, "%s: a RESCALE epilogue needs an integer accumulator", op);
        tb200_status st = make_rescale_dev(ctx, &e->rescale, TB200_INT32, out_dt, channels, &info->rs);
        if (st != TB200_OK)
            return st;
        info->has_rescale = true;
    }
    else
        TB200_ERROR_IF(ctx, int_path && out_dt != TB200_INT32, "%s: integer accumulator output must be INT32", op);
    if (e->has_clamp)
    {
        TB200_ERROR_IF(ctx, int_path && !e->has_rescale, "%s: CLAMP is not defined on INT32 tensors", op);
        if (int_path)
        {
            TB200_ERROR_IF(ctx, e->clamp_max_i < e->clamp_min_i, "OpClamp: max smaller than min");
            info->clamp_lo = e->clamp_min_i;
            info->clamp_hi = e->clamp_max_i;
        }
        else
        {
            TB200_ERROR_IF(ctx, std::isnan(e->clamp_min_f) || std::isnan(e->clamp_max_f), "OpClamp: min/max cannot be NaN");
            TB200_ERROR_IF(ctx, e->clamp_max_f < e->clamp_min_f, "OpClamp: max smaller than min");
            info->clamp_lo_f = e->clamp_min_f;
            info->clamp_hi_f = e->clamp_max_f;
        }
        info->has_clamp = true;
    }
    return TB200_OK;
}

static void fill_conv_dev(ConvDev* d, const EpiInfo& e)
{
    d->has_rescale = e.has_rescale;
    d->rs          = e.rs;
    d->has_clamp   = e.has_clamp;
    d->clamp_lo    = e.clamp_lo;
    d->clamp_hi    = e.clamp_hi;
    d->clamp_lo_f  = e.clamp_lo_f;
    d->clamp_hi_f  = e.clamp_hi_f;
}

// Tensor-core epilogue fields shared by conv and matmul.
static void fill_tc_epilogue(TcProblem* q, const EpiInfo& e, tb200_dtype out_dt)
{
    q->out_dtype = out_dt;
    q->has_clamp = e.has_clamp;
    if (e.has_rescale)
    {
        q->epi          = TC_EPI_RESCALE;
        q->double_round = e.rs.rounding == TB200_DOUBLE_ROUND;
        q->out_zp       = (int32_t)e.rs.out_zp_ext;
        int64_t lo = e.rs.qmin, hi = e.rs.qmax;
        if (e.has_clamp)
        {
            // clip to [qmin, qmax] followed by CLAMP [cmin, cmax] is one clip to [L, H]
            lo = std::min<int64_t>(std::max<int64_t>(e.rs.qmin, e.clamp_lo), e.clamp_hi);
            hi = std::min<int64_t>(std::max<int64_t>(e.rs.qmax, e.clamp_lo), e.clamp_hi);
        }
        q->clamp_lo = (int32_t)lo;
        q->clamp_hi = (int32_t)hi;
    }
    q->clamp_lo_f = e.clamp_lo_f;
    q->clamp_hi_f = e.clamp_hi_f;
}

}    // namespace tb200

// =================================================================================================== context
extern "C" tb200_status tb200_ctx_create(int device, void* stream, tb200_ctx** out)
{
    if (!out)
        return TB200_ERROR;
    *out          = nullptr;
    tb200_ctx* c  = new (std::nothrow) tb200_ctx();
    if (!c)
        return TB200_INTERNAL;
    c->device = device;
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess)
    {
        fprintf(stderr, "tb200_ctx_create: cudaSetDevice(%d) failed: %s\n", device, cudaGetErrorString(e));
        delete c;
        return TB200_INTERNAL;
    }
    if (stream)
        c->stream = reinterpret_cast<cudaStream_t>(stream);
    else
    {
        if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess)
        {
            delete c;
            return TB200_INTERNAL;
        }
        c->owns_stream = true;
    }
    int attr_val = 0;
    if (cudaDeviceGetAttribute(&attr_val, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && attr_val > 0)
        c->num_sms = attr_val;
    if (cudaDeviceGetAttribute(&attr_val, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) == cudaSuccess && attr_val > 0)
        c->max_smem_optin = attr_val;
    if (cudaMalloc(&c->d_status, sizeof(int)) != cudaSuccess || cudaMallocHost(&c->h_status, sizeof(int)) != cudaSuccess ||
        cudaMemsetAsync(c->d_status, 0, sizeof(int), c->stream) != cudaSuccess)
    {
        fprintf(stderr, "tb200_ctx_create: status word allocation failed: %s\n", cudaGetErrorString(cudaGetLastError()));
        delete c;
        return TB200_INTERNAL;
    }
    c->policy = diag_env_int("TB200_KERNEL_POLICY", 0);
    *out = c;
    return TB200_OK;
}

extern "C" tb200_status tb200_ctx_destroy(tb200_ctx* ctx)
{
    if (!ctx)
        return TB200_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    tb200_comm_destroy(ctx);
    for (auto& e : ctx->prepared)
        if (e->block)
            cudaFree(e->block);
    ctx->prepared.clear();
    for (void* b : ctx->retired)
        cudaFree(b);
    ctx->retired.clear();
    if (ctx->scratch)
        cudaFree(ctx->scratch);
    if (ctx->stage)
        cudaFree(ctx->stage);
    if (ctx->io_pinned)
        cudaFreeHost(ctx->io_pinned);
    if (ctx->join_table)
        cudaFree(ctx->join_table);
    if (ctx->pair_flags)
        cudaFree(ctx->pair_flags);
    if (ctx->pipe.ready)
    {
        cudaStreamSynchronize(ctx->pipe.h2d);
        cudaStreamSynchronize(ctx->pipe.d2h);
        for (int i = 0; i < 2; i++)
        {
            if (ctx->pipe.buf[i])
                cudaFree(ctx->pipe.buf[i]);
            cudaEventDestroy(ctx->pipe.up[i]);
            cudaEventDestroy(ctx->pipe.done[i]);
            cudaEventDestroy(ctx->pipe.down[i]);
        }
        cudaStreamDestroy(ctx->pipe.h2d);
        cudaStreamDestroy(ctx->pipe.d2h);
    }
    if (ctx->d_status)
        cudaFree(ctx->d_status);
    if (ctx->h_status)
        cudaFreeHost(ctx->h_status);
    if (ctx->owns_stream)
        cudaStreamDestroy(ctx->stream);
    delete ctx;
    return TB200_OK;
}

extern "C" const char* tb200_last_error(const tb200_ctx* ctx)
{
    return ctx ? ctx->err.c_str() : "null context";
}

extern "C" uint64_t tb200_launch_count(const tb200_ctx* ctx)
{
    return ctx ? ctx->launches : 0;
}

extern "C" tb200_status tb200_timer_enable(tb200_ctx* ctx, int32_t on)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    ctx->timing = on != 0;
    return TB200_OK;
}

extern "C" tb200_status tb200_timer_read(tb200_ctx* ctx, double* total_ms, int32_t* launches)
{
    if (!ctx || !total_ms || !launches)
        return TB200_ERROR;
    TB200_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    double sum = 0.0;
    int n      = 0;
    for (auto& pr : ctx->timed)
    {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, pr.first, pr.second) == cudaSuccess)
        {
            sum += ms;
            n++;
        }
        cudaEventDestroy(pr.first);
        cudaEventDestroy(pr.second);
    }
    ctx->timed.clear();
    *total_ms = sum;
    *launches = n;
    return TB200_OK;
}

extern "C" tb200_status tb200_capture_begin(tb200_ctx* ctx)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, ctx->capturing, "capture already in progress");
    TB200_ERROR_IF(ctx, ctx->timing, "disable the kernel timer before capturing");
    TB200_CUDA_CHECK(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    ctx->capturing = true;
    return TB200_OK;
}

extern "C" tb200_status tb200_capture_end(tb200_ctx* ctx, tb200_graph** out)
{
    if (!ctx || !out)
        return TB200_ERROR;
    *out = nullptr;
    TB200_ERROR_IF(ctx, !ctx->capturing, "no capture in progress");
    ctx->capturing   = false;
    cudaGraph_t g    = nullptr;
    cudaError_t e    = cudaStreamEndCapture(ctx->stream, &g);
    if (e != cudaSuccess || !g)
        return fail(ctx, TB200_INTERNAL, "cudaStreamEndCapture failed: %s", cudaGetErrorString(e));
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, g, 0);
    if (e != cudaSuccess)
    {
        cudaGraphDestroy(g);
        return fail(ctx, TB200_INTERNAL, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
    }
    tb200_graph* tg = new (std::nothrow) tb200_graph();
    if (!tg)
    {
        cudaGraphExecDestroy(exec);
        cudaGraphDestroy(g);
        return fail(ctx, TB200_INTERNAL, "out of host memory");
    }
    tg->graph = g;
    tg->exec  = exec;
    ctx->live_graphs++;
    size_t n  = 0;
    if (cudaGraphGetNodes(g, nullptr, &n) == cudaSuccess)
        tg->launches = n;
    *out = tg;
    return TB200_OK;
}

extern "C" tb200_status tb200_graph_launch(tb200_ctx* ctx, tb200_graph* graph)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !graph || !graph->exec, "null graph");
    TB200_ERROR_IF(ctx, ctx->capturing, "a captured graph cannot be launched while capturing");
    TB200_CUDA_CHECK(ctx, cudaGraphLaunch(graph->exec, ctx->stream));
    ctx->launches += graph->launches;
    ctx->last_kernel = "cuda_graph_replay";
    return TB200_OK;
}

extern "C" tb200_status tb200_graph_destroy(tb200_ctx* ctx, tb200_graph* graph)
{
    if (!graph)
        return TB200_OK;
    if (ctx)
        cudaStreamSynchronize(ctx->stream);
    if (graph->exec)
        cudaGraphExecDestroy(graph->exec);
    if (graph->graph)
        cudaGraphDestroy(graph->graph);
    delete graph;
    if (ctx && ctx->live_graphs > 0 && --ctx->live_graphs == 0)
    {
        // no graph can hold the parked blocks' addresses any more
        for (void* b : ctx->retired)
            cudaFree(b);
        ctx->retired.clear();
    }
    return TB200_OK;
}

extern "C" int tb200_set_kernel_policy(tb200_ctx* ctx, int policy)
{
    int old     = ctx->policy;
    ctx->policy = policy;
    return old;
}

extern "C" tb200_status tb200_set_wait_limit(tb200_ctx* ctx, uint64_t sm_cycles)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, sm_cycles == 0 || sm_cycles > (uint64_t)1 << 62, "wait limit out of range");
    ctx->wait_limit_cycles = (long long)sm_cycles;
    return TB200_OK;
}

extern "C" tb200_status tb200_set_shared_gpu(tb200_ctx* ctx, int32_t shared)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    ctx->shared_gpu = shared != 0;
    return TB200_OK;
}

extern "C" tb200_status tb200_set_launch_overlap(tb200_ctx* ctx, int32_t on)
{
    if (!ctx)
        return TB200_ERROR;
    ctx->launch_overlap = on ? 1 : 0;
    return TB200_OK;
}

extern "C" tb200_status tb200_const_cache_control(tb200_ctx* ctx, int32_t action)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    switch (action)
    {
        case TB200_CACHE_OFF:
            cache_clear(ctx);
            ctx->const_cache_on = false;
            return TB200_OK;
        case TB200_CACHE_ON:
            ctx->const_cache_on = true;
            return TB200_OK;
        case TB200_CACHE_CLEAR:
            cache_clear(ctx);
            return TB200_OK;
    }
    return fail(ctx, TB200_ERROR, "unknown cache action %d", (int)action);
}

extern "C" int32_t tb200_const_cache_entries(const tb200_ctx* ctx)
{
    return ctx ? (int32_t)ctx->prepared.size() : 0;
}

extern "C" const char* tb200_last_kernel(const tb200_ctx* ctx)
{
    return ctx ? ctx->last_kernel : "none";
}

extern "C" tb200_status tb200_sync(tb200_ctx* ctx)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, ctx->capturing, "tb200_sync is not allowed while capturing");
    TB200_CUDA_CHECK(ctx, cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    TB200_CUDA_CHECK(ctx, cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream));
    TB200_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    const int s = *ctx->h_status;
    if (s & TB200_DEV_TIMEOUT)
        return fail(ctx, TB200_INTERNAL, "a kernel gave up waiting on its pipeline (device status 0x%x)", s);
    if (s & TB200_DEV_UNPREDICTABLE)
        return fail(ctx, TB200_UNPREDICTABLE, "a REQUIRE condition failed on the device (RESCALE range / ADD overflow)");
    return TB200_OK;
}

// =================================================================================================== tensors
static tb200_status make_tensor(tb200_ctx* ctx, tb200_dtype dtype, int rank, const int32_t* shape, void* ptr, bool owns,
                                tb200_tensor** out)
{
    TB200_ERROR_IF(ctx, !out, "null output handle");
    *out = nullptr;
    TB200_ERROR_IF(ctx, rank < 0 || rank > 6, "tensor rank %d out of range", rank);
    TB200_ERROR_IF(ctx, dtype_size(dtype) == 0, "unsupported dtype %d", (int)dtype);
    int64_t n = 1;
    for (int i = 0; i < rank; i++)
    {
        TB200_ERROR_IF(ctx, shape[i] < 0, "negative dimension");
        n *= shape[i];
        // the reference caps tensors at 2^31-1 elements (reference_model/src/subgraph_traverser.cpp:583-598)
        TB200_ERROR_IF(ctx, n > 2147483647LL, "tensor exceeds 2^31-1 elements");
    }
    tb200_tensor* t = new (std::nothrow) tb200_tensor();
    if (!t)
        return fail(ctx, TB200_INTERNAL, "out of host memory");
    t->dtype = dtype;
    t->rank  = rank;
    for (int i = 0; i < 6; i++)
        t->shape[i] = i < rank ? shape[i] : 1;
    t->bytes = (size_t)n * dtype_size(dtype);
    t->owns  = owns;
    t->data  = ptr;
    int64_t st = 1;
    for (int i = 5; i >= 0; i--)
    {
        t->stride[i] = st;
        st *= t->shape[i];
    }
    // shape[] is padded with ones after `rank`, so the loop above yields row-major strides for the first `rank` dims
    t->contiguous = true;
    if (owns)
    {
        cudaError_t e = cudaMalloc(&t->data, std::max<size_t>(t->bytes, 16));
        if (e != cudaSuccess)
        {
            delete t;
            return fail(ctx, TB200_INTERNAL, "cudaMalloc of %zu bytes failed: %s", t->bytes, cudaGetErrorString(e));
        }
    }
    *out = t;
    return TB200_OK;
}

extern "C" tb200_status tb200_tensor_alloc(tb200_ctx* ctx, tb200_dtype dtype, int rank, const int32_t* shape,
                                           tb200_tensor** out)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    return make_tensor(ctx, dtype, rank, shape, nullptr, true, out);
}

extern "C" tb200_status tb200_tensor_wrap(tb200_ctx* ctx, tb200_dtype dtype, int rank, const int32_t* shape,
                                          void* device_ptr, tb200_tensor** out)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !device_ptr, "null device pointer");
    TB200_ERROR_IF(ctx, (reinterpret_cast<uintptr_t>(device_ptr) & 15) != 0, "device pointer must be 16-byte aligned");
    return make_tensor(ctx, dtype, rank, shape, device_ptr, false, out);
}

extern "C" tb200_status tb200_tensor_free(tb200_ctx* ctx, tb200_tensor* t)
{
    if (!t)
        return TB200_OK;
    if (ctx && t->data)
        cache_note_free(ctx, t->data, std::max<size_t>(t->bytes, 1));
    if (t->owns && t->data)
    {
        if (ctx)
            cudaStreamSynchronize(ctx->stream);
        cudaFree(t->data);
    }
    delete t;
    return TB200_OK;
}

extern "C" tb200_status tb200_tensor_upload(tb200_ctx* ctx, tb200_tensor* t, const void* host, size_t bytes)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !t || !host, "null tensor or host buffer");
    TB200_ERROR_IF(ctx, !t->contiguous, "upload needs a contiguous tensor");
    TB200_ERROR_IF(ctx, ctx->capturing, "uploads are not allowed while capturing");
    TB200_ERROR_IF(ctx, bytes != t->bytes, "upload of %zu bytes into a tensor of %zu bytes", bytes, t->bytes);
    if (bytes)
    {
        TB200_CUDA_CHECK(ctx, cudaMemcpyAsync(t->data, host, bytes, cudaMemcpyHostToDevice, ctx->stream));
        // tables derived from this tensor (it may be a weight, bias, multiplier or shift) follow the new contents
        return cache_note_upload(ctx, t->data, bytes);
    }
    return TB200_OK;
}

extern "C" tb200_status tb200_tensor_download(tb200_ctx* ctx, const tb200_tensor* t, void* host, size_t bytes)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !t || !host, "null tensor or host buffer");
    TB200_ERROR_IF(ctx, !t->contiguous, "download needs a contiguous tensor");
    TB200_ERROR_IF(ctx, ctx->capturing, "downloads are not allowed while capturing");
    TB200_ERROR_IF(ctx, bytes != t->bytes, "download of %zu bytes from a tensor of %zu bytes", bytes, t->bytes);
    if (bytes)
        TB200_CUDA_CHECK(ctx, cudaMemcpyAsync(host, t->data, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return tb200_sync(ctx);
}

extern "C" void* tb200_tensor_data(const tb200_tensor* t)
{
    return t ? t->data : nullptr;
}

extern "C" size_t tb200_tensor_bytes(const tb200_tensor* t)
{
    return t ? t->bytes : 0;
}

// SLICE as a zero-copy view (OpSlice::eval, reference_model/src/ops/data_layout.cpp:369-398): same ERROR_IFs, the
// view keeps the parent's pitch.  Views are accepted as the input of tb200_conv2d; other operators need contiguous
// tensors and report TB200_ERROR for a view.
extern "C" tb200_status tb200_tensor_slice(tb200_ctx* ctx, const tb200_tensor* parent, const int32_t* start,
                                           const int32_t* size, tb200_tensor** out)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !parent || !start || !size || !out, "OpSlice: null operand");
    *out = nullptr;
    int64_t offset = 0, n = 1;
    for (int i = 0; i < parent->rank; i++)
    {
        const int32_t b = start[i], sz = size[i];
        TB200_ERROR_IF(ctx, b < 0 || b >= parent->shape[i], "OpSlice: start out of boundary");
        TB200_ERROR_IF(ctx, (b + sz) < 0 || (b + sz) > parent->shape[i], "OpSlice: (start+size) out of boundary");
        TB200_ERROR_IF(ctx, sz <= 0, "OpSlice: output must be positive");
        offset += (int64_t)b * parent->stride[i];
        n *= sz;
    }
    const size_t es = dtype_size(parent->dtype);
    TB200_ERROR_IF(ctx, ((offset * (int64_t)es) & 15) != 0, "OpSlice: a zero-copy view must start on a 16-byte boundary");
    tb200_tensor* t = new (std::nothrow) tb200_tensor(*parent);
    if (!t)
        return fail(ctx, TB200_INTERNAL, "out of host memory");
    t->owns = false;
    t->data = reinterpret_cast<uint8_t*>(parent->data) + offset * (int64_t)es;
    bool contig = parent->contiguous;
    for (int i = 0; i < parent->rank; i++)
    {
        if (size[i] != parent->shape[i] && i != 0)
            contig = false;    // anything but a cut along the outermost dimension leaves gaps
        t->shape[i] = size[i];
    }
    t->bytes      = (size_t)n * es;
    t->contiguous = contig;
    *out          = t;
    return TB200_OK;
}

// RESHAPE as a zero-copy view of a contiguous tensor (OpReshape::eval, reference_model/src/ops/data_layout.cpp:227-):
// element counts must match.
extern "C" tb200_status tb200_tensor_reshape(tb200_ctx* ctx, const tb200_tensor* parent, int rank, const int32_t* shape,
                                             tb200_tensor** out)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !parent || !shape || !out, "OpReshape: null operand");
    TB200_ERROR_IF(ctx, !parent->contiguous, "OpReshape: a zero-copy reshape needs a contiguous tensor");
    int64_t n = 1;
    for (int i = 0; i < rank; i++)
        n *= shape[i];
    TB200_ERROR_IF(ctx, rank < 0 || rank > 6 || n != numel(parent), "OpReshape: input and output element counts differ");
    return make_tensor(ctx, parent->dtype, rank, shape, parent->data, false, out);
}

// =================================================================================================== CONV2D
// One phase of a TRANSPOSE_CONV2D writes its [N][OH][OW] pixel grid into a strided subset of the output tensor:
// pixel (oy, ox) lands at (oy * sy + y0, ox * sx + x0).  Only the tensor-core kernel takes such a view; conv2d_impl
// answers kNeedsDenseOutput (before launching anything) when the problem would go to another kernel.
struct ConvOutView
{
    int OH, OW, sy, sx, y0, x0;
    // d2s_oc != 0: the weight rows are (ky, kx, oc) blocks of d2s_oc channels and block (ky, kx) of pixel (oy, ox)
    // lands at (oy * sy + ky, ox * sx + kx); d2s_kw is the stamp's width
    int d2s_oc, d2s_kw;
};
static const tb200_status kNeedsDenseOutput = (tb200_status)-77;

// The word a builder left at `offset` of a cache entry's block (e.g. "every column's lean RESCALE record is usable"),
// read back once per build: a copy and a stream synchronisation at the first use of the entry, nothing afterwards.
// An entry that is rebuilt on every use, or that is first met while capturing, stays unread: the caller then takes
// the path that needs no verdict.
static tb200_status read_host_flag(tb200_ctx* ctx, Prepared* e, size_t offset)
{
    if (e->host_flag >= 0 || e->unstable || ctx->capturing || !e->valid)
        return TB200_OK;
    TB200_CUDA_CHECK(ctx, cudaMemcpyAsync(ctx->h_status, reinterpret_cast<const uint8_t*>(e->block) + offset, sizeof(int),
                                          cudaMemcpyDeviceToHost, ctx->stream));
    TB200_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    e->host_flag = *ctx->h_status != 0 ? 1 : 0;
    return TB200_OK;
}

static tb200_status conv2d_impl(tb200_ctx* ctx, const tb200_tensor* input, const tb200_tensor* weight,
                                const tb200_tensor* bias, int32_t input_zp, int32_t weight_zp, const int32_t pad[4],
                                const int32_t stride[2], const int32_t dilation[2], const tb200_epilogue* epilogue,
                                tb200_tensor* output, const ConvOutView* view, bool dry_run, bool use_cache)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !input || !weight || !bias || !output || !pad || !stride || !dilation, "OpConv2d: null operand");
    TB200_ERROR_IF(ctx, !all_contiguous({ weight, bias, output }), "%s: zero-copy views are accepted only as the CONV2D input; this operand must be contiguous", "OpConv2d");
    // OpConv2d::checkTensorAttributes (reference_model/src/ops/tensor_ops.cpp:690-720)
    TB200_ERROR_IF(ctx, input->rank != 4 || weight->rank != 4 || output->rank != 4 || bias->rank != 1,
                   "OpConv2d: input, weight and output must be rank 4 and bias rank 1");
    const int N = input->shape[0], IH = input->shape[1], IW = input->shape[2], IC = input->shape[3];
    const int OC = weight->shape[0], KH = weight->shape[1], KW = weight->shape[2];
    const int OH = view ? view->OH : output->shape[1], OW = view ? view->OW : output->shape[2];
    tb200_status st = check_conv_attr(ctx, "OpConv2d", IH, IW, OH, OW, KH, KW, pad, stride, dilation);
    if (st != TB200_OK)
        return st;
    // OpConv2d::eval ERROR_IFs (:742-748)
    TB200_ERROR_IF(ctx, N != output->shape[0], "OpConv2d: tensor batch mismatch %d != %d", N, output->shape[0]);
    TB200_ERROR_IF(ctx, weight->shape[3] != IC, "OpConv2d: tensor input channel mismatch %d != %d", weight->shape[3], IC);
    TB200_ERROR_IF(ctx, OC != output->shape[3] && !(view && view->d2s_oc), "OpConv2d: tensor output channel mismatch %d != %d",
                   OC, output->shape[3]);
    TB200_ERROR_IF(ctx, bias->shape[0] != OC && bias->shape[0] != 1, "OpConv2d: bias channel mismatch %d != %d",
                   bias->shape[0], OC);
    const bool int_path = input->dtype == TB200_INT8;
    TB200_ERROR_IF(ctx, weight->dtype != input->dtype, "OpConv2d: input and weight dtypes differ");
    if (int_path)
        TB200_ERROR_IF(ctx, bias->dtype != TB200_INT32, "OpConv2d: INT8 convolution needs an INT32 bias");
    else
    {
        TB200_ERROR_IF(ctx, !dtype_is_float(input->dtype) && !dtype_is_fp8(input->dtype), "OpConv2d: unsupported input dtype %d",
                       (int)input->dtype);
        if (dtype_is_fp8(input->dtype))    // <FP8, FP8, FP16, FP16>, reference_model/src/ops/tensor_ops.cpp:2228-2229
            TB200_ERROR_IF(ctx, bias->dtype != TB200_FP16 || output->dtype != TB200_FP16,
                           "OpConv2d: an FP8 convolution has an FP16 bias and output");
        else
            TB200_ERROR_IF(ctx, bias->dtype != input->dtype || output->dtype != input->dtype,
                           "OpConv2d: floating bias and output must have the input dtype");
        // :805,811
        TB200_ERROR_IF(ctx, input_zp != 0, "Input zero point must be zero for non int8_t data");
        TB200_ERROR_IF(ctx, weight_zp != 0, "Weight zero point must be zero for non int8_t data");
    }
    TB200_ERROR_IF(ctx, input_zp < -128 || input_zp > 127 || weight_zp < -128 || weight_zp > 127,
                   "OpConv2d: zero point outside the int8 range");
    EpiInfo epi;
    st = parse_epilogue(ctx, "OpConv2d", epilogue, int_path, OC, output->dtype, &epi);
    if (st != TB200_OK)
        return st;
    if (numel(output) == 0)
        return TB200_OK;
    if (!dry_run)
        cache_note_write(ctx, output->data, output->bytes);

    // ---- tensor-core path
    const bool tc_rescale_ok = !epi.has_rescale || (epi.rs.scale32 && epi.rs.rounding != TB200_INEXACT_ROUND &&
                                                    !epi.rs.out_unsigned);
    if (ctx->policy == 0 && (!int_path || weight_zp == 0) && tc_rescale_ok &&
        (int_path || input->dtype != TB200_FP32))
    {
        TcProblem q;
        memset(&q, 0, sizeof(q));
        q.in_dtype = input->dtype;
        q.a        = input->data;
        q.N = N; q.IH = IH; q.IW = IW; q.IC = IC;
        q.a_stride_w = input->stride[2]; q.a_stride_h = input->stride[1]; q.a_stride_n = input->stride[0];
        q.OH = OH; q.OW = OW; q.OC = OC;
        q.KH = KH; q.KW = KW;
        q.pad_t = pad[0]; q.pad_l = pad[2];
        q.stride_y = stride[0]; q.stride_x = stride[1];
        q.dil_y = dilation[0]; q.dil_x = dilation[1];
        q.b   = weight->data;
        q.out = output->data;
        if (view)
        {
            q.out_OH = output->shape[1]; q.out_OW = output->shape[2];
            q.out_sy = view->sy; q.out_sx = view->sx; q.out_y0 = view->y0; q.out_x0 = view->x0;
            q.d2s_oc = view->d2s_oc; q.d2s_kw = view->d2s_kw;
        }
        q.epi = int_path ? TC_EPI_I32 : TC_EPI_FLOAT;
        fill_tc_epilogue(&q, epi, output->dtype);
        std::string why;
        if (tc_gemm_supported(q, &why))
        {
            const int OCpad = (OC + 255) / 256 * 256;
            if (dry_run && !int_path)
                return TB200_OK;
            if (int_path)
            {
                const bool padded  = pad[0] || pad[1] || pad[2] || pad[3];
                const bool classes = input_zp != 0 && padded;
                const size_t ncls  = classes ? (size_t)(KH + 1) * (KH + 1) * (KW + 1) * (KW + 1) : 1;
                // block: prefix | corr | mult_pad | shift_pad
                // block: prefix | corr | mult_pad | shift_pad | records of the lean RESCALE form | border deltas
                const size_t prefix_elems = ((size_t)(KH + 1) * (KW + 1) * OC + 3) & ~(size_t)3;
                const size_t corr_elems   = ncls * OCpad;
                const size_t rec_off      = ((prefix_elems + corr_elems + OCpad) * sizeof(int32_t) + OCpad + 63) & ~(size_t)63;
                const bool want_rec       = epi.has_rescale;
                const size_t delta_off    = rec_off + (want_rec ? (size_t)OCpad * 8 * sizeof(int32_t) : 0);
                const size_t flag_off     = delta_off + ((want_rec && classes) ? corr_elems * sizeof(int32_t) : 0);
                const size_t bytes        = flag_off + 64;
                if (bytes <= ((size_t)64 << 20))
                {
                    if (dry_run)
                        return TB200_OK;
                    const int8_t* wp   = reinterpret_cast<const int8_t*>(weight->data);
                    const int32_t* bp  = reinterpret_cast<const int32_t*>(bias->data);
                    const int32_t* mp  = epi.has_rescale ? reinterpret_cast<const int32_t*>(epi.rs.mult) : nullptr;
                    const int8_t* sp   = epi.has_rescale ? epi.rs.shift : nullptr;
                    const int bias_n = bias->shape[0], per_ch = epi.rs.per_channel, has_rs = epi.has_rescale ? 1 : 0;
                    const int cls_i = classes ? 1 : 0;
                    const int dr_i  = epi.has_rescale && epi.rs.rounding == TB200_DOUBLE_ROUND ? 1 : 0;
                    const int32_t ozp_i = epi.has_rescale ? (int32_t)epi.rs.out_zp_ext : 0;
                    auto build = [=](tb200_ctx* c, void* block) -> tb200_status {
                        int32_t* prefix   = reinterpret_cast<int32_t*>(block);
                        int32_t* corr     = prefix + prefix_elems;
                        int32_t* mult_pad = corr + corr_elems;
                        int8_t* shift_pad = reinterpret_cast<int8_t*>(mult_pad + OCpad);
                        int32_t* rec      = want_rec ? reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(block) + rec_off) : nullptr;
                        int32_t* delta    = (want_rec && cls_i) ? reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(block) + delta_off) : nullptr;
                        int* all_ok       = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(block) + flag_off);
                        TB200_CUDA_CHECK(c, cudaMemsetAsync(all_ok, want_rec ? 1 : 0, sizeof(int), c->stream));
                        conv_epilogue_tables_kernel<<<(OCpad * 32 + 127) / 128, 128, 0, c->stream>>>(
                            wp, bp, bias_n, OC, OCpad, KH, KW, IC, input_zp, cls_i, mp, sp, per_ch, prefix, corr,
                            has_rs ? mult_pad : nullptr, shift_pad, rec, delta, dr_i, ozp_i, all_ok);
                        return post_launch(c, "conv_epilogue_tables");
                    };
                    void* block = nullptr;
                    Prepared* e = nullptr;
                    if (use_cache && ctx->const_cache_on)
                    {
                        std::string key;
                        key_add(&key, (int)0);
                        key_add(&key, wp); key_add(&key, bp); key_add(&key, mp); key_add(&key, sp);
                        key_add(&key, OC); key_add(&key, KH); key_add(&key, KW); key_add(&key, IC); key_add(&key, bias_n);
                        key_add(&key, input_zp); key_add(&key, per_ch); key_add(&key, has_rs); key_add(&key, cls_i);
                        key_add(&key, dr_i); key_add(&key, ozp_i);
                        e = cache_find(ctx, key);
                        if (!e)
                        {
                            std::vector<std::pair<const char*, size_t>> ops = {
                                { reinterpret_cast<const char*>(wp), weight->bytes }, { reinterpret_cast<const char*>(bp), bias->bytes } };
                            if (has_rs)
                            {
                                ops.push_back({ reinterpret_cast<const char*>(mp), epilogue->rescale.multiplier->bytes });
                                ops.push_back({ reinterpret_cast<const char*>(sp), epilogue->rescale.shift->bytes });
                            }
                            e = cache_insert(ctx, key, std::move(ops), bytes, build);
                        }
                    }
                    bool lean_ok = false;
                    if (e)
                    {
                        st = cache_use(ctx, e);
                        if (st != TB200_OK)
                            return st;
                        block = e->block;
                        st    = read_host_flag(ctx, e, flag_off);
                        if (st != TB200_OK)
                            return st;
                        lean_ok = e->host_flag == 1;
                    }
                    else
                    {
                        st = ensure_scratch(ctx, bytes);
                        if (st != TB200_OK)
                            return st;
                        st = build(ctx, ctx->scratch);
                        if (st != TB200_OK)
                            return st;
                        block = ctx->scratch;
                    }
                    q.lean_ok         = lean_ok ? 1 : 0;
                    int32_t* corr     = reinterpret_cast<int32_t*>(block) + prefix_elems;
                    int32_t* mult_pad = corr + corr_elems;
                    q.corr         = corr;
                    q.corr_stride  = OCpad;
                    q.corr_classes = cls_i;
                    q.mult_pad     = mult_pad;
                    q.shift_pad    = reinterpret_cast<int8_t*>(mult_pad + OCpad);
                    // the lean form packs with int8 saturation: it serves RESCALEs to signed int8 only
                    const bool lean_out = want_rec && output->dtype == TB200_INT8 && !epi.rs.out_unsigned;
                    q.rec   = lean_out ? reinterpret_cast<const int32_t*>(reinterpret_cast<const uint8_t*>(block) + rec_off) : nullptr;
                    q.delta = (lean_out && classes)
                                  ? reinterpret_cast<const int32_t*>(reinterpret_cast<const uint8_t*>(block) + delta_off)
                                  : nullptr;
                    return tc_gemm_launch(ctx, q);
                }
            }
            else
            {
                const void* bp   = bias->data;
                const int bias_n = bias->shape[0];
                const bool b16   = bias->dtype == TB200_FP16;
                auto build = [=](tb200_ctx* c, void* block) -> tb200_status {
                    float* bf = reinterpret_cast<float*>(block);
                    if (b16)
                        bias_to_f32_kernel<__half><<<(OCpad + 127) / 128, 128, 0, c->stream>>>(
                            reinterpret_cast<const __half*>(bp), bias_n, OC, bf, OCpad);
                    else
                        bias_to_f32_kernel<__nv_bfloat16><<<(OCpad + 127) / 128, 128, 0, c->stream>>>(
                            reinterpret_cast<const __nv_bfloat16*>(bp), bias_n, OC, bf, OCpad);
                    return post_launch(c, "bias_to_f32");
                };
                Prepared* e = nullptr;
                if (use_cache && ctx->const_cache_on)
                {
                    std::string key;
                    key_add(&key, (int)2);
                    key_add(&key, bp); key_add(&key, bias_n); key_add(&key, OC); key_add(&key, (int)bias->dtype);
                    e = cache_find(ctx, key);
                    if (!e)
                        e = cache_insert(ctx, key, { { reinterpret_cast<const char*>(bp), bias->bytes } },
                                         (size_t)OCpad * sizeof(float), build);
                }
                void* block = nullptr;
                if (e)
                {
                    st = cache_use(ctx, e);
                    if (st != TB200_OK)
                        return st;
                    block = e->block;
                }
                else
                {
                    st = ensure_scratch(ctx, (size_t)OCpad * sizeof(float));
                    if (st != TB200_OK)
                        return st;
                    st = build(ctx, ctx->scratch);
                    if (st != TB200_OK)
                        return st;
                    block = ctx->scratch;
                }
                q.bias_f_pad  = reinterpret_cast<const float*>(block);
                q.corr_stride = OCpad;
                return tc_gemm_launch(ctx, q);
            }
        }
    }

    if (view || dry_run)
        return kNeedsDenseOutput;

    // ---- few-channel int8 convolutions with a horizontal stride of 2 (the RGB stem), parity-split form: four bytes per
    // pixel and one padded copy per parity of the output column make the KW taps a 32-byte window at a 16-byte pitch,
    // half the MMAs of the 64-byte window of the form below.  Only tc_conv_lean_kernel maps the (image, parity) batch
    // back to output columns, so this form needs cached, host-proven tables; anything else takes the form below.
    if (ctx->policy == 0 && int_path && weight_zp == 0 && tc_rescale_ok && input->contiguous && IC <= 4 && stride[1] == 2 &&
        KW >= 2 && KW <= 8 && dilation[0] == 1 && dilation[1] == 1 && use_cache && ctx->const_cache_on && epi.has_rescale &&
        output->dtype == TB200_INT8 && !epi.rs.out_unsigned && N < (1 << 29))
    {
        const int win   = 32;
        const int OWp   = (OW + 1) / 2;    // output columns of parity 0 (parity 1 has OW / 2)
        const int Hp    = IH + pad[0] + pad[1];
        const int Wq    = (std::max(IW + pad[2] + pad[3], 4 * (OWp - 1) + 8 + 2) + 3) & ~3;
        const int OCpad = (OC + 255) / 256 * 256;
        const size_t xq_bytes = ((size_t)N * 2 * Hp * Wq * 4 + 255) & ~(size_t)255;
        const size_t wr_bytes = ((size_t)OC * KH * win + 255) & ~(size_t)255;
        const size_t prefix_elems = ((size_t)(KH + 1) * 2 * OC + 3) & ~(size_t)3;
        const size_t rec_off   = ((prefix_elems + 2 * (size_t)OCpad) * sizeof(int32_t) + OCpad + 63) & ~(size_t)63;
        const size_t flag_off  = rec_off + (size_t)OCpad * 8 * sizeof(int32_t);
        const size_t tab_bytes = flag_off + 64;
        if (xq_bytes + wr_bytes + tab_bytes <= ((size_t)8 << 30))
        {
            TcProblem q;
            memset(&q, 0, sizeof(q));
            q.in_dtype = TB200_INT8;
            q.N = 2 * N; q.IH = Hp; q.IW = OWp; q.IC = win;
            q.a_stride_w = 16; q.a_stride_h = (int64_t)Wq * 4; q.a_stride_n = (int64_t)Hp * Wq * 4;
            q.OH = OH; q.OW = OWp; q.OC = OC;
            q.KH = KH; q.KW = 1;
            q.stride_y = stride[0]; q.stride_x = 1; q.dil_y = 1; q.dil_x = 1;
            q.out = output->data;
            q.epi = TC_EPI_I32;
            q.xpar = 1;
            q.out_ow_real = OW;
            fill_tc_epilogue(&q, epi, output->dtype);
            const int8_t* wp  = reinterpret_cast<const int8_t*>(weight->data);
            const int32_t* bp = reinterpret_cast<const int32_t*>(bias->data);
            const int32_t* mp = reinterpret_cast<const int32_t*>(epi.rs.mult);
            const int8_t* sp  = epi.rs.shift;
            const int bias_n = bias->shape[0], per_ch = epi.rs.per_channel;
            const int block  = 256;
            const int dr_i   = epi.rs.rounding == TB200_DOUBLE_ROUND ? 1 : 0;
            const int32_t ozp_i = (int32_t)epi.rs.out_zp_ext;
            auto build = [=](tb200_ctx* c, void* blk) -> tb200_status {
                int8_t* wr        = reinterpret_cast<int8_t*>(blk);
                int32_t* prefix   = reinterpret_cast<int32_t*>(wr + wr_bytes);
                int32_t* corr     = prefix + prefix_elems;
                int32_t* mult_pad = corr + OCpad;
                int8_t* shift_pad = reinterpret_cast<int8_t*>(mult_pad + OCpad);
                int32_t* rec      = reinterpret_cast<int32_t*>(wr + wr_bytes + rec_off);
                int* all_ok       = reinterpret_cast<int*>(wr + wr_bytes + flag_off);
                TB200_CUDA_CHECK(c, cudaMemsetAsync(all_ok, 1, sizeof(int), c->stream));
                repack_weights_smallc_kernel<<<(int)(((int64_t)OC * KH * win + block - 1) / block), block, 0, c->stream>>>(
                    wp, wr, OC, KH, KW, IC, 4, win);
                conv_epilogue_tables_kernel<<<(OCpad * 32 + 127) / 128, 128, 0, c->stream>>>(
                    wr, bp, bias_n, OC, OCpad, KH, 1, win, input_zp, 0, mp, sp, per_ch, prefix, corr, mult_pad, shift_pad, rec,
                    nullptr, dr_i, ozp_i, all_ok);
                return post_launch(c, "conv_window_tables", 2);
            };
            std::string key;
            key_add(&key, (int)7);
            key_add(&key, wp); key_add(&key, bp); key_add(&key, mp); key_add(&key, sp);
            key_add(&key, OC); key_add(&key, KH); key_add(&key, KW); key_add(&key, IC); key_add(&key, bias_n);
            key_add(&key, input_zp); key_add(&key, per_ch); key_add(&key, dr_i); key_add(&key, ozp_i);
            Prepared* e = cache_find(ctx, key);
            if (!e)
            {
                std::vector<std::pair<const char*, size_t>> ops = {
                    { reinterpret_cast<const char*>(wp), weight->bytes }, { reinterpret_cast<const char*>(bp), bias->bytes },
                    { reinterpret_cast<const char*>(mp), epilogue->rescale.multiplier->bytes },
                    { reinterpret_cast<const char*>(sp), epilogue->rescale.shift->bytes } };
                e = cache_insert(ctx, key, std::move(ops), wr_bytes + tab_bytes, build);
            }
            if (e)
            {
                st = cache_use(ctx, e);
                if (st == TB200_OK)
                    st = read_host_flag(ctx, e, wr_bytes + flag_off);
                if (st != TB200_OK)
                    return st;
                int8_t* wr        = reinterpret_cast<int8_t*>(e->block);
                int32_t* corr     = reinterpret_cast<int32_t*>(wr + wr_bytes) + prefix_elems;
                int32_t* mult_pad = corr + OCpad;
                q.b           = wr;
                q.corr        = corr;
                q.corr_stride = OCpad;
                q.mult_pad    = mult_pad;
                q.shift_pad   = reinterpret_cast<int8_t*>(mult_pad + OCpad);
                q.rec         = reinterpret_cast<const int32_t*>(wr + wr_bytes + rec_off);
                q.lean_ok     = e->host_flag == 1 ? 1 : 0;
                // the scratch address enters the plan only as a pointer: any 16-byte aligned value serves the dry run
                q.a = ctx->scratch ? ctx->scratch : reinterpret_cast<const void*>(static_cast<uintptr_t>(256));
                if (q.lean_ok && tc_gemm_lean_supported(ctx, q))
                {
                    st = ensure_scratch(ctx, xq_bytes);
                    if (st != TB200_OK)
                        return st;
                    int8_t* xq = reinterpret_cast<int8_t*>(ctx->scratch);
                    q.a        = xq;
                    pad_expand_parity_i8_kernel<<<grid_for(ctx, (int64_t)N * 2 * Hp * (Wq / 4), block), block, 0, ctx->stream>>>(
                        reinterpret_cast<const int8_t*>(input->data), xq, N, IH, IW, IC, Hp, Wq, pad[0], pad[2], input_zp);
                    st = post_launch(ctx, "conv_window_relayout", 1);
                    if (st != TB200_OK)
                        return st;
                    st = tc_gemm_launch(ctx, q);
                    // a driver that refuses the overlapping-window tensor map sends this shape to the form below
                    if (!(st == TB200_INTERNAL && ctx->err.find("rejected") != std::string::npos))
                        return st;
                }
            }
        }
    }

    // ---- few-channel int8 convolutions (IC <= 8, e.g. the RGB stem): window re-layout + tensor cores
    if (ctx->policy == 0 && int_path && weight_zp == 0 && tc_rescale_ok && input->contiguous && IC <= 8 &&
        (IC % 32) != 0 && dilation[0] == 1 && dilation[1] == 1 && KW >= 2)
    {
        const int Cp  = (stride[1] % 2 == 0) ? 8 : 16;
        int win       = KW * Cp;
        win           = win <= 32 ? 32 : win <= 64 ? 64 : win <= 128 ? 128 : 0;
        const int Hp  = IH + pad[0] + pad[1];
        const int Wp0 = IW + pad[2] + pad[3];
        // every window [ox*stride*Cp, +win) must stay inside its row
        const int Wp  = std::max(Wp0, ((OW - 1) * stride[1] * Cp + win + Cp - 1) / Cp);
        const int OCpad = (OC + 255) / 256 * 256;
        const size_t xp_bytes = ((size_t)N * Hp * Wp * Cp + 255) & ~(size_t)255;
        const size_t wr_bytes = ((size_t)OC * KH * win + 255) & ~(size_t)255;
        const size_t prefix_elems = ((size_t)(KH + 1) * 2 * OC + 3) & ~(size_t)3;
        const size_t rec_off   = ((prefix_elems + 2 * (size_t)OCpad) * sizeof(int32_t) + OCpad + 63) & ~(size_t)63;
        const size_t flag_off  = rec_off + (size_t)OCpad * 8 * sizeof(int32_t);
        const size_t tab_bytes = flag_off + 64;
        if (win != 0 && xp_bytes + wr_bytes + tab_bytes <= ((size_t)8 << 30))
        {
            TcProblem q;
            memset(&q, 0, sizeof(q));
            q.in_dtype = TB200_INT8;
            q.N = N; q.IH = Hp; q.IW = OW; q.IC = win;
            q.a_stride_w = (int64_t)stride[1] * Cp; q.a_stride_h = (int64_t)Wp * Cp; q.a_stride_n = (int64_t)Hp * Wp * Cp;
            q.OH = OH; q.OW = OW; q.OC = OC;
            q.KH = KH; q.KW = 1;
            q.stride_y = stride[0]; q.stride_x = 1; q.dil_y = 1; q.dil_x = 1;
            q.out = output->data;
            q.epi = TC_EPI_I32;
            fill_tc_epilogue(&q, epi, output->dtype);
            // Derived from the constants alone (cached): weights re-packed to [OC][KH][win] and the epilogue tables.
            // Derived from the input (context scratch, every call): the border- and channel-padded copy.
            const int8_t* wp  = reinterpret_cast<const int8_t*>(weight->data);
            const int32_t* bp = reinterpret_cast<const int32_t*>(bias->data);
            const int32_t* mp = epi.has_rescale ? reinterpret_cast<const int32_t*>(epi.rs.mult) : nullptr;
            const int8_t* sp  = epi.has_rescale ? epi.rs.shift : nullptr;
            const int bias_n = bias->shape[0], per_ch = epi.rs.per_channel, has_rs = epi.has_rescale ? 1 : 0;
            const int block  = 256;
            const int dr_i   = epi.has_rescale && epi.rs.rounding == TB200_DOUBLE_ROUND ? 1 : 0;
            const int32_t ozp_i = epi.has_rescale ? (int32_t)epi.rs.out_zp_ext : 0;
            auto build = [=](tb200_ctx* c, void* blk) -> tb200_status {
                int8_t* wr        = reinterpret_cast<int8_t*>(blk);
                int32_t* prefix   = reinterpret_cast<int32_t*>(wr + wr_bytes);
                int32_t* corr     = prefix + prefix_elems;
                int32_t* mult_pad = corr + OCpad;
                int8_t* shift_pad = reinterpret_cast<int8_t*>(mult_pad + OCpad);
                int32_t* rec      = has_rs ? reinterpret_cast<int32_t*>(wr + wr_bytes + rec_off) : nullptr;
                int* all_ok       = reinterpret_cast<int*>(wr + wr_bytes + flag_off);
                TB200_CUDA_CHECK(c, cudaMemsetAsync(all_ok, has_rs ? 1 : 0, sizeof(int), c->stream));
                repack_weights_smallc_kernel<<<(int)(((int64_t)OC * KH * win + block - 1) / block), block, 0, c->stream>>>(
                    wp, wr, OC, KH, KW, IC, Cp, win);
                // the border holds the zero point, so every tap is in scope and one correction row serves all pixels
                // (the re-packed rows are `win` bytes of which KW * IC carry weights: the value bound counts them all,
                // which only makes it more cautious)
                conv_epilogue_tables_kernel<<<(OCpad * 32 + 127) / 128, 128, 0, c->stream>>>(
                    wr, bp, bias_n, OC, OCpad, KH, 1, win, input_zp, 0, mp, sp, per_ch, prefix, corr,
                    has_rs ? mult_pad : nullptr, shift_pad, rec, nullptr, dr_i, ozp_i, all_ok);
                return post_launch(c, "conv_window_tables", 2);
            };
            Prepared* e = nullptr;
            if (use_cache && ctx->const_cache_on)
            {
                std::string key;
                key_add(&key, (int)1);
                key_add(&key, wp); key_add(&key, bp); key_add(&key, mp); key_add(&key, sp);
                key_add(&key, OC); key_add(&key, KH); key_add(&key, KW); key_add(&key, IC); key_add(&key, bias_n);
                key_add(&key, input_zp); key_add(&key, per_ch); key_add(&key, has_rs); key_add(&key, Cp); key_add(&key, win);
                key_add(&key, dr_i); key_add(&key, ozp_i);
                e = cache_find(ctx, key);
                if (!e)
                {
                    std::vector<std::pair<const char*, size_t>> ops = {
                        { reinterpret_cast<const char*>(wp), weight->bytes }, { reinterpret_cast<const char*>(bp), bias->bytes } };
                    if (has_rs)
                    {
                        ops.push_back({ reinterpret_cast<const char*>(mp), epilogue->rescale.multiplier->bytes });
                        ops.push_back({ reinterpret_cast<const char*>(sp), epilogue->rescale.shift->bytes });
                    }
                    e = cache_insert(ctx, key, std::move(ops), wr_bytes + tab_bytes, build);
                }
            }
            st = ensure_scratch(ctx, xp_bytes + (e ? 0 : wr_bytes + tab_bytes));
            if (st != TB200_OK)
                return st;
            int8_t* xp = reinterpret_cast<int8_t*>(ctx->scratch);
            int8_t* wr = e ? reinterpret_cast<int8_t*>(e->block) : xp + xp_bytes;
            q.a = xp;
            q.b = wr;
            std::string why;
            if (tc_gemm_supported(q, &why))
            {
                if (e)
                {
                    st = cache_use(ctx, e);
                    if (st == TB200_OK)
                        st = read_host_flag(ctx, e, wr_bytes + flag_off);
                    q.lean_ok = e->host_flag == 1 ? 1 : 0;
                }
                else
                    st = build(ctx, wr);
                if (st != TB200_OK)
                    return st;
                int32_t* corr     = reinterpret_cast<int32_t*>(wr + wr_bytes) + prefix_elems;
                int32_t* mult_pad = corr + OCpad;
                pad_expand_i8_kernel<<<grid_for(ctx, (int64_t)N * Hp * Wp, block), block, 0, ctx->stream>>>(
                    reinterpret_cast<const int8_t*>(input->data), xp, N, IH, IW, IC, Hp, Wp, Cp, pad[0], pad[2], input_zp);
                st = post_launch(ctx, "conv_window_relayout", 1);
                if (st != TB200_OK)
                    return st;
                q.corr        = corr;
                q.corr_stride = OCpad;
                q.mult_pad    = mult_pad;
                q.shift_pad   = reinterpret_cast<int8_t*>(mult_pad + OCpad);
                if (has_rs && output->dtype == TB200_INT8 && !epi.rs.out_unsigned)
                    q.rec = reinterpret_cast<const int32_t*>(wr + wr_bytes + rec_off);
                st = tc_gemm_launch(ctx, q);
                // a driver that refuses the overlapping-window tensor map sends this shape to the CUDA-core kernel
                if (!(st == TB200_INTERNAL && ctx->err.find("rejected") != std::string::npos))
                    return st;
            }
        }
    }

    // ---- CUDA-core path
    ConvDev d;
    memset(&d, 0, sizeof(d));
    d.N = N; d.IH = IH; d.IW = IW; d.IC = IC; d.OH = OH; d.OW = OW; d.OC = OC; d.KH = KH; d.KW = KW; d.M = 1;
    d.pad_t = pad[0]; d.pad_l = pad[2]; d.sy = stride[0]; d.sx = stride[1]; d.dy = dilation[0]; d.dx = dilation[1];
    d.in_zp = input_zp; d.w_zp = weight_zp; d.bias_n = bias->shape[0];
    d.in_sn = input->stride[0]; d.in_sh = input->stride[1]; d.in_sw = input->stride[2];
    TB200_ERROR_IF(ctx, input->stride[3] != 1, "OpConv2d: the channel dimension of the input must be dense");
    fill_conv_dev(&d, epi);
    const int block = 256;
    const int grid  = grid_for(ctx, numel(output), block);
    if (int_path)
    {
        const int8_t* in  = reinterpret_cast<const int8_t*>(input->data);
        const int8_t* w   = reinterpret_cast<const int8_t*>(weight->data);
        const int32_t* b  = reinterpret_cast<const int32_t*>(bias->data);
        switch (dtype_size(output->dtype))
        {
            case 1:
                conv2d_direct_i8_kernel<int8_t><<<grid, block, 0, ctx->stream>>>(in, w, b, reinterpret_cast<int8_t*>(output->data), d, ctx->d_status);
                break;
            case 2:
                conv2d_direct_i8_kernel<int16_t><<<grid, block, 0, ctx->stream>>>(in, w, b, reinterpret_cast<int16_t*>(output->data), d, ctx->d_status);
                break;
            default:
                conv2d_direct_i8_kernel<int32_t><<<grid, block, 0, ctx->stream>>>(in, w, b, reinterpret_cast<int32_t*>(output->data), d, ctx->d_status);
                break;
        }
    }
    else if (input->dtype == TB200_FP8E4M3)
        conv2d_direct_fp_kernel<__nv_fp8_e4m3, __half><<<grid, block, 0, ctx->stream>>>(
            reinterpret_cast<const __nv_fp8_e4m3*>(input->data), reinterpret_cast<const __nv_fp8_e4m3*>(weight->data),
            reinterpret_cast<const __half*>(bias->data), reinterpret_cast<__half*>(output->data), d);
    else if (input->dtype == TB200_FP8E5M2)
        conv2d_direct_fp_kernel<__nv_fp8_e5m2, __half><<<grid, block, 0, ctx->stream>>>(
            reinterpret_cast<const __nv_fp8_e5m2*>(input->data), reinterpret_cast<const __nv_fp8_e5m2*>(weight->data),
            reinterpret_cast<const __half*>(bias->data), reinterpret_cast<__half*>(output->data), d);
    else if (input->dtype == TB200_FP16)
        conv2d_direct_fp_kernel<__half><<<grid, block, 0, ctx->stream>>>(
            reinterpret_cast<const __half*>(input->data), reinterpret_cast<const __half*>(weight->data),
            reinterpret_cast<const __half*>(bias->data), reinterpret_cast<__half*>(output->data), d);
    else if (input->dtype == TB200_BF16)
        conv2d_direct_fp_kernel<__nv_bfloat16><<<grid, block, 0, ctx->stream>>>(
            reinterpret_cast<const __nv_bfloat16*>(input->data), reinterpret_cast<const __nv_bfloat16*>(weight->data),
            reinterpret_cast<const __nv_bfloat16*>(bias->data), reinterpret_cast<__nv_bfloat16*>(output->data), d);
    else
        conv2d_direct_fp_kernel<float><<<grid, block, 0, ctx->stream>>>(
            reinterpret_cast<const float*>(input->data), reinterpret_cast<const float*>(weight->data),
            reinterpret_cast<const float*>(bias->data), reinterpret_cast<float*>(output->data), d);
    return post_launch(ctx, "conv2d_direct");
}

extern "C" tb200_status tb200_conv2d(tb200_ctx* ctx, const tb200_tensor* input, const tb200_tensor* weight,
                                     const tb200_tensor* bias, int32_t input_zp, int32_t weight_zp, const int32_t pad[4],
                                     const int32_t stride[2], const int32_t dilation[2], const tb200_epilogue* epilogue,
                                     tb200_tensor* output)
{
    return conv2d_impl(ctx, input, weight, bias, input_zp, weight_zp, pad, stride, dilation, epilogue, output, nullptr,
                       false, true);
}

// =================================================================================================== TRANSPOSE_CONV2D
// Staging that must outlive a nested tb200_conv2d call (which owns ctx->scratch).
static tb200_status ensure_stage(tb200_ctx* ctx, size_t bytes)
{
    if (bytes <= ctx->stage_bytes)
        return TB200_OK;
    if (ctx->capturing)
        return fail(ctx, TB200_ERROR, "staging memory would have to grow during capture; evaluate once eagerly first");
    release_block(ctx, ctx->stage);
    ctx->stage       = nullptr;
    ctx->stage_bytes = 0;
    TB200_CUDA_CHECK(ctx, cudaMalloc(&ctx->stage, bytes));
    ctx->stage_bytes = bytes;
    return TB200_OK;
}

template <typename U>
static void launch_spread(tb200_ctx* ctx, const void* in, void* out, int N, int IH, int IW, int units, int DH, int DW, int sy,
                          int sx, U fill)
{
    const int block = 256;
    spread_pixels_kernel<U><<<grid_for(ctx, (int64_t)N * DH * DW * units, block), block, 0, ctx->stream>>>(
        reinterpret_cast<const U*>(in), reinterpret_cast<U*>(out), N, IH, IW, units, DH, DW, sy, sx, fill);
}

template <typename U>
static void launch_mirror_u(tb200_ctx* ctx, const void* in, void* out, int OC, int KH, int KW, int units, int ky0, int sy,
                            int Ty, int kx0, int sx, int Tx)
{
    const int block = 256;
    mirror_weights_kernel<U><<<grid_for(ctx, (int64_t)OC * Ty * Tx * units, block), block, 0, ctx->stream>>>(
        reinterpret_cast<const U*>(in), reinterpret_cast<U*>(out), OC, KH, KW, units, ky0, sy, Ty, kx0, sx, Tx);
}

// run = bytes of one pixel's channel run; 16-byte units when the run and both pointers allow it
static void launch_mirror(tb200_ctx* ctx, const void* in, void* out, int OC, int KH, int KW, int IC, size_t es, bool vec,
                          int ky0, int sy, int Ty, int kx0, int sx, int Tx)
{
    if (vec)
        launch_mirror_u<uint4>(ctx, in, out, OC, KH, KW, (int)(IC * es / 16), ky0, sy, Ty, kx0, sx, Tx);
    else if (es == 1)
        launch_mirror_u<uint8_t>(ctx, in, out, OC, KH, KW, IC, ky0, sy, Ty, kx0, sx, Tx);
    else if (es == 2)
        launch_mirror_u<uint16_t>(ctx, in, out, OC, KH, KW, IC, ky0, sy, Ty, kx0, sx, Tx);
    else
        launch_mirror_u<uint32_t>(ctx, in, out, OC, KH, KW, IC, ky0, sy, Ty, kx0, sx, Tx);
}

// One axis of one phase of a strided TRANSPOSE_CONV2D.  Output positions o = p + s*j (j < J) only see the taps
// k = k0 + s*t (t < T) with k0 = (p - out_pad) mod s, and read input index j + c - t with c = (p - out_pad - k0) / s
// (OpTransposeConv2d::eval, reference_model/src/ops/tensor_ops.cpp:2148-2171, solved for the taps whose division is
// exact).  With the taps mirrored this is a stride-1 convolution over input rows [start, start + len) with pads
// (pad0, pad1).  T == 0: no tap reaches this phase (its outputs are the bias alone).
struct PhaseAxis
{
    int J, k0, T, start, len, pad0, pad1;
};

static PhaseAxis plan_phase_axis(int I, int K, int O, int s, int out_pad0, int p)
{
    PhaseAxis a = {};
    a.J         = O > p ? (O - p + s - 1) / s : 0;
    a.k0        = ((p - out_pad0) % s + s) % s;
    a.T         = K > a.k0 ? (K - a.k0 + s - 1) / s : 0;
    if (a.J == 0 || a.T == 0)
        return a;
    const int c = (p - out_pad0 - a.k0) / s;    // exact by the choice of k0
    a.pad0      = (a.T - 1) - c;
    if (a.pad0 < 0)
    {
        a.start = -a.pad0;
        a.pad0  = 0;
    }
    a.len  = I - a.start;
    a.pad1 = a.J - a.len - a.pad0 + a.T - 1;
    if (a.pad1 < 0)
    {
        a.len += a.pad1;
        a.pad1 = 0;
    }
    if (a.len <= 0)
        a.T = 0;
    return a;
}

// CONV2D 1x1 -> CLAMP -> DEPTHWISE_CONV2D 3x3 -> CLAMP in one kernel (expand_dw.cu); see include/tb200.h.
extern "C" tb200_status tb200_conv2d_depthwise(tb200_ctx* ctx, const tb200_tensor* input, const tb200_tensor* weight,
                                               const tb200_tensor* bias, const tb200_epilogue* conv_epilogue,
                                               const tb200_tensor* dw_weight, const tb200_tensor* dw_bias,
                                               const int32_t dw_pad[4], const int32_t dw_stride[2],
                                               const tb200_epilogue* dw_epilogue, tb200_tensor* expanded,
                                               tb200_tensor* output)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !input || !weight || !bias || !dw_weight || !dw_bias || !dw_pad || !dw_stride || !output,
                   "OpConv2d + OpDepthwiseConv2d: null operand");
    TB200_ERROR_IF(ctx, !all_contiguous({ input, weight, bias, dw_weight, dw_bias, output }),
                   "OpConv2d + OpDepthwiseConv2d: every operand must be contiguous");
    TB200_ERROR_IF(ctx, input->rank != 4 || weight->rank != 4 || dw_weight->rank != 4 || output->rank != 4 || bias->rank != 1 ||
                            dw_bias->rank != 1,
                   "OpConv2d + OpDepthwiseConv2d: tensors must be rank 4 and biases rank 1");
    const int N = input->shape[0], IH = input->shape[1], IW = input->shape[2], IC = input->shape[3];
    const int C  = weight->shape[0];
    const int OH = output->shape[1], OW = output->shape[2];
    const int32_t one[2]  = { 1, 1 };
    const int32_t zero[4] = { 0, 0, 0, 0 };
    const tb200_dtype dt  = input->dtype;
    bool fusable = weight->shape[1] == 1 && weight->shape[2] == 1 && weight->shape[3] == IC && dw_weight->shape[0] == 3 &&
                   dw_weight->shape[1] == 3 && dw_weight->shape[2] == C && dw_weight->shape[3] == 1 && output->shape[0] == N &&
                   output->shape[3] == C && (bias->shape[0] == C || bias->shape[0] == 1) &&
                   (dw_bias->shape[0] == C || dw_bias->shape[0] == 1) && weight->dtype == dt && bias->dtype == dt &&
                   dw_weight->dtype == dt && dw_bias->dtype == dt && output->dtype == dt && numel(output) > 0 && numel(input) > 0;
    ExpandDwProblem q;
    memset(&q, 0, sizeof(q));
    if (fusable)
    {
        // the checks of the two operators the kernel stands for (the CONV2D's output shape is implied: [N, IH, IW, C])
        tb200_status st = check_conv_attr(ctx, "OpDepthwiseConv2d", IH, IW, OH, OW, 3, 3, dw_pad, dw_stride, one);
        if (st != TB200_OK)
            return st;
        EpiInfo e1, e2;
        st = parse_epilogue(ctx, "OpConv2d", conv_epilogue, false, C, dt, &e1);
        if (st != TB200_OK)
            return st;
        st = parse_epilogue(ctx, "OpDepthwiseConv2d", dw_epilogue, false, C, dt, &e2);
        if (st != TB200_OK)
            return st;
        q.dtype = dt;
        q.in = input->data; q.w1 = weight->data; q.b1 = bias->data; q.wd = dw_weight->data; q.bd = dw_bias->data;
        q.out = output->data;
        q.b1_n = bias->shape[0]; q.bd_n = dw_bias->shape[0];
        q.N = N; q.IH = IH; q.IW = IW; q.IC = IC; q.C = C; q.OH = OH; q.OW = OW;
        q.pad_t = dw_pad[0]; q.pad_l = dw_pad[2]; q.sy = dw_stride[0]; q.sx = dw_stride[1];
        q.clamp1 = e1.has_clamp; q.lo1 = e1.clamp_lo_f; q.hi1 = e1.clamp_hi_f;
        q.clamp2 = e2.has_clamp; q.lo2 = e2.clamp_lo_f; q.hi2 = e2.clamp_hi_f;
        std::string why;
        fusable = ctx->policy == 0 && expand_dw_supported(ctx, q, &why);
    }
    if (fusable)
    {
        cache_note_write(ctx, output->data, output->bytes);
        return expand_dw_launch(ctx, q);
    }
    // shapes the kernel does not take: the two operators one after the other, through the caller's tensor
    TB200_ERROR_IF(ctx, !expanded,
                   "OpConv2d + OpDepthwiseConv2d: this shape does not run as one kernel and no tensor for the CONV2D output was given");
    tb200_status st = tb200_conv2d(ctx, input, weight, bias, 0, 0, zero, one, one, conv_epilogue, expanded);
    if (st != TB200_OK && st != TB200_UNPREDICTABLE)
        return st;
    const tb200_status st2 = tb200_depthwise_conv2d(ctx, expanded, dw_weight, dw_bias, 0, 0, dw_pad, dw_stride, one, dw_epilogue, output);
    return st2 != TB200_OK ? st2 : st;
}

// check_conv_attribute with conv_dimension 3 (reference_model/src/ops/tensor_ops.cpp:120-226): pad = (d0, d1, top, bottom,
// left, right), stride and dilation = (d, y, x)
static tb200_status check_conv3d_attr(tb200_ctx* ctx, const int in[3], const int out[3], const int k[3], const int32_t* pad,
                                      const int32_t* stride, const int32_t* dilation)
{
    const char* op = "OpConv3d";
    for (int i = 0; i < 6; i++)
        TB200_ERROR_IF(ctx, pad[i] < 0, "%s: At least one pad is smaller than zero", op);
    for (int i = 0; i < 3; i++)
        TB200_ERROR_IF(ctx, stride[i] < 1, "%s: At least one stride dimension is smaller than one", op);
    for (int i = 0; i < 3; i++)
        TB200_ERROR_IF(ctx, dilation[i] < 1, "%s: At least one dilation dimension is smaller than one", op);
    int full[3];
    for (int a = 0; a < 3; a++)
        full[a] = in[a] - 1 + pad[2 * a] + pad[2 * a + 1] - (k[a] - 1) * dilation[a];
    TB200_ERROR_IF(ctx, (full[0] % stride[0] != 0) || (full[1] % stride[1] != 0) || (full[2] % stride[2] != 0),
                   "%s: Parameters must yield exact integer output dimensions", op);
    TB200_ERROR_IF(ctx, out[0] != full[0] / stride[0] + 1 || out[1] != full[1] / stride[1] + 1 || out[2] != full[2] / stride[2] + 1,
                   "%s: Mismatch between output shape provided and expected output shape (%d,%d,%d)", op,
                   full[0] / stride[0] + 1, full[1] / stride[1] + 1, full[2] / stride[2] + 1);
    return TB200_OK;
}

// A contiguous rank-4 view [a, b, c, d] over a tensor's memory (no ownership).
static tb200_tensor view4(const tb200_tensor* t, int a, int b, int c, int d)
{
    tb200_tensor v = *t;
    v.rank         = 4;
    v.shape[0] = a; v.shape[1] = b; v.shape[2] = c; v.shape[3] = d;
    v.stride[3] = 1; v.stride[2] = d; v.stride[1] = (int64_t)c * d; v.stride[0] = (int64_t)b * c * d;
    v.owns       = false;
    v.contiguous = true;
    return v;
}

// CONV3D; see include/tb200.h.
extern "C" tb200_status tb200_conv3d(tb200_ctx* ctx, const tb200_tensor* input, const tb200_tensor* weight,
                                     const tb200_tensor* bias, int32_t input_zp, int32_t weight_zp, const int32_t pad[6],
                                     const int32_t stride[3], const int32_t dilation[3], const tb200_epilogue* epilogue,
                                     tb200_tensor* output)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !input || !weight || !bias || !output || !pad || !stride || !dilation, "OpConv3d: null operand");
    TB200_ERROR_IF(ctx, !all_contiguous({ input, weight, bias, output }), "OpConv3d: every operand must be contiguous");
    TB200_ERROR_IF(ctx, input->rank != 5 || weight->rank != 5 || output->rank != 5 || bias->rank != 1,
                   "OpConv3d: input, weight and output must be rank 5 and bias rank 1");
    const int N = input->shape[0], ID = input->shape[1], IH = input->shape[2], IW = input->shape[3], IC = input->shape[4];
    const int OC = weight->shape[0], KD = weight->shape[1], KH = weight->shape[2], KW = weight->shape[3];
    const int OD = output->shape[1], OH = output->shape[2], OW = output->shape[3];
    const int in3[3] = { ID, IH, IW }, out3[3] = { OD, OH, OW }, k3[3] = { KD, KH, KW };
    tb200_status st = check_conv3d_attr(ctx, in3, out3, k3, pad, stride, dilation);
    if (st != TB200_OK)
        return st;
    // OpConv3d::eval ERROR_IFs (reference_model/src/ops/tensor_ops.cpp:961-967)
    TB200_ERROR_IF(ctx, N != output->shape[0], "OpConv3d: tensor batch mismatch %d != %d", N, output->shape[0]);
    TB200_ERROR_IF(ctx, weight->shape[4] != IC, "OpConv3d: tensor input channel mismatch %d != %d", weight->shape[4], IC);
    TB200_ERROR_IF(ctx, OC != output->shape[4], "OpConv3d: tensor output channel mismatch %d != %d", OC, output->shape[4]);
    TB200_ERROR_IF(ctx, bias->shape[0] != OC && bias->shape[0] != 1, "OpConv3d: bias channel mismatch %d != %d", bias->shape[0], OC);
    const bool int_path = input->dtype == TB200_INT8;
    TB200_ERROR_IF(ctx, weight->dtype != input->dtype, "OpConv3d: input and weight dtypes differ");
    if (int_path)
        TB200_ERROR_IF(ctx, bias->dtype != TB200_INT32, "OpConv3d: INT8 convolution needs an INT32 bias");
    else
    {
        TB200_ERROR_IF(ctx, !dtype_is_float(input->dtype), "OpConv3d: unsupported input dtype");
        TB200_ERROR_IF(ctx, bias->dtype != input->dtype || output->dtype != input->dtype,
                       "OpConv3d: floating bias and output must have the input dtype");
        TB200_ERROR_IF(ctx, input_zp != 0, "Input zero point must be zero for non int8_t data");
        TB200_ERROR_IF(ctx, weight_zp != 0, "Weight zero point must be zero for non int8_t data");
    }
    TB200_ERROR_IF(ctx, input_zp < -128 || input_zp > 127 || weight_zp < -128 || weight_zp > 127,
                   "OpConv3d: zero point outside the int8 range");
    EpiInfo epi;
    st = parse_epilogue(ctx, "OpConv3d", epilogue, int_path, OC, output->dtype, &epi);
    if (st != TB200_OK)
        return st;
    if (numel(output) == 0)
        return TB200_OK;
    // One depth tap, depth stride 1, no depth padding: every depth slice is an image of a CONV2D with the same weights
    // (output depth od reads input depth od only), so the batch of N x ID images takes CONV2D's kernels, the tensor-core
    // ones included.
    if (KD == 1 && stride[0] == 1 && pad[0] == 0 && pad[1] == 0 && (int64_t)N * ID < ((int64_t)1 << 31))
    {
        const tb200_tensor in4 = view4(input, N * ID, IH, IW, IC), w4 = view4(weight, OC, KH, KW, IC);
        tb200_tensor out4      = view4(output, N * OD, OH, OW, OC);
        return tb200_conv2d(ctx, &in4, &w4, bias, input_zp, weight_zp, pad + 2, stride + 1, dilation + 1, epilogue, &out4);
    }
    // Any other kernel whose depth taps make whole 32-byte runs of K: the taps of every output depth are gathered beside
    // the channels (staging of KD times the input) and the weights re-ordered to match, which leaves a CONV2D over
    // N x OD images with KD x IC channels for the tensor-core kernels.  The sum runs over the same products in another
    // order: exact for integers, inside the floating-point rule like every tensor-core sum.
    const size_t es  = dtype_size(input->dtype);
    const size_t run = (size_t)IC * es;
    if (ctx->policy == 0 && ((size_t)KD * run) % 32 == 0 && (int64_t)N * OD < ((int64_t)1 << 31) && (int64_t)KD * IC < (1 << 24))
    {
        const int64_t pixels = (int64_t)IH * IW;
        const size_t w_bytes = ((size_t)OC * KH * KW * KD * run + 255) & ~(size_t)255;
        const size_t x_bytes = (size_t)N * OD * pixels * KD * run;
        st                   = ensure_stage(ctx, w_bytes + x_bytes + 256);
        if (st != TB200_OK)
            return st;
        uint8_t* wm = reinterpret_cast<uint8_t*>(ctx->stage);
        uint8_t* xm = wm + w_bytes;
        const int block = 256;
        const uint32_t zb = (uint32_t)(uint8_t)(int8_t)input_zp * 0x01010101u;    // floating types: zero point 0
        if (run % 16 == 0)
        {
            const int units = (int)(run / 16);
            const uint4 fill = es == 1 ? make_uint4(zb, zb, zb, zb) : make_uint4(0, 0, 0, 0);
            conv3d_unfold_depth_kernel<uint4><<<grid_for(ctx, (int64_t)N * OD * pixels * KD * units, block), block, 0, ctx->stream>>>(
                reinterpret_cast<const uint4*>(input->data), reinterpret_cast<uint4*>(xm), N, ID, OD, KD, pixels, units, stride[0],
                dilation[0], pad[0], fill);
            conv3d_fold_weights_kernel<uint4><<<grid_for(ctx, (int64_t)OC * KH * KW * KD * units, block), block, 0, ctx->stream>>>(
                reinterpret_cast<const uint4*>(weight->data), reinterpret_cast<uint4*>(wm), OC, KD, KH * KW, units);
        }
        else if (es == 1)
        {
            conv3d_unfold_depth_kernel<uint8_t><<<grid_for(ctx, (int64_t)N * OD * pixels * KD * IC, block), block, 0, ctx->stream>>>(
                reinterpret_cast<const uint8_t*>(input->data), xm, N, ID, OD, KD, pixels, IC, stride[0], dilation[0], pad[0],
                (uint8_t)(int8_t)input_zp);
            conv3d_fold_weights_kernel<uint8_t><<<grid_for(ctx, (int64_t)OC * KH * KW * KD * IC, block), block, 0, ctx->stream>>>(
                reinterpret_cast<const uint8_t*>(weight->data), wm, OC, KD, KH * KW, IC);
        }
        else if (es == 2)
        {
            conv3d_unfold_depth_kernel<uint16_t><<<grid_for(ctx, (int64_t)N * OD * pixels * KD * IC, block), block, 0, ctx->stream>>>(
                reinterpret_cast<const uint16_t*>(input->data), reinterpret_cast<uint16_t*>(xm), N, ID, OD, KD, pixels, IC, stride[0],
                dilation[0], pad[0], (uint16_t)0);
            conv3d_fold_weights_kernel<uint16_t><<<grid_for(ctx, (int64_t)OC * KH * KW * KD * IC, block), block, 0, ctx->stream>>>(
                reinterpret_cast<const uint16_t*>(weight->data), reinterpret_cast<uint16_t*>(wm), OC, KD, KH * KW, IC);
        }
        else
        {
            conv3d_unfold_depth_kernel<uint32_t><<<grid_for(ctx, (int64_t)N * OD * pixels * KD * IC, block), block, 0, ctx->stream>>>(
                reinterpret_cast<const uint32_t*>(input->data), reinterpret_cast<uint32_t*>(xm), N, ID, OD, KD, pixels, IC, stride[0],
                dilation[0], pad[0], 0u);
            conv3d_fold_weights_kernel<uint32_t><<<grid_for(ctx, (int64_t)OC * KH * KW * KD * IC, block), block, 0, ctx->stream>>>(
                reinterpret_cast<const uint32_t*>(weight->data), reinterpret_cast<uint32_t*>(wm), OC, KD, KH * KW, IC);
        }
        st = post_launch(ctx, "conv3d_depth_staging", 2);
        if (st != TB200_OK)
            return st;
        tb200_tensor xin = view4(input, N * OD, IH, IW, KD * IC), wst = view4(weight, OC, KH, KW, KD * IC);
        xin.data  = xm;
        xin.bytes = x_bytes;
        wst.data  = wm;
        wst.bytes = (size_t)OC * KH * KW * KD * run;
        tb200_tensor out4 = view4(output, N * OD, OH, OW, OC);
        // (input and weights live in staging that the next call overwrites: nothing derived from them is cached)
        st = conv2d_impl(ctx, &xin, &wst, bias, input_zp, weight_zp, pad + 2, stride + 1, dilation + 1, epilogue, &out4, nullptr,
                         false, false);
        if (st != TB200_OK && ctx->err.compare(0, 8, "OpConv2d") == 0)
            ctx->err = "OpConv3d (as CONV2D): " + ctx->err;
        return st;
    }
    cache_note_write(ctx, output->data, output->bytes);
    ConvDev d;
    memset(&d, 0, sizeof(d));
    d.N = N; d.IH = IH; d.IW = IW; d.IC = IC; d.OH = OH; d.OW = OW; d.OC = OC; d.KH = KH; d.KW = KW; d.M = 1;
    d.pad_t = pad[2]; d.pad_l = pad[4]; d.sy = stride[1]; d.sx = stride[2]; d.dy = dilation[1]; d.dx = dilation[2];
    d.in_zp = input_zp; d.w_zp = weight_zp; d.bias_n = bias->shape[0];
    fill_conv_dev(&d, epi);
    ConvDepthDev z;
    z.ID = ID; z.OD = OD; z.KD = KD; z.pad_d = pad[0]; z.sd = stride[0]; z.dd = dilation[0];
    const int block = 256;
    const int grid  = grid_for(ctx, numel(output), block);
    if (int_path)
    {
        const int8_t* in = reinterpret_cast<const int8_t*>(input->data);
        const int8_t* w  = reinterpret_cast<const int8_t*>(weight->data);
        const int32_t* b = reinterpret_cast<const int32_t*>(bias->data);
        switch (dtype_size(output->dtype))
        {
            case 1:
                conv3d_direct_i8_kernel<int8_t><<<grid, block, 0, ctx->stream>>>(in, w, b, reinterpret_cast<int8_t*>(output->data), d, z, ctx->d_status);
                break;
            case 2:
                conv3d_direct_i8_kernel<int16_t><<<grid, block, 0, ctx->stream>>>(in, w, b, reinterpret_cast<int16_t*>(output->data), d, z, ctx->d_status);
                break;
            default:
                conv3d_direct_i8_kernel<int32_t><<<grid, block, 0, ctx->stream>>>(in, w, b, reinterpret_cast<int32_t*>(output->data), d, z, ctx->d_status);
                break;
        }
    }
    else if (input->dtype == TB200_FP16)
        conv3d_direct_fp_kernel<__half><<<grid, block, 0, ctx->stream>>>(
            reinterpret_cast<const __half*>(input->data), reinterpret_cast<const __half*>(weight->data),
            reinterpret_cast<const __half*>(bias->data), reinterpret_cast<__half*>(output->data), d, z);
    else if (input->dtype == TB200_BF16)
        conv3d_direct_fp_kernel<__nv_bfloat16><<<grid, block, 0, ctx->stream>>>(
            reinterpret_cast<const __nv_bfloat16*>(input->data), reinterpret_cast<const __nv_bfloat16*>(weight->data),
            reinterpret_cast<const __nv_bfloat16*>(bias->data), reinterpret_cast<__nv_bfloat16*>(output->data), d, z);
    else
        conv3d_direct_fp_kernel<float><<<grid, block, 0, ctx->stream>>>(
            reinterpret_cast<const float*>(input->data), reinterpret_cast<const float*>(weight->data),
            reinterpret_cast<const float*>(bias->data), reinterpret_cast<float*>(output->data), d, z);
    return post_launch(ctx, "conv3d_direct");
}

extern "C" tb200_status tb200_transpose_conv2d(tb200_ctx* ctx, const tb200_tensor* input, const tb200_tensor* weight,
                                               const tb200_tensor* bias, int32_t input_zp, int32_t weight_zp,
                                               const int32_t out_pad[4], const int32_t stride[2],
                                               const tb200_epilogue* epilogue, tb200_tensor* output)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !input || !weight || !bias || !output || !out_pad || !stride, "OpTransposeConv2d: null operand");
    TB200_ERROR_IF(ctx, !all_contiguous({ input, weight, bias, output }), "OpTransposeConv2d: operands must be contiguous");
    // OpTransposeConv2d::checkTensorAttributes (reference_model/src/ops/tensor_ops.cpp:1982-2056)
    TB200_ERROR_IF(ctx, input->rank != 4 || weight->rank != 4 || output->rank != 4 || bias->rank != 1,
                   "OpTransposeConv2d: input, weight and output must be rank 4 and bias rank 1");
    TB200_ERROR_IF(ctx, stride[0] < 1 || stride[1] < 1, "OpTransposeConv2d: At least one stride is smaller than one");
    const int N = input->shape[0], IH = input->shape[1], IW = input->shape[2], IC = input->shape[3];
    const int OC = weight->shape[0], KH = weight->shape[1], KW = weight->shape[2];
    const int OH = output->shape[1], OW = output->shape[2];
    for (int i = 0; i < 4; i++)
        TB200_ERROR_IF(ctx, out_pad[i] <= -weight->shape[i / 2 + 1],
                       "OpTransposeConv2d: At least one out_pad value is larger than kernel size");
    const int64_t H = (int64_t)(IH - 1) * stride[0] + out_pad[0] + out_pad[1] + KH;
    const int64_t W = (int64_t)(IW - 1) * stride[1] + out_pad[2] + out_pad[3] + KW;
    TB200_ERROR_IF(ctx, OH != H || OW != W,
                   "OpTransposeConv2d: Mismatch between output shape provided and expected output shape (%lld,%lld)",
                   (long long)H, (long long)W);
    // OpTransposeConv2d::eval ERROR_IFs (:2085-2091, :2116-2122)
    TB200_ERROR_IF(ctx, N != output->shape[0], "OpTransposeConv2d: tensor batch mismatch %d != %d", N, output->shape[0]);
    TB200_ERROR_IF(ctx, weight->shape[3] != IC, "OpTransposeConv2d: tensor input channel mismatch %d != %d",
                   weight->shape[3], IC);
    TB200_ERROR_IF(ctx, OC != output->shape[3], "OpTransposeConv2d: tensor output channel mismatch %d != %d", OC,
                   output->shape[3]);
    TB200_ERROR_IF(ctx, bias->shape[0] != OC && bias->shape[0] != 1, "OpTransposeConv2d: bias channels mismatch %d != %d",
                   bias->shape[0], OC);
    TB200_ERROR_IF(ctx, weight->dtype != input->dtype, "OpTransposeConv2d: input and weight dtypes differ");
    if (input->dtype != TB200_INT8)
    {
        TB200_ERROR_IF(ctx, !dtype_is_float(input->dtype) && !dtype_is_fp8(input->dtype),
                       "OpTransposeConv2d: unsupported input dtype %d", (int)input->dtype);
        TB200_ERROR_IF(ctx, input_zp != 0, "Input zero point must be zero for non int8_t data");
        TB200_ERROR_IF(ctx, weight_zp != 0, "Weight zero point must be zero for non int8_t data");
    }
    TB200_ERROR_IF(ctx, input_zp < -128 || input_zp > 127 || weight_zp < -128 || weight_zp > 127,
                   "OpTransposeConv2d: zero point outside the int8 range");
    if (numel(output) == 0 || numel(input) == 0)
        TB200_ERROR_IF(ctx, numel(output) != 0, "OpTransposeConv2d: empty input with a non-empty output");
    if (numel(output) == 0)
        return TB200_OK;

    const size_t es  = dtype_size(input->dtype);
    const size_t run = (size_t)IC * es;    // bytes of one pixel's channel run
    const bool vec   = (run % 16) == 0 && (reinterpret_cast<uintptr_t>(input->data) % 16) == 0 &&
                     (reinterpret_cast<uintptr_t>(weight->data) % 16) == 0;
    const int32_t one[2] = { 1, 1 };
    const int sy = stride[0], sx = stride[1];
    tb200_status st;

    // ---- all phases as column blocks of ONE stride-1 convolution (see embed_phase_operands_kernel): its window covers
    // the input rows any phase reads for a macro-pixel, each phase's taps sit in it mirrored with zeros elsewhere, and
    // block (py, px) of a row is stored at output pixel (j*sy + py, i*sx + px).  With kernel == stride and no out_pad
    // the window is one pixel and nothing is wasted; otherwise zero weights are multiplied too, which the tensor pipe
    // has room for as long as the window is small against the kernel.
    if ((sy > 1 || sx > 1) && sy <= PhaseEmbed::kMax && sx <= PhaseEmbed::kMax && OC % 32 == 0 &&
        (int64_t)sy * sx * OC <= 65536 && (reinterpret_cast<uintptr_t>(output->data) & 31) == 0)
    {
        struct Axis
        {
            int J, U, pad0, pad1, start, len;
            bool ok;
        };
        PhaseEmbed pe;
        memset(&pe, 0, sizeof(pe));
        pe.sy = sy;
        pe.sx = sx;
        auto plan_axis = [](int I, int K, int O, int s, int out_pad0, int* k0, int* T, int* sh, int* U_out) {
            Axis a = {};
            a.J    = (O + s - 1) / s;
            int c[PhaseEmbed::kMax];
            int cmax = INT_MIN;
            for (int p = 0; p < s; p++)
            {
                k0[p] = ((p - out_pad0) % s + s) % s;
                T[p]  = K > k0[p] ? (K - k0[p] + s - 1) / s : 0;
                c[p]  = (p - out_pad0 - k0[p]) / s;    // exact by the choice of k0
                if (T[p] > 0)
                    cmax = std::max(cmax, c[p]);
            }
            if (cmax == INT_MIN)
                return a;
            int U = 0;
            for (int p = 0; p < s; p++)
            {
                sh[p] = cmax - c[p];
                if (T[p] > 0)
                    U = std::max(U, T[p] + sh[p]);
            }
            a.U    = U;
            a.pad0 = (U - 1) - cmax;
            if (a.pad0 < 0)
            {
                a.start = -a.pad0;
                a.pad0  = 0;
            }
            a.len  = I - a.start;
            a.pad1 = a.J - a.len - a.pad0 + U - 1;
            if (a.pad1 < 0)
            {
                a.len += a.pad1;
                a.pad1 = 0;
            }
            a.ok   = a.len > 0;
            *U_out = U;
            return a;
        };
        const Axis ay = plan_axis(IH, KH, OH, sy, out_pad[0], pe.k0y, pe.Ty, pe.shy, &pe.Uy);
        const Axis ax = plan_axis(IW, KW, OW, sx, out_pad[2], pe.k0x, pe.Tx, pe.shx, &pe.Ux);
        // multiplied weights against useful ones: 1 for kernel == stride, 2.25 for a 4x4 kernel with stride 2
        const double waste = ay.ok && ax.ok ? (double)pe.Uy * pe.Ux * sy * sx / ((double)KH * KW) : 1e9;
        if (ay.ok && ax.ok && waste <= 4.5)
        {
            const int blocks = sy * sx, cols = blocks * OC;
            const bool rs        = epilogue && epilogue->has_rescale && epilogue->rescale.multiplier && epilogue->rescale.shift;
            const bool rs_per_ch = rs && epilogue->rescale.per_channel && epilogue->rescale.multiplier->shape[0] == OC &&
                                   epilogue->rescale.shift->shape[0] == OC;
            const size_t bias_es = dtype_size(bias->dtype);
            const size_t mult_es = rs_per_ch ? dtype_size(epilogue->rescale.multiplier->dtype) : 0;
            auto up256           = [](size_t v) { return (v + 255) & ~(size_t)255; };
            const size_t w_off = 0, b_off = up256((size_t)cols * pe.Uy * pe.Ux * run),
                         m_off = b_off + up256((size_t)cols * bias_es), s_off = m_off + up256((size_t)cols * mult_es),
                         total = s_off + up256((size_t)cols);
            tb200_tensor xin = *input, wst = *weight, bst = *bias, mst = {}, sst = {};
            xin.owns = wst.owns = bst.owns = false;
            xin.data       = reinterpret_cast<uint8_t*>(input->data) + ((size_t)ay.start * IW + ax.start) * run;
            xin.shape[1]   = ay.len;
            xin.shape[2]   = ax.len;
            xin.contiguous = ay.len == IH && ax.len == IW;
            wst.shape[0] = cols; wst.shape[1] = pe.Uy; wst.shape[2] = pe.Ux;
            wst.stride[2] = IC; wst.stride[1] = (int64_t)pe.Ux * IC; wst.stride[0] = (int64_t)pe.Uy * pe.Ux * IC;
            wst.bytes     = (size_t)cols * pe.Uy * pe.Ux * run;
            const bool rep_b = bias->shape[0] == OC;
            if (rep_b)
            {
                bst.shape[0] = cols;
                bst.bytes    = (size_t)cols * bias_es;
            }
            tb200_epilogue epi2;
            if (epilogue)
                epi2 = *epilogue;
            if (rs_per_ch)
            {
                mst = *epilogue->rescale.multiplier;
                sst = *epilogue->rescale.shift;
                mst.owns = sst.owns = false;
                mst.shape[0] = sst.shape[0] = cols;
                mst.bytes                   = (size_t)cols * mult_es;
                sst.bytes                   = (size_t)cols;
                epi2.rescale.multiplier     = &mst;
                epi2.rescale.shift          = &sst;
            }
            const int32_t pad[4]   = { ay.pad0, ay.pad1, ax.pad0, ax.pad1 };
            const ConvOutView view = { ay.J, ax.J, sy, sx, 0, 0, OC, sx };
            // the probe only looks at shapes and alignment: the unstaged operands stand in
            st = conv2d_impl(ctx, &xin, &wst, &bst, input_zp, weight_zp, pad, one, one, epilogue ? &epi2 : nullptr, output,
                             &view, true, false);
            if (st == TB200_OK)
            {
                st = ensure_stage(ctx, total);
                if (st != TB200_OK)
                    return st;
                uint8_t* base    = reinterpret_cast<uint8_t*>(ctx->stage);
                const int block  = 256;
                const void* b_in = rep_b ? bias->data : nullptr;
                const void* m_in = rs_per_ch ? epilogue->rescale.multiplier->data : nullptr;
                const uint8_t* s_in = rs_per_ch ? reinterpret_cast<const uint8_t*>(epilogue->rescale.shift->data) : nullptr;
                const int64_t wunits = (int64_t)cols * pe.Uy * pe.Ux;
                if (vec)
                    embed_phase_operands_kernel<uint4><<<grid_for(ctx, wunits * (int64_t)(run / 16), block), block, 0, ctx->stream>>>(
                        reinterpret_cast<const uint4*>(weight->data), reinterpret_cast<uint4*>(base + w_off), OC, KH, KW,
                        (int)(run / 16), pe, b_in, base + b_off, (int)bias_es, m_in, base + m_off, (int)mult_es, s_in, base + s_off);
                else if (es == 1)
                    embed_phase_operands_kernel<uint8_t><<<grid_for(ctx, wunits * IC, block), block, 0, ctx->stream>>>(
                        reinterpret_cast<const uint8_t*>(weight->data), base + w_off, OC, KH, KW, IC, pe, b_in, base + b_off,
                        (int)bias_es, m_in, base + m_off, (int)mult_es, s_in, base + s_off);
                else
                    embed_phase_operands_kernel<uint16_t><<<grid_for(ctx, wunits * IC, block), block, 0, ctx->stream>>>(
                        reinterpret_cast<const uint16_t*>(weight->data), reinterpret_cast<uint16_t*>(base + w_off), OC, KH, KW,
                        IC, pe, b_in, base + b_off, (int)bias_es, m_in, base + m_off, (int)mult_es, s_in, base + s_off);
                wst.data = base + w_off;
                if (rep_b)
                    bst.data = base + b_off;
                if (rs_per_ch)
                {
                    mst.data = base + m_off;
                    sst.data = base + s_off;
                }
                st = post_launch(ctx, "transpose_conv_embed_operands", 1);
                if (st != TB200_OK)
                    return st;
                st = conv2d_impl(ctx, &xin, &wst, &bst, input_zp, weight_zp, pad, one, one, epilogue ? &epi2 : nullptr, output,
                                 &view, false, false);
                return st == kNeedsDenseOutput ? fail(ctx, TB200_INTERNAL, "OpTransposeConv2d: plan changed") : st;
            }
            if (st != kNeedsDenseOutput)
                return st;
        }
    }

    // ---- strided: one stride-1 convolution per output phase, each over the original input with the taps that reach
    // the phase, written straight into its pixels of the output.  Needs the tensor-core kernel for every phase.
    if ((sy > 1 || sx > 1) && sy * sx <= PhaseWeights::kMax)
    {
        struct Phase
        {
            PhaseAxis y, x;
            int py, px;
            size_t w_off;
        };
        std::vector<Phase> phases;
        size_t w_total = 0;
        bool ok        = true;
        for (int py = 0; py < sy && ok; py++)
            for (int px = 0; px < sx && ok; px++)
            {
                Phase ph = { plan_phase_axis(IH, KH, OH, sy, out_pad[0], py), plan_phase_axis(IW, KW, OW, sx, out_pad[2], px),
                             py, px, w_total };
                if (ph.y.J == 0 || ph.x.J == 0)
                    continue;    // no output pixel in this phase
                if (ph.y.T == 0 || ph.x.T == 0)
                    ok = false;    // bias-only pixels: left to the dense form below
                w_total += ((size_t)OC * ph.y.T * ph.x.T * run + 255) & ~(size_t)255;
                phases.push_back(ph);
            }
        auto run_phase = [&](const Phase& ph, void* wbuf, bool dry) {
            tb200_tensor xin = *input, wsub = *weight;
            xin.owns = wsub.owns = false;
            xin.data       = reinterpret_cast<uint8_t*>(input->data) + ((size_t)ph.y.start * IW + ph.x.start) * run;
            xin.shape[1]   = ph.y.len;
            xin.shape[2]   = ph.x.len;
            xin.contiguous = false;
            wsub.data      = wbuf;
            wsub.shape[1]  = ph.y.T;
            wsub.shape[2]  = ph.x.T;
            wsub.bytes     = (size_t)OC * ph.y.T * ph.x.T * run;
            wsub.stride[2] = IC;
            wsub.stride[1] = (int64_t)ph.x.T * IC;
            wsub.stride[0] = (int64_t)ph.y.T * ph.x.T * IC;
            const int32_t pad[4]   = { ph.y.pad0, ph.y.pad1, ph.x.pad0, ph.x.pad1 };
            const ConvOutView view = { ph.y.J, ph.x.J, sy, sx, ph.py, ph.px, 0, 0 };
            return conv2d_impl(ctx, &xin, &wsub, bias, input_zp, weight_zp, pad, one, one, epilogue, output, &view, dry, false);
        };
        if (ok && !phases.empty())
        {
            // the probe only looks at shapes and alignment; any 256-byte aligned address stands in for the weights
            for (const Phase& ph : phases)
            {
                st = run_phase(ph, weight->data, true);
                if (st == kNeedsDenseOutput)
                {
                    ok = false;
                    break;
                }
                if (st != TB200_OK)
                    return st;
            }
        }
        if (ok && !phases.empty())
        {
            st = ensure_stage(ctx, w_total);
            if (st != TB200_OK)
                return st;
            uint8_t* wbase = reinterpret_cast<uint8_t*>(ctx->stage);
            // all sub-kernels in one launch; the copy unit is 16 bytes when the channel run allows it, else one element
            const size_t unit_bytes = vec ? 16 : es;
            const int units         = (int)(run / unit_bytes);
            PhaseWeights pw;
            pw.count    = (int)phases.size();
            pw.first[0] = 0;
            for (int i = 0; i < pw.count; i++)
            {
                const Phase& ph = phases[i];
                pw.ky0[i] = ph.y.k0; pw.Ty[i] = ph.y.T; pw.kx0[i] = ph.x.k0; pw.Tx[i] = ph.x.T;
                pw.out_off[i]   = (long long)(ph.w_off / unit_bytes);
                pw.first[i + 1] = pw.first[i] + (long long)OC * ph.y.T * ph.x.T * units;
            }
            const int block = 256;
            const int grid  = grid_for(ctx, pw.first[pw.count], block);
            if (vec)
                mirror_phase_weights_kernel<uint4><<<grid, block, 0, ctx->stream>>>(
                    reinterpret_cast<const uint4*>(weight->data), reinterpret_cast<uint4*>(wbase), OC, KH, KW, units, sy, sx, pw);
            else if (es == 1)
                mirror_phase_weights_kernel<uint8_t><<<grid, block, 0, ctx->stream>>>(
                    reinterpret_cast<const uint8_t*>(weight->data), wbase, OC, KH, KW, units, sy, sx, pw);
            else
                mirror_phase_weights_kernel<uint16_t><<<grid, block, 0, ctx->stream>>>(
                    reinterpret_cast<const uint16_t*>(weight->data), reinterpret_cast<uint16_t*>(wbase), OC, KH, KW, units, sy,
                    sx, pw);
            st = post_launch(ctx, "transpose_conv_phase_weights", 1);
            if (st != TB200_OK)
                return st;
            for (const Phase& ph : phases)
            {
                st = run_phase(ph, wbase + ph.w_off, false);
                if (st != TB200_OK)
                    return st == kNeedsDenseOutput ? fail(ctx, TB200_INTERNAL, "OpTransposeConv2d: phase plan changed") : st;
            }
            return TB200_OK;
        }
    }

    // ---- dense form: a stride-1 CONV2D over the input spread out by the stride, with the whole kernel mirrored
    const bool spread = sy > 1 || sx > 1;
    const int DH = (IH - 1) * sy + 1, DW = (IW - 1) * sx + 1;
    const size_t w_bytes = ((size_t)OC * KH * KW * run + 255) & ~(size_t)255;
    const size_t d_bytes = spread ? (size_t)N * DH * DW * run : 0;
    st                   = ensure_stage(ctx, w_bytes + d_bytes + 256);
    if (st != TB200_OK)
        return st;
    uint8_t* wm = reinterpret_cast<uint8_t*>(ctx->stage);
    uint8_t* dx = wm + w_bytes;
    int launches = 1;
    launch_mirror(ctx, weight->data, wm, OC, KH, KW, IC, es, vec, 0, 1, KH, 0, 1, KW);
    if (spread)
    {
        launches = 2;
        // floating types have zero point 0, whose bit pattern is 0 in every format
        const uint32_t b  = (uint32_t)(uint8_t)(int8_t)input_zp;
        const uint32_t b4 = es == 1 ? b * 0x01010101u : 0u;
        if (vec)
            launch_spread<uint4>(ctx, input->data, dx, N, IH, IW, (int)(run / 16), DH, DW, sy, sx, make_uint4(b4, b4, b4, b4));
        else if (es == 1)
            launch_spread<uint8_t>(ctx, input->data, dx, N, IH, IW, IC, DH, DW, sy, sx, (uint8_t)b);
        else if (es == 2)
            launch_spread<uint16_t>(ctx, input->data, dx, N, IH, IW, IC, DH, DW, sy, sx, (uint16_t)0);
        else
            launch_spread<uint32_t>(ctx, input->data, dx, N, IH, IW, IC, DH, DW, sy, sx, 0u);
    }
    st = post_launch(ctx, "transpose_conv_staging", launches);
    if (st != TB200_OK)
        return st;

    tb200_tensor din = *input, wmir = *weight;
    din.owns = wmir.owns = false;
    wmir.data            = wm;
    if (spread)
    {
        din.data      = dx;
        din.shape[1]  = DH;
        din.shape[2]  = DW;
        din.bytes     = d_bytes;
        din.stride[3] = 1;
        din.stride[2] = IC;
        din.stride[1] = (int64_t)DW * IC;
        din.stride[0] = (int64_t)DH * DW * IC;
    }
    const int32_t pad[4] = { KH - 1 + out_pad[0], KH - 1 + out_pad[1], KW - 1 + out_pad[2], KW - 1 + out_pad[3] };
    // (the mirrored weights live in staging that the next call overwrites: nothing derived from them is cached)
    st = conv2d_impl(ctx, &din, &wmir, bias, input_zp, weight_zp, pad, one, one, epilogue, output, nullptr, false, false);
    if (st != TB200_OK && ctx->err.compare(0, 8, "OpConv2d") == 0)
        ctx->err = "OpTransposeConv2d (as CONV2D): " + ctx->err;
    return st;
}

// =================================================================================================== DEPTHWISE
extern "C" tb200_status tb200_depthwise_conv2d(tb200_ctx* ctx, const tb200_tensor* input, const tb200_tensor* weight,
                                               const tb200_tensor* bias, int32_t input_zp, int32_t weight_zp,
                                               const int32_t pad[4], const int32_t stride[2], const int32_t dilation[2],
                                               const tb200_epilogue* epilogue, tb200_tensor* output)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !input || !weight || !bias || !output || !pad || !stride || !dilation,
                   "OpDepthwiseConv2d: null operand");
    TB200_ERROR_IF(ctx, !all_contiguous({ input, weight, bias, output }), "%s: zero-copy views are accepted only as the CONV2D input; this operand must be contiguous", "OpDepthwiseConv2d");
    TB200_ERROR_IF(ctx, input->rank != 4 || weight->rank != 4 || output->rank != 4 || bias->rank != 1,
                   "OpDepthwiseConv2d: input, weight and output must be rank 4 and bias rank 1");
    const int N = input->shape[0], IH = input->shape[1], IW = input->shape[2], C = input->shape[3];
    const int KH = weight->shape[0], KW = weight->shape[1], M = weight->shape[3];
    const int OH = output->shape[1], OW = output->shape[2];
    // kernel dims start at offset 0 of the weight shape (reference_model/src/ops/tensor_ops.cpp:1139-1169)
    tb200_status st = check_conv_attr(ctx, "OpDepthwiseConv2d", IH, IW, OH, OW, KH, KW, pad, stride, dilation);
    if (st != TB200_OK)
        return st;
    // OpDepthwiseConv2d::eval ERROR_IFs (:1196-1205)
    TB200_ERROR_IF(ctx, N != output->shape[0], "OpDepthwiseConv2d: tensor batch mismatch %d != %d", N, output->shape[0]);
    TB200_ERROR_IF(ctx, weight->shape[2] != C, "OpDepthwiseConv2d: tensor input channel mismatch %d != %d",
                   weight->shape[2], C);
    TB200_ERROR_IF(ctx, C * M != output->shape[3], "OpDepthwiseConv2d: tensor output channel mismatch %d != %d", C * M,
                   output->shape[3]);
    TB200_ERROR_IF(ctx, bias->shape[0] != C * M && bias->shape[0] != 1,
                   "OpDepthwiseConv2d: bias channels mismatch %d != %d", bias->shape[0], C * M);
    const bool int_path = input->dtype == TB200_INT8;
    TB200_ERROR_IF(ctx, weight->dtype != input->dtype, "OpDepthwiseConv2d: input and weight dtypes differ");
    if (int_path)
        TB200_ERROR_IF(ctx, bias->dtype != TB200_INT32, "OpDepthwiseConv2d: INT8 convolution needs an INT32 bias");
    else
    {
        TB200_ERROR_IF(ctx, !dtype_is_float(input->dtype) && !dtype_is_fp8(input->dtype),
                       "OpDepthwiseConv2d: unsupported input dtype");
        if (dtype_is_fp8(input->dtype))    // <FP8, FP8, FP16, FP16>, reference_model/src/ops/tensor_ops.cpp:2250-2251
            TB200_ERROR_IF(ctx, bias->dtype != TB200_FP16 || output->dtype != TB200_FP16,
                           "OpDepthwiseConv2d: an FP8 convolution has an FP16 bias and output");
        else
            TB200_ERROR_IF(ctx, bias->dtype != input->dtype || output->dtype != input->dtype,
                           "OpDepthwiseConv2d: floating bias and output must have the input dtype");
        TB200_ERROR_IF(ctx, input_zp != 0, "Input zero point must be zero for non int8_t data");
        TB200_ERROR_IF(ctx, weight_zp != 0, "Weight zero point must be zero for non int8_t data");
    }
    TB200_ERROR_IF(ctx, input_zp < -128 || input_zp > 127 || weight_zp < -128 || weight_zp > 127,
                   "OpDepthwiseConv2d: zero point outside the int8 range");
    EpiInfo epi;
    st = parse_epilogue(ctx, "OpDepthwiseConv2d", epilogue, int_path, C * M, output->dtype, &epi);
    if (st != TB200_OK)
        return st;
    if (numel(output) == 0)
        return TB200_OK;
    cache_note_write(ctx, output->data, output->bytes);
    ConvDev d;
    memset(&d, 0, sizeof(d));
    d.N = N; d.IH = IH; d.IW = IW; d.IC = C; d.OH = OH; d.OW = OW; d.OC = C * M; d.KH = KH; d.KW = KW; d.M = M;
    d.in_sn = input->stride[0]; d.in_sh = input->stride[1]; d.in_sw = input->stride[2];
    d.pad_t = pad[0]; d.pad_l = pad[2]; d.sy = stride[0]; d.sx = stride[1]; d.dy = dilation[0]; d.dx = dilation[1];
    d.in_zp = input_zp; d.w_zp = weight_zp; d.bias_n = bias->shape[0];
    fill_conv_dev(&d, epi);
    const int block = 256;
    if (int_path && M == 1 && C % 16 == 0 && KH == 3 && KW == 3 && dilation[0] == 1 && dilation[1] == 1 && ctx->policy == 0 &&
        ((reinterpret_cast<uintptr_t>(input->data) | reinterpret_cast<uintptr_t>(weight->data) |
          reinterpret_cast<uintptr_t>(output->data)) & 15) == 0)
    {
        // sixteen channels per thread
        const int grid   = grid_for(ctx, numel(output) / 16, block);
        const int8_t* in = reinterpret_cast<const int8_t*>(input->data);
        const int8_t* w  = reinterpret_cast<const int8_t*>(weight->data);
        const int32_t* b = reinterpret_cast<const int32_t*>(bias->data);
        switch (dtype_size(output->dtype))
        {
            case 1:
                depthwise3x3_i8x16_kernel<int8_t><<<grid, block, 0, ctx->stream>>>(in, w, b, reinterpret_cast<int8_t*>(output->data), d, ctx->d_status);
                break;
            case 2:
                depthwise3x3_i8x16_kernel<int16_t><<<grid, block, 0, ctx->stream>>>(in, w, b, reinterpret_cast<int16_t*>(output->data), d, ctx->d_status);
                break;
            default:
                depthwise3x3_i8x16_kernel<int32_t><<<grid, block, 0, ctx->stream>>>(in, w, b, reinterpret_cast<int32_t*>(output->data), d, ctx->d_status);
                break;
        }
        return post_launch(ctx, "depthwise3x3_i8x16");
    }
    if (int_path)
    {
        const int grid    = grid_for(ctx, numel(output), block);
        const int8_t* in  = reinterpret_cast<const int8_t*>(input->data);
        const int8_t* w   = reinterpret_cast<const int8_t*>(weight->data);
        const int32_t* b  = reinterpret_cast<const int32_t*>(bias->data);
        switch (dtype_size(output->dtype))
        {
            case 1:
                depthwise_direct_i8_kernel<int8_t><<<grid, block, 0, ctx->stream>>>(in, w, b, reinterpret_cast<int8_t*>(output->data), d, ctx->d_status);
                break;
            case 2:
                depthwise_direct_i8_kernel<int16_t><<<grid, block, 0, ctx->stream>>>(in, w, b, reinterpret_cast<int16_t*>(output->data), d, ctx->d_status);
                break;
            default:
                depthwise_direct_i8_kernel<int32_t><<<grid, block, 0, ctx->stream>>>(in, w, b, reinterpret_cast<int32_t*>(output->data), d, ctx->d_status);
                break;
        }
        return post_launch(ctx, "depthwise_direct_i8");
    }
    const bool x8 = (M == 1) && (C % 8 == 0) && (input->dtype == TB200_FP16 || input->dtype == TB200_BF16) && ctx->policy == 0 &&
                    ((reinterpret_cast<uintptr_t>(input->data) | reinterpret_cast<uintptr_t>(weight->data) |
                      reinterpret_cast<uintptr_t>(output->data)) & 15) == 0;
    if (x8)
    {
        const int grid = grid_for(ctx, numel(output) / 8, block);
        if (d.KH == 3 && d.KW == 3 && d.dy == 1 && d.dx == 1)
        {
            if (input->dtype == TB200_FP16)
                depthwise3x3_fp_x8_kernel<__half><<<grid, block, 0, ctx->stream>>>(
                    reinterpret_cast<const __half*>(input->data), reinterpret_cast<const __half*>(weight->data),
                    reinterpret_cast<const __half*>(bias->data), reinterpret_cast<__half*>(output->data), d);
            else
                depthwise3x3_fp_x8_kernel<__nv_bfloat16><<<grid, block, 0, ctx->stream>>>(
                    reinterpret_cast<const __nv_bfloat16*>(input->data), reinterpret_cast<const __nv_bfloat16*>(weight->data),
                    reinterpret_cast<const __nv_bfloat16*>(bias->data), reinterpret_cast<__nv_bfloat16*>(output->data), d);
            return post_launch(ctx, "depthwise_fp_x8");
        }
        if (input->dtype == TB200_FP16)
            depthwise_fp_x8_kernel<__half><<<grid, block, 0, ctx->stream>>>(
                reinterpret_cast<const __half*>(input->data), reinterpret_cast<const __half*>(weight->data),
                reinterpret_cast<const __half*>(bias->data), reinterpret_cast<__half*>(output->data), d);
        else
            depthwise_fp_x8_kernel<__nv_bfloat16><<<grid, block, 0, ctx->stream>>>(
                reinterpret_cast<const __nv_bfloat16*>(input->data), reinterpret_cast<const __nv_bfloat16*>(weight->data),
                reinterpret_cast<const __nv_bfloat16*>(bias->data), reinterpret_cast<__nv_bfloat16*>(output->data), d);
        return post_launch(ctx, "depthwise_fp_x8");
    }
    const int grid = grid_for(ctx, numel(output), block);
    if (input->dtype == TB200_FP8E4M3)
        depthwise_direct_fp_kernel<__nv_fp8_e4m3, __half><<<grid, block, 0, ctx->stream>>>(
            reinterpret_cast<const __nv_fp8_e4m3*>(input->data), reinterpret_cast<const __nv_fp8_e4m3*>(weight->data),
            reinterpret_cast<const __half*>(bias->data), reinterpret_cast<__half*>(output->data), d);
    else if (input->dtype == TB200_FP8E5M2)
        depthwise_direct_fp_kernel<__nv_fp8_e5m2, __half><<<grid, block, 0, ctx->stream>>>(
            reinterpret_cast<const __nv_fp8_e5m2*>(input->data), reinterpret_cast<const __nv_fp8_e5m2*>(weight->data),
            reinterpret_cast<const __half*>(bias->data), reinterpret_cast<__half*>(output->data), d);
    else if (input->dtype == TB200_FP16)
        depthwise_direct_fp_kernel<__half><<<grid, block, 0, ctx->stream>>>(
            reinterpret_cast<const __half*>(input->data), reinterpret_cast<const __half*>(weight->data),
            reinterpret_cast<const __half*>(bias->data), reinterpret_cast<__half*>(output->data), d);
    else if (input->dtype == TB200_BF16)
        depthwise_direct_fp_kernel<__nv_bfloat16><<<grid, block, 0, ctx->stream>>>(
            reinterpret_cast<const __nv_bfloat16*>(input->data), reinterpret_cast<const __nv_bfloat16*>(weight->data),
            reinterpret_cast<const __nv_bfloat16*>(bias->data), reinterpret_cast<__nv_bfloat16*>(output->data), d);
    else
        depthwise_direct_fp_kernel<float><<<grid, block, 0, ctx->stream>>>(
            reinterpret_cast<const float*>(input->data), reinterpret_cast<const float*>(weight->data),
            reinterpret_cast<const float*>(bias->data), reinterpret_cast<float*>(output->data), d);
    return post_launch(ctx, "depthwise_direct_fp");
}

// =================================================================================================== MATMUL
extern "C" tb200_status tb200_matmul(tb200_ctx* ctx, const tb200_tensor* a, const tb200_tensor* b, int32_t a_zp,
                                     int32_t b_zp, const tb200_epilogue* epilogue, tb200_tensor* output)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !a || !b || !output, "OpMatMul: null operand");
    TB200_ERROR_IF(ctx, !all_contiguous({ a, b, output }), "%s: zero-copy views are accepted only as the CONV2D input; this operand must be contiguous", "OpMatMul");
    // OpMatMul::checkTensorAttributes (reference_model/src/ops/tensor_ops.cpp:1347-1420)
    TB200_ERROR_IF(ctx, a->rank != 3 || b->rank != 3 || output->rank != 3, "OpMatMul: operands must be rank 3");
    const int N = a->shape[0], H = a->shape[1], C = a->shape[2], W = b->shape[2];
    TB200_ERROR_IF(ctx, b->shape[0] != N || output->shape[0] != N, "OpMatMul operator a.shape[0], b.shape[0] and output.shape[0] should match");
    TB200_ERROR_IF(ctx, output->shape[1] != H, "OpMatMul operator output.shape[1] should match a.shape[1]");
    TB200_ERROR_IF(ctx, b->shape[1] != C, "OpMatMul operator a.shape[2] should match b.shape[1]");
    TB200_ERROR_IF(ctx, output->shape[2] != W, "OpMatMul operator output.shape[2] should match b.shape[2]");
    // the two fp8 formats may be paired freely (reference_model/src/ops/tensor_ops.cpp:2263-2270)
    const bool fp8 = dtype_is_fp8(a->dtype) && dtype_is_fp8(b->dtype);
    TB200_ERROR_IF(ctx, a->dtype != b->dtype && !fp8, "OpMatMul: operand dtypes differ");
    const bool int_path = a->dtype == TB200_INT8;
    if (!int_path)
    {
        TB200_ERROR_IF(ctx, !dtype_is_float(a->dtype) && !fp8, "OpMatMul: unsupported dtype");
        // :1433-1434
        TB200_ERROR_IF(ctx, a_zp != 0, "OpMatMul: A zeropoint must be zero for non int8_t data");
        TB200_ERROR_IF(ctx, b_zp != 0, "OpMatMul: B zeropoint must be zero for non int8_t data");
        if (fp8)
            TB200_ERROR_IF(ctx, output->dtype != TB200_FP16 && output->dtype != TB200_FP32,
                           "OpMatMul: the output of an FP8 MATMUL must be FP16 or FP32");
        else
            TB200_ERROR_IF(ctx, output->dtype != a->dtype && output->dtype != TB200_FP32,
                           "OpMatMul: output dtype must be the input dtype or FP32");
    }
    TB200_ERROR_IF(ctx, a_zp < -128 || a_zp > 127 || b_zp < -128 || b_zp > 127, "OpMatMul: zero point outside the int8 range");
    EpiInfo epi;
    tb200_status st = parse_epilogue(ctx, "OpMatMul", epilogue, int_path, W, output->dtype, &epi);
    if (st != TB200_OK)
        return st;
    TB200_ERROR_IF(ctx, epi.has_rescale || epi.has_clamp, "OpMatMul: fused epilogues are not available for MATMUL");
    if (numel(output) == 0)
        return TB200_OK;
    cache_note_write(ctx, output->data, output->bytes);

    if (a->dtype == TB200_FP32)
    {
        if (ctx->policy == 0)
            return sgemm_f32_launch(ctx, reinterpret_cast<const float*>(a->data), reinterpret_cast<const float*>(b->data),
                                    reinterpret_cast<float*>(output->data), N, H, C, W);
    }
    else if (ctx->policy == 0)
    {
        TcProblem q;
        memset(&q, 0, sizeof(q));
        q.in_dtype    = a->dtype;
        q.b_fp8_dtype = (fp8 && b->dtype != a->dtype) ? (int)b->dtype : 0;
        q.a           = a->data;
        q.N = 1; q.IH = N; q.IW = H; q.IC = C;
        q.OH = N; q.OW = H; q.OC = W;
        q.KH = 1; q.KW = 1;
        q.stride_y = q.stride_x = q.dil_y = q.dil_x = 1;
        q.b          = b->data;
        q.b_mn_major = 1;
        q.out        = output->data;
        q.epi        = int_path ? TC_EPI_I32 : TC_EPI_FLOAT;
        fill_tc_epilogue(&q, epi, output->dtype);
        // B rows that are not a multiple of 16 bytes cannot be described to TMA: they are copied once into scratch
        // with a padded pitch (the pad columns lie outside the tensor map and read as zero)
        const size_t es_in  = dtype_size(a->dtype);
        const bool pad_b    = ((size_t)W * es_in) % 16 != 0;
        const int64_t b_ld  = pad_b ? (int64_t)((((size_t)W * es_in + 15) & ~(size_t)15) / es_in) : 0;
        const size_t padb_bytes = pad_b ? (((size_t)N * C * b_ld * es_in + 255) & ~(size_t)255) : 0;
        q.b_ld = b_ld;
        std::string why;
        // (the CTA-pair kernel takes K tails the single-CTA kernel does not)
        if (tc_gemm_pair_supported(q, ctx->num_sms) || tc_gemm_supported(q, &why))
        {
            const bool need_sums = int_path && (a_zp != 0 || b_zp != 0);
            const int Wpad       = (W + 255) / 256 * 256;
            const size_t rows = (size_t)N * H, cols = (size_t)N * Wpad;
            const size_t sums_bytes = need_sums ? (((rows + 3) & ~(size_t)3) + cols) * sizeof(int32_t) : 0;
            if (pad_b || need_sums)
            {
                st = ensure_scratch(ctx, padb_bytes + sums_bytes);
                if (st != TB200_OK)
                    return st;
            }
            if (pad_b)
            {
                TB200_CUDA_CHECK(ctx, cudaMemcpy2DAsync(ctx->scratch, (size_t)b_ld * es_in, b->data, (size_t)W * es_in,
                                                        (size_t)W * es_in, (size_t)N * C, cudaMemcpyDeviceToDevice,
                                                        ctx->stream));
                q.b = ctx->scratch;
            }
            if (need_sums)
            {
                int32_t* row_corr = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(ctx->scratch) + padb_bytes);
                int32_t* col_corr = row_corr + ((rows + 3) & ~(size_t)3);
                // The CTA-pair kernel takes the sums from its own tiles while they sit in shared memory: both of them,
                // shared between tiles through flags in global memory (no pass over A or B at all), or the row sums only.
                // The flags carry a per-launch epoch, which a replayed CUDA graph would repeat: not while capturing.
                const bool pair      = tc_gemm_pair_supported(q, ctx->num_sms);
                // Sharing sums between tiles needs every CTA pair of the grid resident at once, which holds on a GPU
                // this context has to itself; tb200_set_shared_gpu(ctx, 1) keeps the sums in separate kernels.
                const bool fuse_all  = pair && !ctx->capturing && !ctx->shared_gpu && diag_env_int("TB200_FUSE_SUMS", 1) != 0;
                const bool fuse_rows = !fuse_all && b_zp != 0 && pair && diag_env_int("TB200_FUSE_ROW_SUMS", 1) != 0;
                if (fuse_all)
                {
                    const size_t words = (size_t)N * 2 * ((H + 255) / 256 + (W + 255) / 256);
                    if (words > ctx->pair_flag_words)
                    {
                        release_block(ctx, ctx->pair_flags);
                        ctx->pair_flags      = nullptr;
                        ctx->pair_flag_words = 0;
                        TB200_CUDA_CHECK(ctx, cudaMalloc(reinterpret_cast<void**>(&ctx->pair_flags), words * sizeof(uint32_t)));
                        TB200_CUDA_CHECK(ctx, cudaMemset(ctx->pair_flags, 0, words * sizeof(uint32_t)));
                        ctx->pair_flag_words = words;
                        ctx->pair_epoch      = 0;
                    }
                    q.fuse_row_sums = 2;
                    q.a_zp          = a_zp;
                    q.b_zp          = b_zp;
                    if (ctx->pair_epoch == 0xffffffffu)
                    {
                        // the epoch is about to repeat: start over from clean flags
                        TB200_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
                        TB200_CUDA_CHECK(ctx, cudaMemset(ctx->pair_flags, 0, ctx->pair_flag_words * sizeof(uint32_t)));
                        ctx->pair_epoch = 0;
                    }
                    q.sum_flags     = ctx->pair_flags;
                    q.sum_epoch     = ++ctx->pair_epoch;
                    q.row_corr      = b_zp != 0 ? row_corr : nullptr;
                    if (a_zp != 0)
                    {
                        q.corr         = col_corr;
                        q.corr_stride  = Wpad;
                        q.corr_ystride = Wpad;
                    }
                    return tc_gemm_launch(ctx, q);
                }
                if (fuse_rows)
                {
                    q.fuse_row_sums = 1;
                    q.a_zp          = a_zp;
                    q.b_zp          = b_zp;
                }
                else if (b_zp != 0)
                    q.row_corr = row_corr;
                if (a_zp != 0)
                {
                    q.corr         = col_corr;
                    q.corr_stride  = Wpad;
                    q.corr_ystride = Wpad;
                }
                // zero-point sums of batches [lo, hi) on `stream`
                auto launch_sums = [&](cudaStream_t stream, int lo, int hi) -> tb200_status {
                    const int nb  = hi - lo;
                    int launches  = 0;
                    if (b_zp != 0 && !fuse_rows)
                    {
                        const int block = 256;
                        matmul_row_corr_kernel<<<grid_for(ctx, (int64_t)nb * H * 32, block), block, 0, stream>>>(
                            reinterpret_cast<const int8_t*>(a->data) + (size_t)lo * H * C, row_corr + (size_t)lo * H,
                            (int64_t)nb * H, C, a_zp, b_zp);
                        launches++;
                    }
                    if (a_zp != 0)
                    {
                        TB200_CUDA_CHECK(ctx, cudaMemsetAsync(col_corr + (size_t)lo * Wpad, 0,
                                                              (size_t)nb * Wpad * sizeof(int32_t), stream));
                        const int xblocks = (W + 511) / 512;
                        int ksplit     = std::max(1, std::min((C + 63) / 64, (4 * ctx->num_sms) / std::max(1, xblocks * nb)));
                        const int kper = ((C + ksplit - 1) / ksplit + 7) / 8 * 8;
                        ksplit         = (C + kper - 1) / kper;
                        dim3 grid(xblocks, ksplit, nb);
                        matmul_col_corr_kernel<<<grid, 256, 0, stream>>>(
                            reinterpret_cast<const int8_t*>(b->data) + (size_t)lo * C * W, col_corr + (size_t)lo * Wpad, C, W,
                            Wpad, kper, a_zp);
                        launches++;
                    }
                    return post_launch(ctx, "matmul_zp_sums", launches);
                };
                // (Running the sums of later batches on a second stream beside tile-range pieces of the GEMM was
                // measured slower than this plain sequence: the memory-bound sums slow the concurrent GEMM by more
                // than they hide.)
                st = launch_sums(ctx->stream, 0, N);
                if (st != TB200_OK)
                    return st;
                return tc_gemm_launch(ctx, q);
            }
            return tc_gemm_launch(ctx, q);
        }
    }

    const int block = 256;
    const int grid  = grid_for(ctx, numel(output), block);
    if (int_path)
        matmul_direct_i8_kernel<<<grid, block, 0, ctx->stream>>>(reinterpret_cast<const int8_t*>(a->data),
                                                                 reinterpret_cast<const int8_t*>(b->data),
                                                                 reinterpret_cast<int32_t*>(output->data), N, H, C, W, a_zp, b_zp);
    else if (fp8)
    {
#define TB200_FP8_MM(TA, TBB, TO)                                                                                     \
    matmul_direct_fp_kernel<TA, TO, TBB><<<grid, block, 0, ctx->stream>>>(                                             \
        reinterpret_cast<const TA*>(a->data), reinterpret_cast<const TBB*>(b->data), reinterpret_cast<TO*>(output->data), \
        N, H, C, W)
        const bool a43 = a->dtype == TB200_FP8E4M3, b43 = b->dtype == TB200_FP8E4M3, o16 = output->dtype == TB200_FP16;
        if (a43 && b43)
        {
            if (o16) TB200_FP8_MM(__nv_fp8_e4m3, __nv_fp8_e4m3, __half); else TB200_FP8_MM(__nv_fp8_e4m3, __nv_fp8_e4m3, float);
        }
        else if (a43)
        {
            if (o16) TB200_FP8_MM(__nv_fp8_e4m3, __nv_fp8_e5m2, __half); else TB200_FP8_MM(__nv_fp8_e4m3, __nv_fp8_e5m2, float);
        }
        else if (b43)
        {
            if (o16) TB200_FP8_MM(__nv_fp8_e5m2, __nv_fp8_e4m3, __half); else TB200_FP8_MM(__nv_fp8_e5m2, __nv_fp8_e4m3, float);
        }
        else
        {
            if (o16) TB200_FP8_MM(__nv_fp8_e5m2, __nv_fp8_e5m2, __half); else TB200_FP8_MM(__nv_fp8_e5m2, __nv_fp8_e5m2, float);
        }
#undef TB200_FP8_MM
    }
    else if (a->dtype == TB200_FP32)
        matmul_direct_fp_kernel<float, float><<<grid, block, 0, ctx->stream>>>(
            reinterpret_cast<const float*>(a->data), reinterpret_cast<const float*>(b->data),
            reinterpret_cast<float*>(output->data), N, H, C, W);
    else if (a->dtype == TB200_FP16 && output->dtype == TB200_FP16)
        matmul_direct_fp_kernel<__half, __half><<<grid, block, 0, ctx->stream>>>(
            reinterpret_cast<const __half*>(a->data), reinterpret_cast<const __half*>(b->data),
            reinterpret_cast<__half*>(output->data), N, H, C, W);
    else if (a->dtype == TB200_FP16)
        matmul_direct_fp_kernel<__half, float><<<grid, block, 0, ctx->stream>>>(
            reinterpret_cast<const __half*>(a->data), reinterpret_cast<const __half*>(b->data),
            reinterpret_cast<float*>(output->data), N, H, C, W);
    else if (output->dtype == TB200_BF16)
        matmul_direct_fp_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, block, 0, ctx->stream>>>(
            reinterpret_cast<const __nv_bfloat16*>(a->data), reinterpret_cast<const __nv_bfloat16*>(b->data),
            reinterpret_cast<__nv_bfloat16*>(output->data), N, H, C, W);
    else
        matmul_direct_fp_kernel<__nv_bfloat16, float><<<grid, block, 0, ctx->stream>>>(
            reinterpret_cast<const __nv_bfloat16*>(a->data), reinterpret_cast<const __nv_bfloat16*>(b->data),
            reinterpret_cast<float*>(output->data), N, H, C, W);
    return post_launch(ctx, "matmul_direct");
}

// =================================================================================================== RESCALE
template <typename TIn>
static void launch_rescale_out(tb200_ctx* ctx, const tb200_tensor* in, tb200_tensor* out, int64_t n, int C,
                               const RescaleDev& r, bool vec4)
{
    const int block = 256;
    const TIn* ip   = reinterpret_cast<const TIn*>(in->data);
#define TB200_RS_LAUNCH(TOUT)                                                                                          \
    if (vec4)                                                                                                          \
        rescale_kernel<TIn, TOUT, 4><<<grid_for(ctx, n / 4, block), block, 0, ctx->stream>>>(                          \
            ip, reinterpret_cast<TOUT*>(out->data), n, C, r, ctx->d_status);                                           \
    else                                                                                                               \
        rescale_kernel<TIn, TOUT, 1><<<grid_for(ctx, n, block), block, 0, ctx->stream>>>(                              \
            ip, reinterpret_cast<TOUT*>(out->data), n, C, r, ctx->d_status);
    switch (dtype_size(out->dtype))
    {
        case 1:
            TB200_RS_LAUNCH(int8_t)
            break;
        case 2:
            TB200_RS_LAUNCH(int16_t)
            break;
        default:
            TB200_RS_LAUNCH(int32_t)
            break;
    }
#undef TB200_RS_LAUNCH
}

extern "C" tb200_status tb200_rescale(tb200_ctx* ctx, const tb200_tensor* input, const tb200_rescale_attr* attr,
                                      tb200_tensor* output)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !input || !attr || !output, "OpRescale: null operand");
    TB200_ERROR_IF(ctx, !all_contiguous({ input, output, attr->multiplier, attr->shift }), "%s: zero-copy views are accepted only as the CONV2D input; this operand must be contiguous", "OpRescale");
    TB200_ERROR_IF(ctx, !same_shape(input, output), "OpRescale: input and output shapes differ");
    const int C = input->rank > 0 ? input->shape[input->rank - 1] : 1;
    RescaleDev r;
    tb200_status st = make_rescale_dev(ctx, attr, input->dtype, output->dtype, C, &r);
    if (st != TB200_OK)
        return st;
    const int64_t n = numel(input);
    if (n == 0)
        return TB200_OK;
    cache_note_write(ctx, output->data, output->bytes);
    const bool aligned = ((reinterpret_cast<uintptr_t>(input->data) | reinterpret_cast<uintptr_t>(output->data)) & 15) == 0;
    const bool vec4    = aligned && (n % 4 == 0) && (!attr->per_channel || C % 4 == 0);
    switch (dtype_size(input->dtype))
    {
        case 1:
            launch_rescale_out<int8_t>(ctx, input, output, n, C, r, vec4);
            break;
        case 2:
            launch_rescale_out<int16_t>(ctx, input, output, n, C, r, vec4);
            break;
        default:
            launch_rescale_out<int32_t>(ctx, input, output, n, C, r, vec4);
            break;
    }
    return post_launch(ctx, "rescale");
}

// =================================================================================================== CLAMP
extern "C" tb200_status tb200_clamp(tb200_ctx* ctx, const tb200_tensor* input, int32_t min_i, int32_t max_i, float min_f,
                                    float max_f, int32_t nan_ignore, tb200_tensor* output)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !input || !output, "OpClamp: null operand");
    TB200_ERROR_IF(ctx, !all_contiguous({ input, output }), "%s: zero-copy views are accepted only as the CONV2D input; this operand must be contiguous", "OpClamp");
    TB200_ERROR_IF(ctx, !same_shape(input, output) || input->dtype != output->dtype,
                   "OpClamp: input and output must have the same shape and dtype");
    const int64_t n = numel(input);
    const int block = 256;
    const int grid  = grid_for(ctx, std::max<int64_t>(1, n / 8), block);
    cache_note_write(ctx, output->data, output->bytes);
    switch (input->dtype)
    {
        case TB200_INT8:
            TB200_ERROR_IF(ctx, max_i < min_i, "OpClamp: max smaller than min");
            if (n)
                clamp_int_kernel<int8_t><<<grid, block, 0, ctx->stream>>>(reinterpret_cast<const int8_t*>(input->data), reinterpret_cast<int8_t*>(output->data), n, min_i, max_i);
            break;
        case TB200_INT16:
            TB200_ERROR_IF(ctx, max_i < min_i, "OpClamp: max smaller than min");
            if (n)
                clamp_int_kernel<int16_t><<<grid, block, 0, ctx->stream>>>(reinterpret_cast<const int16_t*>(input->data), reinterpret_cast<int16_t*>(output->data), n, min_i, max_i);
            break;
        case TB200_FP16:
        case TB200_BF16:
        case TB200_FP32:
            TB200_ERROR_IF(ctx, std::isnan(min_f) || std::isnan(max_f), "OpClamp: min/max cannot be NaN");
            TB200_ERROR_IF(ctx, max_f < min_f, "OpClamp: max smaller than min");
            if (n)
            {
                if (input->dtype == TB200_FP16)
                    clamp_fp_kernel<__half><<<grid, block, 0, ctx->stream>>>(reinterpret_cast<const __half*>(input->data), reinterpret_cast<__half*>(output->data), n, min_f, max_f, nan_ignore);
                else if (input->dtype == TB200_BF16)
                    clamp_fp_kernel<__nv_bfloat16><<<grid, block, 0, ctx->stream>>>(reinterpret_cast<const __nv_bfloat16*>(input->data), reinterpret_cast<__nv_bfloat16*>(output->data), n, min_f, max_f, nan_ignore);
                else
                    clamp_fp_kernel<float><<<grid, block, 0, ctx->stream>>>(reinterpret_cast<const float*>(input->data), reinterpret_cast<float*>(output->data), n, min_f, max_f, nan_ignore);
            }
            break;
        default:
            // the reference instantiates CLAMP for INT8, INT16 and the floating types only
            return fail(ctx, TB200_ERROR, "OpClamp: unsupported TOSA_REF_TYPE %d", (int)input->dtype);
    }
    if (n == 0)
        return TB200_OK;
    return post_launch(ctx, "clamp");
}

// =================================================================================================== ADD
extern "C" tb200_status tb200_add(tb200_ctx* ctx, const tb200_tensor* a, const tb200_tensor* b, tb200_tensor* output)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !a || !b || !output, "OpAdd: null operand");
    TB200_ERROR_IF(ctx, !all_contiguous({ a, b, output }), "%s: zero-copy views are accepted only as the CONV2D input; this operand must be contiguous", "OpAdd");
    // BinaryNodeBase::checkTensorAttributes / broadcast (reference_model/src/ops/ewise_binary.cpp:40-111)
    TB200_ERROR_IF(ctx, a->rank != b->rank || a->dtype != b->dtype, "Binary operator input types must match");
    TB200_ERROR_IF(ctx, output->rank != a->rank, "Binary operators ADD lhs input and output rank/shape must match");
    TB200_ERROR_IF(ctx, output->dtype != a->dtype, "Binary operator type doesn't match");
    BcastDev bc;
    memset(&bc, 0, sizeof(bc));
    bc.rank       = a->rank;
    bc.same_shape = 1;
    for (int i = 0; i < a->rank; i++)
    {
        int cs = a->shape[i];
        if (cs == 1)
            cs = b->shape[i];
        else
            TB200_ERROR_IF(ctx, b->shape[i] != 1 && b->shape[i] != cs,
                           "Broadcast_shape failure, input shapes are not compatible");
        TB200_ERROR_IF(ctx, cs != output->shape[i], "Broadcast_shape failure, calculated_shape and result_shape don't match");
        bc.oshape[i] = output->shape[i];
        if (a->shape[i] != output->shape[i] || b->shape[i] != output->shape[i])
            bc.same_shape = 0;
    }
    int64_t as = 1, bs = 1;
    for (int i = a->rank - 1; i >= 0; i--)
    {
        bc.astride[i] = (a->shape[i] == 1 && output->shape[i] != 1) ? 0 : as;
        bc.bstride[i] = (b->shape[i] == 1 && output->shape[i] != 1) ? 0 : bs;
        as *= a->shape[i];
        bs *= b->shape[i];
    }
    const int64_t n = numel(output);
    if (n == 0)
        return TB200_OK;
    cache_note_write(ctx, output->data, output->bytes);
    if (((reinterpret_cast<uintptr_t>(a->data) | reinterpret_cast<uintptr_t>(b->data) |
          reinterpret_cast<uintptr_t>(output->data)) & 15) != 0 && bc.same_shape)
    {
        // unaligned views take the indexed path
        bc.same_shape = 0;
    }
    const int block = 256;
    const int grid  = grid_for(ctx, bc.same_shape ? std::max<int64_t>(1, n / 4) : n, block);
    switch (a->dtype)
    {
        case TB200_INT32:
            add_kernel<int32_t><<<grid, block, 0, ctx->stream>>>(reinterpret_cast<const int32_t*>(a->data), reinterpret_cast<const int32_t*>(b->data), reinterpret_cast<int32_t*>(output->data), n, bc, ctx->d_status);
            break;
        case TB200_FP32:
            add_kernel<float><<<grid, block, 0, ctx->stream>>>(reinterpret_cast<const float*>(a->data), reinterpret_cast<const float*>(b->data), reinterpret_cast<float*>(output->data), n, bc, ctx->d_status);
            break;
        case TB200_FP16:
            add_kernel<__half><<<grid, block, 0, ctx->stream>>>(reinterpret_cast<const __half*>(a->data), reinterpret_cast<const __half*>(b->data), reinterpret_cast<__half*>(output->data), n, bc, ctx->d_status);
            break;
        case TB200_BF16:
            add_kernel<__nv_bfloat16><<<grid, block, 0, ctx->stream>>>(reinterpret_cast<const __nv_bfloat16*>(a->data), reinterpret_cast<const __nv_bfloat16*>(b->data), reinterpret_cast<__nv_bfloat16*>(output->data), n, bc, ctx->d_status);
            break;
        default:
            // integer ADD exists for INT32 only (reference_model/src/ops/op_factory.cpp:189-195)
            return fail(ctx, TB200_ERROR, "OpAdd: unsupported TOSA_REF_TYPE %d", (int)a->dtype);
    }
    return post_launch(ctx, "add");
}

extern "C" tb200_status tb200_residual_add(tb200_ctx* ctx, const tb200_tensor* a, const tb200_rescale_attr* a_attr,
                                           const tb200_tensor* b, const tb200_rescale_attr* b_attr,
                                           const tb200_rescale_attr* out_attr, int32_t has_clamp, int32_t clamp_min,
                                           int32_t clamp_max, tb200_tensor* output)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !a || !b || !output || !a_attr || !b_attr || !out_attr, "residual_add: null operand");
    TB200_ERROR_IF(ctx, !all_contiguous({ a, b, output }), "%s: zero-copy views are accepted only as the CONV2D input; this operand must be contiguous", "residual_add");
    TB200_ERROR_IF(ctx, !same_shape(a, b) || !same_shape(a, output), "residual_add: operand shapes differ");
    TB200_ERROR_IF(ctx, a->dtype != TB200_INT8 || b->dtype != TB200_INT8 || output->dtype != TB200_INT8,
                   "residual_add: INT8 tensors only");
    TB200_ERROR_IF(ctx, has_clamp && clamp_max < clamp_min, "OpClamp: max smaller than min");
    const int C = a->rank > 0 ? a->shape[a->rank - 1] : 1;
    ResidualDev r;
    memset(&r, 0, sizeof(r));
    tb200_status st = make_rescale_dev(ctx, a_attr, TB200_INT8, TB200_INT32, C, &r.ra);
    if (st == TB200_OK)
        st = make_rescale_dev(ctx, b_attr, TB200_INT8, TB200_INT32, C, &r.rb);
    if (st == TB200_OK)
        st = make_rescale_dev(ctx, out_attr, TB200_INT32, TB200_INT8, C, &r.ro);
    if (st != TB200_OK)
        return st;
    r.has_clamp = has_clamp;
    r.clamp_min = clamp_min;
    r.clamp_max = clamp_max;
    const int64_t n = numel(a);
    if (n == 0)
        return TB200_OK;
    cache_note_write(ctx, output->data, output->bytes);
    const bool aligned = ((reinterpret_cast<uintptr_t>(a->data) | reinterpret_cast<uintptr_t>(b->data) |
                           reinterpret_cast<uintptr_t>(output->data)) & 15) == 0;
    const bool pc = a_attr->per_channel || b_attr->per_channel || out_attr->per_channel;
    const int block = 256;
    const bool simple = !pc && a_attr->scale32 && b_attr->scale32 && out_attr->scale32 &&
                        a_attr->rounding_mode != TB200_INEXACT_ROUND && b_attr->rounding_mode != TB200_INEXACT_ROUND &&
                        out_attr->rounding_mode != TB200_INEXACT_ROUND && !a_attr->input_unsigned &&
                        !b_attr->input_unsigned && !out_attr->output_unsigned && ctx->policy == 0;
    if (simple && aligned && n % 16 == 0)
    {
        ResidualFast f;
        auto leg = [](const tb200_rescale_attr* at) {
            ResidualLeg l;
            l.mult         = reinterpret_cast<const int32_t*>(at->multiplier->data);
            l.shift        = reinterpret_cast<const int8_t*>(at->shift->data);
            l.zp_in        = (int32_t)(int8_t)at->input_zp;
            l.zp_out       = (int32_t)(int8_t)at->output_zp;
            l.double_round = at->rounding_mode == TB200_DOUBLE_ROUND;
            return l;
        };
        f.a = leg(a_attr);
        f.b = leg(b_attr);
        f.o = leg(out_attr);
        f.o.zp_in = 0;    // INT32 input of the last leg has no zero point (checked above)
        // clip to int8, then CLAMP: one clip to [lo, hi]
        f.lo = has_clamp ? std::min(std::max(-128, clamp_min), clamp_max) : -128;
        f.hi = has_clamp ? std::min(std::max(127, clamp_min), clamp_max) : 127;
        // Large joins pay for tabulating all 65536 byte pairs first (two launches, one lookup per element after that)
        if (n >= ((int64_t)1 << 22))
        {
            constexpr size_t kTableSmem = kJoinTableBytes + kJoinBadWords * sizeof(uint32_t);
            // the table depends on the three RESCALEs' constants and the clip range alone: built once per join, cached
            auto build = [=](tb200_ctx* c, void* block) -> tb200_status {
                uint8_t* tab = reinterpret_cast<uint8_t*>(block);
                residual_table_kernel<<<256, 256, 0, c->stream>>>(f, tab, reinterpret_cast<uint32_t*>(tab + kJoinTableBytes));
                return post_launch(c, "residual_table");
            };
            Prepared* e = nullptr;
            if (ctx->const_cache_on)
            {
                std::string key;
                key_add(&key, (int)3);
                for (const ResidualLeg* l : { &f.a, &f.b, &f.o })
                {
                    key_add(&key, l->mult); key_add(&key, l->shift);
                    key_add(&key, l->zp_in); key_add(&key, l->zp_out); key_add(&key, l->double_round);
                }
                key_add(&key, f.lo); key_add(&key, f.hi);
                e = cache_find(ctx, key);
                if (!e)
                {
                    std::vector<std::pair<const char*, size_t>> ops;
                    for (const tb200_rescale_attr* at : { a_attr, b_attr, out_attr })
                    {
                        ops.push_back({ reinterpret_cast<const char*>(at->multiplier->data), at->multiplier->bytes });
                        ops.push_back({ reinterpret_cast<const char*>(at->shift->data), at->shift->bytes });
                    }
                    e = cache_insert(ctx, key, std::move(ops), kTableSmem, build);
                }
            }
            uint8_t* table = nullptr;
            if (e)
            {
                st = cache_use(ctx, e);
                if (st != TB200_OK)
                    return st;
                table = reinterpret_cast<uint8_t*>(e->block);
            }
            else if (ctx->join_table != nullptr || !ctx->capturing)
            {
                if (ctx->join_table == nullptr)
                    TB200_CUDA_CHECK(ctx, cudaMalloc(&ctx->join_table, kTableSmem));
                st = build(ctx, ctx->join_table);
                if (st != TB200_OK)
                    return st;
                table = reinterpret_cast<uint8_t*>(ctx->join_table);
            }
            if (table != nullptr)
            {
                st = raise_smem_limit(ctx, 16, reinterpret_cast<const void*>(residual_add_i8_table_kernel), (int)kTableSmem);
                if (st != TB200_OK)
                    return st;
                uint32_t* bad_bits = reinterpret_cast<uint32_t*>(table + kJoinTableBytes);
                const int tblock   = 512;
                const int tgrid    = (int)std::min<int64_t>((n / 16 + tblock - 1) / tblock, (int64_t)ctx->num_sms * 2);
                if (ctx->join_stream && n / 16 >= (int64_t)ctx->num_sms * kJoinStreamChunkVecs * 4)
                {
                    // streaming form: operands through a ring of bulk copies (large joins only: every SM needs a few chunks)
                    st = raise_smem_limit(ctx, 17, reinterpret_cast<const void*>(residual_add_i8_stream_kernel), (int)kJoinStreamSmem);
                    if (st != TB200_OK)
                        return st;
                    cudaLaunchConfig_t cfg;
                    memset(&cfg, 0, sizeof(cfg));
                    cfg.gridDim          = dim3((unsigned)ctx->num_sms);
                    cfg.blockDim         = dim3((unsigned)kJoinStreamThreads);
                    cfg.dynamicSmemBytes = kJoinStreamSmem;
                    cfg.stream           = ctx->stream;
                    cudaLaunchAttribute at[1];
                    at[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
                    at[0].val.programmaticStreamSerializationAllowed = 1;
                    cfg.attrs    = at;
                    cfg.numAttrs = ctx->launch_overlap ? 1 : 0;
                    cudaLaunchKernelEx(&cfg, residual_add_i8_stream_kernel, reinterpret_cast<const int8_t*>(a->data),
                                       reinterpret_cast<const int8_t*>(b->data), reinterpret_cast<int8_t*>(output->data),
                                       (int64_t)(n / 16), reinterpret_cast<const uint8_t*>(table),
                                       reinterpret_cast<const uint32_t*>(bad_bits), ctx->d_status, ctx->wait_limit_cycles);
                    return post_launch(ctx, "residual_add_i8_stream");
                }
                {
                    cudaLaunchConfig_t cfg;
                    memset(&cfg, 0, sizeof(cfg));
                    cfg.gridDim          = dim3((unsigned)tgrid);
                    cfg.blockDim         = dim3((unsigned)tblock);
                    cfg.dynamicSmemBytes = kTableSmem;
                    cfg.stream           = ctx->stream;
                    cudaLaunchAttribute at[1];
                    at[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
                    at[0].val.programmaticStreamSerializationAllowed = 1;
                    cfg.attrs    = at;
                    cfg.numAttrs = ctx->launch_overlap ? 1 : 0;
                    cudaLaunchKernelEx(&cfg, residual_add_i8_table_kernel, reinterpret_cast<const int8_t*>(a->data),
                                       reinterpret_cast<const int8_t*>(b->data), reinterpret_cast<int8_t*>(output->data),
                                       (int64_t)(n / 16), reinterpret_cast<const uint8_t*>(table),
                                       reinterpret_cast<const uint32_t*>(bad_bits), ctx->d_status);
                }
                return post_launch(ctx, "residual_add_i8_table");
            }
        }
        residual_add_i8_fast_kernel<<<grid_for(ctx, n / 16, block), block, 0, ctx->stream>>>(
            reinterpret_cast<const int8_t*>(a->data), reinterpret_cast<const int8_t*>(b->data),
            reinterpret_cast<int8_t*>(output->data), n / 16, f, ctx->d_status);
        return post_launch(ctx, "residual_add_i8_fast");
    }
    if (aligned && n % 16 == 0 && (!pc || C % 16 == 0))
        residual_add_i8_kernel<16><<<grid_for(ctx, n / 16, block), block, 0, ctx->stream>>>(
            reinterpret_cast<const int8_t*>(a->data), reinterpret_cast<const int8_t*>(b->data),
            reinterpret_cast<int8_t*>(output->data), n, C, r, ctx->d_status);
    else
        residual_add_i8_kernel<1><<<grid_for(ctx, n, block), block, 0, ctx->stream>>>(
            reinterpret_cast<const int8_t*>(a->data), reinterpret_cast<const int8_t*>(b->data),
            reinterpret_cast<int8_t*>(output->data), n, C, r, ctx->d_status);
    return post_launch(ctx, "residual_add_i8");
}

// =================================================================================================== pools
static tb200_status pool_common(tb200_ctx* ctx, const char* op, const tb200_tensor* input, const int32_t* kernel,
                                const int32_t* pad, const int32_t* stride, const tb200_tensor* output, PoolDev* p)
{
    TB200_ERROR_IF(ctx, !input || !output || !kernel || !pad || !stride, "%s: null operand", op);
    TB200_ERROR_IF(ctx, !all_contiguous({ input, output }), "%s: zero-copy views are accepted only as the CONV2D input; this operand must be contiguous", op);
    TB200_ERROR_IF(ctx, input->rank != 4 || output->rank != 4, "%s: input and output must be rank 4", op);
    TB200_ERROR_IF(ctx, input->dtype != output->dtype, "%s: input and output dtypes differ", op);
    tb200_status st = check_pool_attr(ctx, op, input->shape[1], input->shape[2], output->shape[1], output->shape[2],
                                      kernel, pad, stride);
    if (st != TB200_OK)
        return st;
    TB200_ERROR_IF(ctx, input->shape[0] != output->shape[0], "%s: tensor batch mismatch %d != %d", op, input->shape[0],
                   output->shape[0]);
    TB200_ERROR_IF(ctx, input->shape[3] != output->shape[3], "%s: tensor channel mismatch %d != %d", op, input->shape[3],
                   output->shape[3]);
    p->N = input->shape[0]; p->IH = input->shape[1]; p->IW = input->shape[2]; p->C = input->shape[3];
    p->OH = output->shape[1]; p->OW = output->shape[2];
    p->ky = kernel[0]; p->kx = kernel[1]; p->pad_t = pad[0]; p->pad_l = pad[2]; p->sy = stride[0]; p->sx = stride[1];
    return TB200_OK;
}

extern "C" tb200_status tb200_max_pool2d(tb200_ctx* ctx, const tb200_tensor* input, const int32_t kernel[2],
                                         const int32_t pad[4], const int32_t stride[2], tb200_tensor* output)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    PoolDev p;
    tb200_status st = pool_common(ctx, "OpMaxPool2d", input, kernel, pad, stride, output, &p);
    if (st != TB200_OK)
        return st;
    const int64_t n = numel(output);
    if (n == 0)
        return TB200_OK;
    cache_note_write(ctx, output->data, output->bytes);
    const int block = 256;
    const bool aligned = ((reinterpret_cast<uintptr_t>(input->data) | reinterpret_cast<uintptr_t>(output->data)) & 15) == 0;
    switch (input->dtype)
    {
        case TB200_INT8:
            if (p.C % 16 == 0 && aligned && ctx->policy == 0 && p.ky == 3 && p.kx == 3)
                max_pool3x3_i8x16_kernel<<<grid_for(ctx, n / 16, block), block, 0, ctx->stream>>>(
                    reinterpret_cast<const int8_t*>(input->data), reinterpret_cast<int8_t*>(output->data), p);
            else if (p.C % 16 == 0 && aligned && ctx->policy == 0)
                max_pool_i8x16_kernel<<<grid_for(ctx, n / 16, block), block, 0, ctx->stream>>>(
                    reinterpret_cast<const int8_t*>(input->data), reinterpret_cast<int8_t*>(output->data), p);
            else
                max_pool_kernel<int8_t, int32_t><<<grid_for(ctx, n, block), block, 0, ctx->stream>>>(
                    reinterpret_cast<const int8_t*>(input->data), reinterpret_cast<int8_t*>(output->data), p, -128);
            break;
        case TB200_INT16:
            max_pool_kernel<int16_t, int32_t><<<grid_for(ctx, n, block), block, 0, ctx->stream>>>(
                reinterpret_cast<const int16_t*>(input->data), reinterpret_cast<int16_t*>(output->data), p, -32768);
            break;
        case TB200_FP16:
            max_pool_kernel<__half, float><<<grid_for(ctx, n, block), block, 0, ctx->stream>>>(
                reinterpret_cast<const __half*>(input->data), reinterpret_cast<__half*>(output->data), p, -65504.0f);
            break;
        case TB200_BF16:
            max_pool_kernel<__nv_bfloat16, float><<<grid_for(ctx, n, block), block, 0, ctx->stream>>>(
                reinterpret_cast<const __nv_bfloat16*>(input->data), reinterpret_cast<__nv_bfloat16*>(output->data), p,
                -3.3895313892515355e38f);
            break;
        case TB200_FP32:
            max_pool_kernel<float, float><<<grid_for(ctx, n, block), block, 0, ctx->stream>>>(
                reinterpret_cast<const float*>(input->data), reinterpret_cast<float*>(output->data), p, -3.402823466e38f);
            break;
        default:
            return fail(ctx, TB200_ERROR, "OpMaxPool2d: unsupported dtype %d", (int)input->dtype);
    }
    return post_launch(ctx, "max_pool2d");
}

extern "C" tb200_status tb200_avg_pool2d(tb200_ctx* ctx, const tb200_tensor* input, const int32_t kernel[2],
                                         const int32_t pad[4], const int32_t stride[2], int32_t input_zp,
                                         int32_t output_zp, tb200_tensor* output)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    PoolDev p;
    tb200_status st = pool_common(ctx, "OpAvgPool2d", input, kernel, pad, stride, output, &p);
    if (st != TB200_OK)
        return st;
    // reference_model/src/ops/tensor_ops.cpp:568-571
    TB200_ERROR_IF(ctx, input->dtype != TB200_INT8 && input_zp != 0, "OpAvgPool2d: Input zeropoint must be zero for non int8_t data");
    TB200_ERROR_IF(ctx, input->dtype != TB200_INT8 && output_zp != 0, "OpAvgPool2d: Output zeropoint must be zero for non int8_t data");
    TB200_ERROR_IF(ctx, input_zp < -128 || input_zp > 127 || output_zp < -128 || output_zp > 127,
                   "OpAvgPool2d: zero point outside the int8 range");
    const int64_t n = numel(output);
    if (n == 0)
        return TB200_OK;
    cache_note_write(ctx, output->data, output->bytes);
    const int block = 256;
    const int grid  = grid_for(ctx, n, block);
    switch (input->dtype)
    {
        case TB200_INT8:
            if (p.C % 4 == 0 && ctx->policy == 0 &&
                ((reinterpret_cast<uintptr_t>(input->data) | reinterpret_cast<uintptr_t>(output->data)) & 3) == 0)
                avg_pool_i8x4_kernel<<<grid_for(ctx, n / 4, block), block, 0, ctx->stream>>>(
                    reinterpret_cast<const int8_t*>(input->data), reinterpret_cast<int8_t*>(output->data), p, input_zp, output_zp,
                    -128, 127, ctx->d_status);
            else
                avg_pool_int_kernel<int8_t><<<grid, block, 0, ctx->stream>>>(reinterpret_cast<const int8_t*>(input->data), reinterpret_cast<int8_t*>(output->data), p, input_zp, output_zp, -128, 127, ctx->d_status);
            break;
        case TB200_INT16:
            avg_pool_int_kernel<int16_t><<<grid, block, 0, ctx->stream>>>(reinterpret_cast<const int16_t*>(input->data), reinterpret_cast<int16_t*>(output->data), p, 0, 0, -32768, 32767, ctx->d_status);
            break;
        case TB200_FP16:
            avg_pool_fp_kernel<__half><<<grid, block, 0, ctx->stream>>>(reinterpret_cast<const __half*>(input->data), reinterpret_cast<__half*>(output->data), p);
            break;
        case TB200_BF16:
            avg_pool_fp_kernel<__nv_bfloat16><<<grid, block, 0, ctx->stream>>>(reinterpret_cast<const __nv_bfloat16*>(input->data), reinterpret_cast<__nv_bfloat16*>(output->data), p);
            break;
        case TB200_FP32:
            avg_pool_fp_kernel<float><<<grid, block, 0, ctx->stream>>>(reinterpret_cast<const float*>(input->data), reinterpret_cast<float*>(output->data), p);
            break;
        default:
            return fail(ctx, TB200_ERROR, "OpAvgPool2d: unsupported dtype %d", (int)input->dtype);
    }
    return post_launch(ctx, "avg_pool2d");
}

// =================================================================================================== host buffers
static tb200_status pipe_prepare(tb200_ctx* ctx, size_t bytes_per_slot)
{
    auto& p = ctx->pipe;
    if (!p.ready)
    {
        TB200_CUDA_CHECK(ctx, cudaStreamCreateWithFlags(&p.h2d, cudaStreamNonBlocking));
        TB200_CUDA_CHECK(ctx, cudaStreamCreateWithFlags(&p.d2h, cudaStreamNonBlocking));
        for (int i = 0; i < 2; i++)
        {
            TB200_CUDA_CHECK(ctx, cudaEventCreateWithFlags(&p.up[i], cudaEventDisableTiming));
            TB200_CUDA_CHECK(ctx, cudaEventCreateWithFlags(&p.done[i], cudaEventDisableTiming));
            TB200_CUDA_CHECK(ctx, cudaEventCreateWithFlags(&p.down[i], cudaEventDisableTiming));
        }
        p.ready = true;
    }
    if (bytes_per_slot > p.cap)
    {
        TB200_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
        TB200_CUDA_CHECK(ctx, cudaStreamSynchronize(p.h2d));
        TB200_CUDA_CHECK(ctx, cudaStreamSynchronize(p.d2h));
        for (int i = 0; i < 2; i++)
        {
            if (p.buf[i])
                cudaFree(p.buf[i]);
            p.buf[i] = nullptr;
        }
        p.cap = 0;
        for (int i = 0; i < 2; i++)
            TB200_CUDA_CHECK(ctx, cudaMalloc(&p.buf[i], bytes_per_slot));
        p.cap = bytes_per_slot;
    }
    return TB200_OK;
}

// MATMUL on host buffers.  The batch is cut into chunks that flow through two device staging slots: while chunk i
// is multiplied, chunk i+1 is uploaded and chunk i-1 downloaded on separate copy streams, so that the PCIe link
// carries both directions at once.  Pinned host buffers make the copies asynchronous; pageable ones still work.
extern "C" tb200_status tb200_matmul_host(tb200_ctx* ctx, tb200_dtype in_dtype, tb200_dtype out_dtype, const void* a,
                                          const void* b, int32_t N, int32_t H, int32_t C, int32_t W, int32_t a_zp,
                                          int32_t b_zp, void* out)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !a || !b || !out, "matmul_host: null buffer");
    TB200_ERROR_IF(ctx, N < 0 || H < 0 || C < 0 || W < 0, "matmul_host: negative dimension");
    const size_t es_in = dtype_size(in_dtype), es_out = dtype_size(out_dtype);
    TB200_ERROR_IF(ctx, es_in == 0 || es_out == 0, "matmul_host: unsupported dtype");
    if (N == 0 || H == 0 || W == 0)
        return TB200_OK;
    const size_t a_b = (size_t)H * C * es_in, b_b = (size_t)C * W * es_in, o_b = (size_t)H * W * es_out;
    auto up256 = [](size_t v) { return (v + 255) & ~(size_t)255; };
    // About 64 MB of A per chunk in the steady state (smaller chunks were measured slower: per-chunk launch work adds
    // up).  The link is the bottleneck, so the first chunks are small and double in size (the first product starts after
    // one batch has been uploaded, not eight) and the last ones halve again (little is left to download after the last
    // upload).
    const size_t chunk_target = (size_t)std::max(1, diag_env_int("TB200_HOST_CHUNK_MB", 64)) << 20;
    int nb = (int)std::max<size_t>(1, std::min<size_t>((size_t)N, chunk_target / std::max<size_t>(a_b, 1)));
    std::vector<int> sizes;
    {
        std::vector<int> tail;
        int left = N;
        for (int c = 1; c < nb && left > 2 * c; c *= 2)
        {
            sizes.push_back(c);
            tail.push_back(c);
            left -= 2 * c;
        }
        while (left > 0)
        {
            const int c = std::min(nb, left);
            sizes.push_back(c);
            left -= c;
        }
        sizes.insert(sizes.end(), tail.rbegin(), tail.rend());
    }
    const size_t off_b = up256((size_t)nb * a_b), off_o = off_b + up256((size_t)nb * b_b);
    const size_t slot_bytes = off_o + up256((size_t)nb * o_b);
    tb200_status st = pipe_prepare(ctx, slot_bytes);
    if (st != TB200_OK)
        return st;
    auto& p = ctx->pipe;
    // order the copy streams after whatever the caller queued on the compute stream, and clear stale events
    TB200_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    int chunk_idx = 0;
    for (int n0 = 0; n0 < N; n0 += sizes[chunk_idx], chunk_idx++)
    {
        const int cnt  = sizes[chunk_idx];
        const int slot = chunk_idx & 1;
        uint8_t* base  = reinterpret_cast<uint8_t*>(p.buf[slot]);
        if (chunk_idx >= 2)
        {
            // the slot's inputs are free once its previous product is done; its output once that was downloaded
            TB200_CUDA_CHECK(ctx, cudaStreamWaitEvent(p.h2d, p.done[slot], 0));
            TB200_CUDA_CHECK(ctx, cudaStreamWaitEvent(ctx->stream, p.down[slot], 0));
        }
        TB200_CUDA_CHECK(ctx, cudaMemcpyAsync(base, reinterpret_cast<const uint8_t*>(a) + (size_t)n0 * a_b,
                                              (size_t)cnt * a_b, cudaMemcpyHostToDevice, p.h2d));
        TB200_CUDA_CHECK(ctx, cudaMemcpyAsync(base + off_b, reinterpret_cast<const uint8_t*>(b) + (size_t)n0 * b_b,
                                              (size_t)cnt * b_b, cudaMemcpyHostToDevice, p.h2d));
        TB200_CUDA_CHECK(ctx, cudaEventRecord(p.up[slot], p.h2d));
        TB200_CUDA_CHECK(ctx, cudaStreamWaitEvent(ctx->stream, p.up[slot], 0));
        tb200_tensor ta{ in_dtype, 3, { cnt, H, C, 1, 1, 1 }, base, (size_t)cnt * a_b, false, { 0, 0, 0, 0, 0, 0 }, true };
        tb200_tensor tbm{ in_dtype, 3, { cnt, C, W, 1, 1, 1 }, base + off_b, (size_t)cnt * b_b, false, { 0, 0, 0, 0, 0, 0 }, true };
        tb200_tensor to{ out_dtype, 3, { cnt, H, W, 1, 1, 1 }, base + off_o, (size_t)cnt * o_b, false, { 0, 0, 0, 0, 0, 0 }, true };
        st = tb200_matmul(ctx, &ta, &tbm, a_zp, b_zp, nullptr, &to);
        if (st != TB200_OK)
            break;
        TB200_CUDA_CHECK(ctx, cudaEventRecord(p.done[slot], ctx->stream));
        TB200_CUDA_CHECK(ctx, cudaStreamWaitEvent(p.d2h, p.done[slot], 0));
        TB200_CUDA_CHECK(ctx, cudaMemcpyAsync(reinterpret_cast<uint8_t*>(out) + (size_t)n0 * o_b, base + off_o,
                                              (size_t)cnt * o_b, cudaMemcpyDeviceToHost, p.d2h));
        TB200_CUDA_CHECK(ctx, cudaEventRecord(p.down[slot], p.d2h));
    }
    cudaError_t e1 = cudaStreamSynchronize(p.h2d);
    cudaError_t e2 = cudaStreamSynchronize(p.d2h);
    tb200_status sync_st = tb200_sync(ctx);
    if (st != TB200_OK)
        return st;
    if (e1 != cudaSuccess || e2 != cudaSuccess)
        return fail(ctx, TB200_INTERNAL, "matmul_host: copy stream failed: %s", cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
    return sync_st;
}
