/*
 * tb200 — C ABI of the B200 (sm_100a) compute path for the TOSA reference model's
 * CONV2D / DEPTHWISE_CONV2D / MATMUL / RESCALE / CLAMP / ADD / MAX_POOL2D / AVG_POOL2D nodes.
 *
 * This is the boundary a reference-side adapter binds: a GraphNode subclass's eval()
 * (reference_model/src/graph_node.h:176-179) or a CustomOpInterface::eval()
 * (reference_model/include/custom_op_interface.h:25-35) calls one entry point per node.
 * Plain C: opaque handles, pointers and sizes only; nothing throws or aborts across it.
 *
 * Conventions
 *  - Tensors are row-major in TOSA shape order at their true element width (int8 is 1 byte,
 *    fp16/bf16 2 bytes): NHWC activations, OHWI CONV2D weights, [KH,KW,C,M] DEPTHWISE weights,
 *    [N,H,C] x [N,C,W] MATMUL operands.  This is the layout of every external buffer of the
 *    reference (reference_model/src/tensor.cpp:2157-2179), not its internal column-major Eigen storage.
 *  - Zero points are passed as scalars; the adapter reads element (0) of the reference's rank-1
 *    zero-point operands (reference_model/src/ops/tensor_ops.cpp:804,810).
 *  - Every call returns a tb200_status.  Shape / attribute violations (the reference's ERROR_IF)
 *    are detected on the host before any launch and return TB200_ERROR.  Data-dependent REQUIRE
 *    failures (RESCALE range checks, int32 ADD overflow) are recorded by the kernels in a device
 *    status word and reported by tb200_sync / tb200_tensor_download as TB200_UNPREDICTABLE.
 *  - All work is asynchronous on the context's stream.  Calls on one context must be serialised
 *    by the caller (the reference is single-threaded, reference_model/src/model_runner.cpp:22-23).
 */
#ifndef TB200_H
#define TB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C"
{
#endif

#if defined(__GNUC__)
#define TB200_API __attribute__((visibility("default")))
#else
#define TB200_API
#endif

    /* Mirrors GraphStatus {TOSA_VALID, TOSA_UNPREDICTABLE, TOSA_ERROR}
     * (reference_model/include/graph_status.h:18-23); TB200_INTERNAL covers CUDA / driver failures,
     * which the adapter should surface as TOSA_ERROR. */
    typedef enum tb200_status
    {
        TB200_OK            = 0,
        TB200_UNPREDICTABLE = 1,
        TB200_ERROR         = 2,
        TB200_INTERNAL      = 3
    } tb200_status;

    /* Same numeric values as tosa_datatype_t (reference_model/include/types.h:27-44). */
    typedef enum tb200_dtype
    {
        TB200_BF16   = 0,
        TB200_FP16   = 2,
        TB200_FP32   = 3,
        TB200_INT16  = 4,
        TB200_INT32  = 5,
        TB200_INT8   = 8,
        TB200_UINT16 = 9,
        TB200_UINT8  = 10,
        TB200_FP8E4M3 = 12, /* 1-4-3, bias 7, no infinities; operands of MATMUL and the convolutions */
        TB200_FP8E5M2 = 13  /* 1-5-2, bias 15; operands of MATMUL and the convolutions */
    } tb200_dtype;

    /* RoundingMode of the RESCALE attribute (reference_model/src/ops/type_conversion.cpp:229-231). */
    typedef enum tb200_rounding
    {
        TB200_SINGLE_ROUND  = 0,
        TB200_DOUBLE_ROUND  = 1,
        TB200_INEXACT_ROUND = 2
    } tb200_rounding;

    typedef struct tb200_ctx tb200_ctx;
    typedef struct tb200_tensor tb200_tensor;

    /* ---- context ------------------------------------------------------------------------------ */

    /* Creates a context on CUDA device `device`.  `stream` is a cudaStream_t the caller owns, or NULL
     * to let the context create its own.  One context per (process, device); stands where the reference
     * has its process-wide model state (reference_model/src/model_runner_impl.cpp:24-28). */
    TB200_API tb200_status tb200_ctx_create(int device, void* stream, tb200_ctx** out);
    TB200_API tb200_status tb200_ctx_destroy(tb200_ctx* ctx);
    /* Text of the last error recorded on this context (never NULL). */
    TB200_API const char* tb200_last_error(const tb200_ctx* ctx);
    /* Waits for the stream, then reports and clears the device status word: TB200_OK,
     * TB200_UNPREDICTABLE (a REQUIRE failed in some kernel since the last sync) or TB200_INTERNAL.
     * Stands where SubgraphTraverser reads the graph status after evaluateAll
     * (reference_model/src/model_runner_impl.cpp:56-126). */
    TB200_API tb200_status tb200_sync(tb200_ctx* ctx);
    /* Number of kernels this context has launched since creation (for accounting in benchmarks). */
    TB200_API uint64_t tb200_launch_count(const tb200_ctx* ctx);
    /* Measurement aid with no counterpart in the reference (which has no timers): while enabled, the main
     * kernel of every CONV2D / MATMUL call (the tensor-core GEMM or the fp32 SGEMM, not its small preparation
     * kernels) is bracketed by CUDA events on the context's stream.  tb200_timer_read synchronises, returns the
     * summed device time in milliseconds and the number of bracketed launches since the last read, and clears. */
    TB200_API tb200_status tb200_timer_enable(tb200_ctx* ctx, int32_t on);
    TB200_API tb200_status tb200_timer_read(tb200_ctx* ctx, double* total_ms, int32_t* launches);

    /* Whole-evaluation replay.  The reference evaluates a graph node by node from its ready list
     * (reference_model/src/subgraph_traverser.cpp:1190-1202); on the device the same sequence of operator calls can
     * be recorded once into a CUDA graph and replayed with a single launch.  Between tb200_capture_begin and
     * tb200_capture_end the operator entry points enqueue nothing for execution, they only record; no call may
     * need to grow the context's scratch memory or build a cache entry (run the sequence once eagerly first), and
     * uploads / downloads / tb200_sync are not allowed.  Operands must stay allocated for as long as the graph is
     * replayed.  A graph records the addresses of the context's internal blocks (scratch, staging, cached tables):
     * while any graph of a context is alive, a block that a later eager call has to grow or drop is not freed but
     * parked until the last graph is destroyed, so a replay never touches freed memory.  Constants changed through
     * tb200_tensor_upload are picked up by a replay (the tables derived from them are rebuilt in place behind the
     * copy). */
    typedef struct tb200_graph tb200_graph;
    TB200_API tb200_status tb200_capture_begin(tb200_ctx* ctx);
    TB200_API tb200_status tb200_capture_end(tb200_ctx* ctx, tb200_graph** out);
    TB200_API tb200_status tb200_graph_launch(tb200_ctx* ctx, tb200_graph* graph);
    TB200_API tb200_status tb200_graph_destroy(tb200_ctx* ctx, tb200_graph* graph);

    /* Every wait a kernel makes on its own pipeline (TMA arrival, accumulator hand-over, zero-point sums published by
     * another CTA) gives up after `sm_cycles` SM clock cycles, about two seconds by default: the kernel then drains,
     * frees its tensor memory and exits, its output is incomplete, and the next tb200_sync / download reports
     * TB200_INTERNAL.  The context stays usable.  No counterpart in the reference (a host interpreter cannot stall on
     * a device pipeline); the setter exists so that a host can bound its worst case and so that the give-up path can
     * be exercised. */
    TB200_API tb200_status tb200_set_wait_limit(tb200_ctx* ctx, uint64_t sm_cycles);
    /* shared != 0: other work may occupy SMs of this GPU while the context runs.  Kernels then never wait for another
     * CTA of their own grid: the CTA-pair MATMUL takes its zero-point sums from separate kernels instead of exchanging
     * them between tiles through flags (which needs the whole grid resident at once, true on a GPU the context has to
     * itself, the default). */
    TB200_API tb200_status tb200_set_shared_gpu(tb200_ctx* ctx, int32_t shared);
    /* on != 0 (the default): the kernels that support it (the int8 CONV2D + RESCALE kernel, the residual join) are
     * launched with programmatic stream serialization, so that one kernel's set-up and its reads of constants overlap
     * the end of the kernel before it on the same stream; each waits for its predecessor (griddepcontrol.wait) before
     * it reads an activation or writes an output, so results and ordering are those of plain stream order.  The
     * reference evaluates node after node on one host thread and has no counterpart; the switch is there for hosts
     * that want plain launches (for instance to read per-kernel times from a profiler's timeline). */
    TB200_API tb200_status tb200_set_launch_overlap(tb200_ctx* ctx, int32_t on);

    /* Constant-operand cache.  The reference decodes a graph's constants once
     * (reference_model/src/subgraph_traverser.cpp:617-781); here everything an operator derives from constants alone
     * (zero-point correction rows, per-channel RESCALE records, re-packed weights of few-channel layers, the byte-pair
     * table of a residual join) is built on the first call that sees those operands and reused afterwards, keyed by the
     * operands' device addresses and the attributes.  tb200_tensor_upload / tb200_tensor_load_npy into an operand
     * rebuild what was derived from it; an operator writing into an operand makes its entries rebuild on every use;
     * tb200_tensor_free drops them.  Memory handed over with tb200_tensor_wrap and then modified by the caller behind
     * the library's back is the one case that needs TB200_CACHE_CLEAR. */
    typedef enum tb200_cache_action
    {
        TB200_CACHE_OFF   = 0, /* drop every entry and build nothing new: every call recomputes its tables */
        TB200_CACHE_ON    = 1, /* the default */
        TB200_CACHE_CLEAR = 2  /* drop every entry, stay on */
    } tb200_cache_action;
    TB200_API tb200_status tb200_const_cache_control(tb200_ctx* ctx, int32_t action);
    TB200_API int32_t tb200_const_cache_entries(const tb200_ctx* ctx);

    /* ---- tensors -------------------------------------------------------------------------------
     * Device-resident replacements for TensorTemplate<Eigen::Tensor<T,R>> buffers
     * (reference_model/src/tensor.h:365-440): allocate stands for Tensor::allocate (:380-398),
     * upload / download for setTensorValue* / getTensorValue* (reference_model/src/tensor.cpp:2157-2179, :3662). */
    TB200_API tb200_status tb200_tensor_alloc(tb200_ctx* ctx, tb200_dtype dtype, int rank, const int32_t* shape,
                                              tb200_tensor** out);
    /* Wraps device memory the caller owns (for hosts that manage device buffers themselves). */
    TB200_API tb200_status tb200_tensor_wrap(tb200_ctx* ctx, tb200_dtype dtype, int rank, const int32_t* shape,
                                             void* device_ptr, tb200_tensor** out);
    TB200_API tb200_status tb200_tensor_free(tb200_ctx* ctx, tb200_tensor* t);
    /* `host` holds `bytes` = element count x element width, row-major.  Upload is asynchronous when `host`
     * is pinned; download synchronises the stream and returns the status tb200_sync would. */
    TB200_API tb200_status tb200_tensor_upload(tb200_ctx* ctx, tb200_tensor* t, const void* host, size_t bytes);
    TB200_API tb200_status tb200_tensor_download(tb200_ctx* ctx, const tb200_tensor* t, void* host, size_t bytes);
    /* SLICE as a zero-copy view: replaces OpSlice<Rank,T>::eval (reference_model/src/ops/data_layout.cpp:369-398)
     * with the same start / size rules.  The view shares its parent's memory (free the view before the parent) and
     * keeps its pitch; it is accepted as the input of tb200_conv2d (e.g. the 55x55 cut that makes a stride-2 1x1
     * shortcut convolution legal under the exact-division rule); other operators need contiguous tensors. */
    TB200_API tb200_status tb200_tensor_slice(tb200_ctx* ctx, const tb200_tensor* parent, const int32_t* start,
                                              const int32_t* size, tb200_tensor** out);
    /* RESHAPE as a zero-copy view of a contiguous tensor: replaces OpReshape::eval
     * (reference_model/src/ops/data_layout.cpp:227-). */
    TB200_API tb200_status tb200_tensor_reshape(tb200_ctx* ctx, const tb200_tensor* parent, int rank,
                                                const int32_t* shape, tb200_tensor** out);
    TB200_API void* tb200_tensor_data(const tb200_tensor* t);
    TB200_API size_t tb200_tensor_bytes(const tb200_tensor* t);

    /* ---- NumPy files ----------------------------------------------------------------------------
     * Replace Tensor::readFromNpyFile / Tensor::writeToNpyFile (reference_model/src/tensor.cpp:96-421, :423-640).
     * Loading accepts the file types the reference's tools produce for a tensor of `dtype`: an int32 file for every
     * integer tensor (:164-171; narrowed on the device, a value outside the tensor type's range is TB200_ERROR), the
     * tensor's own width (what writeToNpyFile emits for INT8 / INT16 results, :574-600), float16 for FP16, float32
     * for FP32, and 2-byte raw words or float32 (rounded to nearest even) for BF16.  Row-major files only.
     * Saving writes format 1.0 with the tensor's own element type.  The payload moves through one pinned 64 MiB
     * host buffer; no widened copy of the tensor is made on either side.
     * tb200_npy_probe reads only the header (no context, no GPU): descr such as "<i4", rank, shape, payload offset;
     * `err` receives the reason when it returns TB200_ERROR. */
    TB200_API tb200_status tb200_npy_probe(const char* path, char descr[8], int32_t* rank, int32_t shape[6],
                                           uint64_t* data_offset, char* err, size_t err_len);
    TB200_API tb200_status tb200_tensor_load_npy(tb200_ctx* ctx, const char* path, tb200_dtype dtype,
                                                 tb200_tensor** out);
    TB200_API tb200_status tb200_tensor_save_npy(tb200_ctx* ctx, const tb200_tensor* t, const char* path);

    /* ---- fused epilogue ------------------------------------------------------------------------
     * Lets the host collapse CONV2D/MATMUL -> RESCALE -> CLAMP chains whose intermediates have a single
     * consumer (reference_model/src/tensor.h:92-100).  NULL means the plain op. */
    typedef struct tb200_rescale_attr
    {
        const tb200_tensor* multiplier; /* INT32 when scale32 else INT16; [C] when per_channel else [1] */
        const tb200_tensor* shift;      /* INT8; same length as multiplier */
        int32_t input_zp;
        int32_t output_zp;
        int32_t scale32;
        int32_t rounding_mode; /* tb200_rounding */
        int32_t per_channel;
        int32_t input_unsigned;
        int32_t output_unsigned;
    } tb200_rescale_attr;

    typedef struct tb200_epilogue
    {
        int32_t has_rescale; /* integer paths only: int32 accumulator -> `out` dtype */
        tb200_rescale_attr rescale;
        int32_t has_clamp;
        int32_t clamp_min_i; /* integer outputs */
        int32_t clamp_max_i;
        float clamp_min_f; /* floating outputs */
        float clamp_max_f;
    } tb200_epilogue;

    /* ---- operators -----------------------------------------------------------------------------*/

    /* CONV2D.  Replaces OpConv2d<In,W,Acc,Out>::eval (reference_model/src/ops/tensor_ops.cpp:723-882) and the
     * checks of check_conv_attribute (:120-226) / OpConv2d::checkTensorAttributes (:690-720).
     * input NHWC, weight OHWI, bias [OC] or [1]; pad = {top,bottom,left,right}, stride = {y,x}, dilation = {y,x}.
     * Supported tuples (in/weight/bias/out): INT8/INT8/INT32/INT32, FP16/FP16/FP16/FP16, BF16/BF16/BF16/BF16,
     * FP32/FP32/FP32/FP32, FP8E4M3/FP8E4M3/FP16/FP16, FP8E5M2/FP8E5M2/FP16/FP16 (:2228-2229); floating types
     * accumulate in fp32.  With an epilogue carrying RESCALE the output is the RESCALE's output dtype. */
    TB200_API tb200_status tb200_conv2d(tb200_ctx* ctx, const tb200_tensor* input, const tb200_tensor* weight,
                                        const tb200_tensor* bias, int32_t input_zp, int32_t weight_zp,
                                        const int32_t pad[4], const int32_t stride[2], const int32_t dilation[2],
                                        const tb200_epilogue* epilogue, tb200_tensor* output);

    /* DEPTHWISE_CONV2D.  Replaces OpDepthwiseConv2d::eval (reference_model/src/ops/tensor_ops.cpp:1172-1334).
     * weight [KH,KW,C,M]; output channel c*M+m.  Type tuples as for CONV2D (fp8 operands: :2250-2251). */
    TB200_API tb200_status tb200_depthwise_conv2d(tb200_ctx* ctx, const tb200_tensor* input,
                                                  const tb200_tensor* weight, const tb200_tensor* bias,
                                                  int32_t input_zp, int32_t weight_zp, const int32_t pad[4],
                                                  const int32_t stride[2], const int32_t dilation[2],
                                                  const tb200_epilogue* epilogue, tb200_tensor* output);

    /* CONV2D with a 1x1 kernel (stride 1, no padding) -> optional CLAMP -> DEPTHWISE_CONV2D with a 3x3 kernel
     * (multiplier 1, no dilation) -> optional CLAMP, evaluated as ONE kernel for FP16 and BF16: the tensor between the
     * two operators (the largest tensor of an inverted-residual block, with a single consumer,
     * reference_model/src/tensor.h:92-100) never reaches device memory.  Stands for OpConv2d::eval
     * (reference_model/src/ops/tensor_ops.cpp:723-882), OpClamp (reference_model/src/ops/activation_funcs.cpp:27-128),
     * OpDepthwiseConv2d::eval (tensor_ops.cpp:1172-1334) and OpClamp again, with the CONV2D result rounded to the
     * storage type before the window runs over it, as the reference's intermediate tensor is.
     * input NHWC [N,IH,IW,IC], weight [C,1,1,IC], bias [C] or [1]; dw_weight [3,3,C,1], dw_bias [C] or [1];
     * dw_pad = {top,bottom,left,right}, dw_stride = {y,x}; output [N,OH,OW,C].  The one-kernel form needs IC of 16, 32
     * or 64, C a multiple of 64, IW <= 128 and strides of 1 or 2 (tb200_last_kernel then names expand_dw_f16 or
     * expand_dw_bf16, and `expanded` is not touched).  Any other shape runs tb200_conv2d into `expanded`
     * ([N,IH,IW,C]) and tb200_depthwise_conv2d out of it; with `expanded` NULL such a shape is TB200_ERROR. */
    TB200_API tb200_status tb200_conv2d_depthwise(tb200_ctx* ctx, const tb200_tensor* input, const tb200_tensor* weight,
                                                  const tb200_tensor* bias, const tb200_epilogue* conv_epilogue,
                                                  const tb200_tensor* dw_weight, const tb200_tensor* dw_bias,
                                                  const int32_t dw_pad[4], const int32_t dw_stride[2],
                                                  const tb200_epilogue* dw_epilogue, tb200_tensor* expanded,
                                                  tb200_tensor* output);

    /* CONV3D.  Replaces OpConv3d<In,W,Acc,Out>::eval (reference_model/src/ops/tensor_ops.cpp:934-1120) and the checks of
     * check_conv_attribute with conv_dimension 3 (:120-226) / OpConv3d::checkTensorAttributes (:902-931).
     * input [N,ID,IH,IW,IC], weight [OC,KD,KH,KW,IC], bias [OC] or [1]; pad = {d0,d1,top,bottom,left,right}, stride and
     * dilation = {d,y,x}; output [N,OD,OH,OW,OC].  Type tuples INT8/INT8/INT32/INT32 (or, with a RESCALE epilogue, the
     * RESCALE's output type), FP16, BF16 and FP32 with fp32 accumulation (:2231-2235); taps outside the input are skipped,
     * order kd, ky, kx, ic.  A kernel of depth 1 with depth stride 1 and no depth padding runs as a CONV2D over N * ID
     * images (tb200_conv2d's kernels, tensor cores included); a shape whose KD * IC elements make whole 32-byte runs is
     * staged (depth taps gathered beside the channels, weights re-ordered) and runs as a CONV2D over N * OD images with
     * KD * IC channels, the same products summed in another order; every other shape runs a CUDA-core kernel, one thread
     * per output. */
    TB200_API tb200_status tb200_conv3d(tb200_ctx* ctx, const tb200_tensor* input, const tb200_tensor* weight,
                                        const tb200_tensor* bias, int32_t input_zp, int32_t weight_zp, const int32_t pad[6],
                                        const int32_t stride[3], const int32_t dilation[3], const tb200_epilogue* epilogue,
                                        tb200_tensor* output);

    /* TRANSPOSE_CONV2D.  Replaces OpTransposeConv2d::eval (reference_model/src/ops/tensor_ops.cpp:2059-2197) and
     * OpTransposeConv2d::checkTensorAttributes (:1982-2056).  input NHWC, weight OHWI, bias [OC] or [1];
     * out_pad = {top,bottom,left,right} (each > -kernel), stride = {y,x}; the output must be
     * (IH-1)*stride_y + out_pad_top + out_pad_bottom + KH by the same in x.  Type tuples and the epilogue are
     * those of tb200_conv2d.  Never scatters: the output phases (rows and columns modulo the stride) become column
     * blocks of one stride-1 CONV2D over the original input, stored straight at their output pixels; shapes that form
     * cannot take run one stride-1 CONV2D per phase, or a stride-1 CONV2D over the input spread out by the stride
     * (gaps hold the input zero point) with the kernel mirrored.  All three end in tb200_conv2d's kernels. */
    TB200_API tb200_status tb200_transpose_conv2d(tb200_ctx* ctx, const tb200_tensor* input,
                                                  const tb200_tensor* weight, const tb200_tensor* bias,
                                                  int32_t input_zp, int32_t weight_zp, const int32_t out_pad[4],
                                                  const int32_t stride[2], const tb200_epilogue* epilogue,
                                                  tb200_tensor* output);

    /* MATMUL.  Replaces OpMatMul<A,B,Out>::eval (reference_model/src/ops/tensor_ops.cpp:1423-1492, checks :1347-1420).
     * a [N,H,C], b [N,C,W], output [N,H,W]; INT8xINT8->INT32, FP16/BF16->same or FP32, FP32->FP32 (FFMA, no TF32),
     * FP8E4M3 / FP8E5M2 in any pairing of a and b -> FP16 or FP32 (:2263-2270; fp32 accumulation on the tensor cores,
     * `kind::f8f6f4`, rounded once to the output type). */
    TB200_API tb200_status tb200_matmul(tb200_ctx* ctx, const tb200_tensor* a, const tb200_tensor* b, int32_t a_zp,
                                        int32_t b_zp, const tb200_epilogue* epilogue, tb200_tensor* output);

    /* RESCALE.  Replaces OpRescale<Rank,In,Out>::eval (reference_model/src/ops/type_conversion.cpp:223-422, checks
     * :71-154) with QuantUtil::apply_scale_32 / apply_scale_16 (reference_model/src/quant_util.h:45-108). */
    TB200_API tb200_status tb200_rescale(tb200_ctx* ctx, const tb200_tensor* input, const tb200_rescale_attr* attr,
                                         tb200_tensor* output);

    /* CLAMP.  Replaces OpClamp<Rank,T> (reference_model/src/ops/activation_funcs.cpp:27-128).  Integer tensors use
     * min_i/max_i, floating tensors min_f/max_f; nan_ignore selects NanPropagationMode_IGNORE. */
    TB200_API tb200_status tb200_clamp(tb200_ctx* ctx, const tb200_tensor* input, int32_t min_i, int32_t max_i,
                                       float min_f, float max_f, int32_t nan_ignore, tb200_tensor* output);

    /* ADD.  Replaces OpAdd<Rank,T> (reference_model/src/ops/ewise_binary.cpp:144-173) including the size-1
     * broadcast of BinaryNodeBase::broadcast (:81-111).  INT32, FP16, BF16, FP32. */
    TB200_API tb200_status tb200_add(tb200_ctx* ctx, const tb200_tensor* a, const tb200_tensor* b,
                                     tb200_tensor* output);

    /* Residual join of a quantized graph in one pass: RESCALE(a) and RESCALE(b) to INT32, ADD, RESCALE to the output
     * dtype, CLAMP.  Equivalent to the five reference nodes evaluated one after another (INT32 ADD is the only integer
     * ADD, reference_model/src/ops/op_factory.cpp:189-195). */
    TB200_API tb200_status tb200_residual_add(tb200_ctx* ctx, const tb200_tensor* a, const tb200_rescale_attr* a_attr,
                                              const tb200_tensor* b, const tb200_rescale_attr* b_attr,
                                              const tb200_rescale_attr* out_attr, int32_t has_clamp, int32_t clamp_min,
                                              int32_t clamp_max, tb200_tensor* output);

    /* MAX_POOL2D.  Replaces OpMaxPool2d<T>::eval (reference_model/src/ops/tensor_ops.cpp:1545-1641; checks :28-117).
     * kernel = {y,x}. */
    TB200_API tb200_status tb200_max_pool2d(tb200_ctx* ctx, const tb200_tensor* input, const int32_t kernel[2],
                                            const int32_t pad[4], const int32_t stride[2], tb200_tensor* output);

    /* AVG_POOL2D.  Replaces OpAvgPool2d<T,Acc>::eval (reference_model/src/ops/tensor_ops.cpp:542-671) with
     * QuantUtil::reciprocal_scale (reference_model/src/quant_util.h:32-43). */
    TB200_API tb200_status tb200_avg_pool2d(tb200_ctx* ctx, const tb200_tensor* input, const int32_t kernel[2],
                                            const int32_t pad[4], const int32_t stride[2], int32_t input_zp,
                                            int32_t output_zp, tb200_tensor* output);

    /* ---- host-buffer conveniences --------------------------------------------------------------
     * One call per node for hosts that keep tensors in host memory: upload the operands, run the node,
     * download the result, synchronise.  The timed end-to-end path of the benchmark. */
    TB200_API tb200_status tb200_matmul_host(tb200_ctx* ctx, tb200_dtype in_dtype, tb200_dtype out_dtype,
                                             const void* a, const void* b, int32_t N, int32_t H, int32_t C,
                                             int32_t W, int32_t a_zp, int32_t b_zp, void* out);

    /* ---- several GPUs ---------------------------------------------------------------------------
     * The operators of this path are independent across the batch dimension (reference_model/src/ops/tensor_ops.cpp:828,
     * :1283, :1454-1483 index N only on the output side), so a graph is split by giving every GPU its own process,
     * context and slice of the batch; the one exchange is the gather of the output shards.  The reference itself is a
     * single-process interpreter and has no counterpart.  NCCL is looked up at run time (libnccl.so.2 already in the
     * process, else from the loader path); without it these calls return TB200_INTERNAL and nothing else is affected.
     *  - tb200_comm_unique_id: rank 0 calls it and hands the 128 bytes to the other ranks by any means the host has.
     *  - tb200_comm_init: collective over all ranks; creates the context's communicator on the context's device.
     *  - tb200_comm_attach: uses a communicator (ncclComm_t) the host already has instead; the host keeps ownership.
     *  - tb200_gather_output: all ranks call it with their shard; `gathered` receives the shards in rank order along
     *    the shard's outermost dimension larger than one (every other dimension equal), on the context's stream.  With
     *    one rank (no communicator) it is a device copy. */
#define TB200_COMM_ID_BYTES 128
    TB200_API tb200_status tb200_comm_unique_id(char id_out[TB200_COMM_ID_BYTES]);
    TB200_API tb200_status tb200_comm_init(tb200_ctx* ctx, const char id[TB200_COMM_ID_BYTES], int32_t rank, int32_t nranks);
    TB200_API tb200_status tb200_comm_attach(tb200_ctx* ctx, void* nccl_comm);
    TB200_API tb200_status tb200_comm_destroy(tb200_ctx* ctx);
    TB200_API int32_t tb200_comm_rank(const tb200_ctx* ctx);
    TB200_API int32_t tb200_comm_size(const tb200_ctx* ctx);
    TB200_API tb200_status tb200_gather_output(tb200_ctx* ctx, const tb200_tensor* shard, tb200_tensor* gathered);

    /* Largest N*(H + W rounded up to a multiple of 256) the built-in scratch of tb200_matmul_i8_noalloc holds
     * (int32 entries, 1 MiB in total). */
#define TB200_NOALLOC_MAX_SUMS 262144

    /* INT8 MATMUL with zero points, out[N,H,W] (INT32) = (a[N,H,C] - a_zp) x (b[N,C,W] - b_zp), on raw device
     * pointers, performing no device allocation.  It has no counterpart in the reference, which allocates freely
     * on the host; it exists for hosts that must not allocate device memory at evaluation time: an adapter that
     * was handed a fixed set of device buffers by the application embedding it (all device memory belongs to that
     * application's pool), or a latency-bound evaluation loop that cannot take the device-wide synchronisation of
     * cudaMalloc / cudaFree.  tb200_matmul keeps its zero-point row / column sums in context scratch obtained with
     * cudaMalloc; this variant keeps them in a fixed array inside the library image instead, which every GPU that
     * loads the library holds until the process exits (1 MiB + 256 bytes).
     *
     *  - Limit: roundup(N*H, 4) + N*roundup(W, 256) <= TB200_NOALLOC_MAX_SUMS, otherwise TB200_ERROR with a message
     *    naming the limit.
     *  - The CUDA device that owns the pointers must be current.  The first call on each device looks up the
     *    device address of the built-in array (a one-time set-up); make that first call outside any stream
     *    capture.  No call invokes cudaMalloc, cudaFree or any allocating library routine.
     *  - All calls on a device share the one array, and it keeps the previous call's contents.  The status word
     *    in it is cleared at the start of each call; the sums are rewritten for the extent in use.  Two calls
     *    whose kernels overlap on the GPU (different streams without ordering) race on it: order them.
     *  - a, b, out: 16-byte aligned device pointers, row-major.  `stream` is a cudaStream_t (NULL = default).
     *    Work is enqueued on `stream`; with synchronize != 0 the call also waits for it and reports a kernel
     *    that gave up on its pipeline as TB200_INTERNAL.  With synchronize == 0 nobody reads the device status
     *    word (the next call clears it): a caller that needs to know about a kernel that gave up passes
     *    synchronize != 0, which is refused with TB200_ERROR while `stream` is being captured (a synchronisation
     *    would invalidate the capture).  `err` (may be NULL) receives a message on failure. */
    TB200_API tb200_status tb200_matmul_i8_noalloc(void* stream, const int8_t* a, const int8_t* b, int32_t* out,
                                                   int32_t N, int32_t H, int32_t C, int32_t W, int32_t a_zp,
                                                   int32_t b_zp, int32_t synchronize, char* err, size_t err_len);

    /* Selects kernels: 0 = automatic (tensor-core kernels where the shape qualifies), 1 = force the
     * CUDA-core kernels (for A/B checks).  Returns the previous value. */
    TB200_API int tb200_set_kernel_policy(tb200_ctx* ctx, int policy);
    /* Name of the kernel family the last operator call used ("tc_gemm_i8", "direct_conv", ...). */
    TB200_API const char* tb200_last_kernel(const tb200_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* TB200_H */
