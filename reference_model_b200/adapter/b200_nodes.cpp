// See b200_nodes.h.  Compiled inside the reference's tree only.
#include "b200_nodes.h"

#include <cstdlib>
#include <cstring>

#include "func_debug.h"

using namespace TosaReference;
using namespace tosa;

namespace b200
{

// ------------------------------------------------------------------------------------------------ runtime
Runtime& Runtime::get()
{
    static Runtime rt;
    static bool tried = false;
    if (!tried)
    {
        tried            = true;
        const char* want = getenv("TOSA_B200");
        if (want && atoi(want) == 1)
        {
            const char* dev = getenv("TOSA_B200_DEVICE");
            if (tb200_ctx_create(dev ? atoi(dev) : 0, nullptr, &rt.ctx) == TB200_OK)
                rt.buffers = new Buffers(rt.ctx);
            else
                rt.ctx = nullptr;
            // the context lives until the process ends: the reference keeps its tensors until its traverser is
            // destroyed (reference_model/src/subgraph_traverser.cpp:56-80) and release() needs the table until then
        }
    }
    return rt;
}

bool to_tb200_dtype(TOSA_REF_TYPE ref, tb200_dtype* out)
{
    switch (ref)
    {
        case TOSA_REF_TYPE_INT8: *out = TB200_INT8; return true;
        case TOSA_REF_TYPE_UINT8: *out = TB200_UINT8; return true;
        case TOSA_REF_TYPE_INT16: *out = TB200_INT16; return true;
        case TOSA_REF_TYPE_UINT16: *out = TB200_UINT16; return true;
        case TOSA_REF_TYPE_INT32: *out = TB200_INT32; return true;
        case TOSA_REF_TYPE_FP16: *out = TB200_FP16; return true;
        case TOSA_REF_TYPE_BF16: *out = TB200_BF16; return true;
        case TOSA_REF_TYPE_FP32: *out = TB200_FP32; return true;
        case TOSA_REF_TYPE_FP8E4M3: *out = TB200_FP8E4M3; return true;
        case TOSA_REF_TYPE_FP8E5M2: *out = TB200_FP8E5M2; return true;
        default: return false;
    }
}

HostView view_of(Tensor* t)
{
    HostView v;
    v.key   = t;
    v.shape = t->getShape();
    to_tb200_dtype(t->getDtype(), &v.dtype);
    // FP16 / BF16 / FP8 / FP32 tensors are held as float, the integer types as int32_t
    // (reference_model/src/ops/template_types.h:67-147)
    v.is_float_storage = v.dtype == TB200_FP16 || v.dtype == TB200_BF16 || v.dtype == TB200_FP32 || v.dtype == TB200_FP8E4M3 ||
                         v.dtype == TB200_FP8E5M2;
    v.host_data = t->is_allocated() ? t->b200RawData() : nullptr;
    return v;
}

void sync_host(Tensor* t)
{
    Runtime& rt = Runtime::get();
    if (!rt.enabled())
        return;
    std::string err;
    const tb200_status st = rt.buffers->host(view_of(t), &err);
    // a REQUIRE that failed in some kernel since the last read surfaces here, as it would have in the stock eval()
    if (st == TB200_UNPREDICTABLE && t->getProducer())
        t->getProducer()->getParentSGT()->setGraphStatus(GraphStatus::TOSA_UNPREDICTABLE);
    else if ((st == TB200_ERROR || st == TB200_INTERNAL) && t->getProducer())
    {
        fprintf(g_func_debug.func_debug_file, "b200: cannot bring %s back to the host: %s\n", t->getName().c_str(), err.c_str());
        t->getProducer()->getParentSGT()->setGraphStatus(GraphStatus::TOSA_ERROR);
    }
}

void release(Tensor* t)
{
    Runtime& rt = Runtime::get();
    if (rt.enabled())
        rt.buffers->release(t);
}

// ------------------------------------------------------------------------------------------------ base node
NodeB200::NodeB200(SubgraphTraverser* sgt, Op op, uint64_t id, GraphNode* stock)
    : GraphNode(sgt, op, id)
    , stock_(stock)
{}

NodeB200::~NodeB200()
{}

int NodeB200::checkTensorAttributes()
{
    // the stock node validates operand counts, ranks, dtypes and attributes (and prints its own messages); it sees the
    // same tensors this node was wired to (reference_model/src/subgraph_traverser.cpp:1100-1130)
    for (Tensor* t : inputs)
        stock_->addInputTensor(t);
    for (Tensor* t : outputs)
        stock_->addOutputTensor(t);
    return stock_->checkTensorAttributes();
}

tb200_tensor* NodeB200::in(size_t i)
{
    std::string err;
    Tensor* t        = inputs[i];
    // a tensor a CPU node produced is current on the host only; Buffers uploads it once
    tb200_tensor* d  = Runtime::get().buffers->device(view_of(t), &err);
    if (!d)
        fprintf(g_func_debug.func_debug_file, "b200: operand %s: %s\n", t->getName().c_str(), err.c_str());
    return d;
}

tb200_tensor* NodeB200::out(size_t i)
{
    std::string err;
    tb200_tensor* d = Runtime::get().buffers->device_for_output(view_of(outputs[i]), &err);
    if (!d)
        fprintf(g_func_debug.func_debug_file, "b200: output %s: %s\n", outputs[i]->getName().c_str(), err.c_str());
    return d;
}

int32_t NodeB200::scalar_i32(size_t i)
{
    Tensor* t = inputs[i];
    sync_host(t);    // zero points are CONST outputs: already on the host, this is a table lookup
    return t->is_allocated() ? static_cast<const int32_t*>(t->b200RawData())[0] : 0;
}

int NodeB200::finish(tb200_status st)
{
    if (st == TB200_ERROR || st == TB200_INTERNAL)
    {
        fprintf(g_func_debug.func_debug_file, "b200: %s\n", tb200_last_error(Runtime::get().ctx));
        if (parent_sgt->getGraphStatus() != GraphStatus::TOSA_UNPREDICTABLE)
            parent_sgt->setGraphStatus(GraphStatus::TOSA_ERROR);
        return 1;
    }
    for (Tensor* t : outputs)
        Runtime::get().buffers->produced(view_of(t));
    return GraphNode::eval();
}

// ------------------------------------------------------------------------------------------------ operators
Conv2dB200::Conv2dB200(SubgraphTraverser* sgt, TosaAttributeBase* attribute, uint64_t id, GraphNode* stock, bool depthwise)
    : NodeB200(sgt, depthwise ? Op_DEPTHWISE_CONV2D : Op_CONV2D, id, stock)
{
    if (depthwise)
        dw_ = std::make_unique<TosaDepthwiseConv2dAttribute>(dynamic_cast<TosaDepthwiseConv2dAttribute*>(attribute));
    else
        conv_ = std::make_unique<TosaConv2dAttribute>(dynamic_cast<TosaConv2dAttribute*>(attribute));
}

int Conv2dB200::eval()
{
    // operands [input, weight, bias, input_zp, weight_zp] (reference_model/src/ops/tensor_ops.cpp:690-720, :804-811)
    const std::vector<int32_t>& pad      = conv_ ? conv_->pad() : dw_->pad();
    const std::vector<int32_t>& stride   = conv_ ? conv_->stride() : dw_->stride();
    const std::vector<int32_t>& dilation = conv_ ? conv_->dilation() : dw_->dilation();
    tb200_tensor *x = in(0), *w = in(1), *b = in(2), *y = out(0);
    if (!x || !w || !b || !y)
        return finish(TB200_INTERNAL);
    const int32_t in_zp = scalar_i32(3), w_zp = scalar_i32(4);
    tb200_ctx* ctx = Runtime::get().ctx;
    const tb200_status st =
        conv_ ? tb200_conv2d(ctx, x, w, b, in_zp, w_zp, pad.data(), stride.data(), dilation.data(), nullptr, y)
              : tb200_depthwise_conv2d(ctx, x, w, b, in_zp, w_zp, pad.data(), stride.data(), dilation.data(), nullptr, y);
    return finish(st);
}

int MatMulB200::eval()
{
    // operands [a, b, a_zp, b_zp] (reference_model/src/ops/tensor_ops.cpp:1347-1420)
    tb200_tensor *a = in(0), *b = in(1), *y = out(0);
    if (!a || !b || !y)
        return finish(TB200_INTERNAL);
    return finish(tb200_matmul(Runtime::get().ctx, a, b, scalar_i32(2), scalar_i32(3), nullptr, y));
}

RescaleB200::RescaleB200(SubgraphTraverser* sgt, TosaAttributeBase* attribute, uint64_t id, GraphNode* stock)
    : NodeB200(sgt, Op_RESCALE, id, stock)
    , attr_(std::make_unique<TosaRescaleAttribute>(dynamic_cast<TosaRescaleAttribute*>(attribute)))
{}

int RescaleB200::eval()
{
    // operands [input, multiplier, shift, input_zp, output_zp] (reference_model/src/ops/type_conversion.cpp:71-154)
    tb200_tensor *x = in(0), *m = in(1), *s = in(2), *y = out(0);
    if (!x || !m || !s || !y)
        return finish(TB200_INTERNAL);
    tb200_rescale_attr a;
    memset(&a, 0, sizeof(a));
    a.multiplier      = m;
    a.shift           = s;
    a.input_zp        = scalar_i32(3);
    a.output_zp       = scalar_i32(4);
    a.scale32         = attr_->scale32();
    a.rounding_mode   = attr_->rounding_mode() == RoundingMode_DOUBLE_ROUND    ? TB200_DOUBLE_ROUND
                        : attr_->rounding_mode() == RoundingMode_INEXACT_ROUND ? TB200_INEXACT_ROUND
                                                                               : TB200_SINGLE_ROUND;
    a.per_channel     = attr_->per_channel();
    a.input_unsigned  = attr_->input_unsigned();
    a.output_unsigned = attr_->output_unsigned();
    return finish(tb200_rescale(Runtime::get().ctx, x, &a, y));
}

ClampB200::ClampB200(SubgraphTraverser* sgt, TosaAttributeBase* attribute, uint64_t id, GraphNode* stock)
    : NodeB200(sgt, Op_CLAMP, id, stock)
    , attr_(std::make_unique<TosaClampAttribute>(dynamic_cast<TosaClampAttribute*>(attribute)))
{}

int ClampB200::eval()
{
    // min / max arrive as bytes in the input's serialization dtype (reference_model/src/ops/activation_funcs.cpp:41-95)
    tb200_tensor *x = in(0), *y = out(0);
    if (!x || !y)
        return finish(TB200_INTERNAL);
    int32_t lo_i = 0, hi_i = 0;
    float lo_f = 0.f, hi_f = 0.f;
    const std::vector<uint8_t>&mn = attr_->min_val(), &mx = attr_->max_val();
    switch (inputs[0]->getDtype())
    {
        case TOSA_REF_TYPE_INT8:
            lo_i = (int8_t)mn[0];
            hi_i = (int8_t)mx[0];
            break;
        case TOSA_REF_TYPE_INT16:
            lo_i = (int16_t)(mn[0] | (mn[1] << 8));
            hi_i = (int16_t)(mx[0] | (mx[1] << 8));
            break;
        case TOSA_REF_TYPE_FP32:
            memcpy(&lo_f, mn.data(), 4);
            memcpy(&hi_f, mx.data(), 4);
            break;
        default:
        {
            // FP16 / BF16 bounds: decode with the serialization library, as the stock node does
            std::vector<float> a, b;
            if (inputs[0]->getDtype() == TOSA_REF_TYPE_FP16)
            {
                std::vector<half_float::half> ha, hb;
                TosaSerializationHandler::ConvertU8toF16(mn, 1, ha);
                TosaSerializationHandler::ConvertU8toF16(mx, 1, hb);
                lo_f = (float)ha[0];
                hi_f = (float)hb[0];
            }
            else
            {
                std::vector<bf16> ba, bb;
                TosaSerializationHandler::ConvertU8toBF16(mn, 1, ba);
                TosaSerializationHandler::ConvertU8toBF16(mx, 1, bb);
                lo_f = (float)ba[0];
                hi_f = (float)bb[0];
            }
        }
    }
    const int nan_ignore = attr_->nan_mode() == NanPropagationMode_IGNORE;
    return finish(tb200_clamp(Runtime::get().ctx, x, lo_i, hi_i, lo_f, hi_f, nan_ignore, y));
}

int AddB200::eval()
{
    tb200_tensor *a = in(0), *b = in(1), *y = out(0);
    if (!a || !b || !y)
        return finish(TB200_INTERNAL);
    return finish(tb200_add(Runtime::get().ctx, a, b, y));
}

Pool2dB200::Pool2dB200(SubgraphTraverser* sgt, TosaAttributeBase* attribute, uint64_t id, GraphNode* stock, bool average)
    : NodeB200(sgt, average ? Op_AVG_POOL2D : Op_MAX_POOL2D, id, stock)
{
    if (average)
        avg_ = std::make_unique<TosaAvgPool2dAttribute>(dynamic_cast<TosaAvgPool2dAttribute*>(attribute));
    else
        max_ = std::make_unique<TosaMaxPool2dAttribute>(dynamic_cast<TosaMaxPool2dAttribute*>(attribute));
}

int Pool2dB200::eval()
{
    tb200_tensor *x = in(0), *y = out(0);
    if (!x || !y)
        return finish(TB200_INTERNAL);
    tb200_ctx* ctx = Runtime::get().ctx;
    if (max_)
        return finish(tb200_max_pool2d(ctx, x, max_->kernel().data(), max_->pad().data(), max_->stride().data(), y));
    // AVG_POOL2D operands [input, input_zp, output_zp] (reference_model/src/ops/tensor_ops.cpp:476, :509-512)
    return finish(tb200_avg_pool2d(ctx, x, avg_->kernel().data(), avg_->pad().data(), avg_->stride().data(), scalar_i32(1),
                                   scalar_i32(2), y));
}

// ------------------------------------------------------------------------------------------------ factory hook
GraphNode* newOpB200(SubgraphTraverser* sgt, Op op, TosaAttributeBase* attribute, uint64_t id, TOSA_REF_TYPE inputDTYPE,
                     TOSA_REF_TYPE outputDTYPE, TOSA_REF_TYPE weightDTYPE, GraphNode* stock)
{
    if (!stock || !Runtime::get().enabled() || g_func_config.precise_mode || g_func_config.bounds_mode)
        return nullptr;    // the fp64 precise / bounds runs stay on the CPU: they are the oracle's modes, not this path's
    const bool i8 = inputDTYPE == TOSA_REF_TYPE_INT8;
    const bool fl = inputDTYPE == TOSA_REF_TYPE_FP16 || inputDTYPE == TOSA_REF_TYPE_BF16 || inputDTYPE == TOSA_REF_TYPE_FP32;
    switch (op)
    {
        case Op_CONV2D:
        case Op_DEPTHWISE_CONV2D:
            // <INT8,INT8,INT32,INT32> and the floating tuples with fp32 accumulation
            // (reference_model/src/ops/tensor_ops.cpp:2220-2229, :2241-2251)
            if ((i8 && weightDTYPE == TOSA_REF_TYPE_INT8 && outputDTYPE == TOSA_REF_TYPE_INT32) || (fl && weightDTYPE == inputDTYPE))
                return new Conv2dB200(sgt, attribute, id, stock, op == Op_DEPTHWISE_CONV2D);
            return nullptr;
        case Op_MATMUL:
            if ((i8 && outputDTYPE == TOSA_REF_TYPE_INT32) || fl)
                return new MatMulB200(sgt, op, id, stock);
            return nullptr;
        case Op_RESCALE:
            return new RescaleB200(sgt, attribute, id, stock);
        case Op_CLAMP:
            if (i8 || inputDTYPE == TOSA_REF_TYPE_INT16 || fl)
                return new ClampB200(sgt, attribute, id, stock);
            return nullptr;
        case Op_ADD:
            if (inputDTYPE == TOSA_REF_TYPE_INT32 || fl)
                return new AddB200(sgt, op, id, stock);
            return nullptr;
        case Op_MAX_POOL2D:
        case Op_AVG_POOL2D:
            if (i8 || inputDTYPE == TOSA_REF_TYPE_INT16 || fl)
                return new Pool2dB200(sgt, attribute, id, stock, op == Op_AVG_POOL2D);
            return nullptr;
        default:
            return nullptr;
    }
}

}    // namespace b200
