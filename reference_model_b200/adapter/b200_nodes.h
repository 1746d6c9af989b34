// GraphNode subclasses that evaluate CONV2D / DEPTHWISE_CONV2D / MATMUL / RESCALE / CLAMP / ADD / MAX_POOL2D /
// AVG_POOL2D on the B200 through the tb200 C ABI.  Built inside the reference's tree (it needs graph_node.h, tensor.h,
// the serialization library's attribute classes and Eigen); not compiled by this repository's own build.
//
// How they enter the reference: OpFactory::newOp (reference_model/src/ops/op_factory.cpp:36-131) returns from inside its
// type switch, so the adapter's patch renames that body to newOpStock and adds a newOp that builds the stock node first
// and then offers it to b200::newOpB200, keeping the stock node when that returns nullptr.  Each node here wraps the
// stock node the factory built: checkTensorAttributes() is the stock node's own (same ERROR_IFs, same messages), eval()
// replaces the scalar loops and ends in GraphNode::eval(), which marks the outputs valid and counts the evaluation
// (reference_model/src/graph_node.cpp:77-89), exactly as the stock eval() bodies do (e.g.
// reference_model/src/ops/tensor_ops.cpp:881).
#ifndef B200_NODES_H
#define B200_NODES_H

#include <memory>
#include <string>

#include "attribute.h"
#include "graph_node.h"
#include "subgraph_traverser.h"
#include "tensor.h"

#include "b200_buffers.h"

namespace b200
{

// One tb200 context and one device side-table per process (the reference keeps its configuration in process globals
// too: reference_model/src/model_runner.cpp:22-23).  Created at the first B200 node, destroyed at exit.
struct Runtime
{
    tb200_ctx* ctx   = nullptr;
    Buffers* buffers = nullptr;
    static Runtime& get();
    bool enabled() const
    {
        return ctx != nullptr;
    }
};

// What the side-table needs to know about a reference tensor.  `b200RawData()` is the one accessor the adapter adds to
// TosaReference::Tensor (a virtual returning Eigen::Tensor::data() of the concrete TensorTemplate).
HostView view_of(TosaReference::Tensor* t);
// TOSA_REF_TYPE -> tb200_dtype; false for types this path does not take (INT4, INT48, FP64, BOOL, SHAPE).
bool to_tb200_dtype(TOSA_REF_TYPE ref, tb200_dtype* out);
// Called from TensorTemplate<T>::getTensor() (reference_model/src/tensor.h:409-412) before the host container is
// handed out, and from TensorTemplate<T>::deallocate() (:389-398): the two hooks that keep CPU readers and the
// traverser's freeing of dead tensors (reference_model/src/subgraph_traverser.cpp:864-903) correct.
void sync_host(TosaReference::Tensor* t);
void release(TosaReference::Tensor* t);

// Base of the B200 nodes: owns the stock node, forwards the graph wiring to it, converts tb200 statuses.
class NodeB200 : public TosaReference::GraphNode
{
public:
    NodeB200(TosaReference::SubgraphTraverser* sgt, tosa::Op op, uint64_t id, TosaReference::GraphNode* stock);
    ~NodeB200() override;
    int checkTensorAttributes() override;

protected:
    // device tensor holding operand i's current value / device tensor that will receive output i
    tb200_tensor* in(size_t i);
    tb200_tensor* out(size_t i);
    // first element of a rank-1, size-1 integer operand (zero points: reference_model/src/ops/tensor_ops.cpp:804,810)
    int32_t scalar_i32(size_t i);
    // TB200_OK -> outputs are current on the device, return GraphNode::eval(); TB200_ERROR / TB200_INTERNAL -> graph
    // status TOSA_ERROR and 1 (stop evaluation), as ERROR_IF does (reference_model/include/func_debug.h:147-163).
    // TB200_UNPREDICTABLE never comes back from an operator call: REQUIRE failures surface when a result is read
    // (b200::sync_host) or at the end of the run, and set TOSA_UNPREDICTABLE there.
    int finish(tb200_status st);
    std::unique_ptr<TosaReference::GraphNode> stock_;
};

class Conv2dB200 : public NodeB200
{
public:
    Conv2dB200(TosaReference::SubgraphTraverser* sgt, tosa::TosaAttributeBase* attribute, uint64_t id,
               TosaReference::GraphNode* stock, bool depthwise);
    int eval() override;

private:
    std::unique_ptr<tosa::TosaConv2dAttribute> conv_;
    std::unique_ptr<tosa::TosaDepthwiseConv2dAttribute> dw_;
};

class MatMulB200 : public NodeB200
{
public:
    using NodeB200::NodeB200;
    int eval() override;
};

class RescaleB200 : public NodeB200
{
public:
    RescaleB200(TosaReference::SubgraphTraverser* sgt, tosa::TosaAttributeBase* attribute, uint64_t id,
                TosaReference::GraphNode* stock);
    int eval() override;

private:
    std::unique_ptr<tosa::TosaRescaleAttribute> attr_;
};

class ClampB200 : public NodeB200
{
public:
    ClampB200(TosaReference::SubgraphTraverser* sgt, tosa::TosaAttributeBase* attribute, uint64_t id,
              TosaReference::GraphNode* stock);
    int eval() override;

private:
    std::unique_ptr<tosa::TosaClampAttribute> attr_;
};

class AddB200 : public NodeB200
{
public:
    using NodeB200::NodeB200;
    int eval() override;
};

class Pool2dB200 : public NodeB200
{
public:
    Pool2dB200(TosaReference::SubgraphTraverser* sgt, tosa::TosaAttributeBase* attribute, uint64_t id,
               TosaReference::GraphNode* stock, bool average);
    int eval() override;

private:
    std::unique_ptr<tosa::TosaMaxPool2dAttribute> max_;
    std::unique_ptr<tosa::TosaAvgPool2dAttribute> avg_;
};

// The factory hook.  `stock` is the node the reference's own switch built for the same arguments (the hook is called
// after it, so that type dispatch stays the reference's); ownership passes to the returned node.  Returns nullptr (and
// leaves `stock` alone) for operators or type tuples this path does not take, or when TOSA_B200 is not set to 1.
TosaReference::GraphNode* newOpB200(TosaReference::SubgraphTraverser* sgt, tosa::Op op, tosa::TosaAttributeBase* attribute,
                                    uint64_t id, TOSA_REF_TYPE inputDTYPE, TOSA_REF_TYPE outputDTYPE,
                                    TOSA_REF_TYPE weightDTYPE, TosaReference::GraphNode* stock);

}    // namespace b200
#endif
