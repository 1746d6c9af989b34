// Device side-table of the B200 adapter: which host tensor has a device copy, and which of the two is current.
//
// The reference keeps every tensor in an Eigen container that is column-major and wider than the TOSA type: INT8 and
// INT16 values sit in int32_t, FP16 / BF16 in float (reference_model/src/ops/template_types.h:67-147).  Its external
// buffers are row-major at the same widened element type (Tensor::setTensorValue* / getTensorValue*,
// reference_model/src/tensor.cpp:2157-2179, :3662).  The device keeps tensors row-major at their true width
// (include/tb200.h).  This file holds the two conversions (column-major widened <-> row-major true width) and the
// table that decides when one has to run:
//
//   * device(t)  is called by a B200 node for each operand: uploads (marshal + copy) only if the device copy is stale;
//   * produced(t) is called for each output of a B200 node: the device copy is now the current one;
//   * host(t)    is called before anything on the CPU side reads the tensor (a stock operator, an output writer,
//                --dump_intermediates): downloads and converts only if the host copy is stale;
//   * release(t) is called from TensorTemplate::deallocate().
//
// Between two B200 nodes nothing is copied: the tensor stays on the device (the replacement for the Eigen TensorMap
// buffers between consecutive nodes).  The file depends on tb200.h only, not on Eigen or the reference's headers, so
// that the same code serves the adapter inside the reference's build and the stand-alone host test.
#ifndef B200_BUFFERS_H
#define B200_BUFFERS_H

#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/tb200.h"

namespace b200
{

// ---- conversions between the reference's column-major widened storage and row-major true-width buffers
// `shape` is the TOSA shape (outermost first).  Column-major means the first index moves fastest.
// narrow: false is returned when a value does not fit the true type (the reference would never have produced it).
bool col_major_i32_to_row_major(const int32_t* src, const std::vector<int>& shape, tb200_dtype dtype, void* dst);
void row_major_to_col_major_i32(const void* src, const std::vector<int>& shape, tb200_dtype dtype, int32_t* dst);
// float storage: FP32 is copied, FP16 / BF16 are rounded to nearest even on the way down (values the reference holds
// for such tensors are already representable, so the rounding is exact) and widened exactly on the way up
void col_major_f32_to_row_major(const float* src, const std::vector<int>& shape, tb200_dtype dtype, void* dst);
void row_major_to_col_major_f32(const void* src, const std::vector<int>& shape, tb200_dtype dtype, float* dst);
size_t dtype_bytes(tb200_dtype dtype);

// What the table needs to know about a host tensor; the adapter fills it from TosaReference::Tensor, the stand-alone
// test from its own struct.
struct HostView
{
    const void* key = nullptr;     // identity of the host tensor (its address)
    std::vector<int> shape;        // TOSA shape
    tb200_dtype dtype = TB200_INT8;
    bool is_float_storage = false; // host container holds float (FP16 / BF16 / FP32) rather than int32_t
    void* host_data = nullptr;     // column-major container data (Eigen::Tensor::data()), may be null if not allocated
};

class Buffers
{
public:
    explicit Buffers(tb200_ctx* ctx)
        : ctx_(ctx)
    {}
    ~Buffers();
    Buffers(const Buffers&)            = delete;
    Buffers& operator=(const Buffers&) = delete;

    // Device tensor with the host tensor's current value (uploads if the device copy is missing or stale).
    tb200_tensor* device(const HostView& t, std::string* err);
    // Device tensor to be written by a node (allocates if missing; no copy); afterwards call produced().
    tb200_tensor* device_for_output(const HostView& t, std::string* err);
    void produced(const HostView& t);
    // Brings the host container up to date (download + convert) if the device copy is newer.  Returns the status of
    // the download, which carries the device status word (TB200_UNPREDICTABLE for a failed REQUIRE).
    tb200_status host(const HostView& t, std::string* err);
    // The host container was written by a CPU operator: the device copy, if any, is stale.
    void host_written(const void* key);
    void release(const void* key);
    size_t resident() const
    {
        return table_.size();
    }
    // counters for tests and for the single-shot latency report
    uint64_t uploads = 0, downloads = 0, bytes_up = 0, bytes_down = 0;

private:
    struct Entry
    {
        tb200_tensor* dev = nullptr;
        bool dev_valid    = false;
        bool host_valid   = true;
    };
    tb200_ctx* ctx_;
    std::unordered_map<const void*, Entry> table_;
    std::vector<uint8_t> staging_;
    Entry* ensure(const HostView& t, std::string* err);
};

}    // namespace b200
#endif
