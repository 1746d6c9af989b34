// Custom-operator plugin for the stock reference binary: the second way in, for hosts that cannot patch the factory.
//
//     tosa_reference_model --custom_op_lib_path libtosa_b200_plugin.so ...
//
// The CLI loads the library, calls getCustomOpCreationFuncs once and closes the library again while keeping the
// function pointers it was given (reference_model/src/main.cpp:262-284), so this library must be linked with
// -Wl,-z,nodelete (see the CMake fragment).  OpCustom looks an operator up as "domain::name" and calls its eval with
// the node's tensors and the attribute string (reference_model/src/ops/custom.cpp:34-63); the instance is never
// deleted.  Operators registered here, all in domain "b200":
//
//     conv2d_rescale_clamp   inputs [x, weight, bias, multiplier, shift], one output; attributes
//                            "pad=t,b,l,r;stride=y,x;dilation=y,x;input_zp=Z;output_zp=Z;double_round=0|1;per_channel=0|1;
//                             clamp=lo,hi"   (clamp optional)
//     matmul                 inputs [a, b], one output; attributes "a_zp=Z;b_zp=Z"
//
// Tensors arrive as TosaReference::Tensor*; their Eigen containers are reached through the accessor the adapter adds
// (Tensor::b200RawData(), a virtual returning Eigen::Tensor::data() of the concrete TensorTemplate).  Inputs are uploaded and the output downloaded around every call: a
// custom operator stands alone between CPU nodes, there is no neighbour on the device to hand the tensor to.
#include <cstdlib>
#include <cstring>
#include <map>
#include <sstream>

#include "custom_op_interface.h"
#include "custom_registry.h"

#include "b200_nodes.h"

using namespace tosa;

namespace TosaReference
{

namespace
{

std::map<std::string, std::vector<int32_t>> parse_attrs(const std::string& text)
{
    std::map<std::string, std::vector<int32_t>> out;
    std::stringstream ss(text);
    std::string item;
    while (std::getline(ss, item, ';'))
    {
        const size_t eq = item.find('=');
        if (eq == std::string::npos)
            continue;
        std::string key = item.substr(0, eq);
        key.erase(0, key.find_first_not_of(" \n\t"));
        std::vector<int32_t> vals;
        std::stringstream vs(item.substr(eq + 1));
        std::string v;
        while (std::getline(vs, v, ','))
            vals.push_back((int32_t)strtol(v.c_str(), nullptr, 0));
        out[key] = vals;
    }
    return out;
}

int32_t first(const std::map<std::string, std::vector<int32_t>>& a, const char* key, int32_t dflt)
{
    auto it = a.find(key);
    return it == a.end() || it->second.empty() ? dflt : it->second[0];
}

class B200Op : public CustomOpInterface
{
public:
    explicit B200Op(std::string name)
        : name_(std::move(name))
    {}
    std::string getDomainName() const override
    {
        return "b200";
    }
    std::string getOperatorName() const override
    {
        return name_;
    }
    std::string getVersion() const override
    {
        return "1.0";
    }

    int eval(std::vector<Tensor*>& in, std::vector<Tensor*>& out, const std::string& attrs) override
    {
        b200::Runtime& rt = b200::Runtime::get();
        if (!rt.enabled() || out.size() != 1)
            return 1;
        auto a = parse_attrs(attrs);
        std::string err;
        std::vector<tb200_tensor*> d;
        for (Tensor* t : in)
        {
            rt.buffers->host_written(t);    // a CPU node may have rewritten it since the last call
            d.push_back(rt.buffers->device(b200::view_of(t), &err));
            if (!d.back())
                return 1;
        }
        tb200_tensor* y = rt.buffers->device_for_output(b200::view_of(out[0]), &err);
        if (!y)
            return 1;
        tb200_status st = TB200_ERROR;
        if (name_ == "matmul" && in.size() == 2)
            st = tb200_matmul(rt.ctx, d[0], d[1], first(a, "a_zp", 0), first(a, "b_zp", 0), nullptr, y);
        else if (name_ == "conv2d_rescale_clamp" && in.size() == 5 && a["pad"].size() == 4 && a["stride"].size() == 2 &&
                 a["dilation"].size() == 2)
        {
            tb200_epilogue e;
            memset(&e, 0, sizeof(e));
            e.has_rescale           = 1;
            e.rescale.multiplier    = d[3];
            e.rescale.shift         = d[4];
            e.rescale.output_zp     = first(a, "output_zp", 0);
            e.rescale.scale32       = 1;
            e.rescale.rounding_mode = first(a, "double_round", 1) ? TB200_DOUBLE_ROUND : TB200_SINGLE_ROUND;
            e.rescale.per_channel   = first(a, "per_channel", 1);
            if (a.count("clamp") && a["clamp"].size() == 2)
            {
                e.has_clamp   = 1;
                e.clamp_min_i = a["clamp"][0];
                e.clamp_max_i = a["clamp"][1];
            }
            st = tb200_conv2d(rt.ctx, d[0], d[1], d[2], first(a, "input_zp", 0), 0, a["pad"].data(), a["stride"].data(),
                              a["dilation"].data(), &e, y);
        }
        if (st != TB200_OK)
            return 1;
        rt.buffers->produced(b200::view_of(out[0]));
        // OpCustom ignores the return value and the next node reads the Eigen container directly: bring it back now
        st = rt.buffers->host(b200::view_of(out[0]), &err);
        return st == TB200_OK ? 0 : 1;
    }

private:
    std::string name_;
};

CustomOpInterface* make_conv()
{
    return new B200Op("conv2d_rescale_clamp");
}
CustomOpInterface* make_matmul()
{
    return new B200Op("matmul");
}

}    // namespace

extern "C" __attribute__((visibility("default"))) int getCustomOpCreationFuncs(registration_callback_t registration_func)
{
    int rc = registration_func("b200", "conv2d_rescale_clamp", &make_conv);
    rc |= registration_func("b200", "matmul", &make_matmul);
    return rc;
}

}    // namespace TosaReference
