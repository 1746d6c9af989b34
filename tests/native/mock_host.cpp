// A stand-in for the reference's host, small enough to build with g++ alone, that drives the adapter's device
// side-table (reference_model_b200/adapter/b200_buffers.{h,cpp}) the way the reference's traverser would:
//
//   * tensors live in column-major containers widened to int32_t, as the reference's Eigen tensors do
//     (reference_model/src/ops/template_types.h:67-147);
//   * nodes are evaluated in order, every operand is requested from the side-table, every output is marked produced;
//   * after a node has run, an operand whose consumers have all been evaluated is deallocated
//     (reference_model/src/subgraph_traverser.cpp:864-903);
//   * a node that runs on the CPU reads its operand through host() and marks its result host_written(), as the two
//     hooks in TensorTemplate::getTensor() / the stock eval() path do in the patched reference.
//
//   mock_host marshal     conversions only (no GPU): every type, ranks 1..5, against a plain index loop
//   mock_host run         CONV2D -> RESCALE -> CLAMP -> [CPU node] -> CONV2D 1x1 on the device, compared with the
//                         CPU oracle of this repository; checks copy counts and the freeing of dead tensors
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <random>
#include <string>
#include <vector>

#include "../../reference_model_b200/adapter/b200_buffers.h"

extern "C"
{
    void orc_conv2d_i32(const int32_t* in, const int32_t* w, const int32_t* bias, int bias_n, int N, int IH, int IW,
                        int IC, int OC, int KH, int KW, int OH, int OW, const int* pad, const int* stride,
                        const int* dilation, int32_t in_zp, int32_t w_zp, int32_t* out, int nthreads);
    int orc_rescale(const int32_t* in, int64_t outer, int C, const int32_t* multiplier, const int32_t* shift,
                    int per_channel, int scale32, int rounding_mode, int32_t input_zp, int32_t output_zp, int in_bits,
                    int out_bits, int input_unsigned, int output_unsigned, int32_t* out);
    int orc_clamp_i32(const int32_t* in, int64_t n, int32_t min_val, int32_t max_val, int32_t* out);
}

namespace
{

int g_fail = 0;
#define CHECK(cond, ...)                                                                                               \
    do                                                                                                                 \
    {                                                                                                                  \
        if (!(cond))                                                                                                   \
        {                                                                                                              \
            printf("FAIL %s:%d: ", __FILE__, __LINE__);                                                                \
            printf(__VA_ARGS__);                                                                                       \
            printf("\n");                                                                                              \
            g_fail++;                                                                                                  \
        }                                                                                                              \
    } while (0)

size_t count_of(const std::vector<int>& shape)
{
    size_t n = 1;
    for (int d : shape)
        n *= (size_t)d;
    return n;
}

// position of row-major element `i` in a column-major container of the same shape (first index fastest)
size_t col_major_pos(size_t i, const std::vector<int>& shape)
{
    std::vector<size_t> idx(shape.size());
    for (int d = (int)shape.size() - 1; d >= 0; d--)
    {
        idx[d] = i % (size_t)shape[d];
        i /= (size_t)shape[d];
    }
    size_t pos = 0, stride = 1;
    for (size_t d = 0; d < shape.size(); d++)
    {
        pos += idx[d] * stride;
        stride *= (size_t)shape[d];
    }
    return pos;
}

// ---- a host tensor of the mock: column-major, widened
struct HostTensor
{
    std::string name;
    std::vector<int> shape;
    tb200_dtype dtype;
    std::vector<int32_t> data;    // column-major
    int consumers = 0, consumed = 0;
    bool is_output = false;

    b200::HostView view()
    {
        b200::HostView v;
        v.key              = this;
        v.shape            = shape;
        v.dtype            = dtype;
        v.is_float_storage = false;
        v.host_data        = data.empty() ? nullptr : data.data();
        return v;
    }
    void set_row_major(const std::vector<int32_t>& rm)
    {
        data.resize(rm.size());
        for (size_t i = 0; i < rm.size(); i++)
            data[col_major_pos(i, shape)] = rm[i];
    }
    std::vector<int32_t> row_major() const
    {
        std::vector<int32_t> rm(data.size());
        for (size_t i = 0; i < rm.size(); i++)
            rm[i] = data[col_major_pos(i, shape)];
        return rm;
    }
};

// ---------------------------------------------------------------------------------------------------------------------
int marshal_selftest()
{
    std::mt19937 rng(1234);
    const struct
    {
        tb200_dtype dt;
        int lo, hi;
    } int_types[] = { { TB200_INT8, -128, 127 }, { TB200_INT16, -32768, 32767 }, { TB200_INT32, INT32_MIN, INT32_MAX } };
    const std::vector<std::vector<int>> shapes = { { 7 }, { 3, 5 }, { 2, 3, 4 }, { 2, 5, 3, 4 }, { 2, 3, 1, 4, 5 }, { 1, 1, 1, 1 } };
    size_t checked = 0;
    for (auto& ty : int_types)
        for (auto& shape : shapes)
        {
            const size_t n = count_of(shape);
            std::uniform_int_distribution<int64_t> dist(ty.lo, ty.hi);
            std::vector<int32_t> rm(n), cm(n), back(n);
            for (auto& v : rm)
                v = (int32_t)dist(rng);
            for (size_t i = 0; i < n; i++)
                cm[col_major_pos(i, shape)] = rm[i];
            std::vector<uint8_t> dev(n * b200::dtype_bytes(ty.dt));
            CHECK(b200::col_major_i32_to_row_major(cm.data(), shape, ty.dt, dev.data()), "narrowing refused in-range values");
            for (size_t i = 0; i < n; i++)
            {
                int32_t got = ty.dt == TB200_INT8    ? (int32_t)((int8_t*)dev.data())[i]
                              : ty.dt == TB200_INT16 ? (int32_t)((int16_t*)dev.data())[i]
                                                     : ((int32_t*)dev.data())[i];
                if (got != rm[i])
                {
                    CHECK(false, "down: dtype %d rank %zu element %zu: %d != %d", (int)ty.dt, shape.size(), i, got, rm[i]);
                    break;
                }
            }
            b200::row_major_to_col_major_i32(dev.data(), shape, ty.dt, back.data());
            CHECK(back == cm, "up: dtype %d rank %zu round trip differs", (int)ty.dt, shape.size());
            checked += n;
        }
    // a value outside the type must be refused, not wrapped
    {
        std::vector<int32_t> cm = { 1, 2, 300 };
        int8_t dev[3];
        CHECK(!b200::col_major_i32_to_row_major(cm.data(), { 3 }, TB200_INT8, dev), "300 accepted as INT8");
    }
    // floating storage: fp32 verbatim; fp16 / bf16 values that are representable survive the round trip bit for bit
    const tb200_dtype f_types[] = { TB200_FP32, TB200_FP16, TB200_BF16 };
    for (tb200_dtype dt : f_types)
        for (auto& shape : shapes)
        {
            const size_t n = count_of(shape);
            std::vector<float> rm(n), cm(n), back(n);
            for (size_t i = 0; i < n; i++)
            {
                // integers up to 255 scaled by powers of two are exact in all three types (8 significant bits)
                const int mant = (int)(rng() % 511) - 255;
                const int ex   = (int)(rng() % 13) - 6;    // |value| <= 255 * 64, inside fp16
                rm[i]          = std::ldexp((float)mant, ex);
            }
            if (n > 2)
            {
                rm[0] = -0.0f;
                rm[1] = INFINITY;
            }
            for (size_t i = 0; i < n; i++)
                cm[col_major_pos(i, shape)] = rm[i];
            std::vector<uint8_t> dev(n * b200::dtype_bytes(dt));
            b200::col_major_f32_to_row_major(cm.data(), shape, dt, dev.data());
            if (dt == TB200_FP32)
                CHECK(memcmp(dev.data(), rm.data(), n * 4) == 0, "fp32 row-major bytes differ");
            b200::row_major_to_col_major_f32(dev.data(), shape, dt, back.data());
            CHECK(memcmp(back.data(), cm.data(), n * 4) == 0, "float dtype %d rank %zu round trip differs", (int)dt, shape.size());
            checked += n;
        }
    // known encodings: 1.0 -> 0x3C00 (fp16), 0x3F80 (bf16); round to nearest even on the way down
    {
        float one = 1.0f;
        uint16_t h, b;
        b200::col_major_f32_to_row_major(&one, { 1 }, TB200_FP16, &h);
        b200::col_major_f32_to_row_major(&one, { 1 }, TB200_BF16, &b);
        CHECK(h == 0x3C00 && b == 0x3F80, "1.0 encodes as %04x / %04x", h, b);
        float tie = 1.0f + 1.0f / 2048.0f;    // halfway between two fp16 values, even neighbour is 1.0
        b200::col_major_f32_to_row_major(&tie, { 1 }, TB200_FP16, &h);
        CHECK(h == 0x3C00, "fp16 tie rounds to %04x", h);
    }
    printf("marshal checked=%zu failures=%d\n", checked, g_fail);
    return g_fail ? 1 : 0;
}

// ---------------------------------------------------------------------------------------------------------------------
struct Node
{
    std::string name;
    std::vector<HostTensor*> in;
    HostTensor* out;
    bool on_device;
    std::function<tb200_status(std::vector<tb200_tensor*>&, tb200_tensor*)> dev_eval;
    std::function<void()> cpu_eval;
};

int run_graph()
{
    tb200_ctx* ctx = nullptr;
    if (tb200_ctx_create(0, nullptr, &ctx) != TB200_OK)
    {
        printf("FAIL: no context\n");
        return 1;
    }
    int rc = 0;
    {
        b200::Buffers buffers(ctx);
        std::mt19937 rng(99);
        auto fill = [&](HostTensor& t, int lo, int hi) {
            std::uniform_int_distribution<int> d(lo, hi);
            std::vector<int32_t> rm(count_of(t.shape));
            for (auto& v : rm)
                v = d(rng);
            t.set_row_major(rm);
        };
        const int N = 2, H = 12, W = 12, IC = 16, OC = 32, OC2 = 48;
        HostTensor x{ "x", { N, H, W, IC }, TB200_INT8 }, w1{ "w1", { OC, 3, 3, IC }, TB200_INT8 }, b1{ "b1", { OC }, TB200_INT32 },
            m1{ "m1", { OC }, TB200_INT32 }, s1{ "s1", { OC }, TB200_INT8 }, a1{ "a1", { N, H, W, OC }, TB200_INT32 },
            r1{ "r1", { N, H, W, OC }, TB200_INT8 }, c1{ "c1", { N, H, W, OC }, TB200_INT8 }, h1{ "h1", { N, H, W, OC }, TB200_INT8 },
            w2{ "w2", { OC2, 1, 1, OC }, TB200_INT8 }, b2{ "b2", { OC2 }, TB200_INT32 }, a2{ "a2", { N, H, W, OC2 }, TB200_INT32 };
        fill(x, -128, 127);
        fill(w1, -127, 127);
        fill(b1, -20000, 20000);
        fill(m1, 1 << 30, INT32_MAX);
        fill(s1, 38, 44);
        fill(w2, -127, 127);
        fill(b2, -5000, 5000);
        a2.is_output = true;
        const int in_zp = -3, out_zp = 5;
        const int32_t pad1[4] = { 1, 1, 1, 1 }, pad0[4] = { 0, 0, 0, 0 }, one2[2] = { 1, 1 };

        std::vector<Node> nodes;
        nodes.push_back({ "conv1", { &x, &w1, &b1 }, &a1, true, [&](std::vector<tb200_tensor*>& d, tb200_tensor* y) {
                             return tb200_conv2d(ctx, d[0], d[1], d[2], in_zp, 0, pad1, one2, one2, nullptr, y);
                         },
                          nullptr });
        nodes.push_back({ "rescale1", { &a1, &m1, &s1 }, &r1, true, [&](std::vector<tb200_tensor*>& d, tb200_tensor* y) {
                             tb200_rescale_attr ra;
                             memset(&ra, 0, sizeof(ra));
                             ra.multiplier    = d[1];
                             ra.shift         = d[2];
                             ra.output_zp     = out_zp;
                             ra.scale32       = 1;
                             ra.rounding_mode = TB200_DOUBLE_ROUND;
                             ra.per_channel   = 1;
                             return tb200_rescale(ctx, d[0], &ra, y);
                         },
                          nullptr });
        nodes.push_back({ "clamp1", { &r1 }, &c1, true, [&](std::vector<tb200_tensor*>& d, tb200_tensor* y) {
                             return tb200_clamp(ctx, d[0], -100, 100, 0.f, 0.f, 0, y);
                         },
                          nullptr });
        // a node the device path does not take: runs on the host containers (column-major, element-wise)
        nodes.push_back({ "cpu_negate", { &c1 }, &h1, false, nullptr, [&]() {
                             h1.data.resize(c1.data.size());
                             for (size_t i = 0; i < c1.data.size(); i++)
                                 h1.data[i] = -c1.data[i];
                         } });
        nodes.push_back({ "conv2", { &h1, &w2, &b2 }, &a2, true, [&](std::vector<tb200_tensor*>& d, tb200_tensor* y) {
                             return tb200_conv2d(ctx, d[0], d[1], d[2], out_zp, 0, pad0, one2, one2, nullptr, y);
                         },
                          nullptr });
        for (auto& n : nodes)
            for (auto* t : n.in)
                t->consumers++;

        std::string err;
        size_t resident_peak = 0;
        for (auto& n : nodes)
        {
            // allocate the output's host container, as SubgraphTraverser::allocateTensor does before evaluation
            n.out->data.assign(count_of(n.out->shape), 0);
            if (n.on_device)
            {
                std::vector<tb200_tensor*> d;
                for (auto* t : n.in)
                {
                    d.push_back(buffers.device(t->view(), &err));
                    CHECK(d.back() != nullptr, "%s: operand %s: %s", n.name.c_str(), t->name.c_str(), err.c_str());
                }
                tb200_tensor* y = buffers.device_for_output(n.out->view(), &err);
                CHECK(y != nullptr, "%s: output: %s", n.name.c_str(), err.c_str());
                if (g_fail)
                    break;
                tb200_status st = n.dev_eval(d, y);
                CHECK(st == TB200_OK, "%s: status %d: %s", n.name.c_str(), (int)st, tb200_last_error(ctx));
                buffers.produced(n.out->view());
            }
            else
            {
                for (auto* t : n.in)
                    CHECK(buffers.host(t->view(), &err) == TB200_OK, "%s: reading %s: %s", n.name.c_str(), t->name.c_str(), err.c_str());
                n.cpu_eval();
                buffers.host_written(n.out);
            }
            resident_peak = std::max(resident_peak, buffers.resident());
            for (auto* t : n.in)
                if (++t->consumed == t->consumers && !t->is_output)
                {
                    buffers.release(t);
                    t->data.clear();
                    t->data.shrink_to_fit();
                }
            if (g_fail)
                break;
        }
        if (!g_fail)
        {
            CHECK(buffers.host(a2.view(), &err) == TB200_OK, "reading the output: %s", err.c_str());
            // a second read must not copy again
            const uint64_t before = buffers.downloads;
            CHECK(buffers.host(a2.view(), &err) == TB200_OK && buffers.downloads == before, "second read copied again");
        }

        // ---- the same graph on the CPU oracle, row-major int32 containers
        if (!g_fail)
        {
            // the inputs were freed by the traverser: regenerate them from the same seed
            std::mt19937 rng2(99);
            rng = rng2;
            HostTensor x_{ "x", x.shape, TB200_INT8 }, w1_{ "w1", w1.shape, TB200_INT8 }, b1_{ "b1", b1.shape, TB200_INT32 },
                m1_{ "m1", m1.shape, TB200_INT32 }, s1_{ "s1", s1.shape, TB200_INT8 }, w2_{ "w2", w2.shape, TB200_INT8 },
                b2_{ "b2", b2.shape, TB200_INT32 };
            fill(x_, -128, 127);
            fill(w1_, -127, 127);
            fill(b1_, -20000, 20000);
            fill(m1_, 1 << 30, INT32_MAX);
            fill(s1_, 38, 44);
            fill(w2_, -127, 127);
            fill(b2_, -5000, 5000);
            const int pad1i[4] = { 1, 1, 1, 1 }, pad0i[4] = { 0, 0, 0, 0 }, one[2] = { 1, 1 };
            const size_t n1    = (size_t)N * H * W * OC;
            std::vector<int32_t> o_a1(n1), o_r1(n1), o_c1(n1), o_h1(n1), o_a2((size_t)N * H * W * OC2);
            orc_conv2d_i32(x_.row_major().data(), w1_.row_major().data(), b1_.row_major().data(), OC, N, H, W, IC, OC, 3, 3, H, W,
                           pad1i, one, one, in_zp, 0, o_a1.data(), 1);
            int r = orc_rescale(o_a1.data(), (int64_t)N * H * W, OC, m1_.row_major().data(), s1_.row_major().data(), 1, 1, 1, 0,
                                out_zp, 32, 8, 0, 0, o_r1.data());
            CHECK(r == 0, "oracle rescale status %d", r);
            orc_clamp_i32(o_r1.data(), (int64_t)n1, -100, 100, o_c1.data());
            for (size_t i = 0; i < n1; i++)
                o_h1[i] = -o_c1[i];
            orc_conv2d_i32(o_h1.data(), w2_.row_major().data(), b2_.row_major().data(), OC2, N, H, W, OC, OC2, 1, 1, H, W, pad0i,
                           one, one, out_zp, 0, o_a2.data(), 1);
            std::vector<int32_t> got = a2.row_major();
            size_t bad = 0;
            for (size_t i = 0; i < got.size(); i++)
                bad += got[i] != o_a2[i];
            CHECK(bad == 0, "%zu of %zu output elements differ from the oracle", bad, got.size());
            // copies: x w1 b1 | m1 s1 | h1 w2 b2 up; c1 and a2 down; nothing for a1, r1 (device to device)
            CHECK(buffers.uploads == 8, "uploads %llu, expected 8", (unsigned long long)buffers.uploads);
            CHECK(buffers.downloads == 2, "downloads %llu, expected 2", (unsigned long long)buffers.downloads);
            // dead tensors were freed as the traverser went: only the output is left, and never all twelve at once
            CHECK(buffers.resident() == 1, "resident %zu, expected 1", buffers.resident());
            CHECK(resident_peak <= 6, "peak resident %zu", resident_peak);
            printf("run elements=%zu uploads=%llu downloads=%llu peak_resident=%zu launches=%llu\n", got.size(),
                   (unsigned long long)buffers.uploads, (unsigned long long)buffers.downloads, resident_peak,
                   (unsigned long long)tb200_launch_count(ctx));
        }
        buffers.release(&a2);
        rc = g_fail ? 1 : 0;
    }
    tb200_ctx_destroy(ctx);
    printf("run failures=%d\n", g_fail);
    return rc;
}

}    // namespace

int main(int argc, char** argv)
{
    if (argc >= 2 && !strcmp(argv[1], "marshal"))
        return marshal_selftest();
    if (argc >= 2 && !strcmp(argv[1], "run"))
        return run_graph();
    printf("usage: mock_host marshal|run\n");
    return 2;
}
