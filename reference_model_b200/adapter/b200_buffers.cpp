// See b200_buffers.h.
#include "b200_buffers.h"

#include <cmath>
#include <cstring>

namespace b200
{

size_t dtype_bytes(tb200_dtype d)
{
    switch (d)
    {
        case TB200_INT8:
        case TB200_UINT8:
        case TB200_FP8E4M3:
        case TB200_FP8E5M2:
            return 1;
        case TB200_INT16:
        case TB200_UINT16:
        case TB200_FP16:
        case TB200_BF16:
            return 2;
        default:
            return 4;
    }
}

namespace
{

// Walks a tensor in row-major order and yields, for each element, its column-major offset.  The innermost TOSA
// dimension has the largest column-major stride, so a plain nested counter is enough (no division per element).
template <typename F>
void for_each_row_major(const std::vector<int>& shape, F&& fn)
{
    const int rank = (int)shape.size();
    int64_t total  = 1;
    for (int d : shape)
        total *= d;
    if (total == 0)
        return;
    std::vector<int64_t> cm_stride(rank > 0 ? rank : 1, 1);
    for (int i = 1; i < rank; i++)
        cm_stride[i] = cm_stride[i - 1] * shape[i - 1];
    std::vector<int> idx(rank > 0 ? rank : 1, 0);
    int64_t cm = 0;
    for (int64_t rm = 0; rm < total; rm++)
    {
        fn(rm, cm);
        for (int d = rank - 1; d >= 0; d--)
        {
            cm += cm_stride[d];
            if (++idx[d] < shape[d])
                break;
            cm -= cm_stride[d] * shape[d];
            idx[d] = 0;
        }
    }
}

uint16_t f32_to_f16_bits(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const int32_t exp   = (int32_t)((x >> 23) & 0xff) - 127 + 15;
    uint32_t man        = x & 0x7fffffu;
    if (((x >> 23) & 0xff) == 0xff)
        return (uint16_t)(sign | 0x7c00u | (man ? 0x200u | (man >> 13) : 0));
    if (exp >= 31)
        return (uint16_t)(sign | 0x7c00u);
    if (exp <= 0)
    {
        if (exp < -10)
            return (uint16_t)sign;
        man |= 0x800000u;
        const int shift    = 14 - exp;
        uint32_t half      = man >> shift;
        const uint32_t rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1)))
            half++;
        return (uint16_t)(sign | half);
    }
    uint32_t half      = ((uint32_t)exp << 10) | (man >> 13);
    const uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1)))
        half++;
    return (uint16_t)(sign | half);
}

float f16_bits_to_f32(uint16_t h)
{
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp        = (h >> 10) & 0x1f;
    uint32_t man        = h & 0x3ffu;
    uint32_t x;
    if (exp == 0)
    {
        if (man == 0)
            x = sign;
        else
        {
            int e = -1;
            do
            {
                e++;
                man <<= 1;
            } while (!(man & 0x400u));
            x = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    }
    else if (exp == 31)
        x = sign | 0x7f800000u | (man << 13);
    else
        x = sign | ((exp + 127 - 15) << 23) | (man << 13);
    float f;
    memcpy(&f, &x, 4);
    return f;
}

uint16_t f32_to_bf16_bits(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    if ((x & 0x7f800000u) == 0x7f800000u && (x & 0x7fffffu))
        return (uint16_t)((x >> 16) | 0x40u);
    x += 0x7fffu + ((x >> 16) & 1u);
    return (uint16_t)(x >> 16);
}

}    // namespace

bool col_major_i32_to_row_major(const int32_t* src, const std::vector<int>& shape, tb200_dtype dtype, void* dst)
{
    bool fits = true;
    switch (dtype)
    {
        case TB200_INT8:
            for_each_row_major(shape, [&](int64_t rm, int64_t cm) {
                const int32_t v = src[cm];
                fits &= v >= -128 && v <= 127;
                static_cast<int8_t*>(dst)[rm] = (int8_t)v;
            });
            break;
        case TB200_UINT8:
            for_each_row_major(shape, [&](int64_t rm, int64_t cm) {
                const int32_t v = src[cm];
                fits &= v >= 0 && v <= 255;
                static_cast<uint8_t*>(dst)[rm] = (uint8_t)v;
            });
            break;
        case TB200_INT16:
            for_each_row_major(shape, [&](int64_t rm, int64_t cm) {
                const int32_t v = src[cm];
                fits &= v >= -32768 && v <= 32767;
                static_cast<int16_t*>(dst)[rm] = (int16_t)v;
            });
            break;
        case TB200_UINT16:
            for_each_row_major(shape, [&](int64_t rm, int64_t cm) {
                const int32_t v = src[cm];
                fits &= v >= 0 && v <= 65535;
                static_cast<uint16_t*>(dst)[rm] = (uint16_t)v;
            });
            break;
        default:
            for_each_row_major(shape, [&](int64_t rm, int64_t cm) { static_cast<int32_t*>(dst)[rm] = src[cm]; });
            break;
    }
    return fits;
}

void row_major_to_col_major_i32(const void* src, const std::vector<int>& shape, tb200_dtype dtype, int32_t* dst)
{
    switch (dtype)
    {
        case TB200_INT8:
            for_each_row_major(shape, [&](int64_t rm, int64_t cm) { dst[cm] = static_cast<const int8_t*>(src)[rm]; });
            break;
        case TB200_UINT8:
            for_each_row_major(shape, [&](int64_t rm, int64_t cm) { dst[cm] = static_cast<const uint8_t*>(src)[rm]; });
            break;
        case TB200_INT16:
            for_each_row_major(shape, [&](int64_t rm, int64_t cm) { dst[cm] = static_cast<const int16_t*>(src)[rm]; });
            break;
        case TB200_UINT16:
            for_each_row_major(shape, [&](int64_t rm, int64_t cm) { dst[cm] = static_cast<const uint16_t*>(src)[rm]; });
            break;
        default:
            for_each_row_major(shape, [&](int64_t rm, int64_t cm) { dst[cm] = static_cast<const int32_t*>(src)[rm]; });
            break;
    }
}

void col_major_f32_to_row_major(const float* src, const std::vector<int>& shape, tb200_dtype dtype, void* dst)
{
    if (dtype == TB200_FP16)
        for_each_row_major(shape, [&](int64_t rm, int64_t cm) { static_cast<uint16_t*>(dst)[rm] = f32_to_f16_bits(src[cm]); });
    else if (dtype == TB200_BF16)
        for_each_row_major(shape, [&](int64_t rm, int64_t cm) { static_cast<uint16_t*>(dst)[rm] = f32_to_bf16_bits(src[cm]); });
    else
        for_each_row_major(shape, [&](int64_t rm, int64_t cm) { static_cast<float*>(dst)[rm] = src[cm]; });
}

void row_major_to_col_major_f32(const void* src, const std::vector<int>& shape, tb200_dtype dtype, float* dst)
{
    if (dtype == TB200_FP16)
        for_each_row_major(shape, [&](int64_t rm, int64_t cm) { dst[cm] = f16_bits_to_f32(static_cast<const uint16_t*>(src)[rm]); });
    else if (dtype == TB200_BF16)
        for_each_row_major(shape, [&](int64_t rm, int64_t cm) {
            const uint32_t x = (uint32_t)static_cast<const uint16_t*>(src)[rm] << 16;
            memcpy(&dst[cm], &x, 4);
        });
    else
        for_each_row_major(shape, [&](int64_t rm, int64_t cm) { dst[cm] = static_cast<const float*>(src)[rm]; });
}

// ------------------------------------------------------------------------------------------------ table
Buffers::~Buffers()
{
    for (auto& kv : table_)
        if (kv.second.dev)
            tb200_tensor_free(ctx_, kv.second.dev);
}

Buffers::Entry* Buffers::ensure(const HostView& t, std::string* err)
{
    Entry& e = table_[t.key];
    if (!e.dev)
    {
        std::vector<int32_t> shape(t.shape.begin(), t.shape.end());
        if (tb200_tensor_alloc(ctx_, t.dtype, (int)shape.size(), shape.data(), &e.dev) != TB200_OK)
        {
            if (err)
                *err = tb200_last_error(ctx_);
            table_.erase(t.key);
            return nullptr;
        }
    }
    return &e;
}

tb200_tensor* Buffers::device(const HostView& t, std::string* err)
{
    Entry* e = ensure(t, err);
    if (!e)
        return nullptr;
    if (!e->dev_valid)
    {
        if (!t.host_data)
        {
            if (err)
                *err = "operand has neither a device nor a host value";
            return nullptr;
        }
        const size_t bytes = tb200_tensor_bytes(e->dev);
        staging_.resize(bytes);
        if (t.is_float_storage)
            col_major_f32_to_row_major(static_cast<const float*>(t.host_data), t.shape, t.dtype, staging_.data());
        else if (!col_major_i32_to_row_major(static_cast<const int32_t*>(t.host_data), t.shape, t.dtype, staging_.data()))
        {
            if (err)
                *err = "host tensor holds a value outside its TOSA type";
            return nullptr;
        }
        // the staging vector is reused by the next upload: wait for this copy (pageable memory, synchronous anyway)
        if (tb200_tensor_upload(ctx_, e->dev, staging_.data(), bytes) != TB200_OK || tb200_sync(ctx_) == TB200_INTERNAL)
        {
            if (err)
                *err = tb200_last_error(ctx_);
            return nullptr;
        }
        e->dev_valid = true;
        uploads++;
        bytes_up += bytes;
    }
    return e->dev;
}

tb200_tensor* Buffers::device_for_output(const HostView& t, std::string* err)
{
    Entry* e = ensure(t, err);
    return e ? e->dev : nullptr;
}

void Buffers::produced(const HostView& t)
{
    auto it = table_.find(t.key);
    if (it == table_.end())
        return;
    it->second.dev_valid  = true;
    it->second.host_valid = false;
}

tb200_status Buffers::host(const HostView& t, std::string* err)
{
    auto it = table_.find(t.key);
    if (it == table_.end() || it->second.host_valid)
        return TB200_OK;
    if (!t.host_data)
    {
        if (err)
            *err = "host container is not allocated";
        return TB200_ERROR;
    }
    const size_t bytes = tb200_tensor_bytes(it->second.dev);
    staging_.resize(bytes);
    const tb200_status st = tb200_tensor_download(ctx_, it->second.dev, staging_.data(), bytes);
    if (st == TB200_ERROR || st == TB200_INTERNAL)
    {
        if (err)
            *err = tb200_last_error(ctx_);
        return st;
    }
    if (t.is_float_storage)
        row_major_to_col_major_f32(staging_.data(), t.shape, t.dtype, static_cast<float*>(t.host_data));
    else
        row_major_to_col_major_i32(staging_.data(), t.shape, t.dtype, static_cast<int32_t*>(t.host_data));
    it->second.host_valid = true;
    downloads++;
    bytes_down += bytes;
    return st;    // TB200_OK or TB200_UNPREDICTABLE
}

void Buffers::host_written(const void* key)
{
    auto it = table_.find(key);
    if (it != table_.end())
    {
        it->second.host_valid = true;
        it->second.dev_valid  = false;
    }
}

void Buffers::release(const void* key)
{
    auto it = table_.find(key);
    if (it == table_.end())
        return;
    if (it->second.dev)
        tb200_tensor_free(ctx_, it->second.dev);
    table_.erase(it);
}

}    // namespace b200
