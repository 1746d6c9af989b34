// NumPy files straight into device tensors and back.
//
// Stands where the reference has Tensor::readFromNpyFile / Tensor::writeToNpyFile
// (reference_model/src/tensor.cpp:96-421, :423-640).  The reference reads every INT4/INT8/INT16/INT32 tensor from an
// int32 file into an int32 host buffer and then into an int32 Eigen tensor (:164-171, :288-299), and writes INT8 /
// INT16 outputs with their own width (:574-600).  Here the file's payload goes through one pinned host buffer to the
// device in chunks; int32 payloads of narrower tensors are narrowed on the device (values outside the tensor type's
// range are an error), so no widened copy of the tensor ever exists.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cuda_bf16.h>
#include <string>

#include "common.h"

using namespace tb200;

namespace
{

struct NpyHeader
{
    std::string descr;
    int rank = 0;
    int32_t shape[6] = { 1, 1, 1, 1, 1, 1 };
    uint64_t data_offset = 0;
    int64_t elements     = 1;
};

// Parses the header of format versions 1.0, 2.0 and 3.0: magic, version, little-endian header length, then a Python
// dict literal with the keys descr, fortran_order and shape.  Returns an empty string on success, else the reason.
std::string parse_npy_header(FILE* f, NpyHeader* h)
{
    unsigned char pre[12];
    if (fread(pre, 1, 10, f) != 10)
        return "file shorter than a NumPy header";
    if (memcmp(pre, "\x93NUMPY", 6) != 0)
        return "missing NumPy magic";
    const int major = pre[6];
    size_t hlen     = 0, pre_len = 10;
    if (major == 1)
        hlen = (size_t)pre[8] | ((size_t)pre[9] << 8);
    else if (major == 2 || major == 3)
    {
        if (fread(pre + 10, 1, 2, f) != 2)
            return "file shorter than a NumPy header";
        hlen    = (size_t)pre[8] | ((size_t)pre[9] << 8) | ((size_t)pre[10] << 16) | ((size_t)pre[11] << 24);
        pre_len = 12;
    }
    else
        return "unsupported NumPy format version";
    if (hlen == 0 || hlen > (1u << 20))
        return "implausible header length";
    std::string dict(hlen, '\0');
    if (fread(&dict[0], 1, hlen, f) != hlen)
        return "file shorter than its header length";
    h->data_offset = pre_len + hlen;

    auto value_of = [&](const char* key) -> size_t {
        std::string k = std::string("'") + key + "'";
        size_t p      = dict.find(k);
        if (p == std::string::npos)
            return std::string::npos;
        p = dict.find(':', p + k.size());
        if (p == std::string::npos)
            return std::string::npos;
        p++;
        while (p < dict.size() && dict[p] == ' ')
            p++;
        return p;
    };
    size_t p = value_of("descr");
    if (p == std::string::npos || p >= dict.size() || (dict[p] != '\'' && dict[p] != '"'))
        return "descr is missing or not a plain string (structured dtypes are not supported)";
    size_t q = dict.find(dict[p], p + 1);
    if (q == std::string::npos)
        return "unterminated descr";
    h->descr = dict.substr(p + 1, q - p - 1);
    p        = value_of("fortran_order");
    if (p == std::string::npos)
        return "fortran_order is missing";
    if (dict.compare(p, 5, "False") != 0)
        return "fortran_order must be False (tensors are row-major)";
    p = value_of("shape");
    if (p == std::string::npos || dict[p] != '(')
        return "shape is missing";
    q = dict.find(')', p);
    if (q == std::string::npos)
        return "unterminated shape";
    h->rank     = 0;
    h->elements = 1;
    size_t i    = p + 1;
    while (i < q)
    {
        while (i < q && (dict[i] == ' ' || dict[i] == ','))
            i++;
        if (i >= q)
            break;
        if (dict[i] < '0' || dict[i] > '9')
            return "shape holds something that is not a non-negative integer";
        int64_t v = 0;
        while (i < q && dict[i] >= '0' && dict[i] <= '9')
        {
            v = v * 10 + (dict[i] - '0');
            if (v > 2147483647LL)
                return "dimension exceeds 2^31-1";
            i++;
        }
        if (i < q && dict[i] == 'L')    // written by Python 2
            i++;
        if (h->rank == 6)
            return "rank above 6";
        h->shape[h->rank++] = (int32_t)v;
        h->elements *= v;
        if (h->elements > 2147483647LL)
            return "tensor exceeds 2^31-1 elements";
    }
    return "";
}

int descr_bytes(const std::string& d)
{
    if (d.size() < 3)
        return 0;
    if (d[0] == '>')
        return 0;    // big-endian payloads are not supported
    return atoi(d.c_str() + 2);
}

// how a file payload becomes a tensor of `dtype`: 0 = not accepted, 1 = same bits, 2 = int32 narrowed, 3 = fp32 -> bf16
int load_mode(tb200_dtype dtype, const std::string& d)
{
    const std::string k = d.size() >= 3 ? d.substr(1) : d;    // kind + width, byte-order mark dropped
    switch (dtype)
    {
        case TB200_INT8:   return k == "i4" ? 2 : k == "i1" ? 1 : 0;
        case TB200_INT16:  return k == "i4" ? 2 : k == "i2" ? 1 : 0;
        case TB200_INT32:  return k == "i4" ? 1 : 0;
        case TB200_UINT8:  return k == "i4" ? 2 : k == "u1" ? 1 : 0;
        case TB200_UINT16: return k == "i4" ? 2 : k == "u2" ? 1 : 0;
        case TB200_FP16:   return k == "f2" ? 1 : 0;
        case TB200_FP32:   return k == "f4" ? 1 : 0;
        case TB200_BF16:   return (k == "V2" || k == "u2" || k == "i2") ? 1 : k == "f4" ? 3 : 0;
        default:           return 0;
    }
}

const char* save_descr(tb200_dtype dtype)
{
    switch (dtype)
    {
        case TB200_INT8:   return "|i1";
        case TB200_INT16:  return "<i2";
        case TB200_INT32:  return "<i4";
        case TB200_UINT8:  return "|u1";
        case TB200_UINT16: return "<u2";
        case TB200_FP16:   return "<f2";
        case TB200_FP32:   return "<f4";
        case TB200_BF16:   return "<V2";
        default:           return nullptr;
    }
}

template <typename T>
__global__ void narrow_i32_kernel(const int32_t* __restrict__ in, T* __restrict__ out, int64_t n, int32_t lo, int32_t hi,
                                  int* __restrict__ out_of_range)
{
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    bool bad           = false;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step)
    {
        const int32_t v = in[i];
        bad |= (v < lo) || (v > hi);
        out[i] = (T)v;
    }
    if (bad)
        atomicOr(out_of_range, 1);
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, int64_t n)
{
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step)
        out[i] = __float2bfloat16_rn(in[i]);
}

const size_t kChunkBytes = (size_t)64 << 20;

tb200_status ensure_pinned(tb200_ctx* ctx)
{
    if (ctx->io_pinned)
        return TB200_OK;
    TB200_CUDA_CHECK(ctx, cudaMallocHost(&ctx->io_pinned, kChunkBytes));
    return TB200_OK;
}

}    // namespace

extern "C" tb200_status tb200_npy_probe(const char* path, char descr[8], int32_t* rank, int32_t shape[6],
                                        uint64_t* data_offset, char* err, size_t err_len)
{
    auto say = [&](const std::string& m) {
        if (err && err_len)
            snprintf(err, err_len, "%s", m.c_str());
        return TB200_ERROR;
    };
    if (!path)
        return say("null path");
    FILE* f = fopen(path, "rb");
    if (!f)
        return say(std::string("Cannot open file ") + path);
    NpyHeader h;
    const std::string why = parse_npy_header(f, &h);
    fclose(f);
    if (!why.empty())
        return say("Numpy header parsing error for file: " + std::string(path) + " (" + why + ")");
    if (descr)
        snprintf(descr, 8, "%s", h.descr.c_str());
    if (rank)
        *rank = h.rank;
    if (shape)
        for (int i = 0; i < 6; i++)
            shape[i] = h.shape[i];
    if (data_offset)
        *data_offset = h.data_offset;
    if (err && err_len)
        err[0] = '\0';
    return TB200_OK;
}

extern "C" tb200_status tb200_tensor_load_npy(tb200_ctx* ctx, const char* path, tb200_dtype dtype, tb200_tensor** out)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !path || !out, "readFromNpyFile: null argument");
    *out = nullptr;
    TB200_ERROR_IF(ctx, ctx->capturing, "readFromNpyFile: not allowed while capturing");
    FILE* f = fopen(path, "rb");
    TB200_ERROR_IF(ctx, !f, "readFromNpyFile: Cannot open file %s", path);
    NpyHeader h;
    const std::string why = parse_npy_header(f, &h);
    if (!why.empty())
    {
        fclose(f);
        return fail(ctx, TB200_ERROR, "Numpy header parsing error for file: %s (%s)", path, why.c_str());
    }
    const int mode = load_mode(dtype, h.descr);
    const int fes  = descr_bytes(h.descr);
    if (mode == 0 || fes == 0)
    {
        fclose(f);
        return fail(ctx, TB200_ERROR, "readFromNpyFile: Tensor type %d and Numpy file type '%s' mismatch for filename %s",
                    (int)dtype, h.descr.c_str(), path);
    }
    // the payload must be exactly elements * width bytes
    fseek(f, 0, SEEK_END);
    const long fsize = ftell(f);
    if (fsize < 0 || (uint64_t)fsize != h.data_offset + (uint64_t)h.elements * fes)
    {
        fclose(f);
        return fail(ctx, TB200_ERROR, "Buffer size does not match numpy file size for filename %s", path);
    }
    fseek(f, (long)h.data_offset, SEEK_SET);

    tb200_tensor* t = nullptr;
    tb200_status st = tb200_tensor_alloc(ctx, dtype, h.rank, h.shape, &t);
    if (st == TB200_OK)
        st = ensure_pinned(ctx);
    const size_t tes = dtype_size(dtype);
    if (st == TB200_OK && mode != 1)
        st = ensure_scratch(ctx, kChunkBytes + 256);
    int* flag        = nullptr;
    uint8_t* staging = nullptr;
    if (st == TB200_OK && mode != 1)
    {
        flag    = reinterpret_cast<int*>(ctx->scratch);
        staging = reinterpret_cast<uint8_t*>(ctx->scratch) + 256;
        if (cudaMemsetAsync(flag, 0, sizeof(int), ctx->stream) != cudaSuccess)
            st = fail(ctx, TB200_INTERNAL, "readFromNpyFile: cudaMemsetAsync failed");
    }
    const int64_t per_chunk = (int64_t)(kChunkBytes / fes);
    int launches            = 0;
    for (int64_t done = 0; st == TB200_OK && done < h.elements; done += per_chunk)
    {
        const int64_t n = std::min<int64_t>(per_chunk, h.elements - done);
        if (fread(ctx->io_pinned, fes, (size_t)n, f) != (size_t)n)
        {
            st = fail(ctx, TB200_ERROR, "readFromNpyFile: IO error reading file: %s", path);
            break;
        }
        uint8_t* dst = reinterpret_cast<uint8_t*>(t->data) + (size_t)done * tes;
        cudaError_t e = cudaMemcpyAsync(mode == 1 ? dst : staging, ctx->io_pinned, (size_t)n * fes, cudaMemcpyHostToDevice,
                                        ctx->stream);
        if (e == cudaSuccess && mode != 1)
        {
            const int block = 256;
            const int grid  = (int)std::min<int64_t>((n + block - 1) / block, (int64_t)ctx->num_sms * 16);
            const int32_t* src = reinterpret_cast<const int32_t*>(staging);
            if (mode == 3)
                f32_to_bf16_kernel<<<grid, block, 0, ctx->stream>>>(reinterpret_cast<const float*>(staging),
                                                                     reinterpret_cast<__nv_bfloat16*>(dst), n);
            else if (dtype == TB200_INT8)
                narrow_i32_kernel<int8_t><<<grid, block, 0, ctx->stream>>>(src, reinterpret_cast<int8_t*>(dst), n, -128, 127, flag);
            else if (dtype == TB200_UINT8)
                narrow_i32_kernel<uint8_t><<<grid, block, 0, ctx->stream>>>(src, dst, n, 0, 255, flag);
            else if (dtype == TB200_INT16)
                narrow_i32_kernel<int16_t><<<grid, block, 0, ctx->stream>>>(src, reinterpret_cast<int16_t*>(dst), n, -32768,
                                                                            32767, flag);
            else
                narrow_i32_kernel<uint16_t><<<grid, block, 0, ctx->stream>>>(src, reinterpret_cast<uint16_t*>(dst), n, 0, 65535,
                                                                             flag);
            launches++;
            e = cudaGetLastError();
        }
        // the pinned buffer is reused by the next chunk
        if (e == cudaSuccess)
            e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess)
            st = fail(ctx, TB200_INTERNAL, "readFromNpyFile: copy to the device failed: %s", cudaGetErrorString(e));
    }
    fclose(f);
    if (st == TB200_OK && launches > 0)
    {
        ctx->launches += (uint64_t)launches;
        ctx->last_kernel = "npy_narrow";
        int bad          = 0;
        if (cudaMemcpy(&bad, flag, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
            st = fail(ctx, TB200_INTERNAL, "readFromNpyFile: reading the range flag failed");
        else if (bad)
            st = fail(ctx, TB200_ERROR, "readFromNpyFile: a value of %s lies outside the range of tensor type %d", path,
                      (int)dtype);
    }
    if (st != TB200_OK)
    {
        if (t)
            tb200_tensor_free(ctx, t);
        return st;
    }
    *out = t;
    return TB200_OK;
}

extern "C" tb200_status tb200_tensor_save_npy(tb200_ctx* ctx, const tb200_tensor* t, const char* path)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !t || !path, "writeToNpyFile: null argument");
    TB200_ERROR_IF(ctx, ctx->capturing, "writeToNpyFile: not allowed while capturing");
    TB200_ERROR_IF(ctx, !t->contiguous, "writeToNpyFile: a view must be copied into a dense tensor first");
    const char* descr = save_descr(t->dtype);
    TB200_ERROR_IF(ctx, !descr, "writeToNpyFile: unknown tensor type=%d", (int)t->dtype);
    tb200_status st = ensure_pinned(ctx);
    if (st != TB200_OK)
        return st;
    std::string shape = "(";
    for (int i = 0; i < t->rank; i++)
        shape += std::to_string(t->shape[i]) + (t->rank == 1 || i + 1 < t->rank ? "," : "") + (i + 1 < t->rank ? " " : "");
    shape += ")";
    std::string dict = std::string("{'descr': '") + descr + "', 'fortran_order': False, 'shape': " + shape + ", }";
    // version 1.0: the 10-byte preamble plus the dict, padded with spaces and closed by a newline, is a multiple of 64
    const size_t unpadded = 10 + dict.size() + 1;
    dict.append((64 - unpadded % 64) % 64, ' ');
    dict.push_back('\n');
    FILE* f = fopen(path, "wb");
    TB200_ERROR_IF(ctx, !f, "writeToNpyFile: Cannot open file %s", path);
    const unsigned char pre[10] = { 0x93, 'N', 'U', 'M', 'P', 'Y', 1, 0, (unsigned char)(dict.size() & 255),
                                    (unsigned char)(dict.size() >> 8) };
    bool ok = fwrite(pre, 1, 10, f) == 10 && fwrite(dict.data(), 1, dict.size(), f) == dict.size();
    for (size_t done = 0; ok && st == TB200_OK && done < t->bytes; done += kChunkBytes)
    {
        const size_t n = std::min(kChunkBytes, t->bytes - done);
        cudaError_t e  = cudaMemcpyAsync(ctx->io_pinned, reinterpret_cast<const uint8_t*>(t->data) + done, n,
                                         cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess)
            e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess)
            st = fail(ctx, TB200_INTERNAL, "writeToNpyFile: copy from the device failed: %s", cudaGetErrorString(e));
        else
            ok = fwrite(ctx->io_pinned, 1, n, f) == n;
    }
    ok = (fclose(f) == 0) && ok;
    if (st != TB200_OK)
        return st;
    TB200_ERROR_IF(ctx, !ok, "writeToNpyFile: IO error writing file: %s", path);
    return TB200_OK;
}
