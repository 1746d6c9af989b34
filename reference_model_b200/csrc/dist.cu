// Multi-GPU plumbing behind the C ABI: one context per process and GPU, the batch dimension split over the ranks
// (no operator of this path reduces over it: reference_model/src/ops/tensor_ops.cpp:828, :1283, :1454-1483), and one
// exchange at the end, the gather of the output shards.  NCCL is resolved at run time (the library that is already in
// the process, else libnccl.so.2 from the loader path), so libtb200 has no link-time dependency on it and hosts that
// never gather need no NCCL at all.
#include <dlfcn.h>
#include <mutex>

#include "common.h"

namespace
{

// the slice of NCCL's C ABI this file uses (stable since NCCL 2.x)
typedef struct
{
    char internal[128];
} nccl_unique_id;
typedef int (*fn_get_unique_id)(nccl_unique_id*);
typedef int (*fn_comm_init_rank)(void** comm, int nranks, nccl_unique_id id, int rank);
typedef int (*fn_comm_destroy)(void* comm);
typedef int (*fn_comm_count)(void* comm, int* count);
typedef int (*fn_comm_user_rank)(void* comm, int* rank);
typedef int (*fn_all_gather)(const void* send, void* recv, size_t count, int datatype, void* comm, cudaStream_t stream);
typedef const char* (*fn_get_error_string)(int);

struct NcclApi
{
    void* handle                     = nullptr;
    fn_get_unique_id get_unique_id   = nullptr;
    fn_comm_init_rank comm_init_rank = nullptr;
    fn_comm_destroy comm_destroy     = nullptr;
    fn_comm_count comm_count         = nullptr;
    fn_comm_user_rank comm_user_rank = nullptr;
    fn_all_gather all_gather         = nullptr;
    fn_get_error_string error_string = nullptr;
    bool ok                          = false;
};

NcclApi& nccl_api()
{
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        // a copy that the process already holds (e.g. the one a framework brought along) comes first
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
        if (!h)
            h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (!h)
            h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
        if (!h)
            return;
        api.handle         = h;
        api.get_unique_id  = reinterpret_cast<fn_get_unique_id>(dlsym(h, "ncclGetUniqueId"));
        api.comm_init_rank = reinterpret_cast<fn_comm_init_rank>(dlsym(h, "ncclCommInitRank"));
        api.comm_destroy   = reinterpret_cast<fn_comm_destroy>(dlsym(h, "ncclCommDestroy"));
        api.comm_count     = reinterpret_cast<fn_comm_count>(dlsym(h, "ncclCommCount"));
        api.comm_user_rank = reinterpret_cast<fn_comm_user_rank>(dlsym(h, "ncclCommUserRank"));
        api.all_gather     = reinterpret_cast<fn_all_gather>(dlsym(h, "ncclAllGather"));
        api.error_string   = reinterpret_cast<fn_get_error_string>(dlsym(h, "ncclGetErrorString"));
        api.ok = api.get_unique_id && api.comm_init_rank && api.comm_destroy && api.comm_count && api.comm_user_rank &&
                 api.all_gather;
    });
    return api;
}

const char* nccl_err(const NcclApi& api, int code)
{
    return api.error_string ? api.error_string(code) : "NCCL error";
}

}    // namespace

using namespace tb200;

extern "C" tb200_status tb200_comm_unique_id(char id_out[TB200_COMM_ID_BYTES])
{
    if (!id_out)
        return TB200_ERROR;
    NcclApi& api = nccl_api();
    if (!api.ok)
        return TB200_INTERNAL;
    nccl_unique_id id;
    if (api.get_unique_id(&id) != 0)
        return TB200_INTERNAL;
    static_assert(sizeof(id) == TB200_COMM_ID_BYTES, "NCCL unique id size");
    memcpy(id_out, &id, sizeof(id));
    return TB200_OK;
}

extern "C" tb200_status tb200_comm_init(tb200_ctx* ctx, const char id[TB200_COMM_ID_BYTES], int32_t rank, int32_t nranks)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !id || nranks < 1 || rank < 0 || rank >= nranks, "tb200_comm_init: bad rank %d of %d", (int)rank, (int)nranks);
    TB200_ERROR_IF(ctx, ctx->comm != nullptr, "tb200_comm_init: the context already has a communicator");
    NcclApi& api = nccl_api();
    if (!api.ok)
        return fail(ctx, TB200_INTERNAL, "NCCL is not available in this process (libnccl.so.2 could not be loaded)");
    TB200_CUDA_CHECK(ctx, cudaSetDevice(ctx->device));
    nccl_unique_id uid;
    memcpy(&uid, id, sizeof(uid));
    void* comm  = nullptr;
    const int r = api.comm_init_rank(&comm, (int)nranks, uid, (int)rank);
    if (r != 0 || !comm)
        return fail(ctx, TB200_INTERNAL, "ncclCommInitRank failed: %s", nccl_err(api, r));
    ctx->comm        = comm;
    ctx->comm_owned  = true;
    ctx->comm_rank   = rank;
    ctx->comm_nranks = nranks;
    return TB200_OK;
}

extern "C" tb200_status tb200_comm_attach(tb200_ctx* ctx, void* nccl_comm)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !nccl_comm, "tb200_comm_attach: null communicator");
    TB200_ERROR_IF(ctx, ctx->comm != nullptr, "tb200_comm_attach: the context already has a communicator");
    NcclApi& api = nccl_api();
    if (!api.ok)
        return fail(ctx, TB200_INTERNAL, "NCCL is not available in this process (libnccl.so.2 could not be loaded)");
    int n = 0, r = 0;
    if (api.comm_count(nccl_comm, &n) != 0 || api.comm_user_rank(nccl_comm, &r) != 0)
        return fail(ctx, TB200_INTERNAL, "tb200_comm_attach: the communicator does not answer");
    ctx->comm        = nccl_comm;
    ctx->comm_owned  = false;
    ctx->comm_rank   = r;
    ctx->comm_nranks = n;
    return TB200_OK;
}

extern "C" tb200_status tb200_comm_destroy(tb200_ctx* ctx)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    if (ctx->comm && ctx->comm_owned)
    {
        cudaStreamSynchronize(ctx->stream);
        nccl_api().comm_destroy(ctx->comm);
    }
    ctx->comm        = nullptr;
    ctx->comm_owned  = false;
    ctx->comm_rank   = 0;
    ctx->comm_nranks = 1;
    return TB200_OK;
}

extern "C" int32_t tb200_comm_rank(const tb200_ctx* ctx)
{
    return ctx ? ctx->comm_rank : 0;
}

extern "C" int32_t tb200_comm_size(const tb200_ctx* ctx)
{
    return ctx ? ctx->comm_nranks : 1;
}

// The shard's outermost dimension that is larger than one is the split one (the batch for NHWC tensors, the row block
// for the [1, N, classes] output of a final MATMUL); `gathered` has that dimension multiplied by the number of ranks
// and every other dimension equal.  Shards land in rank order, so `gathered` is the tensor a single GPU would have
// produced for the whole batch, provided the split dimension is the outermost non-unit one.
extern "C" tb200_status tb200_gather_output(tb200_ctx* ctx, const tb200_tensor* shard, tb200_tensor* gathered)
{
    if (!ctx)
        return TB200_ERROR;
    TB200_ENTER(ctx);
    TB200_ERROR_IF(ctx, !shard || !gathered, "tb200_gather_output: null tensor");
    TB200_ERROR_IF(ctx, !shard->contiguous || !gathered->contiguous, "tb200_gather_output: tensors must be contiguous");
    TB200_ERROR_IF(ctx, shard->dtype != gathered->dtype || shard->rank != gathered->rank,
                   "tb200_gather_output: shard and result differ in dtype or rank");
    const int nranks = ctx->comm ? ctx->comm_nranks : 1;
    int split        = 0;
    while (split < shard->rank - 1 && shard->shape[split] == 1 && gathered->shape[split] == 1)
        split++;
    for (int i = 0; i < shard->rank; i++)
    {
        const int64_t want = (int64_t)shard->shape[i] * (i == split ? nranks : 1);
        TB200_ERROR_IF(ctx, gathered->shape[i] != want, "tb200_gather_output: result dimension %d is %d, expected %lld", i,
                       gathered->shape[i], (long long)want);
    }
    if (shard->bytes == 0)
        return TB200_OK;
    cache_note_write(ctx, gathered->data, gathered->bytes);
    if (nranks == 1)
    {
        if (shard->data != gathered->data)
            TB200_CUDA_CHECK(ctx, cudaMemcpyAsync(gathered->data, shard->data, shard->bytes, cudaMemcpyDeviceToDevice, ctx->stream));
        return TB200_OK;
    }
    NcclApi& api = nccl_api();
    // ncclInt8 = 0: the exchange is byte-wise, whatever the element type
    const int r = api.all_gather(shard->data, gathered->data, shard->bytes, 0, ctx->comm, ctx->stream);
    if (r != 0)
        return fail(ctx, TB200_INTERNAL, "ncclAllGather failed: %s", nccl_err(api, r));
    ctx->last_kernel = "nccl_all_gather";
    return TB200_OK;
}
