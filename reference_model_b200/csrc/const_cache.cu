// Cache of device blocks derived from constant operands (see Prepared in common.h).
//
// The reference decodes a graph's constants once, when the CONST nodes' outputs are allocated
// (reference_model/src/subgraph_traverser.cpp:617-781), and evaluates with them from then on.  The device path keeps
// the same split: what depends only on weights, biases, multipliers, shifts and zero points is computed at the first
// call that sees those operands and reused afterwards, so a steady-state CONV2D is one launch.
//
// Staleness is handled by address ranges.  Every entry records the device ranges it was derived from;
//   * an upload or file load into such a range rebuilds the entry at once, on the stream, behind the copy;
//   * an operator writing into such a range marks the entry unstable: it is rebuilt before every use from then on;
//   * freeing such a range drops the entry.
// Memory that the caller wrapped (tb200_tensor_wrap) and changes without going through the library is outside this
// bookkeeping; tb200_const_cache_control(ctx, TB200_CACHE_CLEAR) is the remedy there.
#include <algorithm>

#include "common.h"

namespace tb200
{

namespace
{
constexpr size_t kMaxEntries = 2048;

bool overlaps(const Prepared& e, const char* lo, size_t bytes)
{
    const char* hi = lo + bytes;
    for (const auto& r : e.operands)
        if (r.first < hi && lo < r.first + r.second)
            return true;
    return false;
}
}    // namespace

void release_block(tb200_ctx* ctx, void* block)
{
    if (!block)
        return;
    if (ctx->live_graphs > 0 || ctx->capturing)
    {
        ctx->retired.push_back(block);
        return;
    }
    // kernels queued on the stream may still read it
    cudaStreamSynchronize(ctx->stream);
    cudaFree(block);
}

Prepared* cache_find(tb200_ctx* ctx, const std::string& key)
{
    if (!ctx->const_cache_on)
        return nullptr;
    for (auto& e : ctx->prepared)
        if (e->key == key)
        {
            e->last_use = ++ctx->cache_clock;
            return e.get();
        }
    return nullptr;
}

Prepared* cache_insert(tb200_ctx* ctx, const std::string& key, std::vector<std::pair<const char*, size_t>> operands,
                       size_t bytes, std::function<tb200_status(tb200_ctx*, void*)> rebuild)
{
    if (!ctx->const_cache_on || ctx->capturing || bytes == 0)
        return nullptr;
    if (ctx->prepared.size() >= kMaxEntries)
    {
        // drop the entry that has gone unused the longest
        auto oldest = std::min_element(ctx->prepared.begin(), ctx->prepared.end(),
                                       [](const std::unique_ptr<Prepared>& a, const std::unique_ptr<Prepared>& b) {
                                           return a->last_use < b->last_use;
                                       });
        release_block(ctx, (*oldest)->block);
        ctx->prepared.erase(oldest);
    }
    void* block = nullptr;
    if (cudaMalloc(&block, bytes) != cudaSuccess)
    {
        cudaGetLastError();
        return nullptr;
    }
    std::unique_ptr<Prepared> e(new (std::nothrow) Prepared());
    if (!e)
    {
        cudaFree(block);
        return nullptr;
    }
    e->key      = key;
    e->operands = std::move(operands);
    e->block    = block;
    e->bytes    = bytes;
    e->rebuild  = std::move(rebuild);
    e->last_use = ++ctx->cache_clock;
    ctx->prepared.push_back(std::move(e));
    return ctx->prepared.back().get();
}

tb200_status cache_use(tb200_ctx* ctx, Prepared* e)
{
    if (e->valid && !e->unstable)
        return TB200_OK;
    const tb200_status st = e->rebuild(ctx, e->block);
    e->valid              = st == TB200_OK;
    e->host_flag          = -1;
    return st;
}

void cache_note_write(tb200_ctx* ctx, const void* ptr, size_t bytes)
{
    if (ctx->prepared.empty() || !ptr || bytes == 0)
        return;
    const char* lo = reinterpret_cast<const char*>(ptr);
    for (auto& e : ctx->prepared)
        if (!e->unstable && overlaps(*e, lo, bytes))
            e->unstable = true;
}

tb200_status cache_note_upload(tb200_ctx* ctx, const void* ptr, size_t bytes)
{
    if (ctx->prepared.empty() || !ptr || bytes == 0)
        return TB200_OK;
    const char* lo = reinterpret_cast<const char*>(ptr);
    for (auto& e : ctx->prepared)
        if (overlaps(*e, lo, bytes))
        {
            const tb200_status st = e->rebuild(ctx, e->block);
            e->valid              = st == TB200_OK;
            e->host_flag          = -1;
            if (st != TB200_OK)
                return st;
        }
    return TB200_OK;
}

void cache_note_free(tb200_ctx* ctx, const void* ptr, size_t bytes)
{
    if (ctx->prepared.empty() || !ptr || bytes == 0)
        return;
    const char* lo = reinterpret_cast<const char*>(ptr);
    for (size_t i = 0; i < ctx->prepared.size();)
    {
        if (overlaps(*ctx->prepared[i], lo, bytes))
        {
            release_block(ctx, ctx->prepared[i]->block);
            ctx->prepared.erase(ctx->prepared.begin() + (long)i);
        }
        else
            i++;
    }
}

void cache_clear(tb200_ctx* ctx)
{
    for (auto& e : ctx->prepared)
        release_block(ctx, e->block);
    ctx->prepared.clear();
}

}    // namespace tb200
