// Resident expert cache for mixture-of-experts models larger than device memory: a bounded arena of expert-sized
// slots in HBM, least-recently-used eviction, misses streamed from the host through pinned staging memory.  Counterpart
// of ExpertCache (crates/ojas-cuda/src/expert_cache.rs:34-160); a slot is addressed by its byte offset in the arena,
// which is what the *_slots expert entries take (crates/ojas-cuda/src/kernels/moe.rs:127-178).  Two things differ from
// the reference because of this library's weight layout: the loader hands over an expert's GGUF blocks and the cache
// re-lays them into tiles on the device (the copy lands in a raw buffer, the repack kernel writes the slot), and the
// bookkeeping is a separate object (ExpertLru) so that it can be exercised without a GPU.
#include <algorithm>
#include <unordered_map>
#include <vector>

#include "common.cuh"

// ---- the policy: which slot serves which expert.  Pure host code.
struct ojas_b200_expert_lru {
    struct Slot { bool used = false; uint32_t id = 0; uint64_t tick = 0; };
    std::vector<Slot> slots;
    std::unordered_map<uint32_t, size_t> resident;
    uint64_t tick = 0;
    size_t hits = 0, misses = 0, evictions = 0;
};

extern "C" int ojas_b200_expert_lru_create(size_t slots, ojas_b200_expert_lru **out) {
    if (!out || slots == 0) return OJAS_B200_E_ARG;
    ojas_b200_expert_lru *l = new ojas_b200_expert_lru();
    l->slots.resize(slots);
    *out = l;
    return 0;
}

extern "C" void ojas_b200_expert_lru_destroy(ojas_b200_expert_lru *l) { delete l; }

// For every requested id (in order): the slot that serves it, and whether it has to be loaded (1) or is resident (0).
// A request for more DISTINCT experts than there are slots is refused (it would evict a slot the same request still
// needs) with OJAS_B200_E_LIMIT, and nothing changes.
extern "C" int ojas_b200_expert_lru_plan(ojas_b200_expert_lru *l, const uint32_t *ids, size_t n, uint32_t *slot_out, uint8_t *miss_out) {
    if (!l || (n && (!ids || !slot_out || !miss_out))) return OJAS_B200_E_ARG;
    std::vector<uint32_t> distinct(ids, ids + n);
    std::sort(distinct.begin(), distinct.end());
    distinct.erase(std::unique(distinct.begin(), distinct.end()), distinct.end());
    if (distinct.size() > l->slots.size()) return OJAS_B200_E_LIMIT;
    for (size_t i = 0; i < n; i++) {
        const uint32_t id = ids[i];
        l->tick++;
        auto it = l->resident.find(id);
        if (it != l->resident.end()) {
            l->slots[it->second].tick = l->tick;
            l->hits++;
            slot_out[i] = (uint32_t)it->second;
            miss_out[i] = 0;
            continue;
        }
        size_t slot = l->slots.size();
        for (size_t s = 0; s < l->slots.size(); s++)
            if (!l->slots[s].used) { slot = s; break; }
        if (slot == l->slots.size()) {            // no free slot: the least recently used (never one of this request: those were just ticked)
            uint64_t oldest = ~0ull;
            for (size_t s = 0; s < l->slots.size(); s++)
                if (l->slots[s].tick < oldest) { oldest = l->slots[s].tick; slot = s; }
            l->resident.erase(l->slots[slot].id);
            l->evictions++;
        }
        l->slots[slot].used = true;
        l->slots[slot].id = id;
        l->slots[slot].tick = l->tick;
        l->resident[id] = slot;
        l->misses++;
        slot_out[i] = (uint32_t)slot;
        miss_out[i] = 1;
    }
    return 0;
}

extern "C" void ojas_b200_expert_lru_stats(const ojas_b200_expert_lru *l, size_t out[3]) {
    if (!l || !out) return;
    out[0] = l->hits; out[1] = l->misses; out[2] = l->evictions;
}

// ---- the cache: arena + staging + the policy
struct ojas_b200_expert_cache {
    ojas_b200_ctx *ctx;
    uint32_t type;
    size_t N, K, raw_bytes, slot_bytes, n_slots;
    uint8_t *arena = nullptr;       // n_slots * slot_bytes, device
    uint8_t *raw_dev = nullptr;     // one expert's GGUF blocks, device
    uint8_t *staging = nullptr;     // the same, pinned host
    cudaEvent_t staged = nullptr;   // the upload out of `staging` has been queued and has finished
    ojas_b200_expert_lru *lru = nullptr;
    size_t bytes_streamed = 0;
};

extern "C" int ojas_b200_expert_cache_create(ojas_b200_ctx *ctx, uint32_t type, size_t N, size_t K, size_t budget_bytes,
                                             ojas_b200_expert_cache **out) {
    if (!ctx || !out) return OJAS_B200_E_ARG;
    *out = nullptr;
    if (!type_supported(type) || K == 0 || K % 256 != 0 || N == 0 || N % OJAS_TILE_ROWS != 0)
        return ojas_fail(ctx, OJAS_B200_E_ARG, "expert_cache: type %u, expert [%zu, %zu] (K a multiple of 256, N a multiple of 8)", type, N, K);
    ojas_b200_expert_cache *c = new ojas_b200_expert_cache();
    c->ctx = ctx; c->type = type; c->N = N; c->K = K;
    c->raw_bytes = ojas_b200_raw_bytes(type, N, K);
    c->slot_bytes = repacked_size(type, N, K);
    c->n_slots = budget_bytes / c->slot_bytes;
    if (c->n_slots == 0) c->n_slots = 1;              // at least one expert, as the reference does
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e == cudaSuccess) e = cudaMalloc((void **)&c->arena, c->n_slots * c->slot_bytes);
    if (e == cudaSuccess) e = cudaMalloc((void **)&c->raw_dev, c->raw_bytes);
    if (e == cudaSuccess) e = cudaHostAlloc((void **)&c->staging, c->raw_bytes, cudaHostAllocDefault);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->staged, cudaEventDisableTiming);
    if (e != cudaSuccess || ojas_b200_expert_lru_create(c->n_slots, &c->lru) != 0) {
        if (c->arena) cudaFree(c->arena);
        if (c->raw_dev) cudaFree(c->raw_dev);
        if (c->staging) cudaFreeHost(c->staging);
        if (c->staged) cudaEventDestroy(c->staged);
        delete c;
        return ojas_fail(ctx, OJAS_B200_E_CUDA, "expert_cache: allocating the arena (budget %zu bytes): %s", budget_bytes, cudaGetErrorString(e));
    }
    *out = c;
    return 0;
}

extern "C" void ojas_b200_expert_cache_destroy(ojas_b200_expert_cache *c) {
    if (!c) return;
    cudaSetDevice(c->ctx->device);
    cudaStreamSynchronize(c->ctx->stream);
    cudaFree(c->arena);
    cudaFree(c->raw_dev);
    cudaFreeHost(c->staging);
    cudaEventDestroy(c->staged);
    ojas_b200_expert_lru_destroy(c->lru);
    delete c;
}

extern "C" size_t ojas_b200_expert_cache_slots(const ojas_b200_expert_cache *c) { return c ? c->n_slots : 0; }
extern "C" size_t ojas_b200_expert_cache_slot_bytes(const ojas_b200_expert_cache *c) { return c ? c->slot_bytes : 0; }
extern "C" void *ojas_b200_expert_cache_arena(const ojas_b200_expert_cache *c) { return c ? (void *)c->arena : nullptr; }

// hits, misses, evictions, bytes streamed
extern "C" void ojas_b200_expert_cache_stats(const ojas_b200_expert_cache *c, size_t out[4]) {
    if (!c || !out) return;
    ojas_b200_expert_lru_stats(c->lru, out);
    out[3] = c->bytes_streamed;
}

// Makes every requested expert resident and writes each one's byte offset into the arena, in the order asked for.
// `load(user, id, dst, bytes)` fills dst with the expert's GGUF blocks (bytes = ojas_b200_raw_bytes(type, N, K)) and
// returns 0; it is where a caller reads from its model file.  Misses are copied and re-laid on the context's stream,
// so kernels queued after this call see them without further synchronisation; the call blocks only while the single
// staging buffer is still being read by the copy before.
extern "C" int ojas_b200_expert_cache_gather(ojas_b200_expert_cache *c, const uint32_t *ids, size_t n,
                                             int (*load)(void *user, uint32_t id, void *dst, size_t bytes), void *user, uint64_t *offsets_out) {
    if (!c) return OJAS_B200_E_ARG;
    if (n && (!ids || !offsets_out || !load)) return ojas_fail(c->ctx, OJAS_B200_E_ARG, "expert_cache: null pointer");
    std::vector<uint32_t> slot(n);
    std::vector<uint8_t> miss(n);
    int rc = ojas_b200_expert_lru_plan(c->lru, ids, n, slot.data(), miss.data());
    if (rc == OJAS_B200_E_LIMIT)
        return ojas_fail(c->ctx, OJAS_B200_E_LIMIT, "expert_cache: the request names more distinct experts than the arena's %zu slots; raise the budget", c->n_slots);
    if (rc) return rc;
    for (size_t i = 0; i < n; i++) {
        offsets_out[i] = (uint64_t)slot[i] * c->slot_bytes;
        if (!miss[i]) continue;
        OJAS_CUDA(c->ctx, cudaEventSynchronize(c->staged));          // the staging buffer is free again
        if (load(user, ids[i], c->staging, c->raw_bytes) != 0)
            return ojas_fail(c->ctx, OJAS_B200_E_ARG, "expert_cache: the loader failed for expert %u", ids[i]);
        OJAS_CUDA(c->ctx, cudaMemcpyAsync(c->raw_dev, c->staging, c->raw_bytes, cudaMemcpyHostToDevice, c->ctx->stream));
        OJAS_CUDA(c->ctx, cudaEventRecord(c->staged, c->ctx->stream));
        rc = ojas_b200_repack(c->ctx, c->type, c->raw_dev, c->N, c->K, c->arena + offsets_out[i]);
        if (rc) return rc;
        c->bytes_streamed += c->raw_bytes;
    }
    return 0;
}
