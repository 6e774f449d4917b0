// Expert-slot cache over an HBM-resident pool, filled from pinned host memory.
//
// Host-side counterpart of the reference's PreadExpertStreamer
// (Sources/Mference/Infrastructure/Streaming/PreadExpertStreamer.swift:57-580): the same planning rules - hits keep
// their slots, slots named by the caller as still in use are never handed out, victims are chosen least-frequently-
// used first with recency as the tie break (or purely by recency), a plan that cannot place its misses is refused -
// and the same expert -> slot table (Int16, -1 = not resident) that the FFN kernels read on the device.  What was
// a pread() from SSD into a wired slab is here one cudaMemcpyAsync per missing expert from pinned host memory into
// the slab in HBM; table updates travel on the same stream, so kernels enqueued after a publish see the new slots
// and kernels enqueued before a fill still see the old ones.
#include <algorithm>
#include <mutex>
#include <vector>

#include "common.cuh"

struct mfb_pool {
    uint32_t num_experts = 0, slot_count = 0, policy = 0, flags = 0;
    uint64_t slot_bytes = 0, slot_stride = 0;
    uint8_t* slab = nullptr;          // device, slot_count * slot_stride
    int16_t* slot_of_dev = nullptr;   // device, [num_experts]
    // bookkeeping (PreadExpertStreamer.swift:84-93)
    std::vector<int32_t> slot_expert;       // published expert of each slot, -1 = none / being filled
    std::vector<uint64_t> slot_last_use;
    std::vector<uint64_t> expert_use_count;
    std::vector<int16_t> slot_of_host;      // mirror of the device table
    std::vector<char> in_flight;            // slot is being filled by a speculative or eager read: never a victim
    uint64_t use_clock = 0;
    // pinned snapshots of the table for stream-ordered uploads
    static constexpr int RING = 32;
    int16_t* ring = nullptr;                // pinned, RING * num_experts
    cudaEvent_t ring_done[RING] = {};
    int ring_next = 0;
    std::mutex lock;
};

namespace mfb {
namespace {

// shouldEvictSlot (PreadExpertStreamer.swift:518-531): true when slot a goes before slot b.
bool evict_before(const mfb_pool& p, uint32_t a, uint32_t b) {
    if (p.policy == MFB_POOL_LRU) return p.slot_last_use[a] < p.slot_last_use[b];
    const int32_t ea = p.slot_expert[a], eb = p.slot_expert[b];
    if (ea < 0 || eb < 0) return ea < eb;   // empty slots first
    const uint64_t ca = p.expert_use_count[ea], cb = p.expert_use_count[eb];
    if (ca != cb) return ca < cb;
    return p.slot_last_use[a] < p.slot_last_use[b];
}

void set_slot_expert(mfb_pool& p, uint32_t slot, int32_t expert) {
    const int32_t old = p.slot_expert[slot];
    if (old >= 0 && (uint32_t)old < p.num_experts && p.slot_of_host[old] == (int16_t)slot) p.slot_of_host[old] = -1;
    p.slot_expert[slot] = expert;
    if (expert >= 0 && (uint32_t)expert < p.num_experts) p.slot_of_host[expert] = (int16_t)slot;
}

// Uploads the current table on the stream from a pinned snapshot (so later host-side changes cannot reach it).
int32_t upload_table(mfb_pool& p, cudaStream_t s) {
    if (p.flags & MFB_POOL_HOST_ONLY) return MFB_OK;
    const int slot = p.ring_next;
    p.ring_next = (p.ring_next + 1) % mfb_pool::RING;
    MFB_CUDA(cudaEventSynchronize(p.ring_done[slot]));   // the copy that last used this snapshot has run
    int16_t* snap = p.ring + (size_t)slot * p.num_experts;
    std::copy(p.slot_of_host.begin(), p.slot_of_host.end(), snap);
    MFB_CUDA(cudaMemcpyAsync(p.slot_of_dev, snap, p.num_experts * sizeof(int16_t), cudaMemcpyHostToDevice, s));
    MFB_CUDA(cudaEventRecord(p.ring_done[slot], s));
    return MFB_OK;
}

}  // namespace
}  // namespace mfb

using namespace mfb;

extern "C" int32_t mfb_pool_create(uint32_t num_experts, uint64_t slot_bytes, uint32_t slot_count, uint32_t policy,
                                   uint32_t flags, mfb_pool** out) {
    MFB_REQUIRE(out, MFB_ERR_INVALID_ARGUMENT, "pool_create: NULL argument");
    *out = nullptr;
    MFB_REQUIRE(num_experts >= 1 && num_experts <= MFB_MAX_EXPERTS, MFB_ERR_UNSUPPORTED_SHAPE, "pool_create: num_experts must be in 1..%d", MFB_MAX_EXPERTS);
    MFB_REQUIRE(slot_count >= 1 && slot_count <= 32767, MFB_ERR_INVALID_ARGUMENT, "pool_create: slot_count must be in 1..32767");
    MFB_REQUIRE(slot_bytes >= 1 && policy <= MFB_POOL_LRU, MFB_ERR_INVALID_ARGUMENT, "pool_create: slot_bytes / policy");
    mfb_pool* p = new mfb_pool();
    p->num_experts = num_experts; p->slot_count = slot_count; p->policy = policy; p->flags = flags;
    p->slot_bytes = slot_bytes;
    p->slot_stride = (slot_bytes + 255) & ~(uint64_t)255;
    p->slot_expert.assign(slot_count, -1);
    p->slot_last_use.assign(slot_count, 0);
    p->expert_use_count.assign(num_experts, 0);
    p->slot_of_host.assign(num_experts, (int16_t)-1);
    p->in_flight.assign(slot_count, 0);
    if (!(flags & MFB_POOL_HOST_ONLY)) {
        cudaError_t e = cudaMalloc(&p->slab, p->slot_stride * slot_count);
        if (e == cudaSuccess) e = cudaMalloc(&p->slot_of_dev, num_experts * sizeof(int16_t));
        if (e == cudaSuccess) e = cudaMemset(p->slot_of_dev, 0xFF, num_experts * sizeof(int16_t));
        if (e == cudaSuccess) e = cudaMallocHost(&p->ring, (size_t)mfb_pool::RING * num_experts * sizeof(int16_t));
        for (int i = 0; i < mfb_pool::RING && e == cudaSuccess; ++i) e = cudaEventCreateWithFlags(&p->ring_done[i], cudaEventDisableTiming);
        if (e != cudaSuccess) {
            set_error("pool_create: %s", cudaGetErrorString(e));
            mfb_pool_destroy(p);
            return e == cudaErrorMemoryAllocation ? MFB_ERR_ALLOC : MFB_ERR_CUDA;
        }
    }
    *out = p;
    return MFB_OK;
}

extern "C" int32_t mfb_pool_destroy(mfb_pool* p) {
    if (!p) return MFB_OK;
    for (int i = 0; i < mfb_pool::RING; ++i)
        if (p->ring_done[i]) cudaEventDestroy(p->ring_done[i]);
    if (p->ring) cudaFreeHost(p->ring);
    cudaFree(p->slot_of_dev);
    cudaFree(p->slab);
    delete p;
    return MFB_OK;
}

extern "C" int32_t mfb_pool_info(const mfb_pool* p, void** slab, uint64_t* slot_stride, const int16_t** slot_of_device) {
    MFB_REQUIRE(p, MFB_ERR_INVALID_ARGUMENT, "pool_info: NULL pool");
    if (slab) *slab = p->slab;
    if (slot_stride) *slot_stride = p->slot_stride;
    if (slot_of_device) *slot_of_device = p->slot_of_dev;
    return MFB_OK;
}

extern "C" int32_t mfb_pool_plan(mfb_pool* p, const int32_t* experts, uint32_t n, const int32_t* avoid_slots, uint32_t n_avoid,
                                 int32_t* out_slots, uint8_t* out_miss, uint32_t* out_hits) {
    MFB_REQUIRE(p && (experts || n == 0) && (out_slots || n == 0) && (out_miss || n == 0), MFB_ERR_INVALID_ARGUMENT, "pool_plan: NULL argument");
    MFB_REQUIRE(n <= p->slot_count, MFB_ERR_INVALID_ARGUMENT, "pool_plan: %u experts need at least as many slots (%u)", n, p->slot_count);
    std::lock_guard<std::mutex> g(p->lock);
    std::vector<char> reserved(p->slot_count, 0);
    // hits first, in request order (PreadExpertStreamer.swift:223-230)
    for (uint32_t i = 0; i < n; ++i) {
        out_slots[i] = -1;
        for (uint32_t s = 0; s < p->slot_count; ++s)
            if (!reserved[s] && p->slot_expert[s] == experts[i] && experts[i] >= 0) { out_slots[i] = (int32_t)s; reserved[s] = 1; break; }
    }
    for (uint32_t i = 0; i < n_avoid; ++i)
        if (avoid_slots[i] >= 0 && (uint32_t)avoid_slots[i] < p->slot_count) reserved[avoid_slots[i]] = 1;
    for (uint32_t s = 0; s < p->slot_count; ++s)   // slots a speculative or eager read is filling (PreadExpertStreamer.swift:231-236)
        if (p->in_flight[s]) reserved[s] = 1;
    std::vector<uint32_t> evictable;
    for (uint32_t s = 0; s < p->slot_count; ++s)
        if (!reserved[s]) evictable.push_back(s);
    std::stable_sort(evictable.begin(), evictable.end(), [&](uint32_t a, uint32_t b) { return evict_before(*p, a, b); });
    uint32_t misses = 0;
    for (uint32_t i = 0; i < n; ++i) misses += out_slots[i] < 0 ? 1u : 0u;
    if (misses > evictable.size()) {
        set_error("pool_plan: %u misses cannot be placed in %zu free slots", misses, evictable.size());
        return MFB_ERR_NO_SLOT;   // planExpertsCachedIfPossible == nil
    }
    const uint64_t clock = ++p->use_clock;
    for (uint32_t i = 0; i < n; ++i)
        if (experts[i] >= 0 && (uint32_t)experts[i] < p->num_experts) ++p->expert_use_count[experts[i]];
    uint32_t next = 0, hits = 0;
    for (uint32_t i = 0; i < n; ++i) {
        out_miss[i] = out_slots[i] < 0;
        if (out_slots[i] >= 0) { p->slot_last_use[out_slots[i]] = clock; ++hits; continue; }
        const uint32_t s = evictable[next++];
        out_slots[i] = (int32_t)s;
        set_slot_expert(*p, s, -1);   // its content is undefined until the fill is published
        p->slot_last_use[s] = clock;
    }
    if (out_hits) *out_hits = hits;
    return MFB_OK;
}

extern "C" int32_t mfb_pool_fill_async(mfb_pool* p, void* stream, const int32_t* experts, const int32_t* slots,
                                       const uint8_t* miss, uint32_t n, const void* const* host_blobs, uint64_t blob_bytes) {
    MFB_REQUIRE(p && experts && slots && miss && host_blobs, MFB_ERR_INVALID_ARGUMENT, "pool_fill: NULL argument");
    MFB_REQUIRE(!(p->flags & MFB_POOL_HOST_ONLY), MFB_ERR_INVALID_ARGUMENT, "pool_fill: the pool was created without device memory");
    MFB_REQUIRE(blob_bytes <= p->slot_bytes, MFB_ERR_IO, "pool_fill: blob of %llu bytes exceeds the slot size %llu",
                (unsigned long long)blob_bytes, (unsigned long long)p->slot_bytes);
    cudaStream_t s = (cudaStream_t)stream;
    {
        std::lock_guard<std::mutex> g(p->lock);
        const int32_t rc = upload_table(*p, s);   // victims read -1 on the device before their slots are overwritten
        if (rc) return rc;
    }
    for (uint32_t i = 0; i < n; ++i) {
        if (!miss[i]) continue;
        MFB_REQUIRE(slots[i] >= 0 && (uint32_t)slots[i] < p->slot_count, MFB_ERR_INVALID_ARGUMENT, "pool_fill: slot out of range");
        MFB_REQUIRE(host_blobs[i] != nullptr, MFB_ERR_IO, "pool_fill: no source for expert %d", experts[i]);
        MFB_CUDA(cudaMemcpyAsync(p->slab + (uint64_t)slots[i] * p->slot_stride, host_blobs[i], blob_bytes, cudaMemcpyHostToDevice, s));
    }
    return MFB_OK;
}

extern "C" int32_t mfb_pool_publish(mfb_pool* p, void* stream, const int32_t* experts, const int32_t* slots,
                                    const uint8_t* miss, uint32_t n) {
    MFB_REQUIRE(p && experts && slots && miss, MFB_ERR_INVALID_ARGUMENT, "pool_publish: NULL argument");
    for (uint32_t i = 0; i < n; ++i)   // validated before anything changes: the eviction order indexes per-expert counters by these ids
        MFB_REQUIRE(!miss[i] || (experts[i] >= 0 && (uint32_t)experts[i] < p->num_experts), MFB_ERR_INVALID_ARGUMENT,
                    "pool_publish: expert %d out of range", experts[i]);
    std::lock_guard<std::mutex> g(p->lock);
    for (uint32_t i = 0; i < n; ++i)
        if (miss[i] && slots[i] >= 0 && (uint32_t)slots[i] < p->slot_count) set_slot_expert(*p, (uint32_t)slots[i], experts[i]);
    return upload_table(*p, (cudaStream_t)stream);
}

extern "C" int32_t mfb_pool_reserve_speculative(mfb_pool* p, const int32_t* experts, uint32_t n, uint32_t keep_evictable,
                                               int32_t* out_experts, int32_t* out_slots, uint32_t* out_n) {
    MFB_REQUIRE(p && (experts || n == 0) && out_experts && out_slots && out_n, MFB_ERR_INVALID_ARGUMENT, "pool_reserve_speculative: NULL argument");
    *out_n = 0;
    if (n == 0) return MFB_OK;
    std::lock_guard<std::mutex> g(p->lock);
    std::vector<uint32_t> evictable;
    for (uint32_t s = 0; s < p->slot_count; ++s) {
        bool wanted = false;   // a slot that already holds one of the predicted experts is never a victim
        for (uint32_t i = 0; i < n && !wanted; ++i) wanted = p->slot_expert[s] >= 0 && p->slot_expert[s] == experts[i];
        if (!p->in_flight[s] && !wanted) evictable.push_back(s);
    }
    std::stable_sort(evictable.begin(), evictable.end(), [&](uint32_t a, uint32_t b) { return evict_before(*p, a, b); });
    const size_t room = evictable.size() > keep_evictable ? evictable.size() - keep_evictable : 0;
    const uint32_t budget = (uint32_t)std::min<size_t>(n, room);
    // no use counts and no clock are written: an unconfirmed guess must not shift the eviction policy
    for (uint32_t i = 0; i < budget; ++i) {
        const uint32_t s = evictable[i];
        p->in_flight[s] = 1;
        set_slot_expert(*p, s, -1);
        out_experts[i] = experts[i];
        out_slots[i] = (int32_t)s;
    }
    *out_n = budget;
    return MFB_OK;
}

extern "C" int32_t mfb_pool_mark_in_flight(mfb_pool* p, const int32_t* slots, uint32_t n) {
    MFB_REQUIRE(p && (slots || n == 0), MFB_ERR_INVALID_ARGUMENT, "pool_mark_in_flight: NULL argument");
    std::lock_guard<std::mutex> g(p->lock);
    for (uint32_t i = 0; i < n; ++i)
        if (slots[i] >= 0 && (uint32_t)slots[i] < p->slot_count) p->in_flight[slots[i]] = 1;
    return MFB_OK;
}

extern "C" int32_t mfb_pool_finish_speculative(mfb_pool* p, void* stream, const int32_t* experts, const int32_t* slots,
                                              const uint8_t* loaded, uint32_t n) {
    MFB_REQUIRE(p && (n == 0 || (experts && slots && loaded)), MFB_ERR_INVALID_ARGUMENT, "pool_finish_speculative: NULL argument");
    for (uint32_t i = 0; i < n; ++i)
        MFB_REQUIRE(!loaded[i] || (experts[i] >= 0 && (uint32_t)experts[i] < p->num_experts), MFB_ERR_INVALID_ARGUMENT,
                    "pool_finish_speculative: expert %d out of range", experts[i]);
    std::lock_guard<std::mutex> g(p->lock);
    for (uint32_t i = 0; i < n; ++i) {
        if (slots[i] < 0 || (uint32_t)slots[i] >= p->slot_count) continue;
        if (loaded[i]) set_slot_expert(*p, (uint32_t)slots[i], experts[i]);   // a failed read leaves its slot empty
        p->in_flight[slots[i]] = 0;                                            // the mark is always cleared
    }
    return upload_table(*p, (cudaStream_t)stream);
}

extern "C" int32_t mfb_pool_note_all_hit(mfb_pool* p, const int32_t* experts, uint32_t n) {
    MFB_REQUIRE(p && (experts || n == 0), MFB_ERR_INVALID_ARGUMENT, "pool_note_all_hit: NULL argument");
    std::lock_guard<std::mutex> g(p->lock);
    const uint64_t clock = ++p->use_clock;
    for (uint32_t i = 0; i < n; ++i) {
        if (experts[i] < 0 || (uint32_t)experts[i] >= p->num_experts) continue;
        ++p->expert_use_count[experts[i]];
        const int16_t s = p->slot_of_host[experts[i]];
        if (s >= 0) p->slot_last_use[s] = clock;
    }
    return MFB_OK;
}

extern "C" int32_t mfb_pool_slot_of_host(mfb_pool* p, int16_t* out) {
    MFB_REQUIRE(p && out, MFB_ERR_INVALID_ARGUMENT, "pool_slot_of_host: NULL argument");
    std::lock_guard<std::mutex> g(p->lock);
    std::copy(p->slot_of_host.begin(), p->slot_of_host.end(), out);
    return MFB_OK;
}
