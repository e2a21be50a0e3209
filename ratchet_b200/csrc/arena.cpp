// Activation planner: which intermediate tensors of a resolved node list may share memory.
//
// Restates BufferAllocator::greedy_by_size (crates/ratchet-core/src/gpu/buffer_allocator/allocator.rs:209-271,
// after arXiv 2001.03288 "greedy by size"): every intermediate has a usage record {bytes, producer,
// last_consumer} in execution-order positions (allocator.rs:168-207); the records are visited from the largest
// to the smallest (tensor_usage_record.rs sorts by Reverse(size)); a record takes a shared object none of
// whose tenants is alive at the same time -- the LAST such object in creation order, as the reference's loop
// keeps overwriting `best_obj` -- and otherwise opens a new object of exactly its own size.  Two records are
// alive together when max(producers) <= min(last_consumers) (allocator.rs:226-228).
//
// The reference gives every shared object a buffer of its own from the pool; here the objects are laid end to
// end in ONE arena, each starting on an `alignment` boundary, so an executable makes one allocation.
// Records of equal size are visited in the order given (the reference's order among equals is that of a hash
// map, i.e. unspecified).  No CUDA in this file.
#include <algorithm>
#include <numeric>
#include <vector>

#include "arena.hpp"

namespace rt {

Status plan_arena(const rt_usage_record *rec, int32_t n, uint64_t alignment, ArenaPlan *out) {
    if (n < 0 || (n > 0 && !rec)) return Status::Err(RT_ERR_ARG, "rt_arena_plan: bad record list");
    if (alignment == 0 || (alignment & (alignment - 1)) != 0)
        return Status::Err(RT_ERR_ARG, "rt_arena_plan: alignment must be a power of two");
    for (int32_t i = 0; i < n; i++)
        if (rec[i].producer < 0 || rec[i].last_consumer < rec[i].producer)
            return Status::Err(RT_ERR_ARG, "rt_arena_plan: a record ends before it starts");
    std::vector<int32_t> order((size_t)n);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return rec[a].size > rec[b].size; });

    out->object.assign((size_t)n, -1);
    out->offset.assign((size_t)n, 0);
    out->object_bytes.clear();
    for (int32_t r : order) {
        int32_t best = -1;
        for (int32_t obj = 0; obj < (int32_t)out->object_bytes.size(); obj++) {
            bool suitable = true;
            for (int32_t o = 0; o < n && suitable; o++) {
                if (out->object[(size_t)o] != obj) continue;
                const int32_t max_first = std::max(rec[r].producer, rec[o].producer);
                const int32_t min_last = std::min(rec[r].last_consumer, rec[o].last_consumer);
                if (max_first <= min_last) suitable = false;
            }
            if (suitable) best = obj; // no break: the last suitable object wins
        }
        if (best < 0) {
            best = (int32_t)out->object_bytes.size();
            out->object_bytes.push_back(rec[r].size);
        }
        out->object[(size_t)r] = best;
    }
    std::vector<uint64_t> base(out->object_bytes.size());
    uint64_t at = 0;
    for (size_t o = 0; o < base.size(); o++) {
        base[o] = at;
        at += (out->object_bytes[o] + alignment - 1) & ~(alignment - 1);
    }
    out->arena_bytes = at;
    for (int32_t i = 0; i < n; i++) out->offset[(size_t)i] = base[(size_t)out->object[(size_t)i]];
    return Status::Ok();
}

} // namespace rt

extern "C" rt_status rt_arena_plan(const rt_usage_record *records, int32_t n, uint64_t alignment, int32_t *objects,
                                   uint64_t *offsets, int32_t *n_objects, uint64_t *arena_bytes) {
    rt::ArenaPlan plan;
    rt::Status st = rt::plan_arena(records, n, alignment, &plan);
    if (!st.ok()) return rt::fail(st);
    for (int32_t i = 0; i < n; i++) {
        if (objects) objects[i] = plan.object[(size_t)i];
        if (offsets) offsets[i] = plan.offset[(size_t)i];
    }
    if (n_objects) *n_objects = (int32_t)plan.object_bytes.size();
    if (arena_bytes) *arena_bytes = plan.arena_bytes;
    return RT_OK;
}
