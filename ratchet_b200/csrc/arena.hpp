// Result of the activation planner (arena.cpp).
#pragma once
#include <cstdint>
#include <vector>

#include "ratchet_b200.h"
#include "spec.hpp"

namespace rt {

struct ArenaPlan {
    std::vector<int32_t> object;        // per record: index of its shared object
    std::vector<uint64_t> offset;       // per record: byte offset of that object in the arena
    std::vector<uint64_t> object_bytes; // per shared object: its size (that of its first, largest tenant)
    uint64_t arena_bytes = 0;
};

Status plan_arena(const rt_usage_record *records, int32_t n, uint64_t alignment, ArenaPlan *out);

} // namespace rt
