// Host slot machine of the expert cache: which expert sits in which bank slot, and which
// slot a miss may overwrite.
//
// Mirrors `ExpertCache` of the reference (src/domain/expert_cache.rs:8-134): one flat id per
// (layer, expert), `slot_for_id` / `id_of_slot` maps, `usage[slot]` = last step that touched the
// slot, victims chosen as argmin (usage, slot).  It only plans; copying bytes is the caller's job.
#pragma once

#include <algorithm>
#include <cstdint>
#include <vector>

namespace ftm {

struct ExpertPlan {
    std::vector<uint32_t> misses;      // layer-local expert ids needing a copy, ascending
    std::vector<uint32_t> write_slots; // aligned with misses
    std::vector<int32_t> rewrites;     // aligned with the routed ids: slot or -1
};

class ExpertCache {
   public:
    ExpertCache(size_t layers, size_t experts, size_t cache_size)
        : layers_(layers), experts_(experts), cache_size_(cache_size),
          slot_for_id_(layers * experts, -1), id_of_slot_(cache_size, -1), usage_(cache_size, 0), step_(0) {}

    size_t num_layers() const { return layers_; }
    size_t num_experts() const { return experts_; }
    size_t cache_size() const { return cache_size_; }
    int32_t slot_of(size_t layer, uint32_t expert) const { return slot_for_id_[layer * experts_ + expert]; }

    void reset() {
        std::fill(slot_for_id_.begin(), slot_for_id_.end(), -1);
        std::fill(id_of_slot_.begin(), id_of_slot_.end(), -1);
        std::fill(usage_.begin(), usage_.end(), 0);
        step_ = 0;
    }

    ExpertPlan ensure_experts(size_t layer, const uint32_t* routed, size_t n) {
        const size_t base = layer * experts_;
        std::vector<uint32_t> seen;
        seen.reserve(n);
        for (size_t i = 0; i < n; i++)
            if (std::find(seen.begin(), seen.end(), routed[i]) == seen.end()) seen.push_back(routed[i]);
        const uint64_t step = ++step_;
        for (uint32_t e : seen) {
            int32_t s = slot_for_id_[base + e];
            if (s >= 0) usage_[s] = step;
        }
        ExpertPlan plan;
        for (uint32_t e : seen)
            if (slot_for_id_[base + e] < 0) plan.misses.push_back(e);
        std::sort(plan.misses.begin(), plan.misses.end());
        for (uint32_t e : plan.misses) {
            size_t victim = 0;
            for (size_t s = 1; s < cache_size_; s++)
                if (usage_[s] < usage_[victim]) victim = s;
            int32_t old = id_of_slot_[victim];
            if (old >= 0) slot_for_id_[old] = -1;
            id_of_slot_[victim] = (int32_t)(base + e);
            slot_for_id_[base + e] = (int32_t)victim;
            usage_[victim] = step;
            plan.write_slots.push_back((uint32_t)victim);
        }
        plan.rewrites.reserve(n);
        for (size_t i = 0; i < n; i++) plan.rewrites.push_back(slot_for_id_[base + routed[i]]);
        return plan;
    }

   private:
    size_t layers_, experts_, cache_size_;
    std::vector<int32_t> slot_for_id_, id_of_slot_;
    std::vector<uint64_t> usage_;
    uint64_t step_;
};

}  // namespace ftm
