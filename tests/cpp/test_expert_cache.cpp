// Host-only check of the adapter's slot machine against the reference's LRU cases
// (src/domain/expert_cache.rs:141-283).  Built and run by tests/test_host_logic.py with g++.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../../ferrum-torrens_b200/csrc/expert_cache.hpp"

using ftm::ExpertCache;
using ftm::ExpertPlan;

static int failures = 0;
#define CHECK(cond)                                                      \
    do {                                                                 \
        if (!(cond)) {                                                   \
            std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond);   \
            failures++;                                                  \
        }                                                                \
    } while (0)

static ExpertPlan ens(ExpertCache& c, size_t layer, std::vector<uint32_t> r) {
    return c.ensure_experts(layer, r.data(), r.size());
}
template <typename T>
static bool eq(const std::vector<T>& a, std::vector<T> b) { return a == b; }

int main() {
    {   // fills_free_slots_first_lowest_slot
        ExpertCache c(2, 4, 8);
        auto p = ens(c, 0, {2, 0});
        CHECK(eq(p.misses, {0u, 2u}));
        CHECK(eq(p.write_slots, {0u, 1u}));
        CHECK(eq(p.rewrites, {1, 0}));
        CHECK(c.slot_of(0, 0) == 0 && c.slot_of(0, 2) == 1);
    }
    {   // hits_are_resident_and_noop
        ExpertCache c(1, 4, 8);
        ens(c, 0, {1, 3});
        auto p = ens(c, 0, {3, 1, 3});
        CHECK(p.misses.empty());
        CHECK(eq(p.rewrites, {c.slot_of(0, 3), c.slot_of(0, 1), c.slot_of(0, 3)}));
    }
    {   // full_cache_within_one_layer_never_misses
        ExpertCache c(1, 6, 6);
        CHECK(eq(ens(c, 0, {0, 1, 2, 3, 4, 5}).write_slots, {0u, 1u, 2u, 3u, 4u, 5u}));
        auto p = ens(c, 0, {5, 2, 0});
        CHECK(p.misses.empty());
        CHECK(eq(p.rewrites, {5, 2, 0}));
    }
    {   // lru_victim_is_the_coldest_slot
        ExpertCache c(1, 8, 6);
        ens(c, 0, {0, 1, 2, 3, 4, 5});
        ens(c, 0, {5, 0});
        auto p = ens(c, 0, {6});
        CHECK(eq(p.misses, {6u}));
        CHECK(eq(p.write_slots, {1u}));
        CHECK(c.slot_of(0, 1) == -1 && c.slot_of(0, 5) == 5);
    }
    {   // same_step_hits_not_evicted_while_colder_guests_are
        ExpertCache c(1, 8, 6);
        ens(c, 0, {0, 1, 2, 3, 4, 5});
        ens(c, 0, {0, 1});
        CHECK(eq(ens(c, 0, {6, 7}).write_slots, {2u, 3u}));
        CHECK(c.slot_of(0, 0) == 0 && c.slot_of(0, 1) == 1 && c.slot_of(0, 2) == -1);
    }
    {   // layer_id_space_is_flat + residency_is_cross_layer
        ExpertCache c(2, 4, 8);
        ens(c, 0, {0});
        ens(c, 1, {0, 0});
        CHECK(c.slot_of(0, 0) != -1 && c.slot_of(1, 0) != -1 && c.slot_of(0, 0) != c.slot_of(1, 0));
        ExpertCache d(3, 4, 4);
        ens(d, 0, {1, 3});
        ens(d, 1, {0, 2});
        CHECK(ens(d, 0, {1, 3}).misses.empty());
        CHECK(eq(ens(d, 2, {0}).misses, {0u}));
        CHECK(d.slot_of(2, 0) >= 0);
    }
    {   // duplicate_routed_ids_do_not_multiply + cache_smaller_than_experts_still_deterministic
        ExpertCache c(1, 4, 8);
        auto p = ens(c, 0, {2, 2, 2});
        CHECK(eq(p.misses, {2u}));
        CHECK(eq(p.rewrites, {c.slot_of(0, 2), c.slot_of(0, 2), c.slot_of(0, 2)}));
        ExpertCache d(1, 6, 3);
        auto q = ens(d, 0, {5, 4, 3, 2});
        CHECK(eq(q.misses, {2u, 3u, 4u, 5u}));
        CHECK(eq(q.write_slots, {0u, 1u, 2u, 0u}));
        CHECK(eq(q.rewrites, {d.slot_of(0, 5), d.slot_of(0, 4), d.slot_of(0, 3), d.slot_of(0, 2)}));
        CHECK(d.slot_of(0, 2) == -1);
    }
    std::printf(failures ? "FAILED %d\n" : "OK\n", failures);
    return failures ? 1 : 0;
}
