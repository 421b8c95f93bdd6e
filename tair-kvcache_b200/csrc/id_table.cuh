// Dense ids for a set of 64-bit keys: every distinct key gets a number in [0, D) from an open-addressing table that
// lives in a caller's workspace.  Two passes, each a launch of its own: claim (every key finds or takes a slot, the
// thread that takes it draws the next id), then look up.  Used by the eviction-aware replays (per-configuration
// state as flat arrays indexed by id) and by the batched StartWriteCache (first request that names a key).
#pragma once
#include "kvcm_common.cuh"

namespace kvcm {
namespace {

struct IdTable {
    ulonglong2 *slots;         // {key, id}
    unsigned long long *cells;  // [0] = number of ids handed out, [1] = id of the key equal to kEmptyKey (or ~0)
    uint64_t mask;
};

// Pass 1: every key gets a slot; the thread that claims the slot takes the next id.
__device__ __forceinline__ void ClaimId(const IdTable &t, uint64_t key, uint32_t *status) {
    unsigned long long *words = reinterpret_cast<unsigned long long *>(t.slots);
    if (key == kEmptyKey) {
        if (atomicCAS(&t.cells[1], ~0ull, ~0ull - 1) == ~0ull) t.cells[1] = atomicAdd(&t.cells[0], 1ull);
        return;
    }
    uint64_t slot = Mix(key) & t.mask;
    bool placed = false;
    for (uint64_t probe = 0; probe <= t.mask; ++probe) {
        unsigned long long seen = *reinterpret_cast<volatile unsigned long long *>(&words[2 * slot]);
        if (seen == kEmptyKey) {
            seen = atomicCAS(&words[2 * slot], kEmptyKey, key);
            if (seen == kEmptyKey) {
                words[2 * slot + 1] = atomicAdd(&t.cells[0], 1ull);
                placed = true;
                break;
            }
        }
        if (seen == key) {
            placed = true;
            break;
        }
        slot = (slot + 1) & t.mask;
    }
    if (!placed && status != nullptr) atomicAdd(&status[0], 1u);
}

// Pass 2 (a launch of its own, so every id of pass 1 is visible): key -> id.
__device__ __forceinline__ uint32_t LookupId(const IdTable &t, uint64_t key) {
    if (key == kEmptyKey) return static_cast<uint32_t>(t.cells[1]);
    uint64_t slot = Mix(key) & t.mask;
    for (uint64_t probe = 0; probe <= t.mask; ++probe) {
        const ulonglong2 s = t.slots[slot];
        if (s.x == key) return static_cast<uint32_t>(s.y);
        if (s.x == kEmptyKey) break;  // not reached for a key that pass 1 placed
        slot = (slot + 1) & t.mask;
    }
    return 0u;
}

uint64_t SlotsFor(int64_t n_keys) {
    uint64_t n = 1024;
    while (n < 2ull * static_cast<uint64_t>(n_keys)) n <<= 1;
    return n;
}


}  // namespace
}  // namespace kvcm
