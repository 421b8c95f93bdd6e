// GPU-resident block index and the batched matchers that probe it (sm_100a).
//
// The index is the device replica of MetaIndexer's key -> location-map table
// (kv_cache_manager/meta/meta_indexer.cc:419-440,650-752; kv_cache_manager/meta/meta_local_backend.cc:253-327)
// reduced to what the matchers read: one 64-bit summary word per key (see kvcm_b200.h).
// The matchers stand in for MetaSearcher::PrefixMatch, ReverseRollSlideWindowMatch,
// BatchGetBestLocation and BatchGetLocation (kv_cache_manager/manager/meta_searcher.cc:74-310).
//
// Layout in HBM: a power-of-two array of 16-byte slots {int64 key, uint64 value}, open
// addressing with linear probing at load factor <= 0.5, slot = fmix64(key) (chained block
// hashes are not uniformly mixed in their low bits).  A probe is one aligned 128-bit load; the
// expected chain is under two slots, so a lookup costs one or two 32-byte sectors.  Two key
// values are reserved as EMPTY and TOMBSTONE markers; real keys with those values live in two
// side cells, so every int64 stays a legal key.  All loops are bounded by the slot count.
//
// Beside the slots lies one TAG byte per slot: 0 = the slot was never used, 1 = tombstone,
// 2..255 = an 8-bit fingerprint of the key stored there.  Readers walk the tags and touch a slot
// only where the fingerprint matches.  Most probes of a match are misses that end at a never-used
// slot; with tags they end in a byte array sixteen times smaller than the table (32 MiB for 10 M
// keys), which stays in the 126 MB L2, instead of a random 32-byte sector of HBM per probe.
#include <cstring>

#include "id_table.cuh"
#include "kvcm_common.cuh"

struct kvcm_b200_index {
    void *base;         // one allocation: 256-byte header (the cells), the slots, then one tag byte per slot
    ulonglong2 *slots;
    uint8_t *tags;
    uint64_t *cells;    // [0],[1]: values of the two reserved keys; [2]: live keys; [3]: slots that are not EMPTY
    uint64_t n_slots;
    uint64_t max_live;
    int device;
    // Set by attach_peers: device array of the views of all shards of one logical index (this
    // one included), and the mappings opened from other processes.
    void *d_peer_views;
    uint32_t peer_count;
    void *opened[64];
    int n_opened;
    // Host-side upper bound of the tombstones made since the table was last rebuilt (keys passed to erase and to
    // the status transitions), and the bound at which the next upsert rebuilds the table first (0 = never).
    uint64_t tomb_debt;
    uint64_t auto_rehash_at;
    // Host-side upper bound of the slots in use (every key ever passed to upsert since the last clear; refreshed
    // to the true figure by kvcm_b200_index_usage).  While bound + batch stays under the limit an upsert launch
    // cannot overfill the table and runs without per-key seat atomics.
    uint64_t used_upper;
};

// Exchange area of one rank of a routed query: the inbox the other ranks store the keys this rank owns into,
// and the answer bytes the owners store back.  One allocation, exported to the peers like a shard.
struct kvcm_b200_route_area {
    void *base;
    int64_t *inbox;
    uint8_t *answers;
    uint64_t capacity;
    int device;
    void *d_peer_table;  // device copy of kvcm::RoutePeers, set by attach
    uint32_t peer_count;
    uint32_t self;
    void *opened[64];
    int n_opened;
};

namespace kvcm {
namespace {

constexpr uint64_t kTombKey = 0x8000000000000001ull;
constexpr int kMatchWarps = 8;
constexpr size_t kIndexHeaderBytes = 256;

struct IndexView {
    ulonglong2 *slots;
    uint8_t *tags;
    uint64_t *cells;
    uint64_t mask;
    uint64_t max_live;
    // Shards of the logical index this table is part of (peer GPUs' tables mapped into this
    // address space), indexed by owner; null / 0 when the table stands alone.
    const IndexView *peers;
    uint32_t peer_count;
};

constexpr uint8_t kTagEmpty = 0, kTagTomb = 1;
// Fingerprint 2..255 from the top byte of the mixed hash (the slot comes from its low bits).
__host__ __device__ __forceinline__ uint8_t TagOf(uint64_t mixed) {
    return static_cast<uint8_t>(2u + (static_cast<uint32_t>(mixed >> 56) * 254u >> 8));
}

// Hash-range sharding of one logical index over `shards` GPUs: a key belongs to the shard whose
// range of the mixed 64-bit hash contains it.  shards == 1 owns everything.
struct Shard {
    uint32_t count;
    uint32_t rank;
};
__device__ __forceinline__ bool Owns(const Shard &sh, uint64_t key) {
    return sh.count <= 1 || static_cast<uint32_t>(__umul64hi(Mix(key), sh.count)) == sh.rank;
}

__device__ __forceinline__ ulonglong2 LoadSlot(const ulonglong2 *p) {
    ulonglong2 s;
    asm volatile("ld.global.v2.u64 {%0,%1}, [%2];\n" : "=l"(s.x), "=l"(s.y) : "l"(p));
    return s;
}

__device__ __forceinline__ uint32_t OwnerOf(uint64_t key, uint32_t shards) {
    return static_cast<uint32_t>(__umul64hi(Mix(key), shards));
}

// Value word of a key in one table, 0 when absent (MetaIndexer::Get -> EC_NOENT).
// kExpectHit: the caller mostly asks for keys that are there (the leading keys of a prefix match), so
// the probes read the slots themselves and not the tags: one memory round trip per probe of a hit
// instead of two dependent ones, at the price of a sector of HBM when the key is absent.
template <bool kExpectHit>
__device__ __forceinline__ uint64_t LookupIn(const IndexView &t, uint64_t key) {
    if (key == kEmptyKey) return t.cells[0];
    if (key == kTombKey) return t.cells[1];
    const uint64_t mixed = Mix(key);
    const uint8_t tag = TagOf(mixed);
    uint64_t slot = mixed & t.mask;
    if (kExpectHit) {
        for (uint64_t probe = 0; probe <= t.mask; ++probe) {
            const ulonglong2 s = LoadSlot(t.slots + slot);  // the slot itself says whether it is the key, or empty
            if (s.x == key) return s.y;
            if (s.x == kEmptyKey) return 0;
            slot = (slot + 1) & t.mask;
        }
        return 0;
    }
    for (uint64_t probe = 0; probe <= t.mask; ++probe) {
        const uint8_t seen = t.tags[slot];
        if (seen == kTagEmpty) return 0;
        if (seen == tag) {
            const ulonglong2 s = LoadSlot(t.slots + slot);
            if (s.x == key) return s.y;
        }
        slot = (slot + 1) & t.mask;
    }
    return 0;
}

// Value word of a key.  With peers attached the probe goes to the owner shard's table, which may
// live in another GPU's memory: plain peer loads over NVLink, no collective.
template <bool kExpectHit = false>
__device__ __forceinline__ uint64_t Lookup(const IndexView &ix, uint64_t key) {
    if (ix.peer_count > 1) return LookupIn<kExpectHit>(ix.peers[OwnerOf(key, ix.peer_count)], key);
    return LookupIn<kExpectHit>(ix, key);
}

// A key is a hit for the matchers when some location is SERVING in a storage class whose
// policy weight is > 0 (kv_cache_manager/manager/select_location_policy.cc:8-27).
__device__ __forceinline__ bool Servable(uint64_t value, uint32_t avail_mask) {
    return (static_cast<uint32_t>(value) & avail_mask & 0xFFFFu) != 0;
}

__global__ void ClearKernel(IndexView ix) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i <= ix.mask; i += stride) {
        ix.slots[i] = make_ulonglong2(kEmptyKey, 0);
        ix.tags[i] = kTagEmpty;
    }
    if (blockIdx.x == 0 && threadIdx.x < 4) ix.cells[threadIdx.x] = 0;
}

__device__ __forceinline__ void AddCell(uint64_t *cell, int64_t delta) {
    atomicAdd(reinterpret_cast<unsigned long long *>(cell), static_cast<unsigned long long>(delta));
}

// Inserts or overwrites one key.  The probe runs to the end of the key's chain (the first EMPTY slot) and
// remembers the first tombstone it passes; a key that is not there goes into that tombstone, and only when
// the chain holds none into the EMPTY slot.  So a table under steady insert / erase churn reuses the slots
// of erased keys instead of lengthening its chains.  cells[3] counts the slots that are not EMPTY (live +
// tombstones) and an EMPTY slot is claimed only while that count is below `max_live`, which keeps EMPTY
// slots in the table (every miss ends at one) whatever the history.
// Several threads of one launch may insert the same new key: all of them walk the same chain, free slots
// only get fewer while the launch runs, and a thread whose claim fails looks at what took the slot - the
// key itself (then it only stores the value) or another key (then it walks the chain again).
// kCareful: the launch could push the slots in use past the bound, so every claim of an EMPTY slot takes a seat
// on the shared counter first.  Otherwise (the host knows that even if every key of the launch claimed one the bound
// holds) nothing is counted on the way: the caller sums `d_live` and `d_used` per warp and adds them once.
// What is done to the value word once the key's slot is known: `put(word)`.  Overwrite stores a whole word;
// MergeLocation (further down) adds one location to the word that is there.
struct Overwrite {
    uint64_t value;
    __device__ __forceinline__ void operator()(unsigned long long *word) const { atomicExch(word, value); }
};

template <bool kCareful, typename Put>
__device__ __forceinline__ bool UpsertOne(const IndexView &ix, uint64_t key, Put &put, int32_t *d_live,
                                          int32_t *d_used) {
    unsigned long long *words = reinterpret_cast<unsigned long long *>(ix.slots);
    const uint64_t mixed = Mix(key);
    const uint64_t home = mixed & ix.mask;
    // A seat (one count of cells[3]) is taken before an EMPTY slot is claimed, so that the table can never run
    // out of EMPTY slots, and it is kept while the claim is retried: a thread that lost a slot to another key
    // does not hand its seat back in between, or threads arriving at that moment would be refused although
    // there is room for them.
    bool seated = false;
    bool done = false, stored = false;
    for (int attempt = 0; attempt < 64 && !done; ++attempt) {
        uint64_t slot = home, tomb = ~0ull, empty = ~0ull;
        bool found = false;
        for (uint64_t probe = 0; probe <= ix.mask; ++probe) {
            const uint64_t seen = LoadSlot(ix.slots + slot).x;
            if (seen == key) {  // present already (or inserted by a duplicate of this key in the same batch)
                put(&words[2 * slot + 1]);
                found = true;
                break;
            }
            if (seen == kEmptyKey) {
                empty = slot;
                break;
            }
            if (seen == kTombKey && tomb == ~0ull) tomb = slot;
            slot = (slot + 1) & ix.mask;
        }
        if (found) {
            done = stored = true;
        } else if (tomb != ~0ull) {
            const uint64_t was = atomicCAS(&words[2 * tomb], kTombKey, key);
            if (was == kTombKey || was == key) {
                put(&words[2 * tomb + 1]);
                if (was == kTombKey) {
                    ix.tags[tomb] = TagOf(mixed);  // readers of later launches find the slot through its tag
                    *d_live += 1;
                }
                done = stored = true;
            }  // else another key took the tombstone: walk again
        } else if (empty == ~0ull) {
            done = true;  // no EMPTY slot on the whole table: cannot happen below the limit
        } else {
            if (kCareful && !seated) {
                const uint64_t used = atomicAdd(reinterpret_cast<unsigned long long *>(&ix.cells[3]), 1ull);
                if (used >= ix.max_live) {
                    AddCell(&ix.cells[3], -1);
                    return false;
                }
                seated = true;
            }
            const uint64_t was = atomicCAS(&words[2 * empty], kEmptyKey, key);
            if (was == kEmptyKey) {
                put(&words[2 * empty + 1]);
                ix.tags[empty] = TagOf(mixed);
                *d_live += 1;
                if (!kCareful) *d_used += 1;  // in careful mode the seat is this slot's count already
                return true;
            }
            if (was == key) {
                put(&words[2 * empty + 1]);
                done = stored = true;
            }  // else another key took the slot: walk again, seat kept
        }
    }
    if (seated) AddCell(&ix.cells[3], -1);  // ended without claiming an EMPTY slot
    return stored;
}

// One atomic per warp and counter instead of one per key: every lane of the warp gets here.
__device__ __forceinline__ void AddCellsPerWarp(const IndexView &ix, int32_t d_live, int32_t d_used) {
    const int32_t live = __reduce_add_sync(0xffffffffu, d_live);
    const int32_t used = __reduce_add_sync(0xffffffffu, d_used);
    if (LaneId() == 0) {
        if (live != 0) AddCell(&ix.cells[2], live);
        if (used != 0) AddCell(&ix.cells[3], used);
    }
}

template <bool kCareful>
__global__ void __launch_bounds__(256)
    UpsertKernel(IndexView ix, const int64_t *__restrict__ keys, const uint64_t *__restrict__ values,
                 uint64_t uniform_value, int64_t n, Shard shard, uint32_t *status) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    int32_t d_live = 0, d_used = 0;
    if (i < n) {
        const uint64_t key = static_cast<uint64_t>(keys[i]);
        if (Owns(shard, key)) {
            const uint64_t value = (values != nullptr ? values[i] : uniform_value) | KVCM_VAL_PRESENT;
            if (key == kEmptyKey || key == kTombKey) {
                const uint64_t old =
                    atomicExch(reinterpret_cast<unsigned long long *>(&ix.cells[key - kEmptyKey]), value);
                if (old == 0) d_live = 1;
            } else {
                Overwrite put{value};
                if (!UpsertOne<kCareful>(ix, key, put, &d_live, &d_used) && status != nullptr) {
                    atomicAdd(&status[0], 1u);
                }
            }
        }
    }
    AddCellsPerWarp(ix, d_live, d_used);
}

__device__ __forceinline__ uint64_t LoadKeyCoherent(const ulonglong2 *slot) {
    uint64_t k;
    asm volatile("ld.global.cg.u64 %0, [%1];\n" : "=l"(k) : "l"(slot));  // from L2: sees this launch's atomics
    return k;
}

// The slot of an erased key becomes a tombstone so that the probe chains through it stay whole.  A tombstone
// directly before an EMPTY slot holds no chain together (no key can lie beyond an EMPTY slot), so it is turned
// into an EMPTY slot at once, and so are the tombstones before it: the tail of a cluster is given back.  During
// an erase launch slots only move key -> tombstone -> EMPTY, so "the next slot is EMPTY" stays true once seen.
// The tag of a slot may be written by the thread that made it a tombstone and by the thread that freed it;
// whoever writes a tombstone tag looks at the slot again afterwards, so the tag ends up EMPTY when the slot did.
// Returns the number of slots it turned EMPTY (the caller takes them off the count of slots in use).
__device__ __forceinline__ int32_t ReleaseSlot(const IndexView &ix, uint64_t slot) {
    unsigned long long *words = reinterpret_cast<unsigned long long *>(ix.slots);
    atomicExch(&words[2 * slot + 1], 0ull);
    ix.tags[slot] = kTagTomb;
    if (LoadKeyCoherent(ix.slots + slot) == kEmptyKey) ix.tags[slot] = kTagEmpty;
    if (LoadKeyCoherent(ix.slots + ((slot + 1) & ix.mask)) != kEmptyKey) return 0;
    uint64_t p = slot;
    int32_t freed = 0;
    for (uint64_t n = 0; n <= ix.mask; ++n) {
        if (atomicCAS(&words[2 * p], kTombKey, kEmptyKey) != kTombKey) break;
        ix.tags[p] = kTagEmpty;
        ++freed;
        p = (p - 1) & ix.mask;
    }
    return freed;
}

__global__ void __launch_bounds__(256) EraseKernel(IndexView ix, const int64_t *__restrict__ keys, int64_t n) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    int32_t d_live = 0, d_used = 0;
    if (i < n) {
        const uint64_t key = static_cast<uint64_t>(keys[i]);
        if (key == kEmptyKey || key == kTombKey) {
            const uint64_t old = atomicExch(reinterpret_cast<unsigned long long *>(&ix.cells[key - kEmptyKey]), 0ull);
            if (old != 0) d_live = -1;
        } else {
            unsigned long long *words = reinterpret_cast<unsigned long long *>(ix.slots);
            uint64_t slot = Mix(key) & ix.mask;
            for (uint64_t probe = 0; probe <= ix.mask; ++probe) {
                const uint64_t seen = LoadSlot(ix.slots + slot).x;
                if (seen == kEmptyKey) break;
                if (seen == key) {
                    if (atomicCAS(&words[2 * slot], key, kTombKey) == key) {
                        d_live = -1;
                        d_used = -ReleaseSlot(ix, slot);
                    }
                    break;
                }
                slot = (slot + 1) & ix.mask;
            }
        }
    }
    AddCellsPerWarp(ix, d_live, d_used);
}

// ---- location-status transitions on the value word (MetaSearcher::BatchUpdateLocationStatus,
// BatchCASLocationStatus, BatchCADLocationStatus, BatchDeleteLocation:
// kv_cache_manager/manager/meta_searcher.cc:410-820 over BlockCacheLocationsMeta::UpdateLocationStatus /
// GetLocationStatus / DeleteLocation, kv_cache_manager/manager/cache_location.cc:60-82).
// The word keeps, for storage classes 0..7, the status of the key's location in that class as a 3-bit field
// (0 = no location of the class, else status + 1); a task names the class, so it plays the part of the
// reference's location id.  The summary bits the matchers read are recomputed from the field.
__device__ __forceinline__ uint32_t StatusField(uint64_t word, uint32_t cls) {
    return static_cast<uint32_t>(word >> (KVCM_VAL_STATUS_SHIFT + 3u * cls)) & 7u;
}

constexpr uint64_t kAllStatusFields = ((1ull << 24) - 1) << KVCM_VAL_STATUS_SHIFT;
constexpr uint64_t kLocationBits = 0xFFFFFFFFull | kAllStatusFields;  // anything that says "a location is here"

// The word after the task, or `word` unchanged with *code != KVCM_OK.  A returned 0 means that the last
// location went away: the key leaves the index (MetaIndexer::MA_DELETE, meta_searcher.cc:689-691,790-792).
__device__ __forceinline__ uint64_t ApplyStatusTask(uint64_t word, uint32_t task, int32_t *code) {
    const uint32_t cls = task & 0xFFu, expected = (task >> 8) & 0xFFu, next = (task >> 16) & 0xFFu;
    if (cls > 7 || (expected > 4 && expected != KVCM_STATUS_ANY) ||
        (next > 4 && next != KVCM_STATUS_DELETE && next != KVCM_STATUS_DELETE_KEEP_KEY)) {
        *code = KVCM_EC_BADARGS;
        return word;
    }
    if (word == 0 && next == KVCM_STATUS_DELETE_KEEP_KEY) {
        *code = KVCM_OK;  // BatchDeleteLocation skips a key that is not there (meta_searcher.cc:741-744)
        return 0;
    }
    const uint32_t field = word != 0 ? StatusField(word, cls) : 0;
    if (field == 0) {
        *code = KVCM_EC_NOENT;  // no such key, or no location of this class in its map
        // compare-and-delete drops a key whose map is empty whatever its tasks did (meta_searcher.cc:689-692): a key
        // that BatchDeleteLocation left behind empty goes here, and the task still answers EC_NOENT
        if (word != 0 && next == KVCM_STATUS_DELETE && (word & kLocationBits) == 0) return 0;
        return word;
    }
    if (expected != KVCM_STATUS_ANY && field - 1 != expected) {
        *code = KVCM_EC_MISMATCH;
        return word;
    }
    *code = KVCM_OK;
    uint64_t w = word & ~(7ull << (KVCM_VAL_STATUS_SHIFT + 3u * cls)) & ~KVCM_VAL_SERVING(cls) & ~KVCM_VAL_WRITABLE(cls);
    if (next == KVCM_STATUS_DELETE || next == KVCM_STATUS_DELETE_KEEP_KEY) {
        if ((w & kLocationBits) == 0) return next == KVCM_STATUS_DELETE ? 0 : KVCM_VAL_PRESENT;  // empty map
        return w;
    }
    w |= static_cast<uint64_t>(next + 1) << (KVCM_VAL_STATUS_SHIFT + 3u * cls);
    if (next == 3) w |= KVCM_VAL_SERVING(cls);   // CLS_SERVING
    if (next != 0) w |= KVCM_VAL_WRITABLE(cls);  // anything but CLS_NOT_FOUND
    return w | KVCM_VAL_NONEMPTY | KVCM_VAL_PRESENT;
}

// One task on one key: finds the key's word and runs the compare-and-swap loop; the result code of the task.
__device__ __forceinline__ int32_t RunStatusTask(const IndexView &ix, uint64_t key, uint32_t task) {
    unsigned long long *word_at = nullptr;
    uint64_t slot = 0;
    const bool in_cell = key == kEmptyKey || key == kTombKey;
    if (in_cell) {
        word_at = reinterpret_cast<unsigned long long *>(&ix.cells[key - kEmptyKey]);
    } else {
        slot = Mix(key) & ix.mask;
        for (uint64_t probe = 0; probe <= ix.mask; ++probe) {
            const uint64_t seen = LoadSlot(ix.slots + slot).x;
            if (seen == key) {
                word_at = reinterpret_cast<unsigned long long *>(ix.slots) + 2 * slot + 1;
                break;
            }
            if (seen == kEmptyKey) break;
            slot = (slot + 1) & ix.mask;
        }
    }
    int32_t code = KVCM_EC_NOENT;
    if (word_at == nullptr) {
        ApplyStatusTask(0, task, &code);  // the answer for a key that is not there
        return code;
    }
    // Tasks of one launch that name the same key take turns through the compare-and-swap.
    unsigned long long seen = *reinterpret_cast<volatile unsigned long long *>(word_at);
    for (int turn = 0; turn < 1024; ++turn) {
        const uint64_t next = ApplyStatusTask(seen, task, &code);
        if (next == seen) break;  // nothing to write: a refusal, or a task that leaves the word as it is
        const unsigned long long was = atomicCAS(word_at, seen, next);
        if (was == seen) {
            if (next == 0) {  // the key's last location is gone: the key goes too
                AddCell(&ix.cells[2], -1);
                if (!in_cell) {
                    unsigned long long *words = reinterpret_cast<unsigned long long *>(ix.slots);
                    if (atomicCAS(&words[2 * slot], key, kTombKey) == key) {
                        const int32_t freed = ReleaseSlot(ix, slot);
                        if (freed != 0) AddCell(&ix.cells[3], -freed);
                    }
                }
            }
            break;
        }
        seen = was;
        if (turn == 1023) code = KVCM_EC_ERROR;  // the turns ran out
    }
    return code;
}

__global__ void UpdateStatusKernel(IndexView ix, const int64_t *__restrict__ keys, const uint32_t *__restrict__ tasks,
                                   uint32_t uniform_task, int64_t n, Shard shard, int32_t *__restrict__ results) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t key = static_cast<uint64_t>(keys[i]);
    if (!Owns(shard, key)) return;  // the owner shard answers for this key
    results[i] = RunStatusTask(ix, key, tasks != nullptr ? tasks[i] : uniform_task);
}

// ---- a new location for a key (MetaSearcher::BatchAddLocation, kv_cache_manager/manager/meta_searcher.cc:312-408:
// read the key's location map or start an empty one, add the location in status CLS_WRITING, write the map back).
// Here: find the key's slot or claim one as an insert does, then merge the location of the task's class into the
// word that is there with a compare-and-swap, so that tasks of one launch on the same key take turns and the key's
// other locations stay.  The word keeps one status per class, so a class that holds a location already is refused
// with KVCM_EC_EXIST where the reference would add a second location under a fresh id.
struct MergeLocation {
    uint32_t cls, status;
    int32_t code;
    bool into_empty_word;  // the word was 0 when this location went in
    __device__ __forceinline__ void operator()(unsigned long long *word) {
        unsigned long long seen = *reinterpret_cast<volatile unsigned long long *>(word);
        code = KVCM_EC_ERROR;
        into_empty_word = false;
        for (int turn = 0; turn < 1024; ++turn) {
            if (seen != 0 && StatusField(seen, cls) != 0) {
                code = KVCM_EC_EXIST;
                return;
            }
            const unsigned long long next = seen | KVCM_VAL_PRESENT | KVCM_VAL_LOCATION(cls, status);
            const unsigned long long was = atomicCAS(word, seen, next);
            if (was == seen) {
                code = KVCM_OK;
                into_empty_word = seen == 0;
                return;
            }
            seen = was;
        }
    }
};

template <bool kCareful>
__global__ void __launch_bounds__(256)
    AddLocationKernel(IndexView ix, const int64_t *__restrict__ keys, const uint8_t *__restrict__ classes,
                      uint32_t uniform_class, uint32_t status_of_new, int64_t n, Shard shard,
                      int32_t *__restrict__ results, uint32_t *status) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    int32_t d_live = 0, d_used = 0;
    if (i < n) {
        const uint64_t key = static_cast<uint64_t>(keys[i]);
        if (Owns(shard, key)) {
            MergeLocation put{classes != nullptr ? classes[i] : uniform_class, status_of_new, KVCM_EC_ERROR, false};
            if (put.cls > 7) {
                put.code = KVCM_EC_BADARGS;
            } else if (key == kEmptyKey || key == kTombKey) {
                // the two reserved key values live in cells of the header; an empty cell is an absent key
                put(reinterpret_cast<unsigned long long *>(&ix.cells[key - kEmptyKey]));
                if (put.into_empty_word) d_live = 1;
            } else if (!UpsertOne<kCareful>(ix, key, put, &d_live, &d_used)) {
                put.code = KVCM_EC_NOSPC;  // the table is full
                if (status != nullptr) atomicAdd(&status[0], 1u);
            }
            results[i] = put.code;
        }
    }
    AddCellsPerWarp(ix, d_live, d_used);
}

// ---- rebuilding the table in place: live pairs out to a workspace, table reset, pairs back in.  Drops every
// tombstone, so probe chains are as short again as in a freshly filled table.
__global__ void CollectLiveKernel(IndexView ix, ulonglong2 *__restrict__ pairs, unsigned long long *counter) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    const uint64_t first = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint64_t rounds = (ix.mask + stride) / stride;  // the same for every thread: the ballots stay converged
    for (uint64_t r = 0; r < rounds; ++r) {
        const uint64_t i = first + r * stride;
        ulonglong2 s = make_ulonglong2(kEmptyKey, 0);
        if (i <= ix.mask) s = LoadSlot(ix.slots + i);
        const bool live = s.x != kEmptyKey && s.x != kTombKey && s.y != 0;
        const uint32_t votes = __ballot_sync(0xffffffffu, live);
        if (votes == 0) continue;
        const uint32_t lane = LaneId();
        unsigned long long base = 0;
        if (lane == static_cast<uint32_t>(__ffs(votes) - 1)) base = atomicAdd(counter, static_cast<unsigned long long>(__popc(votes)));
        base = __shfl_sync(0xffffffffu, base, __ffs(votes) - 1);
        if (live) pairs[base + __popc(votes & ((1u << lane) - 1u))] = s;
    }
}

__global__ void ResetSlotsKernel(IndexView ix) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i <= ix.mask; i += stride) {
        ix.slots[i] = make_ulonglong2(kEmptyKey, 0);
        ix.tags[i] = kTagEmpty;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {  // the two reserved keys live in their cells and stay
        ix.cells[2] = (ix.cells[0] != 0 ? 1 : 0) + (ix.cells[1] != 0 ? 1 : 0);
        ix.cells[3] = 0;
    }
}

__global__ void ReinsertKernel(IndexView ix, const ulonglong2 *__restrict__ pairs, const unsigned long long *counter,
                               uint32_t *status) {
    const uint64_t n = *counter;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        int32_t d_live = 0, d_used = 0;
        Overwrite put{pairs[i].y};
        if (!UpsertOne<false>(ix, pairs[i].x, put, &d_live, &d_used) && status != nullptr) {
            atomicAdd(&status[0], 1u);
        }
        if (d_live != 0) AddCell(&ix.cells[2], d_live);  // the pairs fitted before: no bound to watch
        if (d_used != 0) AddCell(&ix.cells[3], d_used);
    }
}

__global__ void LookupKernel(IndexView ix, const int64_t *__restrict__ keys, int64_t n, uint64_t *__restrict__ out) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = Lookup(ix, static_cast<uint64_t>(keys[i]));
}

// The flag byte of batch_get for a value word (0 = absent).
__device__ __forceinline__ uint8_t FlagsOf(uint64_t v, uint32_t avail_mask) {
    uint32_t f = 0;
    if (v != 0) {
        f |= KVCM_FLAG_EXISTS;
        if (v & KVCM_VAL_NONEMPTY) f |= KVCM_FLAG_NONEMPTY;
        if (Servable(v, avail_mask)) f |= KVCM_FLAG_SERVABLE;
        if ((static_cast<uint32_t>(v >> 16) & avail_mask & 0xFFFFu) != 0) f |= KVCM_FLAG_WRITABLE;
    }
    return static_cast<uint8_t>(f);
}

// The flags a write looks at: the ones above, and whether the key already holds a location of the class the write
// goes to (whatever its status).
__device__ __forceinline__ uint8_t WriteFlagsOf(uint64_t v, uint32_t avail_mask, uint32_t cls) {
    uint8_t f = FlagsOf(v, avail_mask);
    if (v != 0 && ((v >> (KVCM_VAL_STATUS_SHIFT + 3u * cls)) & 7u) != 0) f |= KVCM_FLAG_HAS_CLASS;
    return f;
}

__global__ void WriteSnapshotKernel(IndexView ix, const int64_t *__restrict__ keys, int64_t n, uint32_t avail_mask,
                                    uint32_t cls, Shard shard, uint8_t *__restrict__ flags) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t key = static_cast<uint64_t>(keys[i]);
    flags[i] = Owns(shard, key) ? WriteFlagsOf(Lookup(ix, key), avail_mask, cls) : 0;
}

__global__ void BatchGetKernel(IndexView ix, const int64_t *__restrict__ keys, int64_t n, uint32_t avail_mask,
                               Shard shard, uint8_t *__restrict__ flags) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t key = static_cast<uint64_t>(keys[i]);
    // A key of another shard is reported absent without touching the table.
    flags[i] = FlagsOf(Owns(shard, key) ? Lookup(ix, key) : 0, avail_mask);
}

// One warp per request; each pass probes 32 consecutive keys, one per lane, and a ballot finds
// the first unmasked key that is not servable.  The warp leaves at that key: the reference
// probes every key of the request and then stops counting at the first miss, which yields the
// same length.
__global__ void __launch_bounds__(kMatchWarps * 32)
    PrefixMatchKernel(IndexView ix, const int64_t *__restrict__ keys, const int64_t *__restrict__ key_off,
                      int32_t n_req, const int64_t *__restrict__ mask_off, const uint8_t *__restrict__ mask_bits,
                      uint32_t avail_mask, Shard shard, int32_t *__restrict__ len_out) {
    const int32_t req = blockIdx.x * kMatchWarps + (threadIdx.x >> 5);
    if (req >= n_req) return;
    const uint32_t lane = LaneId();
    const int64_t beg = key_off[req];
    const int64_t n = key_off[req + 1] - beg;
    const int64_t skip = mask_off != nullptr ? mask_off[req] : 0;
    int32_t matched = 0;
    for (int64_t base = 0; base < n; base += 32) {
        const int64_t i = base + lane;
        bool counted = false, stop = false;
        if (i < n) {
            const bool masked = i < skip || (mask_bits != nullptr && mask_bits[beg + i] != 0);
            if (!masked) {
                // A key of another shard cannot stop this shard's count: its owner decides, and the
                // caller takes the minimum over shards.
                const uint64_t key = static_cast<uint64_t>(keys[beg + i]);
                const bool hit = !Owns(shard, key) || Servable(Lookup<true>(ix, key), avail_mask);
                counted = hit;
                stop = !hit;
            }
        }
        const uint32_t stops = __ballot_sync(0xffffffffu, stop);
        const uint32_t hits = __ballot_sync(0xffffffffu, counted);
        if (stops != 0) {
            const uint32_t below = (1u << (__ffs(stops) - 1)) - 1u;
            matched += __popc(hits & below);
            break;
        }
        matched += __popc(hits);
    }
    if (lane == 0) len_out[req] = matched;
}

// Rightmost window of `sw` consecutive servable keys.  One warp per request scans 32 keys per
// pass from the right end; `run` is the length of the servable run that ends (exclusively) at
// `right_end` and reaches down to the scan position.  The first time a run reaches `sw` keys
// its right-most `sw` keys are the answer: this is where the reference's roll-back loop stops,
// because every window it skips contains a known miss.
__global__ void __launch_bounds__(kMatchWarps * 32)
    SwMatchKernel(IndexView ix, const int64_t *__restrict__ keys, const int64_t *__restrict__ key_off, int32_t n_req,
                  int32_t sw, uint32_t avail_mask, int32_t *__restrict__ base_out) {
    const int32_t req = blockIdx.x * kMatchWarps + (threadIdx.x >> 5);
    if (req >= n_req) return;
    const uint32_t lane = LaneId();
    const int64_t beg = key_off[req];
    const int64_t n = key_off[req + 1] - beg;
    if (n < sw) {
        if (lane == 0) base_out[req] = -2;
        return;
    }
    int64_t run = 0, right_end = n, found = -1;
    for (int64_t hi = n; hi > 0 && found < 0; hi -= 32) {
        if (hi + run < sw) break;  // not enough keys left for a window
        const int64_t lo = hi - 32;
        const int64_t i = lo + lane;
        const bool hit = i >= 0 && Servable(Lookup(ix, static_cast<uint64_t>(keys[beg + i])), avail_mask);
        const uint32_t bits = __ballot_sync(0xffffffffu, hit);
        int cur = 32;  // bits [0, cur) are still to be scanned, from bit cur-1 downwards
        while (cur > 0) {
            const uint32_t x = bits << (32 - cur);
            int ones = __clz(~x);
            ones = ones < cur ? ones : cur;
            run += ones;
            cur -= ones;
            if (run >= sw) {
                found = right_end - sw;
                break;
            }
            if (cur > 0) {
                int zeros = __clz(bits << (32 - cur));
                zeros = zeros < cur ? zeros : cur;
                cur -= zeros;
                run = 0;
                right_end = lo + cur;
            }
        }
    }
    if (lane == 0) base_out[req] = static_cast<int32_t>(found);
}

// The same right-to-left window search over a per-key servable byte (bit0) instead of index
// probes: the second half of the sharded sliding-window match, run after the per-key flags of all
// shards have been combined.
__global__ void __launch_bounds__(kMatchWarps * 32)
    SwFromFlagsKernel(const uint8_t *__restrict__ flags, const int64_t *__restrict__ key_off, int32_t n_req, int32_t sw,
                      int32_t *__restrict__ base_out) {
    const int32_t req = blockIdx.x * kMatchWarps + (threadIdx.x >> 5);
    if (req >= n_req) return;
    const uint32_t lane = LaneId();
    const int64_t beg = key_off[req];
    const int64_t n = key_off[req + 1] - beg;
    if (n < sw) {
        if (lane == 0) base_out[req] = -2;
        return;
    }
    int64_t run = 0, right_end = n, found = -1;
    for (int64_t hi = n; hi > 0 && found < 0; hi -= 32) {
        if (hi + run < sw) break;
        const int64_t lo = hi - 32;
        const int64_t i = lo + lane;
        const bool hit = i >= 0 && (flags[beg + i] & KVCM_FLAG_SERVABLE) != 0;
        const uint32_t bits = __ballot_sync(0xffffffffu, hit);
        int cur = 32;
        while (cur > 0) {
            const uint32_t x = bits << (32 - cur);
            int ones = __clz(~x);
            ones = ones < cur ? ones : cur;
            run += ones;
            cur -= ones;
            if (run >= sw) {
                found = right_end - sw;
                break;
            }
            if (cur > 0) {
                int zeros = __clz(bits << (32 - cur));
                zeros = zeros < cur ? zeros : cur;
                cur -= zeros;
                run = 0;
                right_end = lo + cur;
            }
        }
    }
    if (lane == 0) base_out[req] = static_cast<int32_t>(found);
}

// ------------------------------------------------------------------------------------------
// Routing a batch of keys to the shards that own them: the two device-side halves of an
// all-to-all exchange (dispatch: bucket the keys by owner; combine: bring the answers back into
// the order of the keys).  A key then crosses NVLink once as 8 bytes and its answer comes back as
// one byte, instead of one or two 32-byte peer loads per probe.
// ------------------------------------------------------------------------------------------
constexpr int kRouteThreads = 256;
constexpr int kRouteKeysPerCta = kRouteThreads * 8;
constexpr int kMaxShards = 64;

// counts[s] += keys of this batch owned by shard s.
__global__ void __launch_bounds__(kRouteThreads)
    RouteCountKernel(const int64_t *__restrict__ keys, int64_t n, uint32_t shards, uint32_t *__restrict__ counts) {
    __shared__ uint32_t local[kMaxShards];
    if (threadIdx.x < kMaxShards) local[threadIdx.x] = 0;
    __syncthreads();
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kRouteKeysPerCta;
    constexpr int kPerThread = kRouteKeysPerCta / kRouteThreads;
    int64_t key[kPerThread];
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) {  // all loads of the thread in flight before the first vote
        const int64_t i = base + j * kRouteThreads + threadIdx.x;
        key[j] = i < n ? keys[i] : 0;
    }
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) {
        if (base + j * kRouteThreads + threadIdx.x < n) {
            const uint32_t owner = OwnerOf(static_cast<uint64_t>(key[j]), shards);
            const uint32_t same = __match_any_sync(__activemask(), owner);  // one atomic per owner and warp
            if (LaneId() == static_cast<uint32_t>(__ffs(same)) - 1u) atomicAdd(&local[owner], __popc(same));
        }
    }
    __syncthreads();
    if (threadIdx.x < shards && local[threadIdx.x] != 0) atomicAdd(&counts[threadIdx.x], local[threadIdx.x]);
}

// cursor[s] holds where shard s's bucket continues in keys_out; every CTA reserves room for its keys of each
// owner with one atomic per owner, then places them.  pos_out[i] = where key i went.
__global__ void __launch_bounds__(kRouteThreads)
    RouteScatterKernel(const int64_t *__restrict__ keys, int64_t n, uint32_t shards, uint32_t *__restrict__ cursor,
                       int64_t *__restrict__ keys_out, int32_t *__restrict__ pos_out) {
    __shared__ uint32_t local[kMaxShards];
    __shared__ uint32_t start[kMaxShards];
    if (threadIdx.x < kMaxShards) local[threadIdx.x] = 0;
    __syncthreads();
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kRouteKeysPerCta;
    uint32_t rank_in_cta[kRouteKeysPerCta / kRouteThreads];
    uint32_t owner[kRouteKeysPerCta / kRouteThreads];
#pragma unroll
    for (int j = 0; j < kRouteKeysPerCta / kRouteThreads; ++j) {
        const int64_t i = base + j * kRouteThreads + threadIdx.x;
        if (i < n) {
            owner[j] = OwnerOf(static_cast<uint64_t>(keys[i]), shards);
            const uint32_t same = __match_any_sync(__activemask(), owner[j]);
            const int leader = __ffs(same) - 1;
            uint32_t first = 0;
            if (static_cast<int>(LaneId()) == leader) first = atomicAdd(&local[owner[j]], __popc(same));
            rank_in_cta[j] = __shfl_sync(same, first, leader) + __popc(same & ((1u << LaneId()) - 1u));
        }
    }
    __syncthreads();
    if (threadIdx.x < shards) start[threadIdx.x] = local[threadIdx.x] ? atomicAdd(&cursor[threadIdx.x], local[threadIdx.x]) : 0;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kRouteKeysPerCta / kRouteThreads; ++j) {
        const int64_t i = base + j * kRouteThreads + threadIdx.x;
        if (i < n) {
            const uint32_t at = start[owner[j]] + rank_in_cta[j];
            keys_out[at] = keys[i];
            pos_out[i] = static_cast<int32_t>(at);
        }
    }
}

__global__ void GatherBytesKernel(const uint8_t *__restrict__ src, const int32_t *__restrict__ pos, int64_t n,
                                  uint8_t *__restrict__ dst) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = src[pos[i]];
}

// PrefixMatchKernel over per-key flag bytes (bit0 = servable) instead of index probes: the second half of a
// routed prefix match.
__global__ void __launch_bounds__(kMatchWarps * 32)
    PrefixFromFlagsKernel(const uint8_t *__restrict__ flags, const int64_t *__restrict__ key_off, int32_t n_req,
                          const int64_t *__restrict__ mask_off, const uint8_t *__restrict__ mask_bits,
                          int32_t *__restrict__ len_out) {
    const int32_t req = blockIdx.x * kMatchWarps + (threadIdx.x >> 5);
    if (req >= n_req) return;
    const uint32_t lane = LaneId();
    const int64_t beg = key_off[req];
    const int64_t n = key_off[req + 1] - beg;
    const int64_t skip = mask_off != nullptr ? mask_off[req] : 0;
    int32_t matched = 0;
    for (int64_t base = 0; base < n; base += 32) {
        const int64_t i = base + lane;
        bool counted = false, stop = false;
        if (i < n && !(i < skip || (mask_bits != nullptr && mask_bits[beg + i] != 0))) {
            counted = (flags[beg + i] & KVCM_FLAG_SERVABLE) != 0;
            stop = !counted;
        }
        const uint32_t stops = __ballot_sync(0xffffffffu, stop);
        const uint32_t hits = __ballot_sync(0xffffffffu, counted);
        if (stops != 0) {
            matched += __popc(hits & ((1u << (__ffs(stops) - 1)) - 1u));
            break;
        }
        matched += __popc(hits);
    }
    if (lane == 0) len_out[req] = matched;
}

// ------------------------------------------------------------------------------------------
// The same exchange over peer memory, without a transport in between: the dispatch kernel stores each
// key straight into its owner's inbox (NVLink peer stores, staged per CTA so that a warp writes
// consecutive addresses), and the owner's answer kernel stores the flag bytes straight into the asking
// rank's answer buffer.  No kernel waits for another rank: the ranks meet at a barrier of the caller's
// between dispatch, answer and collect.
// ------------------------------------------------------------------------------------------
struct RoutePeers {
    int64_t *inbox[kMaxShards];
    uint8_t *answers[kMaxShards];
};
// Per call and per peer s.  Dispatch: a = where this rank's region starts in s's inbox, b = where the bucket
// of s starts in this rank's answer buffer.  Answer: a = where asker s's region starts in this rank's inbox
// (a[shards] = keys in the inbox), b = where this rank's bucket starts in asker s's answer buffer.
struct RouteStarts {
    uint32_t a[kMaxShards + 1];
    uint32_t b[kMaxShards];
};

__global__ void __launch_bounds__(kRouteThreads)
    RouteDispatchKernel(const int64_t *__restrict__ keys, int64_t n, uint32_t shards, const RoutePeers *__restrict__ peers,
                        const RouteStarts starts, uint32_t *__restrict__ cursor, int32_t *__restrict__ pos_out) {
    __shared__ int64_t staged[kRouteKeysPerCta];
    __shared__ uint32_t local[kMaxShards];        // keys of this CTA per owner
    __shared__ uint32_t local_start[kMaxShards + 1];
    __shared__ uint32_t reserved[kMaxShards];     // first index this CTA got in its rank's bucket of the owner
    constexpr int kPerThread = kRouteKeysPerCta / kRouteThreads;
    if (threadIdx.x < kMaxShards) local[threadIdx.x] = 0;
    __syncthreads();
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kRouteKeysPerCta;
    int64_t key[kPerThread];
    uint32_t rank_in_cta[kPerThread];
    uint32_t owner[kPerThread];
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) {  // all loads of the thread in flight before the first vote
        const int64_t i = base + j * kRouteThreads + threadIdx.x;
        key[j] = i < n ? keys[i] : 0;
    }
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) {
        const int64_t i = base + j * kRouteThreads + threadIdx.x;
        if (i < n) {
            owner[j] = OwnerOf(static_cast<uint64_t>(key[j]), shards);
            const uint32_t same = __match_any_sync(__activemask(), owner[j]);
            const int leader = __ffs(same) - 1;
            uint32_t first = 0;
            if (static_cast<int>(LaneId()) == leader) first = atomicAdd(&local[owner[j]], __popc(same));
            rank_in_cta[j] = __shfl_sync(same, first, leader) + __popc(same & ((1u << LaneId()) - 1u));
        }
    }
    __syncthreads();
    if (threadIdx.x < shards) reserved[threadIdx.x] = local[threadIdx.x] ? atomicAdd(&cursor[threadIdx.x], local[threadIdx.x]) : 0;
    if (threadIdx.x == 0) {
        uint32_t sum = 0;
        for (uint32_t s = 0; s < shards; ++s) {
            local_start[s] = sum;
            sum += local[s];
        }
        local_start[shards] = sum;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) {
        const int64_t i = base + j * kRouteThreads + threadIdx.x;
        if (i < n) {
            staged[local_start[owner[j]] + rank_in_cta[j]] = key[j];
            pos_out[i] = static_cast<int32_t>(starts.b[owner[j]] + reserved[owner[j]] + rank_in_cta[j]);
        }
    }
    __syncthreads();
    const uint32_t total = local_start[shards];
    for (uint32_t e = threadIdx.x; e < total; e += kRouteThreads) {
        uint32_t lo = 0, hi = shards;  // the owner whose run of the staged keys holds e
        while (hi - lo > 1) {
            const uint32_t mid = (lo + hi) >> 1;
            if (local_start[mid] <= e) lo = mid; else hi = mid;
        }
        peers->inbox[lo][starts.a[lo] + reserved[lo] + (e - local_start[lo])] = staged[e];
    }
}

__global__ void RouteAnswerKernel(IndexView ix, const int64_t *__restrict__ inbox, uint32_t n_inbox, uint32_t shards,
                                  const RoutePeers *__restrict__ peers, const RouteStarts starts, uint32_t avail_mask) {
    const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n_inbox) return;
    uint32_t lo = 0, hi = shards;  // the asker whose region holds j
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (starts.a[mid] <= j) lo = mid; else hi = mid;
    }
    const uint8_t f = FlagsOf(LookupIn<false>(ix, static_cast<uint64_t>(inbox[j])), avail_mask);
    peers->answers[lo][starts.b[lo] + (j - starts.a[lo])] = f;
}

// CacheManager::FilterWriteCache (kv_cache_manager/manager/cache_manager.cc:589-635) for a batch of
// requests, one warp each.  exists(key) = ExistsForWrite: some location with status != NOT_FOUND and
// weight > 0.  If the keys that exist form a prefix of the request, the answer is the offset of the
// first missing key (offset_out >= 0, new keys = the suffix); otherwise offset_out = -1 and the answer
// is the per-key mask "location map non-empty" written to mask_out (new keys = the rest).
__global__ void __launch_bounds__(kMatchWarps * 32)
    FilterWriteKernel(IndexView ix, const int64_t *__restrict__ keys, const int64_t *__restrict__ key_off,
                      int32_t n_req, uint32_t avail_mask, int32_t *__restrict__ offset_out,
                      uint8_t *__restrict__ mask_out, int32_t *__restrict__ n_new_out) {
    const int32_t req = blockIdx.x * kMatchWarps + (threadIdx.x >> 5);
    if (req >= n_req) return;
    const uint32_t lane = LaneId();
    const int64_t beg = key_off[req];
    const int64_t n = key_off[req + 1] - beg;
    int64_t first_missing = n;   // first key without a writable location
    bool exists_after = false;   // some key at or after first_missing exists
    int32_t n_empty = 0;         // keys whose location map is empty
    for (int64_t base = 0; base < n; base += 32) {
        const int64_t i = base + lane;
        bool exists = false, nonempty = false;
        if (i < n) {
            const uint64_t v = Lookup(ix, static_cast<uint64_t>(keys[beg + i]));
            exists = (static_cast<uint32_t>(v >> 16) & avail_mask & 0xFFFFu) != 0;
            nonempty = (v & KVCM_VAL_NONEMPTY) != 0;
            if (mask_out != nullptr) mask_out[beg + i] = nonempty ? 1 : 0;
        }
        const uint32_t in_range = __ballot_sync(0xffffffffu, i < n);
        const uint32_t ex = __ballot_sync(0xffffffffu, exists);
        const uint32_t ne = __ballot_sync(0xffffffffu, nonempty);
        n_empty += __popc(in_range & ~ne);
        if (first_missing == n) {
            const uint32_t missing = in_range & ~ex;
            if (missing != 0) {
                const int pos = __ffs(missing) - 1;
                first_missing = base + pos;
                if ((ex >> pos) != 0) exists_after = true;  // an existing key later in this pass
            }
        } else if (ex != 0) {
            exists_after = true;
        }
    }
    if (lane == 0) {
        if (!exists_after) {
            offset_out[req] = static_cast<int32_t>(first_missing);
            n_new_out[req] = static_cast<int32_t>(n - first_missing);
        } else {
            offset_out[req] = -1;
            n_new_out[req] = n_empty;
        }
    }
}

// ---- StartWriteCache / FinishWriteCache for a batch of requests (CacheManager::StartWriteCache = FilterWriteCache +
// MetaSearcher::BatchAddLocation, kv_cache_manager/manager/cache_manager.cc:334-430,589-635; FinishWriteCache,
// :432-501), with the answers the reference gives when it serves the requests one after the other in batch order.
// What request r sees of a key is what the index held before the batch plus what the requests before r added.  A
// key with an empty (or no) location map is added by the FIRST request that names it, whatever that request's
// block mask looks like - so "the first request that names the key" (an atomic minimum per key, over dense ids
// of the batch's keys) settles, for all requests at once, both who writes a key and what the later ones see.
// The one thing that stays sequential is a key whose map is not empty but holds nothing writable (only locations
// the policy gives no weight, or locations whose status is CLS_NOT_FOUND): a request whose existing keys form a
// prefix adds a location to it, a request with holes does not, and which of the two a request is may depend on
// such a key.  Requests that name one are rare; they are marked, left out of the parallel pass, and served
// afterwards by one warp in batch order.
struct StartWrite {
    IndexView ix;
    const int64_t *keys;
    const int64_t *key_off;
    int32_t n_req;
    uint32_t avail_mask;
    uint32_t cls;
    IdTable table;
    uint32_t *ids;         // per key occurrence: dense id of the key (keys that are writable already have none)
    uint32_t *first;       // per id: the first request that names the key
    uint8_t *snap;         // per key occurrence: the flags of the key before the batch
    uint8_t *ordered;      // per request: 1 = names a key with a map but nothing writable: served in order
    uint32_t *n_ordered;   // how many requests that is
    uint8_t *late_added;   // per id: such a key got its location from an earlier request of the batch
    int32_t *offset_out;
    uint8_t *mask_out;
    int32_t *n_new_out;
    uint8_t *added_out;    // per key occurrence: 1 = this request gave the key its new location
    int32_t *n_added;      // per request: how many keys that is (the length of its write session)
    // One table of a hash-range-sharded index: every shard runs the call on the same batch (all shards' requests in
    // one order) with the same flags per key - each key's flags come from its owner, snap_in - and merges the
    // locations of the keys it owns; whether a key of another shard takes its location is read off its flags.
    const uint8_t *snap_in;
    const uint8_t *skip;   // optional, per request: 1 = not a request (padding of the gathered batch)
    Shard shard;
    uint32_t *status;      // [0] keys refused because the table is full
};

__global__ void StartWriteInitKernel(IdTable t, uint32_t *first, uint8_t *late_added, uint8_t *ordered,
                                     uint32_t *n_ordered, int64_t n_keys, int32_t n_req) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    const uint64_t at = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (uint64_t i = at; i <= t.mask; i += stride) t.slots[i] = make_ulonglong2(kEmptyKey, ~0ull);
    for (uint64_t i = at; i < static_cast<uint64_t>(n_keys); i += stride) {
        first[i] = 0xFFFFFFFFu;
        late_added[i] = 0;
    }
    for (uint64_t i = at; i < static_cast<uint64_t>(n_req); i += stride) ordered[i] = 0;
    if (at == 0) {
        t.cells[0] = 0ull;
        t.cells[1] = ~0ull;
        *n_ordered = 0u;
    }
}

// Pass 1 (a warp per request): the flags of every key before the batch; keys that are not writable claim an id.
__global__ void __launch_bounds__(kMatchWarps * 32) StartWriteSnapshotKernel(StartWrite p) {
    const int32_t req = blockIdx.x * kMatchWarps + (threadIdx.x >> 5);
    if (req >= p.n_req || (p.skip != nullptr && p.skip[req] != 0)) return;
    const int64_t beg = p.key_off[req], end = p.key_off[req + 1];
    bool late = false;
    for (int64_t i = beg + LaneId(); i < end; i += 32) {
        const uint64_t key = static_cast<uint64_t>(p.keys[i]);
        const uint8_t f = p.snap_in != nullptr ? p.snap_in[i] : WriteFlagsOf(Lookup(p.ix, key), p.avail_mask, p.cls);
        p.snap[i] = f;
        if ((f & KVCM_FLAG_WRITABLE) == 0) {
            ClaimId(p.table, key, nullptr);
            late = late || (f & KVCM_FLAG_NONEMPTY) != 0;
        }
    }
    if (__any_sync(0xffffffffu, late) && LaneId() == 0) {
        p.ordered[req] = 1;
        atomicAdd(p.n_ordered, 1u);
    }
}

// Pass 2 (a warp per request): ids, and per key the first request that names it.
__global__ void __launch_bounds__(kMatchWarps * 32) StartWriteOwnersKernel(StartWrite p) {
    const int32_t req = blockIdx.x * kMatchWarps + (threadIdx.x >> 5);
    if (req >= p.n_req || (p.skip != nullptr && p.skip[req] != 0)) return;
    const int64_t beg = p.key_off[req], end = p.key_off[req + 1];
    for (int64_t i = beg + LaneId(); i < end; i += 32) {
        if ((p.snap[i] & KVCM_FLAG_WRITABLE) != 0) continue;
        const uint32_t id = LookupId(p.table, static_cast<uint64_t>(p.keys[i]));
        p.ids[i] = id;
        if ((p.snap[i] & KVCM_FLAG_NONEMPTY) == 0) atomicMin(&p.first[id], static_cast<uint32_t>(req));
    }
}

// One request, all lanes of a warp: its block mask, and the locations it adds.  kCareful as in UpsertOne: the batch
// could push the slots in use past the table's bound, so every claim of an empty slot takes a seat first.
template <bool kCareful>
__device__ __forceinline__ void StartWriteOne(const StartWrite &p, int32_t req, int32_t *d_live, int32_t *d_used) {
    const uint32_t lane = LaneId();
    const uint32_t full = 0xffffffffu;
    const int64_t beg = p.key_off[req];
    const int64_t n = p.key_off[req + 1] - beg;
    const uint32_t r = static_cast<uint32_t>(req);
    if (p.skip != nullptr && p.skip[req] != 0) {  // padding: no keys of its own, nothing to answer
        for (int64_t i = lane; i < n; i += 32) {
            p.added_out[beg + i] = 0;
            if (p.mask_out != nullptr) p.mask_out[beg + i] = 0;
        }
        if (lane == 0) p.offset_out[req] = p.n_new_out[req] = p.n_added[req] = 0;
        return;
    }
    const bool sharded = p.snap_in != nullptr;
    // what this request sees of key i: (exists for write, location map non-empty, id)
    auto view = [&](int64_t i, bool *exists, bool *nonempty, uint32_t *id) {
        const uint8_t f = p.snap[beg + i];
        *exists = (f & KVCM_FLAG_WRITABLE) != 0;
        *nonempty = (f & KVCM_FLAG_NONEMPTY) != 0;
        *id = 0xFFFFFFFFu;
        if (*exists) return;
        *id = p.ids[beg + i];
        if (*nonempty) {  // a map with nothing writable: writable once an earlier request has added to it
            *exists = *reinterpret_cast<volatile uint8_t *>(&p.late_added[*id]) != 0;
        } else if (p.first[*id] < r) {  // added by an earlier request of the batch (in CLS_WRITING)
            *exists = *nonempty = true;
        }
    };
    int64_t first_missing = n;
    bool exists_after = false;
    int32_t n_empty = 0;
    for (int64_t base = 0; base < n; base += 32) {
        const int64_t i = base + lane;
        bool exists = false, nonempty = false;
        uint32_t id;
        if (i < n) {
            view(i, &exists, &nonempty, &id);
            if (p.mask_out != nullptr) p.mask_out[beg + i] = nonempty ? 1 : 0;
        }
        const uint32_t in_range = __ballot_sync(full, i < n);
        const uint32_t ex = __ballot_sync(full, exists);
        const uint32_t ne = __ballot_sync(full, nonempty);
        n_empty += __popc(in_range & ~ne);
        if (first_missing == n) {
            const uint32_t missing = in_range & ~ex;
            if (missing != 0) {
                const int pos = __ffs(missing) - 1;
                first_missing = base + pos;
                if ((ex >> pos) != 0) exists_after = true;
            }
        } else if (ex != 0) {
            exists_after = true;
        }
    }
    const bool prefix_form = !exists_after;
    if (lane == 0) {
        p.offset_out[req] = prefix_form ? static_cast<int32_t>(first_missing) : -1;
        p.n_new_out[req] = prefix_form ? static_cast<int32_t>(n - first_missing) : n_empty;
    }
    // the new keys: everything from the first missing key on, or the keys whose map is empty
    int32_t session = 0;
    for (int64_t base = 0; base < n; base += 32) {
        const int64_t i = base + lane;
        bool exists = false, nonempty = false;
        uint32_t id = 0xFFFFFFFFu;
        if (i < n) view(i, &exists, &nonempty, &id);
        const bool is_new = i < n && (prefix_form ? i >= first_missing : !nonempty);
        uint8_t added = 0;
        if (is_new) {
            const uint64_t key = static_cast<uint64_t>(p.keys[beg + i]);
            // in a sharded call every shard has to give the same answer: the class is free or it is not, which the
            // key's flags say (a full table shows in the owner's status count only)
            const bool takes_it = (p.snap[beg + i] & KVCM_FLAG_HAS_CLASS) == 0;
            MergeLocation put{p.cls, 2u /* CLS_WRITING */, KVCM_EC_ERROR, false};
            if (!Owns(p.shard, key)) {
                put.code = takes_it ? KVCM_OK : KVCM_EC_EXIST;
            } else if (key == kEmptyKey || key == kTombKey) {
                put(reinterpret_cast<unsigned long long *>(&p.ix.cells[key - kEmptyKey]));
                if (put.into_empty_word) *d_live += 1;
            } else if (!UpsertOne<kCareful>(p.ix, key, put, d_live, d_used)) {
                put.code = KVCM_EC_NOSPC;
                if (p.status != nullptr) atomicAdd(&p.status[0], 1u);
            }
            added = (sharded ? takes_it : put.code == KVCM_OK) ? 1 : 0;
            if (added != 0 && nonempty) p.late_added[id] = 1;
        }
        if (i < n) p.added_out[beg + i] = added;
        session += __popc(__ballot_sync(full, added != 0));
    }
    if (lane == 0) p.n_added[req] = session;
}

// Pass 3: every request that can be served by itself, a warp each.
template <bool kCareful>
__global__ void __launch_bounds__(kMatchWarps * 32) StartWriteParallelKernel(StartWrite p) {
    const int32_t req = blockIdx.x * kMatchWarps + (threadIdx.x >> 5);
    int32_t d_live = 0, d_used = 0;
    if (req < p.n_req && p.ordered[req] == 0) StartWriteOne<kCareful>(p, req, &d_live, &d_used);
    AddCellsPerWarp(p.ix, d_live, d_used);
}

// Pass 4: the others, one warp, in batch order (nothing to do for most batches).
template <bool kCareful>
__global__ void __launch_bounds__(32) StartWriteOrderedKernel(StartWrite p) {
    if (*p.n_ordered == 0u) return;
    int32_t d_live = 0, d_used = 0;
    for (int32_t base = 0; base < p.n_req; base += 32) {
        const int32_t mine = base + static_cast<int32_t>(LaneId());
        uint32_t todo = __ballot_sync(0xffffffffu, mine < p.n_req && p.ordered[mine] != 0);
        while (todo != 0) {
            const int32_t req = base + __ffs(todo) - 1;
            todo &= todo - 1;
            StartWriteOne<kCareful>(p, req, &d_live, &d_used);
            __threadfence();  // what this request added is what the next one sees
            __syncwarp();
        }
    }
    AddCellsPerWarp(p.ix, d_live, d_used);
}

// new_off[r] = session keys of the requests before r (one CTA; a running sum over chunks of 1,024 requests).
__global__ void __launch_bounds__(1024) StartWriteOffsetsKernel(const int32_t *__restrict__ n_new, int32_t n_req,
                                                                 int64_t *__restrict__ new_off) {
    __shared__ int64_t warp_sum[32];
    __shared__ int64_t carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int32_t base = 0; base < n_req; base += 1024) {
        const int32_t r = base + static_cast<int32_t>(threadIdx.x);
        const int64_t mine = r < n_req ? n_new[r] : 0;
        int64_t scan = mine;
        for (int d = 1; d < 32; d <<= 1) {
            const int64_t up = __shfl_up_sync(0xffffffffu, scan, d);
            if (static_cast<int>(LaneId()) >= d) scan += up;
        }
        if (LaneId() == 31) warp_sum[threadIdx.x >> 5] = scan;
        __syncthreads();
        if (threadIdx.x < 32) {
            int64_t w = warp_sum[threadIdx.x];
            for (int d = 1; d < 32; d <<= 1) {
                const int64_t up = __shfl_up_sync(0xffffffffu, w, d);
                if (static_cast<int>(threadIdx.x) >= d) w += up;
            }
            warp_sum[threadIdx.x] = w;
        }
        __syncthreads();
        const int64_t before = carry + ((threadIdx.x >> 5) > 0 ? warp_sum[(threadIdx.x >> 5) - 1] : 0) + scan - mine;
        if (r < n_req) new_off[r] = before;
        __syncthreads();
        if (threadIdx.x == 1023) carry = before + mine;
        __syncthreads();
    }
    if (threadIdx.x == 0) new_off[n_req] = carry;
}

// FinishWriteCache of a batch of sessions (a warp per request): the j-th key a request added (its session's keys,
// in request order) turns CLS_SERVING when the success mask holds it - an offset (j < offset) or one byte per
// session key - and loses its location otherwise.  An invalid mask (an offset beyond the session's keys) leaves the
// session untouched and answers KVCM_EC_BADARGS for the request.
__global__ void __launch_bounds__(kMatchWarps * 32)
    FinishWriteKernel(IndexView ix, const int64_t *__restrict__ keys, const int64_t *__restrict__ key_off, int32_t n_req,
                      const uint8_t *__restrict__ added, const int64_t *__restrict__ new_off,
                      const int64_t *__restrict__ success_off, const uint8_t *__restrict__ success_bits, uint32_t cls,
                      Shard shard, int32_t *__restrict__ results) {
    const int32_t req = blockIdx.x * kMatchWarps + (threadIdx.x >> 5);
    if (req >= n_req) return;
    const uint32_t lane = LaneId();
    const int64_t beg = key_off[req], n = key_off[req + 1] - beg;
    const int64_t mine = new_off[req + 1] - new_off[req];
    if (success_bits == nullptr && (success_off[req] < 0 || success_off[req] > mine)) {
        if (lane == 0) results[req] = KVCM_EC_BADARGS;
        return;
    }
    const uint32_t serve = KVCM_STATUS_TASK(cls, KVCM_STATUS_ANY, 3u);
    const uint32_t drop = KVCM_STATUS_TASK(cls, KVCM_STATUS_ANY, KVCM_STATUS_DELETE);
    int64_t rank = 0;  // session keys in front of this pass
    int32_t worst = KVCM_OK;
    for (int64_t base = 0; base < n; base += 32) {
        const int64_t i = base + lane;
        const bool is_mine = i < n && added[beg + i] != 0;
        const uint32_t m = __ballot_sync(0xffffffffu, is_mine);
        if (is_mine) {
            const int64_t j = rank + __popc(m & ((1u << lane) - 1u));
            const bool ok = success_bits != nullptr ? success_bits[new_off[req] + j] != 0 : j < success_off[req];
            const uint64_t key = static_cast<uint64_t>(keys[beg + i]);
            if (Owns(shard, key)) {  // the owner shard makes the transition
                const int32_t code = RunStatusTask(ix, key, ok ? serve : drop);
                if (ok && code != KVCM_OK) worst = code;
            }
        }
        rank += __popc(m);
    }
    worst = __reduce_max_sync(0xffffffffu, worst);
    if (lane == 0) results[req] = worst;
}

// View for the matchers: probes follow the attached peers.
IndexView View(const kvcm_b200_index *ix) {
    IndexView v;
    v.slots = ix->slots;
    v.tags = ix->tags;
    v.cells = ix->cells;
    v.mask = ix->n_slots - 1;
    v.max_live = ix->max_live;
    v.peers = static_cast<const IndexView *>(ix->d_peer_views);
    v.peer_count = ix->peer_count;
    return v;
}

// View of this table alone, for the kernels that write it.
IndexView LocalView(const kvcm_b200_index *ix) {
    IndexView v = View(ix);
    v.peers = nullptr;
    v.peer_count = 0;
    return v;
}

unsigned GridFor(int64_t n, int threads) { return static_cast<unsigned>((n + threads - 1) / threads); }

}  // namespace
}  // namespace kvcm

extern "C" {

int32_t kvcm_b200_index_create(int64_t max_keys, kvcm_b200_index_t **out) {
    if (out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    *out = nullptr;
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (max_keys < 0 || max_keys > (1ll << 36)) return KVCM_EC_BADARGS;
    uint64_t n_slots = 1024;
    while (n_slots < 2ull * static_cast<uint64_t>(max_keys)) n_slots <<= 1;
    auto *ix = new kvcm_b200_index();
    ix->n_slots = n_slots;
    ix->max_live = n_slots - n_slots / 8;  // the matchers rely on at least one EMPTY slot per chain
    ix->tomb_debt = 0;
    ix->auto_rehash_at = n_slots / 8;
    ix->used_upper = 0;
    cudaGetDevice(&ix->device);
    if (cudaMalloc(&ix->base, kvcm::kIndexHeaderBytes + n_slots * (sizeof(ulonglong2) + 1)) != cudaSuccess) {
        cudaGetLastError();
        delete ix;
        return KVCM_EC_NOSPC;
    }
    ix->cells = static_cast<uint64_t *>(ix->base);
    ix->slots = reinterpret_cast<ulonglong2 *>(static_cast<uint8_t *>(ix->base) + kvcm::kIndexHeaderBytes);
    ix->tags = reinterpret_cast<uint8_t *>(ix->slots + n_slots);
    const int32_t rc = kvcm_b200_index_clear(ix, nullptr);
    if (rc != KVCM_OK || cudaStreamSynchronize(nullptr) != cudaSuccess) {
        cudaFree(ix->base);
        delete ix;
        return KVCM_ER_CUDA_STREAM_SYNCHRONIZE_ERROR;
    }
    *out = ix;
    return KVCM_OK;
}

int32_t kvcm_b200_index_detach_peers(kvcm_b200_index_t *ix) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (ix->d_peer_views != nullptr) cudaFree(ix->d_peer_views);
    ix->d_peer_views = nullptr;
    ix->peer_count = 0;
    for (int i = 0; i < ix->n_opened; ++i) cudaIpcCloseMemHandle(ix->opened[i]);
    ix->n_opened = 0;
    cudaGetLastError();
    return KVCM_OK;
}

int32_t kvcm_b200_index_destroy(kvcm_b200_index_t *ix) {
    if (ix == nullptr) return KVCM_OK;
    kvcm_b200_index_detach_peers(ix);
    cudaFree(ix->base);
    delete ix;
    return KVCM_OK;
}

int32_t kvcm_b200_index_export(kvcm_b200_index_t *ix, kvcm_b200_index_export_t *out) {
    if (ix == nullptr || out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    static_assert(sizeof(cudaIpcMemHandle_t) <= sizeof(out->ipc_handle), "IPC handle does not fit");
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, ix->base) != cudaSuccess) {
        cudaGetLastError();
        return KVCM_EC_ERROR;
    }
    memset(out, 0, sizeof(*out));
    memcpy(out->ipc_handle, &h, sizeof(h));
    out->n_slots = ix->n_slots;
    out->device = ix->device;
    return KVCM_OK;
}

// Uploads the table of shard views; shard_rank's own entry is the local table.
static int32_t InstallPeerViews(kvcm_b200_index_t *ix, int32_t shard_count, const kvcm::IndexView *views) {
    void *d = nullptr;
    if (cudaMalloc(&d, sizeof(kvcm::IndexView) * shard_count) != cudaSuccess ||
        cudaMemcpy(d, views, sizeof(kvcm::IndexView) * shard_count, cudaMemcpyHostToDevice) != cudaSuccess) {
        cudaGetLastError();
        if (d != nullptr) cudaFree(d);
        return KVCM_EC_NOSPC;
    }
    ix->d_peer_views = d;
    ix->peer_count = static_cast<uint32_t>(shard_count);
    return KVCM_OK;
}

int32_t kvcm_b200_index_attach_peers(kvcm_b200_index_t *ix, int32_t shard_count, int32_t shard_rank,
                                     const kvcm_b200_index_export_t *exports) {
    if (ix == nullptr || exports == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (shard_count < 1 || shard_count > 64 || shard_rank < 0 || shard_rank >= shard_count) return KVCM_EC_BADARGS;
    kvcm_b200_index_detach_peers(ix);
    kvcm::IndexView views[64];
    for (int32_t r = 0; r < shard_count; ++r) {
        kvcm::IndexView &v = views[r];
        v.peers = nullptr;
        v.peer_count = 0;
        v.max_live = 0;
        if (r == shard_rank) {
            v = kvcm::LocalView(ix);
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, exports[r].ipc_handle, sizeof(h));
        void *base = nullptr;
        if (cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            cudaGetLastError();
            kvcm_b200_index_detach_peers(ix);
            return KVCM_EC_ERROR;
        }
        ix->opened[ix->n_opened++] = base;
        v.cells = static_cast<uint64_t *>(base);
        v.slots = reinterpret_cast<ulonglong2 *>(static_cast<uint8_t *>(base) + kvcm::kIndexHeaderBytes);
        v.tags = reinterpret_cast<uint8_t *>(v.slots + exports[r].n_slots);
        v.mask = exports[r].n_slots - 1;
    }
    return InstallPeerViews(ix, shard_count, views);
}

int32_t kvcm_b200_index_attach_local_peers(kvcm_b200_index_t *ix, int32_t shard_count, int32_t shard_rank,
                                           kvcm_b200_index_t *const *shards) {
    if (ix == nullptr || shards == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (shard_count < 1 || shard_count > 64 || shard_rank < 0 || shard_rank >= shard_count) return KVCM_EC_BADARGS;
    kvcm_b200_index_detach_peers(ix);
    kvcm::IndexView views[64];
    for (int32_t r = 0; r < shard_count; ++r) {
        if (shards[r] == nullptr) return KVCM_ER_INVALID_ADDRESS;
        views[r] = kvcm::LocalView(shards[r]);
    }
    return InstallPeerViews(ix, shard_count, views);
}

int32_t kvcm_b200_index_clear(kvcm_b200_index_t *ix, kvcm_stream_t stream) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    const unsigned grid = static_cast<unsigned>(kvcm::GetDeviceInfo().sm_count * 8);
    ix->tomb_debt = 0;
    ix->used_upper = 0;
    kvcm::ClearKernel<<<grid, 256, 0, kvcm::AsStream(stream)>>>(kvcm::LocalView(ix));
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_index_stats(kvcm_b200_index_t *ix, int64_t *slots, int64_t *live_keys, kvcm_stream_t stream) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (slots != nullptr) *slots = static_cast<int64_t>(ix->n_slots);
    if (live_keys != nullptr) {
        uint64_t live = 0;
        if (cudaMemcpyAsync(&live, ix->cells + 2, sizeof(live), cudaMemcpyDeviceToHost, kvcm::AsStream(stream)) !=
                cudaSuccess ||
            cudaStreamSynchronize(kvcm::AsStream(stream)) != cudaSuccess) {
            return KVCM_ER_CUDA_STREAM_SYNCHRONIZE_ERROR;
        }
        *live_keys = static_cast<int64_t>(live);
    }
    return KVCM_OK;
}

int32_t kvcm_b200_index_usage(kvcm_b200_index_t *ix, int64_t *slots, int64_t *live_keys, int64_t *used_slots,
                              kvcm_stream_t stream) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    uint64_t cells[2] = {0, 0};
    if (cudaMemcpyAsync(cells, ix->cells + 2, sizeof(cells), cudaMemcpyDeviceToHost, kvcm::AsStream(stream)) !=
            cudaSuccess ||
        cudaStreamSynchronize(kvcm::AsStream(stream)) != cudaSuccess) {
        return KVCM_ER_CUDA_STREAM_SYNCHRONIZE_ERROR;
    }
    if (slots != nullptr) *slots = static_cast<int64_t>(ix->n_slots);
    if (live_keys != nullptr) *live_keys = static_cast<int64_t>(cells[0]);
    if (used_slots != nullptr) *used_slots = static_cast<int64_t>(cells[1]);
    ix->used_upper = cells[1];  // everything enqueued before the read has run: this is the true figure
    return KVCM_OK;
}

int64_t kvcm_b200_index_rehash_workspace_bytes(kvcm_b200_index_t *ix) {
    if (ix == nullptr) return 0;
    return 256 + static_cast<int64_t>(ix->n_slots) * static_cast<int64_t>(sizeof(ulonglong2));
}

int32_t kvcm_b200_index_set_auto_rehash(kvcm_b200_index_t *ix, int64_t erased_keys) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (erased_keys < 0) return KVCM_EC_BADARGS;
    ix->auto_rehash_at = static_cast<uint64_t>(erased_keys);
    return KVCM_OK;
}

// Before an insert: once enough keys have been erased since the last rebuild, rebuild first.  The workspace comes
// from and goes back to the stream-ordered allocator, so nothing waits on the host; when it cannot be had the
// rebuild is skipped and tried again at the next insert.
static void MaybeRehash(kvcm_b200_index_t *ix, kvcm_stream_t stream) {
    if (ix->auto_rehash_at == 0 || ix->tomb_debt < ix->auto_rehash_at) return;
    const int64_t bytes = kvcm_b200_index_rehash_workspace_bytes(ix);
    void *ws = nullptr;
    if (cudaMallocAsync(&ws, static_cast<size_t>(bytes), kvcm::AsStream(stream)) != cudaSuccess) {
        cudaGetLastError();
        return;
    }
    kvcm_b200_index_rehash(ix, ws, bytes, nullptr, stream);
    cudaFreeAsync(ws, kvcm::AsStream(stream));
}

int32_t kvcm_b200_index_rehash(kvcm_b200_index_t *ix, void *d_workspace, int64_t workspace_bytes, uint32_t *d_status,
                               kvcm_stream_t stream) {
    if (ix == nullptr || d_workspace == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if ((reinterpret_cast<uintptr_t>(d_workspace) & 15u) != 0) return KVCM_ER_INVALID_ADDRESS;
    if (workspace_bytes < kvcm_b200_index_rehash_workspace_bytes(ix)) return KVCM_EC_NOSPC;
    cudaStream_t s = kvcm::AsStream(stream);
    auto *counter = static_cast<unsigned long long *>(d_workspace);
    auto *pairs = reinterpret_cast<ulonglong2 *>(static_cast<uint8_t *>(d_workspace) + 256);
    if (cudaMemsetAsync(counter, 0, 256, s) != cudaSuccess) return KVCM_ER_CUDAMEMCPY_ERROR;
    const kvcm::IndexView view = kvcm::LocalView(ix);
    const unsigned grid = static_cast<unsigned>(kvcm::GetDeviceInfo().sm_count * 8);
    kvcm::CollectLiveKernel<<<grid, 256, 0, s>>>(view, pairs, counter);
    kvcm::ResetSlotsKernel<<<grid, 256, 0, s>>>(view);
    kvcm::ReinsertKernel<<<grid, 256, 0, s>>>(view, pairs, counter, d_status);
    ix->tomb_debt = 0;
    return kvcm::LaunchStatus();
}

static int32_t UpdateStatus(kvcm_b200_index_t *ix, const int64_t *d_keys, const uint32_t *d_tasks, uint32_t uniform_task,
                            int64_t n, kvcm::Shard shard, int32_t *d_results, kvcm_stream_t stream) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (n < 0) return KVCM_EC_BADARGS;
    if (d_tasks == nullptr) {
        const uint32_t cls = uniform_task & 0xFFu, expected = (uniform_task >> 8) & 0xFFu,
                       next = (uniform_task >> 16) & 0xFFu;
        if (cls > 7 || (expected > 4 && expected != KVCM_STATUS_ANY) ||
            (next > 4 && next != KVCM_STATUS_DELETE && next != KVCM_STATUS_DELETE_KEEP_KEY)) {
            return KVCM_EC_BADARGS;
        }
    }
    if (n == 0) return KVCM_OK;
    if (d_keys == nullptr || d_results == nullptr) return KVCM_ER_INVALID_ADDRESS;
    ix->tomb_debt += static_cast<uint64_t>(n);  // any of the tasks may remove its key's last location
    kvcm::UpdateStatusKernel<<<kvcm::GridFor(n, 256), 256, 0, kvcm::AsStream(stream)>>>(
        kvcm::LocalView(ix), d_keys, d_tasks, uniform_task, n, shard, d_results);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_index_update_status(kvcm_b200_index_t *ix, const int64_t *d_keys, const uint32_t *d_tasks,
                                      uint32_t uniform_task, int64_t n, int32_t *d_results, kvcm_stream_t stream) {
    return UpdateStatus(ix, d_keys, d_tasks, uniform_task, n, kvcm::Shard{1, 0}, d_results, stream);
}

int32_t kvcm_b200_index_update_status_sharded(kvcm_b200_index_t *ix, const int64_t *d_keys, const uint32_t *d_tasks,
                                              uint32_t uniform_task, int64_t n, int32_t shard_count, int32_t shard_rank,
                                              int32_t *d_results, kvcm_stream_t stream) {
    if (shard_count < 1 || shard_rank < 0 || shard_rank >= shard_count) return KVCM_EC_BADARGS;
    return UpdateStatus(ix, d_keys, d_tasks, uniform_task, n,
                        kvcm::Shard{static_cast<uint32_t>(shard_count), static_cast<uint32_t>(shard_rank)}, d_results,
                        stream);
}

static int32_t AddLocation(kvcm_b200_index_t *ix, const int64_t *d_keys, const uint8_t *d_classes,
                           int32_t uniform_class, int32_t status_of_new, int64_t n, kvcm::Shard shard,
                           int32_t *d_results, uint32_t *d_status, kvcm_stream_t stream) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (n < 0 || status_of_new < 0 || status_of_new > 4 || (d_classes == nullptr && (uniform_class < 0 || uniform_class > 7))) {
        return KVCM_EC_BADARGS;
    }
    if (n == 0) return KVCM_OK;
    if (d_keys == nullptr || d_results == nullptr) return KVCM_ER_INVALID_ADDRESS;
    MaybeRehash(ix, stream);
    const bool careful = ix->used_upper + static_cast<uint64_t>(n) > ix->max_live;
    ix->used_upper += static_cast<uint64_t>(n);
    if (ix->used_upper > ix->n_slots) ix->used_upper = ix->n_slots;
    const unsigned grid = kvcm::GridFor(n, 256);
    const uint32_t cls = static_cast<uint32_t>(d_classes == nullptr ? uniform_class : 0);
    if (careful) {
        kvcm::AddLocationKernel<true><<<grid, 256, 0, kvcm::AsStream(stream)>>>(
            kvcm::LocalView(ix), d_keys, d_classes, cls, static_cast<uint32_t>(status_of_new), n, shard, d_results,
            d_status);
    } else {
        kvcm::AddLocationKernel<false><<<grid, 256, 0, kvcm::AsStream(stream)>>>(
            kvcm::LocalView(ix), d_keys, d_classes, cls, static_cast<uint32_t>(status_of_new), n, shard, d_results,
            d_status);
    }
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_index_add_location(kvcm_b200_index_t *ix, const int64_t *d_keys, const uint8_t *d_classes,
                                     int32_t uniform_class, int32_t status_of_new, int64_t n, int32_t *d_results,
                                     uint32_t *d_status, kvcm_stream_t stream) {
    return AddLocation(ix, d_keys, d_classes, uniform_class, status_of_new, n, kvcm::Shard{1, 0}, d_results, d_status,
                       stream);
}

int32_t kvcm_b200_index_add_location_sharded(kvcm_b200_index_t *ix, const int64_t *d_keys, const uint8_t *d_classes,
                                             int32_t uniform_class, int32_t status_of_new, int64_t n,
                                             int32_t shard_count, int32_t shard_rank, int32_t *d_results,
                                             uint32_t *d_status, kvcm_stream_t stream) {
    if (shard_count < 1 || shard_rank < 0 || shard_rank >= shard_count) return KVCM_EC_BADARGS;
    return AddLocation(ix, d_keys, d_classes, uniform_class, status_of_new, n,
                       kvcm::Shard{static_cast<uint32_t>(shard_count), static_cast<uint32_t>(shard_rank)}, d_results,
                       d_status, stream);
}

static void LaunchUpsert(kvcm_b200_index_t *ix, const int64_t *d_keys, const uint64_t *d_values, uint64_t uniform_value,
                         int64_t n, kvcm::Shard shard, uint32_t *d_status, kvcm_stream_t stream) {
    const bool careful = ix->used_upper + static_cast<uint64_t>(n) > ix->max_live;
    ix->used_upper += static_cast<uint64_t>(n);
    if (ix->used_upper > ix->n_slots) ix->used_upper = ix->n_slots;
    const unsigned grid = kvcm::GridFor(n, 256);
    if (careful) {
        kvcm::UpsertKernel<true><<<grid, 256, 0, kvcm::AsStream(stream)>>>(kvcm::LocalView(ix), d_keys, d_values,
                                                                            uniform_value, n, shard, d_status);
    } else {
        kvcm::UpsertKernel<false><<<grid, 256, 0, kvcm::AsStream(stream)>>>(kvcm::LocalView(ix), d_keys, d_values,
                                                                             uniform_value, n, shard, d_status);
    }
}

int32_t kvcm_b200_index_upsert(kvcm_b200_index_t *ix, const int64_t *d_keys, const uint64_t *d_values,
                               uint64_t uniform_value, int64_t n, uint32_t *d_status, kvcm_stream_t stream) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (n < 0) return KVCM_EC_BADARGS;
    if (n == 0) return KVCM_OK;
    if (d_keys == nullptr) return KVCM_ER_INVALID_ADDRESS;
    MaybeRehash(ix, stream);
    LaunchUpsert(ix, d_keys, d_values, uniform_value, n, kvcm::Shard{1, 0}, d_status, stream);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_index_upsert_sharded(kvcm_b200_index_t *ix, const int64_t *d_keys, const uint64_t *d_values,
                                       uint64_t uniform_value, int64_t n, int32_t shard_count, int32_t shard_rank,
                                       uint32_t *d_status, kvcm_stream_t stream) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (n < 0 || shard_count < 1 || shard_rank < 0 || shard_rank >= shard_count) return KVCM_EC_BADARGS;
    if (n == 0) return KVCM_OK;
    if (d_keys == nullptr) return KVCM_ER_INVALID_ADDRESS;
    MaybeRehash(ix, stream);
    LaunchUpsert(ix, d_keys, d_values, uniform_value, n,
                 kvcm::Shard{static_cast<uint32_t>(shard_count), static_cast<uint32_t>(shard_rank)}, d_status, stream);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_index_erase(kvcm_b200_index_t *ix, const int64_t *d_keys, int64_t n, kvcm_stream_t stream) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (n < 0) return KVCM_EC_BADARGS;
    if (n == 0) return KVCM_OK;
    if (d_keys == nullptr) return KVCM_ER_INVALID_ADDRESS;
    ix->tomb_debt += static_cast<uint64_t>(n);
    kvcm::EraseKernel<<<kvcm::GridFor(n, 256), 256, 0, kvcm::AsStream(stream)>>>(kvcm::LocalView(ix), d_keys, n);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_index_lookup(kvcm_b200_index_t *ix, const int64_t *d_keys, int64_t n, uint64_t *d_values_out,
                               kvcm_stream_t stream) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (n < 0) return KVCM_EC_BADARGS;
    if (n == 0) return KVCM_OK;
    if (d_keys == nullptr || d_values_out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    kvcm::LookupKernel<<<kvcm::GridFor(n, 256), 256, 0, kvcm::AsStream(stream)>>>(kvcm::View(ix), d_keys, n,
                                                                                   d_values_out);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_match_prefix(kvcm_b200_index_t *ix, const int64_t *d_keys, const int64_t *d_key_off, int32_t n_req,
                               const int64_t *d_mask_off, const uint8_t *d_mask_bits, uint32_t avail_mask,
                               int32_t *d_len_out, kvcm_stream_t stream) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (n_req < 0) return KVCM_EC_BADARGS;
    if (n_req == 0) return KVCM_OK;
    if (d_key_off == nullptr || d_len_out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    kvcm::PrefixMatchKernel<<<kvcm::GridFor(n_req, kvcm::kMatchWarps), kvcm::kMatchWarps * 32, 0,
                              kvcm::AsStream(stream)>>>(kvcm::View(ix), d_keys, d_key_off, n_req, d_mask_off,
                                                        d_mask_bits, avail_mask, kvcm::Shard{1, 0}, d_len_out);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_match_prefix_sharded(kvcm_b200_index_t *ix, const int64_t *d_keys, const int64_t *d_key_off,
                                       int32_t n_req, const int64_t *d_mask_off, const uint8_t *d_mask_bits,
                                       uint32_t avail_mask, int32_t shard_count, int32_t shard_rank,
                                       int32_t *d_len_out, kvcm_stream_t stream) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (n_req < 0 || shard_count < 1 || shard_rank < 0 || shard_rank >= shard_count) return KVCM_EC_BADARGS;
    if (n_req == 0) return KVCM_OK;
    if (d_key_off == nullptr || d_len_out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    kvcm::PrefixMatchKernel<<<kvcm::GridFor(n_req, kvcm::kMatchWarps), kvcm::kMatchWarps * 32, 0,
                              kvcm::AsStream(stream)>>>(
        kvcm::View(ix), d_keys, d_key_off, n_req, d_mask_off, d_mask_bits, avail_mask,
        kvcm::Shard{static_cast<uint32_t>(shard_count), static_cast<uint32_t>(shard_rank)}, d_len_out);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_match_sw_from_flags(const uint8_t *d_flags, const int64_t *d_key_off, int32_t n_req,
                                      int32_t sw_blocks, int32_t *d_base_out, kvcm_stream_t stream) {
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (n_req < 0 || sw_blocks <= 0) return KVCM_EC_BADARGS;
    if (n_req == 0) return KVCM_OK;
    if (d_key_off == nullptr || d_base_out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    kvcm::SwFromFlagsKernel<<<kvcm::GridFor(n_req, kvcm::kMatchWarps), kvcm::kMatchWarps * 32, 0,
                              kvcm::AsStream(stream)>>>(d_flags, d_key_off, n_req, sw_blocks, d_base_out);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_route_count(const int64_t *d_keys, int64_t n, int32_t shard_count, uint32_t *d_counts,
                              kvcm_stream_t stream) {
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (n < 0 || n > 0x7fffffffll || shard_count < 1 || shard_count > kvcm::kMaxShards) return KVCM_EC_BADARGS;
    if (d_counts == nullptr || (d_keys == nullptr && n > 0)) return KVCM_ER_INVALID_ADDRESS;
    if (cudaMemsetAsync(d_counts, 0, sizeof(uint32_t) * shard_count, kvcm::AsStream(stream)) != cudaSuccess) {
        cudaGetLastError();
        return KVCM_ER_CUDAMEMCPY_ERROR;
    }
    if (n == 0) return KVCM_OK;
    kvcm::RouteCountKernel<<<kvcm::GridFor(n, kvcm::kRouteKeysPerCta), kvcm::kRouteThreads, 0, kvcm::AsStream(stream)>>>(
        d_keys, n, static_cast<uint32_t>(shard_count), d_counts);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_route_scatter(const int64_t *d_keys, int64_t n, int32_t shard_count, uint32_t *d_cursor,
                                int64_t *d_keys_out, int32_t *d_pos_out, kvcm_stream_t stream) {
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (n < 0 || n > 0x7fffffffll || shard_count < 1 || shard_count > kvcm::kMaxShards) return KVCM_EC_BADARGS;
    if (n == 0) return KVCM_OK;
    if (d_keys == nullptr || d_cursor == nullptr || d_keys_out == nullptr || d_pos_out == nullptr) {
        return KVCM_ER_INVALID_ADDRESS;
    }
    kvcm::RouteScatterKernel<<<kvcm::GridFor(n, kvcm::kRouteKeysPerCta), kvcm::kRouteThreads, 0,
                               kvcm::AsStream(stream)>>>(d_keys, n, static_cast<uint32_t>(shard_count), d_cursor,
                                                         d_keys_out, d_pos_out);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_gather_bytes(const uint8_t *d_src, const int32_t *d_pos, int64_t n, uint8_t *d_dst,
                               kvcm_stream_t stream) {
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (n < 0) return KVCM_EC_BADARGS;
    if (n == 0) return KVCM_OK;
    if (d_src == nullptr || d_pos == nullptr || d_dst == nullptr) return KVCM_ER_INVALID_ADDRESS;
    kvcm::GatherBytesKernel<<<kvcm::GridFor(n, 256), 256, 0, kvcm::AsStream(stream)>>>(d_src, d_pos, n, d_dst);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_match_prefix_from_flags(const uint8_t *d_flags, const int64_t *d_key_off, int32_t n_req,
                                          const int64_t *d_mask_off, const uint8_t *d_mask_bits, int32_t *d_len_out,
                                          kvcm_stream_t stream) {
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (n_req < 0) return KVCM_EC_BADARGS;
    if (n_req == 0) return KVCM_OK;
    if (d_key_off == nullptr || d_len_out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    kvcm::PrefixFromFlagsKernel<<<kvcm::GridFor(n_req, kvcm::kMatchWarps), kvcm::kMatchWarps * 32, 0,
                                  kvcm::AsStream(stream)>>>(d_flags, d_key_off, n_req, d_mask_off, d_mask_bits,
                                                            d_len_out);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_route_area_detach(kvcm_b200_route_area_t *area) {
    if (area == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (area->d_peer_table != nullptr) cudaFree(area->d_peer_table);
    area->d_peer_table = nullptr;
    area->peer_count = 0;
    for (int i = 0; i < area->n_opened; ++i) cudaIpcCloseMemHandle(area->opened[i]);
    area->n_opened = 0;
    cudaGetLastError();
    return KVCM_OK;
}

int32_t kvcm_b200_route_area_destroy(kvcm_b200_route_area_t *area) {
    if (area == nullptr) return KVCM_OK;
    kvcm_b200_route_area_detach(area);
    cudaFree(area->base);
    delete area;
    return KVCM_OK;
}

int32_t kvcm_b200_route_area_create(int64_t capacity_keys, kvcm_b200_route_area_t **out) {
    if (out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    *out = nullptr;
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (capacity_keys < 1 || capacity_keys > 0x7fffffffll) return KVCM_EC_BADARGS;
    auto *area = new kvcm_b200_route_area();
    area->capacity = (static_cast<uint64_t>(capacity_keys) + 255u) & ~uint64_t{255};
    if (cudaGetDevice(&area->device) != cudaSuccess || cudaMalloc(&area->base, area->capacity * 9) != cudaSuccess) {
        cudaGetLastError();
        delete area;
        return KVCM_EC_NOSPC;
    }
    area->inbox = static_cast<int64_t *>(area->base);
    area->answers = reinterpret_cast<uint8_t *>(area->inbox + area->capacity);
    *out = area;
    return KVCM_OK;
}

int32_t kvcm_b200_route_area_export(kvcm_b200_route_area_t *area, kvcm_b200_route_export_t *out) {
    if (area == nullptr || out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) <= sizeof(out->ipc_handle), "IPC handle does not fit");
    if (cudaIpcGetMemHandle(&h, area->base) != cudaSuccess) {
        cudaGetLastError();
        return KVCM_EC_ERROR;
    }
    memset(out, 0, sizeof(*out));
    memcpy(out->ipc_handle, &h, sizeof(h));
    out->capacity_keys = area->capacity;
    out->device = area->device;
    return KVCM_OK;
}

static int32_t InstallRoutePeers(kvcm_b200_route_area_t *area, int32_t shard_count, int32_t shard_rank,
                                 const kvcm::RoutePeers &table) {
    void *d = nullptr;
    if (cudaMalloc(&d, sizeof(table)) != cudaSuccess ||
        cudaMemcpy(d, &table, sizeof(table), cudaMemcpyHostToDevice) != cudaSuccess) {
        cudaGetLastError();
        if (d != nullptr) cudaFree(d);
        return KVCM_EC_NOSPC;
    }
    area->d_peer_table = d;
    area->peer_count = static_cast<uint32_t>(shard_count);
    area->self = static_cast<uint32_t>(shard_rank);
    return KVCM_OK;
}

int32_t kvcm_b200_route_area_attach(kvcm_b200_route_area_t *area, int32_t shard_count, int32_t shard_rank,
                                    const kvcm_b200_route_export_t *exports) {
    if (area == nullptr || exports == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (shard_count < 1 || shard_count > kvcm::kMaxShards || shard_rank < 0 || shard_rank >= shard_count) {
        return KVCM_EC_BADARGS;
    }
    kvcm_b200_route_area_detach(area);
    kvcm::RoutePeers table{};
    for (int32_t r = 0; r < shard_count; ++r) {
        if (r == shard_rank) {
            table.inbox[r] = area->inbox;
            table.answers[r] = area->answers;
            continue;
        }
        if (exports[r].capacity_keys != area->capacity) {  // one capacity for all ranks: the checks are local then
            kvcm_b200_route_area_detach(area);
            return KVCM_EC_BADARGS;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, exports[r].ipc_handle, sizeof(h));
        void *base = nullptr;
        if (cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            cudaGetLastError();
            kvcm_b200_route_area_detach(area);
            return KVCM_EC_ERROR;
        }
        area->opened[area->n_opened++] = base;
        table.inbox[r] = static_cast<int64_t *>(base);
        table.answers[r] = reinterpret_cast<uint8_t *>(table.inbox[r] + exports[r].capacity_keys);
    }
    return InstallRoutePeers(area, shard_count, shard_rank, table);
}

int32_t kvcm_b200_route_area_attach_local(kvcm_b200_route_area_t *area, int32_t shard_count, int32_t shard_rank,
                                          kvcm_b200_route_area_t *const *areas) {
    if (area == nullptr || areas == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (shard_count < 1 || shard_count > kvcm::kMaxShards || shard_rank < 0 || shard_rank >= shard_count) {
        return KVCM_EC_BADARGS;
    }
    kvcm_b200_route_area_detach(area);
    kvcm::RoutePeers table{};
    for (int32_t r = 0; r < shard_count; ++r) {
        if (areas[r] == nullptr) return KVCM_ER_INVALID_ADDRESS;
        if (areas[r]->capacity != area->capacity) return KVCM_EC_BADARGS;
        table.inbox[r] = areas[r]->inbox;
        table.answers[r] = areas[r]->answers;
    }
    return InstallRoutePeers(area, shard_count, shard_rank, table);
}

// h_counts[r * shards + s] = keys rank r sends to shard s (the same matrix on every rank).
static bool RouteFits(const kvcm_b200_route_area_t *area, const uint32_t *h_counts, uint32_t shards) {
    for (uint32_t owner = 0; owner < shards; ++owner) {  // every inbox holds what all ranks send it
        uint64_t sum = 0;
        for (uint32_t r = 0; r < shards; ++r) sum += h_counts[r * shards + owner];
        if (sum > area->capacity) return false;
    }
    for (uint32_t r = 0; r < shards; ++r) {  // every answer buffer holds one byte per key of its rank
        uint64_t sum = 0;
        for (uint32_t owner = 0; owner < shards; ++owner) sum += h_counts[r * shards + owner];
        if (sum > area->capacity) return false;
    }
    return true;
}

int32_t kvcm_b200_route_dispatch(kvcm_b200_route_area_t *area, const int64_t *d_keys, int64_t n,
                                 const uint32_t *h_counts, uint32_t *d_cursor, int32_t *d_pos_out,
                                 kvcm_stream_t stream) {
    if (area == nullptr || h_counts == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (area->d_peer_table == nullptr || n < 0 || n > 0x7fffffffll) return KVCM_EC_BADARGS;
    const uint32_t shards = area->peer_count, self = area->self;
    if (!RouteFits(area, h_counts, shards)) return KVCM_EC_NOSPC;
    uint64_t mine = 0;
    for (uint32_t owner = 0; owner < shards; ++owner) mine += h_counts[self * shards + owner];
    if (mine != static_cast<uint64_t>(n)) return KVCM_EC_BADARGS;
    if (n == 0) return KVCM_OK;
    if (d_keys == nullptr || d_cursor == nullptr || d_pos_out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    kvcm::RouteStarts starts{};
    uint32_t bucket = 0;
    for (uint32_t owner = 0; owner < shards; ++owner) {
        uint32_t before = 0;  // what the ranks below this one send to the same owner
        for (uint32_t r = 0; r < self; ++r) before += h_counts[r * shards + owner];
        starts.a[owner] = before;
        starts.b[owner] = bucket;
        bucket += h_counts[self * shards + owner];
    }
    if (cudaMemsetAsync(d_cursor, 0, sizeof(uint32_t) * shards, kvcm::AsStream(stream)) != cudaSuccess) {
        cudaGetLastError();
        return KVCM_ER_CUDAMEMCPY_ERROR;
    }
    kvcm::RouteDispatchKernel<<<kvcm::GridFor(n, kvcm::kRouteKeysPerCta), kvcm::kRouteThreads, 0,
                                kvcm::AsStream(stream)>>>(d_keys, n, shards,
                                                          static_cast<const kvcm::RoutePeers *>(area->d_peer_table),
                                                          starts, d_cursor, d_pos_out);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_route_answer(kvcm_b200_index_t *ix, kvcm_b200_route_area_t *area, const uint32_t *h_counts,
                               uint32_t avail_mask, kvcm_stream_t stream) {
    if (ix == nullptr || area == nullptr || h_counts == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (area->d_peer_table == nullptr) return KVCM_EC_BADARGS;
    const uint32_t shards = area->peer_count, self = area->self;
    if (!RouteFits(area, h_counts, shards)) return KVCM_EC_NOSPC;
    kvcm::RouteStarts starts{};
    uint32_t arrived = 0;
    for (uint32_t asker = 0; asker < shards; ++asker) {
        starts.a[asker] = arrived;
        arrived += h_counts[asker * shards + self];
        uint32_t bucket = 0;  // where this rank's bucket starts among the asker's keys
        for (uint32_t owner = 0; owner < self; ++owner) bucket += h_counts[asker * shards + owner];
        starts.b[asker] = bucket;
    }
    starts.a[shards] = arrived;
    if (arrived == 0) return KVCM_OK;
    kvcm::RouteAnswerKernel<<<kvcm::GridFor(arrived, 256), 256, 0, kvcm::AsStream(stream)>>>(
        kvcm::LocalView(ix), area->inbox, arrived, shards, static_cast<const kvcm::RoutePeers *>(area->d_peer_table),
        starts, avail_mask);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_route_collect(kvcm_b200_route_area_t *area, const int32_t *d_pos, int64_t n, uint8_t *d_flags_out,
                                kvcm_stream_t stream) {
    if (area == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (n < 0 || static_cast<uint64_t>(n) > area->capacity) return KVCM_EC_BADARGS;
    return kvcm_b200_gather_bytes(area->answers, d_pos, n, d_flags_out, stream);
}

int32_t kvcm_b200_match_sw(kvcm_b200_index_t *ix, const int64_t *d_keys, const int64_t *d_key_off, int32_t n_req,
                           int32_t sw_blocks, uint32_t avail_mask, int32_t *d_base_out, kvcm_stream_t stream) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (n_req < 0 || sw_blocks <= 0) return KVCM_EC_BADARGS;
    if (n_req == 0) return KVCM_OK;
    if (d_key_off == nullptr || d_base_out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    kvcm::SwMatchKernel<<<kvcm::GridFor(n_req, kvcm::kMatchWarps), kvcm::kMatchWarps * 32, 0,
                          kvcm::AsStream(stream)>>>(kvcm::View(ix), d_keys, d_key_off, n_req, sw_blocks, avail_mask,
                                                    d_base_out);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_filter_write(kvcm_b200_index_t *ix, const int64_t *d_keys, const int64_t *d_key_off, int32_t n_req,
                               uint32_t avail_mask, int32_t *d_offset_out, uint8_t *d_mask_out, int32_t *d_n_new_out,
                               kvcm_stream_t stream) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (n_req < 0) return KVCM_EC_BADARGS;
    if (n_req == 0) return KVCM_OK;
    if (d_key_off == nullptr || d_offset_out == nullptr || d_n_new_out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    kvcm::FilterWriteKernel<<<kvcm::GridFor(n_req, kvcm::kMatchWarps), kvcm::kMatchWarps * 32, 0,
                              kvcm::AsStream(stream)>>>(kvcm::View(ix), d_keys, d_key_off, n_req, avail_mask,
                                                        d_offset_out, d_mask_out, d_n_new_out);
    return kvcm::LaunchStatus();
}

namespace {

struct StartWriteLayout {
    // (the first 256 bytes hold the id table's two cells and the count of requests served in order)
    size_t table_off, ids_off, first_off, snap_off, late_off, ordered_off, n_added_off, total;
};

StartWriteLayout StartWriteLayoutFor(int64_t n_keys, int32_t n_req) {
    auto up = [](size_t v) { return (v + 255) & ~static_cast<size_t>(255); };
    const size_t nk = static_cast<size_t>(n_keys > 0 ? n_keys : 1);
    StartWriteLayout l;
    l.table_off = 256;
    l.ids_off = up(l.table_off + kvcm::SlotsFor(n_keys) * sizeof(ulonglong2));
    l.first_off = up(l.ids_off + nk * 4);
    l.snap_off = up(l.first_off + nk * 4);
    l.late_off = up(l.snap_off + nk);
    l.ordered_off = up(l.late_off + nk);
    l.n_added_off = up(l.ordered_off + static_cast<size_t>(n_req > 0 ? n_req : 1));
    l.total = up(l.n_added_off + static_cast<size_t>(n_req > 0 ? n_req : 1) * 4);
    return l;
}

}  // namespace

int64_t kvcm_b200_start_write_workspace_bytes(int64_t n_keys_total, int32_t n_req) {
    if (n_keys_total < 0 || n_keys_total >= (1ll << 31) || n_req < 0) return -1;
    return static_cast<int64_t>(StartWriteLayoutFor(n_keys_total, n_req).total);
}

static int32_t StartWriteImpl(kvcm_b200_index_t *ix, const int64_t *d_keys, const int64_t *d_key_off, int32_t n_req,
                              int64_t n_keys_total, uint32_t avail_mask, int32_t storage_class,
                              const uint8_t *d_snapshot_flags, const uint8_t *d_request_skip, kvcm::Shard shard,
                              void *d_workspace, int64_t workspace_bytes, int32_t *d_offset_out, uint8_t *d_mask_out,
                              int32_t *d_n_new_out, uint8_t *d_added_out, int64_t *d_new_off_out, uint32_t *d_status,
                              kvcm_stream_t stream) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    // the class new locations go to has to count for the policy, or what a request adds would not be there for the next
    if (n_req < 0 || n_keys_total < 0 || storage_class < 0 || storage_class > 7 ||
        ((avail_mask >> storage_class) & 1u) == 0) {
        return KVCM_EC_BADARGS;
    }
    const int64_t need = kvcm_b200_start_write_workspace_bytes(n_keys_total, n_req);
    if (need < 0) return KVCM_EC_OUT_OF_LIMIT;
    if (n_req == 0) return KVCM_OK;
    if (d_key_off == nullptr || d_offset_out == nullptr || d_n_new_out == nullptr || d_added_out == nullptr ||
        d_new_off_out == nullptr || d_workspace == nullptr || (d_keys == nullptr && n_keys_total > 0)) {
        return KVCM_ER_INVALID_ADDRESS;
    }
    if (reinterpret_cast<uintptr_t>(d_workspace) & 255u) return KVCM_ER_INVALID_ADDRESS;
    if (workspace_bytes < need) return KVCM_EC_NOSPC;
    MaybeRehash(ix, stream);
    const bool careful = ix->used_upper + static_cast<uint64_t>(n_keys_total) > ix->max_live;
    ix->used_upper += static_cast<uint64_t>(n_keys_total);
    if (ix->used_upper > ix->n_slots) ix->used_upper = ix->n_slots;
    const StartWriteLayout l = StartWriteLayoutFor(n_keys_total, n_req);
    uint8_t *ws = static_cast<uint8_t *>(d_workspace);
    kvcm::StartWrite p;
    p.ix = kvcm::LocalView(ix);
    p.keys = d_keys;
    p.key_off = d_key_off;
    p.n_req = n_req;
    p.avail_mask = avail_mask;
    p.cls = static_cast<uint32_t>(storage_class);
    p.table.cells = reinterpret_cast<unsigned long long *>(ws);
    p.table.slots = reinterpret_cast<ulonglong2 *>(ws + l.table_off);
    p.table.mask = kvcm::SlotsFor(n_keys_total) - 1;
    p.ids = reinterpret_cast<uint32_t *>(ws + l.ids_off);
    p.first = reinterpret_cast<uint32_t *>(ws + l.first_off);
    p.snap = ws + l.snap_off;
    p.late_added = ws + l.late_off;
    p.ordered = ws + l.ordered_off;
    p.n_ordered = reinterpret_cast<uint32_t *>(ws + 16);  // beside the id table's two cells in the first 256 bytes
    p.n_added = reinterpret_cast<int32_t *>(ws + l.n_added_off);
    p.offset_out = d_offset_out;
    p.mask_out = d_mask_out;
    p.n_new_out = d_n_new_out;
    p.added_out = d_added_out;
    p.status = d_status;
    p.snap_in = d_snapshot_flags;
    p.skip = d_request_skip;
    p.shard = shard;
    cudaStream_t s = kvcm::AsStream(stream);
    const int sms = kvcm::GetDeviceInfo().sm_count;
    const unsigned grid = kvcm::GridFor(n_req, kvcm::kMatchWarps);
    const unsigned threads = kvcm::kMatchWarps * 32;
    kvcm::StartWriteInitKernel<<<sms * 4, 256, 0, s>>>(p.table, p.first, p.late_added, p.ordered, p.n_ordered,
                                                       n_keys_total, n_req);
    kvcm::StartWriteSnapshotKernel<<<grid, threads, 0, s>>>(p);
    kvcm::StartWriteOwnersKernel<<<grid, threads, 0, s>>>(p);
    if (careful) {
        kvcm::StartWriteParallelKernel<true><<<grid, threads, 0, s>>>(p);
        kvcm::StartWriteOrderedKernel<true><<<1, 32, 0, s>>>(p);
    } else {
        kvcm::StartWriteParallelKernel<false><<<grid, threads, 0, s>>>(p);
        kvcm::StartWriteOrderedKernel<false><<<1, 32, 0, s>>>(p);
    }
    kvcm::StartWriteOffsetsKernel<<<1, 1024, 0, s>>>(p.n_added, n_req, d_new_off_out);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_start_write(kvcm_b200_index_t *ix, const int64_t *d_keys, const int64_t *d_key_off, int32_t n_req,
                              int64_t n_keys_total, uint32_t avail_mask, int32_t storage_class, void *d_workspace,
                              int64_t workspace_bytes, int32_t *d_offset_out, uint8_t *d_mask_out,
                              int32_t *d_n_new_out, uint8_t *d_added_out, int64_t *d_new_off_out, uint32_t *d_status,
                              kvcm_stream_t stream) {
    return StartWriteImpl(ix, d_keys, d_key_off, n_req, n_keys_total, avail_mask, storage_class, nullptr, nullptr,
                          kvcm::Shard{1, 0}, d_workspace, workspace_bytes, d_offset_out, d_mask_out, d_n_new_out,
                          d_added_out, d_new_off_out, d_status, stream);
}

int32_t kvcm_b200_start_write_sharded(kvcm_b200_index_t *ix, const int64_t *d_keys, const int64_t *d_key_off,
                                      int32_t n_req, int64_t n_keys_total, uint32_t avail_mask, int32_t storage_class,
                                      const uint8_t *d_snapshot_flags, const uint8_t *d_request_skip,
                                      int32_t shard_count, int32_t shard_rank, void *d_workspace,
                                      int64_t workspace_bytes, int32_t *d_offset_out, uint8_t *d_mask_out,
                                      int32_t *d_n_new_out, uint8_t *d_added_out, int64_t *d_new_off_out,
                                      uint32_t *d_status, kvcm_stream_t stream) {
    if (shard_count < 1 || shard_rank < 0 || shard_rank >= shard_count) return KVCM_EC_BADARGS;
    if (d_snapshot_flags == nullptr && n_keys_total > 0) return KVCM_ER_INVALID_ADDRESS;
    return StartWriteImpl(ix, d_keys, d_key_off, n_req, n_keys_total, avail_mask, storage_class, d_snapshot_flags,
                          d_request_skip, kvcm::Shard{static_cast<uint32_t>(shard_count), static_cast<uint32_t>(shard_rank)},
                          d_workspace, workspace_bytes, d_offset_out, d_mask_out, d_n_new_out, d_added_out,
                          d_new_off_out, d_status, stream);
}

int32_t kvcm_b200_write_snapshot_sharded(kvcm_b200_index_t *ix, const int64_t *d_keys, int64_t n, uint32_t avail_mask,
                                         int32_t storage_class, int32_t shard_count, int32_t shard_rank,
                                         uint8_t *d_flags_out, kvcm_stream_t stream) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (n < 0 || storage_class < 0 || storage_class > 7 || shard_count < 1 || shard_rank < 0 ||
        shard_rank >= shard_count) {
        return KVCM_EC_BADARGS;
    }
    if (n == 0) return KVCM_OK;
    if (d_keys == nullptr || d_flags_out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    kvcm::WriteSnapshotKernel<<<kvcm::GridFor(n, 256), 256, 0, kvcm::AsStream(stream)>>>(
        kvcm::LocalView(ix), d_keys, n, avail_mask, static_cast<uint32_t>(storage_class),
        kvcm::Shard{static_cast<uint32_t>(shard_count), static_cast<uint32_t>(shard_rank)}, d_flags_out);
    return kvcm::LaunchStatus();
}

static int32_t FinishWriteImpl(kvcm_b200_index_t *ix, const int64_t *d_keys, const int64_t *d_key_off, int32_t n_req,
                               const uint8_t *d_added, const int64_t *d_new_off, const int64_t *d_success_off,
                               const uint8_t *d_success_bits, int32_t storage_class, kvcm::Shard shard,
                               int32_t *d_results, kvcm_stream_t stream) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (n_req < 0 || storage_class < 0 || storage_class > 7) return KVCM_EC_BADARGS;
    if (n_req == 0) return KVCM_OK;
    if (d_key_off == nullptr || d_added == nullptr || d_new_off == nullptr || d_results == nullptr ||
        (d_success_off == nullptr && d_success_bits == nullptr)) {
        return KVCM_ER_INVALID_ADDRESS;
    }
    ix->tomb_debt += static_cast<uint64_t>(n_req);  // failed blocks may take their keys with them
    kvcm::FinishWriteKernel<<<kvcm::GridFor(n_req, kvcm::kMatchWarps), kvcm::kMatchWarps * 32, 0,
                              kvcm::AsStream(stream)>>>(kvcm::LocalView(ix), d_keys, d_key_off, n_req, d_added,
                                                        d_new_off, d_success_off, d_success_bits,
                                                        static_cast<uint32_t>(storage_class), shard, d_results);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_finish_write(kvcm_b200_index_t *ix, const int64_t *d_keys, const int64_t *d_key_off, int32_t n_req,
                               const uint8_t *d_added, const int64_t *d_new_off, const int64_t *d_success_off,
                               const uint8_t *d_success_bits, int32_t storage_class, int32_t *d_results,
                               kvcm_stream_t stream) {
    return FinishWriteImpl(ix, d_keys, d_key_off, n_req, d_added, d_new_off, d_success_off, d_success_bits,
                           storage_class, kvcm::Shard{1, 0}, d_results, stream);
}

int32_t kvcm_b200_finish_write_sharded(kvcm_b200_index_t *ix, const int64_t *d_keys, const int64_t *d_key_off,
                                       int32_t n_req, const uint8_t *d_added, const int64_t *d_new_off,
                                       const int64_t *d_success_off, const uint8_t *d_success_bits,
                                       int32_t storage_class, int32_t shard_count, int32_t shard_rank,
                                       int32_t *d_results, kvcm_stream_t stream) {
    if (shard_count < 1 || shard_rank < 0 || shard_rank >= shard_count) return KVCM_EC_BADARGS;
    return FinishWriteImpl(ix, d_keys, d_key_off, n_req, d_added, d_new_off, d_success_off, d_success_bits,
                           storage_class, kvcm::Shard{static_cast<uint32_t>(shard_count), static_cast<uint32_t>(shard_rank)},
                           d_results, stream);
}

int32_t kvcm_b200_batch_get(kvcm_b200_index_t *ix, const int64_t *d_keys, int64_t n, uint32_t avail_mask,
                            uint8_t *d_flags_out, kvcm_stream_t stream) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (n < 0) return KVCM_EC_BADARGS;
    if (n == 0) return KVCM_OK;
    if (d_keys == nullptr || d_flags_out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    kvcm::BatchGetKernel<<<kvcm::GridFor(n, 256), 256, 0, kvcm::AsStream(stream)>>>(
        kvcm::View(ix), d_keys, n, avail_mask, kvcm::Shard{1, 0}, d_flags_out);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_batch_get_sharded(kvcm_b200_index_t *ix, const int64_t *d_keys, int64_t n, uint32_t avail_mask,
                                    int32_t shard_count, int32_t shard_rank, uint8_t *d_flags_out,
                                    kvcm_stream_t stream) {
    if (ix == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (n < 0 || shard_count < 1 || shard_rank < 0 || shard_rank >= shard_count) return KVCM_EC_BADARGS;
    if (n == 0) return KVCM_OK;
    if (d_keys == nullptr || d_flags_out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    kvcm::BatchGetKernel<<<kvcm::GridFor(n, 256), 256, 0, kvcm::AsStream(stream)>>>(
        kvcm::View(ix), d_keys, n, avail_mask,
        kvcm::Shard{static_cast<uint32_t>(shard_count), static_cast<uint32_t>(shard_rank)}, d_flags_out);
    return kvcm::LaunchStatus();
}

}  // extern "C"
