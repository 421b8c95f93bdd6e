// The "random_lru" eviction policy as a warp runs it: RandomLruEvictionPolicy
// (kv_cache_manager/optimizer/eviction_policy/random_lru.cc:5-131, random_lru.h:13-47) over per-key state.
// Shared by the sweep of sampling instances alone (replay_random_lru.cu) and the sweep of groups that mix the
// policies (replay_leaf_lru.cu).
//
// The policy's own state is what the reference keeps: a dense vector of the cached blocks beside their last access
// times, a key's index in it, and the state of its xorshift generator.
//   pos[id]   kNotCached, else the block's index in blk / ts
//   blk[i]    id of the block at index i; ts[i] its last access time; i < size
// A round of evictions (EvictBlocks, random_lru.cc:38-57) draws `sampling_size` indices with replacement
// (FastRand, :121-131), orders the first k of them by access time with std::partial_sort (:59-82) and removes those
// blocks by swap-and-pop (:84-103).  Blocks written or read by one trace share a timestamp, so WHICH of several
// equally old samples go depends on the order std::partial_sort leaves equal elements in.  That order is a
// property of the algorithm the C++ standard library documents for it - heap-select followed by sort-heap on a
// binary max-heap with hole-based sift-down and sift-up - which is restated below, step for step, on the sample
// held in shared memory; the CPU oracle calls std::partial_sort itself, and the parity tests compare the two on
// traces full of tied timestamps.
// The generator is sequential, the heap is sequential: both run in lane 0 (the raw draws first, the modulo of all
// draws then in parallel; the times of the sampled indices are gathered by all lanes).  The removals are
// sequential too - every one changes the index of the block that was last - but run out of shared memory: the
// tail of the block vector is staged there, and the victims' indices are kept current by a warp-wide scan.
#pragma once
#include "kvcm_common.cuh"

namespace kvcm {
namespace {

constexpr uint32_t kMaxSample = KVCM_B200_RANDOM_LRU_MAX_SAMPLE;  // sampled indices per round held in shared memory
constexpr uint32_t kMaxBatch = KVCM_B200_RANDOM_LRU_MAX_BATCH;    // blocks evicted per round
constexpr uint32_t kNotCached = 0xFFFFFFFFu;
constexpr uint64_t kSamplingSeed = 0x12345678ABCDEF01ull;  // random_lru.h:20; every policy object starts from it

// The policy's generator (FastRand, random_lru.cc:121-131) is xorshift64: three shift-and-xor steps, a linear map of
// the 64 state bits over GF(2).  So is its 32nd power, which lets every lane of a warp produce every 32nd draw by
// itself: the first 32 draws are made in sequence, then lane l jumps from draw l to draw l + 32, l + 64, ...  The
// jump is the matrix of that power applied to the state, stored as eight tables of 256 entries (one per state byte:
// the xor of the columns its set bits select), worked out by the compiler.
__host__ __device__ constexpr uint64_t XorShiftStep(uint64_t x) {
    x ^= x << 13;
    x ^= x >> 7;
    x ^= x << 17;
    return x;
}

struct JumpTables {
    uint64_t of_byte[8][256];
};

constexpr JumpTables MakeJump32() {
    JumpTables t{};
    uint64_t column[64] = {};
    for (int bit = 0; bit < 64; ++bit) {
        uint64_t x = 1ull << bit;
        for (int step = 0; step < 32; ++step) x = XorShiftStep(x);
        column[bit] = x;
    }
    for (int byte = 0; byte < 8; ++byte) {
        for (int value = 0; value < 256; ++value) {
            uint64_t x = 0;
            for (int bit = 0; bit < 8; ++bit) {
                if ((value >> bit) & 1) x ^= column[8 * byte + bit];
            }
            t.of_byte[byte][value] = x;
        }
    }
    return t;
}

constexpr JumpTables kHostJump32 = MakeJump32();
__device__ const JumpTables kJump32 = kHostJump32;

__device__ __forceinline__ uint64_t Jump32(uint64_t x) {
    uint64_t r = 0;
#pragma unroll
    for (int byte = 0; byte < 8; ++byte) r ^= kJump32.of_byte[byte][(x >> (8 * byte)) & 255u];
    return r;
}

// One sampled block: its last access time and its index in the block vector, moved together - one 16-byte shared
// memory access each way.
struct __align__(16) SampleEntry {
    int64_t t;
    uint32_t idx;
    uint32_t pad;
};

__host__ __device__ __forceinline__ SampleEntry LoadEntry(const SampleEntry *s, uint32_t i) {
#ifdef __CUDA_ARCH__
    const int4 v = *reinterpret_cast<const int4 *>(s + i);
    SampleEntry e;
    e.t = static_cast<int64_t>(static_cast<uint32_t>(v.x)) | (static_cast<int64_t>(v.y) << 32);
    e.idx = static_cast<uint32_t>(v.z);
    e.pad = 0;
    return e;
#else
    return s[i];
#endif
}

__host__ __device__ __forceinline__ void StoreEntry(SampleEntry *s, uint32_t i, const SampleEntry &e) {
#ifdef __CUDA_ARCH__
    *reinterpret_cast<int4 *>(s + i) = make_int4(static_cast<int>(static_cast<uint32_t>(e.t)),
                                                 static_cast<int>(e.t >> 32), static_cast<int>(e.idx), 0);
#else
    s[i] = e;
#endif
}

// Sift-up of `value` from `hole` towards `top` in a max-heap ordered by time (the standard library's push-heap step).
__host__ __device__ __forceinline__ void PushHeap(SampleEntry *s, uint32_t hole, uint32_t top, const SampleEntry &value) {
    while (hole > top) {
        const uint32_t parent = (hole - 1) / 2;
        const SampleEntry above = LoadEntry(s, parent);
        if (!(above.t < value.t)) break;
        StoreEntry(s, hole, above);
        hole = parent;
    }
    StoreEntry(s, hole, value);
}

// The hole at `hole` sinks to a leaf along the larger children (the right child unless it is smaller than the
// left), then `value` is sifted up from there: the standard library's adjust-heap step.
__host__ __device__ __forceinline__ void AdjustHeap(SampleEntry *s, uint32_t hole, uint32_t len, const SampleEntry &value) {
    const uint32_t top = hole;
    uint32_t child = hole;
    while (child < (len - 1) / 2) {
        child = 2 * (child + 1);
        const SampleEntry right = LoadEntry(s, child), left = LoadEntry(s, child - 1);
        const bool take_left = right.t < left.t;
        if (take_left) --child;
        StoreEntry(s, hole, take_left ? left : right);
        hole = child;
    }
    if ((len & 1u) == 0 && child == (len - 2) / 2) {
        child = 2 * (child + 1);
        StoreEntry(s, hole, LoadEntry(s, child - 1));
        hole = child - 1;
    }
    PushHeap(s, hole, top, value);
}

__host__ __device__ __forceinline__ void MakeHeap(SampleEntry *s, uint32_t k) {
    if (k < 2) return;
    uint32_t parent = (k - 2) / 2;
    while (true) {
        AdjustHeap(s, parent, k, LoadEntry(s, parent));
        if (parent == 0) break;
        --parent;
    }
}

__host__ __device__ __forceinline__ void SortHeap(SampleEntry *s, uint32_t k) {
    for (uint32_t last = k; last > 1;) {
        --last;
        const SampleEntry value = LoadEntry(s, last);
        StoreEntry(s, last, LoadEntry(s, 0));
        AdjustHeap(s, 0, last, value);
    }
}

// std::partial_sort(first, first + k, first + n) by time: make-heap over the first k, heap-select (an element older
// than the heap's top takes its place), sort-heap.  One thread, as the algorithm is written.
__host__ __device__ __forceinline__ void PartialSortByTime(SampleEntry *s, uint32_t k, uint32_t n) {
    if (k == 0) return;
    MakeHeap(s, k);
    for (uint32_t i = k; i < n; ++i) {
        const SampleEntry value = LoadEntry(s, i);
        if (value.t < s[0].t) {
            StoreEntry(s, i, LoadEntry(s, 0));
            AdjustHeap(s, 0, k, value);
        }
    }
    SortHeap(s, k);
}

#ifdef __CUDACC__
// ---- the same heap steps, shared by the lanes of a warp (heaps of up to kWarpHeapMax entries).
// What makes a sift slow in one lane is that every level waits for the level above: load two children, compare,
// store, next address.  Which child is the larger one does not depend on the value being sifted, so that answer is
// kept, for every inner node, as one bit of a 64-bit word all lanes hold (`choice`: 1 = the left child, i.e. the
// right one is smaller).  A sift then is: (1) every lane follows the bits from the hole to a leaf - registers only -
// and lane l keeps the l-th position of that path; (2) lane l loads the entry one step further down; a ballot finds
// where the new value stops on its way back up (the standard library's adjust-heap lets the hole sink to a leaf and
// pushes the value up from there, passing entries that are smaller); (3) the entries above that point move up one
// position, the value goes in, and the positions below stay as they were; (4) the bits of the nodes whose children
// changed are put right.  The array ends up exactly as the one-lane routines above leave it.
constexpr uint32_t kWarpHeapMax = 128;

struct WarpHeap {
    SampleEntry *s;
    uint64_t choice;
    uint32_t lane;

    __device__ __forceinline__ bool LeftIsLarger(uint32_t node) const { return s[2 * node + 2].t < s[2 * node + 1].t; }

    // the bits of all inner nodes of a heap of `len` entries, from the array as it is
    __device__ __forceinline__ void InitChoice(uint32_t len) {
        uint32_t lo = 0, hi = 0;
        for (uint32_t node = lane; 2 * node + 2 < len; node += 32) {
            if (LeftIsLarger(node)) {
                if (node < 32) {
                    lo |= 1u << node;
                } else {
                    hi |= 1u << (node - 32);
                }
            }
        }
        lo = __reduce_or_sync(0xffffffffu, lo);
        hi = __reduce_or_sync(0xffffffffu, hi);
        choice = static_cast<uint64_t>(lo) | (static_cast<uint64_t>(hi) << 32);
    }

    // AdjustHeap(s, hole, len, value) above, all lanes; value is the same in all lanes
    __device__ __forceinline__ void Adjust(uint32_t hole, uint32_t len, int64_t v_t, uint32_t v_idx) {
        const uint32_t full = 0xffffffffu;
        // (1) the path: p_0 = hole, then the larger child each time; lane l keeps p_l, depth = index of the last
        uint32_t mine = hole, child = hole, depth = 0;
        while (child < (len - 1) / 2) {
            child = 2 * child + 2 - static_cast<uint32_t>((choice >> child) & 1ull);
            ++depth;
            if (depth == lane) mine = child;
        }
        if ((len & 1u) == 0 && child == (len - 2) / 2) {  // a node with a left child only
            child = 2 * child + 1;
            ++depth;
            if (depth == lane) mine = child;
        }
        // (2) what sits one step further down, and where the value stops on its way back up
        const uint32_t below = __shfl_down_sync(full, mine, 1);
        SampleEntry e;
        e.t = 0, e.idx = 0, e.pad = 0;
        if (lane < depth) e = LoadEntry(s, below);
        const uint32_t stays = __ballot_sync(full, lane < depth && !(e.t < v_t));  // entries the value does not pass
        const uint32_t stop = stays == 0 ? 0u : 32u - static_cast<uint32_t>(__clz(stays));  // the value ends at p_stop
        __syncwarp();
        // (3) entries above the stop move up one position; the value goes in
        if (lane < stop) {
            StoreEntry(s, mine, e);
        } else if (lane == stop) {
            SampleEntry v;
            v.t = v_t, v.idx = v_idx, v.pad = 0;
            StoreEntry(s, mine, v);
        }
        __syncwarp();
        // (4) the bits of the nodes whose children changed: p_0 .. p_{stop-1}, and the parent of p_0
        uint32_t node = 0xFFFFFFFFu;
        if (lane < stop) {
            node = mine;
        } else if (lane == 31 && hole > 0) {
            node = (hole - 1) / 2;
        }
        uint32_t set_lo = 0, set_hi = 0, clr_lo = 0, clr_hi = 0;
        if (node != 0xFFFFFFFFu && 2 * node + 2 < len) {
            const bool left = LeftIsLarger(node);
            if (node < 32) {
                clr_lo = 1u << node;
                set_lo = left ? clr_lo : 0u;
            } else {
                clr_hi = 1u << (node - 32);
                set_hi = left ? clr_hi : 0u;
            }
        }
        set_lo = __reduce_or_sync(full, set_lo);
        set_hi = __reduce_or_sync(full, set_hi);
        clr_lo = __reduce_or_sync(full, clr_lo);
        clr_hi = __reduce_or_sync(full, clr_hi);
        const uint64_t clr = static_cast<uint64_t>(clr_lo) | (static_cast<uint64_t>(clr_hi) << 32);
        const uint64_t set = static_cast<uint64_t>(set_lo) | (static_cast<uint64_t>(set_hi) << 32);
        choice = (choice & ~clr) | set;
    }

    // the value at position i, read by lane 0 and handed to all lanes
    __device__ __forceinline__ void Fetch(uint32_t i, int64_t *t, uint32_t *idx) const {
        const SampleEntry e = LoadEntry(s, i);  // every lane reads the same entry: a broadcast
        *t = e.t;
        *idx = e.idx;
    }
};

// Heap-select with shared sifts: the heap over s[0, k) is made already; every sample of s[k, n) that is older than
// the heap's top takes its place, in order.  (Measured: a shared sift costs about as much as a one-lane sift of the
// sort-heap phase, where the value stays near the bottom, and clearly less than one of this phase, where the value
// climbs back up several levels - so make-heap and sort-heap keep the one-lane routines.)
__device__ __forceinline__ void HeapSelectShared(SampleEntry *s, uint32_t k, uint32_t n, uint32_t lane) {
    WarpHeap heap{s, 0ull, lane};
    int64_t v_t;
    uint32_t v_idx;
    heap.InitChoice(k);
    for (uint32_t base = k; base < n; base += 32) {
        const uint32_t i = base + lane;
        const int64_t mine = i < n ? s[i].t : 0;
        uint32_t below = __ballot_sync(0xffffffffu, i < n && mine < s[0].t);
        while (below != 0) {
            const uint32_t j = base + static_cast<uint32_t>(__ffs(below)) - 1u;
            below &= below - 1u;
            heap.Fetch(j, &v_t, &v_idx);
            if (!(v_t < s[0].t)) continue;  // the top has got older meanwhile
            __syncwarp();
            if (lane == 0) StoreEntry(s, j, LoadEntry(s, 0));
            __syncwarp();
            heap.Adjust(0, k, v_t, v_idx);
        }
    }
    __syncwarp();
}

// The same for a warp: the heap steps stay lane 0's, in the algorithm's order, but the search for the samples
// that are older than the heap's top - most are not - is a ballot over 32 samples at a time.  The top only gets
// older, so a sample that fails the test once is out for good; lane 0 visits the ones that passed in their order
// and tests each again against the top of that moment, exactly as the loop above does.
__device__ __forceinline__ void PartialSortByTimeWarp(SampleEntry *s, uint32_t k, uint32_t n, uint32_t lane) {
    if (k == 0) return;
    if (lane == 0) MakeHeap(s, k);
    __syncwarp();
    if (k >= 32 && k <= kWarpHeapMax) {  // deep enough for the shared sift to pay, small enough for its word of bits
        HeapSelectShared(s, k, n, lane);
        if (lane == 0) SortHeap(s, k);
        __syncwarp();
        return;
    }
    for (uint32_t base = k; base < n; base += 32) {
        const uint32_t i = base + lane;
        const int64_t mine = i < n ? s[i].t : 0;
        uint32_t below = __ballot_sync(0xffffffffu, i < n && mine < s[0].t);
        if (below == 0) continue;
        if (lane == 0) {
            while (below != 0) {
                const uint32_t j = base + static_cast<uint32_t>(__ffs(below)) - 1u;
                below &= below - 1u;
                const SampleEntry value = LoadEntry(s, j);
                if (value.t < s[0].t) {
                    StoreEntry(s, j, LoadEntry(s, 0));
                    AdjustHeap(s, 0, k, value);
                }
            }
        }
        __syncwarp();
    }
    if (lane == 0) SortHeap(s, k);
    __syncwarp();
}
#endif

// One warp's shared memory for a round of evictions.
struct SamplingScratch {
    SampleEntry sample[kMaxSample];  // the sampled blocks (the raw draws in .t before that)
    int64_t tail_ts[kMaxBatch];      // ts / blk of the last entries of the vector, [j] = index size - 1 - j
    uint32_t v_id[kMaxBatch], v_at[kMaxBatch];  // the round's victims: block id, current index
    uint32_t tail_blk[kMaxBatch];
    uint16_t tail_victim[kMaxBatch];  // which victim the block at that tail position is (kNoVictim: none)
};
constexpr uint16_t kNoVictim = 0xFFFFu;

// RandomLruEvictionPolicy::EvictBlocks(count) (random_lru.cc:38-103) on a block vector of `held` entries; all lanes,
// returns how many blocks went (the caller keeps the vector's length).  *rng is the generator's state, in shared
// memory.
__device__ __forceinline__ uint32_t SamplingEvictRound(SamplingScratch &sc, uint32_t *pos, uint32_t *blk, int64_t *ts,
                                                       int64_t held, uint64_t *rng, uint32_t sampling_size,
                                                       int64_t count, uint32_t lane) {
    if (held == 0) return 0u;
    const uint32_t n_blocks = static_cast<uint32_t>(held);
    const uint32_t want = count < held ? static_cast<uint32_t>(count) : n_blocks;  // total_to_evict
    const uint32_t n_sample = sampling_size < n_blocks ? sampling_size : n_blocks;
    const uint32_t k = want < n_sample ? want : n_sample;
    // the draws: the first 32 in sequence (lane 0), the rest by every lane jumping 32 draws at a time; then their
    // modulo and the sampled blocks' times (all lanes)
    if (lane == 0) {
        uint64_t x = *rng;
        const uint32_t head = n_sample < 32u ? n_sample : 32u;
        for (uint32_t i = 0; i < head; ++i) {
            x = XorShiftStep(x);
            sc.sample[i].t = static_cast<int64_t>(x);
        }
    }
    __syncwarp();
    {
        uint64_t x = lane < n_sample ? static_cast<uint64_t>(sc.sample[lane].t) : 0ull;
        for (uint32_t i = lane + 32u; i < n_sample; i += 32u) {
            x = Jump32(x);
            sc.sample[i].t = static_cast<int64_t>(x);
        }
    }
    __syncwarp();
    if (lane == 0) *rng = static_cast<uint64_t>(sc.sample[n_sample - 1].t);  // the state after the last draw
    __syncwarp();
    for (uint32_t i0 = lane; i0 < n_sample; i0 += 128) {  // four sampled times in flight per lane
        uint32_t at[4];
        int64_t seen[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t i = i0 + 32u * u;
            at[u] = i < n_sample ? static_cast<uint32_t>(static_cast<uint64_t>(sc.sample[i].t) % n_blocks) : 0u;
            seen[u] = i < n_sample ? ts[at[u]] : 0;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t i = i0 + 32u * u;
            if (i < n_sample) StoreEntry(sc.sample, i, SampleEntry{seen[u], at[u], 0u});
        }
    }
    __syncwarp();
    PartialSortByTimeWarp(sc.sample, k, n_sample, lane);
    // the victims as blocks (resolved before the first removal, as the reference resolves them), and the tail
    // of the vector, which the removals read
    const uint32_t n_tail = k < n_blocks ? k : n_blocks;
    for (uint32_t i = lane; i < k; i += 32) {
        sc.v_at[i] = sc.sample[i].idx;
        sc.v_id[i] = blk[sc.sample[i].idx];
    }
    for (uint32_t i = lane; i < n_tail; i += 32) {
        sc.tail_blk[i] = blk[n_blocks - 1 - i];
        sc.tail_ts[i] = ts[n_blocks - 1 - i];
        sc.tail_victim[i] = kNoVictim;
    }
    __syncwarp();
    // A block sampled twice is removed once: every later sample of an index is struck out before the removals start
    // (the reference finds it gone when its turn comes).  Then, for the last n_tail positions of the vector - the only
    // ones a removal ever moves a block away from - which victim sits there.
    for (uint32_t v = lane; v < k; v += 32) {
        const uint32_t at = sc.sample[v].idx;
        bool again = false;
        for (uint32_t u = 0; u < v && !again; ++u) again = sc.sample[u].idx == at;
        if (again) sc.v_at[v] = kNotCached;
    }
    __syncwarp();
    for (uint32_t v = lane; v < k; v += 32) {
        const uint32_t at = sc.v_at[v];
        if (at != kNotCached && n_blocks - 1 - at < n_tail) sc.tail_victim[n_blocks - 1 - at] = static_cast<uint16_t>(v);
    }
    __syncwarp();
    // The removals, swap-and-pop in the victims' order (random_lru.cc:84-103): one lane, no look at the other
    // victims - when the block that sits last is itself a later victim, the table above says so and its index follows.
    uint32_t evicted = 0;
    if (lane == 0) {
        uint32_t size = n_blocks;
        for (uint32_t i = 0; i < k && evicted < want; ++i) {
            const uint32_t at = sc.v_at[i];
            if (at == kNotCached) continue;  // sampled twice: removed already
            const uint32_t id = sc.v_id[i];
            const uint32_t last = size - 1;
            if (at != last) {
                const uint32_t from_end = n_blocks - 1 - last;
                const uint32_t moved = sc.tail_blk[from_end];  // the block that sits last now
                const int64_t moved_t = sc.tail_ts[from_end];
                const uint16_t rider = sc.tail_victim[from_end];  // the later victim that block is, if any
                blk[at] = moved;
                ts[at] = moved_t;
                pos[moved] = at;
                if (rider != kNoVictim) sc.v_at[rider] = at;
                if (n_blocks - 1 - at < n_tail) {  // the staged tail follows
                    sc.tail_blk[n_blocks - 1 - at] = moved;
                    sc.tail_ts[n_blocks - 1 - at] = moved_t;
                    sc.tail_victim[n_blocks - 1 - at] = rider;
                }
            }
            pos[id] = kNotCached;
            --size;
            ++evicted;
        }
    }
    evicted = __shfl_sync(0xffffffffu, evicted, 0);
    __syncwarp();
    return evicted;
}

// One trace of a sampling instance: its leading cached blocks are hits and take the trace's time
// (OnBlockAccessed), then - unless the trace only reads - its missing blocks are appended in key order
// (OnBlockWritten).  ids / mask_bits point at the trace's first key (mask_bits may be null); size is the length of the
// block vector before the trace.  All lanes; the counts come back equal in all lanes.
// type: 0 DialogTurn (InsertWithQuery), 1 GetLocation (PrefixQuery), 2 WriteCache (InsertOnly).
struct SamplingTraceCounts {
    int32_t ext, inte, wr;
};

__device__ __forceinline__ SamplingTraceCounts SamplingReplayTrace(const uint32_t *ids, const uint8_t *mask_bits,
                                                                   int64_t n, uint8_t ty, int64_t skip, int64_t now,
                                                                   uint32_t *pos, uint32_t *blk, int64_t *ts,
                                                                   int64_t size, uint32_t lane) {
    const uint32_t lt = (1u << lane) - 1u;
    SamplingTraceCounts c{0, 0, 0};
    bool alive = ty != 2;  // still inside the leading run of cached blocks
    for (int64_t base = 0; base < n; base += 32) {
        const int64_t i = base + lane;
        const bool have = i < n;
        const uint32_t id = have ? ids[i] : 0u;
        const uint32_t cur = have ? pos[id] : kNotCached;
        const uint32_t in_range = __ballot_sync(0xffffffffu, have);
        const uint32_t cached = __ballot_sync(0xffffffffu, have && cur != kNotCached);
        const uint32_t miss = in_range & ~cached;
        uint32_t touch = 0;  // leading cached blocks: hits, their access time becomes the trace's
        if (alive) {
            touch = miss != 0 ? cached & ((1u << (__ffs(miss) - 1)) - 1u) : cached;
            const uint32_t masked = __ballot_sync(
                0xffffffffu, i < skip || (ty == 1 && mask_bits != nullptr && have && mask_bits[i] != 0));
            c.ext += __popc(touch & ~masked);
            c.inte += __popc(touch & masked);
            if (miss != 0) alive = false;
        }
        const uint32_t write = ty == 1 ? 0u : miss;  // then the missing blocks are written, in order
        if ((touch >> lane) & 1u) {
            ts[cur] = now;
        } else if ((write >> lane) & 1u) {
            const int64_t at = size + __popc(write & lt);
            blk[at] = id;
            ts[at] = now;
            pos[id] = static_cast<uint32_t>(at);
        }
        const uint32_t n_write = __popc(write);
        size += n_write;
        c.wr += static_cast<int32_t>(n_write);
        __syncwarp();
        if (ty == 1 && !alive) break;
    }
    __syncwarp();
    return c;
}

}  // namespace
}  // namespace kvcm
