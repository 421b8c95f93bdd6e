// Optimizer trace replay with LRU eviction, for a sweep of cache quotas at once (sm_100a).
//
// Stands in for OptimizerRunner::RunTraces (kv_cache_manager/optimizer/manager/optimizer_runner.cc:29-215)
// over RadixTreeIndex (kv_cache_manager/optimizer/index/radix_tree_index.cc:19-392) with the "lru"
// eviction policy (kv_cache_manager/optimizer/eviction_policy/lru.cc:6-49) and the quota check after
// every write (OptIndexerManager::CheckAndEvict, kv_cache_manager/optimizer/manager/indexer_manager.cc:55-90;
// OptEvictionManager::EvictByInstanceRough / EvictByInstancePrecise / GetExcessUsageForInstanceInGroup,
// kv_cache_manager/optimizer/manager/eviction_manager.cc:148-266), one instance per group; groups of several
// instances that share the quota (EvictByGroupRough, :86-146) have a kernel of their own further down.
//
// With eviction the replay of ONE configuration is sequential: what trace t hits depends on what
// the traces before it touched and evicted.  The reference's tradeoff-curve scripts run the same
// trace once per (quota, policy) point (kv_cache_manager/optimizer/analysis/script/
// optimizer_analysis_utils.py:95-144,181-207,278-330); those runs are independent, and that is the
// parallel axis here: one warp per configuration, all walking the same trace.
//
// Per configuration the tree collapses to per-key state, because keys are prefix-unique chained
// hashes and because of how the reference orders its recency updates: within one trace it first
// moves the leading cached blocks to the front (in order, stopping at the first evicted or absent
// block) and then writes the missing blocks (in order); blocks that are cached but lie behind the
// first miss are not touched.  So:
//   stamp[key]  0 = not cached, else the sequence number of its last write or access;
//   queue       every write or access appends (key, stamp); an entry is live while it still
//               carries the key's current stamp.  The recency list of the reference is the
//               live entries in queue order, its tail is the oldest live entry.
// A trace is handled 32 keys at a time: ballot for the first miss, ranks from the ballot give
// the stamps and queue positions.  Eviction pops live entries from the head of the queue.
// Keys are renamed to dense ids 0..D-1 once, for all configurations, so that per-configuration
// state is two flat arrays (4 + 8 bytes per key occurrence of the trace).
#include "kvcm_common.cuh"
#include "replay_ids.cuh"

namespace kvcm {
namespace {

constexpr int kEvictWindows = 4;

__global__ void LruInitKernel(IdTable t, uint32_t *stamps, uint64_t n_stamps) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    const uint64_t first = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (uint64_t i = first; i <= t.mask; i += stride) t.slots[i] = make_ulonglong2(kEmptyKey, ~0ull);
    for (uint64_t i = first; i < n_stamps; i += stride) stamps[i] = 0u;
    if (first == 0) {
        t.cells[0] = 0ull;
        t.cells[1] = ~0ull;
    }
}

struct LruSweep {
    const uint32_t *ids;
    const int64_t *key_off;
    const uint8_t *type;
    const int64_t *mask_off;
    const uint8_t *mask_bits;  // optional, per key: 1 = masked (a BlockMaskVector), on top of mask_off
    const int64_t *quota;
    uint32_t *stamps;  // [n_configs][n_keys]
    uint2 *queue;      // [n_configs][n_keys]
    int32_t *ext_hit, *int_hit, *written;  // per trace; all four may be null when only totals are wanted
    int64_t *cache_blocks;
    int64_t *totals;  // [n_configs][4]: external hits, internal hits, written blocks, cached blocks at the end
    int64_t n_keys;
    int32_t n_traces;
    int32_t n_configs;
    int32_t evict_batch;
    int32_t precise;
};

// type: 0 DialogTurn (InsertWithQuery), 1 GetLocation (PrefixQuery), 2 WriteCache (InsertOnly).
__global__ void __launch_bounds__(32) LruSweepKernel(const LruSweep p) {
    const int32_t cfg = blockIdx.x;
    const uint32_t lane = LaneId();
    const uint32_t lt = (1u << lane) - 1u;
    uint32_t *stamp = p.stamps + static_cast<int64_t>(cfg) * p.n_keys;
    uint2 *queue = p.queue + static_cast<int64_t>(cfg) * p.n_keys;
    const int64_t quota = p.quota[cfg];
    const int64_t out0 = static_cast<int64_t>(cfg) * p.n_traces;
    uint32_t counter = 0;  // last stamp handed out
    int64_t head = 0, tail = 0, resident = 0;
    int64_t sum_ext = 0, sum_int = 0, sum_wr = 0;

    // What a trace reads before it touches any state (its extent, kind and the ids of its first 32
    // keys) is fetched one trace ahead, its extent two traces ahead, so that the only load a trace
    // waits for is the one that depends on the traces before it: stamp[id].
    auto extent = [&](int32_t t, int64_t *beg, int64_t *n, uint8_t *ty, int64_t *skip) {
        if (t < p.n_traces) {
            *beg = p.key_off[t];
            *n = p.key_off[t + 1] - *beg;
            *ty = p.type[t];
            *skip = (*ty == 1 && p.mask_off != nullptr) ? p.mask_off[t] : 0;
        } else {
            *beg = 0, *n = 0, *ty = 1, *skip = 0;
        }
    };
    int64_t beg, n, skip, beg1, n1, skip1;
    uint8_t ty, ty1;
    extent(0, &beg, &n, &ty, &skip);
    extent(1, &beg1, &n1, &ty1, &skip1);
    uint32_t first_id = lane < n ? p.ids[beg + lane] : 0u;

    for (int32_t t = 0; t < p.n_traces; ++t) {
        const uint32_t next_first_id = lane < n1 ? p.ids[beg1 + lane] : 0u;
        int64_t beg2, n2, skip2;
        uint8_t ty2;
        extent(t + 2, &beg2, &n2, &ty2, &skip2);
        int32_t ext = 0, inte = 0, wr = 0;
        bool alive = ty != 2;  // still inside the leading run of cached blocks
        for (int64_t base = 0; base < n; base += 32) {
            const int64_t i = base + lane;
            const bool have = i < n;
            const uint32_t id = base == 0 ? first_id : (have ? p.ids[beg + i] : 0u);
            const uint32_t cur = have ? stamp[id] : 0u;
            const uint32_t in_range = __ballot_sync(0xffffffffu, have);
            const uint32_t cached = __ballot_sync(0xffffffffu, have && cur != 0u);
            const uint32_t miss = in_range & ~cached;
            uint32_t touch = 0;  // leading cached blocks: hits, moved to the front in order
            if (alive) {
                touch = miss != 0 ? cached & ((1u << (__ffs(miss) - 1)) - 1u) : cached;
                const uint32_t masked = __ballot_sync(
                    0xffffffffu, i < skip || (ty == 1 && p.mask_bits != nullptr && have && p.mask_bits[beg + i] != 0));
                ext += __popc(touch & ~masked);
                inte += __popc(touch & masked);
                if (miss != 0) alive = false;
            }
            const uint32_t write = ty == 1 ? 0u : miss;  // then the missing blocks are written, in order
            const uint32_t n_touch = __popc(touch), n_write = __popc(write);
            if ((touch >> lane) & 1u) {
                const uint32_t r = __popc(touch & lt);
                stamp[id] = counter + 1 + r;
                queue[tail + r] = make_uint2(id, counter + 1 + r);
            } else if ((write >> lane) & 1u) {
                const uint32_t r = n_touch + __popc(write & lt);
                stamp[id] = counter + 1 + r;
                queue[tail + r] = make_uint2(id, counter + 1 + r);
            }
            counter += n_touch + n_write;
            tail += n_touch + n_write;
            resident += n_write;
            wr += static_cast<int32_t>(n_write);
            __syncwarp();
            if (ty == 1 && !alive) break;
        }
        if (ty != 1 && resident > quota) {
            // CheckAndEvict: whole batches until the excess is covered, or exactly the excess.
            const int64_t excess = resident - quota;
            int64_t need = excess;
            if (p.precise == 0) {
                const int64_t batches = (excess + p.evict_batch - 1) / p.evict_batch;
                need = batches * p.evict_batch;
                if (need > resident) need = resident;
            }
            // The queue is read kEvictWindows x 32 entries at a time: the entries, then their stamps, are
            // independent loads, so a round of ~100 evictions costs two memory round trips, not eight.
            while (need > 0 && head < tail) {
                uint2 e[kEvictWindows];
                bool live[kEvictWindows];
#pragma unroll
                for (int u = 0; u < kEvictWindows; ++u) {
                    const int64_t j = head + u * 32 + lane;
                    e[u] = j < tail ? queue[j] : make_uint2(0u, 0u);
                }
#pragma unroll
                for (int u = 0; u < kEvictWindows; ++u) {
                    const int64_t j = head + u * 32 + lane;
                    live[u] = j < tail && stamp[e[u].x] == e[u].y;
                }
                int64_t advance = 0;
#pragma unroll
                for (int u = 0; u < kEvictWindows; ++u) {
                    const int64_t left = tail - (head + u * 32);  // entries from this window on
                    if (need > 0 && left > 0) {
                        const uint32_t lives = __ballot_sync(0xffffffffu, live[u]);
                        uint32_t take = lives;
                        int64_t step = left < 32 ? left : 32;
                        if (static_cast<int64_t>(__popc(lives)) > need) {
                            // keep only the first `need` live entries of this window; stop right behind the last one
                            const bool mine = live[u] && static_cast<int64_t>(__popc(lives & lt)) < need;
                            take = __ballot_sync(0xffffffffu, mine);
                            step = 32 - __clz(take);
                        }
                        if ((take >> lane) & 1u) stamp[e[u].x] = 0u;
                        const uint32_t n_take = __popc(take);
                        need -= n_take;
                        resident -= n_take;
                        advance += step;
                    }
                }
                head += advance;
                __syncwarp();
            }
        }
        if (lane == 0 && p.ext_hit != nullptr) {
            p.ext_hit[out0 + t] = ext;
            p.int_hit[out0 + t] = inte;
            p.written[out0 + t] = wr;
            p.cache_blocks[out0 + t] = resident;
        }
        sum_ext += ext;
        sum_int += inte;
        sum_wr += wr;
        beg = beg1, n = n1, ty = ty1, skip = skip1, first_id = next_first_id;
        beg1 = beg2, n1 = n2, ty1 = ty2, skip1 = skip2;
    }
    if (lane == 0 && p.totals != nullptr) {
        int64_t *tot = p.totals + static_cast<int64_t>(cfg) * 4;
        tot[0] = sum_ext;
        tot[1] = sum_int;
        tot[2] = sum_wr;
        tot[3] = resident;
    }
}

// ---- several instances that share one group quota -------------------------------------------------------------
// OptEvictionManager::EvictByGroupRough / EvictByInstanceRough / EvictByInstancePrecise over the summed usage of the
// group (kv_cache_manager/optimizer/manager/eviction_manager.cc:86-266).  Every instance has a tree and a recency list
// of its own (kv_cache_manager/optimizer/manager/optimizer_manager.cc:66-99), here a region of the queue per
// instance; ids are unique over (instance, key), so the per-key stamps need no instance.
struct LruGroup {
    const int32_t *trace_inst;  // per trace, 0 .. n_instances-1
    const int64_t *queue_base;  // [n_instances + 1]: where each instance's region of the queue starts
    int64_t *inst_blocks;       // optional, [n_configs][n_instances]: usage per instance at the end
    int64_t *inst_blocks_trace;  // optional, [n_configs][n_traces][n_instances]: usage of every instance after each trace
    int32_t n_instances;
    int32_t mode;               // 1 group rough, 2 instance rough, 3 instance precise
};

__global__ void __launch_bounds__(32) LruGroupSweepKernel(const LruSweep p, const LruGroup g) {
    extern __shared__ int64_t per_inst[];
    const int32_t K = g.n_instances;
    int64_t *head = per_inst, *tail = per_inst + K, *cached = per_inst + 2 * K, *take = per_inst + 3 * K;
    const int32_t cfg = blockIdx.x;
    const uint32_t lane = LaneId();
    const uint32_t lt = (1u << lane) - 1u;
    uint32_t *stamp = p.stamps + static_cast<int64_t>(cfg) * p.n_keys;
    uint2 *queue = p.queue + static_cast<int64_t>(cfg) * p.n_keys;
    const int64_t quota = p.quota[cfg];
    const int64_t out0 = static_cast<int64_t>(cfg) * p.n_traces;
    uint32_t counter = 0;
    int64_t resident = 0;  // of the whole group
    int64_t sum_ext = 0, sum_int = 0, sum_wr = 0;
    for (int32_t j = lane; j < K; j += 32) {
        head[j] = tail[j] = g.queue_base[j];
        cached[j] = 0;
    }
    __syncwarp();

    // As in the single-instance kernel: a trace's extent, kind, instance and first 32 ids are fetched one trace
    // ahead (the extent two ahead), so that the load a trace waits for is stamp[id].
    auto extent = [&](int32_t t, int64_t *beg, int64_t *n, uint8_t *ty, int64_t *skip, int32_t *who) {
        if (t < p.n_traces) {
            *beg = p.key_off[t];
            *n = p.key_off[t + 1] - *beg;
            *ty = p.type[t];
            *skip = (*ty == 1 && p.mask_off != nullptr) ? p.mask_off[t] : 0;
            *who = g.trace_inst[t];
            if (*who < 0 || *who >= K) {  // counted by LruGroupExtentKernel; its keys have no ids: an empty trace
                *who = 0;
                *n = 0;
            }
        } else {
            *beg = 0, *n = 0, *ty = 1, *skip = 0, *who = 0;
        }
    };
    int64_t beg, n, skip, beg1, n1, skip1;
    uint8_t ty, ty1;
    int32_t me, me1;
    extent(0, &beg, &n, &ty, &skip, &me);
    extent(1, &beg1, &n1, &ty1, &skip1, &me1);
    uint32_t first_id = lane < n ? p.ids[beg + lane] : 0u;

    for (int32_t t = 0; t < p.n_traces; ++t) {
        const uint32_t next_first_id = lane < n1 ? p.ids[beg1 + lane] : 0u;
        int64_t beg2, n2, skip2;
        uint8_t ty2;
        int32_t me2;
        extent(t + 2, &beg2, &n2, &ty2, &skip2, &me2);
        int64_t my_tail = tail[me];
        int32_t ext = 0, inte = 0, wr = 0;
        bool alive = ty != 2;
        for (int64_t base = 0; base < n; base += 32) {
            const int64_t i = base + lane;
            const bool have = i < n;
            const uint32_t id = base == 0 ? first_id : (have ? p.ids[beg + i] : 0u);
            const uint32_t cur = have ? stamp[id] : 0u;
            const uint32_t in_range = __ballot_sync(0xffffffffu, have);
            const uint32_t hit = __ballot_sync(0xffffffffu, have && cur != 0u);
            const uint32_t miss = in_range & ~hit;
            uint32_t touch = 0;
            if (alive) {
                touch = miss != 0 ? hit & ((1u << (__ffs(miss) - 1)) - 1u) : hit;
                const uint32_t masked = __ballot_sync(
                    0xffffffffu, i < skip || (ty == 1 && p.mask_bits != nullptr && have && p.mask_bits[beg + i] != 0));
                ext += __popc(touch & ~masked);
                inte += __popc(touch & masked);
                if (miss != 0) alive = false;
            }
            const uint32_t write = ty == 1 ? 0u : miss;
            const uint32_t n_touch = __popc(touch), n_write = __popc(write);
            if ((touch >> lane) & 1u) {
                const uint32_t r = __popc(touch & lt);
                stamp[id] = counter + 1 + r;
                queue[my_tail + r] = make_uint2(id, counter + 1 + r);
            } else if ((write >> lane) & 1u) {
                const uint32_t r = n_touch + __popc(write & lt);
                stamp[id] = counter + 1 + r;
                queue[my_tail + r] = make_uint2(id, counter + 1 + r);
            }
            counter += n_touch + n_write;
            my_tail += n_touch + n_write;
            resident += n_write;
            wr += static_cast<int32_t>(n_write);
            __syncwarp();
            if (ty == 1 && !alive) break;
        }
        int64_t my_cached = cached[me] + wr;
        __syncwarp();
        if (lane == 0) {
            tail[me] = my_tail;
            cached[me] = my_cached;
        }
        __syncwarp();
        if (ty != 1 && resident > quota) {
            const int64_t excess = resident - quota;
            // How many blocks every instance loses.  The instances' lists are independent, so only the counts
            // depend on the order of the reference's rounds, and they follow from the usages alone.
            if (g.mode == 1) {
                if (lane == 0) {
                    for (int32_t j = 0; j < K; ++j) take[j] = 0;
                    int64_t total = 0;
                    while (total < excess) {
                        bool any = false;
                        for (int32_t j = 0; j < K; ++j) {  // a whole round even when the excess is covered midway
                            const int64_t left = cached[j] - take[j];
                            const int64_t got = left < p.evict_batch ? left : p.evict_batch;
                            if (got > 0) {
                                take[j] += got;
                                total += got;
                                any = true;
                            }
                        }
                        if (!any) break;
                    }
                }
            } else {
                int64_t need = excess;
                if (g.mode == 2) need = (excess + p.evict_batch - 1) / p.evict_batch * p.evict_batch;
                if (need > my_cached) need = my_cached;
                for (int32_t j = lane; j < K; j += 32) take[j] = j == me ? need : 0;
            }
            __syncwarp();
            const int32_t first = g.mode == 1 ? 0 : me, last = g.mode == 1 ? K : me + 1;
            for (int32_t j = first; j < last; ++j) {
                int64_t need = take[j];
                if (need == 0) continue;
                int64_t hd = head[j];
                const int64_t tl = tail[j];
                int64_t popped = 0;
                while (need > 0 && hd < tl) {
                    const int64_t q = hd + lane;
                    const uint2 e = q < tl ? queue[q] : make_uint2(0u, 0u);
                    const bool live = q < tl && stamp[e.x] == e.y;
                    const uint32_t lives = __ballot_sync(0xffffffffu, live);
                    uint32_t out = lives;
                    int64_t step = tl - hd < 32 ? tl - hd : 32;
                    if (static_cast<int64_t>(__popc(lives)) > need) {
                        const bool mine = live && static_cast<int64_t>(__popc(lives & lt)) < need;
                        out = __ballot_sync(0xffffffffu, mine);
                        step = 32 - __clz(out);
                    }
                    if ((out >> lane) & 1u) stamp[e.x] = 0u;
                    const int64_t n_out = __popc(out);
                    need -= n_out;
                    popped += n_out;
                    hd += step;
                    __syncwarp();
                }
                resident -= popped;
                if (j == me) my_cached -= popped;
                if (lane == 0) {
                    head[j] = hd;
                    cached[j] -= popped;
                }
                __syncwarp();
            }
        }
        if (lane == 0 && p.ext_hit != nullptr) {
            p.ext_hit[out0 + t] = ext;
            p.int_hit[out0 + t] = inte;
            p.written[out0 + t] = wr;
            p.cache_blocks[out0 + t] = my_cached;
        }
        if (g.inst_blocks_trace != nullptr) {  // ReadRecord::blocks_per_instance of the reference's result records
            __syncwarp();
            int64_t *row = g.inst_blocks_trace + (out0 + t) * K;
            for (int32_t j = lane; j < K; j += 32) row[j] = cached[j];
        }
        sum_ext += ext;
        sum_int += inte;
        sum_wr += wr;
        beg = beg1, n = n1, ty = ty1, skip = skip1, me = me1, first_id = next_first_id;
        beg1 = beg2, n1 = n2, ty1 = ty2, skip1 = skip2, me1 = me2;
    }
    if (lane == 0 && p.totals != nullptr) {
        int64_t *tot = p.totals + static_cast<int64_t>(cfg) * 4;
        tot[0] = sum_ext;
        tot[1] = sum_int;
        tot[2] = sum_wr;
        tot[3] = resident;
    }
    if (g.inst_blocks != nullptr) {
        for (int32_t j = lane; j < K; j += 32) g.inst_blocks[static_cast<int64_t>(cfg) * K + j] = cached[j];
    }
}

struct LruLayout {
    uint64_t table_off, ids_off, stamps_off, queue_off, total;
};

LruLayout LayoutFor(int64_t n_keys, int32_t n_configs) {
    auto up = [](uint64_t v) { return (v + 255u) & ~static_cast<uint64_t>(255u); };
    LruLayout l;
    const uint64_t nk = static_cast<uint64_t>(n_keys > 0 ? n_keys : 1);
    l.table_off = 256;
    l.ids_off = up(l.table_off + SlotsFor(n_keys) * sizeof(ulonglong2));
    l.stamps_off = up(l.ids_off + nk * sizeof(uint32_t));
    l.queue_off = up(l.stamps_off + nk * sizeof(uint32_t) * static_cast<uint64_t>(n_configs));
    l.total = up(l.queue_off + nk * sizeof(uint2) * static_cast<uint64_t>(n_configs));
    return l;
}

}  // namespace
}  // namespace kvcm

extern "C" {

int64_t kvcm_b200_replay_lru_workspace_bytes(int64_t n_keys_total, int32_t n_configs) {
    if (n_keys_total < 0 || n_keys_total >= (1ll << 32) - 1 || n_configs <= 0 || n_configs > 65535) return -1;
    return static_cast<int64_t>(kvcm::LayoutFor(n_keys_total, n_configs).total);
}

int32_t kvcm_b200_replay_lru(const int64_t *d_keys, const int64_t *d_key_off, const uint8_t *d_trace_type,
                             const int64_t *d_mask_off, const uint8_t *d_mask_bits, int32_t n_traces,
                             int64_t n_keys_total, const int64_t *d_quota_blocks, int32_t n_configs, int32_t evict_batch,
                             int32_t precise, void *d_workspace, int64_t workspace_bytes, int32_t *d_ext_hit, int32_t *d_int_hit,
                             int32_t *d_written, int64_t *d_cache_blocks, int64_t *d_totals, uint32_t *d_status,
                             kvcm_stream_t stream) {
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (n_traces < 0 || n_keys_total < 0 || n_configs <= 0 || evict_batch <= 0) return KVCM_EC_BADARGS;
    const int64_t need = kvcm_b200_replay_lru_workspace_bytes(n_keys_total, n_configs);
    if (need < 0) return KVCM_EC_OUT_OF_LIMIT;
    if (n_traces == 0) return KVCM_OK;
    const int per_trace = (d_ext_hit != nullptr) + (d_int_hit != nullptr) + (d_written != nullptr) +
                          (d_cache_blocks != nullptr);
    if (d_key_off == nullptr || d_trace_type == nullptr || d_quota_blocks == nullptr || d_workspace == nullptr ||
        (d_keys == nullptr && n_keys_total > 0) || (per_trace != 0 && per_trace != 4) ||
        (per_trace == 0 && d_totals == nullptr)) {
        return KVCM_ER_INVALID_ADDRESS;
    }
    if (reinterpret_cast<uintptr_t>(d_workspace) & 255u) return KVCM_ER_INVALID_ADDRESS;
    if (workspace_bytes < need) return KVCM_EC_NOSPC;
    const kvcm::LruLayout l = kvcm::LayoutFor(n_keys_total, n_configs);
    uint8_t *ws = static_cast<uint8_t *>(d_workspace);
    kvcm::IdTable t;
    t.cells = reinterpret_cast<unsigned long long *>(ws);
    t.slots = reinterpret_cast<ulonglong2 *>(ws + l.table_off);
    t.mask = kvcm::SlotsFor(n_keys_total) - 1;
    uint32_t *ids = reinterpret_cast<uint32_t *>(ws + l.ids_off);
    uint32_t *stamps = reinterpret_cast<uint32_t *>(ws + l.stamps_off);
    cudaStream_t s = kvcm::AsStream(stream);
    const int sms = kvcm::GetDeviceInfo().sm_count;
    const uint64_t n_stamps = static_cast<uint64_t>(n_keys_total) * static_cast<uint64_t>(n_configs);
    kvcm::LruInitKernel<<<sms * 8, 256, 0, s>>>(t, stamps, n_stamps);
    if (n_keys_total > 0) {
        kvcm::LruClaimIdsKernel<<<sms * 8, 256, 0, s>>>(t, d_keys, n_keys_total, d_status);
        kvcm::LruLookupIdsKernel<<<sms * 8, 256, 0, s>>>(t, d_keys, n_keys_total, ids);
    }
    kvcm::LruSweep p;
    p.ids = ids;
    p.key_off = d_key_off;
    p.type = d_trace_type;
    p.mask_off = d_mask_off;
    p.mask_bits = d_mask_bits;
    p.quota = d_quota_blocks;
    p.stamps = stamps;
    p.queue = reinterpret_cast<uint2 *>(ws + l.queue_off);
    p.ext_hit = d_ext_hit;
    p.int_hit = d_int_hit;
    p.written = d_written;
    p.cache_blocks = d_cache_blocks;
    p.totals = d_totals;
    p.n_keys = n_keys_total > 0 ? n_keys_total : 1;
    p.n_traces = n_traces;
    p.n_configs = n_configs;
    p.evict_batch = evict_batch;
    p.precise = precise;
    kvcm::LruSweepKernel<<<static_cast<unsigned>(n_configs), 32, 0, s>>>(p);
    return kvcm::LaunchStatus();
}

}  // extern "C"

extern "C" {

int64_t kvcm_b200_replay_lru_group_workspace_bytes(int64_t n_keys_total, int32_t n_configs, int32_t n_instances) {
    const int64_t base = kvcm_b200_replay_lru_workspace_bytes(n_keys_total, n_configs);
    if (base < 0 || n_instances <= 0 || n_instances > KVCM_B200_REPLAY_GROUP_MAX_INSTANCES) return -1;
    return base + ((static_cast<int64_t>(n_instances) + 1) * 8 + 255) / 256 * 256;
}

int32_t kvcm_b200_replay_lru_group(const int64_t *d_keys, const int64_t *d_key_off, const uint8_t *d_trace_type,
                                   const int64_t *d_mask_off, const uint8_t *d_mask_bits,
                                   const int32_t *d_trace_instance, int32_t n_instances, int32_t n_traces,
                                   int64_t n_keys_total, const int64_t *d_quota_blocks, int32_t n_configs,
                                   int32_t evict_batch, int32_t eviction_mode, void *d_workspace,
                                   int64_t workspace_bytes, int32_t *d_ext_hit, int32_t *d_int_hit, int32_t *d_written,
                                   int64_t *d_cache_blocks, int64_t *d_totals, int64_t *d_instance_blocks,
                                   uint32_t *d_status, kvcm_stream_t stream) {
    return kvcm_b200_replay_lru_group_records(d_keys, d_key_off, d_trace_type, d_mask_off, d_mask_bits, d_trace_instance,
                                              n_instances, n_traces, n_keys_total, d_quota_blocks, n_configs,
                                              evict_batch, eviction_mode, d_workspace, workspace_bytes, d_ext_hit,
                                              d_int_hit, d_written, d_cache_blocks, d_totals, d_instance_blocks, nullptr,
                                              d_status, stream);
}

int32_t kvcm_b200_replay_lru_group_records(const int64_t *d_keys, const int64_t *d_key_off, const uint8_t *d_trace_type,
                                           const int64_t *d_mask_off, const uint8_t *d_mask_bits,
                                           const int32_t *d_trace_instance, int32_t n_instances, int32_t n_traces,
                                           int64_t n_keys_total, const int64_t *d_quota_blocks, int32_t n_configs,
                                           int32_t evict_batch, int32_t eviction_mode, void *d_workspace,
                                           int64_t workspace_bytes, int32_t *d_ext_hit, int32_t *d_int_hit,
                                           int32_t *d_written, int64_t *d_cache_blocks, int64_t *d_totals,
                                           int64_t *d_instance_blocks, int64_t *d_instance_blocks_per_trace,
                                           uint32_t *d_status, kvcm_stream_t stream) {
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (n_traces < 0 || n_keys_total < 0 || n_configs <= 0 || evict_batch <= 0 || n_instances <= 0 ||
        eviction_mode < 1 || eviction_mode > 3) {
        return KVCM_EC_BADARGS;
    }
    const int64_t need = kvcm_b200_replay_lru_group_workspace_bytes(n_keys_total, n_configs, n_instances);
    if (need < 0) return KVCM_EC_OUT_OF_LIMIT;
    if (n_traces == 0) return KVCM_OK;
    const int per_trace = (d_ext_hit != nullptr) + (d_int_hit != nullptr) + (d_written != nullptr) +
                          (d_cache_blocks != nullptr);
    if (d_key_off == nullptr || d_trace_type == nullptr || d_quota_blocks == nullptr || d_workspace == nullptr ||
        d_trace_instance == nullptr || (d_keys == nullptr && n_keys_total > 0) || (per_trace != 0 && per_trace != 4) ||
        (per_trace == 0 && d_totals == nullptr)) {
        return KVCM_ER_INVALID_ADDRESS;
    }
    if (reinterpret_cast<uintptr_t>(d_workspace) & 255u) return KVCM_ER_INVALID_ADDRESS;
    if (workspace_bytes < need) return KVCM_EC_NOSPC;
    const kvcm::LruLayout l = kvcm::LayoutFor(n_keys_total, n_configs);
    uint8_t *ws = static_cast<uint8_t *>(d_workspace);
    kvcm::IdTable t;
    t.cells = reinterpret_cast<unsigned long long *>(ws);
    t.slots = reinterpret_cast<ulonglong2 *>(ws + l.table_off);
    t.mask = kvcm::SlotsFor(n_keys_total) - 1;
    uint32_t *ids = reinterpret_cast<uint32_t *>(ws + l.ids_off);
    uint32_t *stamps = reinterpret_cast<uint32_t *>(ws + l.stamps_off);
    int64_t *queue_base = reinterpret_cast<int64_t *>(ws + l.total);
    cudaStream_t s = kvcm::AsStream(stream);
    const int sms = kvcm::GetDeviceInfo().sm_count;
    const uint64_t n_stamps = static_cast<uint64_t>(n_keys_total) * static_cast<uint64_t>(n_configs);
    kvcm::LruInitKernel<<<sms * 8, 256, 0, s>>>(t, stamps, n_stamps);
    kvcm::LruGroupExtentKernel<<<1, 1024, sizeof(unsigned long long) * n_instances, s>>>(
        d_key_off, d_trace_instance, n_traces, n_instances, queue_base, d_status);
    if (n_keys_total > 0) {
        // one instance after the other: the table starts empty each time, the id counter runs on
        for (int32_t j = 0; j < n_instances; ++j) {
            if (j > 0) kvcm::IdTableClearKernel<<<sms * 8, 256, 0, s>>>(t);
            kvcm::LruClaimIdsOfInstanceKernel<<<sms * 4, 256, 0, s>>>(t, d_keys, d_key_off, d_trace_instance, n_traces, j,
                                                                     d_status);
            kvcm::LruLookupIdsOfInstanceKernel<<<sms * 4, 256, 0, s>>>(t, d_keys, d_key_off, d_trace_instance, n_traces,
                                                                      j, ids);
        }
    }
    kvcm::LruSweep p;
    p.ids = ids;
    p.key_off = d_key_off;
    p.type = d_trace_type;
    p.mask_off = d_mask_off;
    p.mask_bits = d_mask_bits;
    p.quota = d_quota_blocks;
    p.stamps = stamps;
    p.queue = reinterpret_cast<uint2 *>(ws + l.queue_off);
    p.ext_hit = d_ext_hit;
    p.int_hit = d_int_hit;
    p.written = d_written;
    p.cache_blocks = d_cache_blocks;
    p.totals = d_totals;
    p.n_keys = n_keys_total > 0 ? n_keys_total : 1;
    p.n_traces = n_traces;
    p.n_configs = n_configs;
    p.evict_batch = evict_batch;
    p.precise = eviction_mode == 3;
    kvcm::LruGroup g;
    g.trace_inst = d_trace_instance;
    g.queue_base = queue_base;
    g.inst_blocks = d_instance_blocks;
    g.inst_blocks_trace = d_instance_blocks_per_trace;
    g.n_instances = n_instances;
    g.mode = eviction_mode;
    kvcm::LruGroupSweepKernel<<<static_cast<unsigned>(n_configs), 32, sizeof(int64_t) * 4 * n_instances, s>>>(p, g);
    return kvcm::LaunchStatus();
}

}  // extern "C"
