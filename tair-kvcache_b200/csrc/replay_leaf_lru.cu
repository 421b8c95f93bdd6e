// Optimizer trace replay with the "leaf_aware_lru" eviction policy, for a sweep of cache quotas at once (sm_100a).
//
// Stands in for OptimizerRunner::RunTraces (kv_cache_manager/optimizer/manager/optimizer_runner.cc:29-215) over
// RadixTreeIndex (kv_cache_manager/optimizer/index/radix_tree_index.cc:19-392) with LeafAwareLruEvictionPolicy
// (kv_cache_manager/optimizer/eviction_policy/leaf_aware_lru.cc:20-160) and the quota check after every write
// (OptIndexerManager::CheckAndEvict, kv_cache_manager/optimizer/manager/indexer_manager.cc:55-90;
// OptEvictionManager, kv_cache_manager/optimizer/manager/eviction_manager.cc:86-266), for one instance or for a
// group of instances that share the quota: every instance has a tree and a queue of its own
// (kv_cache_manager/optimizer/manager/optimizer_manager.cc:66-99), here one pool of node numbers whose first
// n_instances entries are the roots, and one pair of queue sentinels per instance; ids are unique over
// (instance, key), so everything that is kept per key needs no instance.
//
// Unlike plain LRU this policy reads the shape of the tree: only blocks of childless nodes queue up for
// eviction, a block whose node has cached children is dropped from the queue when it reaches the cold end, and a
// node whose children have all been emptied gets its blocks queued again, sorted by last access time.  So the
// tree is kept, per configuration, in a form a warp can walk without pointers.  Keys are prefix-unique chained
// hashes: a key fixes the key before it.  Hence
//   occ[id]       a position of key id in the id array - the same for every configuration, built once.  The
//                 ids in front of it there, back to the start of that trace, are the key's chain;
//   node_of[id]   the tree node that holds the block of key id; the key is in the tree while that node has
//                 blocks (removing a node zeroes its block count, node numbers are never reused).  If a key is
//                 in the tree, so is its whole chain, and a trace's walk down the tree is the run of its leading
//                 keys that are in the tree;
//   per node      parent, number of children, number of blocks, last key, cached blocks, cached blocks of the
//                 immediate children (zero = RadixTreeNode::isDataLeaf), cached blocks outside the queue.
// A node's blocks are the end of the chain of its last key.  Splitting a node (radix_tree_index.cc:89-127) gives
// the new number to the UPPER part, whose keys are the ones the splitting trace has just walked.
// The queue is the reference's doubly linked list over key ids (two sentinels), because the sorted re-insertions
// (kv_cache_manager/optimizer/eviction_policy/common_structure.h:62-89) depend on list order, ties included.
//
// One warp per configuration.  Lanes share the scan of a trace's keys, the relabelling at a split, the writes of
// new blocks, the eviction of a group of cold blocks and the re-queueing of a node's blocks; what is left to lane 0
// is the list surgery around them and the walk to a sorted insertion point (latency-bound on L2).
// Every walk carries an iteration limit so that keys that break the prefix-unique premise end in a status
// count, not in an endless loop.
//
// A group may also hold instances of the "random_lru" policy (EvictionPolicyFactory::CreatePolicy makes a policy per
// instance, whatever the others are).  Such an instance needs no tree here - which blocks a trace hits and writes
// depends on per-key state alone - so the second form of the kernel keeps, for those instances, the sampling
// policy's block vector (replay_sampling.cuh) beside the trees and queues of the others, and the quota check calls
// whichever EvictBlocks the instance's policy has.
#include "kvcm_common.cuh"
#include "replay_ids.cuh"
#include "replay_sampling.cuh"

namespace kvcm {
namespace {

constexpr uint32_t kNone = 0xFFFFFFFFu;
constexpr uint8_t kCached = 1, kListed = 2;
constexpr int kNodeFields = 7;

struct LeafSweep {
    const uint32_t *ids;
    const uint32_t *occ;  // one position of each key in ids
    const int64_t *key_off;
    const uint8_t *type;
    const int64_t *mask_off;
    const uint8_t *mask_bits;
    const int64_t *timestamps;  // optional, per trace; the trace number when null
    const int32_t *trace_inst;  // optional, per trace, 0 .. n_instances-1; instance 0 when null
    const int64_t *quota;
    uint32_t *node_of;  // [n_configs][n_keys]
    uint8_t *flags;     // [n_configs][n_keys]
    int64_t *time;      // [n_configs][n_keys]  last_access_time
    uint32_t *lprev;    // [n_configs][n_keys]  towards the hot end; the sentinels' links are in shared memory
    uint32_t *lnext;    // [n_configs][n_keys]  towards the cold end
    uint32_t *evicted;  // [n_configs][n_keys]  the nodes of the blocks evicted after one trace
    uint32_t *nodes;    // [n_configs][kNodeFields][max_nodes]
    int32_t *ext_hit, *int_hit, *written;
    int64_t *cache_blocks;
    int64_t *totals;
    int64_t *inst_blocks;        // optional, [n_configs][n_instances]: usage per instance at the end
    int64_t *inst_blocks_trace;  // optional, [n_configs][n_traces][n_instances]: usage of every instance after each trace
    uint32_t *status;
    int64_t n_keys;
    int64_t n_ids;  // key occurrences in ids (n_keys is this, or 1 for an empty input)
    int64_t max_nodes;
    int32_t n_traces;
    int32_t n_configs;
    int32_t evict_batch;
    int32_t n_instances;
    int32_t mode;  // 1 group rough, 2 instance rough, 3 instance precise
    // bit j set: instance j runs the plain "lru" policy (kv_cache_manager/optimizer/eviction_policy/lru.cc:6-49) over
    // the same tree and queue: every cached block is queued whatever its node's children, the cold end goes first
    uint64_t lru_instances;
    // bit j set: instance j runs "random_lru".  The node_of entry of one of its keys is the block's index in the
    // instance's block vector (kNone = not cached); the vector is the instance's region of blk / ts.
    uint64_t sampling_instances;
    uint32_t *blk;               // [n_configs][n_keys]; null without a sampling instance
    int64_t *ts;                 // [n_configs][n_keys]
    const int64_t *region_base;  // [n_instances + 1]: key occurrences of the instances before (LruGroupExtentKernel)
    uint32_t sampling_size[KVCM_B200_REPLAY_GROUP_MAX_INSTANCES];
};
static_assert(kNone == kNotCached, "a sampling instance's index shares node_of with the tree instances' node numbers");

__global__ void LeafInitKernel(IdTable t, uint32_t *node_of, uint8_t *flags, uint64_t n_state) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    const uint64_t first = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (uint64_t i = first; i <= t.mask; i += stride) t.slots[i] = make_ulonglong2(kEmptyKey, ~0ull);
    for (uint64_t i = first; i < n_state; i += stride) {
        node_of[i] = kNone;
        flags[i] = 0;
    }
    if (first == 0) {
        t.cells[0] = 0ull;
        t.cells[1] = ~0ull;
    }
}

// occ[id] = a position of the key in ids (whichever occurrence writes last).  Keys are prefix-unique, so the ids
// in front of that position, back to the start of its trace, are the key's chain whichever occurrence it is; and
// the ids behind it are a guess at what follows the key in a queue, checked against the queue's links before use.
// Traces that name no instance of the group have no ids and are left out.
__global__ void __launch_bounds__(256)
    LeafOccKernel(const uint32_t *__restrict__ ids, const int64_t *__restrict__ key_off,
                  const int32_t *__restrict__ trace_inst, int32_t n_instances, int32_t n_traces, uint32_t *occ) {
    const int32_t warps = static_cast<int32_t>(gridDim.x * (blockDim.x >> 5));
    const uint32_t lane = LaneId();
    for (int32_t t = static_cast<int32_t>(blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)); t < n_traces;
         t += warps) {
        if (trace_inst != nullptr && (trace_inst[t] < 0 || trace_inst[t] >= n_instances)) continue;
        const int64_t end = key_off[t + 1];
        for (int64_t i = key_off[t] + lane; i < end; i += 32) occ[ids[i]] = static_cast<uint32_t>(i);
    }
}

// Traces of an instance number outside the group are replayed as empty traces (the sweep does the same) and counted.
__global__ void __launch_bounds__(256)
    LeafCheckInstancesKernel(const int32_t *__restrict__ trace_inst, int32_t n_traces, int32_t n_instances,
                             uint32_t *status) {
    const int32_t stride = static_cast<int32_t>(gridDim.x * blockDim.x);
    for (int32_t t = static_cast<int32_t>(blockIdx.x * blockDim.x + threadIdx.x); t < n_traces; t += stride) {
        const int32_t j = trace_inst[t];
        if ((j < 0 || j >= n_instances) && status != nullptr) atomicAdd(&status[0], 1u);
    }
}

// type: 0 DialogTurn (InsertWithQuery), 1 GetLocation (PrefixQuery), 2 WriteCache (InsertOnly).
// kSampling: the group holds "random_lru" instances too (more shared memory, one more branch per trace and per
// round of evictions).
template <bool kSampling>
__global__ void __launch_bounds__(32) LeafSweepKernel(const LeafSweep p) {
    extern __shared__ int64_t cached_of[];  // [n_instances]: cached blocks per instance (EvictionPolicy::size())
    __shared__ uint32_t short_group[32];
    // The sentinels' own links live in shared memory only (the hot and the cold end of every instance's queue are
    // read for every trace and every eviction): the links of keys are in global memory.
    uint32_t *front_of = reinterpret_cast<uint32_t *>(cached_of + p.n_instances);  // [n_instances]: hottest entry
    uint32_t *cold_of = front_of + p.n_instances;                                  // [n_instances]: coldest entry
    // sampling instances: the generator's state, where the block vector starts, the warp's scratch for a round
    uint64_t *rng_of = reinterpret_cast<uint64_t *>(cached_of + 2 * p.n_instances);  // [n_instances]
    int64_t *base_of = cached_of + 3 * p.n_instances;                                // [n_instances]
    SamplingScratch *scratch = reinterpret_cast<SamplingScratch *>(cached_of + 4 * p.n_instances);
    const int64_t cfg = blockIdx.x;
    const uint32_t lane = LaneId();
    const uint32_t full = 0xffffffffu;
    const uint32_t below = (1u << lane) - 1u;
    const int64_t nk = p.n_keys;
    const int32_t K = p.n_instances;
    const uint32_t n_roots = static_cast<uint32_t>(K);  // node j is the root of instance j
    uint32_t *node_of = p.node_of + cfg * nk;
    uint8_t *flags = p.flags + cfg * nk;
    int64_t *time = p.time + cfg * nk;
    uint32_t *lprev = p.lprev + cfg * nk;
    uint32_t *lnext = p.lnext + cfg * nk;
    uint32_t *evicted = p.evicted + cfg * nk;
    uint32_t *node = p.nodes + cfg * kNodeFields * p.max_nodes;
    uint32_t *n_parent = node, *n_children = node + p.max_nodes, *n_blocks = node + 2 * p.max_nodes;
    uint32_t *n_last = node + 3 * p.max_nodes, *n_cached = node + 4 * p.max_nodes;
    uint32_t *n_childc = node + 5 * p.max_nodes;  // cached blocks of the immediate children
    uint32_t *n_unlisted = node + 6 * p.max_nodes;  // cached blocks of the node that are not in the queue
    const int64_t quota = p.quota[cfg];
    const int64_t out0 = cfg * p.n_traces;
    const uint64_t walk_cap = static_cast<uint64_t>(nk) + 2;
    // the queue of instance j lies between the sentinels head_of(j) (hot end) and head_of(j) + 1 (cold end)
    auto head_of = [&](int32_t j) { return static_cast<uint32_t>(nk) + 2u * static_cast<uint32_t>(j); };
    auto plain_lru = [&](int32_t j) { return ((p.lru_instances >> j) & 1ull) != 0; };
    auto sampling = [&](int32_t j) { return kSampling && ((p.sampling_instances >> j) & 1ull) != 0; };
    // x is a key or a sentinel of instance j's queue (hd = its hot-end sentinel)
    auto get_next = [&](uint32_t x, uint32_t hd, int32_t j) { return x == hd ? front_of[j] : lnext[x]; };
    auto get_prev = [&](uint32_t x, uint32_t hd, int32_t j) { return x == hd + 1 ? cold_of[j] : lprev[x]; };
    auto set_next = [&](uint32_t x, uint32_t v, uint32_t hd, int32_t j) {
        if (x == hd) {
            front_of[j] = v;
        } else {
            lnext[x] = v;
        }
    };
    auto set_prev = [&](uint32_t x, uint32_t v, uint32_t hd, int32_t j) {
        if (x == hd + 1) {
            cold_of[j] = v;
        } else {
            lprev[x] = v;
        }
    };

    // owned by lane 0
    uint32_t n_nodes = n_roots, faults = 0;
    int64_t resident = 0, sum_ext = 0, sum_int = 0, sum_wr = 0;  // resident: of the whole group

    auto new_node = [&](uint32_t parent) -> uint32_t {
        uint32_t x = n_nodes;
        if (static_cast<int64_t>(x) >= p.max_nodes) {  // cannot happen: a trace makes at most two nodes
            ++faults;
            x = static_cast<uint32_t>(p.max_nodes - 1);
        } else {
            ++n_nodes;
        }
        n_parent[x] = parent;
        n_children[x] = 0;
        n_blocks[x] = 0;
        n_last[x] = kNone;
        n_cached[x] = 0;
        n_childc[x] = 0;
        n_unlisted[x] = 0;
        return x;
    };
    // Where LinkedList::insert_sorted / insert_sorted_reverse under LeafLRUListNode::compare, picked as
    // insert_sorted_by_priority picks them (leaf_aware_lru.cc:53-83), put a block of time bt into the queue between
    // hd and hd + 1: the entry it goes in front of, and whether the walk came from the hot end.  An insertion from the
    // hot end lands in front of the entries of equal time, one from the cold end behind them.  Lane 0.
    auto insertion_point = [&](int64_t bt, uint32_t hd, int32_t j, bool *from_hot) -> uint32_t {
        const uint32_t tl = hd + 1;
        const uint32_t h = front_of[j];
        *from_hot = true;
        if (h == tl) return tl;
        const uint32_t c = cold_of[j];
        const int64_t ht = time[h], ct = time[c];
        *from_hot = bt >= ht ? true : (bt <= ct ? false : (ht - bt) < (bt - ct));
        uint64_t steps = 0;
        uint32_t before;
        if (*from_hot) {
            uint32_t cur = h;
            while (cur != tl && bt < time[cur] && ++steps < walk_cap) cur = lnext[cur];
            before = cur;
        } else {
            uint32_t cur = c;
            while (cur != hd && time[cur] < bt && ++steps < walk_cap) cur = lprev[cur];
            before = get_next(cur, hd, j);
        }
        if (steps >= walk_cap) ++faults;
        return before;
    };
    // UpdateNodeState (leaf_aware_lru.cc:135-160) for a node that has just become a data leaf: its cached blocks
    // that are outside the queue go back in, in key order, each by sorted insertion.  All lanes.  The node's
    // blocks are the last n_blocks ids of the chain that ends at its last key, read straight out of the id array.
    // Consecutive insertions of one time end up side by side - the second one walks from the same end, stops at
    // the first one and lands in front of it (from the hot end) or behind it (from the cold end), and so on - so a
    // run of blocks that share a time costs one walk for its first block and one splice: lanes write the links
    // inside the run, lane 0 the two links around it.  Blocks written or touched by one trace share a time.
    auto requeue_node = [&](uint32_t u, uint32_t hd, int32_t j) {
        const uint32_t c = n_blocks[u];
        const uint32_t last = n_last[u];
        const int64_t first_pos = last != kNone ? static_cast<int64_t>(p.occ[last]) - static_cast<int64_t>(c) + 1 : -1;
        bool broken = last == kNone || first_pos < 0;
        for (uint32_t base = 0; base < c && !broken; base += 32) {
            const uint32_t k = base + lane;
            const bool have = k < c;
            const uint32_t x = have ? p.ids[first_pos + k] : kNone;
            const bool member = have && node_of[x] == u;
            broken = __any_sync(full, have && !member);
            const bool need = member && (flags[x] & (kCached | kListed)) == kCached;
            const int64_t tm = need ? time[x] : 0;
            const uint32_t need_m = __ballot_sync(full, need);
            const int lower_need = 31 - __clz(need_m & below);  // the needing lane before this one, -1 if none
            const int64_t tm_lower = __shfl_sync(full, tm, lower_need < 0 ? 0 : lower_need);
            uint32_t starts = __ballot_sync(full, need && (lower_need < 0 || tm_lower != tm));
            while (starts != 0) {
                const int first = __ffs(starts) - 1;
                starts &= starts - 1;
                const uint32_t upto = starts != 0 ? ((1u << (__ffs(starts) - 1)) - 1u) : full;
                const uint32_t run = need_m & upto & ~((1u << first) - 1u);
                const int top = 31 - __clz(run);
                const uint32_t x_first = __shfl_sync(full, x, first), x_top = __shfl_sync(full, x, top);
                const int64_t bt = __shfl_sync(full, tm, first);
                uint32_t before = 0, after = 0, hot = 0;  // the run goes between `after` (hotter) and `before`
                if (lane == 0) {
                    bool from_hot;
                    before = insertion_point(bt, hd, j, &from_hot);
                    after = get_prev(before, hd, j);
                    hot = from_hot ? 1u : 0u;
                }
                before = __shfl_sync(full, before, 0);
                after = __shfl_sync(full, after, 0);
                hot = __shfl_sync(full, hot, 0);
                const bool mine = ((run >> lane) & 1u) != 0;
                const int lower = 31 - __clz(run & below);
                const uint32_t above_m = run & ~below & ~(1u << lane);
                const int higher = above_m != 0 ? __ffs(above_m) - 1 : -1;
                const uint32_t x_lower = __shfl_sync(full, x, lower < 0 ? 0 : lower);
                const uint32_t x_higher = __shfl_sync(full, x, higher < 0 ? 0 : higher);
                if (mine) {
                    // from the hot end the later block lies in front of the earlier one; from the cold end behind it
                    const uint32_t colder = hot != 0 ? (lower < 0 ? before : x_lower) : (higher < 0 ? before : x_higher);
                    const uint32_t hotter = hot != 0 ? (higher < 0 ? after : x_higher) : (lower < 0 ? after : x_lower);
                    lnext[x] = colder;
                    lprev[x] = hotter;
                    flags[x] = kCached | kListed;
                }
                if (lane == 0) {
                    set_next(after, hot != 0 ? x_top : x_first, hd, j);
                    set_prev(before, hot != 0 ? x_first : x_top, hd, j);
                }
                __syncwarp();
            }
        }
        if (lane == 0) {
            if (broken) ++faults;
            n_unlisted[u] = 0;
        }
        __syncwarp();
    };

    uint32_t n_ev = 0;   // kept equal in all lanes: entries of `evicted` since the last check began
    uint64_t spins = 0;  // lane 0: steps of the one-by-one path since the last check began
    // LeafAwareLruEvictionPolicy::EvictBlocks(count) of instance j (leaf_aware_lru.cc:85-133), up to 32 blocks at
    // a time; all lanes, returns how many blocks went.  Its set of parents already handled only saves work: a
    // handled parent has nothing left outside the queue.
    auto evict_from = [&](int32_t j, int64_t count) -> int64_t {
        const uint32_t hd = head_of(j), tl = hd + 1;
        const bool lru = plain_lru(j);  // nothing ever leaves this queue but by eviction, nothing is re-queued
        int64_t got = 0;
        while (got < count) {
            const uint32_t want = static_cast<uint32_t>(count - got < 32 ? count - got : 32);
            // The candidates, from the cold end of the queue.  Blocks written by one trace sit in the queue in the
            // trace's key order, so the keys that follow the coldest block in ids are a guess at the blocks that
            // follow it in the queue; each lane checks one link of the guess and the group is the part that the
            // queue's own links confirm.  A short group (keys shared by many traces) falls back to lane 0
            // following the links one by one.
            const uint32_t coldest = cold_of[j];
            if (coldest == hd) break;  // the queue ran out
            const int64_t guess_at = static_cast<int64_t>(p.occ[coldest]) + lane;
            uint32_t cand = lane == 0 ? coldest : (guess_at < p.n_ids ? p.ids[guess_at] : kNone);
            const uint32_t towards_head = cand != kNone ? lprev[cand] : kNone;
            const uint32_t cand_after = __shfl_down_sync(full, cand, 1);
            const uint32_t linked = __ballot_sync(full, lane < 31 && cand_after != kNone && towards_head == cand_after);
            uint32_t m = static_cast<uint32_t>(__ffs(~linked));  // confirmed links + 1 (bit 31 is never set)
            if (m > want) m = want;
            uint32_t after = __shfl_sync(full, towards_head, m - 1);
            if (m < want && m < 8) {
                m = 0;
                if (lane == 0) {
                    uint32_t b = coldest;
                    while (m < want && b != hd) {
                        short_group[m++] = b;
                        b = lprev[b];
                    }
                    after = b;
                }
                m = __shfl_sync(full, m, 0);
                after = __shfl_sync(full, after, 0);
                __syncwarp();
                cand = lane < m ? short_group[lane] : kNone;
                __syncwarp();
            }
            const bool mine = lane < m;
            const uint32_t nd = mine ? node_of[cand] : 0u;
            const uint32_t up = mine ? n_parent[nd] : 0u;
            // The whole group goes at once when every candidate sits in a data leaf and no parent runs out of
            // cached children while it still has blocks outside the queue (nothing is re-queued, so the queue
            // stays as it was followed).
            const uint32_t same_up = __match_any_sync(full, mine ? up : kNone - lane);
            const uint32_t same_nd = __match_any_sync(full, mine ? nd : kNone - lane);
            bool plain = true;
            if (mine && !lru) {
                const uint32_t under = static_cast<uint32_t>(__popc(same_up));
                plain = n_childc[nd] == 0 && (up < n_roots || n_unlisted[up] == 0 || n_childc[up] > under);
            }
            if (__all_sync(full, plain) && static_cast<int64_t>(n_ev) + m <= nk) {
                if (mine) {
                    flags[cand] = 0;
                    evicted[n_ev + lane] = nd;
                    if (static_cast<uint32_t>(__ffs(same_nd) - 1) == lane) {
                        atomicSub(&n_cached[nd], static_cast<uint32_t>(__popc(same_nd)));
                    }
                }
                __syncwarp();  // n_childc is read above for nodes that are parents here
                if (mine && static_cast<uint32_t>(__ffs(same_up) - 1) == lane) {
                    atomicSub(&n_childc[up], static_cast<uint32_t>(__popc(same_up)));
                }
                if (lane == 0) {
                    set_next(after, tl, hd, j);
                    cold_of[j] = after;
                    resident -= m;
                    cached_of[j] -= m;
                }
                __syncwarp();
                n_ev += m;
                got += m;
                continue;
            }
            // otherwise one block after the other, up to the same number; lane 0 stops where a parent has become
            // a data leaf with blocks outside the queue, the warp queues them, lane 0 goes on
            uint32_t g = 0;
            for (;;) {
                uint32_t turned = kNone;
                if (lane == 0) {
                    while (g < want) {
                        const uint32_t b = cold_of[j];
                        if (b == hd) break;
                        if (++spins > 2 * walk_cap || static_cast<int64_t>(n_ev) >= nk) {
                            ++faults;  // a block leaves the queue at most twice per check, and is evicted once
                            break;
                        }
                        const uint32_t a = lprev[b];
                        const uint32_t node_b = node_of[b];
                        set_next(a, tl, hd, j);
                        cold_of[j] = a;
                        if (!lru && n_childc[node_b] != 0) {  // its node has cached children by now: out of the queue
                            flags[b] = kCached;
                            n_unlisted[node_b] += 1;
                            continue;
                        }
                        flags[b] = 0;
                        n_cached[node_b] -= 1;
                        const uint32_t up_b = n_parent[node_b];
                        n_childc[up_b] -= 1;
                        evicted[n_ev++] = node_b;
                        ++g;
                        if (!lru && up_b >= n_roots && n_childc[up_b] == 0 && n_unlisted[up_b] != 0) {
                            turned = up_b;
                            break;
                        }
                    }
                }
                turned = __shfl_sync(full, turned, 0);
                if (turned == kNone) break;
                requeue_node(turned, hd, j);
            }
            g = __shfl_sync(full, g, 0);
            n_ev = __shfl_sync(full, n_ev, 0);
            if (lane == 0) {
                resident -= g;
                cached_of[j] -= g;
            }
            __syncwarp();
            got += g;
            if (g < want) break;  // the queue ran out (or a walk limit did)
        }
        return got;
    };
    // EvictBlocks(count) of instance j, whatever its policy; all lanes, returns how many blocks went
    auto evict_blocks = [&](int32_t j, int64_t count) -> int64_t {
        if (!sampling(j)) return evict_from(j, count);
        const int64_t held = cached_of[j];
        const int64_t got = SamplingEvictRound(*scratch, node_of, p.blk + cfg * nk + base_of[j],
                                               p.ts + cfg * nk + base_of[j], held, &rng_of[j], p.sampling_size[j],
                                               count, lane);
        if (lane == 0) {
            cached_of[j] = held - got;
            resident -= got;
        }
        __syncwarp();
        return got;
    };

    if (lane == 0) {
        for (int32_t j = 0; j < K; ++j) {
            n_parent[j] = kNone;
            n_children[j] = 0;
            n_blocks[j] = 0;
            n_last[j] = kNone;
            n_cached[j] = 0;
            n_childc[j] = 0;
            n_unlisted[j] = 0;
            front_of[j] = head_of(j) + 1;
            cold_of[j] = head_of(j);
            cached_of[j] = 0;
            if (kSampling) {
                rng_of[j] = kSamplingSeed;
                base_of[j] = p.region_base[j];
            }
        }
    }
    __syncwarp();

    // What a trace reads before it touches any state (its extent, kind, time, instance and the ids of its first 32
    // keys) is fetched one trace ahead, its extent two traces ahead: those loads do not wait for the traces before it.
    auto extent = [&](int32_t t, int64_t *beg, int64_t *n, uint8_t *ty, int64_t *skip, int64_t *now, int32_t *who) {
        if (t < p.n_traces) {
            *beg = p.key_off[t];
            *n = p.key_off[t + 1] - *beg;
            *ty = p.type[t];
            *skip = (*ty == 1 && p.mask_off != nullptr) ? p.mask_off[t] : 0;
            *now = p.timestamps != nullptr ? p.timestamps[t] : static_cast<int64_t>(t);
            *who = p.trace_inst != nullptr ? p.trace_inst[t] : 0;
            if (*who < 0 || *who >= K) {  // counted by LeafCheckInstancesKernel; its keys have no ids
                *who = 0;
                *n = 0;
            }
        } else {
            *beg = 0, *n = 0, *ty = 1, *skip = 0, *now = 0, *who = 0;
        }
    };
    int64_t beg, n, skip, now, beg1, n1, skip1, now1;
    uint8_t ty, ty1;
    int32_t me, me1;
    extent(0, &beg, &n, &ty, &skip, &now, &me);
    extent(1, &beg1, &n1, &ty1, &skip1, &now1, &me1);
    uint32_t first_id = lane < n ? p.ids[beg + lane] : 0u;

    for (int32_t t = 0; t < p.n_traces; ++t) {
        const uint32_t next_first_id = lane < n1 ? p.ids[beg1 + lane] : 0u;
        int64_t beg2, n2, skip2, now2;
        uint8_t ty2;
        int32_t me2;
        extent(t + 2, &beg2, &n2, &ty2, &skip2, &now2, &me2);
        int32_t ext = 0, inte = 0, wr = 0;
        const uint32_t my_root = static_cast<uint32_t>(me);
        const uint32_t kHead = head_of(me);
        const bool sampled = sampling(me);  // a trace of a "random_lru" instance: no tree, its block vector only
        if (sampled) {
            const SamplingTraceCounts c = SamplingReplayTrace(
                p.ids + beg, p.mask_bits != nullptr ? p.mask_bits + beg : nullptr, n, ty, skip, now, node_of,
                p.blk + cfg * nk + base_of[me], p.ts + cfg * nk + base_of[me], cached_of[me], lane);
            ext = c.ext, inte = c.inte, wr = c.wr;
            n = 0;  // nothing is left for the tree
        }

        // ---- scan: where the trace leaves the tree (div) and its first block that is not cached (first_gone)
        // A key is in the tree when its node still has blocks: removing a node only zeroes its block count.
        int64_t div = n, first_gone = -1;
        uint32_t at_id = kNone, at_node = my_root;      // the last block inside the tree and its node (the root if none)
        uint32_t carry_id = kNone, carry_node = my_root;  // the same for the previous 32 keys
        for (int64_t base = 0; base < n; base += 32) {
            const int64_t i = base + lane;
            const bool have = i < n;
            const uint32_t id = base == 0 ? first_id : (have ? p.ids[beg + i] : 0u);
            uint32_t nd = have ? node_of[id] : kNone;
            const uint8_t fl = have ? flags[id] : 0;
            // (a cached block's node has blocks for sure, so only the others pay for the second load)
            if (nd != kNone && (fl & kCached) == 0 && n_blocks[nd] == 0) nd = kNone;
            const uint32_t in_range = __ballot_sync(full, have);
            const uint32_t in_tree = __ballot_sync(full, have && nd != kNone);
            const uint32_t cached = __ballot_sync(full, have && nd != kNone && (fl & kCached) != 0);
            const uint32_t out = in_range & ~in_tree;
            const uint32_t valid = out != 0 ? ((1u << (__ffs(out) - 1)) - 1u) : in_range;
            const uint32_t gone = valid & ~cached;
            if (first_gone < 0) {
                if (ty != 2) {
                    const uint32_t lead = gone != 0 ? (valid & ((1u << (__ffs(gone) - 1)) - 1u)) : valid;
                    const uint32_t masked = __ballot_sync(
                        full, i < skip || (ty == 1 && p.mask_bits != nullptr && have && p.mask_bits[beg + i] != 0));
                    ext += __popc(lead & ~masked);
                    inte += __popc(lead & masked);
                }
                if (gone != 0) first_gone = base + __ffs(gone) - 1;
            }
            if (out != 0) {
                const int src = __ffs(out) - 1;
                div = base + src;
                const uint32_t id_before = __shfl_sync(full, id, src > 0 ? src - 1 : 0);
                const uint32_t node_before = __shfl_sync(full, nd, src > 0 ? src - 1 : 0);
                at_id = src > 0 ? id_before : carry_id;
                at_node = src > 0 ? node_before : carry_node;
                break;
            }
            if (ty == 1 && first_gone >= 0) break;
            carry_id = __shfl_sync(full, id, 31);
            carry_node = __shfl_sync(full, nd, 31);
        }
        const int64_t hit_len = ty == 2 ? 0 : (first_gone >= 0 ? first_gone : div);

        // ---- the leading cached blocks are accessed, in order (radix_tree_index.cc:166-172,246-249): each one
        // moves to the front of the queue.  Blocks that already follow each other in the queue the way the moves
        // would leave them (the later one in front of the earlier one) move as one piece; a piece of one block is
        // the plain move.  The links inside a piece are read by all lanes at once, the splice is lane 0's.
        if (ty != 2) {
            for (int64_t base = 0; base < hit_len; base += 32) {
                const int64_t i = base + lane;
                const bool have = i < hit_len;
                const uint32_t id = have ? p.ids[beg + i] : kNone;
                bool listed = false;
                uint32_t ln = kNone, lp = kNone;  // this key's links, kept up to date below; they mean something only when queued
                if (have) {
                    time[id] = now;
                    ln = lnext[id];
                    lp = lprev[id];
                    listed = (flags[id] & kListed) != 0;
                }
                uint32_t front = front_of[me];  // kept equal in all lanes
                const uint32_t id_before = __shfl_up_sync(full, id, 1);
                const uint32_t listed_m = __ballot_sync(full, listed);
                const bool joins = listed && lane > 0 && ((listed_m >> (lane - 1)) & 1u) != 0 && ln == id_before;
                const uint32_t joins_m = __ballot_sync(full, joins);
                uint32_t starts = listed_m & ~joins_m;
                while (starts != 0) {
                    const int first = __ffs(starts) - 1;
                    starts &= starts - 1;
                    const int len = first == 31 ? 0 : __ffs(~(joins_m >> (first + 1))) - 1;
                    const uint32_t piece_tail = __shfl_sync(full, id, first);        // accessed first: ends up deepest
                    const uint32_t piece_head = __shfl_sync(full, id, first + len);  // accessed last: ends up in front
                    const uint32_t b = __shfl_sync(full, ln, first);        // what follows the piece, towards the cold end
                    const uint32_t a = __shfl_sync(full, lp, first + len);  // what precedes it
                    if (a == kHead) continue;  // in front already
                    if (lane == 0) {
                        lnext[a] = b;  // a is a key: the piece is not in front
                        set_prev(b, a, kHead, me);
                        lnext[piece_tail] = front;
                        lprev[front] = piece_tail;  // a key: the queue holds the piece and more
                        lprev[piece_head] = kHead;
                    }
                    // the same five links in the lanes' copies, so that a later piece needs no load
                    if (listed) {
                        if (id == a) ln = b;
                        if (id == b) lp = a;
                        if (id == piece_tail) ln = front;
                        if (id == front) lp = piece_tail;
                        if (id == piece_head) lp = kHead;
                    }
                    front = piece_head;
                }
                if (lane == 0) front_of[me] = front;
                __syncwarp();
            }
        }

        if (ty != 1) {
            // ---- evicted blocks on the walked path get their location back (:60-63,250-252,355-375)
            if (lane == 0) {
                for (int64_t i = hit_len; i < div; ++i) {
                    const uint32_t id = p.ids[beg + i];
                    if ((flags[id] & kCached) != 0) continue;
                    const uint32_t nd = node_of[id];
                    time[id] = now;
                    const uint32_t above = n_parent[nd], kids = n_children[nd];
                    atomicAdd(&n_cached[nd], 1u);
                    atomicAdd(&n_childc[above], 1u);
                    ++wr;
                    if (kids == 0 || plain_lru(me)) {
                        flags[id] = kCached | kListed;
                        const uint32_t f = front_of[me];
                        lnext[id] = f;
                        lprev[id] = kHead;
                        set_prev(f, id, kHead, me);
                        front_of[me] = id;
                    } else {
                        flags[id] = kCached;
                        atomicAdd(&n_unlisted[nd], 1u);
                    }
                }
            }
            __syncwarp();
            if (div < n) {
                // ---- where the rest goes: the end of a childless node, a new child, or a split (:30-87,89-127)
                uint32_t target = 0, child = 0, mid = 0, do_split = 0, old_front = 0;
                uint32_t above_target = 0, above_at = 0;  // lane 0: the parents of the target node and of at_node
                if (lane == 0) {
                    const uint32_t at = at_node;
                    const uint32_t last_of_at = n_last[at], kids = n_children[at];
                    above_at = n_parent[at];
                    old_front = front_of[me];
                    if (div == 0 || last_of_at == at_id) {
                        if (at >= n_roots && kids == 0) {
                            target = at;
                            above_target = above_at;
                        } else {
                            target = new_node(at);
                            n_children[at] = kids + 1;
                            above_target = at;
                        }
                    } else {
                        do_split = 1;
                        child = at;
                        mid = new_node(above_at);
                        target = new_node(mid);
                        above_target = mid;
                    }
                }
                target = __shfl_sync(full, target, 0);
                child = __shfl_sync(full, child, 0);
                mid = __shfl_sync(full, mid, 0);
                do_split = __shfl_sync(full, do_split, 0);
                old_front = __shfl_sync(full, old_front, 0);
                if (do_split != 0) {
                    // the upper part takes the new number: its keys are the walked keys that sit in `child`
                    uint32_t pos = 0, unl = 0;
                    for (int64_t j0 = div - 1; j0 >= 0; j0 -= 32) {
                        const int64_t j = j0 - lane;
                        const bool have = j >= 0;
                        const uint32_t id = have ? p.ids[beg + j] : 0u;
                        const uint32_t nd = have ? node_of[id] : kNone;
                        const uint32_t member = __ballot_sync(full, have && nd == child);
                        const uint32_t run = member == full ? 32u : static_cast<uint32_t>(__ffs(~member) - 1);
                        const bool mine = lane < run;
                        const uint8_t fl = mine ? flags[id] : 0;
                        if (mine) node_of[id] = mid;
                        unl += __popc(__ballot_sync(full, mine && (fl & (kCached | kListed)) == kCached));
                        pos += run;
                        if (run < 32u) break;
                    }
                    if (lane == 0) {
                        // every walked block is cached by now (hit, or just given its location back)
                        const uint32_t up = above_at;
                        n_children[mid] = 2;
                        n_blocks[mid] = pos;
                        n_last[mid] = p.ids[beg + div - 1];
                        n_cached[mid] = pos;
                        n_unlisted[mid] = unl;
                        n_blocks[child] -= pos;
                        n_cached[child] -= pos;
                        n_unlisted[child] -= unl;
                        n_parent[child] = mid;
                        n_childc[mid] = n_cached[child];
                        n_childc[up] -= n_cached[child];
                    }
                }
                __syncwarp();
                // ---- the new blocks, pushed to the front one after the other (:327-343, leaf_aware_lru.cc:20-31)
                for (int64_t base = div; base < n; base += 32) {
                    const int64_t i = base + lane;
                    if (i < n) {
                        const uint32_t id = p.ids[beg + i];
                        node_of[id] = target;
                        flags[id] = kCached | kListed;
                        time[id] = now;
                        lnext[id] = i == div ? old_front : p.ids[beg + i - 1];
                        lprev[id] = i == n - 1 ? kHead : p.ids[beg + i + 1];
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    const uint32_t cnt = static_cast<uint32_t>(n - div);
                    set_prev(old_front, p.ids[beg + div], kHead, me);
                    front_of[me] = p.ids[beg + n - 1];
                    // additions without a returned value do not wait for memory
                    atomicAdd(&n_blocks[target], cnt);
                    atomicAdd(&n_cached[target], cnt);
                    n_last[target] = p.ids[beg + n - 1];
                    atomicAdd(&n_childc[above_target], cnt);
                    wr += static_cast<int32_t>(cnt);
                }
                __syncwarp();
            }
            if (lane == 0) {
                resident += wr;
                cached_of[me] += wr;
            }
            __syncwarp();

            // ---- CheckAndEvict over the usage of the whole group (eviction_manager.cc:86-266): in turns over the
            // instances, a batch each, until a round covers the excess or takes nothing (group rough); or from the
            // writing instance only, whole batches (instance rough) or exactly the excess (instance precise).
            const int64_t resident_now = __shfl_sync(full, resident, 0);
            if (resident_now > quota) {
                const int64_t excess = resident_now - quota;
                int64_t total = 0;  // kept equal in all lanes
                n_ev = 0;
                spins = 0;
                if (p.mode == 1) {
                    while (total < excess) {
                        bool any = false;
                        for (int32_t j = 0; j < K; ++j) {  // a whole round even when the excess is covered midway
                            const int64_t got = evict_blocks(j, p.evict_batch);
                            any = any || got > 0;
                            total += got;
                        }
                        if (!any) break;
                    }
                } else {
                    while (total < excess) {
                        const int64_t rest = excess - total;
                        const int64_t count = p.mode == 3 && rest < p.evict_batch ? rest : p.evict_batch;
                        const int64_t got = evict_blocks(me, count);
                        if (got == 0) break;
                        total += got;
                    }
                }
                // CleanEmptyBlocks (radix_tree_index.cc:284-325), per instance in the reference; the trees do not
                // touch, so one pass over everything evicted does the same: childless nodes without a cached block
                // go, among the nodes that own an evicted block, until nothing more goes.  The lanes look at the
                // nodes of 32 evicted blocks at a time and remove what they find; the order of removals does not
                // change what remains.  Another round is needed only when a removal left a parent childless.
                bool again = n_ev != 0;
                while (again) {
                    again = false;
                    for (uint32_t e0 = 0; e0 < n_ev; e0 += 32) {
                        const uint32_t e = e0 + lane;
                        const uint32_t node_e = e < n_ev ? evicted[e] : 0u;
                        const bool empty = node_e >= n_roots && n_cached[node_e] == 0 && n_children[node_e] == 0 &&
                                           n_blocks[node_e] != 0;
                        const uint32_t same = __match_any_sync(full, empty ? node_e : kNone - lane);
                        bool orphaned = false;
                        if (empty && static_cast<uint32_t>(__ffs(same) - 1) == lane) {  // once per node
                            n_blocks[node_e] = 0;  // its keys are out of the tree from here on
                            const uint32_t above = n_parent[node_e];
                            orphaned = atomicSub(&n_children[above], 1u) == 1u && above >= n_roots;
                        }
                        again = __any_sync(full, orphaned) || again;
                        __syncwarp();
                    }
                }
            }
            __syncwarp();
        }
        if (lane == 0) {
            if (p.ext_hit != nullptr) {
                p.ext_hit[out0 + t] = ext;
                p.int_hit[out0 + t] = inte;
                p.written[out0 + t] = wr;
                p.cache_blocks[out0 + t] = cached_of[me];
            }
            sum_ext += ext;
            sum_int += inte;
            sum_wr += wr;
        }
        if (p.inst_blocks_trace != nullptr) {  // ReadRecord::blocks_per_instance of the reference's result records
            int64_t *row = p.inst_blocks_trace + (out0 + t) * K;
            for (int32_t j = lane; j < K; j += 32) row[j] = cached_of[j];
        }
        beg = beg1, n = n1, ty = ty1, skip = skip1, now = now1, me = me1, first_id = next_first_id;
        beg1 = beg2, n1 = n2, ty1 = ty2, skip1 = skip2, now1 = now2, me1 = me2;
    }
    if (lane == 0) {
        if (p.totals != nullptr) {
            int64_t *tot = p.totals + cfg * 4;
            tot[0] = sum_ext;
            tot[1] = sum_int;
            tot[2] = sum_wr;
            tot[3] = resident;
        }
        if (faults != 0 && p.status != nullptr) atomicAdd(&p.status[0], faults);
    }
    if (p.inst_blocks != nullptr) {
        for (int32_t j = lane; j < K; j += 32) p.inst_blocks[cfg * K + j] = cached_of[j];
    }
}

struct LeafLayout {
    uint64_t table_off, ids_off, occ_off, node_of_off, flags_off, time_off, lprev_off, lnext_off, evicted_off, nodes_off,
        blk_off, ts_off, region_off, total;
    int64_t max_nodes;
};

// with_sampling: the group holds a "random_lru" instance (block vectors and the instances' regions are added)
LeafLayout LayoutFor(int64_t n_keys, int32_t n_traces, int32_t n_configs, int32_t n_instances, bool with_sampling) {
    auto up = [](uint64_t v) { return (v + 255u) & ~static_cast<uint64_t>(255u); };
    LeafLayout l;
    const uint64_t nk = static_cast<uint64_t>(n_keys > 0 ? n_keys : 1);
    const uint64_t nc = static_cast<uint64_t>(n_configs);
    l.max_nodes = 2 * static_cast<int64_t>(n_traces) + n_instances + 1;  // the roots, and at most two new nodes per trace
    l.table_off = 256;
    l.ids_off = up(l.table_off + SlotsFor(n_keys) * sizeof(ulonglong2));
    l.occ_off = up(l.ids_off + nk * 4);
    l.node_of_off = up(l.occ_off + nk * 4);
    l.flags_off = up(l.node_of_off + nk * 4 * nc);
    l.time_off = up(l.flags_off + nk * nc);
    l.lprev_off = up(l.time_off + nk * 8 * nc);
    l.lnext_off = up(l.lprev_off + nk * 4 * nc);
    l.evicted_off = up(l.lnext_off + nk * 4 * nc);
    l.nodes_off = up(l.evicted_off + nk * 4 * nc);
    l.total = up(l.nodes_off + static_cast<uint64_t>(l.max_nodes) * 4 * kNodeFields * nc);
    l.blk_off = l.ts_off = l.region_off = l.total;
    if (with_sampling) {
        l.ts_off = up(l.blk_off + nk * 4 * nc);
        l.region_off = up(l.ts_off + nk * 8 * nc);
        l.total = up(l.region_off + (static_cast<uint64_t>(n_instances) + 1) * 8);
    }
    return l;
}

}  // namespace
}  // namespace kvcm

namespace kvcm {
namespace {

// 1 when some instance runs random_lru, 0 when none does, -1 for a policy byte that names nothing
int SamplingInstances(const uint8_t *h_instance_policy, int32_t n_instances) {
    int found = 0;
    for (int32_t j = 0; h_instance_policy != nullptr && j < n_instances; ++j) {
        if (h_instance_policy[j] > KVCM_POLICY_RANDOM_LRU) return -1;
        if (h_instance_policy[j] == KVCM_POLICY_RANDOM_LRU) found = 1;
    }
    return found;
}

bool GroupShapeOk(int64_t n_keys_total, int32_t n_traces, int32_t n_configs, int32_t n_instances) {
    return n_keys_total >= 0 && n_keys_total < (1ll << 32) - 3 - 2 * KVCM_B200_REPLAY_GROUP_MAX_INSTANCES &&
           n_traces >= 0 && n_traces < (1 << 30) && n_configs > 0 && n_configs <= 65535 && n_instances > 0 &&
           n_instances <= KVCM_B200_REPLAY_GROUP_MAX_INSTANCES;
}

}  // namespace
}  // namespace kvcm

extern "C" {

int64_t kvcm_b200_replay_policy_group_workspace_bytes(int64_t n_keys_total, int32_t n_traces, int32_t n_configs,
                                                      const uint8_t *h_instance_policy, int32_t n_instances) {
    if (!kvcm::GroupShapeOk(n_keys_total, n_traces, n_configs, n_instances)) return -1;
    const int with_sampling = kvcm::SamplingInstances(h_instance_policy, n_instances);
    if (with_sampling < 0) return -1;
    return static_cast<int64_t>(kvcm::LayoutFor(n_keys_total, n_traces, n_configs, n_instances, with_sampling != 0).total);
}

int64_t kvcm_b200_replay_leaf_lru_group_workspace_bytes(int64_t n_keys_total, int32_t n_traces, int32_t n_configs,
                                                        int32_t n_instances) {
    return kvcm_b200_replay_policy_group_workspace_bytes(n_keys_total, n_traces, n_configs, nullptr, n_instances);
}

int64_t kvcm_b200_replay_leaf_lru_workspace_bytes(int64_t n_keys_total, int32_t n_traces, int32_t n_configs) {
    return kvcm_b200_replay_leaf_lru_group_workspace_bytes(n_keys_total, n_traces, n_configs, 1);
}

int32_t kvcm_b200_replay_leaf_lru_group(const int64_t *d_keys, const int64_t *d_key_off, const uint8_t *d_trace_type,
                                        const int64_t *d_mask_off, const uint8_t *d_mask_bits,
                                        const int64_t *d_timestamps, const int32_t *d_trace_instance,
                                        int32_t n_instances, int32_t n_traces, int64_t n_keys_total,
                                        const int64_t *d_quota_blocks, int32_t n_configs, int32_t evict_batch,
                                        int32_t eviction_mode, void *d_workspace, int64_t workspace_bytes,
                                        int32_t *d_ext_hit, int32_t *d_int_hit, int32_t *d_written,
                                        int64_t *d_cache_blocks, int64_t *d_totals, int64_t *d_instance_blocks,
                                        int64_t *d_instance_blocks_per_trace, uint32_t *d_status,
                                        kvcm_stream_t stream) {
    return kvcm_b200_replay_policy_group(d_keys, d_key_off, d_trace_type, d_mask_off, d_mask_bits, d_timestamps,
                                         d_trace_instance, nullptr, nullptr, n_instances, n_traces, n_keys_total,
                                         d_quota_blocks, n_configs, evict_batch, eviction_mode, d_workspace,
                                         workspace_bytes, d_ext_hit, d_int_hit, d_written, d_cache_blocks, d_totals,
                                         d_instance_blocks, d_instance_blocks_per_trace, d_status, stream);
}

int32_t kvcm_b200_replay_tree_group(const int64_t *d_keys, const int64_t *d_key_off, const uint8_t *d_trace_type,
                                    const int64_t *d_mask_off, const uint8_t *d_mask_bits, const int64_t *d_timestamps,
                                    const int32_t *d_trace_instance, const uint8_t *h_instance_policy,
                                    int32_t n_instances, int32_t n_traces, int64_t n_keys_total,
                                    const int64_t *d_quota_blocks, int32_t n_configs, int32_t evict_batch,
                                    int32_t eviction_mode, void *d_workspace, int64_t workspace_bytes,
                                    int32_t *d_ext_hit, int32_t *d_int_hit, int32_t *d_written, int64_t *d_cache_blocks,
                                    int64_t *d_totals, int64_t *d_instance_blocks,
                                    int64_t *d_instance_blocks_per_trace, uint32_t *d_status, kvcm_stream_t stream) {
    if (n_instances > 0 && n_instances <= KVCM_B200_REPLAY_GROUP_MAX_INSTANCES &&
        kvcm::SamplingInstances(h_instance_policy, n_instances) != 0) {
        return KVCM_EC_BADARGS;  // the two queue policies only
    }
    return kvcm_b200_replay_policy_group(d_keys, d_key_off, d_trace_type, d_mask_off, d_mask_bits, d_timestamps,
                                         d_trace_instance, h_instance_policy, nullptr, n_instances, n_traces,
                                         n_keys_total, d_quota_blocks, n_configs, evict_batch, eviction_mode,
                                         d_workspace, workspace_bytes, d_ext_hit, d_int_hit, d_written, d_cache_blocks,
                                         d_totals, d_instance_blocks, d_instance_blocks_per_trace, d_status, stream);
}

int32_t kvcm_b200_replay_policy_group(const int64_t *d_keys, const int64_t *d_key_off, const uint8_t *d_trace_type,
                                      const int64_t *d_mask_off, const uint8_t *d_mask_bits, const int64_t *d_timestamps,
                                      const int32_t *d_trace_instance, const uint8_t *h_instance_policy,
                                      const double *h_sample_rate, int32_t n_instances, int32_t n_traces,
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
    if (!kvcm::GroupShapeOk(n_keys_total, n_traces, n_configs, n_instances)) return KVCM_EC_OUT_OF_LIMIT;
    const int with_sampling = kvcm::SamplingInstances(h_instance_policy, n_instances);
    if (with_sampling < 0) return KVCM_EC_BADARGS;
    kvcm::LeafSweep p;
    uint64_t lru_instances = 0, sampling_instances = 0;
    for (int32_t j = 0; j < KVCM_B200_REPLAY_GROUP_MAX_INSTANCES; ++j) p.sampling_size[j] = 0;
    for (int32_t j = 0; h_instance_policy != nullptr && j < n_instances; ++j) {
        if (h_instance_policy[j] == KVCM_POLICY_LRU) lru_instances |= 1ull << j;
        if (h_instance_policy[j] != KVCM_POLICY_RANDOM_LRU) continue;
        sampling_instances |= 1ull << j;
        // RandomLruEvictionPolicy's constructor (random_lru.cc:5-14): a rate <= 0 means 0.1; the size is a double
        // division cut to an integer
        double rate = h_sample_rate != nullptr ? h_sample_rate[j] : 0.0;
        if (rate <= 0.0) rate = 0.1;
        const double size = static_cast<double>(evict_batch) / rate;
        if (static_cast<uint32_t>(evict_batch) > kvcm::kMaxBatch || size > static_cast<double>(kvcm::kMaxSample) ||
            size < 1.0) {
            return KVCM_EC_OUT_OF_LIMIT;
        }
        p.sampling_size[j] = static_cast<uint32_t>(size);
    }
    if (n_traces == 0) return KVCM_OK;
    const int per_trace = (d_ext_hit != nullptr) + (d_int_hit != nullptr) + (d_written != nullptr) +
                          (d_cache_blocks != nullptr);
    if (d_key_off == nullptr || d_trace_type == nullptr || d_quota_blocks == nullptr || d_workspace == nullptr ||
        (d_trace_instance == nullptr && n_instances > 1) || (d_keys == nullptr && n_keys_total > 0) ||
        (per_trace != 0 && per_trace != 4) || (per_trace == 0 && d_totals == nullptr)) {
        return KVCM_ER_INVALID_ADDRESS;
    }
    if (reinterpret_cast<uintptr_t>(d_workspace) & 255u) return KVCM_ER_INVALID_ADDRESS;
    const kvcm::LeafLayout l = kvcm::LayoutFor(n_keys_total, n_traces, n_configs, n_instances, with_sampling != 0);
    if (workspace_bytes < static_cast<int64_t>(l.total)) return KVCM_EC_NOSPC;
    uint8_t *ws = static_cast<uint8_t *>(d_workspace);
    kvcm::IdTable t;
    t.cells = reinterpret_cast<unsigned long long *>(ws);
    t.slots = reinterpret_cast<ulonglong2 *>(ws + l.table_off);
    t.mask = kvcm::SlotsFor(n_keys_total) - 1;
    uint32_t *ids = reinterpret_cast<uint32_t *>(ws + l.ids_off);
    uint32_t *occ = reinterpret_cast<uint32_t *>(ws + l.occ_off);
    int64_t *region_base = reinterpret_cast<int64_t *>(ws + l.region_off);
    const uint64_t nk = static_cast<uint64_t>(n_keys_total > 0 ? n_keys_total : 1);
    cudaStream_t s = kvcm::AsStream(stream);
    const int sms = kvcm::GetDeviceInfo().sm_count;
    p.ids = ids;
    p.occ = occ;
    p.key_off = d_key_off;
    p.type = d_trace_type;
    p.mask_off = d_mask_off;
    p.mask_bits = d_mask_bits;
    p.timestamps = d_timestamps;
    p.trace_inst = d_trace_instance;
    p.quota = d_quota_blocks;
    p.node_of = reinterpret_cast<uint32_t *>(ws + l.node_of_off);
    p.flags = ws + l.flags_off;
    p.time = reinterpret_cast<int64_t *>(ws + l.time_off);
    p.lprev = reinterpret_cast<uint32_t *>(ws + l.lprev_off);
    p.lnext = reinterpret_cast<uint32_t *>(ws + l.lnext_off);
    p.evicted = reinterpret_cast<uint32_t *>(ws + l.evicted_off);
    p.nodes = reinterpret_cast<uint32_t *>(ws + l.nodes_off);
    p.blk = with_sampling != 0 ? reinterpret_cast<uint32_t *>(ws + l.blk_off) : nullptr;
    p.ts = with_sampling != 0 ? reinterpret_cast<int64_t *>(ws + l.ts_off) : nullptr;
    p.region_base = with_sampling != 0 ? region_base : nullptr;
    p.ext_hit = d_ext_hit;
    p.int_hit = d_int_hit;
    p.written = d_written;
    p.cache_blocks = d_cache_blocks;
    p.totals = d_totals;
    p.inst_blocks = d_instance_blocks;
    p.inst_blocks_trace = d_instance_blocks_per_trace;
    p.status = d_status;
    p.n_keys = static_cast<int64_t>(nk);
    p.n_ids = n_keys_total;
    p.max_nodes = l.max_nodes;
    p.n_traces = n_traces;
    p.n_configs = n_configs;
    p.evict_batch = evict_batch;
    p.n_instances = n_instances;
    p.mode = eviction_mode;
    p.lru_instances = lru_instances;
    p.sampling_instances = sampling_instances;
    kvcm::LeafInitKernel<<<sms * 8, 256, 0, s>>>(t, p.node_of, p.flags, nk * static_cast<uint64_t>(n_configs));
    if (d_trace_instance != nullptr) {
        kvcm::LeafCheckInstancesKernel<<<sms, 256, 0, s>>>(d_trace_instance, n_traces, n_instances, d_status);
    }
    if (with_sampling != 0) {
        if (d_trace_instance != nullptr) {
            kvcm::LruGroupExtentKernel<<<1, 1024, sizeof(unsigned long long) * n_instances, s>>>(
                d_key_off, d_trace_instance, n_traces, n_instances, region_base, nullptr);
        } else {
            cudaMemsetAsync(region_base, 0, 2 * sizeof(int64_t), s);  // one instance: its vector starts at 0
        }
    }
    if (n_keys_total > 0) {
        if (d_trace_instance == nullptr) {
            kvcm::LruClaimIdsKernel<<<sms * 8, 256, 0, s>>>(t, d_keys, n_keys_total, d_status);
            kvcm::LruLookupIdsKernel<<<sms * 8, 256, 0, s>>>(t, d_keys, n_keys_total, ids);
        } else {
            // keys of traces that name no instance of the group keep id 0: the sweep replays those traces as empty
            cudaMemsetAsync(ids, 0, static_cast<size_t>(n_keys_total) * sizeof(uint32_t), s);
            // one instance after the other: the table starts empty each time, the id counter runs on
            for (int32_t j = 0; j < n_instances; ++j) {
                if (j > 0) kvcm::IdTableClearKernel<<<sms * 8, 256, 0, s>>>(t);
                kvcm::LruClaimIdsOfInstanceKernel<<<sms * 4, 256, 0, s>>>(t, d_keys, d_key_off, d_trace_instance,
                                                                         n_traces, j, d_status);
                kvcm::LruLookupIdsOfInstanceKernel<<<sms * 4, 256, 0, s>>>(t, d_keys, d_key_off, d_trace_instance,
                                                                          n_traces, j, ids);
            }
        }
        kvcm::LeafOccKernel<<<sms * 4, 256, 0, s>>>(ids, d_key_off, d_trace_instance, n_instances, n_traces, occ);
    }
    const size_t per_instance = sizeof(int64_t) * static_cast<size_t>(n_instances);
    if (with_sampling != 0) {
        kvcm::LeafSweepKernel<true><<<static_cast<unsigned>(n_configs), 32,
                                      4 * per_instance + sizeof(kvcm::SamplingScratch), s>>>(p);
    } else {
        kvcm::LeafSweepKernel<false><<<static_cast<unsigned>(n_configs), 32, 2 * per_instance, s>>>(p);
    }
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_replay_leaf_lru(const int64_t *d_keys, const int64_t *d_key_off, const uint8_t *d_trace_type,
                                  const int64_t *d_mask_off, const uint8_t *d_mask_bits, const int64_t *d_timestamps,
                                  int32_t n_traces, int64_t n_keys_total, const int64_t *d_quota_blocks,
                                  int32_t n_configs, int32_t evict_batch, int32_t precise, void *d_workspace,
                                  int64_t workspace_bytes, int32_t *d_ext_hit, int32_t *d_int_hit, int32_t *d_written,
                                  int64_t *d_cache_blocks, int64_t *d_totals, uint32_t *d_status,
                                  kvcm_stream_t stream) {
    return kvcm_b200_replay_leaf_lru_group(d_keys, d_key_off, d_trace_type, d_mask_off, d_mask_bits, d_timestamps,
                                           nullptr, 1, n_traces, n_keys_total, d_quota_blocks, n_configs, evict_batch,
                                           precise != 0 ? 3 : 2, d_workspace, workspace_bytes, d_ext_hit, d_int_hit,
                                           d_written, d_cache_blocks, d_totals, nullptr, nullptr, d_status, stream);
}

}  // extern "C"
