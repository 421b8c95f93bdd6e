// Optimizer trace replay with the "random_lru" eviction policy, for a sweep of cache quotas at once (sm_100a).
//
// Stands in for OptimizerRunner::RunTraces (kv_cache_manager/optimizer/manager/optimizer_runner.cc:29-215) over
// RadixTreeIndex (kv_cache_manager/optimizer/index/radix_tree_index.cc:19-392) with RandomLruEvictionPolicy
// (kv_cache_manager/optimizer/eviction_policy/random_lru.cc:5-131, random_lru.h:13-47) and the quota check after
// every write (OptIndexerManager::CheckAndEvict, kv_cache_manager/optimizer/manager/indexer_manager.cc:55-90;
// OptEvictionManager::EvictByGroupRough / EvictByInstanceRough / EvictByInstancePrecise,
// manager/eviction_manager.cc:86-239), for one instance or for a group of instances that share the quota: every
// instance has its own block vector (a region of blk / ts), its own generator and its own sampling size; ids are
// unique over (instance, key).
//
// One warp replays one quota point, as in the "lru" sweep, and the tree collapses to per-key state for the same
// reasons (keys are prefix-unique; a trace touches its leading cached blocks, then writes its missing ones).  The
// policy itself - block vector, sampling, partial sort, swap-and-pop - is in replay_sampling.cuh.
#include "kvcm_common.cuh"
#include "replay_ids.cuh"
#include "replay_sampling.cuh"

namespace kvcm {
namespace {

__global__ void RandomInitKernel(IdTable t, uint32_t *pos, uint64_t n_pos) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    const uint64_t first = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (uint64_t i = first; i <= t.mask; i += stride) t.slots[i] = make_ulonglong2(kEmptyKey, ~0ull);
    for (uint64_t i = first; i < n_pos; i += stride) pos[i] = kNotCached;
    if (first == 0) {
        t.cells[0] = 0ull;
        t.cells[1] = ~0ull;
    }
}

struct RandomSweep {
    const uint32_t *ids;
    const int64_t *key_off;
    const uint8_t *type;
    const int64_t *mask_off;
    const uint8_t *mask_bits;
    const int64_t *timestamps;  // per trace; null = the trace number
    const int64_t *quota;
    uint32_t *pos;  // [n_configs][n_keys]
    uint32_t *blk;  // [n_configs][n_keys]
    int64_t *ts;    // [n_configs][n_keys]
    int32_t *ext_hit, *int_hit, *written;  // per trace; all four may be null when only totals are wanted
    int64_t *cache_blocks;
    int64_t *totals;  // [n_configs][4]
    int64_t n_keys;
    int32_t n_traces;
    int32_t n_configs;
    int32_t evict_batch;
    const int32_t *trace_inst;   // optional, per trace, 0 .. n_instances-1; instance 0 when null
    const int64_t *region_base;  // [n_instances + 1]: where each instance's block vector starts; null = one instance at 0
    int64_t *inst_blocks;        // optional, [n_configs][n_instances]: usage per instance at the end
    int64_t *inst_blocks_trace;  // optional, [n_configs][n_traces][n_instances]: usage of every instance after each trace
    int32_t n_instances;
    int32_t mode;  // 1 group rough, 2 instance rough, 3 instance precise
    uint32_t sampling_size[KVCM_B200_REPLAY_GROUP_MAX_INSTANCES];  // per instance
};

// type: 0 DialogTurn (InsertWithQuery), 1 GetLocation (PrefixQuery), 2 WriteCache (InsertOnly).
__global__ void __launch_bounds__(32) RandomLruSweepKernel(const RandomSweep p) {
    __shared__ SamplingScratch scratch;
    extern __shared__ int64_t per_inst[];
    const int32_t K = p.n_instances;
    int64_t *size_of = per_inst;      // [K] cached blocks of the instance = the length of its block vector
    int64_t *base_of = per_inst + K;  // [K] where its block vector starts in blk / ts
    uint64_t *rng_of = reinterpret_cast<uint64_t *>(per_inst + 2 * K);  // [K] the state of its generator
    const int32_t cfg = blockIdx.x;
    const uint32_t lane = LaneId();
    uint32_t *pos = p.pos + static_cast<int64_t>(cfg) * p.n_keys;
    uint32_t *blk_all = p.blk + static_cast<int64_t>(cfg) * p.n_keys;
    int64_t *ts_all = p.ts + static_cast<int64_t>(cfg) * p.n_keys;
    const int64_t quota = p.quota[cfg];
    const int64_t out0 = static_cast<int64_t>(cfg) * p.n_traces;
    int64_t resident = 0;  // of the whole group
    int64_t sum_ext = 0, sum_int = 0, sum_wr = 0;
    for (int32_t j = lane; j < K; j += 32) {
        size_of[j] = 0;
        base_of[j] = p.region_base != nullptr ? p.region_base[j] : 0;
        rng_of[j] = kSamplingSeed;
    }
    __syncwarp();

    auto evict_round = [&](int32_t j, int64_t count) -> uint32_t {
        const int64_t held = size_of[j];
        const uint32_t got = SamplingEvictRound(scratch, pos, blk_all + base_of[j], ts_all + base_of[j], held,
                                                &rng_of[j], p.sampling_size[j], count, lane);
        if (lane == 0) size_of[j] = held - got;
        __syncwarp();
        return got;
    };

    for (int32_t t = 0; t < p.n_traces; ++t) {
        const int64_t beg = p.key_off[t];
        int64_t n = p.key_off[t + 1] - beg;
        const uint8_t ty = p.type[t];
        const int64_t skip = (ty == 1 && p.mask_off != nullptr) ? p.mask_off[t] : 0;
        const int64_t now = p.timestamps != nullptr ? p.timestamps[t] : static_cast<int64_t>(t);
        int32_t me = p.trace_inst != nullptr ? p.trace_inst[t] : 0;
        if (me < 0 || me >= K) {  // counted by the extent kernel; its keys have no ids: an empty trace
            me = 0;
            n = 0;
        }
        const int64_t my_size = size_of[me];
        const SamplingTraceCounts c = SamplingReplayTrace(
            p.ids + beg, p.mask_bits != nullptr ? p.mask_bits + beg : nullptr, n, ty, skip, now, pos,
            blk_all + base_of[me], ts_all + base_of[me], my_size, lane);
        resident += c.wr;
        if (lane == 0) size_of[me] = my_size + c.wr;
        __syncwarp();
        if (ty != 1 && resident > quota) {
            // CheckAndEvict over the usage of the whole group: in turns over the instances, a batch each, until a
            // round covers the excess or takes nothing (group rough); or from the writing instance only, whole
            // batches (instance rough) or exactly the excess (instance precise).
            const int64_t excess = resident - quota;
            int64_t total = 0;
            if (p.mode == 1) {
                while (total < excess) {
                    bool any = false;
                    for (int32_t j = 0; j < K; ++j) {  // a whole round even when the excess is covered midway
                        const uint32_t got = evict_round(j, p.evict_batch);
                        any = any || got != 0;
                        total += got;
                    }
                    if (!any) break;
                }
            } else {
                while (total < excess) {
                    int64_t count = p.evict_batch;
                    if (p.mode == 3 && excess - total < count) count = excess - total;
                    const uint32_t got = evict_round(me, count);
                    if (got == 0) break;
                    total += got;
                }
            }
            resident -= total;
        }
        if (lane == 0 && p.ext_hit != nullptr) {
            p.ext_hit[out0 + t] = c.ext;
            p.int_hit[out0 + t] = c.inte;
            p.written[out0 + t] = c.wr;
            p.cache_blocks[out0 + t] = size_of[me];
        }
        if (p.inst_blocks_trace != nullptr) {  // ReadRecord::blocks_per_instance of the reference's result records
            int64_t *row = p.inst_blocks_trace + (out0 + t) * K;
            for (int32_t j = lane; j < K; j += 32) row[j] = size_of[j];
        }
        sum_ext += c.ext;
        sum_int += c.inte;
        sum_wr += c.wr;
    }
    if (lane == 0 && p.totals != nullptr) {
        int64_t *tot = p.totals + static_cast<int64_t>(cfg) * 4;
        tot[0] = sum_ext;
        tot[1] = sum_int;
        tot[2] = sum_wr;
        tot[3] = resident;
    }
    if (p.inst_blocks != nullptr) {
        for (int32_t j = lane; j < K; j += 32) p.inst_blocks[static_cast<int64_t>(cfg) * K + j] = size_of[j];
    }
}

struct RandomLayout {
    size_t table_off, ids_off, pos_off, blk_off, ts_off, total;
};

RandomLayout RandomLayoutFor(int64_t n_keys, int32_t n_configs) {
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    const size_t keys = static_cast<size_t>(n_keys > 0 ? n_keys : 1);
    RandomLayout l;
    l.table_off = 256;
    l.ids_off = l.table_off + up(SlotsFor(n_keys) * sizeof(ulonglong2));
    l.pos_off = l.ids_off + up(keys * sizeof(uint32_t));
    l.blk_off = l.pos_off + up(keys * n_configs * sizeof(uint32_t));
    l.ts_off = l.blk_off + up(keys * n_configs * sizeof(uint32_t));
    l.total = l.ts_off + up(keys * n_configs * sizeof(int64_t));
    return l;
}

}  // namespace
}  // namespace kvcm

extern "C" {

int32_t kvcm_b200_selftest_partial_sort(uint32_t *h_idx, int64_t *h_times, uint32_t k, uint32_t n) {
    if (h_idx == nullptr || h_times == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (k > n) return KVCM_EC_BADARGS;
    std::vector<kvcm::SampleEntry> s(n);
    for (uint32_t i = 0; i < n; ++i) s[i] = kvcm::SampleEntry{h_times[i], h_idx[i], 0};
    kvcm::PartialSortByTime(s.data(), k, n);
    for (uint32_t i = 0; i < n; ++i) {
        h_times[i] = s[i].t;
        h_idx[i] = s[i].idx;
    }
    return KVCM_OK;
}

int64_t kvcm_b200_replay_random_lru_group_workspace_bytes(int64_t n_keys_total, int32_t n_configs,
                                                          int32_t n_instances) {
    if (n_keys_total < 0 || n_keys_total >= (1ll << 32) - 1 || n_configs <= 0 || n_configs > 65535 || n_instances <= 0 ||
        n_instances > KVCM_B200_REPLAY_GROUP_MAX_INSTANCES) {
        return -1;
    }
    return static_cast<int64_t>(kvcm::RandomLayoutFor(n_keys_total, n_configs).total) +
           ((static_cast<int64_t>(n_instances) + 1) * 8 + 255) / 256 * 256;
}

int64_t kvcm_b200_replay_random_lru_workspace_bytes(int64_t n_keys_total, int32_t n_configs) {
    return kvcm_b200_replay_random_lru_group_workspace_bytes(n_keys_total, n_configs, 1);
}

int32_t kvcm_b200_replay_random_lru_group(const int64_t *d_keys, const int64_t *d_key_off, const uint8_t *d_trace_type,
                                          const int64_t *d_mask_off, const uint8_t *d_mask_bits,
                                          const int64_t *d_timestamps, const int32_t *d_trace_instance,
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
    const int64_t need = kvcm_b200_replay_random_lru_group_workspace_bytes(n_keys_total, n_configs, n_instances);
    if (need < 0) return KVCM_EC_OUT_OF_LIMIT;
    kvcm::RandomSweep p;
    for (int32_t j = 0; j < n_instances; ++j) {
        // RandomLruEvictionPolicy's constructor (random_lru.cc:5-14): a rate <= 0 means 0.1; the size is a double
        // division cut to an integer
        double rate = h_sample_rate != nullptr ? h_sample_rate[j] : 0.0;
        if (rate <= 0.0) rate = 0.1;
        const double sampling = static_cast<double>(evict_batch) / rate;
        if (static_cast<uint32_t>(evict_batch) > kvcm::kMaxBatch || sampling > static_cast<double>(kvcm::kMaxSample) ||
            sampling < 1.0) {
            return KVCM_EC_OUT_OF_LIMIT;
        }
        p.sampling_size[j] = static_cast<uint32_t>(sampling);
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
    if (workspace_bytes < need) return KVCM_EC_NOSPC;
    const kvcm::RandomLayout l = kvcm::RandomLayoutFor(n_keys_total, n_configs);
    uint8_t *ws = static_cast<uint8_t *>(d_workspace);
    kvcm::IdTable t;
    t.cells = reinterpret_cast<unsigned long long *>(ws);
    t.slots = reinterpret_cast<ulonglong2 *>(ws + l.table_off);
    t.mask = kvcm::SlotsFor(n_keys_total) - 1;
    uint32_t *ids = reinterpret_cast<uint32_t *>(ws + l.ids_off);
    uint32_t *pos = reinterpret_cast<uint32_t *>(ws + l.pos_off);
    int64_t *region_base = reinterpret_cast<int64_t *>(ws + l.total);
    cudaStream_t s = kvcm::AsStream(stream);
    const int sms = kvcm::GetDeviceInfo().sm_count;
    const uint64_t n_pos = static_cast<uint64_t>(n_keys_total > 0 ? n_keys_total : 1) * static_cast<uint64_t>(n_configs);
    kvcm::RandomInitKernel<<<sms * 8, 256, 0, s>>>(t, pos, n_pos);
    if (d_trace_instance == nullptr) {
        if (n_keys_total > 0) {
            kvcm::LruClaimIdsKernel<<<sms * 8, 256, 0, s>>>(t, d_keys, n_keys_total, d_status);
            kvcm::LruLookupIdsKernel<<<sms * 8, 256, 0, s>>>(t, d_keys, n_keys_total, ids);
        }
    } else {
        kvcm::LruGroupExtentKernel<<<1, 1024, sizeof(unsigned long long) * n_instances, s>>>(
            d_key_off, d_trace_instance, n_traces, n_instances, region_base, d_status);
        // one instance after the other: the table starts empty each time, the id counter runs on
        for (int32_t j = 0; n_keys_total > 0 && j < n_instances; ++j) {
            if (j > 0) kvcm::IdTableClearKernel<<<sms * 8, 256, 0, s>>>(t);
            kvcm::LruClaimIdsOfInstanceKernel<<<sms * 4, 256, 0, s>>>(t, d_keys, d_key_off, d_trace_instance, n_traces, j,
                                                                     d_status);
            kvcm::LruLookupIdsOfInstanceKernel<<<sms * 4, 256, 0, s>>>(t, d_keys, d_key_off, d_trace_instance, n_traces,
                                                                      j, ids);
        }
    }
    p.ids = ids;
    p.key_off = d_key_off;
    p.type = d_trace_type;
    p.mask_off = d_mask_off;
    p.mask_bits = d_mask_bits;
    p.timestamps = d_timestamps;
    p.quota = d_quota_blocks;
    p.pos = pos;
    p.blk = reinterpret_cast<uint32_t *>(ws + l.blk_off);
    p.ts = reinterpret_cast<int64_t *>(ws + l.ts_off);
    p.ext_hit = d_ext_hit;
    p.int_hit = d_int_hit;
    p.written = d_written;
    p.cache_blocks = d_cache_blocks;
    p.totals = d_totals;
    p.n_keys = n_keys_total > 0 ? n_keys_total : 1;
    p.n_traces = n_traces;
    p.n_configs = n_configs;
    p.evict_batch = evict_batch;
    p.trace_inst = d_trace_instance;
    p.region_base = d_trace_instance != nullptr ? region_base : nullptr;
    p.inst_blocks = d_instance_blocks;
    p.inst_blocks_trace = d_instance_blocks_per_trace;
    p.n_instances = n_instances;
    p.mode = eviction_mode;
    kvcm::RandomLruSweepKernel<<<static_cast<unsigned>(n_configs), 32, sizeof(int64_t) * 3 * n_instances, s>>>(p);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_replay_random_lru(const int64_t *d_keys, const int64_t *d_key_off, const uint8_t *d_trace_type,
                                    const int64_t *d_mask_off, const uint8_t *d_mask_bits, const int64_t *d_timestamps,
                                    int32_t n_traces, int64_t n_keys_total, const int64_t *d_quota_blocks,
                                    int32_t n_configs, int32_t evict_batch, int32_t precise, double sample_rate,
                                    void *d_workspace, int64_t workspace_bytes, int32_t *d_ext_hit, int32_t *d_int_hit,
                                    int32_t *d_written, int64_t *d_cache_blocks, int64_t *d_totals, uint32_t *d_status,
                                    kvcm_stream_t stream) {
    return kvcm_b200_replay_random_lru_group(d_keys, d_key_off, d_trace_type, d_mask_off, d_mask_bits, d_timestamps,
                                             nullptr, &sample_rate, 1, n_traces, n_keys_total, d_quota_blocks,
                                             n_configs, evict_batch, precise != 0 ? 3 : 2, d_workspace, workspace_bytes,
                                             d_ext_hit, d_int_hit, d_written, d_cache_blocks, d_totals, nullptr, nullptr,
                                             d_status, stream);
}

}  // extern "C"
