// Optimizer trace replay without eviction, as two data-parallel passes (sm_100a).
//
// Stands in for the sequential loop OptimizerRunner::RunTraces
// (kv_cache_manager/optimizer/manager/optimizer_runner.cc:29-215) over RadixTreeIndex
// (kv_cache_manager/optimizer/index/radix_tree_index.cc:19-282).  The reference replays one
// trace at a time because trace t must see exactly the blocks written by traces < t.  Without
// eviction that order dependence collapses to one number per key - the sequence number of the
// first trace that writes it:
//   pass 1  every writing trace t does atomicMin(first_writer[key], t) for each of its keys;
//   pass 2  trace t counts its leading keys with first_writer < t (hits: cached before t) and
//           its keys with first_writer == t (blocks it wrote itself).
// This equals the prefix-tree walk when keys are prefix-unique chained block hashes (a key
// determines its whole prefix), which is what GenKeyVector and ApplyPrefixHash produce.
//
// Scratch: an open-addressing table {int64 key, uint64 first_writer} in caller-provided
// workspace, 16-byte slots, at least twice as many slots as keys.
#include <mutex>

#include <algorithm>
#include <string>
#include <unordered_map>
#include <vector>

#include "kvcm_common.cuh"

// Scratch of kvcm_b200_replay_noalloc: a fixed table that lives in the library's device image.
// Every GPU that loads the library holds these bytes until the process exits.
static __device__ __align__(256) unsigned char g_replay_noalloc_scratch[KVCM_B200_REPLAY_NOALLOC_SCRATCH_BYTES];

namespace kvcm {
namespace {

constexpr uint64_t kNoWriter = ~0ull;
constexpr int kWarps = 8;

struct ReplayTable {
    ulonglong2 *slots;
    unsigned long long *cells;  // first_writer of the key equal to kEmptyKey
    uint64_t mask;
};

__global__ void ReplayInitKernel(ReplayTable t) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i <= t.mask; i += stride) {
        t.slots[i] = make_ulonglong2(kEmptyKey, kNoWriter);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) t.cells[0] = kNoWriter;
}

// Pointer to the first_writer word of `key`, claiming a slot when `insert`.  nullptr when the
// key is absent (lookup) or the bounded probe sequence found no room (insert).
__device__ __forceinline__ unsigned long long *FindWriterWord(const ReplayTable &t, uint64_t key, bool insert) {
    if (key == kEmptyKey) return &t.cells[0];
    unsigned long long *words = reinterpret_cast<unsigned long long *>(t.slots);
    uint64_t slot = Mix(key) & t.mask;
    for (uint64_t probe = 0; probe <= t.mask; ++probe) {
        unsigned long long seen = *reinterpret_cast<volatile unsigned long long *>(&words[2 * slot]);
        if (seen == kEmptyKey && insert) seen = atomicCAS(&words[2 * slot], kEmptyKey, key);
        if (seen == key || (seen == kEmptyKey && insert)) return &words[2 * slot + 1];
        if (seen == kEmptyKey) return nullptr;
        slot = (slot + 1) & t.mask;
    }
    return nullptr;
}

// type: 0 DialogTurn (reads and writes), 1 GetLocation (reads), 2 WriteCache (writes).
__global__ void __launch_bounds__(kWarps * 32)
    ReplayFirstWriterKernel(ReplayTable t, const int64_t *__restrict__ keys, const int64_t *__restrict__ key_off,
                            const uint8_t *__restrict__ type, int32_t n_traces, uint32_t *status) {
    const int32_t trace = blockIdx.x * kWarps + (threadIdx.x >> 5);
    if (trace >= n_traces || type[trace] == 1) return;
    const int64_t beg = key_off[trace], end = key_off[trace + 1];
    for (int64_t i = beg + LaneId(); i < end; i += 32) {
        unsigned long long *w = FindWriterWord(t, static_cast<uint64_t>(keys[i]), true);
        if (w != nullptr) {
            atomicMin(w, static_cast<unsigned long long>(trace));
        } else if (status != nullptr) {
            atomicAdd(&status[0], 1u);
        }
    }
}

__global__ void __launch_bounds__(kWarps * 32)
    ReplayCountKernel(ReplayTable t, const int64_t *__restrict__ keys, const int64_t *__restrict__ key_off,
                      const uint8_t *__restrict__ type, const int64_t *__restrict__ mask_off,
                      const uint8_t *__restrict__ mask_bits, int32_t n_traces,
                      int32_t *__restrict__ ext_hit, int32_t *__restrict__ int_hit, int32_t *__restrict__ written) {
    const int32_t trace = blockIdx.x * kWarps + (threadIdx.x >> 5);
    if (trace >= n_traces) return;
    const uint32_t lane = LaneId();
    const int64_t beg = key_off[trace];
    const int64_t n = key_off[trace + 1] - beg;
    const uint8_t ty = type[trace];
    const int64_t skip = (ty == 1 && mask_off != nullptr) ? mask_off[trace] : 0;
    const unsigned long long me = static_cast<unsigned long long>(trace);
    int32_t ext = 0, inte = 0, wr = 0;
    bool prefix_alive = ty != 2;  // WriteCache traces record no hits
    for (int64_t base = 0; base < n; base += 32) {
        const int64_t i = base + lane;
        unsigned long long first = kNoWriter;
        if (i < n) {
            const unsigned long long *w = FindWriterWord(t, static_cast<uint64_t>(keys[beg + i]), false);
            if (w != nullptr) first = *w;
        }
        const uint32_t in_range = __ballot_sync(0xffffffffu, i < n);
        const uint32_t before = __ballot_sync(0xffffffffu, i < n && first < me);
        const uint32_t mine = __ballot_sync(0xffffffffu, i < n && first == me);
        const uint32_t masked =
            __ballot_sync(0xffffffffu, i < skip || (ty == 1 && mask_bits != nullptr && i < n && mask_bits[beg + i] != 0));
        if (ty != 1) wr += __popc(mine);
        if (prefix_alive) {
            const uint32_t miss = in_range & ~before;
            const uint32_t lead = miss != 0 ? ((1u << (__ffs(miss) - 1)) - 1u) : 0xffffffffu;
            ext += __popc(before & lead & ~masked);
            inte += __popc(before & lead & masked);
            if (miss != 0) prefix_alive = false;
        }
        if (!prefix_alive && ty == 1) break;
    }
    if (lane == 0) {
        ext_hit[trace] = ext;
        int_hit[trace] = inte;
        written[trace] = wr;
    }
}

// cache_blocks[t] = base + written[0] + ... + written[t]; one CTA, each thread owns a contiguous span.
__global__ void __launch_bounds__(1024)
    ReplayRunningSizeKernel(const int32_t *__restrict__ written, int32_t n, int64_t base, int64_t *__restrict__ out) {
    __shared__ int64_t partial[1024];
    const int tid = threadIdx.x;
    const int64_t span = (static_cast<int64_t>(n) + blockDim.x - 1) / blockDim.x;
    const int64_t lo = min(static_cast<int64_t>(n), tid * span), hi = min(static_cast<int64_t>(n), lo + span);
    int64_t sum = 0;
    for (int64_t i = lo; i < hi; ++i) sum += written[i];
    partial[tid] = sum;
    __syncthreads();
    for (int d = 1; d < blockDim.x; d <<= 1) {
        const int64_t add = tid >= d ? partial[tid - d] : 0;
        __syncthreads();
        partial[tid] += add;
        __syncthreads();
    }
    int64_t acc = base + partial[tid] - sum;
    for (int64_t i = lo; i < hi; ++i) {
        acc += written[i];
        out[i] = acc;
    }
}

uint64_t SlotsFor(int64_t n_keys) {
    uint64_t n = 1024;
    while (n < 2ull * static_cast<uint64_t>(n_keys)) n <<= 1;
    return n;
}

}  // namespace
}  // namespace kvcm

extern "C" {

int64_t kvcm_b200_replay_workspace_bytes(int64_t n_keys_total) {
    if (n_keys_total < 0 || n_keys_total > (1ll << 36)) return -1;
    return static_cast<int64_t>(kvcm::SlotsFor(n_keys_total) * sizeof(ulonglong2) + 256);
}

int32_t kvcm_b200_replay(const int64_t *d_keys, const int64_t *d_key_off, const uint8_t *d_trace_type,
                         const int64_t *d_mask_off, const uint8_t *d_mask_bits, int32_t n_traces,
                         int64_t n_keys_total, void *d_workspace,
                         int64_t workspace_bytes, int32_t *d_ext_hit, int32_t *d_int_hit, int32_t *d_written,
                         int64_t *d_cache_blocks, uint32_t *d_status, kvcm_stream_t stream) {
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (n_traces < 0 || n_keys_total < 0) return KVCM_EC_BADARGS;
    if (n_traces == 0) return KVCM_OK;
    if (d_key_off == nullptr || d_trace_type == nullptr || d_ext_hit == nullptr || d_int_hit == nullptr ||
        d_written == nullptr || d_workspace == nullptr || (d_keys == nullptr && n_keys_total > 0)) {
        return KVCM_ER_INVALID_ADDRESS;
    }
    if (reinterpret_cast<uintptr_t>(d_workspace) & 255u) return KVCM_ER_INVALID_ADDRESS;
    const int64_t need = kvcm_b200_replay_workspace_bytes(n_keys_total);
    if (need < 0 || workspace_bytes < need) return KVCM_EC_NOSPC;
    kvcm::ReplayTable t;
    t.cells = static_cast<unsigned long long *>(d_workspace);
    t.slots = reinterpret_cast<ulonglong2 *>(static_cast<uint8_t *>(d_workspace) + 256);
    t.mask = kvcm::SlotsFor(n_keys_total) - 1;
    cudaStream_t s = kvcm::AsStream(stream);
    kvcm::ReplayInitKernel<<<kvcm::GetDeviceInfo().sm_count * 8, 256, 0, s>>>(t);
    const unsigned grid = static_cast<unsigned>((n_traces + kvcm::kWarps - 1) / kvcm::kWarps);
    kvcm::ReplayFirstWriterKernel<<<grid, kvcm::kWarps * 32, 0, s>>>(t, d_keys, d_key_off, d_trace_type, n_traces,
                                                                     d_status);
    kvcm::ReplayCountKernel<<<grid, kvcm::kWarps * 32, 0, s>>>(t, d_keys, d_key_off, d_trace_type, d_mask_off,
                                                               d_mask_bits, n_traces, d_ext_hit, d_int_hit, d_written);
    if (d_cache_blocks != nullptr) {
        kvcm::ReplayRunningSizeKernel<<<1, 1024, 0, s>>>(d_written, n_traces, 0, d_cache_blocks);
    }
    return kvcm::LaunchStatus();
}

// The replay for callers that must not allocate.  Same contract and same kernels as
// kvcm_b200_replay; the scratch table is g_replay_noalloc_scratch instead of caller memory.
//
// In host code the name of a __device__ array is only a stand-in, not an address a kernel can
// use, so the device address is asked for once per device - with that device current - through
// cudaGetSymbolAddress and kept.  The first call on a device performs that query.
int32_t kvcm_b200_replay_noalloc(const int64_t *d_keys, const int64_t *d_key_off, const uint8_t *d_trace_type,
                                 const int64_t *d_mask_off, int32_t n_traces, int64_t n_keys_total,
                                 int32_t *d_ext_hit, int32_t *d_int_hit, int32_t *d_written, int64_t *d_cache_blocks,
                                 uint32_t *d_status, kvcm_stream_t stream) {
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (n_keys_total < 0) return KVCM_EC_BADARGS;
    if (n_keys_total > KVCM_B200_REPLAY_NOALLOC_MAX_KEYS) return KVCM_EC_OUT_OF_LIMIT;

    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static void *scratch_of_device[kMaxDevices] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        return KVCM_ER_NO_DEVICE;
    }
    void *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (scratch_of_device[dev] == nullptr) {
            void *p = nullptr;
            if (cudaGetSymbolAddress(&p, g_replay_noalloc_scratch) != cudaSuccess || p == nullptr) {
                cudaGetLastError();
                return KVCM_ER_INVALID_ADDRESS;
            }
            scratch_of_device[dev] = p;
        }
        scratch = scratch_of_device[dev];
    }
    // The table is rebuilt from its first slot by every call (the init kernel covers every slot
    // the call uses), so what an earlier call left behind is never read.
    return kvcm_b200_replay(d_keys, d_key_off, d_trace_type, d_mask_off, nullptr, n_traces, n_keys_total, scratch,
                            KVCM_B200_REPLAY_NOALLOC_SCRATCH_BYTES, d_ext_hit, d_int_hit, d_written, d_cache_blocks,
                            d_status, stream);
}

// Host-only: the order in which OptimizerLoader::LoadTrace replays the traces of a file.  It sorts them by timestamp
// with std::sort (TraceTimeSorter::SortTracesByTimestamp, kv_cache_manager/optimizer/trace_converter/
// trace_util.cc:6-8,42-45), which is not stable: traces of one timestamp come out in whatever order the standard
// library's introsort leaves them, and since replay order decides hits and evictions that order is part of the
// result.  So the same routine is called here, on trace numbers compared by their timestamps - the sequence of
// comparisons and moves does not depend on what the elements are.
int32_t kvcm_b200_trace_replay_order(const int64_t *h_timestamps, int64_t n_traces, int64_t *h_order_out) {
    if (n_traces < 0) return KVCM_EC_BADARGS;
    if (n_traces == 0) return KVCM_OK;
    if (h_timestamps == nullptr || h_order_out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    std::vector<int64_t> order(static_cast<size_t>(n_traces));
    for (int64_t i = 0; i < n_traces; ++i) order[static_cast<size_t>(i)] = i;
    std::sort(order.begin(), order.end(),
              [h_timestamps](int64_t a, int64_t b) { return h_timestamps[a] < h_timestamps[b]; });
    for (int64_t i = 0; i < n_traces; ++i) h_order_out[i] = order[static_cast<size_t>(i)];
    return KVCM_OK;
}

// Host-only: the order in which a std::unordered_map<std::string, ...> hands back its entries after a sequence of
// assignments (map[key] = ...) and erasures.  The reference's publisher-log reader keeps the writes that were
// started but not finished in such a map and appends what is left in ITERATION order
// (kv_cache_manager/optimizer/trace_converter/publisher_log_converter.cc:207-219, publisher_log_converter.h:50);
// that order is the standard library's (hash function, bucket growth, node list), and - through the unstable sort
// that follows - it decides the replay order of traces with equal timestamps.  So the same container runs here on
// the same operations.  Operation i names key h_keys[h_key_off[i] .. h_key_off[i+1]); h_erase[i] != 0 erases it,
// else it is assigned the value i.  h_order_out receives the values left, in iteration order; *h_n_out how many.
int32_t kvcm_b200_string_map_iteration_order(const char *h_keys, const int64_t *h_key_off, const uint8_t *h_erase,
                                             int64_t n_ops, int64_t *h_order_out, int64_t *h_n_out) {
    if (n_ops < 0) return KVCM_EC_BADARGS;
    if (h_n_out == nullptr || (n_ops > 0 && (h_key_off == nullptr || h_erase == nullptr || h_order_out == nullptr))) {
        return KVCM_ER_INVALID_ADDRESS;
    }
    std::unordered_map<std::string, int64_t> map;
    for (int64_t i = 0; i < n_ops; ++i) {
        const int64_t len = h_key_off[i + 1] - h_key_off[i];
        if (len < 0 || (len > 0 && h_keys == nullptr)) return KVCM_EC_BADARGS;
        const std::string key(len > 0 ? h_keys + h_key_off[i] : "", static_cast<size_t>(len));
        if (h_erase[i] != 0) {
            map.erase(key);
        } else {
            map[key] = i;
        }
    }
    int64_t n = 0;
    for (const auto &entry : map) h_order_out[n++] = entry.second;
    *h_n_out = n;
    return KVCM_OK;
}

}  // extern "C"
