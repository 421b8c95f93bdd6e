// Dense ids for the keys of a trace file: every distinct key gets a number in [0, D), once for all the
// configurations of a sweep, so that per-configuration replay state is flat arrays indexed by id.
// Shared by the eviction-aware replays (replay_lru.cu, replay_leaf_lru.cu).
#pragma once
#include "id_table.cuh"
#include "kvcm_common.cuh"

namespace kvcm {
namespace {

__global__ void __launch_bounds__(256)
    LruClaimIdsKernel(IdTable t, const int64_t *__restrict__ keys, int64_t n_keys, uint32_t *status) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_keys; i += stride) {
        ClaimId(t, static_cast<uint64_t>(keys[i]), status);
    }
}

__global__ void __launch_bounds__(256)
    LruLookupIdsKernel(IdTable t, const int64_t *__restrict__ keys, int64_t n_keys, uint32_t *__restrict__ ids) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_keys; i += stride) {
        ids[i] = LookupId(t, static_cast<uint64_t>(keys[i]));
    }
}

// The same two passes over the traces of ONE instance (a warp per trace).  Instances have separate trees, so the
// same key in two instances is two blocks: the table is cleared between instances while the id counter runs on,
// which makes ids unique over (instance, key).
__global__ void IdTableClearKernel(IdTable t) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    const uint64_t first = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (uint64_t i = first; i <= t.mask; i += stride) t.slots[i] = make_ulonglong2(kEmptyKey, ~0ull);
    if (first == 0) t.cells[1] = ~0ull;
}

__global__ void __launch_bounds__(256)
    LruClaimIdsOfInstanceKernel(IdTable t, const int64_t *__restrict__ keys, const int64_t *__restrict__ key_off,
                                const int32_t *__restrict__ trace_inst, int32_t n_traces, int32_t which,
                                uint32_t *status) {
    const int32_t warps = static_cast<int32_t>(gridDim.x * (blockDim.x >> 5));
    const uint32_t lane = LaneId();
    for (int32_t tr = static_cast<int32_t>(blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)); tr < n_traces;
         tr += warps) {
        if (trace_inst[tr] != which) continue;
        const int64_t end = key_off[tr + 1];
        for (int64_t i = key_off[tr] + lane; i < end; i += 32) ClaimId(t, static_cast<uint64_t>(keys[i]), status);
    }
}

__global__ void __launch_bounds__(256)
    LruLookupIdsOfInstanceKernel(IdTable t, const int64_t *__restrict__ keys, const int64_t *__restrict__ key_off,
                                 const int32_t *__restrict__ trace_inst, int32_t n_traces, int32_t which,
                                 uint32_t *__restrict__ ids) {
    const int32_t warps = static_cast<int32_t>(gridDim.x * (blockDim.x >> 5));
    const uint32_t lane = LaneId();
    for (int32_t tr = static_cast<int32_t>(blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)); tr < n_traces;
         tr += warps) {
        if (trace_inst[tr] != which) continue;
        const int64_t end = key_off[tr + 1];
        for (int64_t i = key_off[tr] + lane; i < end; i += 32) ids[i] = LookupId(t, static_cast<uint64_t>(keys[i]));
    }
}

// Key occurrences per instance, then their running sum: the region of a per-configuration array that belongs to each
// instance of a group (an instance appends at most one entry per occurrence).  Counts the traces whose instance is out
// of range.
__global__ void __launch_bounds__(1024)
    LruGroupExtentKernel(const int64_t *__restrict__ key_off, const int32_t *__restrict__ trace_inst, int32_t n_traces,
                         int32_t n_instances, int64_t *queue_base, uint32_t *status) {
    extern __shared__ unsigned long long count[];
    for (int32_t j = threadIdx.x; j < n_instances; j += blockDim.x) count[j] = 0ull;
    __syncthreads();
    for (int32_t t = threadIdx.x; t < n_traces; t += blockDim.x) {
        const int32_t j = trace_inst[t];
        if (j < 0 || j >= n_instances) {
            if (status != nullptr) atomicAdd(&status[0], 1u);
            continue;
        }
        atomicAdd(&count[j], static_cast<unsigned long long>(key_off[t + 1] - key_off[t]));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int64_t at = 0;
        for (int32_t j = 0; j < n_instances; ++j) {
            queue_base[j] = at;
            at += static_cast<int64_t>(count[j]);
        }
        queue_base[n_instances] = at;
    }
}

}  // namespace
}  // namespace kvcm
