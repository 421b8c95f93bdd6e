// Shared host/device helpers of libkvcm_b200.so (sm_100a only).
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <mutex>
#include <utility>
#include <vector>

#include "kvcm_b200.h"

namespace kvcm {

// Device properties the launchers size their grids from; queried once per device.
struct DeviceInfo {
    int sm_count = 0;
    int64_t l2_bytes = 0;
    bool ok = false;
};

// Properties of the device that is current for the calling thread (kept per device after the first query).
const DeviceInfo &GetDeviceInfo();

inline cudaStream_t AsStream(kvcm_stream_t s) { return static_cast<cudaStream_t>(s); }

// Maps the state of the CUDA runtime after a launch to a return code of the C ABI.
inline int32_t LaunchStatus() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? KVCM_OK : KVCM_ER_CUDAMEMCPY_ERROR;
}

// True when a device is present; every compute entry point checks it first so that a box
// without a GPU gets KVCM_ER_NO_DEVICE instead of a silent no-op.
bool HaveDevice();

// The opt-in to more than 48 KiB of dynamic shared memory is per device and per kernel; this makes it
// once for each pair, whichever host thread gets there first.
template <typename Kernel>
inline void EnsureDynamicSmem(Kernel kernel, int bytes) {
    static std::mutex mu;
    static std::vector<std::pair<int, const void *>> done;
    int device = 0;
    cudaGetDevice(&device);
    const std::pair<int, const void *> key(device, reinterpret_cast<const void *>(kernel));
    std::lock_guard<std::mutex> lock(mu);
    if (std::find(done.begin(), done.end(), key) == done.end()) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        done.push_back(key);
    }
}

__device__ __forceinline__ uint32_t LaneId() { return threadIdx.x & 31u; }

// The key value an empty slot of the library's open-addressing tables holds (INT64_MIN; a real key of that value is
// kept beside the table), and the 64-bit finaliser that spreads keys over their slots and over hash-range shards.
constexpr uint64_t kEmptyKey = 0x8000000000000000ull;

__host__ __device__ __forceinline__ uint64_t Mix(uint64_t k) {
    k ^= k >> 33;
    k *= 0xff51afd7ed558ccdull;
    k ^= k >> 33;
    k *= 0xc4ceb9fe1a85ec53ull;
    k ^= k >> 33;
    return k;
}

// One step of the reference's chained block hash (kv_cache_manager/manager/hash_util.h:8-12):
//   hash ^= value + 0x9e3779b97f4a7c15 + (hash << 12) + (hash >> 32)
// on int64 with wrap-around; `>>` is the arithmetic shift of a signed value.  Written on
// unsigned words so that the device code has no signed overflow.
__host__ __device__ __forceinline__ uint64_t HashStep(uint64_t h, uint64_t v) {
    const uint64_t sra32 = static_cast<uint64_t>(static_cast<int64_t>(h) >> 32);
    return h ^ (v + 0x9e3779b97f4a7c15ull + (h << 12) + sra32);
}

// The same step with `value + 0x9e3779b97f4a7c15` formed by the caller ahead of time.
__host__ __device__ __forceinline__ uint64_t HashStepPre(uint64_t h, uint64_t value_plus_golden) {
    const uint64_t sra32 = static_cast<uint64_t>(static_cast<int64_t>(h) >> 32);
    return h ^ (value_plus_golden + (h << 12) + sra32);
}

// ---- mbarrier and bulk-copy (TMA) primitives shared by the kernels that stage through shared memory ----
// Failed polls of a barrier after which a kernel gives up, raises its error word and returns.
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t SmemAddr(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void MbarInit(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void MbarArriveExpectTx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool MbarTryWait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// The one wait loop of every kernel that waits on an mbarrier: polls until the phase with `parity` completes,
// at most `limit` times.  false = gave up; the caller then raises its error word, waits (again bounded) for the
// copies it may still have in flight, and returns.  kRelaxed: the waiter is far ahead of what it waits for, so
// it sleeps between polls instead of taking issue slots from the warps that do the work.
template <bool kRelaxed = false>
__device__ __forceinline__ bool BoundedWait(uint32_t bar, uint32_t parity, uint32_t limit = kSpinLimit) {
    uint32_t polls = 0;
    while (!MbarTryWait(bar, parity)) {
        if (++polls >= limit) return false;
        if (kRelaxed) __nanosleep(256);
    }
    return true;
}
__device__ __forceinline__ void MbarInval(uint32_t bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void BulkLoad(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                     dst_smem),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void BulkStore(void *dst, uint32_t src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n" ::"l"(dst), "r"(src_smem), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void BulkCommit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void BulkWaitRead() {
    asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(kPending) : "memory");
}
__device__ __forceinline__ void BulkWaitAll() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }
__device__ __forceinline__ void MbarArrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}

}  // namespace kvcm
