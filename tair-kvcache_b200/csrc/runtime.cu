// Device discovery and the small host-only entry points of the C ABI.
#include "kvcm_common.cuh"

namespace kvcm {

const DeviceInfo &GetDeviceInfo() {
    // Kept per device: a process may drive several GPUs (shards attached inside one process), and grid sizes
    // must come from the device the launch goes to, which is the calling thread's current device.
    static std::mutex mu;
    static std::vector<DeviceInfo> known;  // by device ordinal
    static const DeviceInfo none;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) {
        cudaGetLastError();
        return none;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (known.capacity() < 64) known.reserve(64);  // references handed out stay valid
    if (known.size() <= static_cast<size_t>(dev)) known.resize(static_cast<size_t>(dev) + 1);
    DeviceInfo &d = known[static_cast<size_t>(dev)];
    if (!d.ok) {
        cudaDeviceProp prop;
        if (cudaGetDeviceProperties(&prop, dev) == cudaSuccess) {
            d.sm_count = prop.multiProcessorCount;
            d.l2_bytes = prop.l2CacheSize;
            d.ok = true;
        } else {
            cudaGetLastError();
        }
    }
    return d;
}

namespace {

// One warp.  Lane 0 arms an mbarrier for bytes that nothing will ever send - no copy is issued - and runs the
// shared bounded wait with the caller's poll limit; the wait runs out by construction, the status words are
// written, the barrier is invalidated and the kernel returns.  This is the give-up path every kernel with an
// mbarrier takes when a wait does not come through, executed once with nothing in flight.
__global__ void __launch_bounds__(32) BoundedWaitSelfTestKernel(uint32_t limit, uint32_t *status) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        MbarInit(SmemAddr(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        MbarArriveExpectTx(SmemAddr(&bar), 64);
        const bool came_through = BoundedWait(SmemAddr(&bar), 0, limit);
        status[0] = came_through ? 0u : 1u;
        status[1] = limit;
        MbarInval(SmemAddr(&bar));
    }
}

}  // namespace

bool HaveDevice() { return GetDeviceInfo().ok; }

}  // namespace kvcm

extern "C" {

int32_t kvcm_b200_abi_version(void) { return 1; }

int32_t kvcm_b200_set_device(int32_t device) {
    if (cudaSetDevice(device) != cudaSuccess) {
        cudaGetLastError();
        return KVCM_ER_NO_DEVICE;
    }
    return KVCM_OK;
}

const char *kvcm_b200_error_string(int32_t code) {
    switch (code) {
        case KVCM_OK: return "ok";
        case KVCM_ER_INVALID_PARAMS: return "invalid parameters";
        case KVCM_ER_INVALID_ADDRESS: return "invalid or misaligned address";
        case KVCM_ER_UNSUPPORTED_MEMORY_TYPE: return "unsupported memory type";
        case KVCM_ER_CUDAMEMCPY_ERROR: return "CUDA launch or copy failed";
        case KVCM_ER_CUDA_STREAM_SYNCHRONIZE_ERROR: return "CUDA stream synchronize failed";
        case KVCM_ER_NO_DEVICE: return "no CUDA device: this library has no CPU path";
        case KVCM_EC_ERROR: return "error";
        case KVCM_EC_NOENT: return "entry does not exist";
        case KVCM_EC_BADARGS: return "bad arguments";
        case KVCM_EC_NOSPC: return "out of space";
        case KVCM_EC_MISMATCH: return "status differs from the expected one";
        case KVCM_EC_OUT_OF_LIMIT: return "size beyond the fixed limit of this entry point";
        default: return "unknown code";
    }
}

int32_t kvcm_b200_selftest_bounded_wait(uint32_t poll_limit, uint32_t *d_status, kvcm_stream_t stream) {
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (d_status == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (poll_limit == 0 || poll_limit > 65536) return KVCM_ER_INVALID_PARAMS;  // a self test is short
    kvcm::BoundedWaitSelfTestKernel<<<1, 32, 0, kvcm::AsStream(stream)>>>(poll_limit, d_status);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_device_info(int32_t *sm_count, int64_t *l2_bytes, int64_t *free_bytes, int64_t *total_bytes) {
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    const kvcm::DeviceInfo &d = kvcm::GetDeviceInfo();
    if (sm_count != nullptr) *sm_count = d.sm_count;
    if (l2_bytes != nullptr) *l2_bytes = d.l2_bytes;
    if (free_bytes != nullptr || total_bytes != nullptr) {
        size_t f = 0, t = 0;
        if (cudaMemGetInfo(&f, &t) != cudaSuccess) return KVCM_ER_CUDAMEMCPY_ERROR;
        if (free_bytes != nullptr) *free_bytes = static_cast<int64_t>(f);
        if (total_bytes != nullptr) *total_bytes = static_cast<int64_t>(t);
    }
    return KVCM_OK;
}

}  // extern "C"
