// Device discovery and the small host-only entry points of the C ABI.
#include "kvcm_common.cuh"

namespace kvcm {

const DeviceInfo &GetDeviceInfo() {
    // One process drives one GPU; the properties of the device current at first use are kept.
    static DeviceInfo info = [] {
        DeviceInfo d;
        int dev = 0;
        cudaDeviceProp prop;
        if (cudaGetDevice(&dev) == cudaSuccess && cudaGetDeviceProperties(&prop, dev) == cudaSuccess) {
            d.sm_count = prop.multiProcessorCount;
            d.l2_bytes = prop.l2CacheSize;
            d.ok = true;
        } else {
            cudaGetLastError();
        }
        return d;
    }();
    return info;
}

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
        case KVCM_EC_OUT_OF_LIMIT: return "size beyond the fixed limit of this entry point";
        default: return "unknown code";
    }
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
