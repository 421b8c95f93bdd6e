// Batched segment copy and the debug CRC of transferred buffers (sm_100a).
//
// copy_segments stands in for the per-Iov cudaMemcpyAsync loops of LocalFileSdk::DoGet / DoPut
// (kv_cache_manager/client/src/internal/sdk/local_file_sdk.cc:223-245,326-353) and
// Hf3fsUsrbioClient::CopyIovs (kv_cache_manager/client/src/internal/sdk/hf3fs_usrbio_client.cc:478-505):
// one launch moves every segment of a request instead of one runtime call per Iov.
// iov_crc stands in for GetIovsCrcDevice (kv_cache_manager/client/src/internal/sdk/sdk_buffer_check_util.cu:21-44).
#include "kvcm_common.cuh"

namespace kvcm {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 8;
constexpr uint64_t kChunk = static_cast<uint64_t>(kThreads) * 16 * kUnroll;  // 32 KiB

// grid.x strides over segments, grid.y CTAs share the chunks of one segment.
__global__ void __launch_bounds__(kThreads) CopySegmentsKernel(const kvcm_b200_seg_t *__restrict__ segs, int32_t n) {
    const uint32_t tid = threadIdx.x;
    for (int32_t s = blockIdx.x; s < n; s += gridDim.x) {
        uint8_t *dst = static_cast<uint8_t *>(segs[s].dst);
        const uint8_t *src = static_cast<const uint8_t *>(segs[s].src);
        const uint64_t bytes = segs[s].bytes;
        if (dst == nullptr || src == nullptr || bytes == 0) continue;
        const bool aligned = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0;
        const uint64_t vec_bytes = aligned ? (bytes & ~15ull) : 0;
        for (uint64_t base = blockIdx.y * kChunk; base < vec_bytes; base += gridDim.y * kChunk) {
            uint4 v[kUnroll];
            uint64_t off[kUnroll];
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                off[j] = base + (static_cast<uint64_t>(j) * kThreads + tid) * 16;
                if (off[j] < vec_bytes) v[j] = __ldcs(reinterpret_cast<const uint4 *>(src + off[j]));
            }
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                if (off[j] < vec_bytes) __stcs(reinterpret_cast<uint4 *>(dst + off[j]), v[j]);
            }
        }
        // Unaligned segments and the sub-16-byte tail go byte by byte.
        for (uint64_t o = vec_bytes + blockIdx.y * kThreads + tid; o < bytes;
             o += static_cast<uint64_t>(gridDim.y) * kThreads) {
            dst[o] = src[o];
        }
    }
}

__device__ __forceinline__ uint32_t CrcByte(uint32_t crc, uint8_t data) {
    crc ^= data;
#pragma unroll
    for (int i = 0; i < 8; ++i) crc = (crc >> 1) ^ (0xEDB88320u & (0u - (crc & 1u)));
    return crc;
}

__global__ void IovCrcKernel(const kvcm_b200_seg_t *__restrict__ segs, int32_t n, uint64_t cal_bytes,
                             uint32_t *__restrict__ out) {
    const int32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint8_t *p = static_cast<const uint8_t *>(segs[i].src);
    const uint64_t size = segs[i].bytes;
    const uint64_t cal = cal_bytes < size ? cal_bytes : size;
    uint32_t crc = 0xFFFFFFFFu;
    for (uint64_t k = 0; k < cal; ++k) crc = CrcByte(crc, p[k]);
    for (uint64_t k = size - cal; k < size; ++k) crc = CrcByte(crc, p[k]);
    out[i] = ~crc;
}

}  // namespace
}  // namespace kvcm

extern "C" {

int32_t kvcm_b200_copy_segments(const kvcm_b200_seg_t *d_segs, int32_t n_segs, kvcm_stream_t stream) {
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (n_segs < 0) return KVCM_ER_INVALID_PARAMS;
    if (n_segs == 0) return KVCM_OK;
    if (d_segs == nullptr) return KVCM_ER_INVALID_ADDRESS;
    const int resident = kvcm::GetDeviceInfo().sm_count * 8;
    int parts = resident / n_segs;
    parts = parts < 1 ? 1 : (parts > 64 ? 64 : parts);
    dim3 grid(static_cast<unsigned>(n_segs < resident ? n_segs : resident), static_cast<unsigned>(parts));
    kvcm::CopySegmentsKernel<<<grid, kvcm::kThreads, 0, kvcm::AsStream(stream)>>>(d_segs, n_segs);
    return kvcm::LaunchStatus();
}

int32_t kvcm_b200_iovs_to_segments(const kvcm_b200_iov_t *h_iovs, int32_t n_iovs, void *block_string,
                                   int32_t direction, kvcm_b200_seg_t *h_segs_out, int32_t *n_segs_out,
                                   uint64_t *span_bytes_out) {
    if (n_iovs < 0 || (direction != 0 && direction != 1)) return KVCM_ER_INVALID_PARAMS;
    if ((n_iovs > 0 && (h_iovs == nullptr || h_segs_out == nullptr)) || n_segs_out == nullptr) {
        return KVCM_ER_INVALID_ADDRESS;
    }
    uint8_t *str = static_cast<uint8_t *>(block_string);
    uint64_t offset = 0;
    int32_t n = 0;
    for (int32_t i = 0; i < n_iovs; ++i) {
        const kvcm_b200_iov_t &iov = h_iovs[i];
        if (iov.type > 1) return KVCM_ER_UNSUPPORTED_MEMORY_TYPE;
        if (!iov.ignore && iov.base != nullptr && iov.size > 0) {
            if (str == nullptr) return KVCM_ER_INVALID_ADDRESS;
            kvcm_b200_seg_t &seg = h_segs_out[n++];
            seg.bytes = iov.size;
            if (direction == 0) {
                seg.dst = str + offset;
                seg.src = iov.base;
            } else {
                seg.dst = iov.base;
                seg.src = str + offset;
            }
        }
        offset += iov.size;
    }
    *n_segs_out = n;
    if (span_bytes_out != nullptr) *span_bytes_out = offset;
    return KVCM_OK;
}

int32_t kvcm_b200_iov_crc(const kvcm_b200_seg_t *d_segs, int32_t n_segs, uint64_t cal_bytes, uint32_t *d_crc_out,
                          kvcm_stream_t stream) {
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (n_segs < 0) return KVCM_ER_INVALID_PARAMS;
    if (n_segs == 0) return KVCM_OK;
    if (d_segs == nullptr || d_crc_out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    kvcm::IovCrcKernel<<<(n_segs + 255) / 256, 256, 0, kvcm::AsStream(stream)>>>(d_segs, n_segs, cal_bytes, d_crc_out);
    return kvcm::LaunchStatus();
}

}  // extern "C"
