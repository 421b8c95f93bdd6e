// Batched segment copy and the debug CRC of transferred buffers (sm_100a).
//
// copy_segments stands in for the per-Iov cudaMemcpyAsync loops of LocalFileSdk::DoGet / DoPut
// (kv_cache_manager/client/src/internal/sdk/local_file_sdk.cc:223-245,326-353) and
// Hf3fsUsrbioClient::CopyIovs (kv_cache_manager/client/src/internal/sdk/hf3fs_usrbio_client.cc:478-505):
// one launch moves every segment of a request instead of one runtime call per Iov.
// iov_crc stands in for GetIovsCrcDevice (kv_cache_manager/client/src/internal/sdk/sdk_buffer_check_util.cu:21-44).
#include <algorithm>
#include <mutex>
#include <vector>

#include "kvcm_common.cuh"

namespace kvcm {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 8;
constexpr uint64_t kChunk = static_cast<uint64_t>(kThreads) * 16 * kUnroll;  // 32 KiB

// ------------------------------------------------------------------------------------------
// Bulk-copy (TMA) form, used when segments are large: persistent one-warp CTAs, a ring of shared-
// memory stages, one cp.async.bulk load and one cp.async.bulk store per chunk, no thread touching
// the payload (the same machinery as the gather / scatter ring).  CTA b walks segments
// b / parts, b / parts + lanes, ... and of each segment the chunks b % parts, b % parts + parts, ...
// A chunk whose ends are not 16-byte aligned is moved by the warp with plain accesses, as is the
// tail of fewer than 16 bytes.  Every wait is bounded; a CTA that gives up counts itself in
// g_copy_wait_timeouts and returns.
// ------------------------------------------------------------------------------------------
constexpr int kBulkStages = 2;
constexpr uint32_t kBulkChunk = 32 * 1024;  // 48 KiB for segments of 96 KiB and more, see the launcher
constexpr uint64_t kBulkMinSegment = 8 * 1024;  // below this mean size the vector kernel is used

__device__ uint32_t g_copy_wait_timeouts = 0;

struct ChunkItem {
    const uint8_t *src;
    uint8_t *dst;
    uint32_t len;
    uint32_t bulk_len;  // leading bytes moved by bulk copies (0: the warp moves the whole chunk)
};

__global__ void __launch_bounds__(32)
    CopySegmentsBulkKernel(const kvcm_b200_seg_t *__restrict__ segs, int32_t n, uint32_t parts, uint32_t seg_lanes,
                           uint32_t chunk_bytes) {
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ __align__(8) uint64_t bars[kBulkStages];
    const uint32_t lane = threadIdx.x;
    if (lane == 0) {
        for (int s = 0; s < kBulkStages; ++s) MbarInit(SmemAddr(&bars[s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async;\n" ::: "memory");
    }
    __syncwarp();
    const uint32_t my_part = blockIdx.x % parts;
    int64_t seg = blockIdx.x / parts;
    if (seg >= seg_lanes) return;
    uint64_t chunk = my_part;
    // Next chunk of this CTA's walk (warp-uniform); false when the walk is over.
    auto next = [&](ChunkItem *it) -> bool {
        while (seg < n) {
            const uint8_t *src = static_cast<const uint8_t *>(segs[seg].src);
            uint8_t *dst = static_cast<uint8_t *>(segs[seg].dst);
            const uint64_t bytes = (src == nullptr || dst == nullptr) ? 0 : segs[seg].bytes;
            const uint64_t off = chunk * chunk_bytes;
            if (off < bytes) {
                it->src = src + off;
                it->dst = dst + off;
                it->len = bytes - off < chunk_bytes ? static_cast<uint32_t>(bytes - off) : chunk_bytes;
                const bool aligned = ((reinterpret_cast<uintptr_t>(it->src) | reinterpret_cast<uintptr_t>(it->dst)) & 15u) == 0;
                it->bulk_len = aligned ? (it->len & ~15u) : 0u;
                chunk += parts;
                return true;
            }
            seg += seg_lanes;
            chunk = my_part;
        }
        return false;
    };
    const uint32_t ring_base = SmemAddr(ring);
    ChunkItem items[kBulkStages];
    bool live[kBulkStages];
    auto load = [&](int s) {
        live[s] = next(&items[s]);
        if (!live[s]) return;
        const ChunkItem &it = items[s];
        if (lane == 0) {
            MbarArriveExpectTx(SmemAddr(&bars[s]), it.bulk_len);
            if (it.bulk_len > 0) BulkLoad(ring_base + s * chunk_bytes, it.src, it.bulk_len, SmemAddr(&bars[s]));
        }
        for (uint32_t i = it.bulk_len + lane; i < it.len; i += 32) it.dst[i] = it.src[i];  // what bulk copies cannot take
    };
#pragma unroll
    for (int s = 0; s < kBulkStages - 1; ++s) load(s);
    live[kBulkStages - 1] = false;
    bool failed = false;
    uint32_t k = 0;
    while (true) {
        const int s = k % kBulkStages;
        if (!live[s]) break;
        if (lane == 0) failed = !BoundedWait(SmemAddr(&bars[s]), (k / kBulkStages) & 1u);
        failed = __shfl_sync(0xffffffffu, failed ? 1 : 0, 0) != 0;
        __syncwarp();
        if (failed) break;
        if (lane == 0 && items[s].bulk_len > 0) BulkStore(items[s].dst, ring_base + s * chunk_bytes, items[s].bulk_len);
        BulkCommit();
        // The stage refilled next was drained by the store of chunk k-1: let every group but the newest finish
        // reading shared memory first.
        BulkWaitRead<1>();
        __syncwarp();
        load((k + kBulkStages - 1) % kBulkStages);
        ++k;
    }
    if (failed && lane == 0) {
        // Leave no copy in flight behind: the loads of the chunk that was waited for and of the chunks fetched
        // ahead may still be writing this CTA's shared memory; one more bounded wait for each of them.
        for (uint32_t j = k; j < k + kBulkStages - 1; ++j) {
            if (live[j % kBulkStages]) BoundedWait(SmemAddr(&bars[j % kBulkStages]), (j / kBulkStages) & 1u);
        }
    }
    BulkWaitAll();
    if (failed && lane == 0) atomicAdd(&g_copy_wait_timeouts, 1u);
}

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
    return kvcm_b200_copy_segments_sized(d_segs, n_segs, 0, stream);
}

int32_t kvcm_b200_copy_wait_timeouts(uint32_t *h_count_out) {
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (h_count_out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    const cudaError_t e = cudaMemcpyFromSymbol(h_count_out, kvcm::g_copy_wait_timeouts, sizeof(uint32_t));
    return e == cudaSuccess ? KVCM_OK : KVCM_ER_CUDAMEMCPY_ERROR;
}

int32_t kvcm_b200_copy_segments_sized(const kvcm_b200_seg_t *d_segs, int32_t n_segs, uint64_t total_bytes,
                                      kvcm_stream_t stream) {
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (n_segs < 0) return KVCM_ER_INVALID_PARAMS;
    if (n_segs == 0) return KVCM_OK;
    if (d_segs == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (total_bytes / static_cast<uint64_t>(n_segs) >= kvcm::kBulkMinSegment) {
        // Large segments: the bulk-copy ring, two stages of shared memory per one-warp CTA.
        // Geometry from a sweep on B200 (131,072 segments of 128 KiB): 48 KiB chunks x 2 CTAs per SM reach 0.99 of
        // the measured copy peak, 32 KiB x 3 reach 0.97, 64 KiB x 1 0.93; 192 KiB are in flight per SM either way.
        // Short segments would leave most of a 48 KiB stage empty.
        const bool wide = total_bytes / static_cast<uint64_t>(n_segs) >= 96 * 1024;
        const uint32_t chunk_bytes = wide ? 48 * 1024 : kvcm::kBulkChunk;
        const int ctas_per_sm = wide ? 2 : 3;
        const int smem = kvcm::kBulkStages * static_cast<int>(chunk_bytes);
        kvcm::EnsureDynamicSmem(kvcm::CopySegmentsBulkKernel, kvcm::kBulkStages * 48 * 1024);
        const uint32_t grid = static_cast<uint32_t>(kvcm::GetDeviceInfo().sm_count) * ctas_per_sm;
        uint32_t parts = 1, seg_lanes = grid;
        if (static_cast<uint32_t>(n_segs) < grid) {
            parts = grid / static_cast<uint32_t>(n_segs);
            parts = parts > 64 ? 64 : parts;
            seg_lanes = static_cast<uint32_t>(n_segs);
        }
        kvcm::CopySegmentsBulkKernel<<<seg_lanes * parts, 32, smem, kvcm::AsStream(stream)>>>(d_segs, n_segs, parts,
                                                                                            seg_lanes, chunk_bytes);
        return kvcm::LaunchStatus();
    }
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
            if (iov.type == 0) {
                // A CPU iov goes into the table only if a kernel can address it: pinned or registered host
                // memory (or memory the driver knows as device / managed).  Ordinary pageable memory - what the
                // reference copies with std::memcpy - is refused here, before any launch; the caller moves such
                // iovs on the host (IovCopier does) and marks them `ignore`.
                cudaPointerAttributes attr;
                if (cudaPointerGetAttributes(&attr, iov.base) != cudaSuccess) {
                    cudaGetLastError();
                    return KVCM_ER_UNSUPPORTED_MEMORY_TYPE;
                }
                if (attr.type == cudaMemoryTypeUnregistered) return KVCM_ER_UNSUPPORTED_MEMORY_TYPE;
            }
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
