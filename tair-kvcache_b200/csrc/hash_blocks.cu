// Chained token-block hashing for a batch of requests (sm_100a).
//
// Stands in for GenKeyVector (kv_cache_manager/manager/cache_manager.cc:76-87) over
// hashInt64Array (kv_cache_manager/manager/hash_util.h:8-24) and for ApplyPrefixHash
// (kv_cache_manager/optimizer/trace_converter/trace_util.cc:47-56).
//
// The hash of a request is one serial dependency chain over all of its tokens (the state feeds
// the next step and the step is not associative), so the parallelism is across requests only:
// one lane walks one request.  What bounds the kernel is the latency of the chain, not HBM:
// a request of L tokens takes L dependent steps however many SMs are idle.
//
// Token tiles are staged through shared memory.  Each lane owns a ring of kStages x 64 bytes;
// it fills the ring with 16-byte cp.async copies from its own request (src-size clamped to
// the token array's extent, so nothing outside the caller's buffer is read) and consumes a
// stage with four conflict-free 128-bit shared loads.  The ring keeps kStages-1 stages (about
// a hundred tokens) in flight per lane, which hides DRAM latency behind the chain itself.
#include "kvcm_common.cuh"

namespace kvcm {
namespace {

constexpr int kStages = 8;
constexpr int kStageBytes = 64;                         // per lane
constexpr int kPieces = kStageBytes / 16;               // cp.async pieces per lane per stage
constexpr int kWarpRingBytes = kStages * kPieces * 32 * 16;  // 16 KiB
constexpr int kMaxWarpsPerCta = 4;

__device__ __forceinline__ void CpAsync16(uint32_t smem_addr, uint64_t gmem_addr, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr), "l"(gmem_addr), "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void CpAsyncCommit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void CpAsyncWait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(kPending) : "memory");
}

template <typename T>
__device__ __forceinline__ uint64_t Widen(T v);
template <>
__device__ __forceinline__ uint64_t Widen<uint32_t>(uint32_t v) {
    return static_cast<uint64_t>(v);
}
template <>
__device__ __forceinline__ uint64_t Widen<int64_t>(int64_t v) {
    return static_cast<uint64_t>(v);
}

template <typename T>
__global__ void __launch_bounds__(kMaxWarpsPerCta * 32)
    HashBlocksKernel(const T *__restrict__ tokens, int64_t n_tokens_total, const int64_t *__restrict__ tok_off,
                     int32_t n_req, int32_t block_size, int64_t *__restrict__ keys,
                     const int64_t *__restrict__ key_off) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int kPerPiece = 16 / sizeof(T);
    const uint32_t lane = LaneId();
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t warps_per_cta = blockDim.x >> 5;
    const int64_t req = (static_cast<int64_t>(blockIdx.x) * warps_per_cta + warp) * 32 + lane;
    const bool active = req < n_req;

    int64_t first_tok = 0, n_tok = 0, key_base = 0;
    if (active) {
        first_tok = tok_off[req];
        n_tok = tok_off[req + 1] - first_tok;
        key_base = key_off[req];
    }
    // Only whole blocks are hashed; the trailing partial block is never read.
    const int64_t used = n_tok > 0 ? (n_tok / block_size) * block_size : 0;
    const uint64_t arr_beg = reinterpret_cast<uint64_t>(tokens);
    const uint64_t arr_end = arr_beg + static_cast<uint64_t>(n_tokens_total) * sizeof(T);
    const uint64_t beg = arr_beg + static_cast<uint64_t>(first_tok) * sizeof(T);
    const uint64_t end = beg + static_cast<uint64_t>(used) * sizeof(T);
    const uint64_t a0 = beg & ~15ull;  // arr_beg is 16-byte aligned, so a0 >= arr_beg
    const int64_t n_stages = used > 0 ? static_cast<int64_t>((end - a0 + kStageBytes - 1) / kStageBytes) : 0;
    int64_t max_stages = n_stages;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        const int64_t other = __shfl_xor_sync(0xffffffffu, max_stages, d);
        max_stages = other > max_stages ? other : max_stages;
    }

    const uint32_t ring = static_cast<uint32_t>(__cvta_generic_to_shared(smem)) + warp * kWarpRingBytes + lane * 16;
    auto issue = [&](int64_t s) {
        if (s < n_stages) {
            const uint32_t slot = static_cast<uint32_t>(s % kStages);
#pragma unroll
            for (int c = 0; c < kPieces; ++c) {
                const uint64_t a = a0 + static_cast<uint64_t>(s) * kStageBytes + c * 16;
                if (a < end) {
                    const uint64_t left = arr_end - a;
                    CpAsync16(ring + (slot * kPieces + c) * 512, a, left >= 16 ? 16u : static_cast<uint32_t>(left));
                }
            }
        }
        CpAsyncCommit();
    };

#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) issue(s);

    uint64_t h = 0;
    int32_t left_in_block = block_size;
    int64_t *out = keys + key_base;
    for (int64_t k = 0; k < max_stages; ++k) {
        issue(k + kStages - 1);
        CpAsyncWait<kStages - 1>();  // stage k has landed; a lane only reads what it copied itself
        if (k < n_stages) {
            const uint32_t slot = static_cast<uint32_t>(k % kStages);
            const uint64_t stage_lo = a0 + static_cast<uint64_t>(k) * kStageBytes;
            const bool full = stage_lo >= beg && stage_lo + kStageBytes <= end;
#pragma unroll
            for (int c = 0; c < kPieces; ++c) {
                uint4 q;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
                             : "r"(ring + (slot * kPieces + c) * 512));
                T tok[kPerPiece];
                if constexpr (sizeof(T) == 4) {
                    tok[0] = static_cast<T>(q.x);
                    tok[1] = static_cast<T>(q.y);
                    tok[2] = static_cast<T>(q.z);
                    tok[3] = static_cast<T>(q.w);
                } else {
                    tok[0] = static_cast<T>(static_cast<uint64_t>(q.x) | (static_cast<uint64_t>(q.y) << 32));
                    tok[1] = static_cast<T>(static_cast<uint64_t>(q.z) | (static_cast<uint64_t>(q.w) << 32));
                }
#pragma unroll
                for (int i = 0; i < kPerPiece; ++i) {
                    const uint64_t pos = stage_lo + c * 16 + i * sizeof(T);
                    if (full || (pos >= beg && pos < end)) {
                        h = HashStep(h, Widen<T>(tok[i]));
                        if (--left_in_block == 0) {
                            *out++ = static_cast<int64_t>(h);
                            left_in_block = block_size;
                        }
                    }
                }
            }
        }
    }
    CpAsyncWait<0>();
}

template <typename T>
int32_t LaunchHash(const T *d_tokens, int64_t n_tokens_total, const int64_t *d_tok_off, int32_t n_req,
                   int32_t block_size, int64_t *d_keys, const int64_t *d_key_off, kvcm_stream_t stream) {
    if (!HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (n_req < 0 || block_size <= 0 || n_tokens_total < 0) return KVCM_ER_INVALID_PARAMS;
    if (n_req == 0) return KVCM_OK;
    if (d_tok_off == nullptr || d_key_off == nullptr || (d_tokens == nullptr && n_tokens_total > 0)) {
        return KVCM_ER_INVALID_ADDRESS;
    }
    if (n_tokens_total == 0) return KVCM_OK;  // every request is empty: no key to write
    if (d_keys == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (reinterpret_cast<uintptr_t>(d_tokens) & 15u) return KVCM_ER_INVALID_ADDRESS;  // 16-byte staging copies

    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(HashBlocksKernel<uint32_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kMaxWarpsPerCta * kWarpRingBytes);
        cudaFuncSetAttribute(HashBlocksKernel<int64_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kMaxWarpsPerCta * kWarpRingBytes);
        attr_set = true;
    }
    // Few requests: one warp per CTA so the chains spread over as many SMs as possible.
    const int64_t n_warps = (static_cast<int64_t>(n_req) + 31) / 32;
    const int warps_per_cta = n_warps <= 2ll * GetDeviceInfo().sm_count ? 1 : kMaxWarpsPerCta;
    const unsigned grid = static_cast<unsigned>((n_warps + warps_per_cta - 1) / warps_per_cta);
    HashBlocksKernel<T><<<grid, warps_per_cta * 32, warps_per_cta * kWarpRingBytes, AsStream(stream)>>>(
        d_tokens, n_tokens_total, d_tok_off, n_req, block_size, d_keys, d_key_off);
    return LaunchStatus();
}

}  // namespace
}  // namespace kvcm

extern "C" {

int32_t kvcm_b200_hash_blocks_u32(const uint32_t *d_tokens, int64_t n_tokens_total, const int64_t *d_tok_off,
                                  int32_t n_req, int32_t block_size, int64_t *d_keys, const int64_t *d_key_off,
                                  kvcm_stream_t stream) {
    return kvcm::LaunchHash<uint32_t>(d_tokens, n_tokens_total, d_tok_off, n_req, block_size, d_keys, d_key_off,
                                      stream);
}

int32_t kvcm_b200_hash_blocks_i64(const int64_t *d_tokens, int64_t n_tokens_total, const int64_t *d_tok_off,
                                  int32_t n_req, int32_t block_size, int64_t *d_keys, const int64_t *d_key_off,
                                  kvcm_stream_t stream) {
    return kvcm::LaunchHash<int64_t>(d_tokens, n_tokens_total, d_tok_off, n_req, block_size, d_keys, d_key_off,
                                     stream);
}

int32_t kvcm_b200_key_offsets(const int64_t *h_tok_off, int32_t n_req, int32_t block_size, int64_t *h_key_off) {
    if (h_tok_off == nullptr || h_key_off == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (n_req < 0 || block_size <= 0) return KVCM_ER_INVALID_PARAMS;
    int64_t acc = 0;
    h_key_off[0] = 0;
    for (int32_t r = 0; r < n_req; ++r) {
        const int64_t len = h_tok_off[r + 1] - h_tok_off[r];
        if (len < 0) return KVCM_ER_INVALID_PARAMS;
        acc += len / block_size;
        h_key_off[r + 1] = acc;
    }
    return KVCM_OK;
}

}  // extern "C"
