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
#include <algorithm>
#include <vector>

#include "kvcm_common.cuh"

namespace kvcm {
namespace {

constexpr int kStages = 8;  // power of two
constexpr int kStageBytes = 64;                         // per lane
constexpr int kPieces = kStageBytes / 16;               // cp.async pieces per lane per stage
constexpr int kWarpRingBytes = kStages * kPieces * 32 * 16;  // 16 KiB
constexpr int kMaxWarpsPerCta = 4;
constexpr int kMaxHashSmemPerSm = 224 * 1024;
// Batches of up to 16 x SMs x this many requests run with half-filled warps.
constexpr int kHalfWarpSmMultiple = 2;

__device__ __forceinline__ void CpAsync16(uint32_t smem_addr, uint64_t gmem_addr, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr), "l"(gmem_addr), "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void CpAsyncCommit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void CpAsyncWait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(kPending) : "memory");
}

// What bounds this kernel is the latency of ONE lane's dependent chain (the longest request), and
// for a lone warp on an SM the integer pipe takes two cycles per warp instruction.  So the loop is
// shaped to spend as few instructions per token as possible next to the chain itself:
//  * a stage (64 bytes per lane) is unpacked into registers, as `token + C`, one stage ahead of
//    the chain (ping-pong register buffers): shared-memory latency never sits on the chain;
//  * a stage that lies wholly inside the request runs as one unrolled run of steps.  When
//    block_size is a multiple of the tokens per stage, a block can only end at the positions
//    {last, 0 .. tokens-per-16-bytes - 2} of a stage (the request's misalignment against the
//    16-byte copy grid is a per-lane constant), so only those few positions carry a predicated
//    key store; other block sizes check every position;
//  * only the first and last stage of a request, and blocks shorter than a stage, take the
//    per-token checked path; staging copies of inner stages are four unconditional cp.async.
// With few requests (lanes_per_warp = 16) only half of each warp is used, so that twice as many
// SMs work on the batch and the longest chains do not share a warp's issue slots more than needed.
template <typename T, bool kAligned>
__device__ __forceinline__ void RunFullStage(uint64_t &h, const uint64_t (&vc)[kStageBytes / sizeof(T)], int32_t &left,
                                             int64_t *&out, int32_t block_size) {
    constexpr int kPerPiece = 16 / sizeof(T);
    constexpr int kPerStage = kStageBytes / sizeof(T);
    uint32_t hl = static_cast<uint32_t>(h), hh = static_cast<uint32_t>(h >> 32);
#pragma unroll
    for (int i = 0; i < kPerStage; ++i) {
        HashStep32(hl, hh, static_cast<uint32_t>(vc[i]), static_cast<uint32_t>(vc[i] >> 32));
        if (!kAligned || i == kPerStage - 1 || i < kPerPiece - 1) {
            if (i + 1 == left) *out = static_cast<int64_t>(static_cast<uint64_t>(hl) | (static_cast<uint64_t>(hh) << 32));
        }
    }
    h = static_cast<uint64_t>(hl) | (static_cast<uint64_t>(hh) << 32);
    if (left <= kPerStage) {
        ++out;
        left += block_size;
    }
    left -= kPerStage;
}

template <typename T, bool kAligned>
__global__ void __launch_bounds__(kMaxWarpsPerCta * 32)
    HashBlocksKernel(const T *__restrict__ tokens, int64_t n_tokens_total, const int64_t *__restrict__ tok_off,
                     int32_t n_req, int32_t block_size, int64_t *__restrict__ keys,
                     const int64_t *__restrict__ key_off, const int32_t *__restrict__ order,
                     uint32_t lanes_per_warp) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int kPerPiece = 16 / sizeof(T);
    constexpr int kPerStage = kStageBytes / sizeof(T);
    constexpr uint64_t kGolden = 0x9e3779b97f4a7c15ull;
    const uint32_t lane = LaneId();
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t warps_per_cta = blockDim.x >> 5;
    const int64_t pos = (static_cast<int64_t>(blockIdx.x) * warps_per_cta + warp) * lanes_per_warp + lane;
    const bool active = lane < lanes_per_warp && pos < n_req;
    // `order` (optional) lists the requests longest first: lanes of one warp then walk chains of
    // similar length, and the longest chains start first.
    const int64_t req = active && order != nullptr ? order[pos] : pos;

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
    const uint64_t span = used > 0 ? end - a0 : 0;
    const int64_t n_stages = static_cast<int64_t>((span + kStageBytes - 1) / kStageBytes);
    const int64_t n_pieces = static_cast<int64_t>((span + 15) / 16);
    // The last piece may hang over the end of the token array: copy only what exists.
    const uint64_t last_piece = a0 + static_cast<uint64_t>(n_pieces > 0 ? n_pieces - 1 : 0) * 16;
    const uint32_t last_piece_bytes = arr_end - last_piece >= 16 ? 16u : static_cast<uint32_t>(arr_end - last_piece);
    const int head_skip = static_cast<int>((beg - a0) / sizeof(T));  // tokens of stage 0 before the request
    const int tail_count =                                           // valid tokens of the last stage
        static_cast<int>((span - static_cast<uint64_t>(n_stages > 0 ? n_stages - 1 : 0) * kStageBytes) / sizeof(T));
    int64_t max_stages = n_stages;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        const int64_t other = __shfl_xor_sync(0xffffffffu, max_stages, d);
        max_stages = other > max_stages ? other : max_stages;
    }

    const uint32_t ring = static_cast<uint32_t>(__cvta_generic_to_shared(smem)) + warp * kWarpRingBytes + lane * 16;
    auto issue = [&](int64_t s) {
        const uint32_t dst = ring + (static_cast<uint32_t>(s) & (kStages - 1)) * (kPieces * 512);
        const uint64_t src = a0 + static_cast<uint64_t>(s) * kStageBytes;
        if (s + 1 < n_stages) {  // an inner stage: four whole pieces
#pragma unroll
            for (int c = 0; c < kPieces; ++c) CpAsync16(dst + c * 512, src + c * 16, 16u);
        } else if (s < n_stages) {  // the last stage: some pieces may be absent, the last one short
            const int64_t p0 = s * kPieces;
#pragma unroll
            for (int c = 0; c < kPieces; ++c) {
                if (p0 + c < n_pieces) {
                    CpAsync16(dst + c * 512, src + c * 16, p0 + c == n_pieces - 1 ? last_piece_bytes : 16u);
                }
            }
        }
        CpAsyncCommit();
    };

    // Unpacks one stage from the ring into `token + golden` values (garbage beyond the request:
    // the caller never consumes those).
    auto unpack = [&](int64_t s, uint64_t (&vc)[kPerStage]) {
        const uint32_t src = ring + (static_cast<uint32_t>(s) & (kStages - 1)) * (kPieces * 512);
#pragma unroll
        for (int c = 0; c < kPieces; ++c) {
            uint4 q;
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                         : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
                         : "r"(src + c * 512));
            if constexpr (sizeof(T) == 4) {
                vc[c * kPerPiece + 0] = static_cast<uint64_t>(q.x) + kGolden;
                vc[c * kPerPiece + 1] = static_cast<uint64_t>(q.y) + kGolden;
                vc[c * kPerPiece + 2] = static_cast<uint64_t>(q.z) + kGolden;
                vc[c * kPerPiece + 3] = static_cast<uint64_t>(q.w) + kGolden;
            } else {
                vc[c * kPerPiece + 0] = (static_cast<uint64_t>(q.x) | (static_cast<uint64_t>(q.y) << 32)) + kGolden;
                vc[c * kPerPiece + 1] = (static_cast<uint64_t>(q.z) | (static_cast<uint64_t>(q.w) << 32)) + kGolden;
            }
        }
    };

    uint64_t h = 0;
    int32_t left = block_size;  // tokens still to come in the current block, this one included
    int64_t *out = keys + key_base;
    // Runs the chain over stage k, held in `vc`.
    auto consume = [&](int64_t k, const uint64_t (&vc)[kPerStage]) {
        if (k >= n_stages) return;
        const int lo = k == 0 ? head_skip : 0;
        const int hi = k == n_stages - 1 ? tail_count : kPerStage;
        if (lo == 0 && hi == kPerStage && block_size >= kPerStage) {
            RunFullStage<T, kAligned>(h, vc, left, out, block_size);
        } else {
#pragma unroll
            for (int i = 0; i < kPerStage; ++i) {
                if (i >= lo && i < hi) {
                    h = HashStepPre(h, vc[i]);
                    if (--left == 0) {
                        *out++ = static_cast<int64_t>(h);
                        left = block_size;
                    }
                }
            }
        }
    };

#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) issue(s);
    CpAsyncWait<kStages - 2>();  // stage 0 has landed
    uint64_t even[kPerStage], odd[kPerStage];
    unpack(0, even);
    // Stage k+1 is fetched from shared memory while the chain runs over stage k, which is already
    // in registers.  Two stages per trip so that the two register buffers swap roles without copies.
    for (int64_t k = 0; k < max_stages; k += 2) {
        issue(k + kStages - 1);
        CpAsyncWait<kStages - 2>();  // stage k+1 has landed; a lane only reads what it copied itself
        unpack(k + 1, odd);
        consume(k, even);
        issue(k + kStages);
        CpAsyncWait<kStages - 2>();  // stage k+2
        unpack(k + 2, even);
        consume(k + 1, odd);
    }
    CpAsyncWait<0>();
}

template <typename T>
int32_t LaunchHash(const T *d_tokens, int64_t n_tokens_total, const int64_t *d_tok_off, int32_t n_req,
                   int32_t block_size, int64_t *d_keys, const int64_t *d_key_off, const int32_t *d_order,
                   int32_t warps_per_sm, kvcm_stream_t stream) {
    if (!HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (n_req < 0 || block_size <= 0 || n_tokens_total < 0 || warps_per_sm < 0) return KVCM_ER_INVALID_PARAMS;
    if (n_req == 0) return KVCM_OK;
    if (d_tok_off == nullptr || d_key_off == nullptr || (d_tokens == nullptr && n_tokens_total > 0)) {
        return KVCM_ER_INVALID_ADDRESS;
    }
    if (n_tokens_total == 0) return KVCM_OK;  // every request is empty: no key to write
    if (d_keys == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (reinterpret_cast<uintptr_t>(d_tokens) & 15u) return KVCM_ER_INVALID_ADDRESS;  // 16-byte staging copies

    static bool attr_set = false;
    if (!attr_set) {
        const int bytes = kMaxHashSmemPerSm;
        cudaFuncSetAttribute(HashBlocksKernel<uint32_t, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        cudaFuncSetAttribute(HashBlocksKernel<uint32_t, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        cudaFuncSetAttribute(HashBlocksKernel<int64_t, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        cudaFuncSetAttribute(HashBlocksKernel<int64_t, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        attr_set = true;
    }
    // Few requests: half-filled warps, one per CTA, so the chains spread over as many SMs as possible.
    const int sms = GetDeviceInfo().sm_count;
    const uint32_t lanes_per_warp = static_cast<int64_t>(n_req) <= 16ll * sms * kHalfWarpSmMultiple ? 16u : 32u;
    const int64_t n_warps = (static_cast<int64_t>(n_req) + lanes_per_warp - 1) / lanes_per_warp;
    // One warp per CTA while every warp of the batch can be resident at once (16 KiB of shared memory
    // each, 14 per SM): a warp that finishes frees its slot alone and CTAs land on the SMs round-robin.
    // A caller that knows the batch is ruled by its longest chains (kvcm_b200_length_order says so) asks
    // for fewer resident warps per SM: shared memory per CTA is then padded so that only that many
    // one-warp CTAs fit, the longest chains - launched first - run alone on their scheduler, and the
    // shorter ones take over the slots as they free up.
    int warps_per_cta = n_warps <= 14ll * sms ? 1 : kMaxWarpsPerCta;
    size_t smem_per_warp = kWarpRingBytes;
    if (warps_per_sm > 0 && warps_per_sm < 14) {
        warps_per_cta = 1;
        smem_per_warp = (static_cast<size_t>(kMaxHashSmemPerSm) / warps_per_sm) & ~static_cast<size_t>(1023);
        if (smem_per_warp < kWarpRingBytes) smem_per_warp = kWarpRingBytes;
    }
    const size_t smem = static_cast<size_t>(warps_per_cta) * smem_per_warp;
    const unsigned grid = static_cast<unsigned>((n_warps + warps_per_cta - 1) / warps_per_cta);
    const unsigned threads = warps_per_cta * 32;
    constexpr int kPerStage = kStageBytes / sizeof(T);
    if (block_size % kPerStage == 0) {
        HashBlocksKernel<T, true><<<grid, threads, smem, AsStream(stream)>>>(
            d_tokens, n_tokens_total, d_tok_off, n_req, block_size, d_keys, d_key_off, d_order, lanes_per_warp);
    } else {
        HashBlocksKernel<T, false><<<grid, threads, smem, AsStream(stream)>>>(
            d_tokens, n_tokens_total, d_tok_off, n_req, block_size, d_keys, d_key_off, d_order, lanes_per_warp);
    }
    return LaunchStatus();
}

}  // namespace
}  // namespace kvcm

extern "C" {

int32_t kvcm_b200_hash_blocks_u32(const uint32_t *d_tokens, int64_t n_tokens_total, const int64_t *d_tok_off,
                                  int32_t n_req, int32_t block_size, int64_t *d_keys, const int64_t *d_key_off,
                                  const int32_t *d_req_order, int32_t warps_per_sm, kvcm_stream_t stream) {
    return kvcm::LaunchHash<uint32_t>(d_tokens, n_tokens_total, d_tok_off, n_req, block_size, d_keys, d_key_off,
                                      d_req_order, warps_per_sm, stream);
}

int32_t kvcm_b200_hash_blocks_i64(const int64_t *d_tokens, int64_t n_tokens_total, const int64_t *d_tok_off,
                                  int32_t n_req, int32_t block_size, int64_t *d_keys, const int64_t *d_key_off,
                                  const int32_t *d_req_order, int32_t warps_per_sm, kvcm_stream_t stream) {
    return kvcm::LaunchHash<int64_t>(d_tokens, n_tokens_total, d_tok_off, n_req, block_size, d_keys, d_key_off,
                                     d_req_order, warps_per_sm, stream);
}

int32_t kvcm_b200_length_order(const int64_t *h_tok_off, int32_t n_req, int32_t *h_order_out,
                               int32_t *warps_per_sm_out) {
    if (h_tok_off == nullptr || h_order_out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    if (n_req < 0) return KVCM_ER_INVALID_PARAMS;
    if (warps_per_sm_out != nullptr) *warps_per_sm_out = 0;
    std::vector<int32_t> idx(n_req);
    for (int32_t r = 0; r < n_req; ++r) idx[r] = r;
    std::stable_sort(idx.begin(), idx.end(), [&](int32_t a, int32_t b) {
        return h_tok_off[a + 1] - h_tok_off[a] > h_tok_off[b + 1] - h_tok_off[b];
    });
    for (int32_t r = 0; r < n_req; ++r) h_order_out[r] = idx[r];
    if (warps_per_sm_out != nullptr && n_req > 0) {
        // A lone warp advances one token per ~47 cycles (dependent chain); a scheduler shared by several
        // warps issues one token step per ~31 cycles in total.  If the longest chain alone outlasts the
        // whole batch spread over all schedulers, keep one warp per scheduler (4 per SM) so that chain is
        // never slowed down; otherwise fill the SMs.
        const int sms = kvcm::HaveDevice() ? kvcm::GetDeviceInfo().sm_count : 148;
        const double longest = static_cast<double>(h_tok_off[idx[0] + 1] - h_tok_off[idx[0]]);
        double warp_steps = 0;
        for (int32_t r = 0; r < n_req; r += 32) warp_steps += static_cast<double>(h_tok_off[idx[r] + 1] - h_tok_off[idx[r]]);
        *warps_per_sm_out = longest * 47.0 >= warp_steps * 31.0 / (4.0 * sms) ? 4 : 0;
    }
    return KVCM_OK;
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
