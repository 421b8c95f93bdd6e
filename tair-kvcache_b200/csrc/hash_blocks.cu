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
// Tokens are staged through shared memory by a producer warp with bulk copies (TMA); the consumer
// warp runs the chains out of registers.  The two sections below describe the chain loop and the
// staging ring.
#include <algorithm>
#include <mutex>
#include <utility>
#include <vector>

#include "kvcm_common.cuh"

namespace kvcm {
namespace {

constexpr int kStageBytes = 64;            // bytes of one lane unpacked into registers at a time
constexpr int kPieces = kStageBytes / 16;  // 128-bit shared loads per stage
constexpr int kSlots = 3;                  // ring fills per warp: two in flight ahead of the one being hashed
constexpr int kMaxWarpsPerCta = 4;         // consumer warps; a CTA has as many producer warps again
constexpr int kMaxHashSmemPerSm = 224 * 1024;
// Ring geometry for fills of kMinis 64-byte stages per lane: one bulk copy brings kMinis x 64 bytes of a request.
// A bulk copy costs its issuing lane the same ~54 cycles whatever its size (measured, 256 B to 2 KiB), so a warp
// fills a slot in ~1,700 cycles.  A chain that runs at ~21 cycles per token eats 64 tokens in ~1,350 cycles: with
// 256-byte fills the producer would hold it back, with 512-byte fills (kMinis = 8) it does not.  Launches ruled by
// their longest chains take kMinis = 8; launches with many warps per SM, ruled by the integer pipe, keep
// kMinis = 4, whose smaller ring lets twice as many warps stay resident.
template <int kMinis>
struct RingGeo {
    static constexpr int kLaneStride = kMinis * kStageBytes + 16;  // an odd number of 16-byte words
    static constexpr int kFillBytes = kMinis * kStageBytes;        // bytes of one lane in one ring slot
    static constexpr int kSlotBytes = 32 * kLaneStride;            // one ring slot of a warp
    static constexpr int kWarpRingBytes = kSlots * kSlotBytes;     // 25.5 KiB (kMinis 4), 49.5 KiB (kMinis 8)
    // Consumer warps that fit on an SM (1 KiB of shared memory per CTA goes to the system).
    static constexpr int kResidentWarpsPerSm = kMaxHashSmemPerSm / (kWarpRingBytes + 1024);
    static_assert(kMinis % 2 == 0 && (kLaneStride / 16) % 2 == 1, "ring geometry");
};
constexpr int kShallowMinis = 4, kDeepMinis = 8;
// Batches of up to 16 x SMs x this many requests run with half-filled warps.
constexpr int kHalfWarpSmMultiple = 2;

// What bounds this kernel is the latency of ONE lane's dependent chain (the longest request, ~37
// cycles per token), and for a lone warp on an SM the integer pipe takes two cycles per warp instruction.  So the loop is
// shaped to spend as few instructions per token as possible next to the chain itself:
//  * a stage (64 bytes per lane) is unpacked into registers, as `token + C`, one stage ahead of
//    the chain (ping-pong register buffers): shared-memory latency never sits on the chain;
//  * a stage that lies wholly inside the request runs as one unrolled run of steps.  When
//    block_size is a multiple of the tokens per stage, a block can only end at the positions
//    {last, 0 .. tokens-per-16-bytes - 2} of a stage (the request's misalignment against the
//    16-byte copy grid is a per-lane constant), so only those few positions carry a predicated
//    key store; other block sizes check every position;
//  * only the first and last stage of a request, and blocks shorter than a stage, take the
//    per-token checked path.
// With few requests (lanes_per_warp = 16) only half of each warp is used, so that twice as many
// SMs work on the batch and the longest chains do not share a warp's issue slots more than needed.
// One step on a raw 32-bit token, state in two 32-bit halves: hl * 4096 + C in one wide multiply-add (the golden
// constant rides on the addend), hh * 4096 + its high word in a second, then the three-input adds.  Against the
// plain 64-bit step on `token + C` this saves the two integer adds per token that form `token + C` and moves two
// operations from the integer pipe to the multiply-add pipe: measured 6-7 % faster on chain-bound batches.
// 64-bit tokens keep the plain step (their high word would need a fourth addend).
__device__ __forceinline__ void HashStepTok(uint32_t &hl, uint32_t &hh, uint32_t tok) {
    uint64_t w;
    const uint32_t k4096 = 4096u;
    asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(w) : "r"(hl), "r"(k4096), "l"(0x9e3779b97f4a7c15ull));
    uint32_t hi1;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(hi1) : "r"(hh), "r"(k4096), "r"(static_cast<uint32_t>(w >> 32)));
    const uint32_t bh = static_cast<uint32_t>(static_cast<int32_t>(hh) >> 31);
    const uint64_t lo = static_cast<uint64_t>(static_cast<uint32_t>(w)) + hh + tok;
    const uint32_t hi = hi1 + bh + static_cast<uint32_t>(lo >> 32);
    hl ^= static_cast<uint32_t>(lo);
    hh ^= hi;
}

template <typename T, bool kAligned>
__device__ __forceinline__ void RunFullStage(uint64_t &h, const uint64_t (&vc)[kStageBytes / sizeof(T)], int32_t &left,
                                             int64_t *&out, int32_t block_size) {
    constexpr int kPerPiece = 16 / sizeof(T);
    constexpr int kPerStage = kStageBytes / sizeof(T);
    if constexpr (sizeof(T) == 4) {
        uint32_t hl = static_cast<uint32_t>(h), hh = static_cast<uint32_t>(h >> 32);
#pragma unroll
        for (int i = 0; i < kPerStage; ++i) {
            HashStepTok(hl, hh, static_cast<uint32_t>(vc[i]));
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
        return;
    }
    // 64-bit tokens: plain 64-bit steps on `token + C`.
    uint64_t hx = h;
#pragma unroll
    for (int i = 0; i < kPerStage; ++i) {
        hx = HashStepPre(hx, vc[i]);
        if (!kAligned || i == kPerStage - 1 || i < kPerPiece - 1) {
            if (i + 1 == left) *out = static_cast<int64_t>(hx);
        }
    }
    h = hx;
    if (left <= kPerStage) {
        ++out;
        left += block_size;
    }
    left -= kPerStage;
}

// A whole ring fill (kMinis full stages of one lane) straight out of shared memory, for block sizes that are a
// multiple of the tokens per stage.  The loop body is nothing but plain 128-bit shared loads and chain steps: the
// compiler schedules the loads ahead of the chain by itself, and nothing that depends on run-time counters sits
// between two steps (a counter-driven store after every token costs a lone warp 43 cycles per token against 20 for
// the bare chain, measured).  A block can only end after the last token of a stage or after one of its first
// tokens-per-16-bytes - 1 (the request's misalignment against the 16-byte copy grid is a per-lane constant), so
// the hash after those few positions is kept, and once per stage the lane picks the one its block ends on.
template <typename T, int kMinis, bool kPlainStep>
__device__ __forceinline__ void RunFullFill(uint64_t &h, const uint4 *fill, int32_t &left, int64_t *&out,
                                            int32_t block_size) {
    constexpr int kPerPiece = 16 / sizeof(T);
    constexpr int kPerStage = kStageBytes / sizeof(T);
    uint64_t hx = h;
    uint32_t hl = static_cast<uint32_t>(h), hh = static_cast<uint32_t>(h >> 32);
#pragma unroll
    for (int s = 0; s < kMinis; ++s) {
        uint64_t at_end = 0, early[kPerPiece];  // hash after the stage's last token / after token e of the stage
#pragma unroll
        for (int c = 0; c < kPieces; ++c) {
            const uint4 q = fill[s * kPieces + c];
            if constexpr (sizeof(T) == 4) {
                const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if constexpr (kPlainStep) {
                        hx = HashStep(hx, w[j]);
                    } else {
                        HashStepTok(hl, hh, w[j]);
                        hx = static_cast<uint64_t>(hl) | (static_cast<uint64_t>(hh) << 32);
                    }
                    if (c == 0 && j < kPerPiece - 1) early[j] = hx;
                    if (c == kPieces - 1 && j == 3) at_end = hx;
                }
            } else {
                const uint64_t w[2] = {static_cast<uint64_t>(q.x) | (static_cast<uint64_t>(q.y) << 32),
                                       static_cast<uint64_t>(q.z) | (static_cast<uint64_t>(q.w) << 32)};
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    hx = HashStep(hx, w[j]);
                    if (c == 0 && j < kPerPiece - 1) early[j] = hx;
                    if (c == kPieces - 1 && j == 1) at_end = hx;
                }
            }
        }
        if (left <= kPerStage) {  // the block ends in this stage, after token left - 1
            uint64_t key = at_end;
#pragma unroll
            for (int e = 0; e < kPerPiece - 1; ++e) {
                if (left == e + 1) key = early[e];
            }
            *out++ = static_cast<int64_t>(key);
            left += block_size;
        }
        left -= kPerStage;
    }
    h = hx;
}

// ---------------------------------------------------------------------------------------------
// The staging ring.  One lane = one request, so the 32 lanes of a warp read 32 unrelated places of
// the token array.  Fetched with per-lane 16-byte copies that is 32 cache lines per warp instruction,
// and with more than a few warps per SM the L1 tag stage, not the chain, sets the pace (measured:
// 2.6x slower on 65,536 requests of 21k tokens).  Here a request is fetched kMinis x 64 bytes at a
// time with ONE bulk copy (cp.async.bulk, global -> shared, completion counted on an mbarrier),
// which goes through the TMA unit and bypasses L1.  A bulk copy costs its issuing warp some tens of
// cycles per lane (about 900 cycles per warp-wide fill), so the copies are issued by a second warp:
// CTA = consumer warps [0, n) that run the chains + producer warps [n, 2n), producer lane j
// fetching for consumer lane j (a one-consumer CTA may swap the two roles, see the kernel).  Per
// consumer warp and ring slot
// there is a `full` barrier (one arrival by the producer's lane 0 + the bytes in flight) and an `empty` barrier
// (one arrival by the consumer's lane 0 once every lane is through with the slot).  A lane's bytes of a slot are
// contiguous; lanes are kMinis*64+16 bytes apart, an odd number of 16-byte words, so the 128-bit
// reads of a warp stay conflict-free.  Every wait is bounded: after kSpinLimit polls the warp
// raises g_hash_wait_timeouts, waits once more (bounded) for the copies in flight, and returns.
// ---------------------------------------------------------------------------------------------
__device__ uint32_t g_hash_wait_timeouts = 0;

// Where a lane's request lies in the token array, as the staging copies see it.
template <typename T>
struct LaneSpan {
    uint64_t a0;          // 16-byte aligned start of the bytes to fetch
    uint64_t fetch;       // bytes to fetch, a multiple of 16
    uint64_t bulk_total;  // of which bulk copies bring this many (the rest is the piece at the array's end)
    uint32_t over;        // bytes by which the last piece would overrun the token array (0..15)
    int64_t n_stages;     // 64-byte stages
    int64_t n_ring;       // ring fills
    int head_skip;        // tokens of stage 0 that precede the request
    int tail_count;       // valid tokens of the last stage
    int64_t key_base;
};

template <typename T, int kMinis>
__device__ __forceinline__ LaneSpan<T> DescribeLane(const T *tokens, int64_t n_tokens_total, const int64_t *tok_off,
                                                    const int64_t *key_off, const int32_t *order, int64_t pos,
                                                    bool active, int32_t block_size) {
    LaneSpan<T> s;
    const int64_t req = active && order != nullptr ? order[pos] : pos;
    int64_t first_tok = 0, n_tok = 0;
    s.key_base = 0;
    if (active) {
        first_tok = tok_off[req];
        n_tok = tok_off[req + 1] - first_tok;
        s.key_base = key_off[req];
    }
    // Only whole blocks are hashed; the trailing partial block is never read.
    const int64_t used = n_tok > 0 ? (n_tok / block_size) * block_size : 0;
    const uint64_t arr_beg = reinterpret_cast<uint64_t>(tokens);
    const uint64_t arr_end = arr_beg + static_cast<uint64_t>(n_tokens_total) * sizeof(T);
    const uint64_t beg = arr_beg + static_cast<uint64_t>(first_tok) * sizeof(T);
    const uint64_t end = beg + static_cast<uint64_t>(used) * sizeof(T);
    s.a0 = beg & ~15ull;  // arr_beg is 16-byte aligned, so a0 >= arr_beg
    const uint64_t span = used > 0 ? end - s.a0 : 0;
    s.n_stages = static_cast<int64_t>((span + kStageBytes - 1) / kStageBytes);
    s.n_ring = (s.n_stages + kMinis - 1) / kMinis;
    s.fetch = (span + 15) & ~15ull;
    s.over = s.a0 + s.fetch > arr_end ? static_cast<uint32_t>(s.a0 + s.fetch - arr_end) : 0u;
    s.bulk_total = s.over > 0 ? s.fetch - 16 : s.fetch;
    s.head_skip = static_cast<int>((beg - s.a0) / sizeof(T));
    s.tail_count =
        static_cast<int>((span - static_cast<uint64_t>(s.n_stages > 0 ? s.n_stages - 1 : 0) * kStageBytes) / sizeof(T));
    return s;
}

template <typename T, bool kAligned, int kMinis>
__global__ void __launch_bounds__(2 * kMaxWarpsPerCta * 32)
    HashBlocksKernel(const T *__restrict__ tokens, int64_t n_tokens_total, const int64_t *__restrict__ tok_off,
                         int32_t n_req, int32_t block_size, int64_t *__restrict__ keys,
                         const int64_t *__restrict__ key_off, const int32_t *__restrict__ order,
                         uint32_t lanes_per_warp, uint32_t warp_smem_bytes) {
    using Geo = RingGeo<kMinis>;
    static_assert(kSlots >= 2, "ring geometry");
    constexpr int kLaneStride = Geo::kLaneStride;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bars[kMaxWarpsPerCta][kSlots];
    __shared__ __align__(8) uint64_t empty_bars[kMaxWarpsPerCta][kSlots];
    constexpr int kPerPiece = 16 / sizeof(T);
    constexpr int kPerStage = kStageBytes / sizeof(T);
    constexpr uint64_t kGolden = 0x9e3779b97f4a7c15ull;
    constexpr uint32_t kFull = Geo::kFillBytes;   // bytes of one lane in one ring slot
    constexpr uint32_t kSlotBytes = Geo::kSlotBytes;  // one ring slot of a warp
    const uint32_t lane = LaneId();
    const uint32_t n_consumers = blockDim.x >> 6;
    const uint32_t warp_in_cta = threadIdx.x >> 5;
    __shared__ uint32_t swap_roles;

    if (threadIdx.x == 0) {
        // A two-warp CTA sits in warp slots (2k, 2k+1) of its SM and a warp's scheduler is its slot modulo
        // 4, so with the consumer always first the chains of all CTAs of an SM would crowd onto
        // schedulers 0 and 2 (measured: issue-active 57% on two schedulers, 23% on the others).  The first
        // warp reads its slot and the CTA swaps the roles in every other pair of pairs: consumers then
        // land on slots 0, 2, 5, 7, ... = schedulers 0, 2, 1, 3.  Only balance depends on this.
        uint32_t slot_id;
        asm volatile("mov.u32 %0, %%warpid;\n" : "=r"(slot_id));
        swap_roles = n_consumers == 1 ? (slot_id >> 2) & 1u : 0u;
        for (uint32_t w = 0; w < n_consumers; ++w) {
#pragma unroll
            for (int s = 0; s < kSlots; ++s) {
                MbarInit(SmemAddr(&full_bars[w][s]), 1);   // one arrival per fill: the producer's lane 0
                MbarInit(SmemAddr(&empty_bars[w][s]), 1);  // one arrival per fill: the consumer's lane 0
            }
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async;\n" ::: "memory");
    }
    __syncthreads();
    const bool producer = n_consumers == 1 ? (warp_in_cta ^ swap_roles) == 1 : warp_in_cta >= n_consumers;
    const uint32_t warp = n_consumers == 1 ? 0 : (producer ? warp_in_cta - n_consumers : warp_in_cta);  // consumer served
    const int64_t pos = (static_cast<int64_t>(blockIdx.x) * n_consumers + warp) * lanes_per_warp + lane;
    const bool active = lane < lanes_per_warp && pos < n_req;

    const LaneSpan<T> sp =
        DescribeLane<T, kMinis>(tokens, n_tokens_total, tok_off, key_off, order, pos, active, block_size);
    int64_t max_ring = sp.n_ring;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        const int64_t other = __shfl_xor_sync(0xffffffffu, max_ring, d);
        max_ring = other > max_ring ? other : max_ring;
    }
    const uint32_t full0 = SmemAddr(&full_bars[warp][0]);
    const uint32_t empty0 = SmemAddr(&empty_bars[warp][0]);
    const uint32_t ring = SmemAddr(smem) + warp * warp_smem_bytes + lane * kLaneStride;

    if (producer) {
        // Fill r carries this lane's bytes [r*kFull, (r+1)*kFull) of its request into slot r % kSlots.
        // A phase of `full` is one fill of the warp, whether or not every lane still has bytes to fetch.
        bool ok = true;
        uint32_t slot = 0, round = 0;  // r = round * kSlots + slot
        for (int64_t r = 0; r < max_ring && ok; ++r) {
            if (round > 0) ok = BoundedWait<true>(empty0 + slot * 8, (round - 1) & 1u);  // fill r - kSlots was drained
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint32_t bar = full0 + slot * 8;
            const uint64_t at = static_cast<uint64_t>(r) * kFull;
            if (sp.over > 0 && r == sp.n_ring - 1) {  // the piece at the very end of the token array
                const uint64_t tail_at = sp.fetch - 16;
                const T *src = reinterpret_cast<const T *>(sp.a0 + tail_at);
                const uint32_t dst = ring + slot * kSlotBytes + static_cast<uint32_t>(tail_at - at);
                const int n_words = static_cast<int>((16 - sp.over) / sizeof(T));
                for (int w = 0; w < n_words; ++w) {
                    if constexpr (sizeof(T) == 4) {
                        asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(dst + w * 4), "r"(static_cast<uint32_t>(src[w]))
                                     : "memory");
                    } else {
                        asm volatile("st.shared.u64 [%0], %1;\n" ::"r"(dst + w * 8), "l"(static_cast<uint64_t>(src[w]))
                                     : "memory");
                    }
                }
            }
            // One arrival per fill, by lane 0, announcing the bytes of all 32 lanes (a barrier operation is a
            // shared-memory atomic on the pipe the consumers' shared loads use: 32 per fill and warp were felt by
            // the chains of every warp on the SM).  It follows the warp's tail words (__syncwarp orders them before
            // it, its release publishes them) and precedes the copies.
            uint32_t bytes = 0;
            if (r < sp.n_ring && at < sp.bulk_total) {
                bytes = sp.bulk_total - at >= kFull ? kFull : static_cast<uint32_t>(sp.bulk_total - at);
            }
            const uint32_t warp_bytes = __reduce_add_sync(0xffffffffu, bytes);
            __syncwarp();
            if (lane == 0) MbarArriveExpectTx(bar, warp_bytes);
            __syncwarp();
            if (bytes > 0) BulkLoad(ring + slot * kSlotBytes, reinterpret_cast<const void *>(sp.a0 + at), bytes, bar);
            if (++slot == kSlots) {
                slot = 0;
                ++round;
            }
        }
        if (!ok && lane == 0) atomicAdd(&g_hash_wait_timeouts, 1u);
        return;  // copies still in flight land in shared memory that lives until the consumer, which waits for them, is done
    }

    // ---- consumer ----
    // Unpacks 64-byte stage m of the fill held in the slot at `slot_base`: raw 32-bit tokens, or `token + golden`
    // for 64-bit tokens (garbage beyond the request: the caller never consumes those).
    auto unpack = [&](uint32_t slot_base, int m, uint64_t (&vc)[kPerStage]) {
        const uint32_t src = slot_base + m * kStageBytes;
#pragma unroll
        for (int c = 0; c < kPieces; ++c) {
            uint4 q;
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                         : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
                         : "r"(src + c * 16));
            if constexpr (sizeof(T) == 4) {
                vc[c * kPerPiece + 0] = q.x;  // 32-bit tokens stay raw: their step adds the constant itself
                vc[c * kPerPiece + 1] = q.y;
                vc[c * kPerPiece + 2] = q.z;
                vc[c * kPerPiece + 3] = q.w;
            } else {
                vc[c * kPerPiece + 0] = (static_cast<uint64_t>(q.x) | (static_cast<uint64_t>(q.y) << 32)) + kGolden;
                vc[c * kPerPiece + 1] = (static_cast<uint64_t>(q.z) | (static_cast<uint64_t>(q.w) << 32)) + kGolden;
            }
        }
    };

    uint64_t h = 0;
    int32_t left = block_size;  // tokens still to come in the current block, this one included
    int64_t *out = keys + sp.key_base;
    const int64_t n_stages = sp.n_stages;
    // Runs the chain over 64-byte stage k, held in `vc`.
    auto consume = [&](int64_t k, const uint64_t (&vc)[kPerStage]) {
        if (k >= n_stages) return;
        const int lo = k == 0 ? sp.head_skip : 0;
        const int hi = k == n_stages - 1 ? sp.tail_count : kPerStage;
        if (lo == 0 && hi == kPerStage && block_size >= kPerStage) {
            RunFullStage<T, kAligned>(h, vc, left, out, block_size);
        } else {
#pragma unroll
            for (int i = 0; i < kPerStage; ++i) {
                if (i >= lo && i < hi) {
                    h = sizeof(T) == 4 ? HashStep(h, vc[i]) : HashStepPre(h, vc[i]);
                    if (--left == 0) {
                        *out++ = static_cast<int64_t>(h);
                        left = block_size;
                    }
                }
            }
        }
    };

    if constexpr (kAligned) {
        // Block sizes that are a multiple of a stage (16, 32, 64 ... tokens): a fill that lies wholly inside the
        // lane's request runs as one straight piece of code out of shared memory (RunFullFill); the first and the
        // last fill of a request, which hold tokens that are not the request's, go stage by stage through the
        // checked path.  The wait for a fill sits right before its first use: the producer runs two fills ahead,
        // so it returns at once, and the slot is handed back when the fill has been hashed.
        const uint8_t *lane_ring = smem + warp * warp_smem_bytes + lane * kLaneStride;
        bool ok = true;
        uint32_t slot = 0, round = 0;  // fill r = round * kSlots + slot
        int64_t waited = 0;            // fills whose `full` wait has returned
        uint64_t stage[kPerStage];
        for (int64_t r = 0; r < max_ring; ++r) {
            ok = BoundedWait(full0 + slot * 8, round & 1u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            ++waited;
            const int64_t k0 = r * kMinis;
            const bool whole = k0 + kMinis <= n_stages && (k0 > 0 || sp.head_skip == 0) &&
                               (k0 + kMinis < n_stages || sp.tail_count == kPerStage);
            if (whole) {
                RunFullFill<T, kMinis, kMinis == kDeepMinis>(
                    h, reinterpret_cast<const uint4 *>(lane_ring + slot * kSlotBytes), left, out, block_size);
            } else if (k0 < n_stages) {
#pragma unroll 1
                for (int m = 0; m < kMinis; ++m) {
                    unpack(ring + slot * kSlotBytes, m, stage);
                    consume(k0 + m, stage);
                }
            }
            __syncwarp();
            if (lane == 0) MbarArrive(empty0 + slot * 8);  // every lane has hashed its part: the slot may be refilled
            if (++slot == kSlots) {
                slot = 0;
                ++round;
            }
        }
        if (!ok) {
            // Leave no copy in flight behind: one more bounded wait for each fill the producer may have started.
            for (int64_t r = waited; r < max_ring && r < waited + kSlots; ++r) {
                BoundedWait(full0 + static_cast<uint32_t>(r % kSlots) * 8, static_cast<uint32_t>(r / kSlots) & 1u);
            }
            if (lane == 0) atomicAdd(&g_hash_wait_timeouts, 1u);
        }
        return;
    }
    bool ok = max_ring == 0 || BoundedWait(full0, 0);
    ok = __all_sync(0xffffffffu, ok);
    uint64_t even[kPerStage], odd[kPerStage];
    uint32_t slot = 0, round = 0;  // fill r = round * kSlots + slot
    int64_t waited = 1;            // fills whose `full` wait has returned
    if (ok && max_ring > 0) {
        unpack(ring, 0, even);
        for (int64_t r = 0; r < max_ring; ++r) {
            const uint32_t next_slot = slot + 1 == kSlots ? 0 : slot + 1;
            const uint32_t next_round = slot + 1 == kSlots ? round + 1 : round;
            const uint32_t cur = ring + slot * kSlotBytes;
            const uint32_t nxt = ring + next_slot * kSlotBytes;
            const int64_t k0 = r * kMinis;
#pragma unroll
            for (int m = 0; m < kMinis; m += 2) {
                // Stage m+1 is fetched from shared memory while the chain runs over stage m, which is
                // already in registers; two stages per step so the register buffers swap without copies.
                unpack(cur, m + 1, odd);
                consume(k0 + m, even);
                if (m + 2 < kMinis) {
                    unpack(cur, m + 2, even);
                } else {
                    __syncwarp();
                    if (lane == 0) MbarArrive(empty0 + slot * 8);  // this fill now lives in registers: the slot may be refilled
                    if (r + 1 < max_ring) {
                        ok = BoundedWait(full0 + next_slot * 8, next_round & 1u);
                        ok = __all_sync(0xffffffffu, ok);
                        if (ok) {
                            ++waited;
                            unpack(nxt, 0, even);
                        }
                    }
                }
                consume(k0 + m + 1, odd);
            }
            if (!ok) break;
            slot = next_slot;
            round = next_round;
        }
    }
    if (!ok) {
        // Leave no copy in flight behind: one more bounded wait for each fill the producer may have started.
        for (int64_t r = waited; r < max_ring && r < waited + kSlots; ++r) {
            BoundedWait(full0 + static_cast<uint32_t>(r % kSlots) * 8, static_cast<uint32_t>(r / kSlots) & 1u);
        }
        if (lane == 0) atomicAdd(&g_hash_wait_timeouts, 1u);
    }
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

    const int sms = GetDeviceInfo().sm_count;
    // Few requests: half-filled warps, one per CTA, so the chains spread over as many SMs as possible.
    const uint32_t lanes_per_warp = static_cast<int64_t>(n_req) <= 16ll * sms * kHalfWarpSmMultiple ? 16u : 32u;
    const int64_t n_warps = (static_cast<int64_t>(n_req) + lanes_per_warp - 1) / lanes_per_warp;
    // One consumer warp (+ its producer) per CTA while every warp of the batch can be resident at once:
    // a warp that finishes frees its slot alone and CTAs land on the SMs round-robin.
    // A caller that knows the batch is ruled by its longest chains (kvcm_b200_length_order says so) asks
    // for fewer resident warps per SM: shared memory per CTA is then padded so that only that many
    // one-warp CTAs fit, the longest chains - launched first - run alone on their scheduler, and the
    // shorter ones take over the slots as they free up.
    // Ruled by the longest chains (the caller says so, or there are no more warps than schedulers): deep fills.
    const bool deep = (warps_per_sm > 0 && warps_per_sm <= RingGeo<kDeepMinis>::kResidentWarpsPerSm) ||
                      n_warps <= static_cast<int64_t>(RingGeo<kDeepMinis>::kResidentWarpsPerSm) * sms;
    const int ring_bytes = deep ? RingGeo<kDeepMinis>::kWarpRingBytes : RingGeo<kShallowMinis>::kWarpRingBytes;
    const int resident = deep ? RingGeo<kDeepMinis>::kResidentWarpsPerSm : RingGeo<kShallowMinis>::kResidentWarpsPerSm;
    int warps_per_cta = n_warps <= static_cast<int64_t>(resident) * sms ? 1 : kMaxWarpsPerCta;
    size_t smem_per_warp = static_cast<size_t>(ring_bytes);
    if (warps_per_sm > 0 && warps_per_sm < resident) {
        warps_per_cta = 1;
        smem_per_warp = std::max<size_t>(smem_per_warp, (static_cast<size_t>(kMaxHashSmemPerSm) / warps_per_sm - 1024) &
                                                            ~static_cast<size_t>(1023));
    }
    const size_t smem = static_cast<size_t>(warps_per_cta) * smem_per_warp;
    const unsigned grid = static_cast<unsigned>((n_warps + warps_per_cta - 1) / warps_per_cta);
    const unsigned threads = 2 * warps_per_cta * 32;  // consumer warps + their producer warps
    constexpr int kPerStage = kStageBytes / sizeof(T);
    auto launch = [&](auto kernel) {
        EnsureDynamicSmem(kernel, kMaxHashSmemPerSm);
        kernel<<<grid, threads, smem, AsStream(stream)>>>(d_tokens, n_tokens_total, d_tok_off, n_req, block_size, d_keys,
                                                          d_key_off, d_order, lanes_per_warp,
                                                          static_cast<uint32_t>(smem_per_warp));
    };
    if (block_size % kPerStage == 0) {
        deep ? launch(HashBlocksKernel<T, true, kDeepMinis>) : launch(HashBlocksKernel<T, true, kShallowMinis>);
    } else {
        deep ? launch(HashBlocksKernel<T, false, kDeepMinis>) : launch(HashBlocksKernel<T, false, kShallowMinis>);
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

int32_t kvcm_b200_hash_wait_timeouts(uint32_t *h_count_out) {
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (h_count_out == nullptr) return KVCM_ER_INVALID_ADDRESS;
    const cudaError_t e = cudaMemcpyFromSymbol(h_count_out, kvcm::g_hash_wait_timeouts, sizeof(uint32_t));
    return e == cudaSuccess ? KVCM_OK : KVCM_ER_CUDAMEMCPY_ERROR;
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
        // How many hashing warps per SM finish the batch first.  Measured cycles per token of a chain with c
        // hashing warps (and their producers) on its SM: 25 alone, ~29 with 2, ~32 with 3, ~35 with 4; with the
        // SM filled (8 warps, small fills) a chain crawls at ~55 but the SM as a whole does about as many steps
        // per cycle as with 4.  A batch takes the longer of its longest chain at that pace and of all its warp
        // steps spread over the resident warps; pick the c that makes that shortest (0 = fill the SMs).
        const int sms = kvcm::HaveDevice() ? kvcm::GetDeviceInfo().sm_count : 148;
        const double longest = static_cast<double>(h_tok_off[idx[0] + 1] - h_tok_off[idx[0]]);
        double warp_steps = 0;
        for (int32_t r = 0; r < n_req; r += 32) warp_steps += static_cast<double>(h_tok_off[idx[r] + 1] - h_tok_off[idx[r]]);
        const int caps[4] = {2, 3, 4, 0};
        const double pace[4] = {29.0, 32.0, 35.0, 55.0};
        const double steps_per_cycle_per_sm[4] = {2 / 29.0, 3 / 32.0, 4 / 35.0, 4 / 34.0};
        double best = 0;
        for (int i = 0; i < 4; ++i) {
            const double chain = longest * pace[i];
            const double volume = warp_steps / (steps_per_cycle_per_sm[i] * sms);
            const double t = chain > volume ? chain : volume;
            if (i == 0 || t < best) {
                best = t;
                *warps_per_sm_out = caps[i];
            }
        }
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
