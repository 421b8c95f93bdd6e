// Paged-KV gather / scatter for sm_100a.
//
// Stands in for the Triton kernels of
// kv_cache_manager/py_connector/kernel/batch_gather_scatter_helper.py:33-98,139-205 and
// kv_cache_manager/py_connector/kernel/gather_scatter_helper.py:10-107.
//
// Data layout in HBM.  A pool is [pool_rows, row_bytes]; a staging slot is
// [n_pools, rows_per_block, row_bytes].  The (block, pool) pair owns one contiguous *tile* of
// tile_bytes = rows_per_block * row_bytes in staging, made of rows_per_block runs that are
// each contiguous in the pool.  Tiles are cut into fixed chunks of kChunkBytes; chunk ids are
// dealt round-robin to a persistent grid, so neighbouring CTAs stream neighbouring staging
// bytes and every CTA moves the same number of bytes.
//
// The kernel is a pure byte mover bounded by HBM bandwidth: per chunk every thread issues
// kUnroll independent 16-byte loads before the first store (32 KiB in flight per CTA), with
// streaming cache hints because no byte is touched twice.  The row index of a 16-byte vector
// is one 32-bit division by row_bytes and one cached 4-byte table read - the table is read
// per vector from L1, never per element from DRAM.
#include <cstdlib>
#include <cstring>

#include "kvcm_common.cuh"

namespace kvcm {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 8;
constexpr uint32_t kVecBytes = 16;
constexpr uint32_t kChunkBytes = kThreads * kVecBytes * kUnroll;  // 32 KiB

// Cache policy of the 16-byte accesses: 0 default, 1 streaming (evict-first) loads and stores,
// 2 streaming loads with default stores.
template <int kHint>
__device__ __forceinline__ uint4 LoadVec(const void *p) {
    if constexpr (kHint == 0) {
        return *reinterpret_cast<const uint4 *>(p);
    } else {
        return __ldcs(reinterpret_cast<const uint4 *>(p));
    }
}
template <int kHint>
__device__ __forceinline__ void StoreVec(void *p, uint4 v) {
    if constexpr (kHint == 1) {
        __stcs(reinterpret_cast<uint4 *>(p), v);
    } else {
        *reinterpret_cast<uint4 *>(p) = v;
    }
}

struct MoveParams {
    const uint64_t *pool_ptrs;  // device array of base addresses
    uint8_t *staging;
    const int32_t *row_idx;
    const int32_t *slot_idx;  // may be null: slot = block
    uint32_t *status;         // may be null
    int64_t n_slots;
    int64_t pool_rows;
    int64_t sub_stride;  // bytes between the sub-pools addressed through one pointer
    int64_t slot_bytes;  // n_pools * tile_bytes
    uint32_t row_bytes;
    uint32_t tile_bytes;
    uint32_t chunks_per_tile;
    uint32_t total_chunks;
    int32_t n_pools;      // tiles per block = pointers * sub_per_ptr
    int32_t sub_per_ptr;  // 1, or 2 for the legacy [2, total_tokens, hidden] layer tensors
    int32_t rows_per_block;
    int32_t report_skips;  // 0 for the legacy form, which skips silently
    uint32_t chunk_bytes;  // bytes per work item (fixed kChunkBytes for the vector kernel)
    int32_t stages;        // ring depth of the bulk kernel
};

__device__ __forceinline__ void ReportSkip(const MoveParams &p, uint32_t block, uint32_t count) {
    if (p.report_skips && p.status != nullptr) {
        atomicAdd(&p.status[0], count);
        atomicMax(&p.status[1], block + 1u);
    }
}

// kGather: pool -> staging.  !kGather: staging -> pool.
template <bool kGather, int kHint>
__global__ void __launch_bounds__(kThreads) MoveRowsKernel(const MoveParams p) {
    const uint32_t tid = threadIdx.x;
    for (uint32_t chunk = blockIdx.x; chunk < p.total_chunks; chunk += gridDim.x) {
        const uint32_t tile = chunk / p.chunks_per_tile;
        const uint32_t chunk_in_tile = chunk - tile * p.chunks_per_tile;
        const uint32_t block = tile / static_cast<uint32_t>(p.n_pools);
        const uint32_t pool = tile - block * static_cast<uint32_t>(p.n_pools);

        const int64_t slot = p.slot_idx != nullptr ? static_cast<int64_t>(__ldg(p.slot_idx + block))
                                                   : static_cast<int64_t>(block);
        if (slot < 0 || slot >= p.n_slots) {
            if (tid == 0 && chunk_in_tile == 0) ReportSkip(p, block, static_cast<uint32_t>(p.rows_per_block));
            continue;
        }
        const uint32_t ptr_i = pool / static_cast<uint32_t>(p.sub_per_ptr);
        const uint32_t sub_i = pool - ptr_i * static_cast<uint32_t>(p.sub_per_ptr);
        uint8_t *pool_base = reinterpret_cast<uint8_t *>(__ldg(p.pool_ptrs + ptr_i)) + sub_i * p.sub_stride;
        uint8_t *stage = p.staging + slot * p.slot_bytes + static_cast<int64_t>(pool) * p.tile_bytes;
        const int32_t *rows = p.row_idx + static_cast<int64_t>(block) * p.rows_per_block;
        const uint32_t chunk_off = chunk_in_tile * kChunkBytes;

        const bool aligned =
            ((reinterpret_cast<uintptr_t>(pool_base) | reinterpret_cast<uintptr_t>(stage) | p.row_bytes) & 15u) == 0;
        if (aligned) {
            uint4 v[kUnroll];
            uint8_t *in_pool[kUnroll];
            uint32_t off[kUnroll];
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                off[j] = chunk_off + (static_cast<uint32_t>(j) * kThreads + tid) * kVecBytes;
                in_pool[j] = nullptr;
                if (off[j] < p.tile_bytes) {
                    const uint32_t r = off[j] / p.row_bytes;
                    const uint32_t within = off[j] - r * p.row_bytes;
                    const int64_t row = __ldg(rows + r);
                    if (row >= 0 && row < p.pool_rows) {
                        in_pool[j] = pool_base + row * p.row_bytes + within;
                    } else if (within == 0) {
                        ReportSkip(p, block, 1u);
                    }
                }
            }
            if (kGather) {
#pragma unroll
                for (int j = 0; j < kUnroll; ++j) {
                    if (in_pool[j] != nullptr) v[j] = LoadVec<kHint>(in_pool[j]);
                }
#pragma unroll
                for (int j = 0; j < kUnroll; ++j) {
                    if (in_pool[j] != nullptr) StoreVec<kHint>(stage + off[j], v[j]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < kUnroll; ++j) {
                    if (in_pool[j] != nullptr) v[j] = LoadVec<kHint>(stage + off[j]);
                }
#pragma unroll
                for (int j = 0; j < kUnroll; ++j) {
                    if (in_pool[j] != nullptr) StoreVec<kHint>(in_pool[j], v[j]);
                }
            }
        } else {
            // Any alignment: one byte per thread per step.  Correct for odd row sizes and
            // unaligned base addresses; not a fast path.
            const uint32_t end = min(p.tile_bytes, chunk_off + kChunkBytes);
            for (uint32_t o = chunk_off + tid; o < end; o += kThreads) {
                const uint32_t r = o / p.row_bytes;
                const uint32_t within = o - r * p.row_bytes;
                const int64_t row = __ldg(rows + r);
                if (row >= 0 && row < p.pool_rows) {
                    uint8_t *q = pool_base + row * p.row_bytes + within;
                    if (kGather) {
                        stage[o] = *q;
                    } else {
                        *q = stage[o];
                    }
                } else if (within == 0) {
                    ReportSkip(p, block, 1u);
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// Bulk-copy (TMA) mover.  One warp per CTA; lane 0 drives a ring of kBulkStages shared-memory
// buffers of kChunkBytes with cp.async.bulk: global -> shared completes on an mbarrier,
// shared -> global is tracked by bulk groups.  No thread touches the payload, so the SM spends
// a few hundred instructions per 32 KiB.  Used when rows are large multiples of 16 bytes; a chunk
// whose pool base turns out to be misaligned is copied by the warp with plain byte accesses.
// Every wait is bounded: after kSpinLimit failed polls the CTA raises status[2] and leaves.
// ------------------------------------------------------------------------------------------
constexpr int kBulkMaxStages = 8;
constexpr uint32_t kBulkMinRowBytes = 512;

struct ChunkDesc {
    uint8_t *pool_base;
    uint8_t *stage;  // start of this chunk in staging
    const int32_t *rows;
    uint32_t chunk_off;  // offset of the chunk inside its tile
    uint32_t len;
    uint32_t block;
    bool first_in_tile;
    bool slot_ok;
    bool aligned;
};

__device__ __forceinline__ ChunkDesc Describe(const MoveParams &p, uint32_t chunk) {
    ChunkDesc d;
    const uint32_t tile = chunk / p.chunks_per_tile;
    const uint32_t chunk_in_tile = chunk - tile * p.chunks_per_tile;
    d.block = tile / static_cast<uint32_t>(p.n_pools);
    const uint32_t pool = tile - d.block * static_cast<uint32_t>(p.n_pools);
    const int64_t slot = p.slot_idx != nullptr ? static_cast<int64_t>(__ldg(p.slot_idx + d.block))
                                               : static_cast<int64_t>(d.block);
    d.slot_ok = slot >= 0 && slot < p.n_slots;
    d.first_in_tile = chunk_in_tile == 0;
    d.chunk_off = chunk_in_tile * p.chunk_bytes;
    d.len = min(p.chunk_bytes, p.tile_bytes - d.chunk_off);
    const uint32_t ptr_i = pool / static_cast<uint32_t>(p.sub_per_ptr);
    const uint32_t sub_i = pool - ptr_i * static_cast<uint32_t>(p.sub_per_ptr);
    d.pool_base = reinterpret_cast<uint8_t *>(__ldg(p.pool_ptrs + ptr_i)) + sub_i * p.sub_stride;
    d.stage = p.staging + (d.slot_ok ? slot : 0) * p.slot_bytes + static_cast<int64_t>(pool) * p.tile_bytes +
              d.chunk_off;
    d.rows = p.row_idx + static_cast<int64_t>(d.block) * p.rows_per_block;
    d.aligned = (reinterpret_cast<uintptr_t>(d.pool_base) & 15u) == 0;
    return d;
}

// The runs of a chunk: maximal pieces that are contiguous in the pool (a chunk that starts in
// the middle of a row begins with the rest of that row).  Run j is described without walking
// runs 0..j-1, so the lanes of the warp take runs j = lane, lane + 32, ... independently.
struct RunWalker {
    uint32_t first_row;
    uint32_t first_within;
    uint32_t first_len;
    uint32_t n_runs;
};

__device__ __forceinline__ RunWalker WalkRuns(const MoveParams &p, const ChunkDesc &d) {
    RunWalker w;
    w.first_row = d.chunk_off / p.row_bytes;
    w.first_within = d.chunk_off - w.first_row * p.row_bytes;
    w.first_len = min(p.row_bytes - w.first_within, d.len);
    w.n_runs = 1 + (d.len - w.first_len + p.row_bytes - 1) / p.row_bytes;
    return w;
}

// Run j: offset inside the chunk, address in the pool (nullptr when the row index is out of
// range), length, and whether the run starts its row (the lane that reports a skipped row).
__device__ __forceinline__ void GetRun(const MoveParams &p, const ChunkDesc &d, const RunWalker &w, uint32_t j,
                                       uint32_t *off, uint8_t **addr, uint32_t *len, bool *starts_row) {
    const uint32_t within = j == 0 ? w.first_within : 0;
    *off = j == 0 ? 0 : w.first_len + (j - 1) * p.row_bytes;
    *len = j == 0 ? w.first_len : min(p.row_bytes, d.len - *off);
    *starts_row = within == 0;
    const int64_t row = __ldg(d.rows + w.first_row + j);
    *addr = (row >= 0 && row < p.pool_rows) ? d.pool_base + row * p.row_bytes + within : nullptr;
}

template <bool kGather>
__global__ void __launch_bounds__(32) MoveRowsBulkKernel(const MoveParams p) {
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ __align__(8) uint64_t bars[kBulkMaxStages];
    const uint32_t lane = threadIdx.x;
    const uint32_t n_stages = static_cast<uint32_t>(p.stages);
    if (lane == 0) {
        for (uint32_t s = 0; s < n_stages; ++s) MbarInit(SmemAddr(&bars[s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async;\n" ::: "memory");
    }
    __syncwarp();
    const uint32_t ring_base = SmemAddr(ring);
    const uint32_t n_my =
        p.total_chunks > blockIdx.x ? (p.total_chunks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    uint32_t direct_mask = 0;  // bit s: the chunk in stage s was handled without the ring

    // Fills stage k % n_stages with chunk k.  Gather: one bulk load per run, issued by as many
    // lanes as there are runs.  Scatter: the chunk is contiguous in staging, one load.
    auto load = [&](uint32_t k) {
        const uint32_t s = k % n_stages;
        const uint32_t bar = SmemAddr(&bars[s]);
        const uint32_t buf = ring_base + s * p.chunk_bytes;
        const ChunkDesc d = Describe(p, blockIdx.x + k * gridDim.x);
        direct_mask &= ~(1u << s);
        if (!d.slot_ok) {
            if (lane == 0) {
                if (d.first_in_tile) ReportSkip(p, d.block, static_cast<uint32_t>(p.rows_per_block));
                MbarArriveExpectTx(bar, 0);
            }
            direct_mask |= 1u << s;
            return;
        }
        const RunWalker w = WalkRuns(p, d);
        uint32_t off, len;
        uint8_t *addr;
        bool starts_row;
        if (!d.aligned) {
            // Misaligned pool base: the warp moves the chunk byte by byte, bypassing the ring.
            for (uint32_t j = 0; j < w.n_runs; ++j) {
                GetRun(p, d, w, j, &off, &addr, &len, &starts_row);
                if (addr == nullptr) {
                    if (lane == 0 && starts_row) ReportSkip(p, d.block, 1u);
                    continue;
                }
                for (uint32_t i = lane; i < len; i += 32) {
                    if (kGather) {
                        d.stage[off + i] = addr[i];
                    } else {
                        addr[i] = d.stage[off + i];
                    }
                }
            }
            if (lane == 0) MbarArriveExpectTx(bar, 0);
            direct_mask |= 1u << s;
            return;
        }
        if (kGather) {
            uint32_t total = 0;
            for (uint32_t j = lane; j < w.n_runs; j += 32) {
                GetRun(p, d, w, j, &off, &addr, &len, &starts_row);
                if (addr != nullptr) {
                    total += len;
                } else if (starts_row) {
                    ReportSkip(p, d.block, 1u);
                }
            }
#pragma unroll
            for (int delta = 16; delta > 0; delta >>= 1) total += __shfl_xor_sync(0xffffffffu, total, delta);
            if (lane == 0) MbarArriveExpectTx(bar, total);
            __syncwarp();
            for (uint32_t j = lane; j < w.n_runs; j += 32) {
                GetRun(p, d, w, j, &off, &addr, &len, &starts_row);
                if (addr != nullptr) BulkLoad(buf + off, addr, len, bar);
            }
        } else if (lane == 0) {
            MbarArriveExpectTx(bar, d.len);
            BulkLoad(buf, d.stage, d.len, bar);
        }
    };

    // Drains stage k % n_stages: one bulk store per run, spread over the lanes.  Bulk groups are
    // per thread, so every lane commits one group per chunk (empty for lanes without a run).
    auto store = [&](uint32_t k) {
        const uint32_t s = k % n_stages;
        if (((direct_mask >> s) & 1u) == 0) {
            const uint32_t buf = ring_base + s * p.chunk_bytes;
            const ChunkDesc d = Describe(p, blockIdx.x + k * gridDim.x);
            const RunWalker w = WalkRuns(p, d);
            for (uint32_t j = lane; j < w.n_runs; j += 32) {
                uint32_t off, len;
                uint8_t *addr;
                bool starts_row;
                GetRun(p, d, w, j, &off, &addr, &len, &starts_row);
                if (addr != nullptr) {
                    BulkStore(kGather ? d.stage + off : addr, buf + off, len);
                } else if (!kGather && starts_row) {
                    ReportSkip(p, d.block, 1u);
                }
            }
        }
        BulkCommit();
    };

    const uint32_t ahead = n_stages - 1;
    for (uint32_t k = 0; k < ahead && k < n_my; ++k) load(k);
    bool failed = false;
    uint32_t fail_k = 0;
    for (uint32_t k = 0; k < n_my; ++k) {
        const uint32_t s = k % n_stages;
        if (lane == 0) failed = !BoundedWait(SmemAddr(&bars[s]), (k / n_stages) & 1u);
        failed = __shfl_sync(0xffffffffu, failed ? 1 : 0, 0) != 0;
        __syncwarp();  // the lanes that store out of the stage are ordered after the poll that saw it filled
        if (failed) {
            fail_k = k;
            break;
        }
        store(k);
        if (k + ahead < n_my) {
            // The stage about to be refilled was drained by the stores of chunk k-1: every lane
            // lets all of its bulk groups but the newest finish reading shared memory first.
            BulkWaitRead<1>();
            __syncwarp();
            load(k + ahead);
        }
    }
    if (failed && lane == 0) {
        // Leave no copy in flight behind: the loads of the chunk that was waited for and of the chunks fetched
        // ahead may still be writing this CTA's shared memory; one more bounded wait for each of them.
        for (uint32_t k = fail_k; k < n_my && k < fail_k + n_stages - 1; ++k) {
            BoundedWait(SmemAddr(&bars[k % n_stages]), (k / n_stages) & 1u);
        }
    }
    BulkWaitAll();
    if (lane == 0 && failed && p.status != nullptr) atomicExch(&p.status[2], 1u);
}

// 0 = plain 16-byte loads/stores, 1 = bulk-copy ring.  KVCM_B200_MOVER=ldg|bulk overrides the default;
// KVCM_B200_MOVER_HINT=0|1|2 picks the cache policy of the plain mover.
struct MoverConfig {
    int mover = 1;
    int hint = 0;
    uint32_t bulk_min_row_bytes = kBulkMinRowBytes;  // shorter rows use the vector kernel
    // Ring geometry; chunk 0 = choose from the shape (see BulkGeometryFor).
    int bulk_stages = 2;
    int bulk_ctas_per_sm = 3;
    uint32_t bulk_chunk_bytes = 0;
};

struct BulkGeometry {
    int stages;
    int ctas_per_sm;
    uint32_t chunk_bytes;
};

// Ring geometry from the shape, from sweeps on B200 (2 stages throughout; what matters is ~192 KiB
// in flight per SM, enough CTAs to issue the copies of short rows in parallel, and chunks that split
// a tile evenly, because chunk ids are dealt round-robin and a short tail chunk always lands on the
// same CTAs):
//   rows < 2 KiB (token rows)                       -> 16 KiB chunks, 6 CTAs per SM
//   rows >= 8 KiB in tiles >= 96 KiB (Llama-8B pages) -> 48 KiB chunks, 2 CTAs per SM
//   otherwise                                        -> tile split into equal chunks <= 32 KiB, 3 CTAs per SM
BulkGeometry BulkGeometryFor(const MoverConfig &cfg, int64_t tile_bytes, int64_t row_bytes) {
    if (cfg.bulk_chunk_bytes != 0) return {cfg.bulk_stages, cfg.bulk_ctas_per_sm, cfg.bulk_chunk_bytes};
    if (row_bytes < 2048) return {2, 6, 16 * 1024};
    if (row_bytes >= 8192 && tile_bytes >= 96 * 1024) return {2, 2, 48 * 1024};
    const int64_t n = (tile_bytes + 32 * 1024 - 1) / (32 * 1024);
    int64_t chunk = (tile_bytes + n - 1) / n;
    chunk = (chunk + 1023) / 1024 * 1024;
    return {2, 3, static_cast<uint32_t>(chunk)};
}

MoverConfig &GetMoverConfig() {
    static MoverConfig cfg = [] {
        MoverConfig c;
        if (const char *m = getenv("KVCM_B200_MOVER")) {
            if (strcmp(m, "ldg") == 0) c.mover = 0;
            if (strcmp(m, "bulk") == 0) c.mover = 1;
        }
        if (const char *h = getenv("KVCM_B200_MOVER_HINT")) {
            if (h[0] >= '0' && h[0] <= '2') c.hint = h[0] - '0';
        }
        return c;
    }();
    return cfg;
}

template <bool kGather, int kHint>
int ResidentCtas() {
    static int cached = 0;
    if (cached == 0) {
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, MoveRowsKernel<kGather, kHint>, kThreads, 0) !=
                cudaSuccess ||
            per_sm < 1) {
            cudaGetLastError();
            per_sm = 1;
        }
        cached = per_sm * GetDeviceInfo().sm_count;
    }
    return cached;
}

// Number of SMs a launch may occupy.  0 = the library's choice: every SM when staging is device
// memory (the transfer is HBM-bound), kHostStagingSms when staging is host memory - the transfer
// is then bound by the PCIe link, a few SMs saturate it, and the rest stay free for the engine's
// own kernels and for a transfer in the other direction.
constexpr int kHostStagingSms = 16;

// Returns 0 when `staging` is plain pageable host memory, which a kernel cannot address.
int SmBudget(int32_t max_sms, const void *staging) {
    const int all = GetDeviceInfo().sm_count;
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, staging) != cudaSuccess) {
        cudaGetLastError();
        return max_sms > 0 && max_sms < all ? max_sms : all;
    }
    if (attr.type == cudaMemoryTypeUnregistered) return 0;
    if (max_sms > 0) return max_sms < all ? max_sms : all;
    if (attr.type == cudaMemoryTypeHost) return kHostStagingSms < all ? kHostStagingSms : all;
    return all;
}

template <bool kGather, int kHint>
void LaunchPlain(const MoveParams &p, int sms, cudaStream_t stream) {
    const int64_t resident = static_cast<int64_t>(ResidentCtas<kGather, kHint>()) / GetDeviceInfo().sm_count * sms;
    const unsigned grid = static_cast<unsigned>(p.total_chunks < resident ? p.total_chunks : resident);
    MoveRowsKernel<kGather, kHint><<<grid, kThreads, 0, stream>>>(p);
}

constexpr int kBulkMaxSmem = 224 * 1024;

template <bool kGather>
void LaunchBulk(const MoveParams &p, int ctas_per_sm, int sms, cudaStream_t stream) {
    EnsureDynamicSmem(MoveRowsBulkKernel<kGather>, kBulkMaxSmem);
    const int smem = p.stages * static_cast<int>(p.chunk_bytes);
    const int64_t resident = static_cast<int64_t>(sms) * ctas_per_sm;
    const unsigned grid = static_cast<unsigned>(p.total_chunks < resident ? p.total_chunks : resident);
    MoveRowsBulkKernel<kGather><<<grid, 32, smem, stream>>>(p);
}

int32_t LaunchMove(bool gather, const void *const *d_ptrs, int32_t n_ptrs, int32_t sub_per_ptr, int64_t sub_stride,
                   void *staging, int64_t n_slots, const int32_t *d_row_idx, const int32_t *d_slot_idx,
                   int32_t n_blocks, int32_t rows_per_block, int64_t row_bytes, int64_t pool_rows, uint32_t *d_status,
                   bool report_skips, int32_t max_sms, kvcm_stream_t stream) {
    if (!HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (max_sms < 0) return KVCM_ER_INVALID_PARAMS;
    if (n_blocks < 0 || n_ptrs <= 0 || rows_per_block <= 0 || row_bytes <= 0 || pool_rows < 0 || n_slots < 0) {
        return KVCM_ER_INVALID_PARAMS;
    }
    if (n_blocks == 0) return KVCM_OK;
    if (d_ptrs == nullptr || staging == nullptr || d_row_idx == nullptr) return KVCM_ER_INVALID_ADDRESS;
    const int64_t tile_bytes = static_cast<int64_t>(rows_per_block) * row_bytes;
    const int64_t n_pools = static_cast<int64_t>(n_ptrs) * sub_per_ptr;
    if (tile_bytes >= (1ll << 31) || n_pools >= (1ll << 31)) return KVCM_ER_INVALID_PARAMS;
    const MoverConfig &cfg = GetMoverConfig();
    // The bulk ring needs 16-byte granularity everywhere and rows long enough to amortise one
    // copy instruction each; the sub-pool stride of the legacy layout must keep that alignment.
    const bool bulk_ok = cfg.mover == 1 && row_bytes % 16 == 0 && row_bytes >= cfg.bulk_min_row_bytes &&
                         (reinterpret_cast<uintptr_t>(staging) & 15u) == 0 && sub_stride % 16 == 0;
    const BulkGeometry geo = BulkGeometryFor(cfg, tile_bytes, row_bytes);
    const int64_t chunk_bytes = bulk_ok ? geo.chunk_bytes : kChunkBytes;
    const int64_t chunks_per_tile = (tile_bytes + chunk_bytes - 1) / chunk_bytes;
    const int64_t total_chunks = chunks_per_tile * n_pools * n_blocks;
    if (total_chunks >= (1ll << 32) - (1ll << 20)) return KVCM_ER_INVALID_PARAMS;

    MoveParams p;
    p.pool_ptrs = reinterpret_cast<const uint64_t *>(d_ptrs);
    p.staging = static_cast<uint8_t *>(staging);
    p.row_idx = d_row_idx;
    p.slot_idx = d_slot_idx;
    p.status = d_status;
    p.n_slots = n_slots;
    p.pool_rows = pool_rows;
    p.sub_stride = sub_stride;
    p.slot_bytes = n_pools * tile_bytes;
    p.row_bytes = static_cast<uint32_t>(row_bytes);
    p.tile_bytes = static_cast<uint32_t>(tile_bytes);
    p.chunks_per_tile = static_cast<uint32_t>(chunks_per_tile);
    p.total_chunks = static_cast<uint32_t>(total_chunks);
    p.n_pools = static_cast<int32_t>(n_pools);
    p.sub_per_ptr = sub_per_ptr;
    p.rows_per_block = rows_per_block;
    p.report_skips = report_skips ? 1 : 0;
    p.chunk_bytes = static_cast<uint32_t>(chunk_bytes);
    p.stages = geo.stages;

    cudaStream_t s = AsStream(stream);
    const int sms = SmBudget(max_sms, staging);
    if (sms == 0) return KVCM_ER_UNSUPPORTED_MEMORY_TYPE;  // pageable host memory: pin it or use save/load_rows
    if (bulk_ok) {
        if (gather) {
            LaunchBulk<true>(p, geo.ctas_per_sm, sms, s);
        } else {
            LaunchBulk<false>(p, geo.ctas_per_sm, sms, s);
        }
    } else if (cfg.hint == 0) {
        gather ? LaunchPlain<true, 0>(p, sms, s) : LaunchPlain<false, 0>(p, sms, s);
    } else if (cfg.hint == 2) {
        gather ? LaunchPlain<true, 2>(p, sms, s) : LaunchPlain<false, 2>(p, sms, s);
    } else {
        gather ? LaunchPlain<true, 1>(p, sms, s) : LaunchPlain<false, 1>(p, sms, s);
    }
    return LaunchStatus();
}

}  // namespace
}  // namespace kvcm

extern "C" {

int32_t kvcm_b200_set_mover(int32_t mover, int32_t cache_hint) {
    if (mover > 1 || cache_hint > 2) return KVCM_ER_INVALID_PARAMS;
    kvcm::MoverConfig &cfg = kvcm::GetMoverConfig();
    if (mover >= 0) cfg.mover = mover;
    if (cache_hint >= 0) cfg.hint = cache_hint;
    return KVCM_OK;
}

int32_t kvcm_b200_set_bulk_min_row_bytes(int32_t row_bytes) {
    if (row_bytes < 16 || row_bytes % 16 != 0) return KVCM_ER_INVALID_PARAMS;
    kvcm::GetMoverConfig().bulk_min_row_bytes = static_cast<uint32_t>(row_bytes);
    return KVCM_OK;
}

int32_t kvcm_b200_set_bulk_geometry(int32_t stages, int32_t ctas_per_sm, int32_t chunk_bytes) {
    if (stages == 0 && ctas_per_sm == 0 && chunk_bytes == 0) {
        kvcm::GetMoverConfig().bulk_chunk_bytes = 0;  // back to the shape-driven choice
        return KVCM_OK;
    }
    if (stages < 2 || stages > kvcm::kBulkMaxStages || ctas_per_sm < 1 || ctas_per_sm > 8 || chunk_bytes < 1024 ||
        chunk_bytes % 1024 != 0 ||
        static_cast<int64_t>(stages) * chunk_bytes * ctas_per_sm > kvcm::kBulkMaxSmem) {
        return KVCM_ER_INVALID_PARAMS;
    }
    kvcm::MoverConfig &cfg = kvcm::GetMoverConfig();
    cfg.bulk_stages = stages;
    cfg.bulk_ctas_per_sm = ctas_per_sm;
    cfg.bulk_chunk_bytes = static_cast<uint32_t>(chunk_bytes);
    return KVCM_OK;
}

int32_t kvcm_b200_gather_tokens(const void *const *d_pool_ptrs, int32_t n_pools, void *staging, int64_t n_slots,
                                const int32_t *d_token_idx, const int32_t *d_slot_idx, int32_t n_blocks,
                                int32_t tokens_per_block, int64_t bytes_per_token, int64_t pool_tokens,
                                uint32_t *d_status, int32_t max_sms, kvcm_stream_t stream) {
    return kvcm::LaunchMove(true, d_pool_ptrs, n_pools, 1, 0, staging, n_slots, d_token_idx, d_slot_idx, n_blocks,
                            tokens_per_block, bytes_per_token, pool_tokens, d_status, true, max_sms, stream);
}

int32_t kvcm_b200_scatter_tokens(const void *const *d_pool_ptrs, int32_t n_pools, const void *staging, int64_t n_slots,
                                 const int32_t *d_token_idx, const int32_t *d_slot_idx, int32_t n_blocks,
                                 int32_t tokens_per_block, int64_t bytes_per_token, int64_t pool_tokens,
                                 uint32_t *d_status, int32_t max_sms, kvcm_stream_t stream) {
    return kvcm::LaunchMove(false, d_pool_ptrs, n_pools, 1, 0, const_cast<void *>(staging), n_slots, d_token_idx,
                            d_slot_idx, n_blocks, tokens_per_block, bytes_per_token, pool_tokens, d_status, true,
                            max_sms, stream);
}

int32_t kvcm_b200_gather_pages(const void *const *d_pool_ptrs, int32_t n_pools, void *staging, int64_t n_slots,
                               const int32_t *d_page_table, const int32_t *d_slot_idx, int32_t n_blocks,
                               int32_t pages_per_block, int64_t page_bytes, int64_t pool_pages, uint32_t *d_status, int32_t max_sms, kvcm_stream_t stream) {
    return kvcm::LaunchMove(true, d_pool_ptrs, n_pools, 1, 0, staging, n_slots, d_page_table, d_slot_idx, n_blocks,
                            pages_per_block, page_bytes, pool_pages, d_status, true, max_sms, stream);
}

int32_t kvcm_b200_scatter_pages(const void *const *d_pool_ptrs, int32_t n_pools, const void *staging, int64_t n_slots,
                                const int32_t *d_page_table, const int32_t *d_slot_idx, int32_t n_blocks,
                                int32_t pages_per_block, int64_t page_bytes, int64_t pool_pages, uint32_t *d_status, int32_t max_sms, kvcm_stream_t stream) {
    return kvcm::LaunchMove(false, d_pool_ptrs, n_pools, 1, 0, const_cast<void *>(staging), n_slots, d_page_table,
                            d_slot_idx, n_blocks, pages_per_block, page_bytes, pool_pages, d_status, true, max_sms, stream);
}

// Legacy form: one block, layer tensors [2, total_tokens, hidden]; the K and V halves of a
// layer are two sub-pools total_tokens * hidden_bytes apart behind one pointer, and the
// staging order [layer][kv][token] is the tile order pool = layer * 2 + kv.
int32_t kvcm_b200_gather_legacy(const void *const *d_layer_ptrs, int32_t n_layers, int64_t total_tokens, void *staging,
                                const int32_t *d_token_idx, int32_t n_tokens, int64_t hidden_bytes,
                                kvcm_stream_t stream) {
    if (n_tokens == 0) return KVCM_OK;
    return kvcm::LaunchMove(true, d_layer_ptrs, n_layers, 2, total_tokens * hidden_bytes, staging, 1, d_token_idx,
                            nullptr, 1, n_tokens, hidden_bytes, total_tokens, nullptr, false, 0, stream);
}

int32_t kvcm_b200_scatter_legacy(const void *const *d_layer_ptrs, int32_t n_layers, int64_t total_tokens,
                                 const void *staging, const int32_t *d_token_idx, int32_t n_tokens,
                                 int64_t hidden_bytes, kvcm_stream_t stream) {
    if (n_tokens == 0) return KVCM_OK;
    return kvcm::LaunchMove(false, d_layer_ptrs, n_layers, 2, total_tokens * hidden_bytes,
                            const_cast<void *>(staging), 1, d_token_idx, nullptr, 1, n_tokens, hidden_bytes,
                            total_tokens, nullptr, false, 0, stream);
}

// Save / load with staging in HOST memory, the PCIe leg done by the copy engines.
//
// SM-issued loads and stores over PCIe saturate one direction (about 52 GB/s on a Gen5 x16 link)
// but a save and a load running at once reach only ~35 GB/s each; the DMA engines sustain ~50 GB/s
// each way at the same time.  So blocks are gathered into a device bounce buffer at HBM speed and
// leave through cudaMemcpyAsync (save), or arrive through cudaMemcpyAsync and are scattered (load).
//
// The bounce buffer is used as two halves and the copies run on a copy stream of the library's own
// (one per device and direction), tied to the caller's stream by events: while the copy engine moves
// the blocks of one half across PCIe, the kernel fills (or empties) the other half, so neither the
// link nor the caller's stream idles between groups.  To the caller everything is still ordered on
// `stream`: the first copy waits for the work that precedes the call, and the stream waits for the
// last copy before the call's successors run.
namespace {

struct CopyLane {
    cudaStream_t copy = nullptr;
    cudaEvent_t entry = nullptr;      // recorded on the caller's stream when a load begins
    cudaEvent_t filled[2] = {};       // save: half gathered (caller's stream); load: half arrived (copy stream)
    cudaEvent_t drained[2] = {};      // save: half copied out (copy stream); load: half scattered (caller's stream)
    std::mutex mu;                    // one call at a time enqueues on a lane: the events are shared
    bool ok = false;
};

// Lane of the current device for one direction (0 = save, 1 = load), created at first use.
CopyLane *GetCopyLane(int direction) {
    static std::mutex mu;
    static std::vector<CopyLane *> lanes;  // [device * 2 + direction]; never freed: they live as long as the library
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(mu);
    const size_t slot = static_cast<size_t>(device) * 2 + direction;
    if (lanes.size() <= slot) lanes.resize(slot + 1, nullptr);
    if (lanes[slot] == nullptr) {
        CopyLane *lane = new CopyLane;
        bool ok = cudaStreamCreateWithFlags(&lane->copy, cudaStreamNonBlocking) == cudaSuccess;
        ok = ok && cudaEventCreateWithFlags(&lane->entry, cudaEventDisableTiming) == cudaSuccess;
        for (int h = 0; h < 2; ++h) {
            ok = ok && cudaEventCreateWithFlags(&lane->filled[h], cudaEventDisableTiming) == cudaSuccess;
            ok = ok && cudaEventCreateWithFlags(&lane->drained[h], cudaEventDisableTiming) == cudaSuccess;
        }
        if (!ok) cudaGetLastError();
        lane->ok = ok;
        lanes[slot] = lane;
    }
    return lanes[slot]->ok ? lanes[slot] : nullptr;
}

// One cudaMemcpyAsync per run of blocks whose host slots are consecutive.
int32_t CopyGroup(bool save, uint8_t *host, uint8_t *bounce, const int32_t *h_slot_idx, int64_t first, int32_t n,
                  int64_t n_slots, int64_t block_bytes, cudaStream_t copy) {
    for (int32_t i = 0; i < n;) {
        const int64_t slot = h_slot_idx != nullptr ? h_slot_idx[first + i] : first + i;
        if (slot < 0 || slot >= n_slots) return KVCM_ER_INVALID_PARAMS;
        int32_t j = i + 1;
        while (j < n && (h_slot_idx != nullptr ? h_slot_idx[first + j] : first + j) == slot + (j - i)) ++j;
        if (slot + (j - i) > n_slots) return KVCM_ER_INVALID_PARAMS;
        const size_t bytes = static_cast<size_t>(j - i) * block_bytes;
        const cudaError_t e = save ? cudaMemcpyAsync(host + slot * block_bytes, bounce + i * block_bytes, bytes,
                                                     cudaMemcpyDeviceToHost, copy)
                                   : cudaMemcpyAsync(bounce + i * block_bytes, host + slot * block_bytes, bytes,
                                                     cudaMemcpyHostToDevice, copy);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return KVCM_ER_CUDAMEMCPY_ERROR;
        }
        i = j;
    }
    return KVCM_OK;
}

inline bool Ok(cudaError_t e) {
    if (e == cudaSuccess) return true;
    cudaGetLastError();
    return false;
}

}  // namespace

static int32_t MoveRowsThroughBounce(bool save, const void *const *d_pool_ptrs, int32_t n_pools, void *h_staging,
                                     int64_t n_slots, const int32_t *d_row_idx, const int32_t *h_slot_idx,
                                     int32_t n_blocks, int32_t rows_per_block, int64_t row_bytes, int64_t pool_rows,
                                     void *d_bounce, int64_t bounce_bytes, uint32_t *d_status, kvcm_stream_t stream) {
    if (!kvcm::HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (n_blocks < 0 || n_pools <= 0 || rows_per_block <= 0 || row_bytes <= 0 || n_slots < 0) {
        return KVCM_ER_INVALID_PARAMS;
    }
    if (n_blocks == 0) return KVCM_OK;
    if (h_staging == nullptr || d_bounce == nullptr || d_row_idx == nullptr) return KVCM_ER_INVALID_ADDRESS;
    const int64_t block_bytes = static_cast<int64_t>(n_pools) * rows_per_block * row_bytes;
    if (bounce_bytes / block_bytes < 1) return KVCM_ER_INVALID_PARAMS;
    if (h_slot_idx != nullptr) {  // refuse a bad slot before anything is launched or copied
        for (int32_t b = 0; b < n_blocks; ++b) {
            if (h_slot_idx[b] < 0 || h_slot_idx[b] >= n_slots) return KVCM_ER_INVALID_PARAMS;
        }
    } else if (n_blocks > n_slots) {
        return KVCM_ER_INVALID_PARAMS;
    }
    cudaStream_t s = kvcm::AsStream(stream);
    uint8_t *host = static_cast<uint8_t *>(h_staging);
    uint8_t *bounce = static_cast<uint8_t *>(d_bounce);

    // Two halves when each holds at least one block and there is more than one block to move; the second half
    // starts on a 256-byte boundary.  Otherwise (a bounce buffer of one block) the groups run back to back on
    // the caller's stream.
    const int64_t half_bytes = (bounce_bytes / 2) & ~int64_t{255};
    CopyLane *lane = (n_blocks > 1 && half_bytes >= block_bytes) ? GetCopyLane(save ? 0 : 1) : nullptr;
    if (lane == nullptr) {
        const int64_t group = bounce_bytes / block_bytes;
        for (int64_t first = 0; first < n_blocks; first += group) {
            const int32_t n = static_cast<int32_t>(first + group <= n_blocks ? group : n_blocks - first);
            const int32_t *rows = d_row_idx + first * rows_per_block;
            int32_t rc = KVCM_OK;
            if (save) {
                rc = kvcm::LaunchMove(true, d_pool_ptrs, n_pools, 1, 0, bounce, n, rows, nullptr, n, rows_per_block,
                                      row_bytes, pool_rows, d_status, true, 0, stream);
            }
            if (rc == KVCM_OK) rc = CopyGroup(save, host, bounce, h_slot_idx, first, n, n_slots, block_bytes, s);
            if (rc == KVCM_OK && !save) {
                rc = kvcm::LaunchMove(false, d_pool_ptrs, n_pools, 1, 0, bounce, n, rows, nullptr, n, rows_per_block,
                                      row_bytes, pool_rows, d_status, true, 0, stream);
            }
            if (rc != KVCM_OK) return rc;
        }
        return KVCM_OK;
    }

    std::lock_guard<std::mutex> lock(lane->mu);
    // No more blocks per group than needed to cut the transfer in two: a short transfer is pipelined too.
    int64_t group = half_bytes / block_bytes;
    if (group > (n_blocks + 1) / 2) group = (n_blocks + 1) / 2;
    if (!save && !Ok(cudaEventRecord(lane->entry, s))) return KVCM_ER_CUDAMEMCPY_ERROR;
    int32_t rc = KVCM_OK;
    bool used[2] = {false, false};
    int64_t k = 0;
    for (int64_t first = 0; first < n_blocks && rc == KVCM_OK; first += group, ++k) {
        const int h = static_cast<int>(k & 1);
        const int32_t n = static_cast<int32_t>(first + group <= n_blocks ? group : n_blocks - first);
        const int32_t *rows = d_row_idx + first * rows_per_block;
        uint8_t *half = bounce + h * half_bytes;
        bool ok = true;
        if (save) {
            // the kernel may refill a half once the copy engine has emptied it (an event that was never
            // recorded counts as complete)
            ok = Ok(cudaStreamWaitEvent(s, lane->drained[h], 0));
            if (ok) {
                rc = kvcm::LaunchMove(true, d_pool_ptrs, n_pools, 1, 0, half, n, rows, nullptr, n, rows_per_block,
                                      row_bytes, pool_rows, d_status, true, 0, stream);
                if (rc != KVCM_OK) break;
            }
            ok = ok && Ok(cudaEventRecord(lane->filled[h], s)) && Ok(cudaStreamWaitEvent(lane->copy, lane->filled[h], 0));
            if (ok) rc = CopyGroup(true, host, half, h_slot_idx, first, n, n_slots, block_bytes, lane->copy);
            ok = ok && Ok(cudaEventRecord(lane->drained[h], lane->copy));
        } else {
            // the copy engine may refill a half once the kernel has scattered it; the first copies wait for
            // whatever precedes this call on the caller's stream
            ok = Ok(cudaStreamWaitEvent(lane->copy, k < 2 ? lane->entry : lane->drained[h], 0));
            if (ok) rc = CopyGroup(false, host, half, h_slot_idx, first, n, n_slots, block_bytes, lane->copy);
            ok = ok && Ok(cudaEventRecord(lane->filled[h], lane->copy)) && Ok(cudaStreamWaitEvent(s, lane->filled[h], 0));
            if (ok && rc == KVCM_OK) {
                rc = kvcm::LaunchMove(false, d_pool_ptrs, n_pools, 1, 0, half, n, rows, nullptr, n, rows_per_block,
                                      row_bytes, pool_rows, d_status, true, 0, stream);
            }
            ok = ok && Ok(cudaEventRecord(lane->drained[h], s));
        }
        used[h] = true;
        if (!ok && rc == KVCM_OK) rc = KVCM_ER_CUDAMEMCPY_ERROR;
    }
    // Whatever was enqueued on the copy stream is joined back into the caller's stream, on the error paths too.
    if (save) {
        for (int h = 0; h < 2; ++h) {
            if (used[h] && !Ok(cudaStreamWaitEvent(s, lane->drained[h], 0)) && rc == KVCM_OK) rc = KVCM_ER_CUDAMEMCPY_ERROR;
        }
    } else {
        for (int h = 0; h < 2; ++h) {
            if (used[h] && !Ok(cudaStreamWaitEvent(s, lane->filled[h], 0)) && rc == KVCM_OK) rc = KVCM_ER_CUDAMEMCPY_ERROR;
        }
    }
    return rc;
}

int32_t kvcm_b200_save_rows_to_host(const void *const *d_pool_ptrs, int32_t n_pools, void *h_staging, int64_t n_slots,
                                    const int32_t *d_row_idx, const int32_t *h_slot_idx, int32_t n_blocks,
                                    int32_t rows_per_block, int64_t row_bytes, int64_t pool_rows, void *d_bounce,
                                    int64_t bounce_bytes, uint32_t *d_status, kvcm_stream_t stream) {
    return MoveRowsThroughBounce(true, d_pool_ptrs, n_pools, h_staging, n_slots, d_row_idx, h_slot_idx, n_blocks,
                                 rows_per_block, row_bytes, pool_rows, d_bounce, bounce_bytes, d_status, stream);
}

int32_t kvcm_b200_load_rows_from_host(const void *const *d_pool_ptrs, int32_t n_pools, const void *h_staging,
                                      int64_t n_slots, const int32_t *d_row_idx, const int32_t *h_slot_idx,
                                      int32_t n_blocks, int32_t rows_per_block, int64_t row_bytes, int64_t pool_rows,
                                      void *d_bounce, int64_t bounce_bytes, uint32_t *d_status,
                                      kvcm_stream_t stream) {
    return MoveRowsThroughBounce(false, d_pool_ptrs, n_pools, const_cast<void *>(h_staging), n_slots, d_row_idx,
                                 h_slot_idx, n_blocks, rows_per_block, row_bytes, pool_rows, d_bounce, bounce_bytes,
                                 d_status, stream);
}

}  // extern "C"
