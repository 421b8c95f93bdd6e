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
#include "kvcm_common.cuh"

namespace kvcm {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 8;
constexpr uint32_t kVecBytes = 16;
constexpr uint32_t kChunkBytes = kThreads * kVecBytes * kUnroll;  // 32 KiB

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
};

__device__ __forceinline__ void ReportSkip(const MoveParams &p, uint32_t block, uint32_t count) {
    if (p.report_skips && p.status != nullptr) {
        atomicAdd(&p.status[0], count);
        atomicMax(&p.status[1], block + 1u);
    }
}

// kGather: pool -> staging.  !kGather: staging -> pool.
template <bool kGather>
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
                    if (in_pool[j] != nullptr) v[j] = __ldcs(reinterpret_cast<const uint4 *>(in_pool[j]));
                }
#pragma unroll
                for (int j = 0; j < kUnroll; ++j) {
                    if (in_pool[j] != nullptr) __stcs(reinterpret_cast<uint4 *>(stage + off[j]), v[j]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < kUnroll; ++j) {
                    if (in_pool[j] != nullptr) v[j] = __ldcs(reinterpret_cast<const uint4 *>(stage + off[j]));
                }
#pragma unroll
                for (int j = 0; j < kUnroll; ++j) {
                    if (in_pool[j] != nullptr) __stcs(reinterpret_cast<uint4 *>(in_pool[j]), v[j]);
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

int ResidentCtas(bool gather) {
    static int cached[2] = {0, 0};
    int &slot = cached[gather ? 0 : 1];
    if (slot == 0) {
        int per_sm = 0;
        cudaError_t e = gather ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, MoveRowsKernel<true>, kThreads, 0)
                               : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, MoveRowsKernel<false>, kThreads, 0);
        if (e != cudaSuccess || per_sm < 1) per_sm = 1;
        slot = per_sm * GetDeviceInfo().sm_count;
    }
    return slot;
}

int32_t LaunchMove(bool gather, const void *const *d_ptrs, int32_t n_ptrs, int32_t sub_per_ptr, int64_t sub_stride,
                   void *staging, int64_t n_slots, const int32_t *d_row_idx, const int32_t *d_slot_idx,
                   int32_t n_blocks, int32_t rows_per_block, int64_t row_bytes, int64_t pool_rows, uint32_t *d_status,
                   bool report_skips, kvcm_stream_t stream) {
    if (!HaveDevice()) return KVCM_ER_NO_DEVICE;
    if (n_blocks < 0 || n_ptrs <= 0 || rows_per_block <= 0 || row_bytes <= 0 || pool_rows < 0 || n_slots < 0) {
        return KVCM_ER_INVALID_PARAMS;
    }
    if (n_blocks == 0) return KVCM_OK;
    if (d_ptrs == nullptr || staging == nullptr || d_row_idx == nullptr) return KVCM_ER_INVALID_ADDRESS;
    const int64_t tile_bytes = static_cast<int64_t>(rows_per_block) * row_bytes;
    const int64_t n_pools = static_cast<int64_t>(n_ptrs) * sub_per_ptr;
    if (tile_bytes >= (1ll << 31) || n_pools >= (1ll << 31)) return KVCM_ER_INVALID_PARAMS;
    const int64_t chunks_per_tile = (tile_bytes + kChunkBytes - 1) / kChunkBytes;
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

    const int64_t resident = ResidentCtas(gather);
    const unsigned grid = static_cast<unsigned>(total_chunks < resident ? total_chunks : resident);
    if (gather) {
        MoveRowsKernel<true><<<grid, kThreads, 0, AsStream(stream)>>>(p);
    } else {
        MoveRowsKernel<false><<<grid, kThreads, 0, AsStream(stream)>>>(p);
    }
    return LaunchStatus();
}

}  // namespace
}  // namespace kvcm

extern "C" {

int32_t kvcm_b200_gather_tokens(const void *const *d_pool_ptrs, int32_t n_pools, void *staging, int64_t n_slots,
                                const int32_t *d_token_idx, const int32_t *d_slot_idx, int32_t n_blocks,
                                int32_t tokens_per_block, int64_t bytes_per_token, int64_t pool_tokens,
                                uint32_t *d_status, kvcm_stream_t stream) {
    return kvcm::LaunchMove(true, d_pool_ptrs, n_pools, 1, 0, staging, n_slots, d_token_idx, d_slot_idx, n_blocks,
                            tokens_per_block, bytes_per_token, pool_tokens, d_status, true, stream);
}

int32_t kvcm_b200_scatter_tokens(const void *const *d_pool_ptrs, int32_t n_pools, const void *staging, int64_t n_slots,
                                 const int32_t *d_token_idx, const int32_t *d_slot_idx, int32_t n_blocks,
                                 int32_t tokens_per_block, int64_t bytes_per_token, int64_t pool_tokens,
                                 uint32_t *d_status, kvcm_stream_t stream) {
    return kvcm::LaunchMove(false, d_pool_ptrs, n_pools, 1, 0, const_cast<void *>(staging), n_slots, d_token_idx,
                            d_slot_idx, n_blocks, tokens_per_block, bytes_per_token, pool_tokens, d_status, true,
                            stream);
}

int32_t kvcm_b200_gather_pages(const void *const *d_pool_ptrs, int32_t n_pools, void *staging, int64_t n_slots,
                               const int32_t *d_page_table, const int32_t *d_slot_idx, int32_t n_blocks,
                               int32_t pages_per_block, int64_t page_bytes, int64_t pool_pages, uint32_t *d_status,
                               kvcm_stream_t stream) {
    return kvcm::LaunchMove(true, d_pool_ptrs, n_pools, 1, 0, staging, n_slots, d_page_table, d_slot_idx, n_blocks,
                            pages_per_block, page_bytes, pool_pages, d_status, true, stream);
}

int32_t kvcm_b200_scatter_pages(const void *const *d_pool_ptrs, int32_t n_pools, const void *staging, int64_t n_slots,
                                const int32_t *d_page_table, const int32_t *d_slot_idx, int32_t n_blocks,
                                int32_t pages_per_block, int64_t page_bytes, int64_t pool_pages, uint32_t *d_status,
                                kvcm_stream_t stream) {
    return kvcm::LaunchMove(false, d_pool_ptrs, n_pools, 1, 0, const_cast<void *>(staging), n_slots, d_page_table,
                            d_slot_idx, n_blocks, pages_per_block, page_bytes, pool_pages, d_status, true, stream);
}

// Legacy form: one block, layer tensors [2, total_tokens, hidden]; the K and V halves of a
// layer are two sub-pools total_tokens * hidden_bytes apart behind one pointer, and the
// staging order [layer][kv][token] is the tile order pool = layer * 2 + kv.
int32_t kvcm_b200_gather_legacy(const void *const *d_layer_ptrs, int32_t n_layers, int64_t total_tokens, void *staging,
                                const int32_t *d_token_idx, int32_t n_tokens, int64_t hidden_bytes,
                                kvcm_stream_t stream) {
    if (n_tokens == 0) return KVCM_OK;
    return kvcm::LaunchMove(true, d_layer_ptrs, n_layers, 2, total_tokens * hidden_bytes, staging, 1, d_token_idx,
                            nullptr, 1, n_tokens, hidden_bytes, total_tokens, nullptr, false, stream);
}

int32_t kvcm_b200_scatter_legacy(const void *const *d_layer_ptrs, int32_t n_layers, int64_t total_tokens,
                                 const void *staging, const int32_t *d_token_idx, int32_t n_tokens,
                                 int64_t hidden_bytes, kvcm_stream_t stream) {
    if (n_tokens == 0) return KVCM_OK;
    return kvcm::LaunchMove(false, d_layer_ptrs, n_layers, 2, total_tokens * hidden_bytes,
                            const_cast<void *>(staging), 1, d_token_idx, nullptr, 1, n_tokens, hidden_bytes,
                            total_tokens, nullptr, false, stream);
}

}  // extern "C"
