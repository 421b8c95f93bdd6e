/*
 * kvcm_b200.h - C ABI of libkvcm_b200.so, the sm_100a implementation of the Tair KVCache
 * Manager (KVCM) data-parallel hot path:
 *
 *   (1) paged-KV block gather / scatter between an engine's per-layer K/V page pools and the
 *       contiguous staging blocks that storage backends read and write;
 *   (2) chained 64-bit token-block hashing, a GPU-resident block index, and batched prefix /
 *       sliding-window / batch-get matching against it.
 *
 * Every entry point names the interface of alibaba/tair-kvcache it stands in for (file:line
 * relative to that project's root).  Conventions:
 *   - plain pointers and sizes only; pointers prefixed d_ are device addresses (staging buffers
 *     may also be pinned host memory reachable from the device);
 *   - every call is asynchronous on `stream` (a cudaStream_t passed as void*, NULL = default
 *     stream) unless its comment says it synchronises;
 *   - the int32 return value is 0 (KVCM_OK) or one of the codes below; nothing throws and
 *     nothing traps on the device.  Problems only the device can see (an index out of range,
 *     a full table) are skipped and counted in a caller-owned status word.
 *   - there is no CPU fallback: without a CUDA device every compute entry point returns
 *     KVCM_ER_NO_DEVICE.
 */
#ifndef KVCM_B200_H_
#define KVCM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define KVCM_API __attribute__((visibility("default")))
#else
#define KVCM_API
#endif

/* ------------------------------------------------------------------------------------------
 * Return codes.  Transfer-side values are numerically those of ClientErrorCode
 * (kv_cache_manager/client/include/common.h:11-63); manager-side values (index, match) are
 * those of ErrorCode (kv_cache_manager/common/error_code.h:6-28) offset by KVCM_EC_BASE so the
 * two families cannot collide in one int32.
 * ---------------------------------------------------------------------------------------- */
#define KVCM_OK 0
#define KVCM_ER_INVALID_PARAMS 3                    /* ER_INVALID_PARAMS */
#define KVCM_ER_INVALID_ADDRESS 107                 /* ER_INVALID_ADDRESS */
#define KVCM_ER_UNSUPPORTED_MEMORY_TYPE 109         /* ER_UNSUPPORTED_MEMORY_TYPE */
#define KVCM_ER_CUDAMEMCPY_ERROR 112                /* ER_CUDAMEMCPY_ERROR: a launch or copy failed */
#define KVCM_ER_CUDA_STREAM_SYNCHRONIZE_ERROR 115   /* ER_CUDA_STREAM_SYNCHRONIZE_ERROR */
#define KVCM_ER_NO_DEVICE 900                       /* no CUDA device / driver: there is no CPU path */
#define KVCM_EC_BASE 1000
#define KVCM_EC_ERROR (KVCM_EC_BASE + 1)            /* EC_ERROR */
#define KVCM_EC_NOENT (KVCM_EC_BASE + 2)            /* EC_NOENT */
#define KVCM_EC_EXIST (KVCM_EC_BASE + 4)            /* EC_EXIST: the key has a location of that class already */
#define KVCM_EC_BADARGS (KVCM_EC_BASE + 6)          /* EC_BADARGS */
#define KVCM_EC_NOSPC (KVCM_EC_BASE + 9)            /* EC_NOSPC: index full */
#define KVCM_EC_OUT_OF_LIMIT (KVCM_EC_BASE + 14)    /* EC_OUT_OF_LIMIT: size beyond a fixed limit */
#define KVCM_EC_MISMATCH (KVCM_EC_BASE + 16)        /* EC_MISMATCH: a compare-and-set found another status */

typedef void *kvcm_stream_t; /* cudaStream_t */

KVCM_API int32_t kvcm_b200_abi_version(void);
/* Binds the calling thread to CUDA device `device` for the calls that follow (one process drives
 * one GPU; a host that already selected its device through the CUDA runtime it shares with this
 * library need not call it).  Grid sizes come from the properties of the calling thread's current device,
 * which the library keeps per device. */
KVCM_API int32_t kvcm_b200_set_device(int32_t device);
KVCM_API const char *kvcm_b200_error_string(int32_t code);
/* Self test of the give-up path of the kernels' bounded waits.  Every kernel here that waits on an mbarrier
 * (the bulk-copy rings of gather / scatter, of the segment copy and of the hash) polls through one shared helper
 * and, when the poll limit runs out, raises an error word (status[2] of gather / scatter,
 * kvcm_b200_copy_wait_timeouts, kvcm_b200_hash_wait_timeouts), waits - bounded again - for the copies it still
 * has in flight and returns.  This entry point runs that helper once, in one warp, on a barrier armed for bytes
 * that are never sent (no copy is issued), with `poll_limit` polls (1..65536): the wait runs out by
 * construction, d_status[0] = 1 (gave up) and d_status[1] = poll_limit are written, and the kernel returns;
 * nothing faults, traps or hangs, and the context stays usable.  No counterpart in the reference. */
KVCM_API int32_t kvcm_b200_selftest_bounded_wait(uint32_t poll_limit, uint32_t *d_status, kvcm_stream_t stream);
/* Number of SMs and L2 bytes of the current device (synchronous, cached). */
KVCM_API int32_t kvcm_b200_device_info(int32_t *sm_count, int64_t *l2_bytes, int64_t *free_bytes,
                                       int64_t *total_bytes);

/* ------------------------------------------------------------------------------------------
 * (1) Gather / scatter of paged KV.
 *
 * Replaces the Triton kernels kv_cache_batch_gather_kernel / kv_cache_batch_scatter_kernel and
 * their wrappers batch_gather_kv_caches / batch_scatter_kv_caches
 * (kv_cache_manager/py_connector/kernel/batch_gather_scatter_helper.py:33-136, 139-248).
 *
 * A pool is one K or V tensor of one layer, row-major [pool_rows, row_bytes].  d_pool_ptrs is
 * the device array of n_pools pool base addresses (the reference's int64 `kv_caches_ptrs_tensor`,
 * order layer0.K, layer0.V, layer1.K, ...).  Block b owns rows_per_block rows
 * d_row_idx[b*rows_per_block + t] of every pool, and staging slot d_slot_idx[b] (NULL = slot b).
 * A staging slot is [n_pools, rows_per_block, row_bytes] contiguous bytes:
 *
 *   gather :  staging[slot][p][t][:] = pool_p[row_idx[b][t]][:]
 *   scatter:  pool_p[row_idx[b][t]][:] = staging[slot][p][t][:]
 *
 * "tokens" form: a row is one token (row_bytes = dim * itemsize) and d_row_idx is the reference's
 * flat block_token_indices.  "pages" form: a row is one engine page (row_bytes = page_tokens *
 * dim * itemsize) and d_row_idx is the engine's block table itself, which removes
 * generate_blocks_idx (kv_cache_manager/py_connector/vllm/v1_connector.py:308-320).  The byte
 * result is identical when the token indices of a block are whole pages.
 *
 * Rows outside [0, pool_rows) and slots outside [0, n_slots) are skipped, never dereferenced.
 * d_status, when not NULL, points to four caller-zeroed uint32 words: [0] is incremented once per
 * skipped (pool,row) pair, [1] keeps 1 + the largest offending block number, [2] becomes 1 if a
 * bounded wait inside the kernel ran out (the copy is then incomplete), [3] is reserved.
 * max_sms bounds the SMs the launch occupies - the role of the reference's `sm_count` argument
 * (batch_gather_scatter_helper.py:110,115).  0 = the library's choice: every SM when staging is device
 * memory, 16 when staging is host memory (the PCIe link is then the bound, and the other SMs stay free
 * for the engine and for a transfer in the opposite direction on another stream).
 * Staging in pageable (unpinned, unregistered) host memory is refused with
 * KVCM_ER_UNSUPPORTED_MEMORY_TYPE: pin or register it, or use the save / load entry points below.
 * Scattering the same row twice in one call is a data race, as in the reference.
 * Fastest when row_bytes and all base addresses are multiples of 16; any alignment is correct.
 * ---------------------------------------------------------------------------------------- */
KVCM_API int32_t kvcm_b200_gather_tokens(const void *const *d_pool_ptrs, int32_t n_pools, void *staging,
                                         int64_t n_slots, const int32_t *d_token_idx, const int32_t *d_slot_idx,
                                         int32_t n_blocks, int32_t tokens_per_block, int64_t bytes_per_token,
                                         int64_t pool_tokens, uint32_t *d_status, int32_t max_sms,
                                         kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_scatter_tokens(const void *const *d_pool_ptrs, int32_t n_pools, const void *staging,
                                          int64_t n_slots, const int32_t *d_token_idx, const int32_t *d_slot_idx,
                                          int32_t n_blocks, int32_t tokens_per_block, int64_t bytes_per_token,
                                          int64_t pool_tokens, uint32_t *d_status, int32_t max_sms,
                                         kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_gather_pages(const void *const *d_pool_ptrs, int32_t n_pools, void *staging,
                                        int64_t n_slots, const int32_t *d_page_table, const int32_t *d_slot_idx,
                                        int32_t n_blocks, int32_t pages_per_block, int64_t page_bytes,
                                        int64_t pool_pages, uint32_t *d_status, int32_t max_sms,
                                         kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_scatter_pages(const void *const *d_pool_ptrs, int32_t n_pools, const void *staging,
                                         int64_t n_slots, const int32_t *d_page_table, const int32_t *d_slot_idx,
                                         int32_t n_blocks, int32_t pages_per_block, int64_t page_bytes,
                                         int64_t pool_pages, uint32_t *d_status, int32_t max_sms,
                                         kvcm_stream_t stream);

/* Save / load with the staging blocks in HOST memory (pinned), the form the vLLM connector runs in
 * production (kv_cache_manager/py_connector/vllm/v1_connector.py:431-432,
 * kv_cache_manager/py_connector/vllm/data_transfer.py:119-150, 205-217).  Same layout rule as gather /
 * scatter above (a row is a token or a page), but the PCIe leg is done by the copy engines: blocks are
 * gathered into the caller's device bounce buffer and copied out (save), or copied in and scattered
 * (load).  The buffer is used as two halves of floor(bounce_bytes / 2 / block_bytes) blocks: the copies
 * run on a copy stream that the library keeps per device and direction, so that one half crosses PCIe
 * while the kernel works on the other; events tie that stream to `stream`, on which the whole call is
 * ordered as seen by the caller (nothing is copied before the work that precedes the call, and what
 * follows the call on `stream` sees every block in place).  A bounce buffer smaller than two blocks is
 * used whole, group after group, on `stream` alone.  A save on one stream and a load on another use
 * both PCIe directions at full rate, which kernels writing host memory directly do not.  Calls of one
 * direction on one device are enqueued one at a time (a mutex); they may come from any thread.  h_slot_idx is a HOST array of staging slots (NULL = slot b); slots
 * outside [0, n_slots) return KVCM_ER_INVALID_PARAMS before anything is launched or copied.
 * d_bounce: device memory, 16-byte aligned, at least one block (n_pools * rows_per_block * row_bytes). */
KVCM_API int32_t kvcm_b200_save_rows_to_host(const void *const *d_pool_ptrs, int32_t n_pools, void *h_staging,
                                             int64_t n_slots, const int32_t *d_row_idx, const int32_t *h_slot_idx,
                                             int32_t n_blocks, int32_t rows_per_block, int64_t row_bytes,
                                             int64_t pool_rows, void *d_bounce, int64_t bounce_bytes,
                                             uint32_t *d_status, kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_load_rows_from_host(const void *const *d_pool_ptrs, int32_t n_pools,
                                               const void *h_staging, int64_t n_slots, const int32_t *d_row_idx,
                                               const int32_t *h_slot_idx, int32_t n_blocks, int32_t rows_per_block,
                                               int64_t row_bytes, int64_t pool_rows, void *d_bounce,
                                               int64_t bounce_bytes, uint32_t *d_status, kvcm_stream_t stream);

/* Tuning knob, process-wide: which of the two gather/scatter kernels large aligned rows use.
 * mover 0 = 16-byte vector loads and stores, 1 = shared-memory ring driven by bulk async copies
 * (default); cache_hint 0|1|2 = default / streaming / streaming-loads-only policy of the vector
 * kernel; -1 leaves a setting unchanged.  Results are byte-identical in every setting.  The
 * environment variables KVCM_B200_MOVER=ldg|bulk and KVCM_B200_MOVER_HINT=0|1|2 set the initial
 * values.  Not stream-ordered: call it while no gather/scatter call is being issued. */
KVCM_API int32_t kvcm_b200_set_mover(int32_t mover, int32_t cache_hint);
/* Geometry of the bulk-copy ring: stages (2..8) of chunk_bytes (multiple of 1024) per CTA and CTAs
 * per SM; stages * chunk_bytes * ctas_per_sm must fit the SM's 224 KiB of shared memory.
 * (0, 0, 0) restores the default, which picks the geometry from the tile size.  Same calling rule as kvcm_b200_set_mover. */
KVCM_API int32_t kvcm_b200_set_bulk_geometry(int32_t stages, int32_t ctas_per_sm, int32_t chunk_bytes);
/* Rows shorter than this many bytes (multiple of 16, default 512) use the vector kernel even when the
 * bulk-copy ring is selected.  Same calling rule as kvcm_b200_set_mover. */
KVCM_API int32_t kvcm_b200_set_bulk_min_row_bytes(int32_t row_bytes);

/* Legacy single-block form: kv_cache_gather_kernel / kv_cache_scatter_kernel and gather_kv_caches /
 * scatter_kv_caches (kv_cache_manager/py_connector/kernel/gather_scatter_helper.py:10-172).
 * d_layer_ptrs[l] is a layer tensor [2, total_tokens, hidden_bytes]; staging is
 * [n_layers, 2, n_tokens, hidden_bytes].  A token index >= total_tokens (or < 0) is skipped
 * silently, as the reference kernels do (:36-38, :87-89). */
KVCM_API int32_t kvcm_b200_gather_legacy(const void *const *d_layer_ptrs, int32_t n_layers, int64_t total_tokens,
                                         void *staging, const int32_t *d_token_idx, int32_t n_tokens,
                                         int64_t hidden_bytes, kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_scatter_legacy(const void *const *d_layer_ptrs, int32_t n_layers, int64_t total_tokens,
                                          const void *staging, const int32_t *d_token_idx, int32_t n_tokens,
                                          int64_t hidden_bytes, kvcm_stream_t stream);

/* Batched iov copy: replaces the per-Iov cudaMemcpyAsync loops of LocalFileSdk::DoGet / DoPut
 * (kv_cache_manager/client/src/internal/sdk/local_file_sdk.cc:223-245, 326-353) and
 * Hf3fsUsrbioClient::CopyIovs (kv_cache_manager/client/src/internal/sdk/hf3fs_usrbio_client.cc:478-505)
 * with one launch.  Segment i copies d_segs[i].bytes bytes from src to dst; the host helper
 * kvcm_b200_iovs_to_segments lays the reference's Iov list (kv_cache_manager/client/include/common.h:99-116)
 * against a contiguous block string, honouring `ignore` (bytes skipped, offset still advanced). */
typedef struct kvcm_b200_seg {
    void *dst;
    const void *src;
    uint64_t bytes;
} kvcm_b200_seg_t;

typedef struct kvcm_b200_iov {
    uint8_t type;   /* MemoryType: 0 CPU, 1 GPU */
    uint8_t ignore; /* bool */
    uint8_t pad_[6];
    void *base;
    uint64_t size;
} kvcm_b200_iov_t;

KVCM_API int32_t kvcm_b200_copy_segments(const kvcm_b200_seg_t *d_segs, int32_t n_segs, kvcm_stream_t stream);
/* The same copy for callers that know how many bytes the segments hold in total (the span that
 * kvcm_b200_iovs_to_segments returns, minus ignored iovs): with a mean segment of 8 KiB or more the copy runs on
 * the bulk-copy (TMA) ring at the HBM roofline; segments whose ends are not 16-byte aligned are then moved by
 * one warp with byte accesses, so callers with large unaligned segments pass total_bytes = 0 (= the call above).
 * The waits of the ring are bounded; kvcm_b200_copy_wait_timeouts reads the per-device count of CTAs that gave
 * up (0 in any healthy run; synchronises with the device). */
KVCM_API int32_t kvcm_b200_copy_segments_sized(const kvcm_b200_seg_t *d_segs, int32_t n_segs, uint64_t total_bytes,
                                               kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_copy_wait_timeouts(uint32_t *h_count_out);
/* Host-only: direction 0 = iovs -> block string (Put), 1 = block string -> iovs (Get).  Writes at
 * most n_iovs segments to h_segs_out, returns their number in *n_segs_out and the bytes the iov
 * list spans in *span_bytes_out.  Every address it emits is one a kernel may touch: an iov of type CPU
 * is accepted only when the driver knows its base as pinned, registered, managed or device memory;
 * ordinary pageable memory - which the reference copies with std::memcpy
 * (kv_cache_manager/client/src/internal/sdk/local_file_sdk.cc:231-233, 339-341) - returns
 * KVCM_ER_UNSUPPORTED_MEMORY_TYPE before anything is launched.  A caller with such iovs copies them on
 * the host and passes them with `ignore` set, as the IovCopier adapter does. */
KVCM_API int32_t kvcm_b200_iovs_to_segments(const kvcm_b200_iov_t *h_iovs, int32_t n_iovs, void *block_string,
                                            int32_t direction, kvcm_b200_seg_t *h_segs_out, int32_t *n_segs_out,
                                            uint64_t *span_bytes_out);

/* Debug check of transferred buffers: replaces the GetIovsCrcDevice kernel
 * (kv_cache_manager/client/src/internal/sdk/sdk_buffer_check_util.cu:21-44).  d_crc_out[i] = reflected
 * CRC-32 (poly 0xEDB88320) of the first and last cal_bytes bytes of segment i (src, bytes). */
KVCM_API int32_t kvcm_b200_iov_crc(const kvcm_b200_seg_t *d_segs, int32_t n_segs, uint64_t cal_bytes,
                                   uint32_t *d_crc_out, kvcm_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * (2a) Chained token-block hash.
 *
 * Replaces GenKeyVector (kv_cache_manager/manager/cache_manager.cc:76-87) over hashInt64Array
 * (kv_cache_manager/manager/hash_util.h:8-24) for a whole batch of requests, and ApplyPrefixHash
 * (kv_cache_manager/optimizer/trace_converter/trace_util.cc:47-56) with block_size = 1.
 * Request r owns tokens[tok_off[r], tok_off[r+1]) and writes floor(len/block_size) keys at
 * d_keys[key_off[r] ...]; the hash state starts at 0 per request and is carried across blocks;
 * a trailing partial block is dropped.  u32 tokens are zero-extended (token ids are non-negative).
 * n_tokens_total is the extent of d_tokens (reads stay inside it).  d_tokens must be 16-byte aligned.
 * d_req_order (optional, NULL = request order) is a permutation of [0, n_req) saying which request
 * each lane takes; listing requests longest first (kvcm_b200_length_order) groups chains of similar
 * length into one warp and starts the longest chains first, which matters for ragged batches.
 * warps_per_sm (0 = fill the SMs) caps the hashing warps resident per SM.  A chain advances one token per
 * ~25 cycles alone on its SM, ~29 / ~32 / ~35 with 2 / 3 / 4 hashing warps there and ~55 on a full SM, so a
 * batch ruled by a few very long requests wants a small cap and a batch of many requests none
 * (kvcm_b200_length_order suggests the value).  A cap of 1..4 also selects 512-byte fills of the staging
 * ring (one bulk copy per lane and fill), without which the copies could not keep up with a lone chain.
 * The keys written depend on neither.
 * Tokens reach shared memory by bulk copies that complete on mbarriers; every wait on one is bounded,
 * and a warp whose wait ran out stops writing keys and counts itself in a per-device counter that
 * kvcm_b200_hash_wait_timeouts reads (0 in any healthy run).
 * ---------------------------------------------------------------------------------------- */
KVCM_API int32_t kvcm_b200_hash_blocks_u32(const uint32_t *d_tokens, int64_t n_tokens_total, const int64_t *d_tok_off,
                                           int32_t n_req, int32_t block_size, int64_t *d_keys,
                                           const int64_t *d_key_off, const int32_t *d_req_order,
                                           int32_t warps_per_sm, kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_hash_blocks_i64(const int64_t *d_tokens, int64_t n_tokens_total, const int64_t *d_tok_off,
                                           int32_t n_req, int32_t block_size, int64_t *d_keys,
                                           const int64_t *d_key_off, const int32_t *d_req_order,
                                           int32_t warps_per_sm, kvcm_stream_t stream);
/* *h_count_out = warps of kvcm_b200_hash_blocks_* launches on the current device that gave up on a
 * bounded wait since the library was loaded.  Synchronises with the device.  (No counterpart in the
 * reference, whose hash runs on the CPU.) */
KVCM_API int32_t kvcm_b200_hash_wait_timeouts(uint32_t *h_count_out);
/* Host-only helper: h_order_out = requests sorted by token count, longest first (stable);
 * *warps_per_sm_out (optional) = the residency cap to pass along with that order. */
KVCM_API int32_t kvcm_b200_length_order(const int64_t *h_tok_off, int32_t n_req, int32_t *h_order_out,
                                        int32_t *warps_per_sm_out);
/* Host-only helper: key_off[r] = sum_{q<r} floor((tok_off[q+1]-tok_off[q]) / block_size); n_req+1 entries. */
KVCM_API int32_t kvcm_b200_key_offsets(const int64_t *h_tok_off, int32_t n_req, int32_t block_size,
                                       int64_t *h_key_off);

/* ------------------------------------------------------------------------------------------
 * (2b) Block index: the GPU-resident replica of MetaIndexer's key -> locations map that the
 * matchers probe (kv_cache_manager/meta/meta_indexer.cc:419-440, 650-752;
 * kv_cache_manager/meta/meta_local_backend.cc:253-327; kv_cache_manager/common/concurrent_hash_map.h).
 * Open addressing, 16-byte slots {int64 key, uint64 value} plus one tag byte per slot (0 = never used,
 * else an 8-bit fingerprint) that lets a miss end in the L2-resident tag array instead of HBM.
 * Every int64 is a legal key.  17 bytes per slot, two slots per key of capacity.
 *
 * The value word summarises the key's location map for the matchers
 * (kv_cache_manager/manager/select_location_policy.cc:8-38).  A location has a status
 * (kv_cache_manager/manager/cache_location.h:44-50) and a storage class c in [0,16) - the
 * DataStorageType, or a per-storage id under a named policy:
 *   bit c        (0..15)  some location of class c is CLS_SERVING
 *   bit 16 + c   (16..31) some location of class c has status != CLS_NOT_FOUND
 *   bit 32                the location map is non-empty
 *   bits 33 + 3c .. 35 + 3c, c in [0,8)   status of the key's location in class c: 0 = the map has no
 *                         location of that class, else CacheLocationStatus + 1.  Read and written only by
 *                         kvcm_b200_index_update_status; the matchers read the summary bits above, which
 *                         that entry point keeps in step.  KVCM_VAL_LOCATION(c, status) builds all three.
 *   bit 63                always set in a stored value (lookups return 0 for an absent key)
 * `avail_mask` arguments carry bit c set when the active SelectLocationPolicy gives class c a
 * weight > 0 (all classes with the default static weights).
 * ---------------------------------------------------------------------------------------- */
#define KVCM_VAL_SERVING(c) (1ull << (c))
#define KVCM_VAL_WRITABLE(c) (1ull << (16 + (c)))
#define KVCM_VAL_NONEMPTY (1ull << 32)
#define KVCM_VAL_PRESENT (1ull << 63)
#define KVCM_VAL_STATUS_SHIFT 33u
/* The bits one location of class c in [0,8) with CacheLocationStatus `status` contributes to a value word. */
#define KVCM_VAL_LOCATION(c, status)                                                                  \
    (KVCM_VAL_NONEMPTY | ((uint64_t)((status) + 1) << (KVCM_VAL_STATUS_SHIFT + 3u * (c))) |            \
     ((status) == 3 ? KVCM_VAL_SERVING(c) : 0ull) | ((status) != 0 ? KVCM_VAL_WRITABLE(c) : 0ull))
#define KVCM_AVAIL_ALL 0xFFFFu

typedef struct kvcm_b200_index kvcm_b200_index_t;

/* Allocates a table for at least max_keys keys at load factor <= 0.5 on the current device
 * (synchronous).  Insertions beyond the capacity are refused and counted, never spin. */
KVCM_API int32_t kvcm_b200_index_create(int64_t max_keys, kvcm_b200_index_t **out);
KVCM_API int32_t kvcm_b200_index_destroy(kvcm_b200_index_t *index);
KVCM_API int32_t kvcm_b200_index_clear(kvcm_b200_index_t *index, kvcm_stream_t stream);
/* Number of slots, and (synchronous on `stream`) the number of live keys. */
KVCM_API int32_t kvcm_b200_index_stats(kvcm_b200_index_t *index, int64_t *slots, int64_t *live_keys,
                                       kvcm_stream_t stream);
/* Insert or overwrite: value[i] (or `uniform_value` when d_values is NULL) is stored with
 * KVCM_VAL_PRESENT or-ed in.  Mirrors the write side MetaIndexer::Put / Update reduces to for the
 * matchers.  d_status[0] counts keys refused because the table is full. */
KVCM_API int32_t kvcm_b200_index_upsert(kvcm_b200_index_t *index, const int64_t *d_keys, const uint64_t *d_values,
                                        uint64_t uniform_value, int64_t n, uint32_t *d_status, kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_index_erase(kvcm_b200_index_t *index, const int64_t *d_keys, int64_t n,
                                       kvcm_stream_t stream);
/* Number of slots and, synchronous on `stream`, the live keys and the slots in use (live keys + the
 * tombstones erased keys leave behind).  An insert reuses the first tombstone on its key's probe chain, so
 * under steady insert / erase churn `used_slots` levels off; it only claims a never-used slot while
 * used_slots < 7/8 of the slots, and is refused (d_status[0] of upsert) beyond that even though
 * live_keys may be far below the capacity: time for kvcm_b200_index_rehash. */
KVCM_API int32_t kvcm_b200_index_usage(kvcm_b200_index_t *index, int64_t *slots, int64_t *live_keys,
                                       int64_t *used_slots, kvcm_stream_t stream);
/* Rebuilds the table in place without its tombstones: the live {key, value} pairs are copied to the
 * caller's device workspace (16-byte aligned, at least kvcm_b200_index_rehash_workspace_bytes), the slots
 * are reset and the pairs inserted again.  Three launches on `stream`; no other call may use the index
 * while they run.  d_status[0] (may be NULL) counts pairs that could not be put back (never, unless the
 * index is written concurrently).  Counterpart of nothing in the reference, whose std::unordered_map
 * (kv_cache_manager/meta/meta_local_backend.h:60) frees a node when a key is deleted. */
KVCM_API int64_t kvcm_b200_index_rehash_workspace_bytes(kvcm_b200_index_t *index);
/* By default the library rebuilds the table by itself: it adds up, on the host, the keys passed to erase and
 * to the status transitions since the last rebuild, and once that sum reaches slots / 8 the next upsert runs
 * the rebuild first, on the upsert's stream, with a workspace taken from and returned to the stream-ordered
 * allocator (cudaMallocAsync; when that fails the rebuild is put off to the next upsert).  So tombstones
 * never take more than an eighth of the slots and probe chains stay short under any amount of insert /
 * erase churn.  erased_keys = 0 turns this off for callers that call kvcm_b200_index_rehash themselves. */
KVCM_API int32_t kvcm_b200_index_set_auto_rehash(kvcm_b200_index_t *index, int64_t erased_keys);
KVCM_API int32_t kvcm_b200_index_rehash(kvcm_b200_index_t *index, void *d_workspace, int64_t workspace_bytes,
                                        uint32_t *d_status, kvcm_stream_t stream);

/* Location-status transitions, one task per key, applied with a compare-and-swap on the key's value word:
 * the device-side counterpart of MetaSearcher::BatchUpdateLocationStatus, BatchCASLocationStatus,
 * BatchCADLocationStatus and BatchDeleteLocation (kv_cache_manager/manager/meta_searcher.cc:410-487,
 * 489-580, 582-717, 719-820).  A task names the storage class of the location (the stand-in for the
 * reference's location id: the word keeps one status per class, classes 0..7), the status it must have
 * (KVCM_STATUS_ANY = unconditional update / delete) and the status it gets (KVCM_STATUS_DELETE removes the
 * location and, with the key's last location, the key, as BatchCADLocationStatus does;
 * KVCM_STATUS_DELETE_KEEP_KEY removes the location the way BatchDeleteLocation does: an absent key is
 * KVCM_OK, and a key that loses its last location stays in the index with an empty location map).  d_tasks[i] = KVCM_STATUS_TASK(class, expected, new), or NULL and every key gets `uniform_task`.
 * d_results[i]: KVCM_OK; KVCM_EC_NOENT when the key is absent or has no location of that class
 * (BlockCacheLocationsMeta::UpdateLocationStatus / GetLocationStatus, kv_cache_manager/manager/cache_location.cc:60-82);
 * KVCM_EC_MISMATCH when the status differs from the expected one; KVCM_EC_BADARGS for a malformed task.
 * A key whose last location is deleted by KVCM_STATUS_DELETE leaves the index, as MetaIndexer::MA_DELETE does; so does
 * a key whose map is ALREADY empty (left behind by KVCM_STATUS_DELETE_KEEP_KEY) when a KVCM_STATUS_DELETE task names
 * it, while the task itself answers KVCM_EC_NOENT: the reference's compare-and-delete drops a key with an empty map
 * whatever its tasks did (meta_searcher.cc:689-692).  Several tasks of
 * one call may name the same key; they are applied one after the other in an unspecified order.  A key
 * with more than one location in one class cannot be represented: keep such a key's map on the host and
 * write its word with kvcm_b200_index_upsert.  The _sharded form touches only the keys this shard owns
 * and leaves the d_results entries of the other keys as they were. */
#define KVCM_STATUS_ANY 0xFFu
#define KVCM_STATUS_DELETE 0xFFu
#define KVCM_STATUS_DELETE_KEEP_KEY 0xFEu
#define KVCM_STATUS_TASK(cls, expected, next) \
    ((uint32_t)(cls) | ((uint32_t)(expected) << 8) | ((uint32_t)(next) << 16))
KVCM_API int32_t kvcm_b200_index_update_status(kvcm_b200_index_t *index, const int64_t *d_keys,
                                               const uint32_t *d_tasks, uint32_t uniform_task, int64_t n,
                                               int32_t *d_results, kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_index_update_status_sharded(kvcm_b200_index_t *index, const int64_t *d_keys,
                                                       const uint32_t *d_tasks, uint32_t uniform_task, int64_t n,
                                                       int32_t shard_count, int32_t shard_rank,
                                                       int32_t *d_results, kvcm_stream_t stream);

/* One new location per key, merged into the key's location map on the device: the counterpart of
 * MetaSearcher::BatchAddLocation (kv_cache_manager/manager/meta_searcher.cc:312-408), which reads the key's map or
 * starts an empty one, adds the location and writes the map back.  Key i gets a location of storage class
 * d_classes[i] (or `uniform_class` when d_classes is NULL; classes 0..7) in status `status_of_new` -
 * BatchAddLocation always adds in CLS_WRITING (2); a key that is absent is inserted, a key that is present keeps its
 * other locations (the merge is a compare-and-swap on the value word, so several tasks of one launch on the same key
 * take turns).  d_results[i]: KVCM_OK; KVCM_EC_EXIST when the key already holds a location of that class - the
 * word keeps one status per class, where the reference would add a second location under a fresh id;
 * KVCM_EC_NOSPC when the table is full (also counted in d_status[0], as kvcm_b200_index_upsert counts it);
 * KVCM_EC_BADARGS for a class above 7.  The sharded form touches only the keys the shard owns and leaves the other
 * results as they are. */
KVCM_API int32_t kvcm_b200_index_add_location(kvcm_b200_index_t *index, const int64_t *d_keys,
                                              const uint8_t *d_classes, int32_t uniform_class, int32_t status_of_new,
                                              int64_t n, int32_t *d_results, uint32_t *d_status, kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_index_add_location_sharded(kvcm_b200_index_t *index, const int64_t *d_keys,
                                                      const uint8_t *d_classes, int32_t uniform_class,
                                                      int32_t status_of_new, int64_t n, int32_t shard_count,
                                                      int32_t shard_rank, int32_t *d_results, uint32_t *d_status,
                                                      kvcm_stream_t stream);

/* d_values_out[i] = stored value of key i, 0 when absent (MetaIndexer::Get -> EC_NOENT). */
KVCM_API int32_t kvcm_b200_index_lookup(kvcm_b200_index_t *index, const int64_t *d_keys, int64_t n,
                                        uint64_t *d_values_out, kvcm_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * (2b) Matchers.  Requests are given in CSR form: request r owns d_keys[key_off[r], key_off[r+1]).
 * ---------------------------------------------------------------------------------------- */

/* MetaSearcher::PrefixMatch (kv_cache_manager/manager/meta_searcher.cc:120-145 over :74-118).
 * Keys with IsIndexInMaskRange true (kv_cache_manager/manager/cache_location.cc:9-21) are removed
 * first: d_mask_off[r] masks the first mask_off[r] keys of request r (BlockMaskOffset);
 * d_mask_bits is a per-key byte array aligned with d_keys (BlockMaskVector, padded with 0);
 * either or both may be NULL.  d_len_out[r] = number of leading unmasked keys that have a
 * SERVING location with weight > 0. */
KVCM_API int32_t kvcm_b200_match_prefix(kvcm_b200_index_t *index, const int64_t *d_keys, const int64_t *d_key_off,
                                        int32_t n_req, const int64_t *d_mask_off, const uint8_t *d_mask_bits,
                                        uint32_t avail_mask, int32_t *d_len_out, kvcm_stream_t stream);

/* MetaSearcher::ReverseRollSlideWindowMatch (kv_cache_manager/manager/meta_searcher.cc:196-265)
 * with the argument guard of kv_cache_manager/manager/cache_manager.cc:993-997.
 * d_base_out[r] = start of the rightmost window of sw_blocks consecutive servable keys, -1 when
 * there is none, -2 when the request has fewer than sw_blocks keys (EC_BADARGS for that request).
 * sw_blocks <= 0 returns KVCM_EC_BADARGS for the call (0 never terminates in the reference). */
KVCM_API int32_t kvcm_b200_match_sw(kvcm_b200_index_t *index, const int64_t *d_keys, const int64_t *d_key_off,
                                    int32_t n_req, int32_t sw_blocks, uint32_t avail_mask, int32_t *d_base_out,
                                    kvcm_stream_t stream);

/* CacheManager::StartWriteCache for a batch of requests (kv_cache_manager/manager/cache_manager.cc:334-430):
 * FilterWriteCache, then MetaSearcher::BatchAddLocation of the keys still to be written, with the answers the
 * reference gives when it serves the requests one after the other in batch order - what request r sees is the
 * index before the call plus what requests 0..r-1 of the batch added.  Per request: d_offset_out / d_mask_out /
 * d_n_new_out exactly as kvcm_b200_filter_write returns them (under that view); per key, d_added_out[i] = 1 when
 * this request gave key i its new location (storage_class, CLS_WRITING) - those keys, in request order, are the
 * request's write session; d_new_off_out[r] (n_req + 1 entries) = session keys of the requests before r.  (A new
 * key that cannot take the location - its map holds one of that class already, in whatever status, or the table is
 * full - counts in d_n_new_out as in the reference's answer but is not part of the session.)
 * A key that several requests of the batch name is written by the first of them; the later ones see it as being
 * written, as they would in the reference.  storage_class (0..7) must be a class avail_mask counts.  The keys of one
 * request are taken to be distinct (chained hashes are).  d_status[0] counts keys refused because the table is full
 * (their d_added_out stays 0).  The workspace (kvcm_b200_start_write_workspace_bytes, 256-byte aligned) is scratch.
 *
 * kvcm_b200_finish_write is CacheManager::FinishWriteCache (:432-501) for the sessions of such a batch - the same
 * d_keys / d_key_off / d_added / d_new_off: the j-th session key of request r turns CLS_SERVING when the success mask
 * holds it (j < d_success_off[r], or d_success_bits[d_new_off[r] + j] != 0 when d_success_bits is given: one byte per
 * session key of the batch) and loses its location otherwise (what the reference leaves to its reclaimer).
 * d_results[r]: KVCM_OK; KVCM_EC_BADARGS for an offset beyond the session's keys (nothing is touched); else the code
 * of a transition that failed. */
KVCM_API int64_t kvcm_b200_start_write_workspace_bytes(int64_t n_keys_total, int32_t n_req);
KVCM_API int32_t kvcm_b200_start_write(kvcm_b200_index_t *index, const int64_t *d_keys, const int64_t *d_key_off,
                                       int32_t n_req, int64_t n_keys_total, uint32_t avail_mask, int32_t storage_class,
                                       void *d_workspace, int64_t workspace_bytes, int32_t *d_offset_out,
                                       uint8_t *d_mask_out, int32_t *d_n_new_out, uint8_t *d_added_out,
                                       int64_t *d_new_off_out, uint32_t *d_status, kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_finish_write(kvcm_b200_index_t *index, const int64_t *d_keys, const int64_t *d_key_off,
                                        int32_t n_req, const uint8_t *d_added, const int64_t *d_new_off,
                                        const int64_t *d_success_off, const uint8_t *d_success_bits,
                                        int32_t storage_class, int32_t *d_results, kvcm_stream_t stream);
/* The same two calls for ONE table of a hash-range-sharded index .  Every shard runs them on
 * the same batch - all shards' requests in one order, e.g. gathered rank after rank - and gets the same answers:
 *   1. kvcm_b200_write_snapshot_sharded: d_flags_out[i] = the flags of key i (KVCM_FLAG_*, with KVCM_FLAG_HAS_CLASS)
 *      where this shard owns it, 0 elsewhere; a bytewise maximum over the shards (an all-reduce) gives every shard
 *      every key's flags as its owner sees them before the batch.
 *   2. kvcm_b200_start_write_sharded with those flags: block masks and write sessions for all requests, computed
 *      alike on every shard; each shard merges the new locations of the keys it owns.  Whether a key takes its
 *      location is read off its flags (the class is free or not), so the sessions agree everywhere; a full table
 *      shows in the owner's d_status[0] only.  d_request_skip (optional, one byte per request) marks entries of
 *      the batch that are no requests (padding of a gathered batch): they get empty answers.
 *   3. kvcm_b200_finish_write_sharded: every shard makes the transitions of the session keys it owns; d_results[r]
 *      holds this shard's part (a maximum over the shards gives the request's code).
 * No kernel of these reads another shard's table. */
KVCM_API int32_t kvcm_b200_write_snapshot_sharded(kvcm_b200_index_t *index, const int64_t *d_keys, int64_t n,
                                                  uint32_t avail_mask, int32_t storage_class, int32_t shard_count,
                                                  int32_t shard_rank, uint8_t *d_flags_out, kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_start_write_sharded(kvcm_b200_index_t *index, const int64_t *d_keys,
                                               const int64_t *d_key_off, int32_t n_req, int64_t n_keys_total,
                                               uint32_t avail_mask, int32_t storage_class,
                                               const uint8_t *d_snapshot_flags, const uint8_t *d_request_skip,
                                               int32_t shard_count, int32_t shard_rank, void *d_workspace,
                                               int64_t workspace_bytes, int32_t *d_offset_out, uint8_t *d_mask_out,
                                               int32_t *d_n_new_out, uint8_t *d_added_out, int64_t *d_new_off_out,
                                               uint32_t *d_status, kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_finish_write_sharded(kvcm_b200_index_t *index, const int64_t *d_keys,
                                                const int64_t *d_key_off, int32_t n_req, const uint8_t *d_added,
                                                const int64_t *d_new_off, const int64_t *d_success_off,
                                                const uint8_t *d_success_bits, int32_t storage_class,
                                                int32_t shard_count, int32_t shard_rank, int32_t *d_results,
                                                kvcm_stream_t stream);

/* MetaSearcher::BatchGetBestLocation / BatchGetLocation (kv_cache_manager/manager/meta_searcher.cc:147-194,
 * 267-310): per key, no early stop.  d_flags_out[i]: bit0 a location would be returned (servable),
 * bit1 key exists, bit2 location map non-empty, bit3 ExistsForWrite (select_location_policy.cc:29-38). */
#define KVCM_FLAG_SERVABLE 1u
#define KVCM_FLAG_EXISTS 2u
#define KVCM_FLAG_NONEMPTY 4u
#define KVCM_FLAG_WRITABLE 8u
#define KVCM_FLAG_HAS_CLASS 16u /* only in the flags of kvcm_b200_write_snapshot_sharded: the key holds a location of the write's class */
KVCM_API int32_t kvcm_b200_batch_get(kvcm_b200_index_t *index, const int64_t *d_keys, int64_t n, uint32_t avail_mask,
                                     uint8_t *d_flags_out, kvcm_stream_t stream);

/* CacheManager::FilterWriteCache (kv_cache_manager/manager/cache_manager.cc:589-635) for a batch of
 * StartWriteCache requests: which keys still have to be written.  A key "exists" when it has a location
 * with status != CLS_NOT_FOUND and weight > 0 (ExistsForWrite).  If the existing keys of request r form
 * a prefix, d_offset_out[r] = index of the first missing key (the BlockMaskOffset the reference returns)
 * and d_n_new_out[r] = keys after it.  Otherwise d_offset_out[r] = -1, the answer is the BlockMaskVector
 * d_mask_out (per key, aligned with d_keys: 1 = location map non-empty; always written when not NULL)
 * and d_n_new_out[r] = keys whose map is empty. */
KVCM_API int32_t kvcm_b200_filter_write(kvcm_b200_index_t *index, const int64_t *d_keys, const int64_t *d_key_off,
                                        int32_t n_req, uint32_t avail_mask, int32_t *d_offset_out,
                                        uint8_t *d_mask_out, int32_t *d_n_new_out, kvcm_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Hash-range-sharded index: one logical index split over shard_count GPUs.  Key k belongs to shard
 * floor(fmix64(k) * shard_count / 2^64).  Each GPU holds an ordinary index with the keys it owns;
 * the exchange between GPUs (all-gather of keys, min / max reduction of results) is the caller's,
 * over NCCL.  The reference has no sharded index (one MetaIndexer per instance,
 * kv_cache_manager/meta/meta_indexer_manager.cc:9-30); these entry points keep the results of the
 * matchers above identical when the table is split:
 *   upsert_sharded        inserts only the keys this shard owns out of the full batch;
 *   match_prefix_sharded  as match_prefix, but keys of other shards never stop the count, so
 *                         min over shards of d_len_out = the unsharded prefix length;
 *   batch_get_sharded     as batch_get, 0 for keys of other shards without probing, so a byte-wise
 *                         max over shards of the flags = the unsharded flags;
 *   match_sw_from_flags   the sliding-window search of match_sw over such combined flags (bit0).
 * ---------------------------------------------------------------------------------------- */
KVCM_API int32_t kvcm_b200_index_upsert_sharded(kvcm_b200_index_t *index, const int64_t *d_keys,
                                                const uint64_t *d_values, uint64_t uniform_value, int64_t n,
                                                int32_t shard_count, int32_t shard_rank, uint32_t *d_status,
                                                kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_match_prefix_sharded(kvcm_b200_index_t *index, const int64_t *d_keys,
                                                const int64_t *d_key_off, int32_t n_req, const int64_t *d_mask_off,
                                                const uint8_t *d_mask_bits, uint32_t avail_mask, int32_t shard_count,
                                                int32_t shard_rank, int32_t *d_len_out, kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_batch_get_sharded(kvcm_b200_index_t *index, const int64_t *d_keys, int64_t n,
                                             uint32_t avail_mask, int32_t shard_count, int32_t shard_rank,
                                             uint8_t *d_flags_out, kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_match_sw_from_flags(const uint8_t *d_flags, const int64_t *d_key_off, int32_t n_req,
                                               int32_t sw_blocks, int32_t *d_base_out, kvcm_stream_t stream);

/* Routed exchange: the device-side halves of an all-to-all that sends every key to the shard that owns it and
 * brings one answer byte back (the transport in between is the caller's: NCCL all-to-all, or its own).  A key
 * crosses the link once as 8 bytes instead of being probed remotely with 32-byte loads.
 *   route_count    d_counts[s] = keys of the batch owned by shard s (the array is cleared first);
 *   route_scatter  d_cursor[s] = where shard s's bucket starts in d_keys_out (the exclusive prefix sums of the
 *                  counts; advanced by the call); keys land in their owner's bucket in no particular order and
 *                  d_pos_out[i] says where key i went;
 *   gather_bytes   d_dst[i] = d_src[d_pos[i]]: the answers, which arrive in bucket order, back in key order;
 *   match_prefix_from_flags  match_prefix over per-key flag bytes (KVCM_FLAG_SERVABLE) instead of index probes,
 *                  as match_sw_from_flags is to match_sw.
 * The owner of a key is the shard of kvcm_b200_index_upsert_sharded.  n < 2^31, shard_count <= 64.  (No
 * counterpart in the reference, whose index is not sharded.) */
KVCM_API int32_t kvcm_b200_route_count(const int64_t *d_keys, int64_t n, int32_t shard_count, uint32_t *d_counts,
                                       kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_route_scatter(const int64_t *d_keys, int64_t n, int32_t shard_count, uint32_t *d_cursor,
                                         int64_t *d_keys_out, int32_t *d_pos_out, kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_gather_bytes(const uint8_t *d_src, const int32_t *d_pos, int64_t n, uint8_t *d_dst,
                                        kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_match_prefix_from_flags(const uint8_t *d_flags, const int64_t *d_key_off, int32_t n_req,
                                                   const int64_t *d_mask_off, const uint8_t *d_mask_bits,
                                                   int32_t *d_len_out, kvcm_stream_t stream);

/* The routed exchange over peer memory (one NVLink / NVSwitch box), with no transport between the two halves:
 * every rank owns an exchange area (an inbox of capacity_keys keys and as many answer bytes), exports it once and
 * maps the others' (CUDA IPC, as for the shards above).  Per batch, with h_counts the shard_count x shard_count
 * matrix of route_count results of all ranks (h_counts[r * shard_count + s] = keys rank r sends to shard s, host
 * memory, the same on every rank):
 *   route_dispatch  stores each of this rank's keys into its owner's inbox (peer stores, staged per CTA so that
 *                   warps write consecutive addresses) and records in d_pos_out[i] where key i's answer will land;
 *                   d_cursor is scratch of shard_count words;
 *   -- all ranks meet (their dispatch kernels have completed) --
 *   route_answer    looks up the keys that arrived in this rank's inbox and stores each flag byte (batch_get's)
 *                   into the asking rank's answer buffer;
 *   -- all ranks meet --
 *   route_collect   d_flags_out[i] = the answer for key i, in key order.
 * No kernel waits on another rank; the meeting points are the caller's (a barrier collective enqueued on the
 * same stream, or stream synchronisation plus a host barrier).  The next batch may be dispatched once every
 * rank has enqueued its collect behind the second meeting point.  EC_NOSPC when some inbox or answer buffer
 * would overflow (nothing is launched; the same verdict on every rank, since all hold the same matrix and
 * capacity).  attach_local is for areas that live in one process.  (No counterpart in the reference.) */
typedef struct kvcm_b200_route_area kvcm_b200_route_area_t;
typedef struct kvcm_b200_route_export {
    uint8_t ipc_handle[64];
    uint64_t capacity_keys;
    int32_t device;
    int32_t reserved_;
} kvcm_b200_route_export_t;
KVCM_API int32_t kvcm_b200_route_area_create(int64_t capacity_keys, kvcm_b200_route_area_t **out);
KVCM_API int32_t kvcm_b200_route_area_destroy(kvcm_b200_route_area_t *area);
KVCM_API int32_t kvcm_b200_route_area_export(kvcm_b200_route_area_t *area, kvcm_b200_route_export_t *out);
KVCM_API int32_t kvcm_b200_route_area_attach(kvcm_b200_route_area_t *area, int32_t shard_count, int32_t shard_rank,
                                             const kvcm_b200_route_export_t *exports);
KVCM_API int32_t kvcm_b200_route_area_attach_local(kvcm_b200_route_area_t *area, int32_t shard_count,
                                                   int32_t shard_rank, kvcm_b200_route_area_t *const *areas);
KVCM_API int32_t kvcm_b200_route_area_detach(kvcm_b200_route_area_t *area);
KVCM_API int32_t kvcm_b200_route_dispatch(kvcm_b200_route_area_t *area, const int64_t *d_keys, int64_t n,
                                          const uint32_t *h_counts, uint32_t *d_cursor, int32_t *d_pos_out,
                                          kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_route_answer(kvcm_b200_index_t *index, kvcm_b200_route_area_t *area,
                                        const uint32_t *h_counts, uint32_t avail_mask, kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_route_collect(kvcm_b200_route_area_t *area, const int32_t *d_pos, int64_t n,
                                         uint8_t *d_flags_out, kvcm_stream_t stream);

/* Peer-attached shards: the collective-free way to query a sharded index on one NVLink / NVSwitch
 * box.  Every GPU exports its shard once; each GPU maps the others' shards (CUDA IPC, peer access)
 * and attaches them to its own handle.  From then on match_prefix, match_sw, batch_get and
 * index_lookup on that handle resolve every key in the table of the shard that owns it, with plain
 * 16-byte peer loads over NVLink - a rank matches its own requests against the whole index without
 * any exchange step.  Writes (upsert_sharded, erase, clear) stay local to the shard; after a batch
 * of writes the ranks synchronise their streams and meet at a host barrier before anyone queries.
 * A process must detach (or destroy the index) before a peer frees its shard, and must not leave
 * while peers may still be probing its memory.  attach_local_peers is the same for shards that live
 * in one process (several GPUs driven by one process with peer access enabled, or tests). */
typedef struct kvcm_b200_index_export {
    uint8_t ipc_handle[64];
    uint64_t n_slots;
    int32_t device;
    int32_t reserved_;
} kvcm_b200_index_export_t;
KVCM_API int32_t kvcm_b200_index_export(kvcm_b200_index_t *index, kvcm_b200_index_export_t *out);
KVCM_API int32_t kvcm_b200_index_attach_peers(kvcm_b200_index_t *index, int32_t shard_count, int32_t shard_rank,
                                              const kvcm_b200_index_export_t *exports);
KVCM_API int32_t kvcm_b200_index_attach_local_peers(kvcm_b200_index_t *index, int32_t shard_count,
                                                    int32_t shard_rank, kvcm_b200_index_t *const *shards);
KVCM_API int32_t kvcm_b200_index_detach_peers(kvcm_b200_index_t *index);

/* ------------------------------------------------------------------------------------------
 * (2c) Optimizer trace replay, no eviction.
 *
 * Replaces the sequential loop OptimizerRunner::RunTraces
 * (kv_cache_manager/optimizer/manager/optimizer_runner.cc:29-215) over RadixTreeIndex::InsertWithQuery /
 * PrefixQuery / InsertOnly (kv_cache_manager/optimizer/index/radix_tree_index.cc:198-282, 129-196, 19-87)
 * for one instance.  Traces are given in replay order (sorted by timestamp) in CSR form; the order
 * is the trace number.  d_trace_type[t]: 0 DialogTurn (query + insert of total_keys), 1 GetLocation
 * (query; the first d_mask_off[t] keys are masked, d_mask_off may be NULL; d_mask_bits, optional, one byte per
 * key of the batch, masks single keys on top of that - a BlockMaskVector with holes), 2 WriteCache (insert).
 * Outputs per trace, as the ReadRecord / WriteRecord of the reference hold them: external hit
 * blocks, internal (masked) hit blocks, blocks newly written, and - if d_cache_blocks is not NULL -
 * the number of cached blocks after the trace.  Exact for prefix-unique chained keys (the output of
 * the hash entry points); capacity-driven eviction is not modelled.
 * d_workspace: caller-owned scratch of at least kvcm_b200_replay_workspace_bytes(n_keys_total)
 * bytes, 256-byte aligned, contents irrelevant before and after.  d_status[0] counts keys that
 * found no room in the scratch table (cannot happen with the stated size).
 * ---------------------------------------------------------------------------------------- */
KVCM_API int64_t kvcm_b200_replay_workspace_bytes(int64_t n_keys_total);
KVCM_API int32_t kvcm_b200_replay(const int64_t *d_keys, const int64_t *d_key_off, const uint8_t *d_trace_type,
                                  const int64_t *d_mask_off, const uint8_t *d_mask_bits, int32_t n_traces,
                                  int64_t n_keys_total, void *d_workspace, int64_t workspace_bytes,
                                  int32_t *d_ext_hit, int32_t *d_int_hit, int32_t *d_written,
                                  int64_t *d_cache_blocks, uint32_t *d_status, kvcm_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * (2c') Optimizer trace replay with LRU eviction, for a sweep of quotas in one call.
 *
 * Replaces one run of OptimizerRunner::RunTraces per tradeoff-curve point
 * (kv_cache_manager/optimizer/analysis/script/optimizer_analysis_utils.py:95-144,278-330 start one
 * optimizer run per (capacity, policy) pair) for the "lru" policy
 * (kv_cache_manager/optimizer/eviction_policy/lru.cc:6-49) on the shared tier with one instance per
 * group: after every DialogTurn / WriteCache trace the cached blocks beyond the quota are evicted
 * from the cold end of the recency list (OptIndexerManager::CheckAndEvict,
 * kv_cache_manager/optimizer/manager/indexer_manager.cc:55-90).  precise = 0: whole batches of
 * evict_batch blocks until the excess is covered (EVICTION_MODE_GROUP_ROUGH / INSTANCE_ROUGH,
 * kv_cache_manager/optimizer/manager/eviction_manager.cc:86-192); precise != 0: exactly the excess
 * (EVICTION_MODE_INSTANCE_PRECISE, :194-239).  d_quota_blocks[c] is configuration c's
 * size_t(quota_capacity * used_percentage) (:249-266).
 * Trace encoding as kvcm_b200_replay.  Per-trace outputs are [n_configs][n_traces], configuration-major; pass
 * all four or none (NULL).  d_totals (optional, [n_configs][4] int64) receives per configuration the sums of
 * external hits, internal hits and written blocks over the trace and the cached blocks at its end - all a
 * tradeoff curve needs, so a large sweep can skip the per-trace arrays.
 * Exact for prefix-unique chained keys without repeats inside one trace.  Configurations are
 * independent and run in parallel (one warp each); one configuration is replayed in trace order.
 * d_workspace: kvcm_b200_replay_lru_workspace_bytes(n_keys_total, n_configs) bytes (-1: too large:
 * n_keys_total < 2^32 - 1, n_configs <= 65535), 256-byte aligned, contents irrelevant before and after.
 * Not covered here: leaf_aware_lru (kvcm_b200_replay_leaf_lru below), several instances sharing one group
 * quota (kvcm_b200_replay_lru_group below), random_lru (kvcm_b200_replay_random_lru below).  A group with
 * hierarchical_eviction_enabled differs for a replay only in the capacity its quota derives from (the first
 * storage tier's, eviction_manager.cc:247-258): the caller passes that quota.
 * ---------------------------------------------------------------------------------------- */
KVCM_API int64_t kvcm_b200_replay_lru_workspace_bytes(int64_t n_keys_total, int32_t n_configs);
KVCM_API int32_t kvcm_b200_replay_lru(const int64_t *d_keys, const int64_t *d_key_off, const uint8_t *d_trace_type,
                                      const int64_t *d_mask_off, const uint8_t *d_mask_bits, int32_t n_traces,
                                      int64_t n_keys_total,
                                      const int64_t *d_quota_blocks, int32_t n_configs, int32_t evict_batch,
                                      int32_t precise, void *d_workspace, int64_t workspace_bytes,
                                      int32_t *d_ext_hit, int32_t *d_int_hit, int32_t *d_written,
                                      int64_t *d_cache_blocks, int64_t *d_totals, uint32_t *d_status,
                                      kvcm_stream_t stream);

/* The LRU sweep for an instance group whose instances share one quota
 * (OptEvictionManager::EvictByGroupRough / EvictByInstanceRough / EvictByInstancePrecise and
 * GetExcessUsageForInstanceInGroup, kv_cache_manager/optimizer/manager/eviction_manager.cc:86-266).  Every instance
 * has a tree and a recency list of its own (kv_cache_manager/optimizer/manager/optimizer_manager.cc:66-99), so the
 * same key in two instances is two blocks; after a write the usage of all instances is summed against the quota.
 * d_trace_instance[t] in [0, n_instances) names the instance of trace t; the traces of all instances come in one
 * replay (timestamp) order.  eviction_mode: 1 = EVICTION_MODE_GROUP_ROUGH (rounds of evict_batch blocks from every
 * instance of the group), 2 = INSTANCE_ROUGH and 3 = INSTANCE_PRECISE (from the writing instance only).
 * d_cache_blocks[c][t] is the usage of trace t's own instance after the trace (GetCurrentInstanceUsage,
 * kv_cache_manager/optimizer/manager/optimizer_runner.cc:116,196), d_totals[c][3] the usage of the group at the end,
 * d_instance_blocks (optional, [n_configs][n_instances]) that of every instance.  Otherwise as kvcm_b200_replay_lru
 * ("lru" policy in every instance; kvcm_b200_replay_leaf_lru_group is the "leaf_aware_lru" twin).  A trace whose
 * instance is out of range is replayed as an empty trace and counted in d_status[0]. */
#define KVCM_B200_REPLAY_GROUP_MAX_INSTANCES 64
KVCM_API int64_t kvcm_b200_replay_lru_group_workspace_bytes(int64_t n_keys_total, int32_t n_configs,
                                                            int32_t n_instances);
KVCM_API int32_t kvcm_b200_replay_lru_group(const int64_t *d_keys, const int64_t *d_key_off,
                                            const uint8_t *d_trace_type, const int64_t *d_mask_off,
                                            const uint8_t *d_mask_bits, const int32_t *d_trace_instance,
                                            int32_t n_instances, int32_t n_traces, int64_t n_keys_total,
                                            const int64_t *d_quota_blocks, int32_t n_configs, int32_t evict_batch,
                                            int32_t eviction_mode, void *d_workspace, int64_t workspace_bytes,
                                            int32_t *d_ext_hit, int32_t *d_int_hit, int32_t *d_written,
                                            int64_t *d_cache_blocks, int64_t *d_totals, int64_t *d_instance_blocks,
                                            uint32_t *d_status, kvcm_stream_t stream);
/* The same call with one more output: d_instance_blocks_per_trace (optional, int64 [n_configs][n_traces][n_instances])
 * = the usage of EVERY instance of the group after each trace, i.e. ReadRecord::blocks_per_instance, which the
 * reference writes into the CachedBlocksPerInstance / CachedBlocksAllInstance columns of its hit-rate CSV
 * (kv_cache_manager/optimizer/analysis/result_analysis.cc:96-113).  Instances are numbered as d_trace_instance
 * numbers them (the reference lists them in the order of an unordered_map). */
KVCM_API int32_t kvcm_b200_replay_lru_group_records(
    const int64_t *d_keys, const int64_t *d_key_off, const uint8_t *d_trace_type, const int64_t *d_mask_off,
    const uint8_t *d_mask_bits, const int32_t *d_trace_instance, int32_t n_instances, int32_t n_traces,
    int64_t n_keys_total, const int64_t *d_quota_blocks, int32_t n_configs, int32_t evict_batch, int32_t eviction_mode,
    void *d_workspace, int64_t workspace_bytes, int32_t *d_ext_hit, int32_t *d_int_hit, int32_t *d_written,
    int64_t *d_cache_blocks, int64_t *d_totals, int64_t *d_instance_blocks, int64_t *d_instance_blocks_per_trace,
    uint32_t *d_status, kvcm_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * (2d) The same sweep under the "random_lru" eviction policy
 * (kv_cache_manager/optimizer/eviction_policy/random_lru.cc:5-131, random_lru.h:13-47): the cached blocks sit in a
 * dense vector beside their last access times; a round of evictions draws sampling_size = evict_batch /
 * sample_rate indices with the policy's xorshift generator (sample_rate <= 0 means 0.1, as in the reference's
 * constructor), orders the first k of them by access time with std::partial_sort and removes those blocks by
 * swap-and-pop.  Equal access times are common (the blocks of one trace share one), and which of several
 * equally old samples go is decided by the order partial_sort leaves equal elements in: the kernel restates
 * that algorithm (heap-select + sort-heap) step for step, and every configuration starts from the reference's
 * generator seed, so the victims are the reference's.
 * Arguments as kvcm_b200_replay_lru, plus d_timestamps (optional, int64 per trace: the traces' timestamp_us;
 * the trace number when NULL) and sample_rate.  evict_batch <= KVCM_B200_RANDOM_LRU_MAX_BATCH and
 * sampling_size <= KVCM_B200_RANDOM_LRU_MAX_SAMPLE (the sample lives in shared memory), else
 * KVCM_EC_OUT_OF_LIMIT.  Exact for prefix-unique chained keys without repeats inside one trace.  One warp per
 * configuration; the generator, the heap and the removals are sequential, so a round of evictions costs tens of
 * microseconds.  d_workspace: kvcm_b200_replay_random_lru_workspace_bytes(n_keys_total, n_configs) bytes
 * (16 bytes per key occurrence for each configuration; -1: too large), 256-byte aligned.
 * ---------------------------------------------------------------------------------------- */
#define KVCM_B200_RANDOM_LRU_MAX_SAMPLE 2048
#define KVCM_B200_RANDOM_LRU_MAX_BATCH 512
KVCM_API int64_t kvcm_b200_replay_random_lru_workspace_bytes(int64_t n_keys_total, int32_t n_configs);
/* Host-only self test: runs, on host arrays, the very routine the sweep kernel orders its samples with
 * (h_idx[i] travels with h_times[i]; afterwards the first k entries are the k smallest times in ascending
 * order, equal times in the order std::partial_sort leaves them).  Lets a box without a GPU check the
 * restatement against the standard library.  No counterpart in the reference. */
KVCM_API int32_t kvcm_b200_selftest_partial_sort(uint32_t *h_idx, int64_t *h_times, uint32_t k, uint32_t n);
KVCM_API int32_t kvcm_b200_replay_random_lru(const int64_t *d_keys, const int64_t *d_key_off,
                                             const uint8_t *d_trace_type, const int64_t *d_mask_off,
                                             const uint8_t *d_mask_bits, const int64_t *d_timestamps,
                                             int32_t n_traces, int64_t n_keys_total, const int64_t *d_quota_blocks,
                                             int32_t n_configs, int32_t evict_batch, int32_t precise,
                                             double sample_rate, void *d_workspace, int64_t workspace_bytes,
                                             int32_t *d_ext_hit, int32_t *d_int_hit, int32_t *d_written,
                                             int64_t *d_cache_blocks, int64_t *d_totals, uint32_t *d_status,
                                             kvcm_stream_t stream);
/* The random_lru sweep for an instance group whose instances share one quota: every instance has its own block
 * vector, its own generator (each policy object starts from the reference's seed) and its own sampling size;
 * h_sample_rate (HOST memory, n_instances doubles, NULL = the default rate everywhere) is each instance's
 * eviction_policy_params.sample_rate.  d_trace_instance, n_instances, eviction_mode, d_cache_blocks, d_totals,
 * d_instance_blocks and d_instance_blocks_per_trace exactly as in kvcm_b200_replay_lru_group_records, everything else
 * as in kvcm_b200_replay_random_lru, which is this call with one instance and eviction_mode 3 (precise) or 2.  A
 * group-rough round draws a fresh sample in every instance in the configuration's order
 * (kv_cache_manager/optimizer/manager/eviction_manager.cc:86-146), so the generators advance as the reference's do.
 * A trace whose instance is out of range is replayed as an empty trace and counted in d_status[0]. */
KVCM_API int64_t kvcm_b200_replay_random_lru_group_workspace_bytes(int64_t n_keys_total, int32_t n_configs,
                                                                   int32_t n_instances);
KVCM_API int32_t kvcm_b200_replay_random_lru_group(
    const int64_t *d_keys, const int64_t *d_key_off, const uint8_t *d_trace_type, const int64_t *d_mask_off,
    const uint8_t *d_mask_bits, const int64_t *d_timestamps, const int32_t *d_trace_instance,
    const double *h_sample_rate, int32_t n_instances, int32_t n_traces, int64_t n_keys_total,
    const int64_t *d_quota_blocks, int32_t n_configs, int32_t evict_batch, int32_t eviction_mode, void *d_workspace,
    int64_t workspace_bytes, int32_t *d_ext_hit, int32_t *d_int_hit, int32_t *d_written, int64_t *d_cache_blocks,
    int64_t *d_totals, int64_t *d_instance_blocks, int64_t *d_instance_blocks_per_trace, uint32_t *d_status,
    kvcm_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * (2c'') The same sweep under the "leaf_aware_lru" eviction policy
 * (kv_cache_manager/optimizer/eviction_policy/leaf_aware_lru.cc:20-160; chosen by eviction_policy_type in
 * the optimizer's startup configuration, kv_cache_manager/optimizer/eviction_policy/policy_factory.cc:8-47).
 * Only blocks of childless tree nodes queue up for eviction; a block whose node has cached children leaves
 * the queue when it reaches the cold end; a node whose children hold no cached block any more gets its
 * blocks queued again, placed by last access time.  The tree of RadixTreeIndex
 * (kv_cache_manager/optimizer/index/radix_tree_index.cc:19-392) is therefore kept per configuration, with
 * the reference's node splits and its removal of emptied leaves.
 * Arguments as kvcm_b200_replay_lru, plus d_timestamps (optional, int64 per trace: the traces' timestamp_us,
 * which order re-queued blocks; the trace number when NULL) and n_traces in the workspace size.
 * d_status[0] (optional) counts keys the id table refused and walks that hit their iteration limit; non-zero
 * means the input broke the premise below and the results are void.
 * Exact for prefix-unique chained keys without repeats inside one trace.  One warp per configuration; the
 * walk to a sorted insertion point and the list surgery around a group of blocks run in one lane, so a
 * configuration costs more than under plain LRU.
 * d_workspace: kvcm_b200_replay_leaf_lru_workspace_bytes(n_keys_total, n_traces, n_configs) bytes
 * (about 25 bytes per key occurrence and 56 per trace for each configuration; -1: too large), 256-byte aligned.
 * ---------------------------------------------------------------------------------------- */
KVCM_API int64_t kvcm_b200_replay_leaf_lru_workspace_bytes(int64_t n_keys_total, int32_t n_traces,
                                                           int32_t n_configs);
KVCM_API int32_t kvcm_b200_replay_leaf_lru(const int64_t *d_keys, const int64_t *d_key_off,
                                           const uint8_t *d_trace_type, const int64_t *d_mask_off,
                                           const uint8_t *d_mask_bits, const int64_t *d_timestamps, int32_t n_traces,
                                           int64_t n_keys_total, const int64_t *d_quota_blocks, int32_t n_configs,
                                           int32_t evict_batch, int32_t precise, void *d_workspace,
                                           int64_t workspace_bytes, int32_t *d_ext_hit, int32_t *d_int_hit,
                                           int32_t *d_written, int64_t *d_cache_blocks, int64_t *d_totals,
                                           uint32_t *d_status, kvcm_stream_t stream);
/* The leaf_aware_lru sweep for an instance group whose instances share one quota: every instance has its own tree
 * and its own leaf-aware queue, the usage of all of them is summed against the quota after a write, and blocks
 * go in rounds over the instances or from the writing instance only - d_trace_instance, n_instances (up to
 * KVCM_B200_REPLAY_GROUP_MAX_INSTANCES), eviction_mode, d_cache_blocks, d_totals, d_instance_blocks and
 * d_instance_blocks_per_trace exactly as in kvcm_b200_replay_lru_group_records, everything else as in
 * kvcm_b200_replay_leaf_lru.  A round asks every instance for evict_batch blocks in the configuration's order
 * (LeafAwareLruEvictionPolicy::EvictBlocks per instance, kv_cache_manager/optimizer/manager/
 * eviction_manager.cc:86-146), and the emptied leaves of every instance are removed afterwards
 * (OptIndexerManager::CheckAndEvict, kv_cache_manager/optimizer/manager/indexer_manager.cc:55-90).
 * A trace whose instance is out of range is replayed as an empty trace and counted in d_status[0].
 * d_trace_instance may be NULL when n_instances is 1.  kvcm_b200_replay_leaf_lru is this call with one instance
 * and eviction_mode 3 (precise) or 2. */
KVCM_API int64_t kvcm_b200_replay_leaf_lru_group_workspace_bytes(int64_t n_keys_total, int32_t n_traces,
                                                                 int32_t n_configs, int32_t n_instances);
/* The same replay for a group whose instances do not all use one policy: h_instance_policy (HOST memory,
 * n_instances bytes, NULL = all leaf-aware) names every instance's eviction_policy_type, KVCM_POLICY_LEAF_AWARE_LRU or
 * KVCM_POLICY_LRU (EvictionPolicyFactory::CreatePolicy per instance, kv_cache_manager/optimizer/eviction_policy/
 * policy_factory.cc:8-47).  An "lru" instance keeps its tree and its queue in the same form; all its cached blocks
 * stay queued whatever their node's children, and a round takes its coldest blocks (lru.cc:28-49).  Workspace as for
 * kvcm_b200_replay_leaf_lru_group, whose arguments the others are.  A group of "lru" instances only is cheaper
 * through kvcm_b200_replay_lru_group, which needs no tree. */
#define KVCM_POLICY_LEAF_AWARE_LRU 0
#define KVCM_POLICY_LRU 1
KVCM_API int32_t kvcm_b200_replay_tree_group(
    const int64_t *d_keys, const int64_t *d_key_off, const uint8_t *d_trace_type, const int64_t *d_mask_off,
    const uint8_t *d_mask_bits, const int64_t *d_timestamps, const int32_t *d_trace_instance,
    const uint8_t *h_instance_policy, int32_t n_instances, int32_t n_traces, int64_t n_keys_total,
    const int64_t *d_quota_blocks, int32_t n_configs, int32_t evict_batch, int32_t eviction_mode, void *d_workspace,
    int64_t workspace_bytes, int32_t *d_ext_hit, int32_t *d_int_hit, int32_t *d_written, int64_t *d_cache_blocks,
    int64_t *d_totals, int64_t *d_instance_blocks, int64_t *d_instance_blocks_per_trace, uint32_t *d_status,
    kvcm_stream_t stream);
KVCM_API int32_t kvcm_b200_replay_leaf_lru_group(
    const int64_t *d_keys, const int64_t *d_key_off, const uint8_t *d_trace_type, const int64_t *d_mask_off,
    const uint8_t *d_mask_bits, const int64_t *d_timestamps, const int32_t *d_trace_instance, int32_t n_instances,
    int32_t n_traces, int64_t n_keys_total, const int64_t *d_quota_blocks, int32_t n_configs, int32_t evict_batch,
    int32_t eviction_mode, void *d_workspace, int64_t workspace_bytes, int32_t *d_ext_hit, int32_t *d_int_hit,
    int32_t *d_written, int64_t *d_cache_blocks, int64_t *d_totals, int64_t *d_instance_blocks,
    int64_t *d_instance_blocks_per_trace, uint32_t *d_status, kvcm_stream_t stream);
/* Any mix of the three policies in one group, as the reference's configuration allows it (every instance of a group
 * names its own eviction_policy_type; kv_cache_manager/optimizer/manager/eviction_manager.cc:21-60 makes one policy
 * object per instance): h_instance_policy may also hold KVCM_POLICY_RANDOM_LRU, and h_sample_rate (HOST memory,
 * n_instances doubles, read for the random_lru instances only; NULL or <= 0 = the policy's default 0.1) gives those
 * instances' eviction_policy_params.sample_rate.  A random_lru instance keeps the policy's block vector, access times
 * and generator instead of a tree and a queue, exactly as in kvcm_b200_replay_random_lru_group, whose limits on
 * evict_batch and evict_batch / sample_rate apply when such an instance is present; a round of the quota check asks
 * every instance in the configuration's order, each through its own EvictBlocks.  The workspace grows by the block
 * vectors when a random_lru instance is present: kvcm_b200_replay_policy_group_workspace_bytes takes the policy bytes.
 * Everything else as in kvcm_b200_replay_tree_group, which is this call without sample rates and refuses
 * KVCM_POLICY_RANDOM_LRU. */
#define KVCM_POLICY_RANDOM_LRU 2
KVCM_API int64_t kvcm_b200_replay_policy_group_workspace_bytes(int64_t n_keys_total, int32_t n_traces,
                                                               int32_t n_configs, const uint8_t *h_instance_policy,
                                                               int32_t n_instances);
KVCM_API int32_t kvcm_b200_replay_policy_group(
    const int64_t *d_keys, const int64_t *d_key_off, const uint8_t *d_trace_type, const int64_t *d_mask_off,
    const uint8_t *d_mask_bits, const int64_t *d_timestamps, const int32_t *d_trace_instance,
    const uint8_t *h_instance_policy, const double *h_sample_rate, int32_t n_instances, int32_t n_traces,
    int64_t n_keys_total, const int64_t *d_quota_blocks, int32_t n_configs, int32_t evict_batch,
    int32_t eviction_mode, void *d_workspace, int64_t workspace_bytes, int32_t *d_ext_hit, int32_t *d_int_hit,
    int32_t *d_written, int64_t *d_cache_blocks, int64_t *d_totals, int64_t *d_instance_blocks,
    int64_t *d_instance_blocks_per_trace, uint32_t *d_status, kvcm_stream_t stream);

/* Host-only helper: h_order_out[i] = the number of the trace replayed i-th when a trace file's traces are put in
 * timestamp order the way OptimizerLoader::LoadTrace does it - std::sort by timestamp
 * (kv_cache_manager/optimizer/trace_converter/trace_util.cc:6-8,42-45), which is not stable, so traces of equal
 * timestamps come out in the standard library's order.  The same routine runs here, so a replay of a file with
 * repeated timestamps visits the traces in the reference's order. */
KVCM_API int32_t kvcm_b200_trace_replay_order(const int64_t *h_timestamps, int64_t n_traces, int64_t *h_order_out);
/* Host-only helper: the order in which a std::unordered_map<std::string, ...> iterates after n_ops operations -
 * operation i names key h_keys[h_key_off[i] .. h_key_off[i+1]) and either erases it (h_erase[i] != 0) or assigns it
 * the value i.  h_order_out receives the values left in iteration order, *h_n_out their number.  The reference's
 * publisher-log reader appends its unfinished writes in that order
 * (kv_cache_manager/optimizer/trace_converter/publisher_log_converter.cc:207-219); the same container runs here. */
KVCM_API int32_t kvcm_b200_string_map_iteration_order(const char *h_keys, const int64_t *h_key_off,
                                                      const uint8_t *h_erase, int64_t n_ops, int64_t *h_order_out,
                                                      int64_t *h_n_out);

/* Trace replay for callers that cannot allocate device memory.  (No counterpart in the reference: it
 * exists for how this library gets embedded, not for a reference interface.)
 *
 * Who needs it: a connector or optimizer hook that runs inside an inference engine's process after
 * the engine has claimed nearly all of HBM for weights and KV pools - a cudaMalloc at that point can
 * fail, and even when it succeeds it synchronises the device and stalls the engine's streams - and
 * plugin hosts whose rules simply forbid allocator calls on the serving path.  Such a caller owns its
 * inputs and outputs but has nowhere to get the replay's scratch table from.
 *
 * Same arguments, results and kernels as kvcm_b200_replay minus the workspace pair and the per-key mask
 * bytes (offset masks only): the scratch table
 * is a fixed array inside the library's device image, KVCM_B200_REPLAY_NOALLOC_SCRATCH_BYTES (8 MiB +
 * 256 B) held by every GPU that loads the library until the process exits.  Limits and rules:
 *   - at most KVCM_B200_REPLAY_NOALLOC_MAX_KEYS keys per call; more returns KVCM_EC_OUT_OF_LIMIT
 *     ("size beyond the fixed limit of this entry point") before anything is launched;
 *   - the call performs no cudaMalloc / cudaFree and calls no allocating library routine;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress with that
 *     device current); make that first call before any stream capture begins;
 *   - every call on a device shares the one array.  Each call rebuilds the part of the table it uses
 *     before reading it, so results never depend on the previous call, but two calls that overlap on
 *     the GPU (different streams, or threads without ordering) race on it: serialise them. */
#define KVCM_B200_REPLAY_NOALLOC_MAX_KEYS 262144
#define KVCM_B200_REPLAY_NOALLOC_SCRATCH_BYTES (524288 * 16 + 256)
KVCM_API int32_t kvcm_b200_replay_noalloc(const int64_t *d_keys, const int64_t *d_key_off,
                                          const uint8_t *d_trace_type, const int64_t *d_mask_off, int32_t n_traces,
                                          int64_t n_keys_total, int32_t *d_ext_hit, int32_t *d_int_hit,
                                          int32_t *d_written, int64_t *d_cache_blocks, uint32_t *d_status,
                                          kvcm_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* KVCM_B200_H_ */
