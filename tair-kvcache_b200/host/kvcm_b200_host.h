// C++ host adapters over the C ABI of libkvcm_b200.so, with the shapes of the reference's own
// operators so that C++ callers (CacheManager, MetaSearcher, the Optimizer, TransferClient SDKs)
// can switch without touching CUDA:
//
//   GenKeyVector / GenKeyVectorBatch / ApplyPrefixHash
//       kv_cache_manager/manager/cache_manager.cc:76-87, kv_cache_manager/optimizer/trace_converter/trace_util.cc:47-56
//   GpuBlockIndex        the device replica of MetaIndexer's table (kv_cache_manager/meta/meta_indexer.cc:419-440)
//   GpuMetaSearcher      PrefixMatch / ReverseRollSlideWindowMatch / BatchGet
//       kv_cache_manager/manager/meta_searcher.cc:74-265, batch-of-one and batched forms
//   GpuTraceReplayer     OptimizerRunner::RunTraces (kv_cache_manager/optimizer/manager/optimizer_runner.cc:29-215) without
//                        eviction, or with the "lru" policy at many quota points at once
//   IovCopier            the per-Iov loops of kv_cache_manager/client/src/internal/sdk/local_file_sdk.cc:223-245,326-353
//
// Header-only, C++17, needs only <cuda_runtime.h> and kvcm_b200.h.  Every call stages its
// arguments through pinned host buffers owned by the adapter, runs on the adapter's stream and
// synchronises before returning (the reference operators are synchronous too).  Return values are
// the C ABI's codes: 0 = ok, transfer side = ClientErrorCode numbers, manager side = 1000 + ErrorCode.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <variant>
#include <vector>

#include "kvcm_b200.h"

namespace kvcm_b200 {

using KeyVector = std::vector<int64_t>;       // kv_cache_manager/manager/cache_manager.h:53-56
using TokenIdsVector = std::vector<int64_t>;
using BlockMaskVector = std::vector<bool>;    // kv_cache_manager/manager/cache_location.h:52-57
using BlockMaskOffset = size_t;
using BlockMask = std::variant<BlockMaskVector, BlockMaskOffset>;

// kv_cache_manager/manager/cache_location.h:44-50
enum CacheLocationStatus : int32_t { CLS_NOT_FOUND = 0, CLS_NEW = 1, CLS_WRITING = 2, CLS_SERVING = 3, CLS_DELETING = 4 };

struct LocationSummary {
    CacheLocationStatus status;
    int32_t storage_class;  // DataStorageType, or a per-storage id under a named policy; clamped to [0, 15]
};

// Value word of a key from its location map (the facts SelectForMatch / ExistsForWrite read,
// kv_cache_manager/manager/select_location_policy.cc:8-38).
inline uint64_t EncodeLocations(const std::vector<LocationSummary> &locations) {
    uint64_t word = 0;
    for (const LocationSummary &l : locations) {
        const int c = l.storage_class < 0 ? 0 : (l.storage_class > 15 ? 15 : l.storage_class);
        word |= KVCM_VAL_NONEMPTY;
        if (l.status == CLS_SERVING) word |= KVCM_VAL_SERVING(c);
        if (l.status != CLS_NOT_FOUND) word |= KVCM_VAL_WRITABLE(c);
    }
    return word;
}

namespace detail {

// Grow-only pair of a pinned host buffer and a device buffer of the same size.
class Mirror {
public:
    Mirror() = default;
    Mirror(const Mirror &) = delete;
    Mirror &operator=(const Mirror &) = delete;
    ~Mirror() { Release(); }
    // device_only: no pinned twin (scratch that never crosses PCIe).
    bool Reserve(size_t bytes, bool device_only = false) {
        if (bytes <= capacity_) return true;
        Release();
        size_t cap = 4096;
        while (cap < bytes) cap <<= 1;
        if ((!device_only && cudaMallocHost(&host_, cap) != cudaSuccess) || cudaMalloc(&dev_, cap) != cudaSuccess) {
            cudaGetLastError();
            Release();
            return false;
        }
        capacity_ = cap;
        return true;
    }
    template <class T>
    T *host() { return static_cast<T *>(host_); }
    template <class T>
    T *dev() { return static_cast<T *>(dev_); }
    bool ToDevice(size_t bytes, cudaStream_t s) {
        return bytes == 0 || cudaMemcpyAsync(dev_, host_, bytes, cudaMemcpyHostToDevice, s) == cudaSuccess;
    }
    bool ToHost(size_t bytes, cudaStream_t s) {
        return bytes == 0 || cudaMemcpyAsync(host_, dev_, bytes, cudaMemcpyDeviceToHost, s) == cudaSuccess;
    }

private:
    void Release() {
        if (host_) cudaFreeHost(host_);
        if (dev_) cudaFree(dev_);
        host_ = dev_ = nullptr;
        capacity_ = 0;
    }
    void *host_ = nullptr;
    void *dev_ = nullptr;
    size_t capacity_ = 0;
};

inline int32_t Sync(cudaStream_t s) {
    return cudaStreamSynchronize(s) == cudaSuccess ? KVCM_OK : KVCM_ER_CUDA_STREAM_SYNCHRONIZE_ERROR;
}

}  // namespace detail

// Batched chained block hash.  One instance per thread (it owns staging buffers).
class GpuKeyGenerator {
public:
    explicit GpuKeyGenerator(cudaStream_t stream = nullptr) : stream_(stream) {}

    // GenKeyVector for many requests: keys[r] = chained hashes of the whole blocks of tokens[r].
    int32_t GenKeyVectorBatch(const std::vector<TokenIdsVector> &tokens, int64_t block_size,
                              std::vector<KeyVector> *keys) {
        keys->assign(tokens.size(), {});
        if (block_size <= 0) return KVCM_EC_BADARGS;
        const int32_t n_req = static_cast<int32_t>(tokens.size());
        if (n_req == 0) return KVCM_OK;
        int64_t n_tok = 0;
        for (const auto &t : tokens) n_tok += static_cast<int64_t>(t.size());
        const size_t off_bytes = sizeof(int64_t) * (n_req + 1);
        if (!tok_.Reserve(sizeof(int64_t) * (n_tok + 2)) || !tok_off_.Reserve(off_bytes) ||
            !key_off_.Reserve(off_bytes)) {
            return KVCM_EC_NOSPC;
        }
        int64_t at = 0;
        for (int32_t r = 0; r < n_req; ++r) {
            tok_off_.host<int64_t>()[r] = at;
            if (!tokens[r].empty()) std::memcpy(tok_.host<int64_t>() + at, tokens[r].data(), sizeof(int64_t) * tokens[r].size());
            at += static_cast<int64_t>(tokens[r].size());
        }
        tok_off_.host<int64_t>()[n_req] = at;
        int32_t rc = kvcm_b200_key_offsets(tok_off_.host<int64_t>(), n_req, static_cast<int32_t>(block_size),
                                           key_off_.host<int64_t>());
        if (rc != KVCM_OK) return rc;
        const int64_t n_keys = key_off_.host<int64_t>()[n_req];
        if (!keys_.Reserve(sizeof(int64_t) * (n_keys + 1))) return KVCM_EC_NOSPC;
        if (!tok_.ToDevice(sizeof(int64_t) * n_tok, stream_) || !tok_off_.ToDevice(off_bytes, stream_) ||
            !key_off_.ToDevice(off_bytes, stream_)) {
            return KVCM_ER_CUDAMEMCPY_ERROR;
        }
        rc = kvcm_b200_hash_blocks_i64(tok_.dev<int64_t>(), n_tok, tok_off_.dev<int64_t>(), n_req,
                                       static_cast<int32_t>(block_size), keys_.dev<int64_t>(),
                                       key_off_.dev<int64_t>(), nullptr, 0, stream_);
        if (rc != KVCM_OK) return rc;
        if (!keys_.ToHost(sizeof(int64_t) * n_keys, stream_)) return KVCM_ER_CUDAMEMCPY_ERROR;
        rc = detail::Sync(stream_);
        if (rc != KVCM_OK) return rc;
        for (int32_t r = 0; r < n_req; ++r) {
            const int64_t b = key_off_.host<int64_t>()[r], e = key_off_.host<int64_t>()[r + 1];
            (*keys)[r].assign(keys_.host<int64_t>() + b, keys_.host<int64_t>() + e);
        }
        return KVCM_OK;
    }

    // The reference's single-request operator: a batch of one.
    KeyVector GenKeyVector(const TokenIdsVector &tokens, int64_t block_size) {
        std::vector<KeyVector> out;
        GenKeyVectorBatch({tokens}, block_size, &out);
        return out.empty() ? KeyVector{} : out[0];
    }

    // One chained key per id (block size 1).
    KeyVector ApplyPrefixHash(const std::vector<int64_t> &hash_ids) { return GenKeyVector(hash_ids, 1); }

private:
    cudaStream_t stream_;
    detail::Mirror tok_, tok_off_, key_off_, keys_;
};

// Device-resident block index of one instance.
class GpuBlockIndex {
public:
    explicit GpuBlockIndex(int64_t max_keys, cudaStream_t stream = nullptr) : stream_(stream) {
        kvcm_b200_index_create(max_keys, &index_);
    }
    GpuBlockIndex(const GpuBlockIndex &) = delete;
    GpuBlockIndex &operator=(const GpuBlockIndex &) = delete;
    ~GpuBlockIndex() { kvcm_b200_index_destroy(index_); }
    bool ok() const { return index_ != nullptr; }
    kvcm_b200_index_t *handle() const { return index_; }

    // Mirrors a MetaIndexer::Put / Update batch: key i gets value word values[i] (EncodeLocations).
    int32_t Put(const KeyVector &keys, const std::vector<uint64_t> &values) {
        if (keys.size() != values.size()) return KVCM_EC_BADARGS;
        const size_t n = keys.size();
        if (n == 0) return KVCM_OK;
        if (!keys_.Reserve(sizeof(int64_t) * n) || !vals_.Reserve(sizeof(uint64_t) * n)) return KVCM_EC_NOSPC;
        std::memcpy(keys_.host<int64_t>(), keys.data(), sizeof(int64_t) * n);
        std::memcpy(vals_.host<uint64_t>(), values.data(), sizeof(uint64_t) * n);
        if (!keys_.ToDevice(sizeof(int64_t) * n, stream_) || !vals_.ToDevice(sizeof(uint64_t) * n, stream_)) {
            return KVCM_ER_CUDAMEMCPY_ERROR;
        }
        const int32_t rc = kvcm_b200_index_upsert(index_, keys_.dev<int64_t>(), vals_.dev<uint64_t>(), 0,
                                                  static_cast<int64_t>(n), nullptr, stream_);
        return rc != KVCM_OK ? rc : detail::Sync(stream_);
    }

    int32_t Erase(const KeyVector &keys) {
        const size_t n = keys.size();
        if (n == 0) return KVCM_OK;
        if (!keys_.Reserve(sizeof(int64_t) * n)) return KVCM_EC_NOSPC;
        std::memcpy(keys_.host<int64_t>(), keys.data(), sizeof(int64_t) * n);
        if (!keys_.ToDevice(sizeof(int64_t) * n, stream_)) return KVCM_ER_CUDAMEMCPY_ERROR;
        const int32_t rc = kvcm_b200_index_erase(index_, keys_.dev<int64_t>(), static_cast<int64_t>(n), stream_);
        return rc != KVCM_OK ? rc : detail::Sync(stream_);
    }

    // MetaSearcher::BatchAddLocation (kv_cache_manager/manager/meta_searcher.cc:312-408) on the replica: key i gets a
    // location of storage class `classes[i]` (DataStorageType's number; one entry = the same class for all) in
    // CLS_WRITING, merged into the key's map on the device.  (*results)[i]: KVCM_OK, KVCM_EC_EXIST, KVCM_EC_NOSPC.
    int32_t AddLocation(const KeyVector &keys, const std::vector<uint8_t> &classes, std::vector<int32_t> *results,
                        int32_t status = 2 /* CLS_WRITING */) {
        const size_t n = keys.size();
        results->assign(n, KVCM_OK);
        if (classes.size() != n && classes.size() != 1) return KVCM_EC_BADARGS;
        if (n == 0) return KVCM_OK;
        const bool uniform = classes.size() == 1 && n != 1;
        if (!keys_.Reserve(sizeof(int64_t) * n) || !vals_.Reserve(sizeof(uint64_t) * n) ||
            !codes_.Reserve(sizeof(int32_t) * n)) {
            return KVCM_EC_NOSPC;
        }
        std::memcpy(keys_.host<int64_t>(), keys.data(), sizeof(int64_t) * n);
        if (!uniform) std::memcpy(vals_.host<uint8_t>(), classes.data(), n);
        if (!keys_.ToDevice(sizeof(int64_t) * n, stream_) || (!uniform && !vals_.ToDevice(n, stream_))) {
            return KVCM_ER_CUDAMEMCPY_ERROR;
        }
        const int32_t rc = kvcm_b200_index_add_location(index_, keys_.dev<int64_t>(),
                                                        uniform ? nullptr : vals_.dev<uint8_t>(),
                                                        uniform ? classes[0] : 0, status, static_cast<int64_t>(n),
                                                        codes_.dev<int32_t>(), nullptr, stream_);
        return rc != KVCM_OK ? rc : FetchCodes(n, results);
    }

    // MetaSearcher::BatchUpdateLocationStatus / BatchCASLocationStatus / BatchCADLocationStatus / BatchDeleteLocation
    // (meta_searcher.cc:410-820) on the replica: tasks[i] = KVCM_STATUS_TASK(class, expected, new); one entry = the
    // same task for all keys (FinishWriteCache of a batch).  (*results)[i]: KVCM_OK, KVCM_EC_NOENT, KVCM_EC_MISMATCH.
    int32_t UpdateLocationStatus(const KeyVector &keys, const std::vector<uint32_t> &tasks,
                                 std::vector<int32_t> *results) {
        const size_t n = keys.size();
        results->assign(n, KVCM_OK);
        if (tasks.size() != n && tasks.size() != 1) return KVCM_EC_BADARGS;
        if (n == 0) return KVCM_OK;
        const bool uniform = tasks.size() == 1 && n != 1;
        if (!keys_.Reserve(sizeof(int64_t) * n) || !vals_.Reserve(sizeof(uint64_t) * n) ||
            !codes_.Reserve(sizeof(int32_t) * n)) {
            return KVCM_EC_NOSPC;
        }
        std::memcpy(keys_.host<int64_t>(), keys.data(), sizeof(int64_t) * n);
        if (!uniform) std::memcpy(vals_.host<uint32_t>(), tasks.data(), sizeof(uint32_t) * n);
        if (!keys_.ToDevice(sizeof(int64_t) * n, stream_) || (!uniform && !vals_.ToDevice(sizeof(uint32_t) * n, stream_))) {
            return KVCM_ER_CUDAMEMCPY_ERROR;
        }
        const int32_t rc = kvcm_b200_index_update_status(index_, keys_.dev<int64_t>(),
                                                         uniform ? nullptr : vals_.dev<uint32_t>(),
                                                         uniform ? tasks[0] : 0, static_cast<int64_t>(n),
                                                         codes_.dev<int32_t>(), stream_);
        return rc != KVCM_OK ? rc : FetchCodes(n, results);
    }

private:
    int32_t FetchCodes(size_t n, std::vector<int32_t> *results) {
        if (!codes_.ToHost(sizeof(int32_t) * n, stream_)) return KVCM_ER_CUDAMEMCPY_ERROR;
        const int32_t rc = detail::Sync(stream_);
        if (rc != KVCM_OK) return rc;
        std::memcpy(results->data(), codes_.host<int32_t>(), sizeof(int32_t) * n);
        return KVCM_OK;
    }

    cudaStream_t stream_;
    kvcm_b200_index_t *index_ = nullptr;
    detail::Mirror keys_, vals_, codes_;
};

// The matchers of MetaSearcher over a GpuBlockIndex.  Results are lengths / window starts / flags;
// turning matched keys into CacheLocation objects stays with the caller's CPU-side table.
class GpuMetaSearcher {
public:
    GpuMetaSearcher(GpuBlockIndex *index, uint32_t avail_mask = KVCM_AVAIL_ALL, cudaStream_t stream = nullptr)
        : index_(index), avail_mask_(avail_mask), stream_(stream) {}

    // Batched PrefixMatch: out_len[r] = number of leading unmasked servable keys of request r.
    int32_t PrefixMatchBatch(const std::vector<KeyVector> &keys, const std::vector<BlockMask> &masks,
                             std::vector<int32_t> *out_len) {
        const int32_t n_req = static_cast<int32_t>(keys.size());
        out_len->assign(n_req, 0);
        if (!masks.empty() && masks.size() != keys.size()) return KVCM_EC_BADARGS;
        if (n_req == 0) return KVCM_OK;
        int32_t rc = Stage(keys);
        if (rc != KVCM_OK) return rc;
        const int64_t n_keys = key_off_.host<int64_t>()[n_req];
        // Offsets and vectors both become a per-key byte mask: index i is masked when
        // IsIndexInMaskRange says so (kv_cache_manager/manager/cache_location.cc:9-21).
        const uint8_t *d_bits = nullptr;
        if (!masks.empty()) {
            if (!bits_.Reserve(static_cast<size_t>(n_keys) + 1)) return KVCM_EC_NOSPC;
            uint8_t *bits = bits_.host<uint8_t>();
            std::memset(bits, 0, static_cast<size_t>(n_keys));
            for (int32_t r = 0; r < n_req; ++r) {
                uint8_t *b = bits + key_off_.host<int64_t>()[r];
                const size_t n = keys[r].size();
                if (std::holds_alternative<BlockMaskVector>(masks[r])) {
                    const auto &v = std::get<BlockMaskVector>(masks[r]);
                    for (size_t i = 0; i < n && i < v.size(); ++i) b[i] = v[i] ? 1 : 0;
                } else {
                    const size_t off = std::get<BlockMaskOffset>(masks[r]);
                    for (size_t i = 0; i < n && i < off; ++i) b[i] = 1;
                }
            }
            if (!bits_.ToDevice(static_cast<size_t>(n_keys), stream_)) return KVCM_ER_CUDAMEMCPY_ERROR;
            d_bits = bits_.dev<uint8_t>();
        }
        if (!out_.Reserve(sizeof(int32_t) * n_req)) return KVCM_EC_NOSPC;
        rc = kvcm_b200_match_prefix(index_->handle(), keys_.dev<int64_t>(), key_off_.dev<int64_t>(), n_req, nullptr,
                                    d_bits, avail_mask_, out_.dev<int32_t>(), stream_);
        if (rc != KVCM_OK) return rc;
        if (!out_.ToHost(sizeof(int32_t) * n_req, stream_)) return KVCM_ER_CUDAMEMCPY_ERROR;
        rc = detail::Sync(stream_);
        if (rc == KVCM_OK) std::memcpy(out_len->data(), out_.host<int32_t>(), sizeof(int32_t) * n_req);
        return rc;
    }

    // MetaSearcher::PrefixMatch for one request.
    int32_t PrefixMatch(const KeyVector &keys, const BlockMask &mask, size_t *out_len) {
        std::vector<int32_t> len;
        const int32_t rc = PrefixMatchBatch({keys}, {mask}, &len);
        *out_len = rc == KVCM_OK ? static_cast<size_t>(len[0]) : 0;
        return rc;
    }

    // Batched ReverseRollSlideWindowMatch: out_base[r] = start of the matched window, -1 none,
    // -2 when request r has fewer than sw_size keys.  sw_size <= 0 -> KVCM_EC_BADARGS.
    int32_t ReverseRollSlideWindowMatchBatch(const std::vector<KeyVector> &keys, int32_t sw_size,
                                             std::vector<int32_t> *out_base) {
        const int32_t n_req = static_cast<int32_t>(keys.size());
        out_base->assign(n_req, -1);
        if (sw_size <= 0) return KVCM_EC_BADARGS;
        if (n_req == 0) return KVCM_OK;
        int32_t rc = Stage(keys);
        if (rc != KVCM_OK) return rc;
        if (!out_.Reserve(sizeof(int32_t) * n_req)) return KVCM_EC_NOSPC;
        rc = kvcm_b200_match_sw(index_->handle(), keys_.dev<int64_t>(), key_off_.dev<int64_t>(), n_req, sw_size,
                                avail_mask_, out_.dev<int32_t>(), stream_);
        if (rc != KVCM_OK) return rc;
        if (!out_.ToHost(sizeof(int32_t) * n_req, stream_)) return KVCM_ER_CUDAMEMCPY_ERROR;
        rc = detail::Sync(stream_);
        if (rc == KVCM_OK) std::memcpy(out_base->data(), out_.host<int32_t>(), sizeof(int32_t) * n_req);
        return rc;
    }

    // One request, with the reference's argument guard (kv_cache_manager/manager/cache_manager.cc:993-997).
    int32_t ReverseRollSlideWindowMatch(const KeyVector &keys, int32_t sw_size, int64_t *out_base) {
        *out_base = -1;
        if (sw_size <= 0 || keys.size() < static_cast<size_t>(sw_size)) return KVCM_EC_BADARGS;
        std::vector<int32_t> base;
        const int32_t rc = ReverseRollSlideWindowMatchBatch({keys}, sw_size, &base);
        if (rc == KVCM_OK) *out_base = base[0];
        return rc;
    }

    // BatchGetBestLocation / BatchGetLocation: flags per key (KVCM_FLAG_*), no early stop.
    int32_t BatchGet(const KeyVector &keys, std::vector<uint8_t> *flags) {
        flags->assign(keys.size(), 0);
        if (keys.empty()) return KVCM_OK;
        int32_t rc = Stage({keys});
        if (rc != KVCM_OK) return rc;
        if (!out_.Reserve(keys.size())) return KVCM_EC_NOSPC;
        rc = kvcm_b200_batch_get(index_->handle(), keys_.dev<int64_t>(), static_cast<int64_t>(keys.size()),
                                 avail_mask_, out_.dev<uint8_t>(), stream_);
        if (rc != KVCM_OK) return rc;
        if (!out_.ToHost(keys.size(), stream_)) return KVCM_ER_CUDAMEMCPY_ERROR;
        rc = detail::Sync(stream_);
        if (rc == KVCM_OK) std::memcpy(flags->data(), out_.host<uint8_t>(), keys.size());
        return rc;
    }

    // CacheManager::StartWriteCache for a batch of requests, answered as if they were served in batch order
    // (kv_cache_manager/manager/cache_manager.cc:334-430): (*masks)[r] is the block mask FilterWriteCache gives
    // request r, (*new_keys)[r] the keys that got a location of `storage_class` in CLS_WRITING - the request's write
    // session.  The batch stays staged on the device for FinishWriteCacheBatch.
    int32_t StartWriteCacheBatch(const std::vector<KeyVector> &keys, int32_t storage_class,
                                 std::vector<BlockMask> *masks, std::vector<KeyVector> *new_keys) {
        const int32_t n_req = static_cast<int32_t>(keys.size());
        masks->assign(n_req, BlockMask{BlockMaskOffset{0}});
        new_keys->assign(n_req, KeyVector{});
        session_requests_ = 0;
        if (n_req == 0) return KVCM_OK;
        int32_t rc = Stage(keys);
        if (rc != KVCM_OK) return rc;
        const int64_t *off = key_off_.host<int64_t>();
        const int64_t n_keys = off[n_req];
        const int64_t ws_bytes = kvcm_b200_start_write_workspace_bytes(n_keys, n_req);
        if (ws_bytes < 0) return KVCM_EC_OUT_OF_LIMIT;
        const size_t per_req = sizeof(int32_t) * n_req, per_key = static_cast<size_t>(n_keys) + 1;
        if (!ws_.Reserve(static_cast<size_t>(ws_bytes), true) || !out_.Reserve(per_req) || !n_new_.Reserve(per_req) ||
            !bits_.Reserve(per_key) || !added_.Reserve(per_key) || !new_off_.Reserve(sizeof(int64_t) * (n_req + 1))) {
            return KVCM_EC_NOSPC;
        }
        rc = kvcm_b200_start_write(index_->handle(), keys_.dev<int64_t>(), key_off_.dev<int64_t>(), n_req, n_keys,
                                   avail_mask_, storage_class, ws_.dev<void>(), ws_bytes, out_.dev<int32_t>(),
                                   bits_.dev<uint8_t>(), n_new_.dev<int32_t>(), added_.dev<uint8_t>(),
                                   new_off_.dev<int64_t>(), nullptr, stream_);
        if (rc != KVCM_OK) return rc;
        if (!out_.ToHost(per_req, stream_) || !bits_.ToHost(per_key - 1, stream_) ||
            !added_.ToHost(per_key - 1, stream_) || !new_off_.ToHost(sizeof(int64_t) * (n_req + 1), stream_)) {
            return KVCM_ER_CUDAMEMCPY_ERROR;
        }
        rc = detail::Sync(stream_);
        if (rc != KVCM_OK) return rc;
        for (int32_t r = 0; r < n_req; ++r) {
            const int32_t first = out_.host<int32_t>()[r];
            if (first >= 0) {
                (*masks)[r] = BlockMask{BlockMaskOffset{static_cast<size_t>(first)}};
            } else {
                BlockMaskVector held(keys[r].size());
                for (size_t i = 0; i < keys[r].size(); ++i) held[i] = bits_.host<uint8_t>()[off[r] + i] != 0;
                (*masks)[r] = BlockMask{std::move(held)};
            }
            for (size_t i = 0; i < keys[r].size(); ++i) {
                if (added_.host<uint8_t>()[off[r] + i] != 0) (*new_keys)[r].push_back(keys[r][i]);
            }
        }
        session_requests_ = n_req;
        session_class_ = storage_class;
        return KVCM_OK;
    }

    // CacheManager::FinishWriteCache (:432-501) for the sessions of the last StartWriteCacheBatch: success_masks[r]
    // is over request r's session keys (an offset, or a vector of exactly that many entries); the keys inside it turn
    // CLS_SERVING, the others lose their location.  (*codes)[r]: KVCM_OK, KVCM_EC_BADARGS for an invalid mask.
    int32_t FinishWriteCacheBatch(const std::vector<BlockMask> &success_masks, std::vector<int32_t> *codes) {
        const int32_t n_req = session_requests_;
        codes->assign(n_req, KVCM_OK);
        if (static_cast<int32_t>(success_masks.size()) != n_req) return KVCM_EC_BADARGS;
        if (n_req == 0) return KVCM_OK;
        const int64_t *new_off = new_off_.host<int64_t>();
        const size_t n_session = static_cast<size_t>(new_off[n_req]);
        if (!bits_.Reserve(n_session + 1) || !out_.Reserve(sizeof(int32_t) * n_req)) return KVCM_EC_NOSPC;
        uint8_t *bits = bits_.host<uint8_t>();
        std::vector<bool> invalid(n_req, false);
        for (int32_t r = 0; r < n_req; ++r) {  // IsBlockMaskValid / IsIndexInMaskRange (cache_location.cc:9-31)
            const size_t mine = static_cast<size_t>(new_off[r + 1] - new_off[r]);
            uint8_t *b = bits + new_off[r];
            if (std::holds_alternative<BlockMaskVector>(success_masks[r])) {
                const auto &v = std::get<BlockMaskVector>(success_masks[r]);
                invalid[r] = v.size() != mine;
                for (size_t j = 0; j < mine; ++j) b[j] = (!invalid[r] && v[j]) ? 1 : 0;
            } else {
                const size_t upto = std::get<BlockMaskOffset>(success_masks[r]);
                invalid[r] = upto > mine;
                for (size_t j = 0; j < mine; ++j) b[j] = (!invalid[r] && j < upto) ? 1 : 0;
            }
        }
        for (int32_t r = 0; r < n_req; ++r) {
            if (invalid[r]) return KVCM_EC_BADARGS;  // as the reference: nothing of an invalid call is applied
        }
        if (!bits_.ToDevice(n_session, stream_)) return KVCM_ER_CUDAMEMCPY_ERROR;
        int32_t rc = kvcm_b200_finish_write(index_->handle(), keys_.dev<int64_t>(), key_off_.dev<int64_t>(), n_req,
                                            added_.dev<uint8_t>(), new_off_.dev<int64_t>(), nullptr,
                                            bits_.dev<uint8_t>(), session_class_, out_.dev<int32_t>(), stream_);
        if (rc != KVCM_OK) return rc;
        if (!out_.ToHost(sizeof(int32_t) * n_req, stream_)) return KVCM_ER_CUDAMEMCPY_ERROR;
        rc = detail::Sync(stream_);
        if (rc == KVCM_OK) std::memcpy(codes->data(), out_.host<int32_t>(), sizeof(int32_t) * n_req);
        session_requests_ = 0;
        return rc;
    }

private:
    // Copies the requests to the device in CSR form.
    int32_t Stage(const std::vector<KeyVector> &keys) {
        const size_t n_req = keys.size();
        size_t n_keys = 0;
        for (const auto &k : keys) n_keys += k.size();
        if (!keys_.Reserve(sizeof(int64_t) * (n_keys + 1)) || !key_off_.Reserve(sizeof(int64_t) * (n_req + 1))) {
            return KVCM_EC_NOSPC;
        }
        int64_t at = 0;
        for (size_t r = 0; r < n_req; ++r) {
            key_off_.host<int64_t>()[r] = at;
            if (!keys[r].empty()) std::memcpy(keys_.host<int64_t>() + at, keys[r].data(), sizeof(int64_t) * keys[r].size());
            at += static_cast<int64_t>(keys[r].size());
        }
        key_off_.host<int64_t>()[n_req] = at;
        if (!keys_.ToDevice(sizeof(int64_t) * n_keys, stream_) ||
            !key_off_.ToDevice(sizeof(int64_t) * (n_req + 1), stream_)) {
            return KVCM_ER_CUDAMEMCPY_ERROR;
        }
        return KVCM_OK;
    }

    GpuBlockIndex *index_;
    uint32_t avail_mask_;
    cudaStream_t stream_;
    detail::Mirror keys_, key_off_, bits_, out_, n_new_, added_, new_off_, ws_;
    int32_t session_requests_ = 0, session_class_ = 0;
};

// Trace replay without eviction, the loop of OptimizerRunner::RunTraces
// (kv_cache_manager/optimizer/manager/optimizer_runner.cc:29-215) for the traces of one instance.
enum class TraceKind : uint8_t { DialogTurn = 0, GetLocation = 1, WriteCache = 2 };

struct ReplayTrace {
    TraceKind kind;
    KeyVector keys;            // DialogTurn: total_keys; GetLocation / WriteCache: keys
    BlockMaskOffset mask = 0;  // GetLocation: number of leading masked (engine-resident) keys
};

// What the reference records per trace (ReadRecord / WriteRecord,
// kv_cache_manager/optimizer/analysis/result_structure.h:15-32).
struct ReplayRecord {
    int32_t external_hit_blocks;
    int32_t internal_hit_blocks;
    int32_t write_blocks;
    int64_t current_cache_blocks;
};

class GpuTraceReplayer {
public:
    explicit GpuTraceReplayer(cudaStream_t stream = nullptr) : stream_(stream) {}

    // Traces in replay (timestamp) order; keys must be prefix-unique chained block keys.
    int32_t RunTraces(const std::vector<ReplayTrace> &traces, std::vector<ReplayRecord> *records) {
        const int32_t n = static_cast<int32_t>(traces.size());
        records->assign(n, ReplayRecord{0, 0, 0, 0});
        if (n == 0) return KVCM_OK;
        int64_t n_keys = 0;
        int32_t rc = Pack(traces, &n_keys);
        if (rc != KVCM_OK) return rc;
        const int64_t ws_bytes = kvcm_b200_replay_workspace_bytes(n_keys);
        if (ws_bytes < 0) return KVCM_EC_BADARGS;
        if (!Outputs(n, 1) || !workspace_.Reserve(static_cast<size_t>(ws_bytes), true)) return KVCM_EC_NOSPC;
        rc = kvcm_b200_replay(keys_.dev<int64_t>(), off_.dev<int64_t>(), kind_.dev<uint8_t>(), mask_.dev<int64_t>(),
                              nullptr, n, n_keys, workspace_.dev<void>(), ws_bytes, ext_.dev<int32_t>(), int_.dev<int32_t>(),
                              wr_.dev<int32_t>(), size_.dev<int64_t>(), nullptr, stream_);
        if (rc != KVCM_OK) return rc;
        rc = Fetch(static_cast<size_t>(n));
        if (rc != KVCM_OK) return rc;
        for (int32_t i = 0; i < n; ++i) (*records)[i] = Record(i);
        return KVCM_OK;
    }

    // The same traces replayed with the "lru" eviction policy once per entry of quota_blocks (the points of a
    // tradeoff curve; quota_capacity * used_percentage in blocks), all in one launch.  evict_batch and precise are
    // eviction_batch_size_per_instance and the eviction mode (false = the rough modes, which evict whole batches;
    // true = INSTANCE_PRECISE).  (*records)[c][t] belongs to quota c and trace t.  leaf_aware = true replays under
    // the "leaf_aware_lru" policy instead (kv_cache_manager/optimizer/eviction_policy/leaf_aware_lru.cc:20-160); the
    // traces' order stands in for their timestamps.
    int32_t RunTracesLru(const std::vector<ReplayTrace> &traces, const std::vector<int64_t> &quota_blocks,
                         int32_t evict_batch, bool precise, std::vector<std::vector<ReplayRecord>> *records,
                         bool leaf_aware = false) {
        const int32_t n = static_cast<int32_t>(traces.size());
        const int32_t n_cfg = static_cast<int32_t>(quota_blocks.size());
        records->assign(n_cfg, std::vector<ReplayRecord>(n, ReplayRecord{0, 0, 0, 0}));
        if (n_cfg == 0) return KVCM_EC_BADARGS;
        if (n == 0) return KVCM_OK;
        int64_t n_keys = 0;
        int32_t rc = Pack(traces, &n_keys);
        if (rc != KVCM_OK) return rc;
        const int64_t ws_bytes = leaf_aware ? kvcm_b200_replay_leaf_lru_workspace_bytes(n_keys, n, n_cfg)
                                            : kvcm_b200_replay_lru_workspace_bytes(n_keys, n_cfg);
        if (ws_bytes < 0) return KVCM_EC_OUT_OF_LIMIT;
        if (!Outputs(n, n_cfg) || !quota_.Reserve(sizeof(int64_t) * n_cfg) ||
            !workspace_.Reserve(static_cast<size_t>(ws_bytes), true)) {
            return KVCM_EC_NOSPC;
        }
        std::memcpy(quota_.host<int64_t>(), quota_blocks.data(), sizeof(int64_t) * n_cfg);
        if (!quota_.ToDevice(sizeof(int64_t) * n_cfg, stream_)) return KVCM_ER_CUDAMEMCPY_ERROR;
        if (leaf_aware) {
            rc = kvcm_b200_replay_leaf_lru(keys_.dev<int64_t>(), off_.dev<int64_t>(), kind_.dev<uint8_t>(),
                                           mask_.dev<int64_t>(), nullptr, nullptr, n, n_keys, quota_.dev<int64_t>(),
                                           n_cfg, evict_batch, precise ? 1 : 0, workspace_.dev<void>(), ws_bytes,
                                           ext_.dev<int32_t>(), int_.dev<int32_t>(), wr_.dev<int32_t>(),
                                           size_.dev<int64_t>(), nullptr, nullptr, stream_);
        } else {
            rc = kvcm_b200_replay_lru(keys_.dev<int64_t>(), off_.dev<int64_t>(), kind_.dev<uint8_t>(),
                                      mask_.dev<int64_t>(), nullptr, n, n_keys, quota_.dev<int64_t>(), n_cfg,
                                      evict_batch, precise ? 1 : 0, workspace_.dev<void>(), ws_bytes,
                                      ext_.dev<int32_t>(), int_.dev<int32_t>(), wr_.dev<int32_t>(),
                                      size_.dev<int64_t>(), nullptr, nullptr, stream_);
        }
        if (rc != KVCM_OK) return rc;
        rc = Fetch(static_cast<size_t>(n) * n_cfg);
        if (rc != KVCM_OK) return rc;
        for (int32_t c = 0; c < n_cfg; ++c) {
            for (int32_t i = 0; i < n; ++i) (*records)[c][i] = Record(static_cast<size_t>(c) * n + i);
        }
        return KVCM_OK;
    }

    // Several instances that share one group quota (OptEvictionManager::EvictByGroupRough / EvictByInstanceRough /
    // EvictByInstancePrecise, kv_cache_manager/optimizer/manager/eviction_manager.cc:86-239): the traces of all
    // instances of the group in replay order, instance_of[t] in [0, n_instances) for each, eviction_mode as in the
    // configuration (1 group rough, 2 instance rough, 3 instance precise), the "lru" policy in every instance, or
    // "leaf_aware_lru" in every instance with leaf_aware = true (the traces' order stands in for their timestamps).
    // (*records)[t].current_cache_blocks is the usage of trace t's own instance; *instance_blocks (optional) receives
    // the usage of every instance at the end.
    int32_t RunTracesLruGroup(const std::vector<ReplayTrace> &traces, const std::vector<int32_t> &instance_of,
                              int32_t n_instances, int64_t quota_blocks, int32_t evict_batch, int32_t eviction_mode,
                              std::vector<ReplayRecord> *records, std::vector<int64_t> *instance_blocks = nullptr,
                              bool leaf_aware = false) {
        if (n_instances <= 0) {
            records->assign(traces.size(), ReplayRecord{0, 0, 0, 0});
            return KVCM_EC_BADARGS;
        }
        const std::vector<uint8_t> policy_of(static_cast<size_t>(n_instances),
                                             leaf_aware ? KVCM_POLICY_LEAF_AWARE_LRU : KVCM_POLICY_LRU);
        return RunTracesPolicyGroup(traces, instance_of, policy_of, {}, quota_blocks, evict_batch, eviction_mode, records,
                                    instance_blocks);
    }

    // The same for a group whose instances name their eviction_policy_type one by one, as the reference's
    // configuration lets them (EvictionPolicyFactory::CreatePolicy per instance,
    // kv_cache_manager/optimizer/eviction_policy/policy_factory.cc:8-47): policy_of[j] is KVCM_POLICY_LRU,
    // KVCM_POLICY_LEAF_AWARE_LRU or KVCM_POLICY_RANDOM_LRU, sample_rate_of[j] the eviction_policy_params.sample_rate
    // of a random_lru instance (empty = the policy's default for all).
    int32_t RunTracesPolicyGroup(const std::vector<ReplayTrace> &traces, const std::vector<int32_t> &instance_of,
                                 const std::vector<uint8_t> &policy_of, const std::vector<double> &sample_rate_of,
                                 int64_t quota_blocks, int32_t evict_batch, int32_t eviction_mode,
                                 std::vector<ReplayRecord> *records, std::vector<int64_t> *instance_blocks = nullptr) {
        const int32_t n = static_cast<int32_t>(traces.size());
        const int32_t n_instances = static_cast<int32_t>(policy_of.size());
        records->assign(n, ReplayRecord{0, 0, 0, 0});
        if (instance_blocks != nullptr) instance_blocks->assign(n_instances, 0);
        if (instance_of.size() != traces.size() || n_instances <= 0 ||
            (!sample_rate_of.empty() && sample_rate_of.size() != policy_of.size())) {
            return KVCM_EC_BADARGS;
        }
        if (n == 0) return KVCM_OK;
        bool queues_only = true;  // every instance "lru": the sweep that keeps no tree
        for (uint8_t policy : policy_of) queues_only = queues_only && policy == KVCM_POLICY_LRU;
        int64_t n_keys = 0;
        int32_t rc = Pack(traces, &n_keys);
        if (rc != KVCM_OK) return rc;
        const int64_t ws_bytes =
            queues_only ? kvcm_b200_replay_lru_group_workspace_bytes(n_keys, 1, n_instances)
                        : kvcm_b200_replay_policy_group_workspace_bytes(n_keys, n, 1, policy_of.data(), n_instances);
        if (ws_bytes < 0) return KVCM_EC_OUT_OF_LIMIT;
        if (!Outputs(n, 1) || !quota_.Reserve(sizeof(int64_t)) || !inst_.Reserve(sizeof(int32_t) * n) ||
            !inst_blocks_.Reserve(sizeof(int64_t) * n_instances) ||
            !workspace_.Reserve(static_cast<size_t>(ws_bytes), true)) {
            return KVCM_EC_NOSPC;
        }
        quota_.host<int64_t>()[0] = quota_blocks;
        std::memcpy(inst_.host<int32_t>(), instance_of.data(), sizeof(int32_t) * n);
        if (!quota_.ToDevice(sizeof(int64_t), stream_) || !inst_.ToDevice(sizeof(int32_t) * n, stream_)) {
            return KVCM_ER_CUDAMEMCPY_ERROR;
        }
        if (!queues_only) {
            rc = kvcm_b200_replay_policy_group(
                keys_.dev<int64_t>(), off_.dev<int64_t>(), kind_.dev<uint8_t>(), mask_.dev<int64_t>(), nullptr, nullptr,
                inst_.dev<int32_t>(), policy_of.data(), sample_rate_of.empty() ? nullptr : sample_rate_of.data(),
                n_instances, n, n_keys, quota_.dev<int64_t>(), 1, evict_batch, eviction_mode, workspace_.dev<void>(),
                ws_bytes, ext_.dev<int32_t>(), int_.dev<int32_t>(), wr_.dev<int32_t>(), size_.dev<int64_t>(), nullptr,
                inst_blocks_.dev<int64_t>(), nullptr, nullptr, stream_);
        } else {
            rc = kvcm_b200_replay_lru_group(keys_.dev<int64_t>(), off_.dev<int64_t>(), kind_.dev<uint8_t>(),
                                            mask_.dev<int64_t>(), nullptr, inst_.dev<int32_t>(), n_instances, n,
                                            n_keys, quota_.dev<int64_t>(), 1, evict_batch, eviction_mode,
                                            workspace_.dev<void>(), ws_bytes, ext_.dev<int32_t>(), int_.dev<int32_t>(),
                                            wr_.dev<int32_t>(), size_.dev<int64_t>(), nullptr,
                                            inst_blocks_.dev<int64_t>(), nullptr, stream_);
        }
        if (rc != KVCM_OK) return rc;
        if (!inst_blocks_.ToHost(sizeof(int64_t) * n_instances, stream_)) return KVCM_ER_CUDAMEMCPY_ERROR;
        rc = Fetch(static_cast<size_t>(n));
        if (rc != KVCM_OK) return rc;
        for (int32_t i = 0; i < n; ++i) (*records)[i] = Record(i);
        if (instance_blocks != nullptr) {
            for (int32_t j = 0; j < n_instances; ++j) (*instance_blocks)[j] = inst_blocks_.host<int64_t>()[j];
        }
        return KVCM_OK;
    }

private:
    // CSR form of the traces in pinned memory, copied to the device.
    int32_t Pack(const std::vector<ReplayTrace> &traces, int64_t *n_keys_out) {
        const int32_t n = static_cast<int32_t>(traces.size());
        int64_t n_keys = 0;
        for (const auto &t : traces) n_keys += static_cast<int64_t>(t.keys.size());
        const size_t off_bytes = sizeof(int64_t) * (n + 1);
        if (!keys_.Reserve(sizeof(int64_t) * (n_keys + 1)) || !off_.Reserve(off_bytes) || !kind_.Reserve(n) ||
            !mask_.Reserve(sizeof(int64_t) * n)) {
            return KVCM_EC_NOSPC;
        }
        int64_t at = 0;
        for (int32_t i = 0; i < n; ++i) {
            off_.host<int64_t>()[i] = at;
            if (!traces[i].keys.empty()) {
                std::memcpy(keys_.host<int64_t>() + at, traces[i].keys.data(), sizeof(int64_t) * traces[i].keys.size());
            }
            at += static_cast<int64_t>(traces[i].keys.size());
            kind_.host<uint8_t>()[i] = static_cast<uint8_t>(traces[i].kind);
            mask_.host<int64_t>()[i] = static_cast<int64_t>(traces[i].mask);
        }
        off_.host<int64_t>()[n] = at;
        if (!keys_.ToDevice(sizeof(int64_t) * n_keys, stream_) || !off_.ToDevice(off_bytes, stream_) ||
            !kind_.ToDevice(n, stream_) || !mask_.ToDevice(sizeof(int64_t) * n, stream_)) {
            return KVCM_ER_CUDAMEMCPY_ERROR;
        }
        *n_keys_out = n_keys;
        return KVCM_OK;
    }
    bool Outputs(int32_t n, int32_t n_cfg) {
        const size_t m = static_cast<size_t>(n) * n_cfg;
        return ext_.Reserve(sizeof(int32_t) * m) && int_.Reserve(sizeof(int32_t) * m) &&
               wr_.Reserve(sizeof(int32_t) * m) && size_.Reserve(sizeof(int64_t) * m);
    }
    int32_t Fetch(size_t m) {
        if (!ext_.ToHost(sizeof(int32_t) * m, stream_) || !int_.ToHost(sizeof(int32_t) * m, stream_) ||
            !wr_.ToHost(sizeof(int32_t) * m, stream_) || !size_.ToHost(sizeof(int64_t) * m, stream_)) {
            return KVCM_ER_CUDAMEMCPY_ERROR;
        }
        return detail::Sync(stream_);
    }
    ReplayRecord Record(size_t i) {
        return ReplayRecord{ext_.host<int32_t>()[i], int_.host<int32_t>()[i], wr_.host<int32_t>()[i],
                            size_.host<int64_t>()[i]};
    }

    cudaStream_t stream_;
    detail::Mirror keys_, off_, kind_, mask_, quota_, ext_, int_, wr_, size_, workspace_, inst_, inst_blocks_;
};

// kv_cache_manager/client/include/common.h:94-116
enum class MemoryType : uint8_t { CPU = 0, GPU = 1 };
struct Iov {
    MemoryType type{MemoryType::GPU};
    void *base{nullptr};
    size_t size{0};
    bool ignore{false};
};
struct BlockBuffer {
    std::vector<Iov> iovs;
};

// One launch for all iovs of a request instead of one cudaMemcpyAsync per Iov.
class IovCopier {
public:
    // through_bounce: a block string in host memory is staged through a device buffer of the same size and crosses
    // PCIe as one copy-engine transfer (a Put and a Get on two streams then use both PCIe directions at full rate);
    // false: the kernel reads / writes the host string itself (no extra device memory).
    explicit IovCopier(cudaStream_t stream = nullptr, bool through_bounce = true)
        : stream_(stream), through_bounce_(through_bounce) {
        cudaEventCreateWithFlags(&staged_, cudaEventDisableTiming);
    }
    IovCopier(const IovCopier &) = delete;
    IovCopier &operator=(const IovCopier &) = delete;
    ~IovCopier() { cudaEventDestroy(staged_); }

    // direction 0: iovs -> block_string (Put), 1: block_string -> iovs (Get).  block_string is device memory, or
    // host memory that is pinned or registered with cudaHostRegister (as the reference's LocalFileSdk does for its
    // mmap); pageable host memory is refused.  Asynchronous on the adapter's stream; the caller keeps the
    // reference's single cudaStreamSynchronize.  *span_bytes = bytes the iov list covers.  Bytes of block_string
    // under ignored, null or empty iovs are never written.  An iov of MemoryType::CPU in ordinary (pageable)
    // memory is moved on the host as the reference moves it and never reaches a kernel; a CPU iov in pinned or
    // registered memory is copied by the kernel like a GPU iov.
    int32_t CopyIovs(const BlockBuffer &buffer, void *block_string, int direction, uint64_t *span_bytes) {
        const int32_t n = static_cast<int32_t>(buffer.iovs.size());
        if (span_bytes) *span_bytes = 0;
        if (n == 0) return KVCM_OK;
        if (direction != 0 && direction != 1) return KVCM_ER_INVALID_PARAMS;
        std::vector<kvcm_b200_iov_t> iovs(n);
        std::vector<uint8_t> on_host(n, 0);  // CPU iovs in pageable memory: moved here, never shown to a kernel
        uint64_t span = 0;
        bool any_on_host = false;
        for (int32_t i = 0; i < n; ++i) {
            iovs[i].type = static_cast<uint8_t>(buffer.iovs[i].type);
            iovs[i].ignore = buffer.iovs[i].ignore ? 1 : 0;
            iovs[i].base = buffer.iovs[i].base;
            iovs[i].size = buffer.iovs[i].size;
            span += buffer.iovs[i].size;
            if (buffer.iovs[i].type == MemoryType::CPU && !buffer.iovs[i].ignore && buffer.iovs[i].base != nullptr &&
                buffer.iovs[i].size > 0) {
                cudaPointerAttributes a{};
                if (cudaPointerGetAttributes(&a, buffer.iovs[i].base) != cudaSuccess) {
                    cudaGetLastError();
                    a.type = cudaMemoryTypeUnregistered;
                }
                if (a.type == cudaMemoryTypeUnregistered) {
                    on_host[i] = 1;
                    any_on_host = true;
                }
            }
        }
        bool host_string = false;
        if (block_string != nullptr) {
            cudaPointerAttributes attr{};
            if (cudaPointerGetAttributes(&attr, block_string) != cudaSuccess) {
                cudaGetLastError();
                return KVCM_ER_INVALID_ADDRESS;
            }
            if (attr.type == cudaMemoryTypeUnregistered) return KVCM_ER_UNSUPPORTED_MEMORY_TYPE;
            host_string = attr.type == cudaMemoryTypeHost;
        }
        if (any_on_host) {
            // What the reference does for MemoryType::CPU (kv_cache_manager/client/src/internal/sdk/
            // local_file_sdk.cc:231-233,339-341): std::memcpy when the block string is host memory too; with a
            // device string the bytes cross with cudaMemcpyAsync on the adapter's stream (the driver stages
            // pageable memory itself).  These iovs are then hidden from the kernel's table.
            if (block_string == nullptr) return KVCM_ER_INVALID_ADDRESS;
            uint64_t at = 0;
            for (int32_t i = 0; i < n; ++i) {
                if (on_host[i]) {
                    uint8_t *in_string = static_cast<uint8_t *>(block_string) + at;
                    if (host_string) {
                        if (direction == 0) {
                            std::memcpy(in_string, iovs[i].base, iovs[i].size);
                        } else {
                            std::memcpy(iovs[i].base, in_string, iovs[i].size);
                        }
                    } else if ((direction == 0 ? cudaMemcpyAsync(in_string, iovs[i].base, iovs[i].size,
                                                                 cudaMemcpyHostToDevice, stream_)
                                               : cudaMemcpyAsync(iovs[i].base, in_string, iovs[i].size,
                                                                 cudaMemcpyDeviceToHost, stream_)) != cudaSuccess) {
                        cudaGetLastError();
                        return KVCM_ER_CUDAMEMCPY_ERROR;
                    }
                    iovs[i].ignore = 1;
                }
                at += iovs[i].size;
            }
        }
        // The pinned segment table and the bounce buffer are reused: wait until the previous call is through.
        if (cudaEventSynchronize(staged_) != cudaSuccess) return KVCM_ER_CUDA_STREAM_SYNCHRONIZE_ERROR;
        if (!segs_.Reserve(sizeof(kvcm_b200_seg_t) * n)) return KVCM_EC_NOSPC;
        void *target = block_string;
        const bool bounce = host_string && through_bounce_ && span > 0;
        if (bounce) {
            if (!bounce_.Reserve(span, true)) return KVCM_EC_NOSPC;
            target = bounce_.dev<void>();
            if (direction == 1 &&
                cudaMemcpyAsync(target, block_string, span, cudaMemcpyHostToDevice, stream_) != cudaSuccess) {
                return KVCM_ER_CUDAMEMCPY_ERROR;
            }
        }
        int32_t n_segs = 0;
        int32_t rc = kvcm_b200_iovs_to_segments(iovs.data(), n, target, direction, segs_.host<kvcm_b200_seg_t>(),
                                                &n_segs, span_bytes);
        if (rc != KVCM_OK) return rc;
        if (!segs_.ToDevice(sizeof(kvcm_b200_seg_t) * n_segs, stream_)) return KVCM_ER_CUDAMEMCPY_ERROR;
        // Device buffers of an engine are 16-byte aligned; an iov list that is not takes the vector kernel.
        uint64_t moved = 0;
        bool aligned = true;
        for (int32_t i = 0; i < n_segs; ++i) {
            const kvcm_b200_seg_t &g = segs_.host<kvcm_b200_seg_t>()[i];
            moved += g.bytes;
            aligned = aligned && ((reinterpret_cast<uintptr_t>(g.dst) | reinterpret_cast<uintptr_t>(g.src)) & 15u) == 0;
        }
        rc = kvcm_b200_copy_segments_sized(segs_.dev<kvcm_b200_seg_t>(), n_segs, aligned ? moved : 0, stream_);
        if (rc == KVCM_OK && bounce && direction == 0) {
            // Back to the host string: one copy per run of bytes that iovs actually filled.
            uint64_t run_begin = 0, at = 0;
            auto flush = [&](uint64_t end) {
                if (end > run_begin && cudaMemcpyAsync(static_cast<uint8_t *>(block_string) + run_begin,
                                                       static_cast<uint8_t *>(target) + run_begin, end - run_begin,
                                                       cudaMemcpyDeviceToHost, stream_) != cudaSuccess) {
                    rc = KVCM_ER_CUDAMEMCPY_ERROR;
                }
            };
            for (int32_t i = 0; i < n; ++i) {
                const bool filled = !iovs[i].ignore && iovs[i].base != nullptr && iovs[i].size > 0;
                if (!filled) {
                    flush(at);
                    run_begin = at + iovs[i].size;
                }
                at += iovs[i].size;
            }
            flush(at);
        }
        cudaEventRecord(staged_, stream_);  // also covers the kernel: the device table may be rewritten after it
        return rc;
    }

private:
    cudaStream_t stream_;
    bool through_bounce_;
    cudaEvent_t staged_ = nullptr;
    detail::Mirror segs_, bounce_;
};

}  // namespace kvcm_b200
