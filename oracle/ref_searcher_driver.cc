// TEST INFRASTRUCTURE ONLY.  A C-callable driver around the REFERENCE's own MetaSearcher over its MetaIndexer and
// local meta backend, compiled from the reference's source files where they lie (oracle/Makefile, target
// ref_searcher): kv_cache_manager/manager/meta_searcher.cc, select_location_policy.cc, cache_location.cc,
// kv_cache_manager/meta/meta_indexer.cc, meta_local_backend.cc, meta_search_cache.cc and the common files they call
// into.  Nothing of the reference is copied here: this file builds the objects the way the reference's own test
// builds them (kv_cache_manager/manager/test/meta_searcher_test.cc:34-79), calls the searcher's public operators and
// hands their results back as plain arrays.  It exists to compare oracle/kvcm_oracle.cc's index, matchers and
// status transitions - the restatement the GPU kernels are compared with - with the reference itself on random
// inputs, beyond the known-answer tables of the reference's tests.
//
// Three symbols the reference's build gets from elsewhere are defined here: the two of its logging back end (alog;
// "nothing is logged") and the meta storage backend factory, whose own source also offers a redis backend (hiredis);
// the factory below makes the reference's local backend only.
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <thread>
#include <utility>
#include <vector>

#include "kv_cache_manager/common/logger.h"
#include "kv_cache_manager/common/request_context.h"
#include "kv_cache_manager/config/meta_indexer_config.h"
#include "kv_cache_manager/config/meta_storage_backend_config.h"
#include "kv_cache_manager/manager/hash_util.h"
#include "kv_cache_manager/manager/meta_searcher.h"
#include "kv_cache_manager/meta/meta_indexer.h"
#include "kv_cache_manager/meta/meta_local_backend.h"
#include "kv_cache_manager/meta/meta_storage_backend_factory.h"

namespace kv_cache_manager {
uint32_t LoggerBroker::base_log_level_ = Logger::LEVEL_UNSET;  // IsLevelEnable() is then false for every level
void LoggerBroker::Log(int, const char *, int, const char *, const char *, ...) {}

std::unique_ptr<MetaStorageBackend>
MetaStorageBackendFactory::CreateAndInitStorageBackend(const std::string &instance_id,
                                                       const std::shared_ptr<MetaStorageBackendConfig> &config) {
    std::unique_ptr<MetaStorageBackend> backend = std::make_unique<MetaLocalBackend>();
    if (backend->Init(instance_id, config) != EC_OK) return nullptr;
    return backend;
}
}  // namespace kv_cache_manager

namespace {

using namespace kv_cache_manager;

struct RefSearcher {
    std::shared_ptr<MetaIndexer> indexer;
    std::shared_ptr<MetaSearcher> searcher;
    std::shared_ptr<RequestContext> context;
    std::map<std::pair<int64_t, int32_t>, std::string> id_of;  // (key, storage type) -> location id
    std::map<std::string, int64_t> key_of;                     // location id -> key
};

std::unique_ptr<SelectLocationPolicy> PolicyFor(const uint32_t *weights) {
    if (weights == nullptr) return std::make_unique<StaticWeightSLPolicy>();
    StaticWeightSLPolicy::WeightArray w{weights[0], weights[1], weights[2], weights[3], weights[4]};
    return std::make_unique<DynamicWeightSLPoliy>(w);
}

BlockMask MaskFor(int32_t mask_kind, int64_t mask_off, const uint8_t *mask_vec, int64_t n) {
    if (mask_kind == 1) return BlockMask(static_cast<BlockMaskOffset>(mask_off));
    BlockMaskVector bits;
    if (mask_kind == 2) {
        bits.resize(static_cast<size_t>(n));
        for (int64_t i = 0; i < n; ++i) bits[static_cast<size_t>(i)] = mask_vec[i] != 0;
    }
    return BlockMask(bits);
}

}  // namespace

extern "C" {

// backend_file: where the local backend keeps its file (a fresh path); empty or null = no storage URI, which is the
// reference's own switch for a local backend that lives in memory only (meta_local_backend.cc:27-34) - with a file it
// rewrites the whole file on every mutation, which makes a large index quadratic to build.
void *kvcm_ref_searcher_create(const char *backend_file, int64_t max_keys) {
    auto backend_config = std::make_shared<MetaStorageBackendConfig>();
    if (backend_file != nullptr && backend_file[0] != 0) {
        backend_config->SetStorageUri(std::string("file://") + backend_file);
    }
    auto config = std::make_shared<MetaIndexerConfig>();
    config->SetMetaStorageBackendConfig(backend_config);
    config->SetMutexShardNum(32);
    config->SetMaxKeyCount(max_keys);
    auto cache = std::make_shared<MetaCachePolicyConfig>();
    cache->SetCapacity(0);
    config->SetMetaCachePolicyConfig(cache);
    auto *h = new RefSearcher();
    h->indexer = std::make_shared<MetaIndexer>();
    if (h->indexer->Init("oracle", config) != EC_OK) {
        delete h;
        return nullptr;
    }
    h->searcher = std::make_shared<MetaSearcher>(h->indexer);
    h->context = std::make_shared<RequestContext>("oracle");
    return h;
}

void kvcm_ref_searcher_destroy(void *handle) { delete static_cast<RefSearcher *>(handle); }

// Gives every key one more location, of storage type `type` (DataStorageType's number), through BatchAddLocation
// (which leaves it WRITING) and then, unless that is what is wanted, BatchUpdateLocationStatus to `status`.
int32_t kvcm_ref_searcher_add(void *handle, const int64_t *keys, int64_t n, int32_t type, int32_t status) {
    auto *h = static_cast<RefSearcher *>(handle);
    MetaSearcher::KeyVector k(keys, keys + n);
    CacheLocationVector locations(static_cast<size_t>(n),
                                  CacheLocation(static_cast<DataStorageType>(type), 1, {LocationSpec("", "")}));
    std::vector<std::string> ids;
    ErrorCode ec = h->searcher->BatchAddLocation(h->context.get(), k, locations, ids);
    if (ec != EC_OK) return static_cast<int32_t>(ec);
    std::vector<std::vector<MetaSearcher::LocationUpdateTask>> tasks(static_cast<size_t>(n));
    for (int64_t i = 0; i < n; ++i) {
        h->id_of[{keys[i], type}] = ids[static_cast<size_t>(i)];
        h->key_of[ids[static_cast<size_t>(i)]] = keys[i];
        tasks[static_cast<size_t>(i)].push_back({ids[static_cast<size_t>(i)], static_cast<CacheLocationStatus>(status)});
    }
    if (status == CLS_WRITING) return 0;
    std::vector<std::vector<ErrorCode>> results;
    return static_cast<int32_t>(h->searcher->BatchUpdateLocationStatus(h->context.get(), k, tasks, results));
}

// MetaSearcher::PrefixMatch: how many locations it returns.  mask_kind 0 none, 1 offset, 2 vector (one byte per key).
int64_t kvcm_ref_searcher_prefix(void *handle, const int64_t *keys, int64_t n, int32_t mask_kind, int64_t mask_off,
                                 const uint8_t *mask_vec, const uint32_t *weights) {
    auto *h = static_cast<RefSearcher *>(handle);
    auto policy = PolicyFor(weights);
    CacheLocationVector out;
    ErrorCode ec = h->searcher->PrefixMatch(h->context.get(), MetaSearcher::KeyVector(keys, keys + n),
                                            MaskFor(mask_kind, mask_off, mask_vec, n), out, policy.get());
    return ec == EC_OK ? static_cast<int64_t>(out.size()) : -static_cast<int64_t>(ec);
}

// The reference's CPU path for a batch of requests: per request the loop of GenKeyVector
// (kv_cache_manager/manager/cache_manager.cc:76-87) around the reference's hashInt64Array, then
// MetaSearcher::PrefixMatch without a mask; matched_out[r] = how many locations it returned.  Requests are dealt to
// `threads` host threads (the index takes concurrent readers: its entries sit behind sharded mutexes); every call
// of PrefixMatch gets a request context of its own.
int32_t kvcm_ref_searcher_prefix_batch(void *handle, const int64_t *tokens, const int64_t *tok_off, int64_t n_req,
                                       int32_t block_size, const uint32_t *weights, int32_t threads,
                                       int32_t *matched_out) {
    auto *h = static_cast<RefSearcher *>(handle);
    if (block_size <= 0 || threads <= 0) return static_cast<int32_t>(EC_BADARGS);
    auto work = [&](int32_t tid) {
        auto policy = PolicyFor(weights);
        for (int64_t r = tid; r < n_req; r += threads) {
            const int64_t *tok = tokens + tok_off[r];
            const int64_t blocks = (tok_off[r + 1] - tok_off[r]) / block_size;
            MetaSearcher::KeyVector keys(static_cast<size_t>(blocks));
            int64_t hash = 0;
            for (int64_t b = 0; b < blocks; ++b) {
                hash = hashInt64Array(hash, tok + b * block_size, tok + (b + 1) * block_size);
                keys[static_cast<size_t>(b)] = hash;
            }
            RequestContext context("oracle");
            CacheLocationVector out;
            h->searcher->PrefixMatch(&context, keys, BlockMask(BlockMaskVector{}), out, policy.get());
            matched_out[r] = static_cast<int32_t>(out.size());
        }
    };
    std::vector<std::thread> pool;
    for (int32_t t = 1; t < threads; ++t) pool.emplace_back(work, t);
    work(0);
    for (auto &t : pool) t.join();
    return 0;
}

// The sliding-window configuration's CPU path per request: GenKeyVector, PrefixMatch and - where the request has at
// least sw_size keys, which the reference asserts - ReverseRollSlideWindowMatch, on `threads` host threads.
// matched_out[r] as above; base_out[r] = where the non-empty entries of the window answer start (-1 none, -2 fewer
// keys than the window).
int32_t kvcm_ref_searcher_window_batch(void *handle, const int64_t *tokens, const int64_t *tok_off, int64_t n_req,
                                       int32_t block_size, int32_t sw, const uint32_t *weights, int32_t threads,
                                       int32_t *matched_out, int32_t *base_out) {
    auto *h = static_cast<RefSearcher *>(handle);
    if (block_size <= 0 || threads <= 0 || sw <= 0) return static_cast<int32_t>(EC_BADARGS);
    auto work = [&](int32_t tid) {
        auto policy = PolicyFor(weights);
        for (int64_t r = tid; r < n_req; r += threads) {
            const int64_t *tok = tokens + tok_off[r];
            const int64_t blocks = (tok_off[r + 1] - tok_off[r]) / block_size;
            MetaSearcher::KeyVector keys(static_cast<size_t>(blocks));
            int64_t hash = 0;
            for (int64_t b = 0; b < blocks; ++b) {
                hash = hashInt64Array(hash, tok + b * block_size, tok + (b + 1) * block_size);
                keys[static_cast<size_t>(b)] = hash;
            }
            RequestContext context("oracle");
            CacheLocationVector out;
            h->searcher->PrefixMatch(&context, keys, BlockMask(BlockMaskVector{}), out, policy.get());
            matched_out[r] = static_cast<int32_t>(out.size());
            base_out[r] = -2;
            if (blocks < sw) continue;
            CacheLocationVector window;
            h->searcher->ReverseRollSlideWindowMatch(&context, keys, sw, window, policy.get());
            base_out[r] = -1;
            for (size_t i = 0; i < window.size(); ++i) {
                if (!window[i].id().empty()) {
                    base_out[r] = static_cast<int32_t>(i);
                    break;
                }
            }
        }
    };
    std::vector<std::thread> pool;
    for (int32_t t = 1; t < threads; ++t) pool.emplace_back(work, t);
    work(0);
    for (auto &t : pool) t.join();
    return 0;
}

// MetaSearcher::ReverseRollSlideWindowMatch.  The reference returns one entry per key, empty but for the matched
// window: the result here is where the non-empty entries start (-1: none; the reference's error code negated when
// it fails), *count_out how many there are.  The reference asserts keys.size() >= sw_size > 0; such calls are not
// made and answer -1000.
int64_t kvcm_ref_searcher_sw(void *handle, const int64_t *keys, int64_t n, int32_t sw, const uint32_t *weights,
                             int64_t *count_out) {
    auto *h = static_cast<RefSearcher *>(handle);
    if (sw <= 0 || n < sw) return -1000;
    auto policy = PolicyFor(weights);
    CacheLocationVector out;
    ErrorCode ec = h->searcher->ReverseRollSlideWindowMatch(h->context.get(), MetaSearcher::KeyVector(keys, keys + n),
                                                            sw, out, policy.get());
    if (ec != EC_OK) return -static_cast<int64_t>(ec);
    int64_t base = -1, count = 0;
    for (size_t i = 0; i < out.size(); ++i) {
        if (out[i].id().empty()) continue;
        if (base < 0) base = static_cast<int64_t>(i);
        ++count;
    }
    if (count_out != nullptr) *count_out = count;
    return base;
}

// Per key: servable_out = BatchGetBestLocation found a location the policy would serve; nonempty_out =
// BatchGetLocation returned a non-empty location map.
int32_t kvcm_ref_searcher_batch_get(void *handle, const int64_t *keys, int64_t n, const uint32_t *weights,
                                    uint8_t *servable_out, uint8_t *nonempty_out) {
    auto *h = static_cast<RefSearcher *>(handle);
    auto policy = PolicyFor(weights);
    MetaSearcher::KeyVector k(keys, keys + n);
    CacheLocationVector best;
    ErrorCode ec = h->searcher->BatchGetBestLocation(h->context.get(), k, best, policy.get());
    if (ec != EC_OK || static_cast<int64_t>(best.size()) != n) return ec != EC_OK ? static_cast<int32_t>(ec) : -1;
    for (int64_t i = 0; i < n; ++i) servable_out[i] = best[static_cast<size_t>(i)].id().empty() ? 0 : 1;
    std::vector<CacheLocationMap> maps;
    ec = h->searcher->BatchGetLocation(h->context.get(), k, BlockMask(BlockMaskVector{}), maps);
    if (ec != EC_OK || static_cast<int64_t>(maps.size()) != n) return ec != EC_OK ? static_cast<int32_t>(ec) : -1;
    for (int64_t i = 0; i < n; ++i) nonempty_out[i] = maps[static_cast<size_t>(i)].empty() ? 0 : 1;
    return 0;
}

// What CacheManager::FilterWriteCache looks at per key (kv_cache_manager/manager/cache_manager.cc:589-635; the
// CacheManager itself needs the RPC stack and is not compiled here): the location map BatchGetLocation returns, and
// whether the reference's own policy object says it exists for a write.
int32_t kvcm_ref_searcher_write_view(void *handle, const int64_t *keys, int64_t n, const uint32_t *weights,
                                     uint8_t *exists_for_write_out, uint8_t *nonempty_out) {
    auto *h = static_cast<RefSearcher *>(handle);
    auto policy = PolicyFor(weights);
    MetaSearcher::KeyVector k(keys, keys + n);
    std::vector<CacheLocationMap> maps;
    ErrorCode ec = h->searcher->BatchGetLocation(h->context.get(), k, BlockMask(static_cast<BlockMaskOffset>(0)), maps);
    if (ec != EC_OK || static_cast<int64_t>(maps.size()) != n) return ec != EC_OK ? static_cast<int32_t>(ec) : -1;
    for (int64_t i = 0; i < n; ++i) {
        exists_for_write_out[i] = policy->ExistsForWrite(maps[static_cast<size_t>(i)]) ? 1 : 0;
        nonempty_out[i] = maps[static_cast<size_t>(i)].empty() ? 0 : 1;
    }
    return 0;
}

// One task per key on the key's location of storage type types[i]: op 0 BatchUpdateLocationStatus (to
// new_status[i]), 1 BatchCASLocationStatus (expected[i] -> new_status[i]), 2 BatchCADLocationStatus (delete when
// expected[i]), 3 BatchDeleteLocation.  results[i] = the ErrorCode of the task.  Returns the call's own ErrorCode.
int32_t kvcm_ref_searcher_status(void *handle, int32_t op, const int64_t *keys, int64_t n, const int32_t *types,
                                 const int32_t *expected, const int32_t *new_status, int32_t *results) {
    auto *h = static_cast<RefSearcher *>(handle);
    MetaSearcher::KeyVector k(keys, keys + n);
    std::vector<std::string> ids(static_cast<size_t>(n));
    for (int64_t i = 0; i < n; ++i) {
        auto it = h->id_of.find({keys[i], types[i]});
        ids[static_cast<size_t>(i)] = it != h->id_of.end() ? it->second : std::string("no-such-location");
    }
    ErrorCode ec = EC_OK;
    std::vector<std::vector<ErrorCode>> batch;
    if (op == 0) {
        std::vector<std::vector<MetaSearcher::LocationUpdateTask>> tasks(static_cast<size_t>(n));
        for (int64_t i = 0; i < n; ++i) {
            tasks[static_cast<size_t>(i)].push_back(
                {ids[static_cast<size_t>(i)], static_cast<CacheLocationStatus>(new_status[i])});
        }
        ec = h->searcher->BatchUpdateLocationStatus(h->context.get(), k, tasks, batch);
    } else if (op == 1) {
        std::vector<std::vector<MetaSearcher::LocationCASTask>> tasks(static_cast<size_t>(n));
        for (int64_t i = 0; i < n; ++i) {
            tasks[static_cast<size_t>(i)].push_back({ids[static_cast<size_t>(i)],
                                                     static_cast<CacheLocationStatus>(expected[i]),
                                                     static_cast<CacheLocationStatus>(new_status[i])});
        }
        ec = h->searcher->BatchCASLocationStatus(h->context.get(), k, tasks, batch);
    } else if (op == 2) {
        std::vector<std::vector<MetaSearcher::LocationCADTask>> tasks(static_cast<size_t>(n));
        for (int64_t i = 0; i < n; ++i) {
            tasks[static_cast<size_t>(i)].push_back(
                {ids[static_cast<size_t>(i)], static_cast<CacheLocationStatus>(expected[i])});
        }
        ec = h->searcher->BatchCADLocationStatus(h->context.get(), k, tasks, batch);
    } else {
        std::vector<ErrorCode> flat;
        ec = h->searcher->BatchDeleteLocation(h->context.get(), k, ids, flat);
        for (int64_t i = 0; i < n; ++i) {
            results[i] = i < static_cast<int64_t>(flat.size()) ? static_cast<int32_t>(flat[static_cast<size_t>(i)]) : -1;
        }
        return static_cast<int32_t>(ec);
    }
    for (int64_t i = 0; i < n; ++i) {
        const bool have = i < static_cast<int64_t>(batch.size()) && !batch[static_cast<size_t>(i)].empty();
        results[i] = have ? static_cast<int32_t>(batch[static_cast<size_t>(i)][0]) : -1;
    }
    return static_cast<int32_t>(ec);
}

}  // extern "C"
