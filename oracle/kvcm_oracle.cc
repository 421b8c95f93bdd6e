// CPU oracle for the KVCM hot path.  TEST INFRASTRUCTURE ONLY.
//
// This file restates, on the CPU, the algorithms of alibaba/tair-kvcache that the
// CUDA library replaces.  It exists to check the CUDA results and to be timed as the
// CPU baseline; the product never links, loads or calls it.  Every function names the
// reference file:line it follows.
//
// Parity pins:
//   * hash chain      - checked against the reference's own header compiled as-is
//                       (oracle/_ref/libkvcm_ref_hash.so, built by oracle/Makefile) and
//                       against tests/golden/hash_kat.json generated from that build.
//   * prefix / SW / batch-get match - checked against the known-answer tables of the
//                       reference's unit tests (tests/golden/match_kat.json).
//   * gather/scatter  - checked against the index rule of the reference's Triton
//                       kernels restated as Python loops in its own test file.
//   * CRC-32          - checked against the three known answers of the reference's test.
//
// Build: make -C oracle   (g++ -O2 -shared -fPIC -pthread)

#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstring>
#include <functional>
#include <list>
#include <memory>
#include <set>
#include <thread>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace {

// ---------------------------------------------------------------------------------
// helpers
// ---------------------------------------------------------------------------------
template <class F>
void ParallelFor(int64_t n, int threads, F &&body) {
    if (threads <= 1 || n <= 1) {
        for (int64_t i = 0; i < n; ++i) body(i);
        return;
    }
    std::atomic<int64_t> next{0};
    std::vector<std::thread> pool;
    pool.reserve(threads);
    for (int t = 0; t < threads; ++t) {
        pool.emplace_back([&] {
            // small dynamic chunks: request lengths are ragged
            for (;;) {
                int64_t i = next.fetch_add(1, std::memory_order_relaxed);
                if (i >= n) break;
                body(i);
            }
        });
    }
    for (auto &th : pool) th.join();
}

// kv_cache_manager/manager/hash_util.h:8-12 (hashInt64Func).  std::hash<int64_t> is the
// identity in libstdc++, the reference's toolchain.  The signed shifts of the original
// are written out on unsigned words so that nothing here is undefined behaviour:
// `hash << 12` keeps the low 64 bits, `hash >> 32` is an arithmetic (sign-extending) shift.
inline int64_t HashStep(int64_t hash, int64_t value) {
    const uint64_t h = static_cast<uint64_t>(hash);
    const uint64_t sra32 = static_cast<uint64_t>(hash >> 32);  // arithmetic on gcc
    const uint64_t mixed = static_cast<uint64_t>(value) + 0x9e3779b97f4a7c15ULL + (h << 12) + sra32;
    return static_cast<int64_t>(h ^ mixed);
}

// One location of a block: kv_cache_manager/manager/cache_location.h:44-50 (status),
// kv_cache_manager/data_storage/storage_config.h:8-13 (storage type).
struct Loc {
    int32_t status;
    int32_t type;
};

// kv_cache_manager/meta/meta_local_backend.h:60 keeps an unordered_map keyed by the int64
// block key; the value's "__uri__" field is the JSON of the location map.  Here the value
// is the decoded location list; an entry with zero locations models an empty location map.
struct OracleIndex {
    std::unordered_map<int64_t, std::vector<Loc>> table;
};

// kv_cache_manager/manager/select_location_policy.cc:40-48 (StaticWeightSLPolicy::GetWeight):
// weight = table[type] when type indexes the table, else DEFAULT (1).
inline uint32_t Weight(int32_t type, const uint32_t *weights, int n_weights) {
    if (type >= 0 && type < n_weights) return weights[type];
    return 1u;
}

// kv_cache_manager/manager/select_location_policy.cc:8-27 (SelectForMatch != nullptr):
// some location is CLS_SERVING (3) and has weight > 0.
inline bool Servable(const std::vector<Loc> &locs, const uint32_t *weights, int n_weights) {
    for (const Loc &l : locs) {
        if (l.status == 3 && Weight(l.type, weights, n_weights) > 0) return true;
    }
    return false;
}

// kv_cache_manager/manager/select_location_policy.cc:29-38 (ExistsForWrite).
inline bool ExistsForWrite(const std::vector<Loc> &locs, const uint32_t *weights, int n_weights) {
    for (const Loc &l : locs) {
        if (l.status != 0 && Weight(l.type, weights, n_weights) > 0) return true;
    }
    return false;
}

// kv_cache_manager/manager/cache_location.cc:9-21 (IsIndexInMaskRange).
// mask_kind 0: bool vector (mask_vec, mask_len); 1: offset (mask_off).
inline bool Masked(int mask_kind, const uint8_t *mask_vec, int64_t mask_len, int64_t mask_off, int64_t i) {
    if (mask_kind == 0) return i < mask_len ? mask_vec[i] != 0 : false;
    return i < mask_off;
}

// The per-key outcome of MetaIndexer::Get as the matchers see it
// (kv_cache_manager/meta/meta_indexer.cc:695-698,735-738): a missing key and a key whose
// "__uri__" is empty both read as EC_NOENT.  The oracle stores decoded location lists, so
// only a missing key is EC_NOENT; an existing key with an empty list is EC_OK with an
// empty location map (meta_searcher.cc:99-103 then stops the prefix match).
inline const std::vector<Loc> *Get(const OracleIndex *ix, int64_t key) {
    auto it = ix->table.find(key);
    return it == ix->table.end() ? nullptr : &it->second;
}

// kv_cache_manager/manager/meta_searcher.cc:120-145 + 74-118 (PrefixMatch).
int64_t PrefixMatchOne(const OracleIndex *ix, const int64_t *keys, int64_t n, int mask_kind,
                       const uint8_t *mask_vec, int64_t mask_len, int64_t mask_off, const uint32_t *w, int nw) {
    std::vector<int64_t> query;
    query.reserve(n);
    for (int64_t i = 0; i < n; ++i) {
        if (!Masked(mask_kind, mask_vec, mask_len, mask_off, i)) query.push_back(keys[i]);
    }
    int64_t len = 0;
    for (int64_t k : query) {
        const std::vector<Loc> *locs = Get(ix, k);
        if (locs == nullptr) break;           // Get != EC_OK
        if (locs->empty()) break;             // location_map.empty()
        if (!Servable(*locs, w, nw)) break;   // SelectForMatch == nullptr
        ++len;
    }
    return len;
}

// kv_cache_manager/manager/meta_searcher.cc:196-265 (ReverseRollSlideWindowMatch), kept in
// its two phases: existence over the whole window first, then the servable predicate.
int64_t SwMatchOne(const OracleIndex *ix, const int64_t *keys, int64_t n, int64_t sw, const uint32_t *w, int nw) {
    for (int64_t base = n - sw; base >= 0;) {
        bool is_match = false;
        for (int64_t off = 0; off < sw; ++off) {
            if (Get(ix, keys[base + off]) == nullptr) {
                base -= sw - off;
                is_match = false;
                break;
            }
            is_match = true;
        }
        if (!is_match) continue;
        for (int64_t off = 0; off < sw; ++off) {
            const std::vector<Loc> *locs = Get(ix, keys[base + off]);
            if (locs->empty() || !Servable(*locs, w, nw)) {
                base -= sw - off;
                is_match = false;
                break;
            }
        }
        if (is_match) return base;
    }
    return -1;
}

}  // namespace

extern "C" {

// ---------------------------------------------------------------------------------
// (2a) chained block hash
// ---------------------------------------------------------------------------------

int64_t kvcm_oracle_hash_step(int64_t hash, int64_t value) { return HashStep(hash, value); }

// kv_cache_manager/manager/cache_manager.cc:76-87 (GenKeyVector): n = tokens/block_size keys,
// the state is carried across blocks, the trailing partial block is dropped.
int64_t kvcm_oracle_gen_key_vector_i64(const int64_t *tokens, int64_t n_tokens, int64_t block_size, int64_t *keys) {
    if (block_size <= 0) return 0;
    const int64_t total_blocks = n_tokens / block_size;
    int64_t hash = 0;
    for (int64_t b = 0; b < total_blocks; ++b) {
        const int64_t *p = tokens + b * block_size;
        for (int64_t t = 0; t < block_size; ++t) hash = HashStep(hash, p[t]);
        keys[b] = hash;
    }
    return total_blocks;
}

// Same loop over uint32 token ids, zero-extended to the int64 the wire format carries
// (kv_cache_manager/protocol/protobuf/meta_service.proto:199).
int64_t kvcm_oracle_gen_key_vector_u32(const uint32_t *tokens, int64_t n_tokens, int64_t block_size, int64_t *keys) {
    if (block_size <= 0) return 0;
    const int64_t total_blocks = n_tokens / block_size;
    int64_t hash = 0;
    for (int64_t b = 0; b < total_blocks; ++b) {
        const uint32_t *p = tokens + b * block_size;
        for (int64_t t = 0; t < block_size; ++t) hash = HashStep(hash, static_cast<int64_t>(p[t]));
        keys[b] = hash;
    }
    return total_blocks;
}

// kv_cache_manager/optimizer/trace_converter/trace_util.cc:47-56 (ApplyPrefixHash): one key per id.
void kvcm_oracle_apply_prefix_hash(const int64_t *ids, int64_t n, int64_t *keys) {
    int64_t hash = 0;
    for (int64_t i = 0; i < n; ++i) {
        hash = HashStep(hash, ids[i]);
        keys[i] = hash;
    }
}

// Batch of requests in CSR form: request r owns tokens[tok_off[r], tok_off[r+1]) and writes
// keys[key_off[r], key_off[r] + len/block_size).  One GenKeyVector per request.
void kvcm_oracle_hash_blocks_u32(const uint32_t *tokens, const int64_t *tok_off, int64_t n_req, int64_t block_size,
                                 int64_t *keys, const int64_t *key_off, int threads) {
    ParallelFor(n_req, threads, [&](int64_t r) {
        kvcm_oracle_gen_key_vector_u32(tokens + tok_off[r], tok_off[r + 1] - tok_off[r], block_size, keys + key_off[r]);
    });
}

void kvcm_oracle_hash_blocks_i64(const int64_t *tokens, const int64_t *tok_off, int64_t n_req, int64_t block_size,
                                 int64_t *keys, const int64_t *key_off, int threads) {
    ParallelFor(n_req, threads, [&](int64_t r) {
        kvcm_oracle_gen_key_vector_i64(tokens + tok_off[r], tok_off[r + 1] - tok_off[r], block_size, keys + key_off[r]);
    });
}

// ---------------------------------------------------------------------------------
// (2b) block index + matchers
// ---------------------------------------------------------------------------------

void *kvcm_oracle_index_create() { return new OracleIndex(); }
void kvcm_oracle_index_destroy(void *h) { delete static_cast<OracleIndex *>(h); }
int64_t kvcm_oracle_index_size(void *h) { return static_cast<int64_t>(static_cast<OracleIndex *>(h)->table.size()); }
void kvcm_oracle_index_reserve(void *h, int64_t n) { static_cast<OracleIndex *>(h)->table.reserve(n); }

// Replace the location list of each key: key i owns statuses/types[loc_off[i], loc_off[i+1]).
void kvcm_oracle_index_put(void *h, const int64_t *keys, int64_t n, const int64_t *loc_off, const int32_t *statuses,
                           const int32_t *types) {
    auto *ix = static_cast<OracleIndex *>(h);
    for (int64_t i = 0; i < n; ++i) {
        std::vector<Loc> locs;
        for (int64_t j = loc_off[i]; j < loc_off[i + 1]; ++j) locs.push_back({statuses[j], types[j]});
        ix->table[keys[i]] = std::move(locs);
    }
}

// Every key gets one location of the given status and storage type.
void kvcm_oracle_index_put_uniform(void *h, const int64_t *keys, int64_t n, int32_t status, int32_t type) {
    auto *ix = static_cast<OracleIndex *>(h);
    for (int64_t i = 0; i < n; ++i) ix->table[keys[i]] = std::vector<Loc>{{status, type}};
}

void kvcm_oracle_index_erase(void *h, const int64_t *keys, int64_t n) {
    auto *ix = static_cast<OracleIndex *>(h);
    for (int64_t i = 0; i < n; ++i) ix->table.erase(keys[i]);
}

// Prefix match of one request; returns the matched length in keys (of the unmasked keys).
int64_t kvcm_oracle_prefix_match(void *h, const int64_t *keys, int64_t n, int mask_kind, const uint8_t *mask_vec,
                                 int64_t mask_len, int64_t mask_off, const uint32_t *weights, int n_weights) {
    return PrefixMatchOne(static_cast<OracleIndex *>(h), keys, n, mask_kind, mask_vec, mask_len, mask_off, weights,
                          n_weights);
}

// Sliding-window match of one request.  *base_out = start of the rightmost fully servable
// window of `sw` keys, or -1.  Return value follows the guard of
// kv_cache_manager/manager/cache_manager.cc:993-997: EC_BADARGS (6) when n < sw or sw < 0.
// sw == 0 never terminates in the reference (meta_searcher.cc:218-229 makes no progress);
// the oracle rejects it with EC_BADARGS as the replacement must.
int32_t kvcm_oracle_sw_match(void *h, const int64_t *keys, int64_t n, int64_t sw, const uint32_t *weights,
                             int n_weights, int64_t *base_out) {
    *base_out = -1;
    if (sw <= 0 || n < sw) return 6;
    *base_out = SwMatchOne(static_cast<OracleIndex *>(h), keys, n, sw, weights, n_weights);
    return 0;
}

// Location-status transitions, one task per key.  Restates the modifiers of
//   MetaSearcher::BatchUpdateLocationStatus  kv_cache_manager/manager/meta_searcher.cc:410-487
//   MetaSearcher::BatchCASLocationStatus     kv_cache_manager/manager/meta_searcher.cc:489-580
//   MetaSearcher::BatchCADLocationStatus     kv_cache_manager/manager/meta_searcher.cc:582-717
//   MetaSearcher::BatchDeleteLocation        kv_cache_manager/manager/meta_searcher.cc:719-820
// over BlockCacheLocationsMeta::UpdateLocationStatus / GetLocationStatus / DeleteLocation
// (kv_cache_manager/manager/cache_location.cc:60-82).  The reference names a location by its id string; here
// the location of key i is named by its storage type types[i] (the first location of that type in the key's
// list).  expected[i] < 0: no comparison (update / delete).  new_status[i] == -1: the location is deleted the
// way BatchCADLocationStatus does it - a key whose location map becomes empty is removed (MA_DELETE, :689-691);
// new_status[i] == -2: the way BatchDeleteLocation does it - a missing key is skipped with EC_OK (:741-744) and
// a key whose last location goes stays, with an empty map (MA_OK, :783-786).  results[i]: 0 EC_OK, 2 EC_NOENT
// (no such key - the modifier's get_ec - or no such location), 16 EC_MISMATCH.
void kvcm_oracle_index_update_status(void *h, const int64_t *keys, int64_t n, const int32_t *types,
                                     const int32_t *expected, const int32_t *new_status, int32_t *results) {
    auto *ix = static_cast<OracleIndex *>(h);
    for (int64_t i = 0; i < n; ++i) {
        auto it = ix->table.find(keys[i]);
        if (it == ix->table.end()) {
            results[i] = new_status[i] == -2 ? 0 : 2;
            continue;
        }
        std::vector<Loc> &locs = it->second;
        size_t at = 0;
        while (at < locs.size() && locs[at].type != types[i]) ++at;
        if (at == locs.size()) {
            results[i] = 2;
            // compare-and-delete drops a key whose map is empty whatever its tasks did (:689-692): a key that an
            // earlier BatchDeleteLocation left behind empty goes here, with the task answering EC_NOENT
            if (new_status[i] == -1 && locs.empty()) ix->table.erase(it);
            continue;
        }
        if (expected[i] >= 0 && locs[at].status != expected[i]) {
            results[i] = 16;
            continue;
        }
        results[i] = 0;
        if (new_status[i] < 0) {
            locs.erase(locs.begin() + static_cast<std::ptrdiff_t>(at));
            if (locs.empty() && new_status[i] == -1) ix->table.erase(it);
        } else {
            locs[at].status = new_status[i];
        }
    }
}

// The location list of one key: returns its length (at most `room` entries are written), -1 for a missing key.
int64_t kvcm_oracle_index_get(void *h, int64_t key, int32_t *statuses, int32_t *types, int64_t room) {
    const std::vector<Loc> *locs = Get(static_cast<OracleIndex *>(h), key);
    if (locs == nullptr) return -1;
    for (size_t j = 0; j < locs->size() && static_cast<int64_t>(j) < room; ++j) {
        statuses[j] = (*locs)[j].status;
        types[j] = (*locs)[j].type;
    }
    return static_cast<int64_t>(locs->size());
}

// kv_cache_manager/manager/meta_searcher.cc:147-194 (BatchGetBestLocation) and
// kv_cache_manager/manager/cache_manager.cc:589-635 (what FilterWriteCache reads from
// BatchGetLocation).  flags[i]: bit0 servable (a location would be returned), bit1 key
// exists, bit2 location map non-empty, bit3 ExistsForWrite.
void kvcm_oracle_batch_get(void *h, const int64_t *keys, int64_t n, const uint32_t *weights, int n_weights,
                           uint8_t *flags) {
    auto *ix = static_cast<OracleIndex *>(h);
    for (int64_t i = 0; i < n; ++i) {
        const std::vector<Loc> *locs = Get(ix, keys[i]);
        uint8_t f = 0;
        if (locs != nullptr) {
            f |= 2;
            if (!locs->empty()) f |= 4;
            if (Servable(*locs, weights, n_weights)) f |= 1;
            if (ExistsForWrite(*locs, weights, n_weights)) f |= 8;
        }
        flags[i] = f;
    }
}

// kv_cache_manager/manager/cache_manager.cc:589-635 (FilterWriteCache).  Returns 1 when the
// result is an offset mask (*offset_out = first key without a writable location), 0 when it
// is a bool vector (mask_out[i] = location map non-empty).  n_new_out = number of keys that
// still have to be written.
int32_t kvcm_oracle_filter_write(void *h, const int64_t *keys, int64_t n, const uint32_t *weights, int n_weights,
                                 int64_t *offset_out, uint8_t *mask_out, int64_t *n_new_out) {
    auto *ix = static_cast<OracleIndex *>(h);
    std::vector<uint8_t> exists(n), nonempty(n);
    for (int64_t i = 0; i < n; ++i) {
        const std::vector<Loc> *locs = Get(ix, keys[i]);
        exists[i] = locs != nullptr && ExistsForWrite(*locs, weights, n_weights);
        nonempty[i] = locs != nullptr && !locs->empty();
    }
    int64_t first_empty = 0;
    while (first_empty < n && exists[first_empty]) ++first_empty;
    bool only_prefix = true;
    for (int64_t i = first_empty; i < n; ++i) only_prefix = only_prefix && !exists[i];
    if (only_prefix) {
        *offset_out = first_empty;
        *n_new_out = n - first_empty;
        return 1;
    }
    int64_t n_new = 0;
    for (int64_t i = 0; i < n; ++i) {
        mask_out[i] = nonempty[i];
        if (!nonempty[i]) ++n_new;
    }
    *offset_out = -1;
    *n_new_out = n_new;
    return 0;
}

// Batched matchers over CSR keys (request r owns keys[key_off[r], key_off[r+1])).
// mask_off may be null (nothing masked); otherwise request r masks its first mask_off[r] keys
// (BlockMaskOffset form, the one the vLLM connector sends).
void kvcm_oracle_prefix_match_batch(void *h, const int64_t *keys, const int64_t *key_off, int64_t n_req,
                                    const int64_t *mask_off, const uint32_t *weights, int n_weights, int32_t *len_out,
                                    int threads) {
    auto *ix = static_cast<OracleIndex *>(h);
    ParallelFor(n_req, threads, [&](int64_t r) {
        len_out[r] = static_cast<int32_t>(PrefixMatchOne(ix, keys + key_off[r], key_off[r + 1] - key_off[r], 1, nullptr,
                                                         0, mask_off ? mask_off[r] : 0, weights, n_weights));
    });
}

// base_out[r] = window start, -1 = no window, -2 = bad arguments for this request.
void kvcm_oracle_sw_match_batch(void *h, const int64_t *keys, const int64_t *key_off, int64_t n_req, int64_t sw,
                                const uint32_t *weights, int n_weights, int32_t *base_out, int threads) {
    auto *ix = static_cast<OracleIndex *>(h);
    ParallelFor(n_req, threads, [&](int64_t r) {
        const int64_t n = key_off[r + 1] - key_off[r];
        if (sw <= 0 || n < sw) {
            base_out[r] = -2;
            return;
        }
        base_out[r] = static_cast<int32_t>(SwMatchOne(ix, keys + key_off[r], n, sw, weights, n_weights));
    });
}

// ---------------------------------------------------------------------------------
// (1) paged-KV gather / scatter
// ---------------------------------------------------------------------------------

// kv_cache_manager/py_connector/kernel/batch_gather_scatter_helper.py:46-98 (gather) and
// :152-205 (scatter), in bytes: a pool is [pool_rows, row_bytes]; block b moves its
// rows_per_block rows row_idx[b][t] to/from staging slot slot_idx[b], whose layout is
// [n_pools, rows_per_block, row_bytes].  A row is one token (the reference's form) or one
// engine page (page-table form); the arithmetic is the same.
// dir 0 = gather (pool -> staging), 1 = scatter (staging -> pool).
// Rows outside [0, pool_rows) and slots outside [0, n_slots) are skipped and counted in the
// return value (the reference's batch kernels do not check; its legacy kernels skip,
// gather_scatter_helper.py:36-38,87-89).
int64_t kvcm_oracle_move_rows(uint8_t *const *pools, int32_t n_pools, uint8_t *staging, int64_t n_slots,
                              const int32_t *row_idx, const int32_t *slot_idx, int64_t n_blocks,
                              int64_t rows_per_block, int64_t row_bytes, int64_t pool_rows, int dir, int threads) {
    std::atomic<int64_t> skipped{0};
    const int64_t slot_bytes = static_cast<int64_t>(n_pools) * rows_per_block * row_bytes;
    ParallelFor(n_blocks, threads, [&](int64_t b) {
        const int64_t slot = slot_idx ? slot_idx[b] : b;
        if (slot < 0 || slot >= n_slots) {
            skipped.fetch_add(static_cast<int64_t>(n_pools) * rows_per_block);
            return;
        }
        for (int32_t p = 0; p < n_pools; ++p) {
            uint8_t *stage = staging + slot * slot_bytes + static_cast<int64_t>(p) * rows_per_block * row_bytes;
            for (int64_t t = 0; t < rows_per_block; ++t) {
                const int64_t row = row_idx[b * rows_per_block + t];
                if (row < 0 || row >= pool_rows) {
                    skipped.fetch_add(1);
                    continue;
                }
                uint8_t *in_pool = pools[p] + row * row_bytes;
                if (dir == 0) {
                    std::memcpy(stage + t * row_bytes, in_pool, row_bytes);
                } else {
                    std::memcpy(in_pool, stage + t * row_bytes, row_bytes);
                }
            }
        }
    });
    return skipped.load();
}

// kv_cache_manager/py_connector/kernel/gather_scatter_helper.py:10-107 (legacy single-block
// kernels): layer tensor [2, total_tokens, hidden] per pointer, staging
// [n_layers, 2, n_tokens, hidden]; a token index >= total_tokens is skipped (:36-38, :87-89).
void kvcm_oracle_move_legacy(uint8_t *const *layers, int32_t n_layers, int64_t total_tokens, uint8_t *staging,
                             const int32_t *token_idx, int64_t n_tokens, int64_t hidden_bytes, int dir) {
    for (int32_t l = 0; l < n_layers; ++l) {
        for (int64_t t = 0; t < n_tokens; ++t) {
            const int64_t tok = token_idx[t];
            if (tok >= total_tokens || tok < 0) continue;
            for (int kv = 0; kv < 2; ++kv) {
                uint8_t *stage = staging + ((static_cast<int64_t>(l) * 2 + kv) * n_tokens + t) * hidden_bytes;
                uint8_t *cache = layers[l] + (kv * total_tokens + tok) * hidden_bytes;
                if (dir == 0) {
                    std::memcpy(stage, cache, hidden_bytes);
                } else {
                    std::memcpy(cache, stage, hidden_bytes);
                }
            }
        }
    }
}

// kv_cache_manager/client/src/internal/sdk/local_file_sdk.cc:223-245 (DoGet) and :326-353
// (DoPut): the iovs of a block are consumed in order against a contiguous byte string; an
// iov with `ignore`, a null base or zero size moves nothing but still advances the offset.
// dir 0 = iov -> block string (Put / save), 1 = block string -> iov (Get / load).
// Returns the number of bytes the iov list spans.
int64_t kvcm_oracle_copy_iovs(uint8_t *const *bases, const int64_t *sizes, const uint8_t *ignore, int64_t n_iovs,
                              uint8_t *block_string, int dir) {
    int64_t offset = 0;
    for (int64_t i = 0; i < n_iovs; ++i) {
        if (!ignore[i] && bases[i] != nullptr && sizes[i] > 0) {
            if (dir == 0) {
                std::memcpy(block_string + offset, bases[i], sizes[i]);
            } else {
                std::memcpy(bases[i], block_string + offset, sizes[i]);
            }
        }
        offset += sizes[i];
    }
    return offset;
}

// kv_cache_manager/client/src/internal/sdk/sdk_buffer_check_util.cu:10-44: reflected CRC-32
// (polynomial 0xEDB88320, init ~0, final complement) over the first and the last
// `cal_bytes` bytes of an iov.
uint32_t kvcm_oracle_iov_crc(const uint8_t *base, int64_t size, int64_t cal_bytes) {
    uint32_t crc = 0xFFFFFFFFu;
    auto feed = [&crc](uint8_t byte) {
        crc ^= byte;
        for (int i = 0; i < 8; ++i) {
            const uint32_t mask = 0u - (crc & 1u);
            crc = (crc >> 1) ^ (0xEDB88320u & mask);
        }
    };
    for (int64_t i = 0; i < cal_bytes; ++i) feed(base[i]);
    for (int64_t i = size - cal_bytes; i < size; ++i) feed(base[i]);
    return ~crc;
}

// ---------------------------------------------------------------------------------
// (2c) Optimizer trace replay
// ---------------------------------------------------------------------------------

}  // extern "C"

namespace {

// The prefix tree of kv_cache_manager/optimizer/index/radix_tree_index.cc, without eviction
// (IsBlockEvict is then always false).  The reference compresses chains of blocks into one
// node and splits nodes on divergence (:89-127); with no eviction that is observationally a
// plain trie with one block per node, which is what is kept here.
struct TrieNode {
    std::unordered_map<int64_t, TrieNode *> children;
    ~TrieNode() {
        for (auto &kv : children) delete kv.second;
    }
};

struct OracleReplay {
    TrieNode root;
    int64_t cached_blocks = 0;
};

}  // namespace

extern "C" {

void *kvcm_oracle_replay_create() { return new OracleReplay(); }
void kvcm_oracle_replay_destroy(void *h) { delete static_cast<OracleReplay *>(h); }

// Replays traces in the given order (the caller sorts by timestamp, as
// kv_cache_manager/optimizer/manager/optimizer_loader.cc:14-20 does).  Trace t owns
// keys[key_off[t], key_off[t+1]).  type: 0 DialogTurn -> RadixTreeIndex::InsertWithQuery
// (radix_tree_index.cc:198-282), 1 GetLocation -> PrefixQuery (:129-196) with the first
// mask_off[t] keys masked, 2 WriteCache -> InsertOnly (:19-87).  Per trace, as
// OptimizerRunner::HandleDialogTurn / HandleGetLocation / HandleWriteCache record them
// (kv_cache_manager/optimizer/manager/optimizer_runner.cc:70-215): external hit blocks,
// internal (masked) hit blocks, newly written blocks, and the cache size after the trace.
void kvcm_oracle_replay_run(void *h, const int64_t *keys, const int64_t *key_off, const uint8_t *type,
                            const int64_t *mask_off, const uint8_t *mask_bits, int64_t n_traces, int32_t *ext_hit,
                            int32_t *int_hit, int32_t *written, int64_t *cache_blocks) {
    auto *st = static_cast<OracleReplay *>(h);
    for (int64_t t = 0; t < n_traces; ++t) {
        const int64_t *k = keys + key_off[t];
        const int64_t n = key_off[t + 1] - key_off[t];
        int32_t ext = 0, inte = 0, wr = 0;
        TrieNode *node = &st->root;
        if (type[t] == 1) {
            // PrefixQuery classifies by key VALUE: a key counts as external when its value occurs
            // at some unmasked position, else internal when it occurs at a masked one (:137-146,:165-173).
            const int64_t mo = mask_off ? mask_off[t] : 0;
            std::unordered_map<int64_t, int> cls;  // 1 = query key, 2 = mask key only
            const uint8_t *bits = mask_bits ? mask_bits + key_off[t] : nullptr;  // a BlockMaskVector, one byte per key
            for (int64_t i = 0; i < n; ++i) {
                if (i < mo || (bits && bits[i])) {
                    cls.emplace(k[i], 2);
                } else {
                    cls[k[i]] = 1;
                }
            }
            for (int64_t i = 0; i < n; ++i) {
                auto it = node->children.find(k[i]);
                if (it == node->children.end()) break;
                if (cls[k[i]] == 1) {
                    ++ext;
                } else {
                    ++inte;
                }
                node = it->second;
            }
        } else {
            int64_t i = 0;
            for (; i < n; ++i) {
                auto it = node->children.find(k[i]);
                if (it == node->children.end()) break;
                node = it->second;
            }
            if (type[t] == 0) ext = static_cast<int32_t>(i);  // leading blocks already cached are the hits
            for (; i < n; ++i) {
                TrieNode *child = new TrieNode();
                node->children.emplace(k[i], child);
                node = child;
                ++wr;
            }
            st->cached_blocks += wr;
        }
        ext_hit[t] = ext;
        int_hit[t] = inte;
        written[t] = wr;
        cache_blocks[t] = st->cached_blocks;
    }
}

}  // extern "C"

// ---------------------------------------------------------------------------------
// (2c') Optimizer trace replay with LRU eviction
// ---------------------------------------------------------------------------------
// Restates, for one instance in a group of its own and the "lru" or the "leaf_aware_lru" policy on the
// shared tier:
//   RadixTreeIndex InsertNode / SplitNode / PrefixQuery / InsertQuery / CleanEmptyBlocks / WriteToTier
//     (kv_cache_manager/optimizer/index/radix_tree_index.cc:19-127,129-196,198-282,284-325,327-392),
//   LruEvictionPolicy (kv_cache_manager/optimizer/eviction_policy/lru.cc:6-49),
//   LeafAwareLruEvictionPolicy (kv_cache_manager/optimizer/eviction_policy/leaf_aware_lru.cc:20-160) with the
//     sorted insertions of LinkedList (eviction_policy/common_structure.h:62-89) and RadixTreeNode::isLeaf /
//     isDataLeaf (kv_cache_manager/optimizer/config/types.h:65-78),
//   OptEvictionManager::EvictByInstanceRough / EvictByInstancePrecise / GetExcessUsageForInstanceInGroup
//     (kv_cache_manager/optimizer/manager/eviction_manager.cc:148-239,249-266; with one instance per
//     group EvictByGroupRough (:86-146) does the same as EvictByInstanceRough),
//   OptIndexerManager::CheckAndEvict (kv_cache_manager/optimizer/manager/indexer_manager.cc:55-90),
//   and the three handlers of OptimizerRunner (optimizer_runner.cc:70-215).
// The tree is kept compressed and split exactly as the reference does, so that this oracle does not
// assume what the GPU replay assumes (that only per-key residency matters).
// Pins: the recency-order cases of kv_cache_manager/optimizer/test/lru_eviction_policy_test.cc:44-146
// restated as traces, the eviction-free replay above when the quota is never reached, and - for everything the
// reference's tests leave out (tree clean-up under eviction, leaf_aware_lru, random_lru, groups of instances) -
// the per-trace records of the reference's own Optimizer, compiled from its sources (ref_optimizer_driver.cc) and
// recorded in tests/golden/optimizer_ref_kat.json; where that library is present the two are also compared live
// (tests/test_optimizer_reference_pins.py).  The cases in tests/test_oracle.py were worked out by hand from the
// cited source lines.

namespace {

struct LruNode;
struct LruBlock {
    int64_t key = 0;
    bool cached = false;  // location_map non-empty
    bool listed = false;  // has a position in the recency list (always while cached under "lru")
    int64_t time = -1;    // last_access_time
    LruNode *owner = nullptr;
    std::list<LruBlock *>::iterator where;  // position in the recency list while listed
    size_t sampled_at = 0;                  // index in the random policy's block vector while cached
};
struct LruNode {
    LruNode *parent = nullptr;
    std::vector<std::unique_ptr<LruBlock>> blocks;
    std::unordered_map<int64_t, std::unique_ptr<LruNode>> children;
    bool leaf() const { return children.empty(); }
    bool data_leaf() const {  // types.h:68-78: no immediate child holds a cached block
        for (const auto &c : children) {
            for (const auto &b : c.second->blocks) {
                if (b->cached) return false;
            }
        }
        return true;
    }
};

struct OracleLruReplay {
    std::unique_ptr<LruNode> root{new LruNode()};
    std::list<LruBlock *> recency;  // front = most recently written or accessed
    int64_t n_cached = 0;           // EvictionPolicy::size(): blocks the policy knows (node_map_)
    int64_t quota = 0;
    int32_t batch = 1;
    bool precise = false;
    bool leaf_aware = false;
    int64_t now = 0;  // timestamp of the trace being replayed
    // "random_lru" (kv_cache_manager/optimizer/eviction_policy/random_lru.cc:5-131, random_lru.h:17-22): every cached
    // block sits in a dense vector beside its last access time; a round of evictions samples `sampling_size`
    // indices with a xorshift generator, orders the first k of them by time with std::partial_sort - called here as
    // the reference calls it, so that equal times come out in the standard library's order - and evicts those.
    bool random = false;
    std::vector<LruBlock *> sampled_blocks;
    std::vector<int64_t> sampled_times;
    uint64_t xor_state = 0x12345678ABCDEF01ULL;
    size_t sampling_size = 0;

    size_t fast_rand(size_t mod) {  // random_lru.cc:121-131
        if (mod == 0) return 0;
        uint64_t x = xor_state;
        x ^= x << 13;
        x ^= x >> 7;
        x ^= x << 17;
        xor_state = x;
        return x % mod;
    }
    void random_remove(LruBlock *b) {  // RemoveBlock, random_lru.cc:84-103: swap with the last entry, pop
        const size_t at = b->sampled_at;
        LruBlock *last = sampled_blocks.back();
        sampled_blocks[at] = last;
        sampled_times[at] = sampled_times.back();
        last->sampled_at = at;
        sampled_blocks.pop_back();
        sampled_times.pop_back();
        b->cached = false;
        --n_cached;
    }
    std::vector<LruBlock *> evict_random_blocks(int64_t count) {  // EvictBlocks + SampleAndPickLru, :38-82
        std::vector<LruBlock *> out;
        if (sampled_blocks.empty()) return out;
        const size_t total = std::min<size_t>(static_cast<size_t>(count), sampled_blocks.size());
        const size_t n = sampled_blocks.size();
        const size_t sample = std::min(sampling_size, n);
        const size_t k = std::min(total, sample);
        std::vector<size_t> indices;
        indices.reserve(sample);
        for (size_t i = 0; i < sample; ++i) indices.push_back(fast_rand(n));
        std::partial_sort(indices.begin(), indices.begin() + static_cast<std::ptrdiff_t>(k), indices.end(),
                          [this](size_t a, size_t b) { return sampled_times[a] < sampled_times[b]; });
        std::vector<LruBlock *> victims;
        for (size_t i = 0; i < k; ++i) victims.push_back(sampled_blocks[indices[i]]);
        for (LruBlock *v : victims) {
            if (!v->cached) continue;  // sampled twice: gone already
            random_remove(v);
            out.push_back(v);
            if (out.size() == total) break;
        }
        return out;
    }

    void on_written(LruBlock *b) {  // lru.cc:6-11; leaf_aware_lru.cc:20-31; times: radix_tree_index.cc:335-336,366-367
        b->cached = true;
        b->time = now;
        ++n_cached;
        if (random) {  // OnBlockWritten, random_lru.cc:17-21
            b->sampled_at = sampled_blocks.size();
            sampled_blocks.push_back(b);
            sampled_times.push_back(b->time);
            return;
        }
        if (leaf_aware && !(b->owner != nullptr && b->owner->leaf())) return;  // only blocks of leaves queue up
        recency.push_front(b);
        b->where = recency.begin();
        b->listed = true;
    }
    void on_accessed(LruBlock *b) {  // lru.cc:18-26; leaf_aware_lru.cc:39-51
        if (!b->cached) return;
        b->time = now;
        if (random) {  // OnBlockAccessed, random_lru.cc:27-35
            sampled_times[b->sampled_at] = now;
            return;
        }
        if (!b->listed) return;
        recency.splice(recency.begin(), recency, b->where);
        b->where = recency.begin();
    }
    // WriteToTier without a callback: new blocks at the end of `node` (radix_tree_index.cc:327-343,377-392)
    void append_new(LruNode *node, const int64_t *k, int64_t n) {
        for (int64_t i = 0; i < n; ++i) {
            std::unique_ptr<LruBlock> b(new LruBlock());
            b->key = k[i];
            b->owner = node;
            LruBlock *raw = b.get();
            node->blocks.push_back(std::move(b));
            on_written(raw);
        }
    }
    // WriteToTier with AppendEvictBlocks: evicted blocks of a node get their location back (:355-375)
    void revive(const std::vector<LruBlock *> &blocks) {
        for (LruBlock *b : blocks) on_written(b);
    }
    void split(LruNode *node, size_t pos, const int64_t *right, int64_t n_right) {  // :89-127
        if (pos == 0 || node->parent == nullptr) return;
        LruNode *parent = node->parent;
        const int64_t edge = node->blocks.front()->key;
        std::unique_ptr<LruNode> old = std::move(parent->children[edge]);
        std::unique_ptr<LruNode> mid(new LruNode());
        LruNode *mid_raw = mid.get();
        for (size_t i = 0; i < pos; ++i) {
            mid_raw->blocks.push_back(std::move(old->blocks[i]));
            mid_raw->blocks.back()->owner = mid_raw;
        }
        mid_raw->parent = parent;
        old->blocks.erase(old->blocks.begin(), old->blocks.begin() + pos);
        old->parent = mid_raw;
        const int64_t old_edge = old->blocks.front()->key;
        mid_raw->children[old_edge] = std::move(old);
        if (n_right > 0) {
            std::unique_ptr<LruNode> fresh(new LruNode());
            fresh->parent = mid_raw;
            append_new(fresh.get(), right, n_right);
            mid_raw->children[right[0]] = std::move(fresh);
        }
        parent->children[edge] = std::move(mid);
    }
    // InsertNode (:30-87) when query == false, InsertQuery (:214-282) when query == true.
    // Returns the number of keys written; `hits` counts the leading cached blocks of a query.
    int64_t insert(LruNode *node, const int64_t *k, int64_t n, bool query, bool alive, int64_t *hits) {
        if (n == 0) return 0;
        if (node->leaf() && node->parent != nullptr) {
            append_new(node, k, n);
            return n;
        }
        auto it = node->children.find(k[0]);
        if (it == node->children.end()) {
            std::unique_ptr<LruNode> fresh(new LruNode());
            fresh->parent = node;
            append_new(fresh.get(), k, n);
            node->children[k[0]] = std::move(fresh);
            return n;
        }
        LruNode *child = it->second.get();
        std::vector<LruBlock *> evicted;
        size_t m = 0;
        while (m < child->blocks.size() && static_cast<int64_t>(m) < n && child->blocks[m]->key == k[m]) {
            LruBlock *b = child->blocks[m].get();
            if (!b->cached) {
                evicted.push_back(b);
                alive = false;
            } else if (query && alive) {
                ++*hits;
                on_accessed(b);
            }
            ++m;
        }
        int64_t wrote = static_cast<int64_t>(evicted.size());
        revive(evicted);
        if (m == child->blocks.size()) return wrote + insert(child, k + m, n - m, query, alive, hits);
        if (static_cast<int64_t>(m) == n) return wrote;
        split(child, m, k + m, n - m);
        return wrote + (n - static_cast<int64_t>(m));
    }
    void prefix_query(const int64_t *k, int64_t n, int64_t mask_off, const uint8_t *bits, int32_t *ext,
                      int32_t *inte) {  // :129-196
        std::unordered_map<int64_t, int> cls;  // 1 = occurs unmasked, 2 = occurs masked only
        for (int64_t i = 0; i < n; ++i) {
            if (i < mask_off || (bits && bits[i])) {
                cls.emplace(k[i], 2);
            } else {
                cls[k[i]] = 1;
            }
        }
        LruNode *node = root.get();
        int64_t at = 0;
        while (at < n) {
            auto it = node->children.find(k[at]);
            if (it == node->children.end()) break;
            LruNode *child = it->second.get();
            size_t m = 0;
            while (m < child->blocks.size() && at + static_cast<int64_t>(m) < n && child->blocks[m]->key == k[at + m]) {
                LruBlock *b = child->blocks[m].get();
                if (!b->cached) break;
                if (cls[k[at + m]] == 1) {
                    ++*ext;
                } else {
                    ++*inte;
                }
                on_accessed(b);
                ++m;
            }
            if (m < child->blocks.size() || at + static_cast<int64_t>(m) == n) break;
            node = child;
            at += static_cast<int64_t>(m);
        }
    }
    std::vector<LruBlock *> evict_blocks(int64_t count) {  // lru.cc:28-49
        if (leaf_aware) return evict_leaf_blocks(count);
        if (random) return evict_random_blocks(count);
        std::vector<LruBlock *> out;
        for (int64_t i = 0; i < count && !recency.empty(); ++i) {
            LruBlock *b = recency.back();
            recency.pop_back();
            b->cached = false;
            b->listed = false;
            --n_cached;
            out.push_back(b);
        }
        return out;
    }
    // LinkedList::insert_sorted / insert_sorted_reverse with LeafLRUListNode::compare (a before b while
    // a's time is smaller), chosen as insert_sorted_by_priority does (leaf_aware_lru.cc:53-83).
    void insert_by_time(LruBlock *b) {
        std::list<LruBlock *>::iterator at;
        if (recency.empty()) {
            at = recency.end();
        } else {
            const int64_t head = recency.front()->time, tail = recency.back()->time, t = b->time;
            bool from_head;
            if (t >= head) {
                from_head = true;
            } else if (t <= tail) {
                from_head = false;
            } else {
                from_head = (head - t) < (t - tail);
            }
            if (from_head) {
                at = recency.begin();
                while (at != recency.end() && t < (*at)->time) ++at;
            } else {
                auto r = recency.rbegin();
                while (r != recency.rend() && (*r)->time < t) ++r;
                at = r.base();  // the position right after *r
            }
        }
        b->where = recency.insert(at, b);
        b->listed = true;
    }
    bool update_node_state(LruNode *node) {  // leaf_aware_lru.cc:135-160
        if (node == nullptr || !node->data_leaf()) return false;
        bool any = false;
        for (const auto &b : node->blocks) {
            if (b->cached && !b->listed) {
                insert_by_time(b.get());
                any = true;
            }
        }
        return any;
    }
    std::vector<LruBlock *> evict_leaf_blocks(int64_t count) {  // leaf_aware_lru.cc:85-133
        std::vector<LruBlock *> out;
        std::set<LruNode *> done;
        while (static_cast<int64_t>(out.size()) < count && !recency.empty()) {
            LruBlock *b = recency.back();
            LruNode *owner = b->owner;
            if (owner != nullptr && !owner->data_leaf()) {  // its node got cached children since: leave the queue
                recency.pop_back();
                b->listed = false;
                continue;
            }
            recency.pop_back();
            b->listed = false;
            b->cached = false;
            --n_cached;
            out.push_back(b);
            if (owner != nullptr && owner->parent != nullptr && done.count(owner->parent) == 0) {
                if (update_node_state(owner->parent)) done.insert(owner->parent);
            }
        }
        return out;
    }
    void clean(const std::vector<LruBlock *> &gone) {  // radix_tree_index.cc:284-325
        std::unordered_set<LruNode *> check;
        for (LruBlock *b : gone) {
            if (!b->cached && b->owner != nullptr && b->owner->parent != nullptr) check.insert(b->owner);
        }
        bool removed = true;
        while (removed) {
            removed = false;
            for (auto it = check.begin(); it != check.end();) {
                LruNode *node = *it;
                bool all_gone = true;
                for (const auto &b : node->blocks) all_gone = all_gone && !b->cached;
                if (all_gone && !node->blocks.empty() && node->parent != nullptr && node->leaf()) {
                    node->parent->children.erase(node->blocks.front()->key);
                    it = check.erase(it);
                    removed = true;
                } else {
                    ++it;
                }
            }
        }
    }
    void check_and_evict() {  // indexer_manager.cc:55-90, eviction_manager.cc:148-266
        const int64_t used = n_cached;
        const int64_t excess = used > quota ? used - quota : 0;
        if (excess == 0) return;
        std::vector<LruBlock *> all;
        int64_t total = 0;
        while (total < excess) {
            const int64_t count = precise ? std::min<int64_t>(batch, excess - total) : batch;
            std::vector<LruBlock *> round = evict_blocks(count);
            if (round.empty()) break;
            total += static_cast<int64_t>(round.size());
            all.insert(all.end(), round.begin(), round.end());
        }
        clean(all);
    }
};

// Several instances that share one group quota (OptEvictionManager::EvictByGroupRough / EvictByInstanceRough /
// EvictByInstancePrecise over GetExcessUsageForInstanceInGroup, eviction_manager.cc:86-266; every instance has a
// tree and a policy of its own, optimizer_manager.cc:66-99; the blocks each instance lost go to that instance's
// CleanEmptyBlocks, indexer_manager.cc:55-90).  mode: 1 group rough, 2 instance rough, 3 instance precise.
struct OracleLruGroup {
    std::vector<std::unique_ptr<OracleLruReplay>> inst;
    int64_t quota = 0;
    int32_t batch = 1;
    int32_t mode = 1;

    void check_and_evict(size_t writer) {
        int64_t used = 0;
        for (const auto &i : inst) used += i->n_cached;
        const int64_t excess = used > quota ? used - quota : 0;
        if (excess == 0) return;
        std::vector<std::vector<LruBlock *>> gone(inst.size());
        int64_t total = 0;
        if (mode == 1) {
            while (total < excess) {
                bool any = false;
                for (size_t j = 0; j < inst.size(); ++j) {  // a whole round even when the excess is covered midway
                    std::vector<LruBlock *> round = inst[j]->evict_blocks(batch);
                    if (round.empty()) continue;
                    any = true;
                    total += static_cast<int64_t>(round.size());
                    gone[j].insert(gone[j].end(), round.begin(), round.end());
                }
                if (!any) break;
            }
        } else {
            while (total < excess) {
                const int64_t count = mode == 3 ? std::min<int64_t>(batch, excess - total) : batch;
                std::vector<LruBlock *> round = inst[writer]->evict_blocks(count);
                if (round.empty()) break;
                total += static_cast<int64_t>(round.size());
                gone[writer].insert(gone[writer].end(), round.begin(), round.end());
            }
        }
        for (size_t j = 0; j < inst.size(); ++j) {
            if (!gone[j].empty()) inst[j]->clean(gone[j]);
        }
    }
};

}  // namespace

extern "C" {

void *kvcm_oracle_lru_group_create(int64_t quota_blocks, int32_t evict_batch, int32_t mode, int32_t n_instances,
                                   int32_t policy) {
    auto *g = new OracleLruGroup();
    g->quota = quota_blocks;
    g->batch = evict_batch;
    g->mode = mode;
    for (int32_t i = 0; i < n_instances; ++i) {
        g->inst.emplace_back(new OracleLruReplay());
        g->inst.back()->leaf_aware = policy == 1;
    }
    return g;
}
void kvcm_oracle_lru_group_destroy(void *h) { delete static_cast<OracleLruGroup *>(h); }
// The eviction_policy_type of one instance of the group (EvictionPolicyFactory::CreatePolicy is called per instance,
// kv_cache_manager/optimizer/manager/eviction_manager.cc:22-55): 0 = "lru", 1 = "leaf_aware_lru".  Before any trace.
void kvcm_oracle_lru_group_set_policy(void *h, int32_t instance, int32_t policy) {
    static_cast<OracleLruGroup *>(h)->inst[static_cast<size_t>(instance)]->leaf_aware = policy == 1;
}
// "random_lru" for one instance of the group, with that instance's sample_rate (RandomLruEvictionPolicy's
// constructor, random_lru.cc:5-14: a rate <= 0 means 0.1, sampling_size = size_t(batch / rate)).  Before any trace.
void kvcm_oracle_lru_group_set_random(void *h, int32_t instance, double sample_rate) {
    auto *g = static_cast<OracleLruGroup *>(h);
    OracleLruReplay *st = g->inst[static_cast<size_t>(instance)].get();
    st->leaf_aware = false;
    st->random = true;
    if (sample_rate <= 0.0) sample_rate = 0.1;
    st->sampling_size = static_cast<size_t>(g->batch / sample_rate);
}

// trace_inst[t]: the instance (0 .. n_instances-1) trace t belongs to; traces in replay order over all instances.
// cache_blocks[t] is the usage of the trace's own instance after the trace (GetCurrentInstanceUsage,
// optimizer_runner.cc:116,196); inst_blocks (optional, [n_instances]) the usage of every instance at the end.
void kvcm_oracle_lru_group_run(void *h, const int64_t *keys, const int64_t *key_off, const uint8_t *type,
                               const int64_t *mask_off, const uint8_t *mask_bits, const int64_t *timestamps,
                               const int32_t *trace_inst, int64_t n_traces, int32_t *ext_hit, int32_t *int_hit,
                               int32_t *written, int64_t *cache_blocks, int64_t *inst_blocks,
                               int64_t *inst_blocks_trace) {
    // inst_blocks_trace (optional, [n_traces][instances]): GetCurrentInstanceUsage of every instance when the
    // trace's record is made (ReadRecord::blocks_per_instance, optimizer_runner.cc:116-124,196-203)
    auto *g = static_cast<OracleLruGroup *>(h);
    for (int64_t t = 0; t < n_traces; ++t) {
        const size_t i = static_cast<size_t>(trace_inst[t]);
        OracleLruReplay *st = g->inst[i].get();
        st->now = timestamps ? timestamps[t] : t;
        const int64_t *k = keys + key_off[t];
        const int64_t n = key_off[t + 1] - key_off[t];
        int32_t ext = 0, inte = 0;
        int64_t wr = 0, hits = 0;
        if (type[t] == 1) {
            if (n > 0) {
                st->prefix_query(k, n, mask_off ? mask_off[t] : 0, mask_bits ? mask_bits + key_off[t] : nullptr, &ext,
                                 &inte);
            }
        } else {
            wr = st->insert(st->root.get(), k, n, type[t] == 0, true, &hits);
            ext = static_cast<int32_t>(hits);
            g->check_and_evict(i);
        }
        ext_hit[t] = ext;
        int_hit[t] = inte;
        written[t] = static_cast<int32_t>(wr);
        cache_blocks[t] = st->n_cached;
        if (inst_blocks_trace != nullptr) {
            for (size_t j = 0; j < g->inst.size(); ++j) {
                inst_blocks_trace[static_cast<size_t>(t) * g->inst.size() + j] = g->inst[j]->n_cached;
            }
        }
    }
    if (inst_blocks != nullptr) {
        for (size_t j = 0; j < g->inst.size(); ++j) inst_blocks[j] = g->inst[j]->n_cached;
    }
}

void *kvcm_oracle_lru_replay_create(int64_t quota_blocks, int32_t evict_batch, int32_t precise) {
    auto *st = new OracleLruReplay();
    st->quota = quota_blocks;
    st->batch = evict_batch;
    st->precise = precise != 0;
    return st;
}
// policy: 0 = "lru", 1 = "leaf_aware_lru"
void *kvcm_oracle_lru_replay_create_policy(int64_t quota_blocks, int32_t evict_batch, int32_t precise,
                                           int32_t policy) {
    auto *st = static_cast<OracleLruReplay *>(kvcm_oracle_lru_replay_create(quota_blocks, evict_batch, precise));
    st->leaf_aware = policy == 1;
    return st;
}
// std::partial_sort exactly as RandomLruEvictionPolicy::SampleAndPickLru calls it (random_lru.cc:72-74): indices
// ordered by the time they point at.  Test infrastructure for the restatement of that algorithm in the sweep kernel.
void kvcm_oracle_partial_sort_by_time(uint64_t *indices, int64_t n, int64_t k, const int64_t *times) {
    std::vector<size_t> idx(indices, indices + n);
    std::partial_sort(idx.begin(), idx.begin() + static_cast<std::ptrdiff_t>(k), idx.end(),
                      [times](size_t a, size_t b) { return times[a] < times[b]; });
    for (int64_t i = 0; i < n; ++i) indices[i] = idx[static_cast<size_t>(i)];
}

// "random_lru": sampling_size = batch / sample_rate as a double division cut to an integer, 0.1 for a rate <= 0
// (RandomLruEvictionPolicy's constructor, random_lru.cc:5-14).
void *kvcm_oracle_random_lru_replay_create(int64_t quota_blocks, int32_t evict_batch, int32_t precise,
                                           double sample_rate) {
    auto *st = static_cast<OracleLruReplay *>(kvcm_oracle_lru_replay_create(quota_blocks, evict_batch, precise));
    st->random = true;
    if (sample_rate <= 0.0) sample_rate = 0.1;
    st->sampling_size = static_cast<size_t>(evict_batch / sample_rate);
    return st;
}
void kvcm_oracle_lru_replay_destroy(void *h) { delete static_cast<OracleLruReplay *>(h); }

// Same trace encoding and outputs as kvcm_oracle_replay_run; cache_blocks[t] is the number of cached
// blocks after trace t (EvictionPolicy::size(), after CheckAndEvict for the writing kinds).
// timestamps (optional): the traces' timestamp_us, which "leaf_aware_lru" orders re-queued blocks by; the
// trace number stands in when it is null.
void kvcm_oracle_lru_replay_run_ts(void *h, const int64_t *keys, const int64_t *key_off, const uint8_t *type,
                                   const int64_t *mask_off, const uint8_t *mask_bits, const int64_t *timestamps,
                                   int64_t n_traces, int32_t *ext_hit, int32_t *int_hit, int32_t *written,
                                   int64_t *cache_blocks) {
    auto *st = static_cast<OracleLruReplay *>(h);
    for (int64_t t = 0; t < n_traces; ++t) {
        st->now = timestamps ? timestamps[t] : t;
        const int64_t *k = keys + key_off[t];
        const int64_t n = key_off[t + 1] - key_off[t];
        int32_t ext = 0, inte = 0;
        int64_t wr = 0, hits = 0;
        if (type[t] == 1) {
            if (n > 0) {
                st->prefix_query(k, n, mask_off ? mask_off[t] : 0, mask_bits ? mask_bits + key_off[t] : nullptr, &ext,
                                 &inte);
            }
        } else {
            wr = st->insert(st->root.get(), k, n, type[t] == 0, true, &hits);
            ext = static_cast<int32_t>(hits);
            st->check_and_evict();
        }
        ext_hit[t] = ext;
        int_hit[t] = inte;
        written[t] = static_cast<int32_t>(wr);
        cache_blocks[t] = st->n_cached;
    }
}
void kvcm_oracle_lru_replay_run(void *h, const int64_t *keys, const int64_t *key_off, const uint8_t *type,
                                const int64_t *mask_off, const uint8_t *mask_bits, int64_t n_traces, int32_t *ext_hit,
                                int32_t *int_hit, int32_t *written, int64_t *cache_blocks) {
    kvcm_oracle_lru_replay_run_ts(h, keys, key_off, type, mask_off, mask_bits, nullptr, n_traces, ext_hit, int_hit,
                                  written, cache_blocks);
}

}  // extern "C"
