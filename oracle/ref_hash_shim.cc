// C wrapper around the reference's OWN hash header, compiled where it lies (never copied).
// TEST INFRASTRUCTURE ONLY: it pins the oracle's hash restatement and can serve as the
// "reference" CPU baseline.  Built by oracle/Makefile into oracle/_ref/ when the reference
// tree is present (KVCM_REF_DIR); nothing in the product loads it.
#include <cstdint>
#include <vector>

#include "kv_cache_manager/manager/hash_util.h"  // hashInt64Func / hashInt64Array, :8-24

extern "C" {

int64_t kvcm_ref_hash_step(int64_t hash, int64_t value) {
    std::hash<int64_t> hasher;
    return kv_cache_manager::hashInt64Func(hasher, hash, value);
}

int64_t kvcm_ref_hash_array(int64_t hash, const int64_t *begin, const int64_t *end) {
    return kv_cache_manager::hashInt64Array(hash, begin, end);
}

// The loop of GenKeyVector (kv_cache_manager/manager/cache_manager.cc:76-87) around the
// reference's hashInt64Array; the function itself sits in an anonymous namespace of a file
// that needs the whole server to compile, so only its three-line loop is restated here.
int64_t kvcm_ref_gen_key_vector(const int64_t *tokens, int64_t n_tokens, int64_t block_size, int64_t *keys) {
    const int64_t total_blocks = n_tokens / block_size;
    int64_t hash = 0;
    for (int64_t index = 0; index < total_blocks; index++) {
        const int64_t pos = index * block_size;
        hash = kv_cache_manager::hashInt64Array(hash, tokens + pos, tokens + pos + block_size);
        keys[index] = hash;
    }
    return total_blocks;
}

// The loop of ApplyPrefixHash (kv_cache_manager/optimizer/trace_converter/trace_util.cc:47-56).
void kvcm_ref_apply_prefix_hash(const int64_t *ids, int64_t n, int64_t *keys) {
    int64_t hash = 0;
    std::hash<int64_t> hasher;
    for (int64_t i = 0; i < n; i++) {
        hash = kv_cache_manager::hashInt64Func(hasher, hash, ids[i]);
        keys[i] = hash;
    }
}

}  // extern "C"
