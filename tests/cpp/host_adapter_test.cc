// Drives the C++ host adapters (tair-kvcache_b200/host/kvcm_b200_host.h) with the known-answer
// tables of the reference's own C++ unit tests, the way those tests call MetaSearcher and
// CacheManager.  Needs a GPU.  Exit code 0 = all checks passed.
//   kv_cache_manager/manager/test/meta_searcher_test.cc:196-274   prefix match, masks
//   kv_cache_manager/manager/test/cache_manager_test.cc:474-786   prefix / batch-get / sliding window
//   hash values: from the reference's hash_util.h compiled as-is (see tests/golden/hash_kat.json)
#include <cstdio>
#include <string>

#include "kvcm_b200_host.h"

using namespace kvcm_b200;

static int g_failed = 0;
#define EXPECT_EQ(a, b)                                                                      \
    do {                                                                                     \
        const auto va = (a);                                                                 \
        const auto vb = (b);                                                                 \
        if (!(va == vb)) {                                                                   \
            std::printf("FAIL %s:%d: %s != %s (%lld vs %lld)\n", __FILE__, __LINE__, #a, #b, \
                        (long long)va, (long long)vb);                                       \
            ++g_failed;                                                                      \
        }                                                                                    \
    } while (0)

static uint64_t Serving(int type) { return EncodeLocations({{CLS_SERVING, type}}); }
static uint64_t Writing(int type) { return EncodeLocations({{CLS_WRITING, type}}); }

static void TestHash() {
    GpuKeyGenerator gen;
    const KeyVector k1 = gen.GenKeyVector({1, 2, 3, 4}, 2);
    EXPECT_EQ(k1.size(), size_t(2));
    EXPECT_EQ(k1[0], -8366447769517741626LL);
    EXPECT_EQ(k1[1], 455111481605203084LL);
    TokenIdsVector t(130);
    for (int i = 0; i < 130; ++i) t[i] = i;
    const KeyVector k2 = gen.GenKeyVector(t, 64);
    EXPECT_EQ(k2.size(), size_t(2));
    EXPECT_EQ(k2[0], 2681637840371060507LL);
    EXPECT_EQ(k2[1], -6990124544746687103LL);
    const KeyVector k3 = gen.ApplyPrefixHash({100, 200, 300});
    EXPECT_EQ(k3.size(), size_t(3));
    EXPECT_EQ(k3[0], -7046029254386353031LL);
    EXPECT_EQ(k3[2], 8024479186332561338LL);
    EXPECT_EQ(gen.GenKeyVector({}, 16).size(), size_t(0));
    EXPECT_EQ(gen.GenKeyVector({1, 2, 3}, 16).size(), size_t(0));
    std::vector<KeyVector> batch;
    EXPECT_EQ(gen.GenKeyVectorBatch({{1, 2, 3, 4}, {}, t}, 2, &batch), KVCM_OK);
    EXPECT_EQ(batch[0][1], 455111481605203084LL);
    EXPECT_EQ(batch[1].size(), size_t(0));
    EXPECT_EQ(batch[2].size(), size_t(65));
}

static void TestPrefixMatch() {
    GpuBlockIndex index(64);
    GpuMetaSearcher searcher(&index);
    size_t len = 99;
    // locations added but not yet SERVING: nothing matches (meta_searcher_test.cc:196-204)
    EXPECT_EQ(index.Put({10, 20, 30}, {Writing(4), Writing(1), Writing(2)}), KVCM_OK);
    EXPECT_EQ(searcher.PrefixMatch({10, 20, 30}, BlockMask{}, &len), KVCM_OK);
    EXPECT_EQ(len, size_t(0));
    EXPECT_EQ(index.Put({10, 20, 30}, {Serving(4), Serving(1), Serving(2)}), KVCM_OK);
    struct Case {
        KeyVector keys;
        size_t want;
    };
    const std::vector<Case> cases = {{{10, 20, 30}, 3}, {{10, 20, 999}, 2}, {{10, 999, 999}, 1}, {{999, 999, 999}, 0},
                                     {{}, 0},           {{10}, 1},          {{10, 20}, 2},       {{10, 999, 30}, 1}};
    for (const Case &c : cases) {
        EXPECT_EQ(searcher.PrefixMatch(c.keys, BlockMask{}, &len), KVCM_OK);
        EXPECT_EQ(len, c.want);
    }
    // masks: vector {true,false,false} and offset 1 both skip the first key (:254-274)
    EXPECT_EQ(searcher.PrefixMatch({10, 20, 30}, BlockMask{BlockMaskVector{true, false, false}}, &len), KVCM_OK);
    EXPECT_EQ(len, size_t(2));
    EXPECT_EQ(searcher.PrefixMatch({10, 20, 30}, BlockMask{BlockMaskOffset{1}}, &len), KVCM_OK);
    EXPECT_EQ(len, size_t(2));
    // batched form, mixed masks
    std::vector<int32_t> lens;
    EXPECT_EQ(searcher.PrefixMatchBatch({{10, 20, 30}, {10, 999, 30}, {}, {999, 10}},
                                        {BlockMask{}, BlockMask{BlockMaskOffset{0}}, BlockMask{},
                                         BlockMask{BlockMaskVector{true}}},
                                        &lens),
              KVCM_OK);
    EXPECT_EQ(lens[0], 3);
    EXPECT_EQ(lens[1], 1);
    EXPECT_EQ(lens[2], 0);
    EXPECT_EQ(lens[3], 1);
    // a storage class the policy has switched off is not servable
    GpuMetaSearcher no_hf3fs(&index, KVCM_AVAIL_ALL & ~(1u << 1));
    EXPECT_EQ(no_hf3fs.PrefixMatch({10, 20, 30}, BlockMask{}, &len), KVCM_OK);
    EXPECT_EQ(len, size_t(1));
    // erase
    EXPECT_EQ(index.Erase({20}), KVCM_OK);
    EXPECT_EQ(searcher.PrefixMatch({10, 20, 30}, BlockMask{}, &len), KVCM_OK);
    EXPECT_EQ(len, size_t(1));
}

static void TestSlidingWindowAndBatchGet() {
    // keys 1..6 started, first five finished: 1..5 SERVING, 6 WRITING (cache_manager_test.cc:666-749)
    GpuBlockIndex index(64);
    GpuMetaSearcher searcher(&index);
    EXPECT_EQ(index.Put({1, 2, 3, 4, 5, 6}, {Serving(4), Serving(4), Serving(4), Serving(4), Serving(4), Writing(4)}),
              KVCM_OK);
    int64_t base = 0;
    EXPECT_EQ(searcher.ReverseRollSlideWindowMatch({1, 2, 3, 4, 5, 6, 7}, 2, &base), KVCM_OK);
    EXPECT_EQ(base, 3);  // non-empty exactly at positions 3,4
    EXPECT_EQ(searcher.ReverseRollSlideWindowMatch({1, 2, 3, 10, 5, 6, 7}, 2, &base), KVCM_OK);
    EXPECT_EQ(base, 1);  // non-empty exactly at positions 1,2
    EXPECT_EQ(searcher.ReverseRollSlideWindowMatch({6, 7, 8}, 2, &base), KVCM_OK);
    EXPECT_EQ(base, -1);
    EXPECT_EQ(searcher.ReverseRollSlideWindowMatch({1}, 2, &base), KVCM_EC_BADARGS);   // keys.size() < sw_size
    EXPECT_EQ(searcher.ReverseRollSlideWindowMatch({1}, -1, &base), KVCM_EC_BADARGS);  // sw_size < 0
    EXPECT_EQ(searcher.ReverseRollSlideWindowMatch({1}, 0, &base), KVCM_EC_BADARGS);   // never ends in the reference
    std::vector<uint8_t> flags;
    EXPECT_EQ(searcher.BatchGet({1, 2, 111, 6}, &flags), KVCM_OK);  // cache_manager_test.cc:547-630
    EXPECT_EQ(flags[0] & KVCM_FLAG_SERVABLE, 1);
    EXPECT_EQ(flags[1] & KVCM_FLAG_SERVABLE, 1);
    EXPECT_EQ(int(flags[2]), 0);
    EXPECT_EQ(flags[3] & KVCM_FLAG_SERVABLE, 0);
    EXPECT_EQ(flags[3] & KVCM_FLAG_WRITABLE, int(KVCM_FLAG_WRITABLE));
}

static void TestWriteCycle() {
    // StartWriteCache -> FinishWriteCache -> reclaim on the replica, without reading a key's map back
    // (MetaSearcher::BatchAddLocation, BatchUpdateLocationStatus, BatchCADLocationStatus:
    // kv_cache_manager/manager/meta_searcher.cc:312-487,582-717; the match table of meta_searcher_test.cc:196-252).
    GpuBlockIndex index(64);
    GpuMetaSearcher searcher(&index);
    std::vector<int32_t> codes;
    size_t len = 99;
    EXPECT_EQ(index.AddLocation({10, 20, 30}, {4}, &codes), KVCM_OK);
    EXPECT_EQ(codes[0] | codes[1] | codes[2], KVCM_OK);
    EXPECT_EQ(searcher.PrefixMatch({10, 20, 30}, BlockMask{}, &len), KVCM_OK);
    EXPECT_EQ(len, size_t(0));  // written, not served yet
    EXPECT_EQ(index.UpdateLocationStatus({10, 20}, {KVCM_STATUS_TASK(4, 2, 3)}, &codes), KVCM_OK);  // WRITING -> SERVING
    EXPECT_EQ(codes[0] | codes[1], KVCM_OK);
    EXPECT_EQ(searcher.PrefixMatch({10, 20, 30}, BlockMask{}, &len), KVCM_OK);
    EXPECT_EQ(len, size_t(2));
    // a second tier for key 20 leaves its served location alone; a second location of one class is refused
    EXPECT_EQ(index.AddLocation({20, 30}, {1, 4}, &codes), KVCM_OK);
    EXPECT_EQ(codes[0], KVCM_OK);
    EXPECT_EQ(codes[1], KVCM_EC_EXIST);
    EXPECT_EQ(searcher.PrefixMatch({10, 20, 30}, BlockMask{}, &len), KVCM_OK);
    EXPECT_EQ(len, size_t(2));
    // compare-and-set on the wrong status, on a missing key; compare-and-delete of the last location drops the key
    EXPECT_EQ(index.UpdateLocationStatus({30, 40, 10}, {KVCM_STATUS_TASK(4, 3, 4), KVCM_STATUS_TASK(4, 2, 3),
                                                        KVCM_STATUS_TASK(4, 3, KVCM_STATUS_DELETE)}, &codes), KVCM_OK);
    EXPECT_EQ(codes[0], KVCM_EC_MISMATCH);
    EXPECT_EQ(codes[1], KVCM_EC_NOENT);
    EXPECT_EQ(codes[2], KVCM_OK);
    std::vector<uint8_t> flags;
    EXPECT_EQ(searcher.BatchGet({10, 20, 30}, &flags), KVCM_OK);
    EXPECT_EQ(int(flags[0]), 0);
    EXPECT_EQ(flags[1] & KVCM_FLAG_SERVABLE, 1);
    EXPECT_EQ(flags[2] & KVCM_FLAG_SERVABLE, 0);
    EXPECT_EQ(index.AddLocation({1, 2}, {1, 2, 3}, &codes), KVCM_EC_BADARGS);
}

static void TestWriteBatch() {
    // Three StartWriteCache requests in one call, answered as if served in order (cache_manager.cc:334-430,589-635):
    // a b c writes all three; a b d e sees a b being written and writes d e; x b sees b and writes x (vector form).
    GpuBlockIndex index(64);
    GpuMetaSearcher searcher(&index);
    std::vector<BlockMask> masks;
    std::vector<KeyVector> fresh;
    EXPECT_EQ(searcher.StartWriteCacheBatch({{11, 12, 13}, {11, 12, 14, 15}, {99, 12}}, 4, &masks, &fresh), KVCM_OK);
    EXPECT_EQ(std::get<BlockMaskOffset>(masks[0]), size_t(0));
    EXPECT_EQ(std::get<BlockMaskOffset>(masks[1]), size_t(2));
    EXPECT_EQ(std::holds_alternative<BlockMaskVector>(masks[2]), true);
    EXPECT_EQ(std::get<BlockMaskVector>(masks[2])[0], false);
    EXPECT_EQ(std::get<BlockMaskVector>(masks[2])[1], true);
    EXPECT_EQ(fresh[0].size(), size_t(3));
    EXPECT_EQ(fresh[1].size(), size_t(2));
    EXPECT_EQ(fresh[1][0], 14);
    EXPECT_EQ(fresh[2].size(), size_t(1));
    EXPECT_EQ(fresh[2][0], 99);
    size_t len = 99;
    EXPECT_EQ(searcher.PrefixMatch({11, 12, 13}, BlockMask{}, &len), KVCM_OK);
    EXPECT_EQ(len, size_t(0));
    std::vector<int32_t> codes;
    // an invalid mask (a vector of the wrong length) refuses the call
    EXPECT_EQ(searcher.FinishWriteCacheBatch({BlockMask{BlockMaskOffset{3}}, BlockMask{BlockMaskVector{true}},
                                              BlockMask{BlockMaskOffset{0}}}, &codes), KVCM_EC_BADARGS);
    EXPECT_EQ(searcher.FinishWriteCacheBatch({BlockMask{BlockMaskOffset{3}}, BlockMask{BlockMaskVector{true, false}},
                                              BlockMask{BlockMaskOffset{0}}}, &codes), KVCM_OK);
    EXPECT_EQ(codes[0] | codes[1] | codes[2], KVCM_OK);
    EXPECT_EQ(searcher.PrefixMatch({11, 12, 14, 15}, BlockMask{}, &len), KVCM_OK);
    EXPECT_EQ(len, size_t(3));  // 15 failed and is gone
    std::vector<uint8_t> flags;
    EXPECT_EQ(searcher.BatchGet({15, 99}, &flags), KVCM_OK);
    EXPECT_EQ(int(flags[0]), 0);
    EXPECT_EQ(int(flags[1]), 0);
}

static void TestIovCopier() {
    // a block of 3 layers x (K,V) iovs with one ignored iov in the middle
    const size_t sz = 4096;
    std::vector<uint8_t> host(6 * sz);
    for (size_t i = 0; i < host.size(); ++i) host[i] = static_cast<uint8_t>(i * 7 + i / sz);
    uint8_t *d_src = nullptr, *d_string = nullptr, *d_back = nullptr;
    cudaMalloc(&d_src, host.size());
    cudaMalloc(&d_string, host.size());
    cudaMalloc(&d_back, host.size());
    cudaMemcpy(d_src, host.data(), host.size(), cudaMemcpyHostToDevice);
    cudaMemset(d_string, 0, host.size());
    cudaMemset(d_back, 0, host.size());
    BlockBuffer put, get;
    for (int i = 0; i < 6; ++i) {
        put.iovs.push_back({MemoryType::GPU, d_src + i * sz, sz, i == 2});
        get.iovs.push_back({MemoryType::GPU, d_back + i * sz, sz, i == 2});
    }
    IovCopier copier;
    uint64_t span = 0;
    EXPECT_EQ(copier.CopyIovs(put, d_string, 0, &span), KVCM_OK);
    EXPECT_EQ(span, uint64_t(6 * sz));
    EXPECT_EQ(copier.CopyIovs(get, d_string, 1, &span), KVCM_OK);
    cudaDeviceSynchronize();
    std::vector<uint8_t> back(host.size());
    cudaMemcpy(back.data(), d_back, back.size(), cudaMemcpyDeviceToHost);
    for (int i = 0; i < 6; ++i) {
        bool same = std::memcmp(back.data() + i * sz, host.data() + i * sz, sz) == 0;
        bool zero = true;
        for (size_t j = 0; j < sz; ++j) zero = zero && back[i * sz + j] == 0;
        EXPECT_EQ(i == 2 ? zero : same, true);
    }
    // The same block with its string in pinned host memory (what LocalFileSdk's registered mmap is), staged through
    // the bounce buffer and read / written by the kernel directly: the bytes under the ignored iov stay as they were.
    uint8_t *h_string = nullptr;
    cudaMallocHost(&h_string, host.size());
    for (int mode = 0; mode < 2; ++mode) {
        IovCopier host_copier(nullptr, mode == 0);
        std::memset(h_string, 0xEE, host.size());
        cudaMemset(d_back, 0, host.size());
        EXPECT_EQ(host_copier.CopyIovs(put, h_string, 0, &span), KVCM_OK);
        cudaDeviceSynchronize();
        for (int i = 0; i < 6; ++i) {
            bool same = std::memcmp(h_string + i * sz, host.data() + i * sz, sz) == 0;
            bool kept = true;
            for (size_t j = 0; j < sz; ++j) kept = kept && h_string[i * sz + j] == 0xEE;
            EXPECT_EQ(i == 2 ? kept : same, true);
        }
        EXPECT_EQ(host_copier.CopyIovs(get, h_string, 1, &span), KVCM_OK);
        cudaDeviceSynchronize();
        cudaMemcpy(back.data(), d_back, back.size(), cudaMemcpyDeviceToHost);
        for (int i = 0; i < 6; ++i) {
            bool same = std::memcmp(back.data() + i * sz, host.data() + i * sz, sz) == 0;
            bool zero = true;
            for (size_t j = 0; j < sz; ++j) zero = zero && back[i * sz + j] == 0;
            EXPECT_EQ(i == 2 ? zero : same, true);
        }
    }
    // pageable host memory is refused, not dereferenced
    std::vector<uint8_t> pageable(host.size());
    EXPECT_EQ(copier.CopyIovs(put, pageable.data(), 0, &span), KVCM_ER_UNSUPPORTED_MEMORY_TYPE);
    // Iovs of MemoryType::CPU in ordinary malloc'ed memory (the reference copies those with std::memcpy,
    // local_file_sdk.cc:231-233,339-341) mixed with GPU iovs: iovs 1 and 4 live on the host.  With a device
    // string, with a pinned host string through the bounce buffer, and with the kernel on the host string itself.
    std::vector<uint8_t> cpu_src(2 * sz), cpu_back(2 * sz);
    std::memcpy(cpu_src.data(), host.data() + 1 * sz, sz);
    std::memcpy(cpu_src.data() + sz, host.data() + 4 * sz, sz);
    BlockBuffer mput = put, mget = get;
    mput.iovs[1] = {MemoryType::CPU, cpu_src.data(), sz, false};
    mput.iovs[4] = {MemoryType::CPU, cpu_src.data() + sz, sz, false};
    mget.iovs[1] = {MemoryType::CPU, cpu_back.data(), sz, false};
    mget.iovs[4] = {MemoryType::CPU, cpu_back.data() + sz, sz, false};
    for (int mode = 0; mode < 3; ++mode) {
        IovCopier mixed(nullptr, mode != 2);
        uint8_t *string = mode == 0 ? d_string : h_string;
        if (mode == 0) {
            cudaMemset(d_string, 0xEE, host.size());
        } else {
            std::memset(h_string, 0xEE, host.size());
        }
        cudaMemset(d_back, 0, host.size());
        std::fill(cpu_back.begin(), cpu_back.end(), 0);
        EXPECT_EQ(mixed.CopyIovs(mput, string, 0, &span), KVCM_OK);
        EXPECT_EQ(span, uint64_t(6 * sz));
        cudaDeviceSynchronize();
        std::vector<uint8_t> str(host.size());
        cudaMemcpy(str.data(), string, str.size(), cudaMemcpyDefault);
        for (int i = 0; i < 6; ++i) {
            bool same = std::memcmp(str.data() + i * sz, host.data() + i * sz, sz) == 0;
            bool kept = true;
            for (size_t j = 0; j < sz; ++j) kept = kept && str[i * sz + j] == 0xEE;
            EXPECT_EQ(i == 2 ? kept : same, true);
        }
        EXPECT_EQ(mixed.CopyIovs(mget, string, 1, &span), KVCM_OK);
        cudaDeviceSynchronize();
        cudaMemcpy(back.data(), d_back, back.size(), cudaMemcpyDeviceToHost);
        for (int i = 0; i < 6; ++i) {
            if (i == 1 || i == 4) {
                EXPECT_EQ(std::memcmp(cpu_back.data() + (i == 1 ? 0 : sz), host.data() + i * sz, sz), 0);
            } else if (i != 2) {
                EXPECT_EQ(std::memcmp(back.data() + i * sz, host.data() + i * sz, sz), 0);
            }
        }
    }
    // the C entry point by itself never puts a pageable CPU base into a table a kernel would read
    {
        kvcm_b200_iov_t one{};
        one.type = 0;
        one.base = cpu_src.data();
        one.size = sz;
        kvcm_b200_seg_t seg{};
        int32_t n_segs = -1;
        EXPECT_EQ(kvcm_b200_iovs_to_segments(&one, 1, d_string, 0, &seg, &n_segs, nullptr),
                  KVCM_ER_UNSUPPORTED_MEMORY_TYPE);
        one.base = h_string;  // pinned: a kernel can address it
        EXPECT_EQ(kvcm_b200_iovs_to_segments(&one, 1, d_string, 0, &seg, &n_segs, nullptr), KVCM_OK);
        EXPECT_EQ(n_segs, 1);
    }
    cudaFreeHost(h_string);
    cudaFree(d_src);
    cudaFree(d_string);
    cudaFree(d_back);
}

static void TestReplay() {
    // kv_cache_manager/optimizer/test/optimizer_manager_py_test.py:57-84: write [1,2,3], query [1,2,4] -> hit 2
    GpuTraceReplayer replayer;
    std::vector<ReplayRecord> rec;
    EXPECT_EQ(replayer.RunTraces({{TraceKind::WriteCache, {1, 2, 3}}, {TraceKind::GetLocation, {1, 2, 4}}}, &rec),
              KVCM_OK);
    EXPECT_EQ(rec[0].write_blocks, 3);
    EXPECT_EQ(rec[1].external_hit_blocks, 2);
    EXPECT_EQ(rec[1].current_cache_blocks, 3);
    // dialog turns read and write in one step; a masked key that is cached counts as an internal hit
    EXPECT_EQ(replayer.RunTraces({{TraceKind::DialogTurn, {1, 2, 3}},
                                  {TraceKind::DialogTurn, {1, 2, 4, 5}},
                                  {TraceKind::GetLocation, {1, 2, 4}, 1}},
                                 &rec),
              KVCM_OK);
    EXPECT_EQ(rec[1].external_hit_blocks, 2);
    EXPECT_EQ(rec[1].write_blocks, 2);
    EXPECT_EQ(rec[2].external_hit_blocks, 2);
    EXPECT_EQ(rec[2].internal_hit_blocks, 1);
    EXPECT_EQ(rec[2].current_cache_blocks, 5);
    EXPECT_EQ(replayer.RunTraces({}, &rec), KVCM_OK);
    // kv_cache_manager/optimizer/test/lru_eviction_policy_test.cc:44-65 as traces: write 1, write 2, read 1; a third
    // block then overflows a quota of 2 and the least recently used block, 2, goes.  With room for all, nothing goes.
    std::vector<std::vector<ReplayRecord>> sweep;
    const std::vector<ReplayTrace> lru = {{TraceKind::WriteCache, {1}},  {TraceKind::WriteCache, {2}},
                                          {TraceKind::GetLocation, {1}}, {TraceKind::WriteCache, {3}},
                                          {TraceKind::GetLocation, {2}}, {TraceKind::GetLocation, {1}}};
    EXPECT_EQ(replayer.RunTracesLru(lru, {2, 100}, 1, true, &sweep), KVCM_OK);
    EXPECT_EQ(sweep.size(), 2u);
    EXPECT_EQ(sweep[0][2].external_hit_blocks, 1);
    EXPECT_EQ(sweep[0][3].current_cache_blocks, 2);
    EXPECT_EQ(sweep[0][4].external_hit_blocks, 0);
    EXPECT_EQ(sweep[0][5].external_hit_blocks, 1);
    EXPECT_EQ(sweep[1][4].external_hit_blocks, 1);
    EXPECT_EQ(sweep[1][5].current_cache_blocks, 3);
    EXPECT_EQ(replayer.RunTracesLru(lru, {}, 1, true, &sweep), KVCM_EC_BADARGS);
    // "leaf_aware_lru" (no test in the reference; worked from eviction_policy/leaf_aware_lru.cc:85-133): [1,2,3] then
    // [1,2,9] splits the node; with room for three blocks the shared prefix 1,2 stays and the leaf block 3 goes, where
    // plain LRU drops block 1.
    const std::vector<ReplayTrace> shared = {{TraceKind::WriteCache, {1, 2, 3}}, {TraceKind::WriteCache, {1, 2, 9}},
                                             {TraceKind::GetLocation, {1, 2, 3}}};
    EXPECT_EQ(replayer.RunTracesLru(shared, {3}, 1, true, &sweep, /*leaf_aware=*/true), KVCM_OK);
    EXPECT_EQ(sweep[0][2].external_hit_blocks, 2);
    EXPECT_EQ(sweep[0][2].current_cache_blocks, 3);
    EXPECT_EQ(replayer.RunTracesLru(shared, {3}, 1, true, &sweep), KVCM_OK);
    EXPECT_EQ(sweep[0][2].external_hit_blocks, 0);
    // Two instances share a quota of 4 blocks (worked from kv_cache_manager/optimizer/manager/eviction_manager.cc:86-192;
    // the reference tests groups of one instance only): a writes 1 2 3, b writes 1 2.  GROUP_ROUGH takes one block
    // from a and one from b; INSTANCE_ROUGH takes one from the writer b only.
    const std::vector<ReplayTrace> two = {{TraceKind::WriteCache, {1, 2, 3}}, {TraceKind::WriteCache, {1, 2}},
                                          {TraceKind::GetLocation, {1, 2, 3}}, {TraceKind::GetLocation, {1, 2}}};
    std::vector<int64_t> usage;
    EXPECT_EQ(replayer.RunTracesLruGroup(two, {0, 1, 0, 1}, 2, 4, 1, 1, &rec, &usage), KVCM_OK);
    EXPECT_EQ(rec[1].current_cache_blocks, 1);
    EXPECT_EQ(rec[2].external_hit_blocks, 0);
    EXPECT_EQ(usage[0], 2);
    EXPECT_EQ(usage[1], 1);
    EXPECT_EQ(replayer.RunTracesLruGroup(two, {0, 1, 0, 1}, 2, 4, 1, 2, &rec, &usage), KVCM_OK);
    EXPECT_EQ(rec[2].external_hit_blocks, 3);
    EXPECT_EQ(usage[0], 3);
    EXPECT_EQ(replayer.RunTracesLruGroup(two, {0, 1}, 2, 4, 1, 2, &rec, &usage), KVCM_EC_BADARGS);
    // The same two instances under "leaf_aware_lru", quota 5, batches of 1, group rough (worked by hand from
    // kv_cache_manager/optimizer/eviction_policy/leaf_aware_lru.cc:85-160 over eviction_manager.cc:86-146): a's split
    // node {1 2} stays while its children {3} and {9} go, is queued again when the last of them has gone, and so
    // a still hits 1 2 at the end; b loses the head of its only chain at once.
    const std::vector<ReplayTrace> leafy = {
        {TraceKind::WriteCache, {1, 2, 3}}, {TraceKind::WriteCache, {1, 2, 9}}, {TraceKind::WriteCache, {1, 2}},
        {TraceKind::GetLocation, {1, 2, 3}}, {TraceKind::GetLocation, {1, 2}}, {TraceKind::WriteCache, {5}},
        {TraceKind::WriteCache, {7, 8}}, {TraceKind::GetLocation, {1, 2, 9}}, {TraceKind::WriteCache, {6}}};
    EXPECT_EQ(replayer.RunTracesLruGroup(leafy, {0, 0, 1, 0, 1, 0, 1, 0, 0}, 2, 5, 1, 1, &rec, &usage, /*leaf_aware=*/true),
              KVCM_OK);
    EXPECT_EQ(rec[3].external_hit_blocks, 2);
    EXPECT_EQ(rec[4].external_hit_blocks, 0);
    EXPECT_EQ(rec[7].external_hit_blocks, 2);
    EXPECT_EQ(rec[6].current_cache_blocks, 2);
    EXPECT_EQ(usage[0], 3);
    EXPECT_EQ(usage[1], 1);
    // An "lru" instance a and a "random_lru" instance b (sample_rate 1, batches of 1: one index is drawn per round)
    // share a quota of 4, group rough.  RandomLruEvictionPolicy's generator (random_lru.h:20, random_lru.cc:121-131)
    // starts at 0x12345678ABCDEF01; its first draw is odd, its second a multiple of 3.  a writes 1 2 3, b writes 4 5:
    // a loses 1 and b - draw mod 2 = 1 - loses 5, where a queue would have taken 4; so b's read of 4 5 hits once.
    // b writes 4 5 7 (two new blocks): a loses 2 and b - draw mod 3 = 0 - loses 4, 7 takes its place.
    const std::vector<ReplayTrace> sampled = {
        {TraceKind::WriteCache, {1, 2, 3}}, {TraceKind::WriteCache, {4, 5}}, {TraceKind::GetLocation, {4, 5}},
        {TraceKind::GetLocation, {1, 2, 3}}, {TraceKind::WriteCache, {4, 5, 7}}, {TraceKind::GetLocation, {4, 5, 7}}};
    EXPECT_EQ(replayer.RunTracesPolicyGroup(sampled, {0, 1, 1, 0, 1, 1}, {KVCM_POLICY_LRU, KVCM_POLICY_RANDOM_LRU},
                                            {0.0, 1.0}, 4, 1, 1, &rec, &usage),
              KVCM_OK);
    EXPECT_EQ(rec[2].external_hit_blocks, 1);
    EXPECT_EQ(rec[3].external_hit_blocks, 0);
    EXPECT_EQ(rec[4].write_blocks, 2);
    EXPECT_EQ(rec[5].external_hit_blocks, 0);
    EXPECT_EQ(usage[0], 1);
    EXPECT_EQ(usage[1], 2);
    EXPECT_EQ(replayer.RunTracesPolicyGroup(sampled, {0, 1, 1, 0, 1, 1}, {KVCM_POLICY_LRU, KVCM_POLICY_LRU}, {}, 4, 1, 1,
                                            &rec, &usage),
              KVCM_OK);
    EXPECT_EQ(rec[2].external_hit_blocks, 0);  // the queue takes 4, and 4 5 is no hit without its first block
    EXPECT_EQ(replayer.RunTracesPolicyGroup(sampled, {0, 1, 1, 0, 1, 1}, {KVCM_POLICY_LRU, 7}, {}, 4, 1, 1, &rec, &usage),
              KVCM_EC_OUT_OF_LIMIT);
}

int main() {
    int32_t sms = 0;
    if (kvcm_b200_device_info(&sms, nullptr, nullptr, nullptr) != KVCM_OK) {
        std::printf("no CUDA device: the adapters have no CPU path\n");
        return 2;
    }
    TestHash();
    TestPrefixMatch();
    TestSlidingWindowAndBatchGet();
    TestWriteCycle();
    TestWriteBatch();
    TestIovCopier();
    TestReplay();
    std::printf(g_failed == 0 ? "host adapter test: all checks passed\n" : "host adapter test: %d checks FAILED\n", g_failed);
    return g_failed == 0 ? 0 : 1;
}
