// TEST INFRASTRUCTURE ONLY.  A C-callable driver around the REFERENCE's own Optimizer, compiled from the
// reference's source files where they lie (oracle/Makefile, target ref_optimizer): its radix tree
// (kv_cache_manager/optimizer/index/radix_tree_index.cc), its three eviction policies
// (kv_cache_manager/optimizer/eviction_policy/{lru,leaf_aware_lru,random_lru}.cc), its eviction and indexer
// managers (kv_cache_manager/optimizer/manager/{eviction_manager,indexer_manager}.cc), its runner
// (manager/optimizer_runner.cc), its trace loaders and its result writer
// (kv_cache_manager/optimizer/analysis/result_analysis.cc).  Nothing of the reference is copied here: this file
// only builds an OptimizerManager from a configuration file, feeds it traces through the runner's own handlers
// and reads the runner's own records back.  It exists to pin oracle/kvcm_oracle.cc - the restatement the GPU
// kernels are compared with - to the reference itself, for the parts of the Optimizer the reference's tests
// do not cover (leaf_aware_lru, random_lru, groups of instances, the hit-rate CSV, the publisher-log reader).
//
// Two things the reference's build links and this one does not have: its logging back end (alog).  The two
// symbols the compiled sources need from it are defined below as "nothing is logged".  JSON comes from the
// header-only rapidjson found on this image at build time.
// Built with -fno-access-control: the manager keeps its runner and its records private, and the reference offers
// no accessor for the per-trace records.
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <memory>
#include <string>
#include <vector>

#include "kv_cache_manager/common/logger.h"
#include "kv_cache_manager/optimizer/config/optimizer_config_loader.h"
#include "kv_cache_manager/optimizer/manager/optimizer_loader.h"
#include "kv_cache_manager/optimizer/manager/optimizer_manager.h"

namespace kv_cache_manager {
uint32_t LoggerBroker::base_log_level_ = Logger::LEVEL_UNSET;  // IsLevelEnable() is then false for every level
void LoggerBroker::Log(int, const char *, int, const char *, const char *, ...) {}
}  // namespace kv_cache_manager

namespace {

struct RefOptimizer {
    std::unique_ptr<kv_cache_manager::OptimizerManager> manager;
};

}  // namespace

extern "C" {

// The configuration file is the Optimizer's own startup configuration (optimizer_startup_config_load.json's format).
void *kvcm_ref_optimizer_create(const char *config_path) {
    kv_cache_manager::OptimizerConfigLoader loader;
    if (config_path == nullptr || !loader.Load(config_path)) return nullptr;
    auto *h = new RefOptimizer();
    h->manager.reset(new kv_cache_manager::OptimizerManager(loader.get_config()));
    if (!h->manager->Init()) {
        delete h;
        return nullptr;
    }
    return h;
}

void kvcm_ref_optimizer_destroy(void *handle) { delete static_cast<RefOptimizer *>(handle); }

// Replays traces through OptimizerRunner::HandleDialogTurn / HandleGetLocation / HandleWriteCache
// (type 0 / 1 / 2) in the order given.  Trace t owns keys[key_off[t], key_off[t+1]) and belongs to
// instance_ids[trace_inst[t]].  A GetLocation trace is masked by the offset mask_off[t] or, when mask_bits is
// given, by the vector mask_bits[key_off[t] ...) (one byte per key).  Outputs per trace: the runner's own record
// (external / internal hit blocks of the read record, write_blocks of the write record) and, asked of the
// eviction manager after the trace, the usage of the trace's instance and of every instance (inst_blocks,
// optional, [n_traces][n_instances] in the order of instance_ids).
int32_t kvcm_ref_optimizer_run(void *handle, const char *const *instance_ids, int32_t n_instances, const int64_t *keys,
                               const int64_t *key_off, const uint8_t *type, const int64_t *mask_off,
                               const uint8_t *mask_bits, const int64_t *timestamps, const int32_t *trace_inst,
                               int64_t n_traces, int32_t *ext_hit, int32_t *int_hit, int32_t *written,
                               int64_t *cache_blocks, int64_t *inst_blocks) {
    using namespace kv_cache_manager;
    auto *h = static_cast<RefOptimizer *>(handle);
    if (h == nullptr || n_instances <= 0) return -1;
    OptimizerManager &m = *h->manager;
    for (int64_t t = 0; t < n_traces; ++t) {
        const int32_t j = trace_inst != nullptr ? trace_inst[t] : 0;
        if (j < 0 || j >= n_instances) return -2;
        const std::string id = instance_ids[j];
        auto result_it = m.result_map_.find(id);
        if (result_it == m.result_map_.end()) return -3;
        Result &result = *result_it->second;
        const std::vector<int64_t> k(keys + key_off[t], keys + key_off[t + 1]);
        const int64_t ts = timestamps != nullptr ? timestamps[t] : t;
        const size_t reads = result.read_results.size(), writes = result.write_results.size();
        if (type[t] == 2) {
            WriteCacheSchemaTrace trace;
            trace.set_instance_id(id);
            trace.set_trace_id("t" + std::to_string(t));
            trace.set_timestamp_us(ts);
            trace.set_keys(k);
            m.optimizer_runner_->HandleWriteCache(trace);
        } else if (type[t] == 1) {
            GetLocationSchemaTrace trace;
            trace.set_instance_id(id);
            trace.set_trace_id("t" + std::to_string(t));
            trace.set_timestamp_us(ts);
            trace.set_keys(k);
            trace.set_query_type("prefix_match");
            if (mask_bits != nullptr) {
                BlockMaskVector bits(k.size());
                for (size_t i = 0; i < k.size(); ++i) bits[i] = mask_bits[key_off[t] + static_cast<int64_t>(i)] != 0;
                trace.set_block_mask(BlockMask(bits));
            } else {
                trace.set_block_mask(BlockMask(static_cast<BlockMaskOffset>(mask_off != nullptr ? mask_off[t] : 0)));
            }
            m.optimizer_runner_->HandleGetLocation(trace);
        } else {
            DialogTurnSchemaTrace trace;
            trace.set_instance_id(id);
            trace.set_trace_id("t" + std::to_string(t));
            trace.set_timestamp_us(ts);
            trace.set_keys(k);
            trace.set_total_keys(k);
            trace.set_query_type("prefix_match");
            m.optimizer_runner_->HandleDialogTurn(trace);
        }
        ext_hit[t] = int_hit[t] = written[t] = 0;
        if (result.read_results.size() > reads) {
            ext_hit[t] = static_cast<int32_t>(result.read_results.back().external_hit_blocks);
            int_hit[t] = static_cast<int32_t>(result.read_results.back().internal_hit_blocks);
        }
        if (result.write_results.size() > writes) {
            written[t] = static_cast<int32_t>(result.write_results.back().write_blocks);
        }
        cache_blocks[t] = static_cast<int64_t>(m.eviction_manager_->GetCurrentInstanceUsage(id));
        if (inst_blocks != nullptr) {
            for (int32_t i = 0; i < n_instances; ++i) {
                inst_blocks[t * n_instances + i] =
                    static_cast<int64_t>(m.eviction_manager_->GetCurrentInstanceUsage(instance_ids[i]));
            }
        }
    }
    return 0;
}

// The traces OptimizerLoader::LoadTrace makes of the trace file the configuration names, in replay order, one line
// per trace into out_path: the kind (0 dialog turn, 1 GetLocation, 2 WriteCache), a space, the trace's own JSON.
// Returns the number of traces, -1 on failure.
int64_t kvcm_ref_optimizer_dump_traces(const char *config_path, const char *out_path) {
    using namespace kv_cache_manager;
    OptimizerConfigLoader loader;
    if (config_path == nullptr || out_path == nullptr || !loader.Load(config_path)) return -1;
    OptimizerConfig config = loader.get_config();
    auto traces = OptimizerLoader::LoadTrace(config);
    std::ofstream out(out_path);
    if (!out.is_open()) return -1;
    for (const auto &trace : traces) {
        int kind = 2;
        if (std::dynamic_pointer_cast<DialogTurnSchemaTrace>(trace)) {
            kind = 0;
        } else if (std::dynamic_pointer_cast<GetLocationSchemaTrace>(trace)) {
            kind = 1;
        }
        out << kind << ' ' << trace->ToJsonString() << '\n';
    }
    return static_cast<int64_t>(traces.size());
}

// What `optimizer_main <config>` does after loading its configuration (kv_cache_manager/optimizer/main.cc): load
// the trace file the configuration names, replay it, write the per-instance hit-rate CSV files.
int32_t kvcm_ref_optimizer_main(const char *config_path) {
    void *handle = kvcm_ref_optimizer_create(config_path);
    if (handle == nullptr) return -1;
    auto *h = static_cast<RefOptimizer *>(handle);
    h->manager->DirectRun();
    h->manager->AnalyzeResults();
    if (getenv("KVCM_DBG_NODESTROY") == nullptr) kvcm_ref_optimizer_destroy(handle);
    return 0;
}

}  // extern "C"
