// pybind11 shim for py_connector: the gather / scatter entry points of libkvcm_b200.so with device
// addresses and the stream passed as integers (tensor.data_ptr(), stream.cuda_stream), the way the
// reference binds its client for Python (kv_cache_manager/client/pybind/py_client_binding.cc:17-125,
// GIL released around every call).  No torch, no CUDA headers: it only forwards to the C ABI.
#include <pybind11/pybind11.h>

#include <cstdint>

#include "kvcm_b200.h"

namespace py = pybind11;

namespace {

template <class T>
T *Ptr(uint64_t address) {
    return reinterpret_cast<T *>(static_cast<uintptr_t>(address));
}

using MoveFn = int32_t (*)(const void *const *, int32_t, void *, int64_t, const int32_t *, const int32_t *, int32_t,
                           int32_t, int64_t, int64_t, uint32_t *, int32_t, kvcm_stream_t);

template <MoveFn fn>
int32_t Move(uint64_t pool_ptrs, int32_t n_pools, uint64_t staging, int64_t n_slots, uint64_t row_idx,
             uint64_t slot_idx, int32_t n_blocks, int32_t rows_per_block, int64_t row_bytes, int64_t pool_rows,
             uint64_t status, int32_t max_sms, uint64_t stream) {
    return fn(Ptr<const void *const>(pool_ptrs), n_pools, Ptr<void>(staging), n_slots, Ptr<const int32_t>(row_idx),
              Ptr<const int32_t>(slot_idx), n_blocks, rows_per_block, row_bytes, pool_rows, Ptr<uint32_t>(status),
              max_sms, Ptr<void>(stream));
}

int32_t ScatterTokens(const void *const *a, int32_t b, void *c, int64_t d, const int32_t *e, const int32_t *f,
                      int32_t g, int32_t h, int64_t i, int64_t j, uint32_t *k, int32_t l, kvcm_stream_t m) {
    return kvcm_b200_scatter_tokens(a, b, c, d, e, f, g, h, i, j, k, l, m);
}
int32_t ScatterPages(const void *const *a, int32_t b, void *c, int64_t d, const int32_t *e, const int32_t *f,
                     int32_t g, int32_t h, int64_t i, int64_t j, uint32_t *k, int32_t l, kvcm_stream_t m) {
    return kvcm_b200_scatter_pages(a, b, c, d, e, f, g, h, i, j, k, l, m);
}

template <bool kSave>
int32_t HostMove(uint64_t pool_ptrs, int32_t n_pools, uint64_t h_staging, int64_t n_slots, uint64_t row_idx,
                 uint64_t h_slot_idx, int32_t n_blocks, int32_t rows_per_block, int64_t row_bytes, int64_t pool_rows,
                 uint64_t bounce, int64_t bounce_bytes, uint64_t status, uint64_t stream) {
    if (kSave) {
        return kvcm_b200_save_rows_to_host(Ptr<const void *const>(pool_ptrs), n_pools, Ptr<void>(h_staging), n_slots,
                                           Ptr<const int32_t>(row_idx), Ptr<const int32_t>(h_slot_idx), n_blocks,
                                           rows_per_block, row_bytes, pool_rows, Ptr<void>(bounce), bounce_bytes,
                                           Ptr<uint32_t>(status), Ptr<void>(stream));
    }
    return kvcm_b200_load_rows_from_host(Ptr<const void *const>(pool_ptrs), n_pools, Ptr<const void>(h_staging),
                                         n_slots, Ptr<const int32_t>(row_idx), Ptr<const int32_t>(h_slot_idx),
                                         n_blocks, rows_per_block, row_bytes, pool_rows, Ptr<void>(bounce),
                                         bounce_bytes, Ptr<uint32_t>(status), Ptr<void>(stream));
}

template <bool kGather>
int32_t Legacy(uint64_t layer_ptrs, int32_t n_layers, int64_t total_tokens, uint64_t staging, uint64_t token_idx,
               int32_t n_tokens, int64_t hidden_bytes, uint64_t stream) {
    if (kGather) {
        return kvcm_b200_gather_legacy(Ptr<const void *const>(layer_ptrs), n_layers, total_tokens, Ptr<void>(staging),
                                       Ptr<const int32_t>(token_idx), n_tokens, hidden_bytes, Ptr<void>(stream));
    }
    return kvcm_b200_scatter_legacy(Ptr<const void *const>(layer_ptrs), n_layers, total_tokens,
                                    Ptr<const void>(staging), Ptr<const int32_t>(token_idx), n_tokens, hidden_bytes,
                                    Ptr<void>(stream));
}

}  // namespace

PYBIND11_MODULE(kvcm_b200_py, m) {
    m.doc() = "pybind shim over the C ABI of libkvcm_b200.so (gather / scatter for py_connector)";
    const auto release = py::call_guard<py::gil_scoped_release>();
    m.def("abi_version", &kvcm_b200_abi_version);
    m.def("set_device", &kvcm_b200_set_device, release);
    m.def("error_string", [](int32_t code) { return std::string(kvcm_b200_error_string(code)); });
    m.def("gather_tokens", &Move<&kvcm_b200_gather_tokens>, release);
    m.def("scatter_tokens", &Move<&ScatterTokens>, release);
    m.def("gather_pages", &Move<&kvcm_b200_gather_pages>, release);
    m.def("scatter_pages", &Move<&ScatterPages>, release);
    m.def("save_rows_to_host", &HostMove<true>, release);
    m.def("load_rows_from_host", &HostMove<false>, release);
    m.def("gather_legacy", &Legacy<true>, release);
    m.def("scatter_legacy", &Legacy<false>, release);
}
