// Bench infrastructure, not product code: the STRUCTURE of the reference's iov copies, for timing
// beside kvcm_b200_copy_segments on the same buffers.  The reference issues one cudaMemcpyAsync per
// iov and synchronises the stream once per request
// (kv_cache_manager/client/src/internal/sdk/local_file_sdk.cc:223-252 for Get, :326-359 for Put;
// kv_cache_manager/client/src/internal/sdk/hf3fs_usrbio_client.cc:478-505).
#include <cuda_runtime.h>

#include <cstdint>

extern "C" {

// Copies n ranges, one call each, then waits for the stream.  Returns 0, or the first CUDA error.
int kvcm_ref_memcpy_loop(void *const *dst, void *const *src, const uint64_t *bytes, int64_t n, void *stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    for (int64_t i = 0; i < n; ++i) {
        const cudaError_t e = cudaMemcpyAsync(dst[i], src[i], bytes[i], cudaMemcpyDefault, s);
        if (e != cudaSuccess) return static_cast<int>(e);
    }
    return static_cast<int>(cudaStreamSynchronize(s));
}

}  // extern "C"
