// ckv_attention_static: the attention entry point for callers that cannot hand the library a
// scratch buffer.  The scratch lives in a fixed array inside the library's own device image.
#include <mutex>

#include "ckv_common.cuh"

namespace ckv {

namespace {

// Every GPU that loads this library carries this array until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[CKV_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void *g_scratch_ptr[kMaxDevices] = {};
std::mutex g_scratch_mutex;   // two host threads may make the first call on a device at the same time

// The array's name is only a host-side handle; kernels need its device address, which differs per
// device and is looked up once per device while that device is current.
int static_scratch_address(void **ptr) {
    int dev = 0;
    CKV_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(CKV_E_UNSUPPORTED, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ptr[dev]) {
        void *p = nullptr;
        CKV_CUDA_CHECK(cudaGetSymbolAddress(&p, g_static_scratch));
        g_scratch_ptr[dev] = p;
    }
    *ptr = g_scratch_ptr[dev];
    return CKV_OK;
}

}  // namespace

}  // namespace ckv

using namespace ckv;

extern "C" size_t ckv_static_scratch_bytes(void) { return (size_t)CKV_STATIC_SCRATCH_BYTES; }

// The status word of the built-in scratch array of the current device (its first four bytes, where
// every attention call keeps it): the caller of ckv_attention_static has no workspace pointer to hand
// to ckv_read_status.  A 4-byte device-to-host copy; allocates nothing.
extern "C" int ckv_static_status(int32_t *status) {
    if (!status) return fail(CKV_E_ARG, "status is null");
    void *scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != CKV_OK) return rc;
    CKV_CUDA_CHECK(cudaMemcpy(status, scratch, 4, cudaMemcpyDeviceToHost));
    return CKV_OK;
}

extern "C" int ckv_attention_static(const ckv_config *cfg, const ckv_layer_state *st, const void *q,
                                    int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_t, const void *key,
                                    const void *value, int64_t kv_stride_b, int64_t kv_stride_h, int64_t kv_stride_t,
                                    int32_t n_tokens, const void *rope, int64_t rope_rows, const float *ema_w_cache,
                                    const void *ema_w_new, void *out, int64_t o_stride_b, int64_t o_stride_h,
                                    int64_t o_stride_t, int32_t flags, void *cuda_stream) {
    const size_t need = ckv_attention_workspace_bytes_for(cfg, n_tokens, flags);
    if (need == 0) return fail(CKV_E_ARG, "invalid configuration or n_tokens");
    if (need > (size_t)CKV_STATIC_SCRATCH_BYTES)
        return fail(CKV_E_WORKSPACE,
                    "this configuration needs %zu bytes of scratch but the built-in array holds %zu; use "
                    "ckv_attention with a caller-provided workspace",
                    need, (size_t)CKV_STATIC_SCRATCH_BYTES);
    void *scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != CKV_OK) return rc;
    return ckv_attention(cfg, st, q, q_stride_b, q_stride_h, q_stride_t, key, value, kv_stride_b, kv_stride_h,
                         kv_stride_t, n_tokens, rope, rope_rows, ema_w_cache, ema_w_new, out, o_stride_b, o_stride_h,
                         o_stride_t, scratch, (size_t)CKV_STATIC_SCRATCH_BYTES, flags, cuda_stream);
}
