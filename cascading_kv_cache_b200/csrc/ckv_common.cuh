// Shared declarations of the cascade_kv_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/cascade_kv_b200.h"

#define CKV_MAX_CASCADES 64

namespace ckv {

// Record a failure message for ckv_last_error() and return the code.
int fail(int code, const char *fmt, ...);

#define CKV_CUDA_CHECK(expr)                                                              \
    do {                                                                                  \
        cudaError_t _e = (expr);                                                          \
        if (_e != cudaSuccess)                                                            \
            return ::ckv::fail(CKV_E_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

struct Dims {
    int B, KVH, H, G, D, NS, W, C, S;
    int dtype, esz;
    int eager_fill, head_reduction, homogeneous, admission;
    double beta;
};

inline int make_dims(const ckv_config *cfg, Dims *d) {
    if (!cfg) return fail(CKV_E_ARG, "cfg is null");
    d->B = cfg->batch; d->KVH = cfg->kv_heads; d->H = cfg->q_heads; d->D = cfg->head_dim;
    d->NS = cfg->num_sinks; d->W = cfg->window; d->C = cfg->cascades;
    d->dtype = cfg->dtype;
    if (d->B <= 0 || d->KVH <= 0 || d->H <= 0 || d->D <= 0 || d->W <= 0 || d->C <= 0 || d->NS < 0)
        return fail(CKV_E_ARG, "non-positive dimension in ckv_config");
    if (d->H % d->KVH != 0) return fail(CKV_E_ARG, "q_heads (%d) is not a multiple of kv_heads (%d)", d->H, d->KVH);
    if (d->C > CKV_MAX_CASCADES) return fail(CKV_E_UNSUPPORTED, "more than %d cascades", CKV_MAX_CASCADES);
    if (d->dtype != CKV_F32 && d->dtype != CKV_F16 && d->dtype != CKV_BF16)
        return fail(CKV_E_ARG, "unknown dtype code %d", d->dtype);
    if ((int64_t)d->W * d->C > (int64_t)1 << 30) return fail(CKV_E_UNSUPPORTED, "cache too long");
    d->G = d->H / d->KVH;
    d->S = d->W * d->C;
    d->esz = d->dtype == CKV_F32 ? 4 : 2;
    d->eager_fill = cfg->eager_fill != 0;
    d->head_reduction = cfg->head_reduction;
    d->homogeneous = cfg->homogeneous_heads != 0;
    d->admission = cfg->admission;
    d->beta = cfg->beta;
    if (d->head_reduction < CKV_REDUCE_MEAN || d->head_reduction > CKV_REDUCE_MEDIAN)
        return fail(CKV_E_ARG, "unknown head_reduction %d", d->head_reduction);
    return CKV_OK;
}

// ---- element type helpers ---------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
    static __device__ __forceinline__ float to_f(float x) { return x; }
    static __device__ __forceinline__ float from_f(float x) { return x; }
};
template <> struct Elem<__half> {
    static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
    static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
};
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
    static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
};

// Round an fp32 value to the storage type and back: the reference computes in the
// activation dtype, so every torch op boundary is a rounding point.
template <typename T> __device__ __forceinline__ float rnd(float x) { return Elem<T>::to_f(Elem<T>::from_f(x)); }

__device__ __forceinline__ long long floor_mod_ll(long long a, long long m) {
    long long r = a % m;
    return r < 0 ? r + m : r;
}

// Lane-invariant slot counters, copied to registers / shared memory.
struct Counters {
    long long stored[CKV_MAX_CASCADES];
    long long start[CKV_MAX_CASCADES];
    long long stored_sinks;
    long long seen;
};

// kernels / launchers implemented across the .cu files --------------------------------------
int launch_update_serial(const Dims &d, const ckv_layer_state *st, const void *key, const void *value,
                         int64_t ksb, int64_t ksh, int64_t kst, const void *scores, int64_t ssb, int64_t ssh,
                         int64_t sst, int n_tokens, cudaStream_t stream);

size_t update_chunk_workspace_bytes(const Dims &d, int n_tokens);
int launch_update_chunk(const Dims &d, const ckv_layer_state *st, const void *key, const void *value, int64_t ksb,
                        int64_t ksh, int64_t kst, const void *scores, int64_t ssb, int64_t ssh, int64_t sst,
                        int n_tokens, void *workspace, size_t workspace_bytes, cudaStream_t stream);
// Parallel chunk update when a workspace is available and the chunk has more than one token,
// otherwise the one-warp-per-lane walk.
inline int launch_update(const Dims &d, const ckv_layer_state *st, const void *key, const void *value, int64_t ksb,
                         int64_t ksh, int64_t kst, const void *scores, int64_t ssb, int64_t ssh, int64_t sst,
                         int n_tokens, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    if (n_tokens >= 2 && workspace && workspace_bytes >= update_chunk_workspace_bytes(d, n_tokens))
        return launch_update_chunk(d, st, key, value, ksb, ksh, kst, scores, ssb, ssh, sst, n_tokens, workspace,
                                   workspace_bytes, stream);
    return launch_update_serial(d, st, key, value, ksb, ksh, kst, scores, ssb, ssh, sst, n_tokens, stream);
}

size_t generic_workspace_bytes(const Dims &d, int n_tokens);
int launch_attention_generic(const Dims &d, const ckv_layer_state *st, const void *q, int64_t qsb, int64_t qsh,
                             int64_t qst, const void *key, const void *value, int64_t ksb, int64_t ksh, int64_t kst,
                             int n_tokens, const void *rope, int64_t rope_rows, const float *ema_w_cache,
                             const void *ema_w_new, void *out, int64_t osb, int64_t osh, int64_t ost, void *workspace,
                             size_t workspace_bytes, int flags, cudaStream_t stream);

// Optional CUDA-event timing of the dominant kernel of a call (see ckv_profile_enable).
struct ProfileHook {
    void before(cudaStream_t stream, const char *kernel_name);
    void after(cudaStream_t stream);
};
ProfileHook *active_profile_hook();  // null when profiling is off
void note_launches(int n);           // kernels launched by the current call

bool decode_tuned_supported(const Dims &d, int n_tokens);
size_t decode_workspace_bytes(const Dims &d);
int launch_decode_tuned(const Dims &d, const ckv_layer_state *st, const void *q, int64_t qsb, int64_t qsh,
                        const void *key, const void *value, int64_t ksb, int64_t ksh, const void *rope,
                        int64_t rope_rows, const float *ema_w_cache, const void *ema_w_new, void *out, int64_t osb,
                        int64_t osh, void *workspace, size_t workspace_bytes, int flags, cudaStream_t stream,
                        ProfileHook *hook);

bool prefill_tuned_supported(const Dims &d, int n_tokens);
size_t prefill_workspace_bytes(const Dims &d, int n_tokens);
int launch_prefill_tuned(const Dims &d, const ckv_layer_state *st, const void *q, int64_t qsb, int64_t qsh,
                         int64_t qst, const void *key, const void *value, int64_t ksb, int64_t ksh, int64_t kst,
                         int n_tokens, const void *rope, int64_t rope_rows, const float *ema_w_cache,
                         const void *ema_w_new, void *out, int64_t osb, int64_t osh, int64_t ost, void *workspace,
                         size_t workspace_bytes, int flags, cudaStream_t stream, ProfileHook *hook);

// Self-tests of the bounded waits: a wait on a barrier phase that nothing completes must give up and raise the
// status word (decode: code 1; prefill: 2 | line << 8).
int launch_decode_wait_selftest(int *status, cudaStream_t stream);
int launch_prefill_wait_selftest(int *status, cudaStream_t stream);

// Kernel attributes (opt-in shared memory sizes) belong to a device's context: a process that drives
// several GPUs has to set them once on each.  Returns true the first time it sees the current device.
inline bool first_use_on_this_device(bool (&seen)[64]) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
    if (seen[dev]) return false;
    seen[dev] = true;
    return true;
}

}  // namespace ckv
