// extern "C" entry points of libckv_b200.so: argument checks and dispatch.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <utility>
#include <vector>

#include "ckv_common.cuh"

namespace ckv {

static thread_local char g_error[512] = "";

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

// ---- profiling hook: library-owned CUDA events around the kernels of each call --------------------
struct TimedLaunch {
    const char *name;
    cudaEvent_t a, b;
};
static bool g_profile_on = false;
static std::vector<TimedLaunch> g_events;
static size_t g_events_used = 0;
static ProfileHook g_hook;
static thread_local int g_launches = 0;
struct KernelTotal {
    const char *name;
    double ms;
    int launches;
};
static std::vector<KernelTotal> g_totals;   // of the last ckv_profile_read, largest total first

void ProfileHook::before(cudaStream_t stream, const char *kernel_name) {
    if (g_events_used == g_events.size()) {
        cudaEvent_t a, b;
        if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return;
        g_events.push_back({kernel_name, a, b});
    }
    g_events[g_events_used].name = kernel_name;
    cudaEventRecord(g_events[g_events_used].a, stream);
}

void ProfileHook::after(cudaStream_t stream) {
    if (g_events_used < g_events.size()) {
        cudaEventRecord(g_events[g_events_used].b, stream);
        g_events_used += 1;
    }
}

ProfileHook *active_profile_hook() { return g_profile_on ? &g_hook : nullptr; }

void note_launches(int n) { g_launches += n; }
void reset_launch_count() { g_launches = 0; }

static int check_state(const ckv_layer_state *st) {
    if (!st) return fail(CKV_E_ARG, "layer state is null");
    if (!st->key_cache || !st->value_cache || !st->score_cache || !st->mask || !st->pos || !st->og_pos ||
        !st->stored_tokens || !st->start_indices || !st->stored_sinks || !st->seen_tokens || !st->every_n)
        return fail(CKV_E_ARG, "layer state has a null pointer");
    return CKV_OK;
}

// Every launch goes to the calling thread's current device.  A cache that lives on another device
// (a process that drives several GPUs and forgot to make the cache's device current) would hand
// this device pointers it cannot reach: refuse on the host instead of faulting on the GPU.
static int check_device(const void *device_ptr, const char *what, void *cuda_stream) {
    // not while the stream is being captured into a graph: the call was checked when it was first made
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing((cudaStream_t)cuda_stream, &capturing) != cudaSuccess) cudaGetLastError();
    if (capturing != cudaStreamCaptureStatusNone) return CKV_OK;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return CKV_OK;  // no usable device: the first launch reports it
    }
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, device_ptr) != cudaSuccess) {
        cudaGetLastError();
        return CKV_OK;
    }
    if (attr.type == cudaMemoryTypeDevice && attr.device != dev)
        return fail(CKV_E_ARG, "%s lives on device %d but device %d is current: make the cache's device current "
                               "before the call", what, attr.device, dev);
    return CKV_OK;
}

static int check_sinks(const Dims &d, const ckv_layer_state *st) {
    if (d.NS > 0 && (!st->sink_keys || !st->sink_values || !st->sink_mask || !st->sink_pos))
        return fail(CKV_E_ARG, "sink buffers are null");
    return CKV_OK;
}

}  // namespace ckv

using namespace ckv;

extern "C" int ckv_abi_version(void) { return CKV_ABI_VERSION; }

extern "C" const char *ckv_last_error(void) { return g_error; }

extern "C" int ckv_cascade_update(const ckv_config *cfg, const ckv_layer_state *st, const void *key, const void *value,
                                  int64_t kv_stride_b, int64_t kv_stride_h, int64_t kv_stride_t, const void *scores,
                                  int64_t s_stride_b, int64_t s_stride_h, int64_t s_stride_t, int32_t n_tokens,
                                  void *workspace, size_t workspace_bytes, void *cuda_stream) {
    Dims d;
    int rc = make_dims(cfg, &d);
    if (rc != CKV_OK) return rc;
    rc = check_state(st);
    if (rc != CKV_OK) return rc;
    if (!key || !value) return fail(CKV_E_ARG, "key/value is null");
    if (n_tokens < 1) return fail(CKV_E_ARG, "n_tokens must be at least 1, got %d", n_tokens);
    if ((rc = check_sinks(d, st)) != CKV_OK) return rc;
    if ((rc = check_device(st->key_cache, "key_cache", cuda_stream)) != CKV_OK) return rc;
    g_launches = 0;
    return launch_update(d, st, key, value, kv_stride_b, kv_stride_h, kv_stride_t, scores, s_stride_b, s_stride_h,
                         s_stride_t, n_tokens, workspace, workspace_bytes, (cudaStream_t)cuda_stream);
}

extern "C" size_t ckv_update_workspace_bytes(const ckv_config *cfg, int32_t n_tokens) {
    Dims d;
    if (make_dims(cfg, &d) != CKV_OK || n_tokens < 1) return 0;
    return update_chunk_workspace_bytes(d, n_tokens);
}

extern "C" size_t ckv_attention_workspace_bytes_for(const ckv_config *cfg, int32_t n_tokens, int32_t flags) {
    Dims d;
    if (make_dims(cfg, &d) != CKV_OK || n_tokens < 1) return 0;
    // the same choice of path as ckv_attention makes
    if (!(flags & CKV_ATTN_FORCE_GENERIC) && decode_tuned_supported(d, n_tokens)) return decode_workspace_bytes(d);
    if (!(flags & CKV_ATTN_FORCE_GENERIC) && prefill_tuned_supported(d, n_tokens))
        return prefill_workspace_bytes(d, n_tokens);
    return generic_workspace_bytes(d, n_tokens);
}

extern "C" size_t ckv_attention_workspace_bytes(const ckv_config *cfg, int32_t n_tokens) {
    const size_t a = ckv_attention_workspace_bytes_for(cfg, n_tokens, 0);
    const size_t b = ckv_attention_workspace_bytes_for(cfg, n_tokens, CKV_ATTN_FORCE_GENERIC);
    return a > b ? a : b;
}

// Host-only: the score-free part of the update state machine (which cascade accepts, which evicts)
// on host copies of the counters, so that a caller can know them without reading the device.
extern "C" int ckv_advance_counters_host(const ckv_config *cfg, const int64_t *every_n, int64_t seen_tokens,
                                         int64_t n_tokens, int64_t *stored_tokens, int64_t *start_indices,
                                         int64_t *stored_sinks) {
    Dims d;
    int rc = make_dims(cfg, &d);
    if (rc != CKV_OK) return rc;
    if (!every_n || !stored_tokens || !start_indices || !stored_sinks) return fail(CKV_E_ARG, "null pointer");
    if (seen_tokens < 0 || n_tokens < 0) return fail(CKV_E_ARG, "negative token count");
    for (int i = 0; i < d.C; ++i)
        if (every_n[i] < 1) return fail(CKV_E_ARG, "every_n[%d] must be at least 1", i);
    int64_t sinks = *stored_sinks;
    for (int64_t j = 0; j < n_tokens; ++j) {
        const int64_t rti = seen_tokens + j + 1;
        if (sinks < d.NS) {
            sinks += 1;
            continue;
        }
        const bool eager = d.eager_fill && (rti - 1 <= (int64_t)d.S + d.NS);
        int i = 0;
        while (i < d.C) {
            const bool do_i = eager || ((rti - 1 - d.NS) % every_n[i] == 0);   // rti - 1 >= NS here
            if ((do_i && stored_tokens[i] < d.W) || (!do_i && stored_tokens[i] == 0)) {
                stored_tokens[i] += 1;
                break;
            } else if (do_i) {
                start_indices[i] = (start_indices[i] + 1) % d.W;
                i += 1;
            } else {
                break;
            }
        }
    }
    *stored_sinks = sinks;
    return CKV_OK;
}

#ifdef CKV_BOUNDS
namespace ckv {
int read_bounds_status_serial(int *out);
int read_bounds_status_chunk(int *out);
int read_bounds_status_decode(int *out);
}  // namespace ckv
#endif

// Debug builds (-DCKV_BOUNDS) only: the first bounds violation the update kernels recorded since the last
// call, 0 if none (4 | source line << 8 otherwise); clears the record.  Synchronises.
extern "C" int ckv_bounds_status(int32_t *status) {
    if (!status) return fail(CKV_E_ARG, "status is null");
#ifdef CKV_BOUNDS
    CKV_CUDA_CHECK(cudaDeviceSynchronize());
    int a = 0, b = 0, c = 0;
    if (read_bounds_status_serial(&a) || read_bounds_status_chunk(&b) || read_bounds_status_decode(&c))
        return fail(CKV_E_CUDA, "reading the bounds status failed");
    *status = a ? a : (b ? b : c);
    return CKV_OK;
#else
    *status = 0;
    return fail(CKV_E_UNSUPPORTED, "this library was built without CKV_BOUNDS");
#endif
}

extern "C" int ckv_last_launch_count(void) { return g_launches; }

extern "C" int ckv_profile_enable(int enable) {
    g_profile_on = enable != 0;
    g_events_used = 0;
    if (!g_profile_on) {
        for (auto &e : g_events) {
            cudaEventDestroy(e.a);
            cudaEventDestroy(e.b);
        }
        g_events.clear();
    }
    return CKV_OK;
}

extern "C" int ckv_profile_read(double *total_ms, int32_t *launches, const char **kernel_name) {
    g_totals.clear();
    for (size_t i = 0; i < g_events_used; ++i) {
        CKV_CUDA_CHECK(cudaEventSynchronize(g_events[i].b));
        float ms = 0.f;
        CKV_CUDA_CHECK(cudaEventElapsedTime(&ms, g_events[i].a, g_events[i].b));
        size_t k = 0;
        while (k < g_totals.size() && strcmp(g_totals[k].name, g_events[i].name) != 0) ++k;
        if (k == g_totals.size()) g_totals.push_back({g_events[i].name, 0.0, 0});
        g_totals[k].ms += ms;
        g_totals[k].launches += 1;
    }
    for (size_t i = 1; i < g_totals.size(); ++i)       // few entries: insertion sort, largest total first
        for (size_t j = i; j > 0 && g_totals[j].ms > g_totals[j - 1].ms; --j) std::swap(g_totals[j], g_totals[j - 1]);
    const bool any = !g_totals.empty();
    if (total_ms) *total_ms = any ? g_totals[0].ms : 0.0;
    if (launches) *launches = any ? g_totals[0].launches : 0;
    if (kernel_name) *kernel_name = any ? g_totals[0].name : "";
    g_events_used = 0;
    return CKV_OK;
}

extern "C" int ckv_profile_kernel(int32_t index, const char **kernel_name, double *total_ms, int32_t *launches) {
    if (index < 0 || (size_t)index >= g_totals.size()) return fail(CKV_E_ARG, "no kernel %d in the last collection", index);
    if (kernel_name) *kernel_name = g_totals[index].name;
    if (total_ms) *total_ms = g_totals[index].ms;
    if (launches) *launches = g_totals[index].launches;
    return CKV_OK;
}

extern "C" int ckv_selftest_bounded_wait(int32_t which, void *workspace, void *cuda_stream) {
    if (!workspace) return fail(CKV_E_ARG, "workspace is null");
    if (which != 1 && which != 2) return fail(CKV_E_ARG, "which must be 1 (decode kernels) or 2 (prefill kernels)");
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    CKV_CUDA_CHECK(cudaMemsetAsync(workspace, 0, 4, stream));
    return which == 1 ? launch_decode_wait_selftest((int *)workspace, stream)
                      : launch_prefill_wait_selftest((int *)workspace, stream);
}

extern "C" int ckv_read_status(const void *workspace, int32_t *status) {
    if (!workspace || !status) return fail(CKV_E_ARG, "workspace/status is null");
    CKV_CUDA_CHECK(cudaMemcpy(status, workspace, 4, cudaMemcpyDeviceToHost));
    return CKV_OK;
}

extern "C" int ckv_attention(const ckv_config *cfg, const ckv_layer_state *st, const void *q, int64_t q_stride_b,
                             int64_t q_stride_h, int64_t q_stride_t, const void *key, const void *value,
                             int64_t kv_stride_b, int64_t kv_stride_h, int64_t kv_stride_t, int32_t n_tokens,
                             const void *rope, int64_t rope_rows, const float *ema_w_cache, const void *ema_w_new,
                             void *out, int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_t, void *workspace,
                             size_t workspace_bytes, int32_t flags, void *cuda_stream) {
    Dims d;
    int rc = make_dims(cfg, &d);
    if (rc != CKV_OK) return rc;
    rc = check_state(st);
    if (rc != CKV_OK) return rc;
    if (!q || !key || !value || !out || !rope) return fail(CKV_E_ARG, "q/key/value/out/rope is null");
    if (n_tokens < 1) return fail(CKV_E_ARG, "n_tokens must be at least 1, got %d", n_tokens);
    if (d.NS < 1) return fail(CKV_E_UNSUPPORTED, "attention needs at least one sink token");
    if ((rc = check_sinks(d, st)) != CKV_OK) return rc;
    if ((rc = check_device(st->key_cache, "key_cache", cuda_stream)) != CKV_OK) return rc;
    g_launches = 0;
    if (!(flags & CKV_ATTN_FORCE_GENERIC) && decode_tuned_supported(d, n_tokens))
        return launch_decode_tuned(d, st, q, q_stride_b, q_stride_h, key, value, kv_stride_b, kv_stride_h, rope,
                                   rope_rows, ema_w_cache, ema_w_new, out, o_stride_b, o_stride_h, workspace,
                                   workspace_bytes, flags, (cudaStream_t)cuda_stream, active_profile_hook());
    if (!(flags & CKV_ATTN_FORCE_GENERIC) && prefill_tuned_supported(d, n_tokens))
        return launch_prefill_tuned(d, st, q, q_stride_b, q_stride_h, q_stride_t, key, value, kv_stride_b, kv_stride_h,
                                    kv_stride_t, n_tokens, rope, rope_rows, ema_w_cache, ema_w_new, out, o_stride_b,
                                    o_stride_h, o_stride_t, workspace, workspace_bytes, flags,
                                    (cudaStream_t)cuda_stream, active_profile_hook());
    return launch_attention_generic(d, st, q, q_stride_b, q_stride_h, q_stride_t, key, value, kv_stride_b,
                                    kv_stride_h, kv_stride_t, n_tokens, rope, rope_rows, ema_w_cache, ema_w_new, out,
                                    o_stride_b, o_stride_h, o_stride_t, workspace, workspace_bytes, flags,
                                    (cudaStream_t)cuda_stream);
}
