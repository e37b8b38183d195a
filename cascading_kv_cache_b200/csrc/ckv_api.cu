// extern "C" entry points of libckv_b200.so: argument checks and dispatch.
#include <stdarg.h>
#include <stdio.h>

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

static int check_state(const ckv_layer_state *st) {
    if (!st) return fail(CKV_E_ARG, "layer state is null");
    if (!st->key_cache || !st->value_cache || !st->score_cache || !st->mask || !st->pos || !st->og_pos ||
        !st->stored_tokens || !st->start_indices || !st->stored_sinks || !st->seen_tokens || !st->every_n)
        return fail(CKV_E_ARG, "layer state has a null pointer");
    return CKV_OK;
}

}  // namespace ckv

using namespace ckv;

extern "C" int ckv_abi_version(void) { return CKV_ABI_VERSION; }

extern "C" const char *ckv_last_error(void) { return g_error; }

extern "C" int ckv_cascade_update(const ckv_config *cfg, const ckv_layer_state *st, const void *key, const void *value,
                                  int64_t kv_stride_b, int64_t kv_stride_h, int64_t kv_stride_t, const void *scores,
                                  int64_t s_stride_b, int64_t s_stride_h, int64_t s_stride_t, int32_t n_tokens,
                                  void *cuda_stream) {
    Dims d;
    int rc = make_dims(cfg, &d);
    if (rc != CKV_OK) return rc;
    rc = check_state(st);
    if (rc != CKV_OK) return rc;
    if (!key || !value) return fail(CKV_E_ARG, "key/value is null");
    if (n_tokens < 1) return fail(CKV_E_ARG, "n_tokens must be at least 1, got %d", n_tokens);
    if (d.NS > 0 && (!st->sink_keys || !st->sink_values || !st->sink_mask || !st->sink_pos))
        return fail(CKV_E_ARG, "sink buffers are null");
    return launch_update_serial(d, st, key, value, kv_stride_b, kv_stride_h, kv_stride_t, scores, s_stride_b,
                                s_stride_h, s_stride_t, n_tokens, (cudaStream_t)cuda_stream);
}

extern "C" size_t ckv_attention_workspace_bytes(const ckv_config *cfg, int32_t n_tokens) {
    Dims d;
    if (make_dims(cfg, &d) != CKV_OK || n_tokens < 1) return 0;
    return generic_workspace_bytes(d, n_tokens);
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
    return launch_attention_generic(d, st, q, q_stride_b, q_stride_h, q_stride_t, key, value, kv_stride_b,
                                    kv_stride_h, kv_stride_t, n_tokens, rope, rope_rows, ema_w_cache, ema_w_new, out,
                                    o_stride_b, o_stride_h, o_stride_t, workspace, workspace_bytes, flags,
                                    (cudaStream_t)cuda_stream);
}
