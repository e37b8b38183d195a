/*
 * cascade_kv_b200 -- C ABI of the B200 (sm_100a) cascading KV cache hot path.
 *
 * Plain pointers and sizes only; no torch types.  Every pointer is a DEVICE
 * pointer unless its comment says "host".  All entry points return 0 on
 * success and a negative CKV_E_* code on failure; ckv_last_error() gives the
 * message of the calling thread's last failure.  Nothing here synchronises the
 * stream or allocates device memory: callers own every buffer, kernels mutate
 * the cache state in place on the stream they are given.
 *
 * One "lane" is one (batch, kv_head) pair.  Cache state of one layer
 * (reference: CascadingKVCache.init_cache, cascade/models/cascading_cache.py:1187-1276):
 *
 *   key_cache, value_cache  [B, KVH, S, D]   cache dtype, contiguous, S = cascades * window
 *   score_cache             [B, KVH, S]      cache dtype
 *   sink_keys, sink_values  [B, KVH, NS, D]  cache dtype
 *   og_pos                  [B, KVH, S]      int64, 1-based stream index of the token in each slot
 *
 * The reference also stores, per lane, quantities that are identical for every
 * lane because they depend only on how many tokens were seen (the slot
 * counters and everything derived from them).  Here they are stored ONCE:
 *
 *   mask       [S]   uint8, 1 = slot empty          (reference: bool [B,KVH,S])
 *   sink_mask  [NS]  uint8, 1 = slot empty          (reference: bool [B,KVH,NS])
 *   pos        [S]   int64 rank of the slot's token (reference: int64 [B,KVH,S])
 *   sink_pos   [NS]  int64
 *   stored_tokens, start_indices [C] int64          (reference: [B,KVH,C])
 *   stored_sinks [1] int64                          (reference: [B,KVH])
 *   seen_tokens  [1] int64                          (reference: seen_tokens_by_layer[l])
 *   every_n      [C] int64  admission stride per cascade (reference: do_cache_every_n)
 *
 * The host-side mirror exposes them as stride-0 expanded views with the
 * reference's shapes.
 */
#ifndef CASCADE_KV_B200_H
#define CASCADE_KV_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CKV_ABI_VERSION 1

enum { CKV_F32 = 0, CKV_F16 = 1, CKV_BF16 = 2 };
enum { CKV_REDUCE_MEAN = 0, CKV_REDUCE_MAX = 1, CKV_REDUCE_MEDIAN = 2 };
/* CKV_ADMIT_STRIDE: every incoming score is zero and the score cache is never
 * touched by attention (reference: update(..., score_states=None),
 * cascading_cache.py:1306-1311).  CKV_ADMIT_EMA: attention feeds EMA scores. */
enum { CKV_ADMIT_STRIDE = 0, CKV_ADMIT_EMA = 1 };

enum {
    CKV_OK = 0,
    CKV_E_ARG = -1,        /* bad shape / dtype / null pointer / alignment */
    CKV_E_UNSUPPORTED = -2,/* configuration outside what the kernels implement */
    CKV_E_WORKSPACE = -3,  /* workspace too small */
    CKV_E_CUDA = -4        /* a CUDA runtime call failed */
};

/* flags of ckv_attention */
enum {
    CKV_ATTN_UPDATE = 1,        /* also run the score EMA (EMA rule) and the cache update */
    CKV_ATTN_FORCE_GENERIC = 2  /* use the plain CUDA-core kernels even where a tuned path exists */
};

typedef struct ckv_config {
    int32_t batch;             /* B */
    int32_t kv_heads;          /* KVH */
    int32_t q_heads;           /* H, a multiple of KVH */
    int32_t head_dim;          /* D */
    int32_t num_sinks;         /* NS */
    int32_t window;            /* W, slots per cascade */
    int32_t cascades;          /* C */
    int32_t dtype;             /* CKV_F32 / CKV_F16 / CKV_BF16 (cache and activations) */
    int32_t eager_fill;        /* reference: CascadingKVCache(eager_fill=...) */
    int32_t head_reduction;    /* CKV_REDUCE_*   (reference: config._head_reduction) */
    int32_t homogeneous_heads; /* reference: config._homogeneous_heads */
    int32_t admission;         /* CKV_ADMIT_* */
    double beta;               /* EMA coefficient (reference: cache.beta) */
} ckv_config;

typedef struct ckv_layer_state {
    void *key_cache;
    void *value_cache;
    void *score_cache;
    void *sink_keys;
    void *sink_values;
    uint8_t *mask;
    uint8_t *sink_mask;
    int64_t *pos;
    int64_t *og_pos;
    int64_t *sink_pos;
    int64_t *stored_tokens;
    int64_t *start_indices;
    int64_t *stored_sinks;
    int64_t *seen_tokens;
    const int64_t *every_n;
} ckv_layer_state;

int ckv_abi_version(void);
const char *ckv_last_error(void);

/*
 * Insert n_tokens new tokens per lane into the cache, in stream order.
 * Replaces: sink_cache(...) / SinkCacheFunc.forward / the Triton kernel
 * _update_kv_cache (cascade/models/cascading_cache.py:962-1028, :777-901,
 * :145-774) and the counter bump in CascadingKVCache.update (:1346).
 *
 *   key, value  [B, KVH, n_tokens, D] cache dtype; element strides for b/h/t are given,
 *               the last dimension is contiguous and every row 16-byte aligned.
 *   scores      [B, >=KVH, n_tokens] cache dtype with element strides, or NULL = all zero
 *               (only heads < KVH are read, as in the reference).
 *   workspace   ckv_update_workspace_bytes(cfg, n_tokens) bytes of scratch for the parallel chunk
 *               update (256-byte aligned).  NULL / too small selects the one-warp-per-lane walk,
 *               which needs no scratch, gives the same result and is much slower for long chunks.
 * seen_tokens is advanced by n_tokens on the device.
 */
size_t ckv_update_workspace_bytes(const ckv_config *cfg, int32_t n_tokens);
int ckv_cascade_update(const ckv_config *cfg, const ckv_layer_state *st,
                       const void *key, const void *value,
                       int64_t kv_stride_b, int64_t kv_stride_h, int64_t kv_stride_t,
                       const void *scores, int64_t s_stride_b, int64_t s_stride_h, int64_t s_stride_t,
                       int32_t n_tokens, void *workspace, size_t workspace_bytes, void *cuda_stream);

/*
 * Host-only helper (no device work): advance HOST copies of the lane-invariant counters by n_tokens
 * tokens, starting from a layer that has seen seen_tokens tokens.  Which cascade accepts or evicts a
 * token depends only on the token's index and the counters, never on scores, so a caller can mirror
 * them and answer CascadingKVCache.get_seq_length() (cascade/models/cascading_cache.py:1129-1132,
 * two .item() synchronisations per call in the reference) without reading the device.
 *   every_n, stored_tokens, start_indices  [cascades] host int64;  stored_sinks  [1] host int64
 */
int ckv_advance_counters_host(const ckv_config *cfg, const int64_t *every_n /* host */, int64_t seen_tokens,
                              int64_t n_tokens, int64_t *stored_tokens /* host */,
                              int64_t *start_indices /* host */, int64_t *stored_sinks /* host */);

/* Bytes of scratch ckv_attention needs for calls of up to n_tokens query tokens, whatever their
 * flags: the larger of the tuned path's need and the generic path's.  (The reference has no
 * counterpart: its eager path allocates the logits and the concatenated, repeated and rotated
 * keys through torch on every call, cascade/models/cascade_attention.py:250-340.) */
size_t ckv_attention_workspace_bytes(const ckv_config *cfg, int32_t n_tokens);

/* The same for calls that pass exactly these flags.  A caller that never sets
 * CKV_ATTN_FORCE_GENERIC needs far less where a tuned kernel exists: the generic path keeps a
 * logit row per (query head, query), the tuned decode path only its split-K partials (Llama-3.1-8B
 * heads, 16 sequences, 8 x 8192 slots, one token: 86 MB instead of 2.3 GB).  Only
 * CKV_ATTN_FORCE_GENERIC changes the answer. */
size_t ckv_attention_workspace_bytes_for(const ckv_config *cfg, int32_t n_tokens, int32_t flags);

/*
 * Attention of n_tokens new tokens over [sinks | cascade cache | the new tokens
 * themselves (causal)], with RoPE applied at cache positions, followed (flag
 * CKV_ATTN_UPDATE) by the EMA score update and the cache update.
 * Replaces: CascadeAttention.forward_cascade position/RoPE logic
 * (cascade/models/cascade_attention.py:114-181), cascade_attn_eager (:250-340),
 * calc_scores (:231-248), and stands in for cascade_attn_flash + the Triton
 * attention(q,k,v,causal,sm_scale,mask,beta) (:202-229,
 * cascade/models/flash_attention.py:540-652) with the eager path's exact score
 * definition.
 *
 * With a 16-bit cache and D = 128 the call is served by tuned kernels: one token by the streaming
 * decode kernels; a chunk that needs column scores (EMA rule with CKV_ATTN_UPDATE) by the two-pass
 * tcgen05 kernels, whose probabilities are normalised and rounded exactly where the reference rounds
 * them; any other chunk by the single-pass tcgen05 kernel.  Everything else, and every call with
 * CKV_ATTN_FORCE_GENERIC, runs on plain CUDA-core kernels.
 *
 *   q           [B, H, n_tokens, D]    un-rotated, element strides for b/h/t
 *   key, value  [B, KVH, n_tokens, D]  un-rotated, element strides for b/h/t
 *   rope        [rope_rows, D] cache dtype: row p = (cos(p*f_0..f_{D/2-1}) | sin(...)),
 *               rope_rows > NS + S + n_tokens
 *   ema_w_cache [n_tokens] float32: weight of query row q for cached slots,
 *               (1-beta)*beta^(n_tokens-1-q)            (cascade_attention.py:315-317)
 *   ema_w_new   [n_tokens] cache dtype: weight at distance j = q - i for new tokens,
 *               (1-beta)*beta^j                         (cascade_attention.py:269-282)
 *               (both may be NULL under CKV_ADMIT_STRIDE)
 *   out         [B, H, n_tokens, D]    element strides for b/h/t
 *   workspace   at least ckv_attention_workspace_bytes_for(cfg, n_tokens, flags) bytes, 256-byte aligned
 */
int ckv_attention(const ckv_config *cfg, const ckv_layer_state *st,
                  const void *q, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_t,
                  const void *key, const void *value,
                  int64_t kv_stride_b, int64_t kv_stride_h, int64_t kv_stride_t,
                  int32_t n_tokens,
                  const void *rope, int64_t rope_rows,
                  const float *ema_w_cache, const void *ema_w_new,
                  void *out, int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_t,
                  void *workspace, size_t workspace_bytes,
                  int32_t flags, void *cuda_stream);

/*
 * Attention over keys and values that the caller has already rotated and laid out as one dense key
 * axis, with per-column attention scores.  Replaces the reference's functional
 * attention(q, k, v, causal, sm_scale, mask, beta) -> (o, scores)
 * (cascade/models/flash_attention.py:540-652, :713), and serves CascadeAttention.cascade_attn_flash /
 * cascade_attn_eager when they are called with materialised tensors
 * (cascade/models/cascade_attention.py:202-229, :250-340).
 *
 *   q      [B, H, n_ctx, D], k, v [B, kv_heads, n_kv, D] (kv_heads divides H; element strides for b/h/t)
 *   mask   [n_kv - n_ctx] uint8, 1 = column masked.  The first n_kv - n_ctx columns obey `mask`, the
 *          last n_ctx columns are causal (column i visible to query rows >= i), as in the reference
 *          kernel (flash_attention.py:54-61), whatever its `causal` argument says.
 *   out    [B, H, n_ctx, D] with element strides; scores [B, H, n_kv] contiguous in the same dtype, or NULL
 *   score_mode CKV_DENSE_SCORES_FLASH: scores[col] = sum_q p[q,col] (1-beta) beta^(n_ctx-1-q), logits
 *          q.k*sm_scale in fp32 (flash_attention.py:63-100; the reference approximates the row
 *          normaliser while it streams, this kernel uses the exact one).
 *          CKV_DENSE_SCORES_EAGER: the eager path's definition and rounding points
 *          (cascade_attention.py:284-323): logits and probabilities rounded to the tensor dtype, masked
 *          columns weighted by ema_w_cache[q] (fp32 [n_ctx]), causal columns by ema_w_new[q - i]
 *          (dtype [n_ctx]) with every product rounded.
 *   workspace  ckv_dense_attention_workspace_bytes(B, H, n_ctx) bytes, 256-byte aligned
 */
enum { CKV_DENSE_SCORES_FLASH = 0, CKV_DENSE_SCORES_EAGER = 1 };
size_t ckv_dense_attention_workspace_bytes(int32_t batch, int32_t q_heads, int32_t n_ctx);
int ckv_dense_attention(const void *q, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_t,
                        const void *k, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_t,
                        const void *v, int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_t,
                        const uint8_t *mask, int32_t batch, int32_t q_heads, int32_t kv_heads,
                        int32_t n_ctx, int32_t n_kv, int32_t head_dim, int32_t dtype, double sm_scale,
                        double beta, int32_t score_mode, const float *ema_w_cache, const void *ema_w_new,
                        void *out, int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_t,
                        void *scores, void *workspace, size_t workspace_bytes, void *cuda_stream);

/*
 * The two element-wise operators of the decoder layer around the attention, for the end-to-end configuration
 * (the reference runs them as chains of framework kernels inside its forked models:
 * cascade/models/llama/modeling_llama.py:113-127 LlamaRMSNorm, :745-770 the residual adds of the decoder layer,
 * :282-313 the SwiGLU gate of LlamaMLP; cascade/models/qwen2/modeling_qwen2.py likewise).  16-bit rows,
 * contiguous, 16-byte aligned, `hidden` / `cols` multiples of 8.
 *
 * ckv_add_rmsnorm: s = x + residual (rounded to the dtype; residual may be null: s = x), written to sum_out
 *   when that is not null; normed = weight * T(s * rsqrt(mean(s^2) + eps)) with the variance in fp32 and the
 *   normalised row rounded to the dtype before the weight is applied, as the reference does.  x, residual,
 *   normed, sum_out: [rows, hidden]; weight: [hidden].  sum_out may alias residual, normed may alias x.
 * ckv_silu_mul: out = T(T(silu(gate)) * up); gate / up: [rows, cols] with row strides ld_gate / ld_up in
 *   elements (the two halves of one fused projection are fine), out: [rows, cols] contiguous.
 */
int ckv_add_rmsnorm(const void *x, const void *residual, const void *weight, void *normed, void *sum_out,
                    int64_t rows, int32_t hidden, double eps, int32_t dtype, void *cuda_stream);
int ckv_silu_mul(const void *gate, const void *up, void *out, int64_t rows, int32_t cols, int64_t ld_gate,
                 int64_t ld_up, int32_t dtype, void *cuda_stream);

/*
 * ckv_attention for callers that may not allocate device memory.
 * (No counterpart in the reference, whose Python layer allocates freely through torch.)
 *
 * Some hosts of this library cannot give it a workspace: a serving runtime that sized all of its
 * device memory at start-up and forbids allocation afterwards, a plugin loaded into a process
 * whose allocator it may not touch, or code running between the capture-safe calls of a
 * framework.  For them the scratch comes from a fixed array of CKV_STATIC_SCRATCH_BYTES bytes
 * that is part of this library's device image: every GPU that loads the library holds those bytes
 * until the process exits.  Arguments are those of ckv_attention minus the workspace pair.
 *
 *  - Calls whose ckv_attention_workspace_bytes_for() exceeds CKV_STATIC_SCRATCH_BYTES are
 *    refused with CKV_E_WORKSPACE; use ckv_attention with your own buffer for those.
 *  - The first call on each device looks up the array's device address (with that device
 *    current); make that first call outside any stream capture.
 *  - No cudaMalloc, cudaFree or other allocating routine is called, on any call.
 *  - All calls on a device share the one array, and it keeps whatever the previous call left;
 *    the words that must start at zero are cleared on the stream at the start of every call.
 *    Two calls that can overlap on the GPU (different streams, no ordering between them) would
 *    race on the array: order them.
 */
#define CKV_STATIC_SCRATCH_BYTES (8u << 20)
size_t ckv_static_scratch_bytes(void);
int ckv_attention_static(const ckv_config *cfg, const ckv_layer_state *st,
                         const void *q, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_t,
                         const void *key, const void *value,
                         int64_t kv_stride_b, int64_t kv_stride_h, int64_t kv_stride_t,
                         int32_t n_tokens,
                         const void *rope, int64_t rope_rows,
                         const float *ema_w_cache, const void *ema_w_new,
                         void *out, int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_t,
                         int32_t flags, void *cuda_stream);
/* ckv_read_status for the built-in array of the current device: a caller of ckv_attention_static has
 * no workspace pointer to pass.  Copies four bytes to the host (synchronises); allocates nothing.
 * (No counterpart in the reference.) */
int ckv_static_status(int32_t *status /* host */);

/* Number of kernels the calling thread's last ckv_attention / ckv_cascade_update call launched. */
int ckv_last_launch_count(void);

/*
 * Optional CUDA-event timing of the kernels of every following ckv_attention call, with events
 * owned by the library.  Replaces the BENCHMARK switch of the reference's sink_cache(), which
 * brackets its launch with CUDA events and prints the time
 * (cascade/models/cascading_cache.py:986-1026).  ckv_profile_read synchronises on the recorded
 * events, sums them per kernel, returns the kernel with the largest total (its summed duration, how
 * many of its launches were timed, its name) and starts a new collection; ckv_profile_kernel then
 * gives the totals of every timed kernel of that collection, largest first (index 0 is the one
 * ckv_profile_read returned; CKV_E_ARG past the end).  Not thread-safe; meant for benchmarks.
 */
int ckv_profile_enable(int enable);
int ckv_profile_read(double *total_ms /* host */, int32_t *launches /* host */, const char **kernel_name /* host */);
int ckv_profile_kernel(int32_t index, const char **kernel_name /* host */, double *total_ms /* host */,
                       int32_t *launches /* host */);

/*
 * Copy the status word of a ckv_attention workspace to the host (synchronises).  0 = no kernel of
 * the last call gave up on a bounded wait; non-zero = a pipeline wait ran out and the results of
 * that call are invalid: low byte 1 (decode kernels) or 2 (prefill kernels, bits 8 and up then hold
 * the source line of the wait that gave up), 3 = the prefill kernel found its shared-memory window
 * misaligned.  (No counterpart in the reference: its kernels have no waits.)  Callers of
 * ckv_attention_static, who hold no workspace pointer, use ckv_static_status instead.
 */
int ckv_read_status(const void *workspace, int32_t *status /* host */);

/*
 * Self-test of the bounded waits: launches one thread that waits, with a short limit, for a barrier phase
 * that nothing completes -- through the very wait routine of the decode kernels (which = 1) or of the
 * prefill kernels (which = 2).  The wait must give up and the kernel end normally; afterwards
 * ckv_read_status(workspace) gives 1 (decode) or 2 | line << 8 (prefill).  This is how the error path of
 * the waits is exercised without making a real pipeline stall.  workspace: at least 4 bytes of device
 * memory, its first word is overwritten.  (No counterpart in the reference.)
 */
int ckv_selftest_bounded_wait(int32_t which, void *workspace, void *cuda_stream);

/*
 * Debug build of the library only (compiled with -DCKV_BOUNDS: `python -m cascading_kv_cache_b200.build
 * --bounds` writes libckv_b200_bounds.so): the update kernels check every slot index and counter before
 * they use it; a violation is recorded and the access skipped, nothing traps.  Returns the first
 * violation since the last call (4 | source line << 8) or 0, and clears the record; synchronises the
 * device.  The ordinary build answers CKV_E_UNSUPPORTED.  (The reference has no counterpart; this stands
 * in for a memory checker where none can be run.)
 */
int ckv_bounds_status(int32_t *status /* host */);

#ifdef __cplusplus
}
#endif
#endif /* CASCADE_KV_B200_H */
