// Functional attention over already rotated, already concatenated keys and values with per-column
// attention scores: the operator behind the reference's
//     attention(q, k, v, causal, sm_scale, mask, beta) -> (o, scores)
// (cascade/models/flash_attention.py:540-652, :713) and behind the bodies of
// CascadeAttention.cascade_attn_flash / cascade_attn_eager when they are called with materialised
// tensors (cascade/models/cascade_attention.py:202-229, :250-340).
//
// The key axis is [n_cached columns governed by `mask` | N_CTX columns governed by causality]
// (flash_attention.py:54-61).  The fused ckv_attention call is the fast path of the model forward;
// this operator serves callers that hold dense tensors.  Plain CUDA-core kernels, any head_dim up to
// 256, fp32 / fp16 / bf16:
//   dense_rows_kernel : one warp per query row, online softmax, output row, row max / sum
//   dense_cols_kernel : one warp per key column, exactly normalised column scores
// Column scores, flash mode (flash_attention.py:71-100): sum_q p[q,col] (1-beta) beta^(N_CTX-1-q),
//   with the exact row normaliser where the reference kernel uses a running approximation.
// Column scores, eager mode (cascade_attention.py:315-323): cached columns as above with caller-made
//   fp32 weights, causal columns sum_{q>=i} T(T(p[q,i]) * w_new[q-i]).
#include "ckv_common.cuh"

namespace ckv {

namespace {

struct DenseParams {
    const void *q, *k, *v;
    long long qsb, qsh, qst, ksb, ksh, kst, vsb, vsh, vst;  // elements
    const uint8_t *mask;                                    // [n_cached], 1 = masked; may be null
    void *out;
    long long osb, osh, ost;
    void *scores;                                           // [B, H, N_KV] in T, or null
    const float *w_cache;                                   // eager mode: [N_CTX] fp32
    const void *w_new;                                      // eager mode: [N_CTX] T
    float *row_m, *row_l;                                   // [B*H*N_CTX]
    int B, H, KVH, G, D, N_CTX, N_KV, n_cached;
    int eager;
    float sm_scale, beta;
};

constexpr int kMaxDPerLane = 8;  // head_dim up to 256

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ bool column_visible(const DenseParams &p, int col, int qrow) {
    if (col < p.n_cached) return p.mask == nullptr || p.mask[col] == 0;
    return (col - p.n_cached) <= qrow;
}

template <typename T>
__device__ __forceinline__ float logit_of(const DenseParams &p, const float (&qv)[kMaxDPerLane], const T *kr,
                                          int lane_id) {
    float part = 0.f;
#pragma unroll
    for (int e = 0; e < kMaxDPerLane; ++e) {
        const int d = lane_id + 32 * e;
        if (d < p.D) part = fmaf(qv[e], Elem<T>::to_f(kr[d]), part);
    }
    const float s = warp_sum(part) * p.sm_scale;
    return p.eager ? rnd<T>(s) : s;   // the eager path's einsum output is a tensor of T
}

template <typename T>
__global__ void __launch_bounds__(128) dense_rows_kernel(DenseParams p) {
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane_id = threadIdx.x & 31;
    const long long n_rows = (long long)p.B * p.H * p.N_CTX;
    if (warp >= n_rows) return;
    const int qi = (int)(warp % p.N_CTX);
    const int bh = (int)(warp / p.N_CTX);
    const int b = bh / p.H, h = bh % p.H, kh = h / p.G;
    const T *qrow = (const T *)p.q + b * p.qsb + h * p.qsh + (long long)qi * p.qst;
    const T *kbase = (const T *)p.k + b * p.ksb + kh * p.ksh;
    const T *vbase = (const T *)p.v + b * p.vsb + kh * p.vsh;
    float qv[kMaxDPerLane], acc[kMaxDPerLane];
#pragma unroll
    for (int e = 0; e < kMaxDPerLane; ++e) {
        const int d = lane_id + 32 * e;
        qv[e] = d < p.D ? Elem<T>::to_f(qrow[d]) : 0.f;
        acc[e] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const int c_end = min(p.N_KV, p.n_cached + qi + 1);
    for (int c = 0; c < c_end; ++c) {
        if (!column_visible(p, c, qi)) continue;
        const float s = logit_of<T>(p, qv, kbase + (long long)c * p.kst, lane_id);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);
        const float pr = expf(s - m_new);
        l = l * corr + pr;
        const T *vr = vbase + (long long)c * p.vst;
#pragma unroll
        for (int e = 0; e < kMaxDPerLane; ++e) {
            const int d = lane_id + 32 * e;
            if (d < p.D) acc[e] = acc[e] * corr + pr * Elem<T>::to_f(vr[d]);
        }
        m = m_new;
    }
    T *orow = (T *)p.out + b * p.osb + h * p.osh + (long long)qi * p.ost;
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int e = 0; e < kMaxDPerLane; ++e) {
        const int d = lane_id + 32 * e;
        if (d < p.D) orow[d] = Elem<T>::from_f(acc[e] * inv);
    }
    if (lane_id == 0) {
        p.row_m[warp] = m;
        p.row_l[warp] = l;
    }
}

template <typename T>
__global__ void __launch_bounds__(128) dense_cols_kernel(DenseParams p) {
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane_id = threadIdx.x & 31;
    const long long n = (long long)p.B * p.H * p.N_KV;
    if (warp >= n) return;
    const int col = (int)(warp % p.N_KV);
    const int bh = (int)(warp / p.N_KV);
    const int b = bh / p.H, h = bh % p.H, kh = h / p.G;
    const bool causal_col = col >= p.n_cached;
    float result = 0.f;
    if (causal_col || p.mask == nullptr || p.mask[col] == 0) {
        const T *kr = (const T *)p.k + b * p.ksb + kh * p.ksh + (long long)col * p.kst;
        float kv[kMaxDPerLane];
#pragma unroll
        for (int e = 0; e < kMaxDPerLane; ++e) {
            const int d = lane_id + 32 * e;
            kv[e] = d < p.D ? Elem<T>::to_f(kr[d]) : 0.f;
        }
        const int q0 = causal_col ? col - p.n_cached : 0;
        const float log2_beta = log2f(p.beta);
        const T *w_new = (const T *)p.w_new;
        float sum = 0.f;
        for (int qi = q0; qi < p.N_CTX; ++qi) {
            const long long row = (long long)bh * p.N_CTX + qi;
            const T *qrow = (const T *)p.q + b * p.qsb + h * p.qsh + (long long)qi * p.qst;
            float part = 0.f;
#pragma unroll
            for (int e = 0; e < kMaxDPerLane; ++e) {
                const int d = lane_id + 32 * e;
                if (d < p.D) part = fmaf(Elem<T>::to_f(qrow[d]), kv[e], part);
            }
            float s = warp_sum(part) * p.sm_scale;
            if (p.eager) s = rnd<T>(s);
            float pr = expf(s - p.row_m[row]) / p.row_l[row];
            if (p.eager) {
                pr = rnd<T>(pr);
                if (causal_col) sum += rnd<T>(__fmul_rn(pr, Elem<T>::to_f(w_new[qi - q0])));
                else sum = fmaf(pr, p.w_cache[qi], sum);
            } else {
                const float w = exp2f((float)(p.N_CTX - 1 - qi) * log2_beta) * (1.f - p.beta);
                sum = fmaf(pr, w, sum);
            }
        }
        result = sum;
    }
    if (lane_id == 0) ((T *)p.scores)[warp] = Elem<T>::from_f(result);
}

template <typename T>
int run_dense(const DenseParams &p, cudaStream_t stream) {
    const long long n_rows = (long long)p.B * p.H * p.N_CTX;
    dense_rows_kernel<T><<<(unsigned)((n_rows + 3) / 4), 128, 0, stream>>>(p);
    CKV_CUDA_CHECK(cudaGetLastError());
    int launches = 1;
    if (p.scores) {
        const long long n_cols = (long long)p.B * p.H * p.N_KV;
        dense_cols_kernel<T><<<(unsigned)((n_cols + 3) / 4), 128, 0, stream>>>(p);
        CKV_CUDA_CHECK(cudaGetLastError());
        launches = 2;
    }
    note_launches(launches);
    return CKV_OK;
}

}  // namespace

void reset_launch_count();

}  // namespace ckv

using namespace ckv;

extern "C" size_t ckv_dense_attention_workspace_bytes(int32_t batch, int32_t q_heads, int32_t n_ctx) {
    if (batch < 1 || q_heads < 1 || n_ctx < 1) return 0;
    return 2 * (((size_t)batch * q_heads * n_ctx * 4 + 255) & ~(size_t)255);
}

extern "C" int ckv_dense_attention(const void *q, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_t,
                                   const void *k, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_t,
                                   const void *v, int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_t,
                                   const uint8_t *mask, int32_t batch, int32_t q_heads, int32_t kv_heads,
                                   int32_t n_ctx, int32_t n_kv, int32_t head_dim, int32_t dtype, double sm_scale,
                                   double beta, int32_t score_mode, const float *ema_w_cache, const void *ema_w_new,
                                   void *out, int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_t,
                                   void *scores, void *workspace, size_t workspace_bytes, void *cuda_stream) {
    if (!q || !k || !v || !out) return fail(CKV_E_ARG, "q/k/v/out is null");
    if (batch < 1 || q_heads < 1 || kv_heads < 1 || n_ctx < 1 || n_kv < n_ctx || head_dim < 1)
        return fail(CKV_E_ARG, "bad shape: batch %d heads %d/%d n_ctx %d n_kv %d head_dim %d", batch, q_heads, kv_heads,
                    n_ctx, n_kv, head_dim);
    if (q_heads % kv_heads != 0) return fail(CKV_E_ARG, "q_heads (%d) is not a multiple of kv_heads (%d)", q_heads, kv_heads);
    if (head_dim > 32 * kMaxDPerLane) return fail(CKV_E_UNSUPPORTED, "head_dim %d above %d", head_dim, 32 * kMaxDPerLane);
    if (dtype != CKV_F32 && dtype != CKV_F16 && dtype != CKV_BF16) return fail(CKV_E_ARG, "unknown dtype code %d", dtype);
    if (score_mode != CKV_DENSE_SCORES_FLASH && score_mode != CKV_DENSE_SCORES_EAGER)
        return fail(CKV_E_ARG, "unknown score mode %d", score_mode);
    if (scores && score_mode == CKV_DENSE_SCORES_EAGER && (!ema_w_cache || !ema_w_new))
        return fail(CKV_E_ARG, "eager score mode needs ema_w_cache and ema_w_new");
    if (n_kv > n_ctx && !mask) return fail(CKV_E_ARG, "mask is null but %d cached columns exist", n_kv - n_ctx);
    const size_t need = ckv_dense_attention_workspace_bytes(batch, q_heads, n_ctx);
    if (!workspace || workspace_bytes < need)
        return fail(CKV_E_WORKSPACE, "workspace of %zu bytes, need %zu", workspace_bytes, need);
    DenseParams p;
    p.q = q; p.k = k; p.v = v;
    p.qsb = q_stride_b; p.qsh = q_stride_h; p.qst = q_stride_t;
    p.ksb = k_stride_b; p.ksh = k_stride_h; p.kst = k_stride_t;
    p.vsb = v_stride_b; p.vsh = v_stride_h; p.vst = v_stride_t;
    p.mask = mask;
    p.out = out; p.osb = o_stride_b; p.osh = o_stride_h; p.ost = o_stride_t;
    p.scores = scores;
    p.w_cache = ema_w_cache; p.w_new = ema_w_new;
    p.row_m = (float *)workspace;
    p.row_l = (float *)((uint8_t *)workspace + need / 2);
    p.B = batch; p.H = q_heads; p.KVH = kv_heads; p.G = q_heads / kv_heads; p.D = head_dim;
    p.N_CTX = n_ctx; p.N_KV = n_kv; p.n_cached = n_kv - n_ctx;
    p.eager = score_mode == CKV_DENSE_SCORES_EAGER;
    p.sm_scale = (float)sm_scale; p.beta = (float)beta;
    reset_launch_count();
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    if (dtype == CKV_F32) return run_dense<float>(p, stream);
    if (dtype == CKV_F16) return run_dense<__half>(p, stream);
    return run_dense<__nv_bfloat16>(p, stream);
}
