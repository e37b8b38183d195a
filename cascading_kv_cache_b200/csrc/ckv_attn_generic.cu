// Plain CUDA-core attention over the cascading cache for every dtype, head_dim
// and chunk length: the path used for fp32 caches and odd head sizes, and the
// in-library cross-check of the tuned kernels.  It follows the reference's eager
// attention (cascade/models/cascade_attention.py:250-340) step by step and rounds
// to the activation dtype wherever a torch op boundary does.
//
// Kernels (all on the caller's stream, scratch in the caller's workspace):
//   1. rope_gather : rotate+scale q and the keys of [sinks | cache | new] at their
//                    cache positions into scratch            (:141-166, :284-291)
//   2. attn_rows   : one warp per query row, online softmax  (:293-313)
//   3. col_scores  : one warp per key column, EMA scores     (:315-323)
//   4. reduce_ema  : head reduction + score-cache decay      (:231-248, :329-330)
//   5. the cache update (ckv_update.cu)
#include "ckv_common.cuh"

namespace ckv {

namespace {

struct GenericParams {
    // inputs
    const void *q, *key, *val;
    long long qsb, qsh, qst, ksb, ksh, kst;  // elements
    const void *rope;
    long long rope_rows;
    const float *ema_w_cache;
    const void *ema_w_new;
    void *out;
    long long osb, osh, ost;
    // state
    const void *sink_k, *sink_v, *cache_k, *cache_v;
    void *cache_s;
    const uint8_t *mask, *sink_mask;
    const long long *pos, *sink_pos, *stored_tokens, *stored_sinks, *seen;
    // scratch
    void *q_rs;      // [B,H,K,D]
    void *k_rot;     // [B,KVH,NS+S+K,D]
    float *row_m;    // [B,H,K]
    float *row_l;    // [B,H,K]
    float *raw;      // [B,H,S+K]
    void *new_scores;  // [B,KVH,K]
    int B, KVH, H, G, D, NS, W, C, S, K;
    int head_reduction, homogeneous;
    float rs;        // sqrt(1/sqrt(D))
    float beta_pow;  // beta^K
};

__device__ __forceinline__ void positions_from_counters(const GenericParams &p, long long &max_pos, long long &shift) {
    const long long seen = *p.seen;
    long long total = 0;
    for (int i = 0; i < p.C; ++i) total += p.stored_tokens[i];
    shift = seen > p.NS ? p.NS : 0;
    // max(sink_pos.amax(), key_pos.amax()) + 1 in closed form (cascade_attention.py:141-148)
    max_pos = seen == 0 ? 0 : (seen <= p.NS ? seen : p.NS + total);
}

template <typename T>
__global__ void rope_gather_kernel(GenericParams p) {
    long long max_pos, shift;
    positions_from_counters(p, max_pos, shift);
    const int half = p.D / 2;
    const int R = p.NS + p.S + p.K;
    const long long n_krows = (long long)p.B * p.KVH * R;
    const long long n_qrows = (long long)p.B * p.H * p.K;
    const long long total = (n_krows + n_qrows) * half;
    const T *rope = (const T *)p.rope;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long rowi = idx / half;
        const int i = (int)(idx % half);
        const T *src;
        T *dst;
        long long pos;
        if (rowi < n_krows) {
            const int r = (int)(rowi % R);
            const long long lane = rowi / R;
            const int b = (int)(lane / p.KVH), h = (int)(lane % p.KVH);
            if (r < p.NS) {
                src = (const T *)p.sink_k + (lane * p.NS + r) * p.D;
                pos = p.sink_pos[r];
            } else if (r < p.NS + p.S) {
                src = (const T *)p.cache_k + (lane * p.S + (r - p.NS)) * p.D;
                pos = p.pos[r - p.NS] + shift;
            } else {
                const int j = r - p.NS - p.S;
                src = (const T *)p.key + b * p.ksb + h * p.ksh + j * p.kst;
                pos = max_pos + j;
            }
            dst = (T *)p.k_rot + rowi * p.D;
        } else {
            const long long qr = rowi - n_krows;
            const int j = (int)(qr % p.K);
            const long long bh = qr / p.K;
            const int b = (int)(bh / p.H), h = (int)(bh % p.H);
            src = (const T *)p.q + b * p.qsb + h * p.qsh + j * p.qst;
            pos = max_pos + j;
            dst = (T *)p.q_rs + qr * p.D;
        }
        if (pos < 0) pos = 0;
        if (pos >= p.rope_rows) pos = p.rope_rows - 1;
        const float c = Elem<T>::to_f(rope[pos * p.D + i]);
        const float s = Elem<T>::to_f(rope[pos * p.D + half + i]);
        const float lo = Elem<T>::to_f(src[i]);
        const float hi = Elem<T>::to_f(src[i + half]);
        // x*cos + rotate_half(x)*sin, each product and the sum rounded to T, then * sqrt(scale)
        const float rlo = rnd<T>(__fadd_rn(rnd<T>(__fmul_rn(lo, c)), rnd<T>(__fmul_rn(-hi, s))));
        const float rhi = rnd<T>(__fadd_rn(rnd<T>(__fmul_rn(hi, c)), rnd<T>(__fmul_rn(lo, s))));
        dst[i] = Elem<T>::from_f(__fmul_rn(rlo, p.rs));
        dst[i + half] = Elem<T>::from_f(__fmul_rn(rhi, p.rs));
    }
}

constexpr int kMaxDPerLane = 8;  // head_dim up to 256

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <typename T>
__device__ __forceinline__ const T *value_row(const GenericParams &p, long long lane, int b, int h, int r) {
    if (r < p.NS) return (const T *)p.sink_v + (lane * p.NS + r) * p.D;
    if (r < p.NS + p.S) return (const T *)p.cache_v + (lane * p.S + (r - p.NS)) * p.D;
    return (const T *)p.val + b * p.ksb + h * p.ksh + (long long)(r - p.NS - p.S) * p.kst;
}

__device__ __forceinline__ bool key_valid(const GenericParams &p, int r, int qrow) {
    if (r < p.NS) return p.sink_mask[r] == 0;
    if (r < p.NS + p.S) return p.mask[r - p.NS] == 0;
    return (r - p.NS - p.S) <= qrow;
}

// One warp per (b, h, q): logits rounded to T as the einsum output is, softmax in fp32.
template <typename T>
__global__ void __launch_bounds__(128) attn_rows_kernel(GenericParams p) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane_id = threadIdx.x & 31;
    const long long n_rows = (long long)p.B * p.H * p.K;
    if (warp >= n_rows) return;
    const int qi = warp % p.K;
    const int bh = warp / p.K;
    const int b = bh / p.H, h = bh % p.H;
    const int kvh = h / p.G;
    const long long lane = (long long)b * p.KVH + kvh;
    const int R = p.NS + p.S + p.K;
    const T *qrow = (const T *)p.q_rs + (long long)warp * p.D;
    const T *krows = (const T *)p.k_rot + lane * R * p.D;
    float qv[kMaxDPerLane], acc[kMaxDPerLane];
#pragma unroll
    for (int e = 0; e < kMaxDPerLane; ++e) {
        const int d = lane_id + 32 * e;
        qv[e] = d < p.D ? Elem<T>::to_f(qrow[d]) : 0.f;
        acc[e] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const int r_end = p.NS + p.S + qi + 1;
    for (int r = 0; r < r_end; ++r) {
        if (!key_valid(p, r, qi)) continue;
        const T *kr = krows + (long long)r * p.D;
        float part = 0.f;
#pragma unroll
        for (int e = 0; e < kMaxDPerLane; ++e) {
            const int d = lane_id + 32 * e;
            if (d < p.D) part = fmaf(qv[e], Elem<T>::to_f(kr[d]), part);
        }
        const float s = rnd<T>(warp_sum(part));
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);
        const float pr = expf(s - m_new);
        l = l * corr + pr;
        const T *vr = value_row<T>(p, lane, b, kvh, r);
#pragma unroll
        for (int e = 0; e < kMaxDPerLane; ++e) {
            const int d = lane_id + 32 * e;
            if (d < p.D) acc[e] = acc[e] * corr + pr * Elem<T>::to_f(vr[d]);
        }
        m = m_new;
    }
    T *orow = (T *)p.out + b * p.osb + h * p.osh + (long long)qi * p.ost;
    const float inv = 1.f / l;
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

// One warp per (b, h, column): column = cache slot (0..S-1) or new token (S..S+K-1).
//   cached slot : sum_q float(T(p[q,col])) * w_cache[q]            -> T   (cascade_attention.py:315-320)
//   new token i : sum_{q>=i} float(T(T(p[q,i]) * w_new[q-i]))      -> T   (:322-323)
template <typename T>
__global__ void __launch_bounds__(128) col_scores_kernel(GenericParams p) {
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane_id = threadIdx.x & 31;
    const int ncol = p.S + p.K;
    const long long n = (long long)p.B * p.H * ncol;
    if (warp >= n) return;
    const int col = (int)(warp % ncol);
    const int bh = (int)(warp / ncol);
    const int b = bh / p.H, h = bh % p.H;
    const int kvh = h / p.G;
    const long long lane = (long long)b * p.KVH + kvh;
    const int R = p.NS + p.S + p.K;
    const bool is_new = col >= p.S;
    const int r = p.NS + col;
    float result = 0.f;
    if (is_new || p.mask[col] == 0) {
        const T *kr = (const T *)p.k_rot + (lane * R + r) * p.D;
        float kv[kMaxDPerLane];
#pragma unroll
        for (int e = 0; e < kMaxDPerLane; ++e) {
            const int d = lane_id + 32 * e;
            kv[e] = d < p.D ? Elem<T>::to_f(kr[d]) : 0.f;
        }
        const int q0 = is_new ? col - p.S : 0;
        const T *w_new = (const T *)p.ema_w_new;
        float sum = 0.f;
        for (int qi = q0; qi < p.K; ++qi) {
            const long long row = (long long)bh * p.K + qi;
            const T *qrow = (const T *)p.q_rs + row * p.D;
            float part = 0.f;
#pragma unroll
            for (int e = 0; e < kMaxDPerLane; ++e) {
                const int d = lane_id + 32 * e;
                if (d < p.D) part = fmaf(Elem<T>::to_f(qrow[d]), kv[e], part);
            }
            const float s = rnd<T>(warp_sum(part));
            const float pr = rnd<T>(expf(s - p.row_m[row]) / p.row_l[row]);
            if (is_new) sum += rnd<T>(__fmul_rn(pr, Elem<T>::to_f(w_new[qi - q0])));
            else sum = fmaf(pr, p.ema_w_cache[qi], sum);
        }
        result = rnd<T>(sum);
    }
    if (lane_id == 0) p.raw[warp] = result;
}

__device__ __forceinline__ float reduce_heads(const float *v, int n, int how) {
    if (how == CKV_REDUCE_MAX) {
        float m = v[0];
        for (int i = 1; i < n; ++i) m = fmaxf(m, v[i]);
        return m;
    }
    if (how == CKV_REDUCE_MEAN) {
        float s = 0.f;
        for (int i = 0; i < n; ++i) s += v[i];
        return s / (float)n;
    }
    // lower median, as torch.median returns for an even count
    const int want = (n - 1) / 2;
    for (int i = 0; i < n; ++i) {
        int less = 0, eq = 0;
        for (int j = 0; j < n; ++j) {
            less += v[j] < v[i];
            eq += v[j] == v[i];
        }
        if (less <= want && want < less + eq) return v[i];
    }
    return v[0];
}

constexpr int kMaxReduceHeads = 128;

// One thread per (b, kv_head, column): reduce the per-head scores over the group
// (or over all heads), then  score_cache = T(T(beta^K * score_cache) + ema)  for
// cached slots and write the reduced new-token scores for the update.
template <typename T>
__global__ void reduce_ema_kernel(GenericParams p) {
    const int ncol = p.S + p.K;
    const long long n = (long long)p.B * p.KVH * ncol;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const int col = (int)(idx % ncol);
    const int bk = (int)(idx / ncol);
    const int b = bk / p.KVH, kvh = bk % p.KVH;
    float v[kMaxReduceHeads];
    const int cnt = p.homogeneous ? p.H : p.G;
    const int h0 = p.homogeneous ? 0 : kvh * p.G;
    for (int i = 0; i < cnt; ++i) v[i] = p.raw[((long long)b * p.H + h0 + i) * ncol + col];
    const float red = rnd<T>(reduce_heads(v, cnt, p.head_reduction));
    if (col < p.S) {
        T *sc = (T *)p.cache_s + (long long)bk * p.S + col;
        const float decayed = rnd<T>(__fmul_rn(Elem<T>::to_f(*sc), p.beta_pow));
        *sc = Elem<T>::from_f(__fadd_rn(decayed, red));
    } else {
        ((T *)p.new_scores)[(long long)bk * p.K + (col - p.S)] = Elem<T>::from_f(red);
    }
}

size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

struct Scratch {
    size_t q_rs, k_rot, row_m, row_l, raw, new_scores, upd, upd_bytes, total;
};

Scratch scratch_layout(const Dims &d, int K) {
    Scratch s;
    size_t off = 256;  // the first 256 bytes of every attention workspace hold the status word
    s.q_rs = off; off += align_up((size_t)d.B * d.H * K * d.D * d.esz);
    s.k_rot = off; off += align_up((size_t)d.B * d.KVH * (d.NS + d.S + K) * d.D * d.esz);
    s.row_m = off; off += align_up((size_t)d.B * d.H * K * 4);
    s.row_l = off; off += align_up((size_t)d.B * d.H * K * 4);
    s.raw = off; off += align_up((size_t)d.B * d.H * (d.S + K) * 4);
    s.new_scores = off; off += align_up((size_t)d.B * d.KVH * K * d.esz);
    s.upd_bytes = update_chunk_workspace_bytes(d, K);
    s.upd = off; off += s.upd_bytes;
    s.total = off;
    return s;
}

template <typename T>
int run_generic(const Dims &d, GenericParams &p, bool ema, cudaStream_t stream) {
    const int half = d.D / 2;
    const long long rope_work = ((long long)d.B * d.KVH * (d.NS + d.S + p.K) + (long long)d.B * d.H * p.K) * half;
    int blocks = (int)((rope_work + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    rope_gather_kernel<T><<<blocks, 256, 0, stream>>>(p);
    CKV_CUDA_CHECK(cudaGetLastError());
    const long long n_rows = (long long)d.B * d.H * p.K;
    ProfileHook *hook = active_profile_hook();
    if (hook) hook->before(stream, "attn_rows_kernel");
    attn_rows_kernel<T><<<(unsigned)((n_rows + 3) / 4), 128, 0, stream>>>(p);
    if (hook) hook->after(stream);
    CKV_CUDA_CHECK(cudaGetLastError());
    if (ema) {
        const long long n_cols = (long long)d.B * d.H * (d.S + p.K);
        col_scores_kernel<T><<<(unsigned)((n_cols + 3) / 4), 128, 0, stream>>>(p);
        CKV_CUDA_CHECK(cudaGetLastError());
        const long long n_red = (long long)d.B * d.KVH * (d.S + p.K);
        reduce_ema_kernel<T><<<(unsigned)((n_red + 127) / 128), 128, 0, stream>>>(p);
        CKV_CUDA_CHECK(cudaGetLastError());
    }
    note_launches(ema ? 4 : 2);
    return CKV_OK;
}

}  // namespace

size_t generic_workspace_bytes(const Dims &d, int n_tokens) { return scratch_layout(d, n_tokens).total; }

int launch_attention_generic(const Dims &d, const ckv_layer_state *st, const void *q, int64_t qsb, int64_t qsh,
                             int64_t qst, const void *key, const void *value, int64_t ksb, int64_t ksh, int64_t kst,
                             int n_tokens, const void *rope, int64_t rope_rows, const float *ema_w_cache,
                             const void *ema_w_new, void *out, int64_t osb, int64_t osh, int64_t ost, void *workspace,
                             size_t workspace_bytes, int flags, cudaStream_t stream) {
    if (d.D % 2 != 0 || d.D > 32 * kMaxDPerLane)
        return fail(CKV_E_UNSUPPORTED, "head_dim %d: need an even value up to %d", d.D, 32 * kMaxDPerLane);
    const bool update = (flags & CKV_ATTN_UPDATE) != 0;
    const bool ema = update && d.admission == CKV_ADMIT_EMA;
    if (ema && (!ema_w_cache || !ema_w_new)) return fail(CKV_E_ARG, "EMA rule needs ema_w_cache and ema_w_new");
    if (ema && (d.homogeneous ? d.H : d.G) > kMaxReduceHeads)
        return fail(CKV_E_UNSUPPORTED, "head reduction over more than %d heads", kMaxReduceHeads);
    const Scratch s = scratch_layout(d, n_tokens);
    if (workspace_bytes < s.total || !workspace)
        return fail(CKV_E_WORKSPACE, "workspace of %zu bytes, need %zu", workspace_bytes, s.total);
    if (rope_rows <= (int64_t)d.NS + d.S + n_tokens)
        return fail(CKV_E_ARG, "rope table has %lld rows, need more than %d", (long long)rope_rows,
                    d.NS + d.S + n_tokens);
    uint8_t *ws = (uint8_t *)workspace;
    CKV_CUDA_CHECK(cudaMemsetAsync(ws, 0, 4, stream));
    GenericParams p;
    p.q = q; p.key = key; p.val = value;
    p.qsb = qsb; p.qsh = qsh; p.qst = qst; p.ksb = ksb; p.ksh = ksh; p.kst = kst;
    p.rope = rope; p.rope_rows = rope_rows;
    p.ema_w_cache = ema_w_cache; p.ema_w_new = ema_w_new;
    p.out = out; p.osb = osb; p.osh = osh; p.ost = ost;
    p.sink_k = st->sink_keys; p.sink_v = st->sink_values; p.cache_k = st->key_cache; p.cache_v = st->value_cache;
    p.cache_s = st->score_cache;
    p.mask = st->mask; p.sink_mask = st->sink_mask;
    p.pos = (const long long *)st->pos; p.sink_pos = (const long long *)st->sink_pos;
    p.stored_tokens = (const long long *)st->stored_tokens;
    p.stored_sinks = (const long long *)st->stored_sinks;
    p.seen = (const long long *)st->seen_tokens;
    p.q_rs = ws + s.q_rs; p.k_rot = ws + s.k_rot;
    p.row_m = (float *)(ws + s.row_m); p.row_l = (float *)(ws + s.row_l);
    p.raw = (float *)(ws + s.raw); p.new_scores = ws + s.new_scores;
    p.B = d.B; p.KVH = d.KVH; p.H = d.H; p.G = d.G; p.D = d.D; p.NS = d.NS; p.W = d.W; p.C = d.C; p.S = d.S;
    p.K = n_tokens;
    p.head_reduction = d.head_reduction; p.homogeneous = d.homogeneous;
    p.rs = (float)sqrt(1.0 / sqrt((double)d.D));
    p.beta_pow = (float)pow(d.beta, (double)n_tokens);
    int rc;
    if (d.dtype == CKV_F32) rc = run_generic<float>(d, p, ema, stream);
    else if (d.dtype == CKV_F16) rc = run_generic<__half>(d, p, ema, stream);
    else rc = run_generic<__nv_bfloat16>(d, p, ema, stream);
    if (rc != CKV_OK) return rc;
    if (update) {
        const void *scores = ema ? p.new_scores : nullptr;
        return launch_update(d, st, key, value, ksb, ksh, kst, scores, (int64_t)d.KVH * n_tokens, n_tokens, 1,
                             n_tokens, ws + s.upd, s.upd_bytes, stream);
    }
    return CKV_OK;
}

}  // namespace ckv
