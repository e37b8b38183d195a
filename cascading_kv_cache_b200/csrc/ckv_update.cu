// Cascade cache update for chunks of any length: one warp per lane walks the
// tokens of the chunk in stream order and moves rows; a second, single-block
// kernel advances the lane-invariant counters and rewrites positions / masks.
//
// Semantics follow the reference state machine
// (cascade/models/cascading_cache.py:381-774) case by case:
//   sink fill (:399-431), append (:492-540), evict-and-carry (:542-604),
//   add into an empty cascade (:606-665), compete with the newest slot
//   (:667-726, floor-mod slot index as in the PyTorch path :1461),
//   position rewrite after the last token of the call (:729-774, :112-142).
#include <stdarg.h>
#include <stdio.h>

#include "ckv_common.cuh"

namespace ckv {

namespace {

struct UpdateParams {
    const uint8_t *key, *val;
    long long ksb, ksh, kst;  // bytes
    const uint8_t *scr;       // may be null (all-zero scores)
    long long ssb, ssh, sst;  // bytes
    uint8_t *sink_k, *sink_v, *cache_k, *cache_v, *cache_s;
    long long *og_pos;
    const long long *stored_tokens, *start_indices, *stored_sinks, *seen, *every_n;
    int KVH, K, NS, W, C, S, row_bytes, esz, dtype, eager_fill;
};

__device__ __forceinline__ float score_bits_to_float(unsigned int bits, int dtype) {
    if (dtype == CKV_F32) return __uint_as_float(bits);
    if (dtype == CKV_BF16) return __uint_as_float(bits << 16);
    return __half2float(__ushort_as_half((unsigned short)bits));
}

__device__ __forceinline__ unsigned int load_score_bits(const uint8_t *p, int esz) {
    return esz == 4 ? *reinterpret_cast<const unsigned int *>(p)
                    : (unsigned int)*reinterpret_cast<const unsigned short *>(p);
}

__device__ __forceinline__ void store_score_bits(uint8_t *p, unsigned int bits, int esz) {
    if (esz == 4) *reinterpret_cast<unsigned int *>(p) = bits;
    else *reinterpret_cast<unsigned short *>(p) = (unsigned short)bits;
}

constexpr int kMaxChunksPerThread = 4;  // rows of up to 32 * 4 * 16 = 2048 bytes

__global__ void __launch_bounds__(32) update_lanes_kernel(UpdateParams p) {
    __shared__ long long s_stored[CKV_MAX_CASCADES];
    __shared__ long long s_start[CKV_MAX_CASCADES];
    __shared__ long long s_every[CKV_MAX_CASCADES];
    const int lane = blockIdx.x;
    const int b = lane / p.KVH, h = lane % p.KVH;
    const int tid = threadIdx.x;
    for (int i = tid; i < p.C; i += 32) {
        s_stored[i] = p.stored_tokens[i];
        s_start[i] = p.start_indices[i];
        s_every[i] = p.every_n[i];
    }
    __syncwarp();
    long long sinks = *p.stored_sinks;
    const long long seen = *p.seen;
    const int nchunk = p.row_bytes / 16;
    const long long row = p.row_bytes;
    uint8_t *ck = p.cache_k + (long long)lane * p.S * row;
    uint8_t *cv = p.cache_v + (long long)lane * p.S * row;
    uint8_t *cs = p.cache_s + (long long)lane * p.S * p.esz;
    long long *og = p.og_pos + (long long)lane * p.S;

    for (int j = 0; j < p.K; ++j) {
        const long long rti = seen + j + 1;
        const uint4 *kin = reinterpret_cast<const uint4 *>(p.key + b * p.ksb + h * p.ksh + j * p.kst);
        const uint4 *vin = reinterpret_cast<const uint4 *>(p.val + b * p.ksb + h * p.ksh + j * p.kst);
        uint4 carry_k[kMaxChunksPerThread], carry_v[kMaxChunksPerThread];
#pragma unroll
        for (int c = 0; c < kMaxChunksPerThread; ++c) {
            int idx = tid + 32 * c;
            if (idx < nchunk) {
                carry_k[c] = kin[idx];
                carry_v[c] = vin[idx];
            }
        }
        if (sinks < p.NS) {
            uint4 *dk = reinterpret_cast<uint4 *>(p.sink_k + ((long long)lane * p.NS + sinks) * row);
            uint4 *dv = reinterpret_cast<uint4 *>(p.sink_v + ((long long)lane * p.NS + sinks) * row);
#pragma unroll
            for (int c = 0; c < kMaxChunksPerThread; ++c) {
                int idx = tid + 32 * c;
                if (idx < nchunk) {
                    dk[idx] = carry_k[c];
                    dv[idx] = carry_v[c];
                }
            }
            sinks += 1;
            continue;
        }
        unsigned int carry_s = 0;
        if (p.scr) carry_s = load_score_bits(p.scr + b * p.ssb + h * p.ssh + j * p.sst, p.esz);
        long long carry_og = rti;
        const bool eager = p.eager_fill && (rti - 1 <= (long long)p.S + p.NS);

        int i = 0;
        while (i < p.C) {
            const long long l = (long long)i * p.W;
            const bool do_i = eager || (floor_mod_ll(rti - 1 - p.NS, s_every[i]) == 0);
            const long long stored_i = s_stored[i];
            const long long start_i = s_start[i];
            if ((do_i && stored_i < p.W) || (!do_i && stored_i == 0)) {
                const long long t = l + start_i + stored_i;
                uint4 *dk = reinterpret_cast<uint4 *>(ck + t * row);
                uint4 *dv = reinterpret_cast<uint4 *>(cv + t * row);
#pragma unroll
                for (int c = 0; c < kMaxChunksPerThread; ++c) {
                    int idx = tid + 32 * c;
                    if (idx < nchunk) {
                        dk[idx] = carry_k[c];
                        dv[idx] = carry_v[c];
                    }
                }
                __syncwarp();
                if (tid == 0) {
                    store_score_bits(cs + t * p.esz, carry_s, p.esz);
                    og[t] = carry_og;
                    s_stored[i] = stored_i + 1;
                }
                __syncwarp();
                break;
            } else if (do_i) {
                const long long t = l + start_i;
                uint4 *dk = reinterpret_cast<uint4 *>(ck + t * row);
                uint4 *dv = reinterpret_cast<uint4 *>(cv + t * row);
#pragma unroll
                for (int c = 0; c < kMaxChunksPerThread; ++c) {
                    int idx = tid + 32 * c;
                    if (idx < nchunk) {
                        uint4 tk = dk[idx], tv = dv[idx];
                        dk[idx] = carry_k[c];
                        dv[idx] = carry_v[c];
                        carry_k[c] = tk;
                        carry_v[c] = tv;
                    }
                }
                const unsigned int next_s = load_score_bits(cs + t * p.esz, p.esz);
                const long long next_og = og[t];
                __syncwarp();
                if (tid == 0) {
                    store_score_bits(cs + t * p.esz, carry_s, p.esz);
                    og[t] = carry_og;
                    s_start[i] = (start_i + 1) % p.W;
                }
                __syncwarp();
                carry_s = next_s;
                carry_og = next_og;
                i += 1;
            } else {
                const long long t = l + floor_mod_ll(start_i - 1, stored_i);
                const unsigned int old_s = load_score_bits(cs + t * p.esz, p.esz);
                if (score_bits_to_float(carry_s, p.dtype) >= score_bits_to_float(old_s, p.dtype)) {
                    uint4 *dk = reinterpret_cast<uint4 *>(ck + t * row);
                    uint4 *dv = reinterpret_cast<uint4 *>(cv + t * row);
#pragma unroll
                    for (int c = 0; c < kMaxChunksPerThread; ++c) {
                        int idx = tid + 32 * c;
                        if (idx < nchunk) {
                            dk[idx] = carry_k[c];
                            dv[idx] = carry_v[c];
                        }
                    }
                    __syncwarp();
                    if (tid == 0) {
                        store_score_bits(cs + t * p.esz, carry_s, p.esz);
                        og[t] = carry_og;
                    }
                }
                __syncwarp();
                break;
            }
        }
    }
}

struct FinalizeParams {
    long long *stored_tokens, *start_indices, *stored_sinks, *seen;
    const long long *every_n;
    long long *pos, *sink_pos;
    uint8_t *mask, *sink_mask;
    int K, NS, W, C, S, eager_fill;
};

// Advance the lane-invariant counters by K tokens.  The branch taken by each
// token depends only on its stream index and the counters, never on scores.
__device__ void advance_counters(long long *stored, long long *start, long long &sinks, long long seen,
                                 const long long *every_n, int K, int NS, int W, int C, int S, int eager_fill) {
    for (int j = 0; j < K; ++j) {
        const long long rti = seen + j + 1;
        if (sinks < NS) {
            sinks += 1;
            continue;
        }
        const bool eager = eager_fill && (rti - 1 <= (long long)S + NS);
        int i = 0;
        while (i < C) {
            const bool do_i = eager || (floor_mod_ll(rti - 1 - NS, every_n[i]) == 0);
            if ((do_i && stored[i] < W) || (!do_i && stored[i] == 0)) {
                stored[i] += 1;
                break;
            } else if (do_i) {
                start[i] = (start[i] + 1) % W;
                i += 1;
            } else {
                break;
            }
        }
    }
}

__global__ void __launch_bounds__(256) update_finalize_kernel(FinalizeParams p) {
    __shared__ long long s_stored[CKV_MAX_CASCADES];
    __shared__ long long s_start[CKV_MAX_CASCADES];
    __shared__ long long s_every[CKV_MAX_CASCADES];
    __shared__ long long s_sinks, s_seen, s_total;
    const int tid = threadIdx.x;
    if (tid == 0) {
        for (int i = 0; i < p.C; ++i) {
            s_stored[i] = p.stored_tokens[i];
            s_start[i] = p.start_indices[i];
            s_every[i] = p.every_n[i];
        }
        long long sinks = *p.stored_sinks;
        const long long seen = *p.seen;
        advance_counters(s_stored, s_start, sinks, seen, s_every, p.K, p.NS, p.W, p.C, p.S, p.eager_fill);
        long long total = 0;
        for (int i = 0; i < p.C; ++i) {
            p.stored_tokens[i] = s_stored[i];
            p.start_indices[i] = s_start[i];
            total += s_stored[i];
        }
        *p.stored_sinks = sinks;
        *p.seen = seen + p.K;
        s_sinks = sinks;
        s_seen = seen + p.K;
        s_total = total;
    }
    __syncthreads();
    for (int s = tid; s < p.NS; s += blockDim.x) {
        if (s < s_sinks) {
            p.sink_pos[s] = s;
            p.sink_mask[s] = 0;
        }
    }
    // positions are rewritten only when the last token of the call went past the sinks
    const bool rewrite = s_seen > p.NS;
    for (int t = tid; t < p.S; t += blockDim.x) {
        const int i = t / p.W, j = t % p.W;
        const long long stored_i = s_stored[i];
        if (j < stored_i) p.mask[t] = 0;
        const long long ub = s_total - (long long)i * p.W;
        const long long seg = stored_i < p.W ? stored_i : p.W;
        if (rewrite && ub > 0 && seg > 0) p.pos[t] = ((j + seg - s_start[i]) % seg) + ub - seg;
    }
}

}  // namespace

int launch_update_serial(const Dims &d, const ckv_layer_state *st, const void *key, const void *value, int64_t ksb,
                         int64_t ksh, int64_t kst, const void *scores, int64_t ssb, int64_t ssh, int64_t sst,
                         int n_tokens, cudaStream_t stream) {
    const int row_bytes = d.D * d.esz;
    if (row_bytes % 16 != 0 || row_bytes > 32 * kMaxChunksPerThread * 16)
        return fail(CKV_E_UNSUPPORTED, "row of %d bytes: need a multiple of 16 and at most %d", row_bytes,
                    32 * kMaxChunksPerThread * 16);
    if (((uintptr_t)key | (uintptr_t)value) % 16 != 0 || (ksb * d.esz) % 16 || (ksh * d.esz) % 16 ||
        (kst * d.esz) % 16)
        return fail(CKV_E_ARG, "key/value rows must be 16-byte aligned");
    UpdateParams p;
    p.key = (const uint8_t *)key; p.val = (const uint8_t *)value;
    p.ksb = ksb * d.esz; p.ksh = ksh * d.esz; p.kst = kst * d.esz;
    p.scr = (const uint8_t *)scores;
    p.ssb = ssb * d.esz; p.ssh = ssh * d.esz; p.sst = sst * d.esz;
    p.sink_k = (uint8_t *)st->sink_keys; p.sink_v = (uint8_t *)st->sink_values;
    p.cache_k = (uint8_t *)st->key_cache; p.cache_v = (uint8_t *)st->value_cache;
    p.cache_s = (uint8_t *)st->score_cache;
    p.og_pos = (long long *)st->og_pos;
    p.stored_tokens = (const long long *)st->stored_tokens;
    p.start_indices = (const long long *)st->start_indices;
    p.stored_sinks = (const long long *)st->stored_sinks;
    p.seen = (const long long *)st->seen_tokens;
    p.every_n = (const long long *)st->every_n;
    p.KVH = d.KVH; p.K = n_tokens; p.NS = d.NS; p.W = d.W; p.C = d.C; p.S = d.S;
    p.row_bytes = row_bytes; p.esz = d.esz; p.dtype = d.dtype; p.eager_fill = d.eager_fill;
    update_lanes_kernel<<<d.B * d.KVH, 32, 0, stream>>>(p);
    CKV_CUDA_CHECK(cudaGetLastError());

    FinalizeParams f;
    f.stored_tokens = (long long *)st->stored_tokens; f.start_indices = (long long *)st->start_indices;
    f.stored_sinks = (long long *)st->stored_sinks; f.seen = (long long *)st->seen_tokens;
    f.every_n = (const long long *)st->every_n;
    f.pos = (long long *)st->pos; f.sink_pos = (long long *)st->sink_pos;
    f.mask = st->mask; f.sink_mask = st->sink_mask;
    f.K = n_tokens; f.NS = d.NS; f.W = d.W; f.C = d.C; f.S = d.S; f.eager_fill = d.eager_fill;
    update_finalize_kernel<<<1, 256, 0, stream>>>(f);
    CKV_CUDA_CHECK(cudaGetLastError());
    return CKV_OK;
}

}  // namespace ckv
