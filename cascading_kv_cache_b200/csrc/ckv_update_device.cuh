// Device-side pieces of the cascade update shared by the chunk update kernels and the
// fused decode kernel: the per-lane token walk and the lane-invariant counter advance.
// Semantics: cascade/models/cascading_cache.py:381-774 of the reference (see ckv_update.cu).
#pragma once

#include "ckv_common.cuh"

namespace ckv {

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

// Walk the K tokens of one lane in stream order with one warp (all 32 threads call this with the
// same arguments).  s_stored / s_start / s_every are per-warp shared scratch of CKV_MAX_CASCADES
// entries; the lane-invariant counters in global memory are only read.
__device__ __forceinline__ void update_lane_walk(const UpdateParams &p, int lane, long long *s_stored,
                                                 long long *s_start, long long *s_every) {
    const int b = lane / p.KVH, h = lane % p.KVH;
    const int tid = threadIdx.x & 31;
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

// Advance the lane-invariant counters by K tokens.  The branch taken by each
// token depends only on its stream index and the counters, never on scores.
static __device__ void advance_counters(long long *stored, long long *start, long long &sinks, long long seen,
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


}  // namespace ckv
