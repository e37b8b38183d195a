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

// ---- debug bounds checks (-DCKV_BOUNDS) ------------------------------------------------------------
// The stand-in for a memory checker on machines where none can be run: every slot index the update
// computes, and the counters it computes them from, are checked before use.  A violation records
// code 4 | (source line << 8) in a per-translation-unit status word and SKIPS the access; nothing
// traps.  ckv_bounds_status() (C ABI) reads and clears the words of all translation units.  In the
// ordinary build the checks compile to nothing.
#ifdef CKV_BOUNDS
static __device__ int g_bounds_status;
__device__ __forceinline__ bool bounds_ok(bool ok, int line) {
    if (!ok) atomicCAS(&g_bounds_status, 0, 4 | (line << 8));
    return ok;
}
#define CKV_IN_BOUNDS(cond) ::ckv::bounds_ok((cond), __LINE__)
static inline int read_bounds_status_of_this_unit(int *out) {
    int zero = 0;
    if (cudaMemcpyFromSymbol(out, g_bounds_status, sizeof(int)) != cudaSuccess) return -1;
    return cudaMemcpyToSymbol(g_bounds_status, &zero, sizeof(int)) == cudaSuccess ? 0 : -1;
}
#else
#define CKV_IN_BOUNDS(cond) true
#endif
// counters of one cascade: at most W tokens stored, ring start inside the window
#define CKV_COUNTERS_OK(stored, start, W) CKV_IN_BOUNDS((stored) >= 0 && (stored) <= (W) && (start) >= 0 && (start) < (W))

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
            if (!CKV_IN_BOUNDS(sinks >= 0)) return;
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
            if (!CKV_COUNTERS_OK(stored_i, start_i, p.W)) return;
            if ((do_i && stored_i < p.W) || (!do_i && stored_i == 0)) {
                const long long t = l + start_i + stored_i;
                if (!CKV_IN_BOUNDS(t < p.S)) return;
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

constexpr int kOneTokenMaxCascades = 8;

// One new token for one lane, rows of 256 bytes, at most kOneTokenMaxCascades cascades: the same
// result as update_lane_walk with K = 1, in one round trip to memory instead of one per cascade.
// Which slot each hop touches follows from the counters alone (the token ripples through the full
// cascades that accept it, then appends or competes with one newest slot), so a warp first reads the
// rows, scores and original positions of every slot on the path at once (thread t < 16 holds 16 bytes
// of each key row, t >= 16 of each value row), then resolves the carry chain in registers and issues
// all stores.  The slots lie in different cascades, so no store can precede a load of the same slot.
// s_stored / s_start / s_every hold the counters BEFORE the token (the caller has them in shared
// memory already), sinks / seen likewise; new_score is the token's incoming score (bits of the cache
// dtype), ignored under the stride rule (p.scr == nullptr means all-zero scores).
__device__ __forceinline__ void update_lane_one_token(const UpdateParams &p, int lane, const long long *s_stored,
                                                      const long long *s_start, const long long *s_every,
                                                      long long sinks, long long seen, unsigned int new_score) {
    const int b = lane / p.KVH, h = lane % p.KVH;
    const int tid = threadIdx.x & 31;
    const long long rti = seen + 1;
    const bool is_v = tid >= 16;
    const int chunk = tid & 15;
    const uint4 *src = reinterpret_cast<const uint4 *>((is_v ? p.val : p.key) + b * p.ksb + h * p.ksh);
    uint4 carry = src[chunk];
    if (sinks < p.NS) {
        if (!CKV_IN_BOUNDS(sinks >= 0)) return;
        uint8_t *dst = (is_v ? p.sink_v : p.sink_k) + ((long long)lane * p.NS + sinks) * 256;
        reinterpret_cast<uint4 *>(dst)[chunk] = carry;
        return;
    }
    uint8_t *rows = (is_v ? p.cache_v : p.cache_k) + (long long)lane * p.S * 256;
    uint8_t *cs = p.cache_s + (long long)lane * p.S * p.esz;
    long long *og = p.og_pos + (long long)lane * p.S;
    const bool eager = p.eager_fill && (rti - 1 <= (long long)p.S + p.NS);

    // the path: slot and kind of every hop (0 = append, 1 = evict and carry on, 2 = compete with the newest slot)
    int slot[kOneTokenMaxCascades], kind[kOneTokenMaxCascades];
    int n_hops = 0;
#pragma unroll
    for (int i = 0; i < kOneTokenMaxCascades; ++i) {
        slot[i] = 0;
        kind[i] = -1;
    }
    {
        bool done = false;
#pragma unroll
        for (int i = 0; i < kOneTokenMaxCascades; ++i) {
            if (i < p.C && !done) {
                const bool do_i = eager || (floor_mod_ll(rti - 1 - p.NS, s_every[i]) == 0);
                const long long stored_i = s_stored[i], start_i = s_start[i], l = (long long)i * p.W;
                if (!CKV_COUNTERS_OK(stored_i, start_i, p.W)) return;
                if ((do_i && stored_i < p.W) || (!do_i && stored_i == 0)) {
                    slot[i] = (int)(l + start_i + stored_i);
                    kind[i] = 0;
                    done = true;
                } else if (do_i) {
                    slot[i] = (int)(l + start_i);
                    kind[i] = 1;
                } else {
                    slot[i] = (int)(l + floor_mod_ll(start_i - 1, stored_i));
                    kind[i] = 2;
                    done = true;
                }
                n_hops = i + 1;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < kOneTokenMaxCascades; ++i)
        if (kind[i] >= 0 && !CKV_IN_BOUNDS(slot[i] >= 0 && slot[i] < p.S)) return;
    // one round of loads: the rows that move on, and the score / original position of every slot on the path
    uint4 row[kOneTokenMaxCascades];
#pragma unroll
    for (int i = 0; i < kOneTokenMaxCascades; ++i)
        if (kind[i] == 1) row[i] = reinterpret_cast<const uint4 *>(rows + (long long)slot[i] * 256)[chunk];
    unsigned int my_s = 0;
    long long my_og = 0;
#pragma unroll
    for (int i = 0; i < kOneTokenMaxCascades; ++i) {
        if (tid == i && kind[i] >= 1) {
            my_s = load_score_bits(cs + (long long)slot[i] * p.esz, p.esz);
            my_og = og[slot[i]];
        }
    }
    unsigned int carry_s = p.scr ? new_score : 0u;
    long long carry_og = rti;
    // resolve the chain and store
#pragma unroll
    for (int i = 0; i < kOneTokenMaxCascades; ++i) {
        if (i < n_hops) {
            const unsigned int slot_s = __shfl_sync(0xffffffffu, my_s, i);
            const long long slot_og = __shfl_sync(0xffffffffu, my_og, i);
            bool write = true;
            if (kind[i] == 2)
                write = score_bits_to_float(carry_s, p.dtype) >= score_bits_to_float(slot_s, p.dtype);
            if (write) {
                reinterpret_cast<uint4 *>(rows + (long long)slot[i] * 256)[chunk] = carry;
                if (tid == 0) {
                    store_score_bits(cs + (long long)slot[i] * p.esz, carry_s, p.esz);
                    og[slot[i]] = carry_og;
                }
            }
            if (kind[i] == 1) {
                carry = row[i];
                carry_s = slot_s;
                carry_og = slot_og;
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
