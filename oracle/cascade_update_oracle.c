/*
 * TEST INFRASTRUCTURE ONLY -- CPU oracle for the cascading KV cache update.
 *
 * Plain-C restatement of the reference's per-lane cache update state machine
 * (cascade/models/cascading_cache.py: _update_kv_cache :145-299,
 * _update_kv_cache_inner :302-774, _update_sink_cache :22-109,
 * _update_positional_idx :112-142).  It is the checker the GPU kernels are
 * compared against and the CPU baseline that the benchmark times; nothing in
 * the shipped package links or calls it.
 *
 * Parity status: pinned.  tests/golden/ holds final cache states produced by
 * the reference's own PyTorch cache (CascadingKVCacheSlow,
 * cascading_cache.py:1496-1843) run on CPU, and tests/test_oracle.py checks
 * this file against them (stride rule).  The score-driven (EMA) branch has no
 * counterpart that the reference can run on a CPU; it follows :667-726 by
 * reading.
 *
 * One "lane" is one (batch, kv_head) pair.  All tensors are contiguous:
 *   key,val        [B,H,K,D]   element size esz (2 or 4 bytes), copied as bytes
 *   scr            [B,*,K]     incoming scores in the cache dtype, strides given
 *   sink_k,sink_v  [B,H,NS,D]
 *   cache_k,cache_v[B,H,S,D]   S = C*W
 *   cache_s        [B,H,S]     cache dtype
 *   sink_mask,mask [B,H,NS] / [B,H,S]  one byte per slot, 1 = empty
 *   sink_pos,pos,og_pos        int64
 *   stored_sinks [B,H], stored_tokens/start_indices [B,H,C]  int64
 *   every_n [C] int64
 */
#include <stdint.h>
#include <string.h>

enum { CKV_F32 = 0, CKV_F16 = 1, CKV_BF16 = 2 };

static float half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static float score_as_float(const uint8_t *p, int dtype) {
    float f;
    if (dtype == CKV_F32) {
        memcpy(&f, p, 4);
    } else if (dtype == CKV_BF16) {
        uint16_t h;
        memcpy(&h, p, 2);
        uint32_t bits = (uint32_t)h << 16;
        memcpy(&f, &bits, 4);
    } else {
        uint16_t h;
        memcpy(&h, p, 2);
        f = half_to_float(h);
    }
    return f;
}

static int64_t floor_mod(int64_t a, int64_t m) {
    int64_t r = a % m;
    return r < 0 ? r + m : r;
}

/* Returns 0 on success, a negative code on invalid arguments. */
int cascade_update_oracle(
    const uint8_t *key, const uint8_t *val,
    const uint8_t *scr, int64_t scr_stride_b, int64_t scr_stride_h, int64_t scr_stride_t,
    uint8_t *sink_k, uint8_t *sink_v,
    uint8_t *cache_k, uint8_t *cache_v, uint8_t *cache_s,
    uint8_t *sink_mask, uint8_t *mask,
    int64_t *sink_pos, int64_t *pos, int64_t *og_pos,
    int64_t *stored_sinks, int64_t *stored_tokens, int64_t *start_indices,
    const int64_t *every_n,
    int64_t B, int64_t H, int64_t K, int64_t D,
    int64_t NS, int64_t W, int64_t C,
    int64_t seen, int64_t max_seq_len, int eager_fill, int dtype)
{
    if (B <= 0 || H <= 0 || K <= 0 || D <= 0 || W <= 0 || C <= 0 || NS < 0) return -1;
    if (dtype != CKV_F32 && dtype != CKV_F16 && dtype != CKV_BF16) return -2;
    const int64_t esz = (dtype == CKV_F32) ? 4 : 2;
    const int64_t row = D * esz;
    const int64_t S = C * W;
    uint8_t carry_k[8192], carry_v[8192], tmp[8192];
    if (row > (int64_t)sizeof(carry_k)) return -3;

    for (int64_t b = 0; b < B; ++b) {
        for (int64_t h = 0; h < H; ++h) {
            const int64_t lane = b * H + h;
            uint8_t *ck = cache_k + lane * S * row;
            uint8_t *cv = cache_v + lane * S * row;
            uint8_t *cs = cache_s + lane * S * esz;
            uint8_t *mk = mask + lane * S;
            int64_t *ps = pos + lane * S;
            int64_t *og = og_pos + lane * S;
            int64_t *st = stored_tokens + lane * C;
            int64_t *sa = start_indices + lane * C;
            int pos_dirty = 0;

            for (int64_t j = 0; j < K; ++j) {
                /* cascading_cache.py:388  rti is the 1-based global index of this token */
                const int64_t rti = seen + j + 1;
                const uint8_t *kin = key + ((lane * K) + j) * row;
                const uint8_t *vin = val + ((lane * K) + j) * row;
                pos_dirty = 0;

                if (stored_sinks[lane] < NS) {
                    /* :22-109 */
                    int64_t s = stored_sinks[lane];
                    memcpy(sink_k + (lane * NS + s) * row, kin, row);
                    memcpy(sink_v + (lane * NS + s) * row, vin, row);
                    sink_pos[lane * NS + s] = s;
                    sink_mask[lane * NS + s] = 0;
                    stored_sinks[lane] = s + 1;
                    continue;
                }

                memcpy(carry_k, kin, row);
                memcpy(carry_v, vin, row);
                uint8_t carry_s[4];
                memcpy(carry_s, scr + (b * scr_stride_b + h * scr_stride_h + j * scr_stride_t) * esz, esz);
                int64_t carry_og = rti;
                /* :440,:471  every cascade accepts every token while the cache first fills */
                const int eager = eager_fill && (rti - 1 <= max_seq_len + NS);

                int64_t i = 0;
                int stop = 0;
                while (i < C && !stop) {
                    const int64_t l = i * W;
                    /* :477-478  the index of the INCOMING token decides, also for a carried evictee */
                    const int do_i = eager || (floor_mod(rti - 1 - NS, every_n[i]) == 0);
                    const int64_t stored_i = st[i];
                    const int64_t start_i = sa[i];
                    if (do_i && stored_i < W) {
                        /* :492-540 append */
                        int64_t t = l + start_i + stored_i;
                        memcpy(ck + t * row, carry_k, row);
                        memcpy(cv + t * row, carry_v, row);
                        memcpy(cs + t * esz, carry_s, esz);
                        og[t] = carry_og;
                        mk[t] = 0;
                        st[i] = stored_i + 1;
                        stop = 1;
                    } else if (do_i) {
                        /* :542-604 evict the oldest slot, carry it to the next cascade */
                        int64_t t = l + start_i;
                        uint8_t ns[4];
                        int64_t nog = og[t];
                        memcpy(tmp, ck + t * row, row);
                        memcpy(ck + t * row, carry_k, row);
                        memcpy(carry_k, tmp, row);
                        memcpy(tmp, cv + t * row, row);
                        memcpy(cv + t * row, carry_v, row);
                        memcpy(carry_v, tmp, row);
                        memcpy(ns, cs + t * esz, esz);
                        memcpy(cs + t * esz, carry_s, esz);
                        memcpy(carry_s, ns, esz);
                        og[t] = carry_og;
                        carry_og = nog;
                        sa[i] = (start_i + 1) % W;
                        i += 1;
                    } else if (stored_i == 0) {
                        /* :606-665 "eager add" into an empty cascade */
                        int64_t t = l + start_i + stored_i;
                        memcpy(ck + t * row, carry_k, row);
                        memcpy(cv + t * row, carry_v, row);
                        memcpy(cs + t * esz, carry_s, esz);
                        og[t] = carry_og;
                        mk[t] = 0;
                        st[i] = stored_i + 1;
                        stop = 1;
                    } else {
                        /* :667-726 compete with the newest slot; floor-mod as in the PyTorch path (:1461) */
                        int64_t t = l + floor_mod(start_i - 1, stored_i);
                        float snew = score_as_float(carry_s, dtype);
                        float sold = score_as_float(cs + t * esz, dtype);
                        if (snew >= sold) {
                            memcpy(ck + t * row, carry_k, row);
                            memcpy(cv + t * row, carry_v, row);
                            memcpy(cs + t * esz, carry_s, esz);
                            og[t] = carry_og;
                        }
                        stop = 1;
                    }
                }
                pos_dirty = 1;
            }

            /* :729-774  positions are rewritten after the last token of the call,
             * only when that token took the non-sink branch */
            if (pos_dirty) {
                int64_t pos_ub = 0;
                for (int64_t i = 0; i < C; ++i) pos_ub += st[i];
                for (int64_t i = 0; i < C; ++i) {
                    int64_t seg = st[i] < W ? st[i] : W;
                    if (seg <= 0) break; /* the reference never reaches an empty cascade here */
                    for (int64_t j = 0; j < W; ++j)
                        ps[i * W + j] = ((j + seg - sa[i]) % seg) + pos_ub - seg;
                    pos_ub -= W;
                    if (pos_ub <= 0) break;
                }
            }
        }
    }
    return 0;
}
