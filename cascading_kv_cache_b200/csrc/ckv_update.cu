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
#include "ckv_update_device.cuh"

namespace ckv {

namespace {

__global__ void __launch_bounds__(32) update_lanes_kernel(UpdateParams p) {
    __shared__ long long s_stored[CKV_MAX_CASCADES];
    __shared__ long long s_start[CKV_MAX_CASCADES];
    __shared__ long long s_every[CKV_MAX_CASCADES];
    update_lane_walk(p, blockIdx.x, s_stored, s_start, s_every);
}

struct FinalizeParams {
    long long *stored_tokens, *start_indices, *stored_sinks, *seen;
    const long long *every_n;
    long long *pos, *sink_pos;
    uint8_t *mask, *sink_mask;
    int K, NS, W, C, S, eager_fill;
};

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
            if (!CKV_COUNTERS_OK(s_stored[i], s_start[i], p.W)) s_stored[i] = s_start[i] = 0;   // keep what follows in range
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
    note_launches(2);
    return CKV_OK;
}

#ifdef CKV_BOUNDS
int read_bounds_status_serial(int *out) { return read_bounds_status_of_this_unit(out); }
#endif

}  // namespace ckv
