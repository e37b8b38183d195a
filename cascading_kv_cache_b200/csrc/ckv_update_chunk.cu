// Parallel cascade cache update for chunks (the fast path of ckv_cascade_update).
//
// The reference walks the chunk token by token per lane (cascade/models/cascading_cache.py:223,
// :381-726).  Two facts make the walk parallel:
//   1. Which branch a token takes in cascade i (append, evict-and-carry, add-into-empty, compete)
//      depends only on its stream index and on counters, never on scores (:471-478, :491-492,
//      :606).  So for the stream of items E_i entering cascade i, "accept" flags are a pure
//      function of position; an exclusive prefix sum over them gives, for every item, the ring slot
//      it is written to, whether it pops the oldest entry, and therefore the stream E_{i+1}.
//   2. Non-accepted items compete with the NEWEST entry only (:667-726): the entry written by
//      accept number a ends up holding the arg-max of {that item, the competitors up to the next
//      accept}, ties going to the later item (score >= old_score, :699).  Each such group is
//      independent of all others.
// One CTA per lane runs C stages (flags -> block scan -> group winners -> popped items = next
// stream) on item ids in shared memory, recording (slot <- item) moves; rows, scores and original
// positions are then moved cascade by cascade from the last to the first, because an item only ever
// moves to a later cascade, so its source is still untouched when it is read.
// A single-block kernel repeats the score-free part to advance the lane-invariant counters.
#include "ckv_common.cuh"
#include "ckv_update_device.cuh"

namespace ckv {

namespace {

constexpr int kChunkMax = 4096;      // tokens per launch (larger chunks are split by the launcher)
constexpr int kThreads = 512;
constexpr int kItemsPerThread = kChunkMax / kThreads;
constexpr int kHdrInts = 2 * CKV_MAX_CASCADES + 1;
constexpr int kSplitMovesFrom = 1024;   // chunks at least this long run their moves as one launch per cascade
constexpr int kMoveBlocks = 32;         // CTAs per lane of such a launch

struct ChunkParams {
    UpdateParams u;
    int *plan;            // [lanes][plan_stride][2]  (destination slot, item id)
    int plan_stride;
    int *hdr;             // [lanes][kHdrInts]: moves of each cascade (offset, count) and the number of stages
    long long *pos, *sink_pos;
    long long *stored_tokens_w, *start_indices_w, *stored_sinks_w, *seen_w;
    uint8_t *mask, *sink_mask;
};

struct Shared {
    int T[2][kChunkMax];      // stream times: index of the chunk token whose arrival caused the event
    int ID[2][kChunkMax];     // stream items: chunk token j (< K) or pre-existing slot t (K + t)
    int ACC[kChunkMax + 1];   // exclusive prefix sum of the accept flags (ACC[L] = number of accepts)
    int WIN[kChunkMax];       // winner item of the group started by accept number a
    int scan_tmp[kThreads];
    long long count[CKV_MAX_CASCADES], start[CKV_MAX_CASCADES], every[CKV_MAX_CASCADES];
    int casc_off[CKV_MAX_CASCADES + 1], casc_cnt[CKV_MAX_CASCADES];
    int win_m1;               // winner of the group of the pre-existing newest entry, or -1
};

// Exclusive block scan of flags held as ACC[x] in {0,1} for x < L; writes ACC[0..L] in place.
__device__ void block_exclusive_scan(Shared &sh, int L) {
    const int tid = threadIdx.x;
    int local[kItemsPerThread];
    int sum = 0;
#pragma unroll
    for (int k = 0; k < kItemsPerThread; ++k) {
        const int x = tid * kItemsPerThread + k;
        local[k] = x < L ? sh.ACC[x] : 0;
        sum += local[k];
    }
    sh.scan_tmp[tid] = sum;
    __syncthreads();
    // scan of kThreads partial sums by the first warp (16 per lane)
    if (tid < 32) {
        constexpr int per = kThreads / 32;
        int part[per];
        int s = 0;
#pragma unroll
        for (int k = 0; k < per; ++k) {
            part[k] = sh.scan_tmp[tid * per + k];
            s += part[k];
        }
        int incl = s;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, off);
            if (tid >= off) incl += v;
        }
        int run = incl - s;
#pragma unroll
        for (int k = 0; k < per; ++k) {
            sh.scan_tmp[tid * per + k] = run;
            run += part[k];
        }
    }
    __syncthreads();
    int run = sh.scan_tmp[tid];
#pragma unroll
    for (int k = 0; k < kItemsPerThread; ++k) {
        const int x = tid * kItemsPerThread + k;
        if (x < L) sh.ACC[x] = run;
        run += local[k];
        if (x == L - 1) sh.ACC[L] = run;
    }
    if (L == 0 && tid == 0) sh.ACC[0] = 0;
    __syncthreads();
}

// Accept flag of stream element x of cascade i (score-free): eager fill, the stride test on the
// INCOMING token's index, or the first item into an empty cascade.
__device__ __forceinline__ int accept_flag(const UpdateParams &u, const Shared &sh, int i, int x, int j, long long seen) {
    const long long rti = seen + j + 1;
    const bool eager = u.eager_fill && (rti - 1 <= (long long)u.S + u.NS);
    const bool stride = floor_mod_ll(rti - 1 - u.NS, sh.every[i]) == 0;
    return (eager || stride || (x == 0 && sh.count[i] == 0)) ? 1 : 0;
}

__device__ __forceinline__ float item_score(const UpdateParams &u, int lane, int b, int h, int id) {
    unsigned int bits;
    if (id < u.K) bits = u.scr ? load_score_bits(u.scr + b * u.ssb + h * u.ssh + (long long)id * u.sst, u.esz) : 0u;
    else bits = load_score_bits(u.cache_s + ((long long)lane * u.S + (id - u.K)) * u.esz, u.esz);
    return score_bits_to_float(bits, u.dtype);
}

// One stage of the plan for cascade i over the stream (T[cur], ID[cur]) of length L.  Returns the
// length of the next stream.  With kData = false only the counters are advanced (no winners).
template <bool kData>
__device__ int cascade_stage(const ChunkParams &p, Shared &sh, int lane, int i, int cur, int L, long long seen,
                             int *plan_lane) {
    const UpdateParams &u = p.u;
    const int tid = threadIdx.x;
    const int b = lane / u.KVH, h = lane % u.KVH;
    const int W = u.W;
    const long long count0 = sh.count[i], start0 = sh.start[i];
    for (int x = tid; x < L; x += kThreads) sh.ACC[x] = accept_flag(u, sh, i, x, sh.T[cur][x], seen);
    if (tid == 0) sh.win_m1 = -1;
    __syncthreads();
    block_exclusive_scan(sh, L);
    const int nA = sh.ACC[L];
    const int f = (int)(W - count0);                       // appends left before the ring is full
    const int newest_pre = count0 > 0 ? (int)floor_mod_ll(start0 - 1, count0) : -1;
    auto slot_of_accept = [&](int a) -> int { return a < f ? (int)(count0 + a) : (int)((start0 + (a - f)) % W); };

    if (kData) {
        // group winners: the item of an accept, then competitors up to the next accept; ties -> later
        for (int x = tid; x < L; x += kThreads) {
            const int a = sh.ACC[x];
            if (sh.ACC[x + 1] != a) {
                int win = sh.ID[cur][x];
                float ws = item_score(u, lane, b, h, win);
                for (int y = x + 1; y < L && sh.ACC[y + 1] == sh.ACC[y]; ++y) {
                    const int c = sh.ID[cur][y];
                    const float cs = item_score(u, lane, b, h, c);
                    if (cs >= ws) {
                        win = c;
                        ws = cs;
                    }
                }
                sh.WIN[a] = win;
            }
        }
        // competitors arriving before the first accept challenge the pre-existing newest entry
        if (tid == 0 && L > 0 && sh.ACC[1] == 0 && newest_pre >= 0) {
            int win = -1;
            float ws = item_score(u, lane, b, h, u.K + i * W + newest_pre);
            for (int y = 0; y < L && sh.ACC[y + 1] == sh.ACC[y]; ++y) {
                const int c = sh.ID[cur][y];
                const float cs = item_score(u, lane, b, h, c);
                if (cs >= ws) {
                    win = c;
                    ws = cs;
                }
            }
            sh.win_m1 = win;
        }
        __syncthreads();
    }
    // popped entries form the next cascade's stream, in order
    const int nxt = cur ^ 1;
    const int n_pop = nA > f ? nA - f : 0;
    for (int x = tid; x < L; x += kThreads) {
        const int a = sh.ACC[x];
        if (sh.ACC[x + 1] != a && a >= f) {
            const int q = a - f;
            sh.T[nxt][q] = sh.T[cur][x];
            if (kData) {
                const int slot = (int)((start0 + q) % W);
                int occ;
                if (a - W >= 0) occ = sh.WIN[a - W];                       // written earlier in this chunk
                else if (slot == newest_pre && sh.win_m1 >= 0) occ = sh.win_m1;
                else occ = u.K + i * W + slot;                              // untouched pre-existing entry
                sh.ID[nxt][q] = occ;
            }
        }
    }
    if (kData) {
        // final (slot <- item) moves of this cascade: the last accept that maps to each slot
        int *plan = plan_lane + 2 * sh.casc_off[i];
        for (int x = tid; x < L; x += kThreads) {
            const int a = sh.ACC[x];
            if (sh.ACC[x + 1] != a && a + W >= nA) {
                const int e = atomicAdd(&sh.casc_cnt[i], 1);
                plan[2 * e] = i * W + slot_of_accept(a);
                plan[2 * e + 1] = sh.WIN[a];
            }
        }
        if (tid == 0 && sh.win_m1 >= 0 && nA < W) {
            const int e = atomicAdd(&sh.casc_cnt[i], 1);
            plan[2 * e] = i * W + newest_pre;
            plan[2 * e + 1] = sh.win_m1;
        }
    }
    __syncthreads();
    if (tid == 0) {
        long long c = count0 + nA;
        sh.count[i] = c < W ? c : W;
        sh.start[i] = (start0 + n_pop) % W;
        if (kData) sh.casc_off[i + 1] = sh.casc_off[i] + (L < W ? L : W) + 1;
    }
    __syncthreads();
    return n_pop;
}

__device__ void load_counters(const UpdateParams &u, Shared &sh) {
    for (int i = threadIdx.x; i < u.C; i += kThreads) {
        sh.count[i] = u.stored_tokens[i];
        sh.start[i] = u.start_indices[i];
        sh.every[i] = u.every_n[i];
        sh.casc_cnt[i] = 0;
        if (!CKV_COUNTERS_OK(sh.count[i], sh.start[i], u.W)) {     // debug build: report, then keep what follows in range
            sh.count[i] = sh.count[i] < 0 ? 0 : (sh.count[i] > u.W ? u.W : sh.count[i]);
            sh.start[i] = floor_mod_ll(sh.start[i], u.W);
        }
    }
    if (threadIdx.x == 0) sh.casc_off[0] = 0;
    __syncthreads();
}

// The moves of one cascade of one lane: 16-byte pieces of the rows, kUnroll of them in flight per
// thread (with few CTAs per lane the copy is bound by the latency of a dependent load-store pair).
// `first` / `step` spread the pieces over the participating threads.
__device__ __forceinline__ void execute_moves(const UpdateParams &u, int lane, const int *plan, int n, long long seen,
                                              int first, int step) {
    const int b = lane / u.KVH, h = lane % u.KVH;
    const int nchunk = u.row_bytes / 16;
    const long long row = u.row_bytes;
    uint8_t *ck = u.cache_k + (long long)lane * u.S * row;
    uint8_t *cv = u.cache_v + (long long)lane * u.S * row;
    uint8_t *cs = u.cache_s + (long long)lane * u.S * u.esz;
    long long *og = u.og_pos + (long long)lane * u.S;
    constexpr int kUnroll = 8;
    const int total = n * nchunk;
    for (int base = first; base < total; base += step * kUnroll) {
        uint4 rk[kUnroll], rv[kUnroll];
        int dsts[kUnroll], cs_[kUnroll];
#pragma unroll
        for (int r = 0; r < kUnroll; ++r) {
            const int idx = base + r * step;
            dsts[r] = -1;
            if (idx < total) {
                const int e = idx / nchunk, c = idx % nchunk;
                const int dst = plan[2 * e], id = plan[2 * e + 1];
                if (!CKV_IN_BOUNDS(dst >= 0 && dst < u.S && id >= 0 && id < u.K + u.S)) continue;
                const uint4 *sk, *sv;
                if (id < u.K) {
                    sk = reinterpret_cast<const uint4 *>(u.key + b * u.ksb + h * u.ksh + (long long)id * u.kst);
                    sv = reinterpret_cast<const uint4 *>(u.val + b * u.ksb + h * u.ksh + (long long)id * u.kst);
                } else {
                    sk = reinterpret_cast<const uint4 *>(ck + (long long)(id - u.K) * row);
                    sv = reinterpret_cast<const uint4 *>(cv + (long long)(id - u.K) * row);
                }
                rk[r] = sk[c];
                rv[r] = sv[c];
                dsts[r] = dst;
                cs_[r] = c;
                if (c == 0) {
                    unsigned int bits;
                    long long o;
                    if (id < u.K) {
                        bits = u.scr ? load_score_bits(u.scr + b * u.ssb + h * u.ssh + (long long)id * u.sst, u.esz) : 0u;
                        o = seen + id + 1;
                    } else {
                        bits = load_score_bits(cs + (long long)(id - u.K) * u.esz, u.esz);
                        o = og[id - u.K];
                    }
                    // a slot is the destination of at most one move of a stage, and a stage's sources
                    // lie in the chunk or in earlier cascades: nothing read in this stage is written in it
                    store_score_bits(cs + (long long)dst * u.esz, bits, u.esz);
                    og[dst] = o;
                }
            }
        }
#pragma unroll
        for (int r = 0; r < kUnroll; ++r) {
            if (dsts[r] >= 0) {
                reinterpret_cast<uint4 *>(ck + (long long)dsts[r] * row)[cs_[r]] = rk[r];
                reinterpret_cast<uint4 *>(cv + (long long)dsts[r] * row)[cs_[r]] = rv[r];
            }
        }
    }
}

template <bool kFused>
__global__ void __launch_bounds__(kThreads) update_chunk_kernel(ChunkParams p) {
    extern __shared__ uint8_t smem_raw[];
    Shared &sh = *reinterpret_cast<Shared *>(smem_raw);
    const UpdateParams &u = p.u;
    const int lane = blockIdx.x, tid = threadIdx.x;
    const int b = lane / u.KVH, h = lane % u.KVH;
    load_counters(u, sh);
    const long long seen = *u.seen;
    const long long sinks0 = *u.stored_sinks;
    const int ns_fill = (int)min((long long)u.K, max(0LL, (long long)u.NS - sinks0));
    const int nchunk = u.row_bytes / 16;
    const long long row = u.row_bytes;
    int *plan_lane = p.plan + (long long)lane * p.plan_stride * 2;

    // sink fill: the first ns_fill tokens of the chunk
    for (int idx = tid; idx < ns_fill * nchunk; idx += kThreads) {
        const int j = idx / nchunk, c = idx % nchunk;
        const uint4 *kin = reinterpret_cast<const uint4 *>(u.key + b * u.ksb + h * u.ksh + (long long)j * u.kst);
        const uint4 *vin = reinterpret_cast<const uint4 *>(u.val + b * u.ksb + h * u.ksh + (long long)j * u.kst);
        reinterpret_cast<uint4 *>(u.sink_k + ((long long)lane * u.NS + sinks0 + j) * row)[c] = kin[c];
        reinterpret_cast<uint4 *>(u.sink_v + ((long long)lane * u.NS + sinks0 + j) * row)[c] = vin[c];
    }
    int L = u.K - ns_fill;
    for (int x = tid; x < L; x += kThreads) {
        sh.T[0][x] = ns_fill + x;
        sh.ID[0][x] = ns_fill + x;
    }
    __syncthreads();
    int cur = 0, n_stage = 0;
    for (int i = 0; i < u.C && L > 0; ++i) {
        L = cascade_stage<true>(p, sh, lane, i, cur, L, seen, plan_lane);
        cur ^= 1;
        n_stage = i + 1;
    }
    __threadfence_block();
    __syncthreads();

    if constexpr (!kFused) {
        // long chunks: the moves run as one launch per cascade with many CTAs per lane
        int *hdr = p.hdr + (long long)lane * kHdrInts;
        if (tid < CKV_MAX_CASCADES) {
            hdr[2 * tid] = tid < n_stage ? sh.casc_off[tid] : 0;
            hdr[2 * tid + 1] = tid < n_stage ? sh.casc_cnt[tid] : 0;
        }
        if (tid == 0) hdr[2 * CKV_MAX_CASCADES] = n_stage;
    } else {
        // execute the moves from the last cascade to the first: sources are chunk rows or entries of
        // EARLIER cascades, which are still untouched when they are read
        for (int i = n_stage - 1; i >= 0; --i) {
            execute_moves(u, lane, plan_lane + 2 * sh.casc_off[i], sh.casc_cnt[i], seen, tid, kThreads);
            __syncthreads();
        }
    }
}

// Moves of cascade `stage` for every lane; launched from the last cascade to the first, so that the
// kernel boundary orders a cascade's reads of the previous cascade's entries before their rewrite.
__global__ void __launch_bounds__(kThreads) update_chunk_move_kernel(ChunkParams p, int stage) {
    const int lane = blockIdx.y;
    const int *hdr = p.hdr + (long long)lane * kHdrInts;
    if (stage >= hdr[2 * CKV_MAX_CASCADES]) return;
    const int *plan = p.plan + (long long)lane * p.plan_stride * 2 + 2 * hdr[2 * stage];
    execute_moves(p.u, lane, plan, hdr[2 * stage + 1], *p.u.seen, blockIdx.x * kThreads + threadIdx.x,
                  gridDim.x * kThreads);
}

// Advance the lane-invariant counters with the same stages (no data), then rewrite positions and
// masks from them (cascading_cache.py:729-774, :112-142).
__global__ void __launch_bounds__(kThreads) update_chunk_finalize_kernel(ChunkParams p) {
    extern __shared__ uint8_t smem_raw[];
    Shared &sh = *reinterpret_cast<Shared *>(smem_raw);
    __shared__ long long s_total, s_sinks, s_seen;
    const UpdateParams &u = p.u;
    const int tid = threadIdx.x;
    load_counters(u, sh);
    const long long seen = *u.seen;
    const long long sinks0 = *u.stored_sinks;
    const int ns_fill = (int)min((long long)u.K, max(0LL, (long long)u.NS - sinks0));
    int L = u.K - ns_fill;
    for (int x = tid; x < L; x += kThreads) sh.T[0][x] = ns_fill + x;
    __syncthreads();
    int cur = 0;
    for (int i = 0; i < u.C && L > 0; ++i) {
        L = cascade_stage<false>(p, sh, 0, i, cur, L, seen, nullptr);
        cur ^= 1;
    }
    if (tid == 0) {
        long long total = 0;
        for (int i = 0; i < u.C; ++i) {
            p.stored_tokens_w[i] = sh.count[i];
            p.start_indices_w[i] = sh.start[i];
            total += sh.count[i];
        }
        *p.stored_sinks_w = sinks0 + ns_fill;
        *p.seen_w = seen + u.K;
        s_total = total;
        s_sinks = sinks0 + ns_fill;
        s_seen = seen + u.K;
    }
    __syncthreads();
    for (int s = tid; s < u.NS; s += kThreads) {
        if (s < s_sinks) {
            p.sink_pos[s] = s;
            p.sink_mask[s] = 0;
        }
    }
    const bool rewrite = s_seen > u.NS;
    for (int t = tid; t < u.S; t += kThreads) {
        const int i = t / u.W, j = t % u.W;
        const long long stored_i = sh.count[i];
        if (j < stored_i) p.mask[t] = 0;
        const long long ub = s_total - (long long)i * u.W;
        const long long seg = stored_i < u.W ? stored_i : u.W;
        if (rewrite && ub > 0 && seg > 0) p.pos[t] = ((j + seg - sh.start[i]) % seg) + ub - seg;
    }
}

size_t up256c(size_t x) { return (x + 255) & ~(size_t)255; }

int plan_stride_for(const Dims &d, int k) {
    const int per = (k < d.W ? k : d.W) + 1;
    return d.C * per;
}

}  // namespace

size_t update_chunk_workspace_bytes(const Dims &d, int n_tokens) {
    const int k = n_tokens < kChunkMax ? n_tokens : kChunkMax;
    return up256c((size_t)d.B * d.KVH * plan_stride_for(d, k) * 2 * sizeof(int)) +
           up256c((size_t)d.B * d.KVH * kHdrInts * sizeof(int));
}

int launch_update_chunk(const Dims &d, const ckv_layer_state *st, const void *key, const void *value, int64_t ksb,
                        int64_t ksh, int64_t kst, const void *scores, int64_t ssb, int64_t ssh, int64_t sst,
                        int n_tokens, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    const int row_bytes = d.D * d.esz;
    if (row_bytes % 16 != 0) return fail(CKV_E_UNSUPPORTED, "row of %d bytes is not a multiple of 16", row_bytes);
    if (((uintptr_t)key | (uintptr_t)value) % 16 != 0 || (ksb * d.esz) % 16 || (ksh * d.esz) % 16 ||
        (kst * d.esz) % 16)
        return fail(CKV_E_ARG, "key/value rows must be 16-byte aligned");
    if (!workspace || workspace_bytes < update_chunk_workspace_bytes(d, n_tokens))
        return fail(CKV_E_WORKSPACE, "update workspace of %zu bytes, need %zu", workspace_bytes,
                    update_chunk_workspace_bytes(d, n_tokens));
    static bool attr_set[64] = {};
    if (first_use_on_this_device(attr_set)) {
        CKV_CUDA_CHECK(cudaFuncSetAttribute(update_chunk_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)sizeof(Shared)));
        CKV_CUDA_CHECK(cudaFuncSetAttribute(update_chunk_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)sizeof(Shared)));
        CKV_CUDA_CHECK(cudaFuncSetAttribute(update_chunk_finalize_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)sizeof(Shared)));
    }
    int launches = 0;
    for (int j0 = 0; j0 < n_tokens; j0 += kChunkMax) {
        const int k = n_tokens - j0 < kChunkMax ? n_tokens - j0 : kChunkMax;
        ChunkParams p;
        UpdateParams &u = p.u;
        u.key = (const uint8_t *)key + (long long)j0 * kst * d.esz;
        u.val = (const uint8_t *)value + (long long)j0 * kst * d.esz;
        u.ksb = ksb * d.esz; u.ksh = ksh * d.esz; u.kst = kst * d.esz;
        u.scr = scores ? (const uint8_t *)scores + (long long)j0 * sst * d.esz : nullptr;
        u.ssb = ssb * d.esz; u.ssh = ssh * d.esz; u.sst = sst * d.esz;
        u.sink_k = (uint8_t *)st->sink_keys; u.sink_v = (uint8_t *)st->sink_values;
        u.cache_k = (uint8_t *)st->key_cache; u.cache_v = (uint8_t *)st->value_cache;
        u.cache_s = (uint8_t *)st->score_cache;
        u.og_pos = (long long *)st->og_pos;
        u.stored_tokens = (const long long *)st->stored_tokens;
        u.start_indices = (const long long *)st->start_indices;
        u.stored_sinks = (const long long *)st->stored_sinks;
        u.seen = (const long long *)st->seen_tokens;
        u.every_n = (const long long *)st->every_n;
        u.KVH = d.KVH; u.K = k; u.NS = d.NS; u.W = d.W; u.C = d.C; u.S = d.S;
        u.row_bytes = row_bytes; u.esz = d.esz; u.dtype = d.dtype; u.eager_fill = d.eager_fill;
        p.plan = (int *)workspace;
        p.plan_stride = plan_stride_for(d, k);
        p.hdr = (int *)((uint8_t *)workspace + up256c((size_t)d.B * d.KVH * plan_stride_for(d, n_tokens < kChunkMax ? n_tokens : kChunkMax) * 2 * sizeof(int)));
        p.pos = (long long *)st->pos; p.sink_pos = (long long *)st->sink_pos;
        p.stored_tokens_w = (long long *)st->stored_tokens; p.start_indices_w = (long long *)st->start_indices;
        p.stored_sinks_w = (long long *)st->stored_sinks; p.seen_w = (long long *)st->seen_tokens;
        p.mask = st->mask; p.sink_mask = st->sink_mask;
        if (k >= kSplitMovesFrom) {
            update_chunk_kernel<false><<<d.B * d.KVH, kThreads, sizeof(Shared), stream>>>(p);
            for (int i = d.C - 1; i >= 0; --i)
                update_chunk_move_kernel<<<dim3(kMoveBlocks, d.B * d.KVH), kThreads, 0, stream>>>(p, i);
            launches += 1 + d.C;
        } else {
            update_chunk_kernel<true><<<d.B * d.KVH, kThreads, sizeof(Shared), stream>>>(p);
            launches += 1;
        }
        CKV_CUDA_CHECK(cudaGetLastError());
        update_chunk_finalize_kernel<<<1, kThreads, sizeof(Shared), stream>>>(p);
        CKV_CUDA_CHECK(cudaGetLastError());
        launches += 1;
    }
    note_launches(launches);
    return CKV_OK;
}

#ifdef CKV_BOUNDS
int read_bounds_status_chunk(int *out) { return read_bounds_status_of_this_unit(out); }
#endif

}  // namespace ckv
