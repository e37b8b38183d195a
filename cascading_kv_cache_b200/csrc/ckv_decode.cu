// Single-token decode over the cascading cache for 16-bit caches with head_dim 128.
//
// Kernel 0, rope_slots_kernel: cache positions do not depend on the lane, so the cos|sin row of every
//   slot is written once per step in slot order (an L2-resident image that TMA can stream).  Two
//   images alternate with the parity of the token count; the finish kernel of a step writes the image
//   of the NEXT step and tags it with the counters it is valid for, so that this kernel returns at
//   once when it finds the tag of its step (it writes the image itself after a prefill chunk, a
//   reset, or any other change of the counters behind the library's back).
//
// Kernel 1, decode_stream_kernel (HBM-bound, persistent, one CTA per SM):
//   The valid keys of all lanes form one flat stream of 64-key tiles; every CTA takes a
//   contiguous range of that stream (a split of the key dimension that ignores lane borders, so
//   all SMs stream the same number of bytes).  Two producer warps move each tile into shared memory
//   with TMA boxes (cp.async.bulk.tensor, 128-byte swizzle, mbarrier completion) through two rings:
//   K lo/hi and V lo/hi from the cache (L2 evict-first) through a 4-stage ring of 32 KB stages, the
//   cos / sin rows of the tile's slots from the image (L2 evict-last) through a 4-stage ring of
//   16 KB stages.  The rings are separate because their sources differ: the K/V bytes come from HBM
//   and need as many stages in flight as the memory latency asks for, the image sits in L2 and its
//   stage is released as soon as the keys are rotated.  Sixteen consumer warps in two groups take
//   alternate tiles; in a group, warp w owns keys [8w, 8w+8): ldmatrix of K and cos/sin fragments,
//   RoPE in packed 16-bit arithmetic on the fragments (the same rounding points as the reference:
//   cascade_attention.py:31-35, :284-291), QK^T on mma.sync m16n8k16 with the GQA group as the M
//   dimension, logits rounded to the cache dtype, online softmax per warp, and
//   out^T += V^T P^T on mma.sync m16n8k8 (dims as M).  At a lane border the warps merge their
//   (max, sum, out) in shared memory into one partial per (CTA, lane); under the EMA rule the
//   logits of every cached slot are also stored (the rounding point of the reference's einsum).
//
// Kernel 2, decode_finish_kernel: the blocks of a lane have roles.  Work blocks merge the partials with
//   the new token's own logit, write the output, turn logits into probabilities, reduce them over
//   the GQA group and apply score_cache = beta*score_cache + ema (cascade_attention.py:315-330);
//   the last of them to finish inserts the new token (the cascade update state machine).  Under the
//   stride rule the insert depends on nothing else and has a block of its own.  Image blocks rewrite
//   the lane-invariant positions / masks and the next step's cos|sin image.  The last block of the
//   whole grid advances the lane-invariant counters.  No host synchronisation anywhere.
#include <cuda.h>

#include "ckv_common.cuh"
#include "ckv_update_device.cuh"

namespace ckv {

namespace {

constexpr int kTile = 64;                       // keys per stage
// Both ring depths are powers of two on purpose: every consumer warp turns the tile index into a stage and
// a barrier phase once per tile, and with any other depth those are integer divisions in the hot loop
// (5 + 3 stages ran 4 % slower than 4 + 4 for that reason alone).
constexpr int kStages = 4;                      // K/V ring
constexpr int kStagesCS = 4;                    // cos/sin ring
static_assert((kStages & (kStages - 1)) == 0 && (kStagesCS & (kStagesCS - 1)) == 0, "ring depths: powers of two");
constexpr int kGroupWarps = 8;                  // warps per consumer group: each owns 8 keys of a tile
constexpr int kGroups = 2;                      // consumer groups working on alternate tiles
constexpr int kComputeWarps = kGroupWarps * kGroups;
constexpr int kStreamThreads = (kComputeWarps + 2) * 32;   // + the K/V producer warp + the cos/sin producer warp
constexpr int kSubBytes = kTile * 128;          // one swizzled 64-row x 128-byte sub-tile
constexpr int kStageBytes = 4 * kSubBytes;      // K lo | K hi | V lo | V hi
constexpr int kStageBytesCS = 2 * kSubBytes;    // cos | sin
constexpr int kOffK = 0, kOffV = 2 * kSubBytes, kOffCos = 0, kOffSin = kSubBytes;
constexpr int kRingBytes = kStages * kStageBytes + kStagesCS * kStageBytesCS;
constexpr int kMaxG = 16;
constexpr int kMergeBytes = (kMaxG * 128 + 2 * kComputeWarps * kMaxG) * 4;  // out[16][128] + m,l per warp
constexpr int kStreamSmem = kRingBytes + 1024 + 256 + kMergeBytes;
constexpr int kPartialStride = 130;             // m, l, out[128] per head row
constexpr unsigned kSpinLimit = 1u << 24;       // bounded mbarrier waits (each probe also sleeps)
constexpr int kFinishThreads = 256;
constexpr int kMaxHomogHeads = 64;              // query heads of one sequence reduced together (homogeneous_heads)
constexpr int kMaxParts = 160;                  // partials of one lane: at most one per stream CTA (one CTA per SM)

struct DecodeParams {
    const void *q;
    long long qsb, qsh;                          // elements
    const void *knew, *vnew;
    long long ksb, ksh;                          // elements
    void *out;
    long long osb, osh;
    const void *rope;
    long long rope_rows;
    const float *ema_w_cache;                    // [1]
    const void *ema_w_new;                       // [1]
    // state
    void *score_cache;
    long long *pos, *sink_pos, *stored_tokens, *start_indices, *stored_sinks, *seen;
    const long long *every_n;
    uint8_t *mask, *sink_mask;
    // scratch
    int *status;                                 // [0] error flag
    unsigned int *sync;                          // [0] lanes done, [1 + lane] blocks done
    void *logits;                                // [B*H][S]
    float *partials;                             // [(grid + lanes)][G][130]: one per (CTA, lane) segment
    void *new_scores;                            // [B*KVH]
    void *rope_slots;                            // 2 x [sink rows padded to 64 | S (+ a tile)][128]: cos|sin per slot
    long long image_bytes;                       // of one of the two images
    long long *image_tag;                        // 2 x 4 words: what each image is valid for
    int sink_rows_pad;
    int B, KVH, H, G, NS, W, C, S;
    int ema, update, head_reduction, eager_fill, dtype;
    int homog;                                   // reduce the scores over all query heads of a sequence
    float *head_stats;                           // homog: [B*H][4] = max, 1/sum, new-token probability of every head
    int stream_grid;
    int finish_chunks, finish_upd, finish_img;   // blocks of a lane in the finish kernel, by role
    float rs, beta_pow;
    UpdateParams upd;                            // the one-token cache update of the finish kernel
};

// ---------------------------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after kSpinLimit probes, raises the status flag and reports failure so
// that the caller leaves its loop instead of hanging the GPU.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, unsigned parity, int *status, unsigned limit = kSpinLimit) {
    for (unsigned n = 0; n < limit; ++n) {
        if (mbar_try_wait(bar, parity)) return true;
        if (n > 64) __nanosleep(64);
        if ((n & 1023) == 1023 && *((volatile int *)status) != 0) return false;
    }
    atomicExch(status, 1);
    return false;
}
// L2 policies: the key/value stream is read once (evict first), the cos/sin table is re-read by
// every lane (evict last).
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *tm, int x, int y, uint64_t *bar,
                                            uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(smem_u32(dst)), "l"(tm), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(policy) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

template <typename T> struct Mma;
template <> struct Mma<__nv_bfloat16> {
    static __device__ __forceinline__ void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};
template <> struct Mma<__half> {
    static __device__ __forceinline__ void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

template <typename T> struct MmaK8;
template <> struct MmaK8<__nv_bfloat16> {
    static __device__ __forceinline__ void run(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
        asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(b0));
    }
};
template <> struct MmaK8<__half> {
    static __device__ __forceinline__ void run(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
        asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(b0));
    }
};

// ---- packed 16-bit arithmetic with one rounding per operation ---------------------------------
template <typename T> struct Pack;
template <> struct Pack<__nv_bfloat16> {
    using T2 = __nv_bfloat162;
    static __device__ __forceinline__ T2 from_u(uint32_t u) { return *reinterpret_cast<T2 *>(&u); }
    static __device__ __forceinline__ uint32_t to_u(T2 v) { return *reinterpret_cast<uint32_t *>(&v); }
    static __device__ __forceinline__ float2 to_f2(T2 v) { return __bfloat1622float2(v); }
    static __device__ __forceinline__ T2 from_f2(float2 f) { return __float22bfloat162_rn(f); }
};
template <> struct Pack<__half> {
    using T2 = __half2;
    static __device__ __forceinline__ T2 from_u(uint32_t u) { return *reinterpret_cast<T2 *>(&u); }
    static __device__ __forceinline__ uint32_t to_u(T2 v) { return *reinterpret_cast<uint32_t *>(&v); }
    static __device__ __forceinline__ float2 to_f2(T2 v) { return __half22float2(v); }
    static __device__ __forceinline__ T2 from_f2(float2 f) { return __float22half2_rn(f); }
};

// (lo, hi) are the element pairs at dims d and d+64.  out = x*cos + rotate_half(x)*sin with each
// product and the sum rounded to T, then times sqrt(scale) in fp32 rounded to T.
template <typename T>
__device__ __forceinline__ void rope_pair(uint32_t &lo, uint32_t &hi, uint32_t c, uint32_t s, float rs) {
    using P = Pack<T>;
    const typename P::T2 l = P::from_u(lo), h = P::from_u(hi), cc = P::from_u(c), ss = P::from_u(s);
    const typename P::T2 nl = __hsub2_rn(__hmul2_rn(l, cc), __hmul2_rn(h, ss));  // _rn: never contracted into fma
    const typename P::T2 nh = __hadd2_rn(__hmul2_rn(h, cc), __hmul2_rn(l, ss));
    float2 fl = P::to_f2(nl), fh = P::to_f2(nh);
    fl.x *= rs; fl.y *= rs; fh.x *= rs; fh.y *= rs;
    lo = P::to_u(P::from_f2(fl));
    hi = P::to_u(P::from_f2(fh));
}

struct Schedule {
    long long seen, sinks, total, shift, max_pos;
    int n_sink_tiles, n_cache_tiles, tiles_per_lane;
    long long n_tiles;
};

__device__ __forceinline__ Schedule make_schedule(const DecodeParams &p) {
    Schedule s;
    s.seen = *p.seen;
    s.sinks = *p.stored_sinks;
    s.total = 0;
    for (int i = 0; i < p.C; ++i) s.total += p.stored_tokens[i];  // uniform loads: the values stay warp-uniform
    s.shift = s.seen > p.NS ? p.NS : 0;
    s.max_pos = s.seen == 0 ? 0 : (s.seen <= p.NS ? s.seen : p.NS + s.total);
    s.n_sink_tiles = (int)((s.sinks + kTile - 1) / kTile);
    s.n_cache_tiles = (int)((s.total + kTile - 1) / kTile);
    s.tiles_per_lane = s.n_sink_tiles + s.n_cache_tiles;
    s.n_tiles = (long long)s.tiles_per_lane * p.B * p.KVH;
    return s;
}

__device__ __forceinline__ long long cta_first_tile(long long cta, long long n_tiles, int grid) {
    return (cta * n_tiles) / grid;
}

// Self-test of the bounded wait: one thread waits, with a short limit, for a barrier phase that nothing will
// ever complete.  The wait must give up, raise the status word and return; the kernel then ends normally.
__global__ void decode_wait_selftest_kernel(int *status) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const bool arrived = mbar_wait(&bar, 0, status, 1u << 12);
        if (arrived) atomicExch(status, -1);     // cannot happen: nobody arrives on this barrier
    }
}

// ------------------------------------------------------------------------------ rope pre-pass
// Positions depend only on the slot, never on the lane: write the cos|sin row of every sink and
// cache slot once per step, in slot order, so that the stream kernel can fetch them with TMA.
// What an image depends on: the counters (hence every position), the table it was taken from, the geometry.
struct ImageTag {
    long long seen, counters, table, geometry;
};

__device__ __forceinline__ ImageTag make_image_tag(const DecodeParams &p, long long seen, long long sinks,
                                                   const long long *stored, const long long *start) {
    ImageTag t;
    t.seen = seen;
    long long h = sinks;
    for (int i = 0; i < p.C; ++i) h = h * 1000003LL + stored[i] * 65537LL + start[i];
    t.counters = h;
    // the table's address, its length, and a few of its values that differ from one RoPE base to another
    // (sines of row 1): a table of another base at a recycled address must not pass for this one
    t.table = (long long)(uintptr_t)p.rope ^ (p.rope_rows << 48) ^
              *reinterpret_cast<const long long *>(reinterpret_cast<const uint8_t *>(p.rope) + 256 + 128 + 32);
    t.geometry = ((long long)p.S << 32) ^ ((long long)p.NS << 16) ^ (long long)p.W ^ ((long long)p.dtype << 60);
    return t;
}

__device__ __forceinline__ uint4 *image_of(const DecodeParams &p, long long seen) {
    return reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(p.rope_slots) + (seen & 1) * p.image_bytes);
}

__global__ void __launch_bounds__(256) rope_slots_kernel(DecodeParams p) {
    const Schedule sc = make_schedule(p);
    if (blockIdx.x == 0 && threadIdx.x == 0) *p.status = 0;     // first kernel of the step: clear the status word
    {
        // the image of this step may already be there (written by the previous step's finish kernel).
        // One thread per block looks: every thread of a large grid reading the same four words would
        // queue up at one L2 bank for longer than the whole kernel otherwise takes.
        __shared__ int s_valid;
        if (threadIdx.x == 0) {
            const ImageTag want = make_image_tag(p, sc.seen, sc.sinks, p.stored_tokens, p.start_indices);
            const volatile long long *tag = p.image_tag + 4 * (sc.seen & 1);
            s_valid = tag[0] == want.seen && tag[1] == want.counters && tag[2] == want.table && tag[3] == want.geometry;
        }
        __syncthreads();
        if (s_valid) return;
    }
    // No block of this grid can see a matching tag from here on: the tag is only ever set by a finish
    // kernel, and the first block marks it invalid because the image now changes under it.
    if (blockIdx.x == 0 && threadIdx.x == 0) p.image_tag[4 * (sc.seen & 1)] = -1;
    const int n_rows = p.sink_rows_pad + p.S;
    const uint4 *rope = reinterpret_cast<const uint4 *>(p.rope);
    uint4 *dst = image_of(p, sc.seen);
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < (long long)n_rows * 16;
         idx += (long long)gridDim.x * blockDim.x) {
        const int row = (int)(idx >> 4), c = (int)(idx & 15);
        long long pos = 0;
        if (row < p.sink_rows_pad) {
            if (row < sc.sinks) pos = p.sink_pos[row];
        } else {
            const int slot = row - p.sink_rows_pad;
            if (slot < sc.total) pos = p.pos[slot] + sc.shift;
        }
        pos = pos < 0 ? 0 : (pos >= p.rope_rows ? p.rope_rows - 1 : pos);
        dst[idx] = rope[pos * 16 + c];
    }
}

// ------------------------------------------------------------------------------ stream kernel
template <typename T, int kRowHalves>
__global__ void __launch_bounds__(kStreamThreads, 1)
decode_stream_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                     const __grid_constant__ CUtensorMap tmSK, const __grid_constant__ CUtensorMap tmSV,
                     const __grid_constant__ CUtensorMap tmR0, const __grid_constant__ CUtensorMap tmR1,
                     DecodeParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *smem_cs = smem + kStages * kStageBytes;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + kRingBytes);
    uint64_t *empty = full + kStages;
    uint64_t *full_cs = empty + kStages;
    uint64_t *empty_cs = full_cs + kStagesCS;
    const int warp = threadIdx.x >> 5, lane_id = threadIdx.x & 31;
    const Schedule sc = make_schedule(p);
    const long long t_begin = cta_first_tile(blockIdx.x, sc.n_tiles, gridDim.x);
    const long long t_end = cta_first_tile(blockIdx.x + 1, sc.n_tiles, gridDim.x);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);    // the producer's expect_tx arrival; TMA completes the bytes
            mbar_init(&empty[s], kGroupWarps);
        }
        for (int s = 0; s < kStagesCS; ++s) {
            mbar_init(&full_cs[s], 1);
            mbar_init(&empty_cs[s], kGroupWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (blockIdx.x == 0) {
        const int n = 1 + p.B * p.KVH;
        for (int i = threadIdx.x; i < n; i += blockDim.x) p.sync[i] = 0;
    }
    __syncthreads();

    if (warp == kComputeWarps) {
        // ------------------------------------------------------------------ K/V producer warp
        // one elected lane issues four TMA boxes per tile: K lo/hi, V lo/hi
        const uint64_t pol_stream = l2_policy_evict_first();
        int lane = (int)(t_begin / sc.tiles_per_lane), ti = (int)(t_begin % sc.tiles_per_lane);
        const int n_it = (int)(t_end - t_begin);
        for (int it = 0; it < n_it; ++it) {
            const int s = it % kStages;
            const bool sink_tile = ti < sc.n_sink_tiles;
            const int row0 = sink_tile ? ti * kTile : (ti - sc.n_sink_tiles) * kTile;
            if (it >= kStages) {
                if (!mbar_wait(&empty[s], ((it / kStages) & 1) ^ 1, p.status)) break;
            }
            uint8_t *stage = smem + s * kStageBytes;
            if (lane_id == 0) {
                mbar_expect_tx(&full[s], 4 * kSubBytes);
                const int y = sink_tile ? lane * p.NS + row0 : lane * p.S + row0;
                const CUtensorMap *mk = sink_tile ? &tmSK : &tmK;
                const CUtensorMap *mv = sink_tile ? &tmSV : &tmV;
                tma_load_2d(stage + kOffK, mk, 0, y, &full[s], pol_stream);
                tma_load_2d(stage + kOffK + kSubBytes, mk, 64, y, &full[s], pol_stream);
                tma_load_2d(stage + kOffV, mv, 0, y, &full[s], pol_stream);
                tma_load_2d(stage + kOffV + kSubBytes, mv, 64, y, &full[s], pol_stream);
            }
            __syncwarp();
            if (++ti == sc.tiles_per_lane) {
                ti = 0;
                ++lane;
            }
        }
    } else if (warp == kComputeWarps + 1) {
        // ------------------------------------------------------------------ cos/sin producer warp
        // the cos / sin rows of each tile's slots from the slot-ordered image the pre-pass wrote
        const uint64_t pol_keep = l2_policy_evict_last();
        const CUtensorMap *tmR = (sc.seen & 1) ? &tmR1 : &tmR0;      // the image of this step
        int ti = (int)(t_begin % sc.tiles_per_lane);
        const int n_it = (int)(t_end - t_begin);
        for (int it = 0; it < n_it; ++it) {
            const int s = it % kStagesCS;
            const bool sink_tile = ti < sc.n_sink_tiles;
            const int row0 = sink_tile ? ti * kTile : (ti - sc.n_sink_tiles) * kTile;
            if (it >= kStagesCS) {
                if (!mbar_wait(&empty_cs[s], ((it / kStagesCS) & 1) ^ 1, p.status)) break;
            }
            uint8_t *stage = smem_cs + s * kStageBytesCS;
            if (lane_id == 0) {
                mbar_expect_tx(&full_cs[s], 2 * kSubBytes);
                const int yr = sink_tile ? row0 : p.sink_rows_pad + row0;
                tma_load_2d(stage + kOffCos, tmR, 0, yr, &full_cs[s], pol_keep);
                tma_load_2d(stage + kOffSin, tmR, 64, yr, &full_cs[s], pol_keep);
            }
            __syncwarp();
            if (++ti == sc.tiles_per_lane) ti = 0;
        }
    } else {
        // ----------------------------------------------------------------- consumer warps
        // Two groups of eight warps take alternate tiles; inside a group warp wk owns keys
        // [8 wk, 8 wk + 8) of the tile.  Every warp walks all iterations so that lane changes (and
        // the block-wide merge they trigger) are seen by all warps alike.
        const int g = lane_id >> 2, tq = lane_id & 3;
        const int group = warp / kGroupWarps, wk = warp % kGroupWarps;
        const T *rope = reinterpret_cast<const T *>(p.rope);
        uint32_t qa[8][4];
        float ot[kRowHalves][8][4];   // out^T: [dims 16 mt + g (+8)][heads 8 nh + 2 tq (+1)]
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
        int cur_lane = -1;
        T *lrow[2] = {nullptr, nullptr};

        float *mg_out = reinterpret_cast<float *>(smem + kRingBytes + 256);              // [kMaxG][128]
        float *mg_m = mg_out + kMaxG * 128;                                              // [warps][kMaxG]
        float *mg_l = mg_m + kComputeWarps * kMaxG;
        const int ctid = threadIdx.x;  // consumer threads are 0 .. kComputeWarps*32 - 1
        auto consumer_sync = [&]() { asm volatile("bar.sync 1, %0;" ::"n"(kComputeWarps * 32) : "memory"); };

        // loop-invariant shared-memory offsets of this thread's ldmatrix rows
        const int krow = 8 * wk + (lane_id & 7);
        const uint32_t rowoff = krow * 128;
        const int sw = krow & 7;
        uint32_t choff[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) choff[u] = rowoff + (uint32_t)(((4 * u + (lane_id >> 3)) ^ sw) << 4);

        // Merge all warps' (max, sum, out) of one (CTA, lane) segment in shared memory and write a
        // single partial.  Runs once per segment, i.e. every few hundred tiles.
        auto flush = [&](int lane) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
                l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
            }
            for (int i = ctid; i < kMaxG * 128; i += kComputeWarps * 32) mg_out[i] = 0.f;
            if (tq == 0) {
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    mg_m[warp * kMaxG + g + 8 * r] = m_run[r];
                    mg_l[warp * kMaxG + g + 8 * r] = l_run[r];
                }
            }
            consumer_sync();
#pragma unroll
            for (int nh = 0; nh < kRowHalves; ++nh) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int head = 8 * nh + 2 * tq + e;
                    if (head < p.G) {
                        float mx = -INFINITY;
                        for (int w = 0; w < kComputeWarps; ++w) mx = fmaxf(mx, mg_m[w * kMaxG + head]);
                        const float mine = mg_m[warp * kMaxG + head];
                        const float sc_w = (mine == -INFINITY) ? 0.f : __expf(mine - mx);
#pragma unroll
                        for (int mt = 0; mt < 8; ++mt) {
                            atomicAdd(&mg_out[head * 128 + 16 * mt + g], ot[nh][mt][e] * sc_w);
                            atomicAdd(&mg_out[head * 128 + 16 * mt + g + 8], ot[nh][mt][2 + e] * sc_w);
                        }
                    }
                }
            }
            consumer_sync();
            float *base = p.partials + (long long)(blockIdx.x + lane) * p.G * kPartialStride;
            for (int i = ctid; i < p.G * 128; i += kComputeWarps * 32)
                base[(i >> 7) * kPartialStride + 2 + (i & 127)] = mg_out[i];
            if (ctid < p.G) {
                float mx = -INFINITY, l = 0.f;
                for (int w = 0; w < kComputeWarps; ++w) mx = fmaxf(mx, mg_m[w * kMaxG + ctid]);
                for (int w = 0; w < kComputeWarps; ++w) {
                    const float mw = mg_m[w * kMaxG + ctid];
                    if (mw != -INFINITY) l += mg_l[w * kMaxG + ctid] * __expf(mw - mx);
                }
                base[ctid * kPartialStride] = mx;
                base[ctid * kPartialStride + 1] = l;
            }
            consumer_sync();
        };

        int lane = (int)(t_begin / sc.tiles_per_lane), ti = (int)(t_begin % sc.tiles_per_lane);
        const int n_it = (int)(t_end - t_begin);
        bool failed = false;
        for (int it = 0; it < n_it; ++it) {
            const int s = it % kStages, scs = it % kStagesCS;
            if (lane != cur_lane) {
                if (cur_lane >= 0) flush(cur_lane);
                cur_lane = lane;
                m_run[0] = m_run[1] = -INFINITY;
                l_run[0] = l_run[1] = 0.f;
#pragma unroll
                for (int nh = 0; nh < kRowHalves; ++nh)
#pragma unroll
                    for (int mt = 0; mt < 8; ++mt) ot[nh][mt][0] = ot[nh][mt][1] = ot[nh][mt][2] = ot[nh][mt][3] = 0.f;
                // A fragments of q (rows = heads of the group), rotated at max_pos and scaled
                const int b = lane / p.KVH, kvh = lane % p.KVH;
                const T *crow = rope + (sc.max_pos < p.rope_rows ? sc.max_pos : p.rope_rows - 1) * 128;
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const int row = g + 8 * r;
                    lrow[r] = reinterpret_cast<T *>(p.logits) + ((long long)b * p.H + kvh * p.G + row) * p.S;
                    if (r < kRowHalves && row < p.G) {
                        const T *qrow = reinterpret_cast<const T *>(p.q) + b * p.qsb + (long long)(kvh * p.G + row) * p.qsh;
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
                            for (int hf = 0; hf < 2; ++hf) {
                                const int d = 16 * ks + 8 * hf + 2 * tq;
                                uint32_t lo = *reinterpret_cast<const uint32_t *>(qrow + d);
                                uint32_t hi = *reinterpret_cast<const uint32_t *>(qrow + d + 64);
                                const uint32_t c = *reinterpret_cast<const uint32_t *>(crow + d);
                                const uint32_t sn = *reinterpret_cast<const uint32_t *>(crow + 64 + d);
                                rope_pair<T>(lo, hi, c, sn, p.rs);
                                qa[ks][r + 2 * hf] = lo;
                                qa[ks + 4][r + 2 * hf] = hi;
                            }
                        }
                    } else {
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks) qa[ks][r] = qa[ks][r + 2] = 0u;
                    }
                }
            }
            if ((it & (kGroups - 1)) == group) {
                if (!mbar_wait(&full[s], (it / kStages) & 1, p.status) ||
                    !mbar_wait(&full_cs[scs], (it / kStagesCS) & 1, p.status)) {
                    failed = true;
                    break;
                }
                const bool sink_tile = ti < sc.n_sink_tiles;
                const int row0 = sink_tile ? ti * kTile : (ti - sc.n_sink_tiles) * kTile;
                const long long limit = sink_tile ? sc.sinks : sc.total;
                const int nvalid = (int)(limit - row0 < kTile ? limit - row0 : kTile);
                const int key0 = 8 * wk;
                if (key0 < nvalid) {
                    const uint32_t stage = smem_u32(smem + s * kStageBytes);
                    const uint32_t stage_cs = smem_u32(smem_cs + scs * kStageBytesCS);
                    float sacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        // k-steps 2u, 2u+1 (dims < 64) with their partners 2u+4, 2u+5 (dims + 64)
                        uint32_t kl[4], kh[4], cs[4], sn[4];
                        ldsm_x4(stage + kOffK + choff[u], kl[0], kl[1], kl[2], kl[3]);
                        ldsm_x4(stage + kOffK + kSubBytes + choff[u], kh[0], kh[1], kh[2], kh[3]);
                        ldsm_x4(stage_cs + kOffCos + choff[u], cs[0], cs[1], cs[2], cs[3]);
                        ldsm_x4(stage_cs + kOffSin + choff[u], sn[0], sn[1], sn[2], sn[3]);
#pragma unroll
                        for (int e = 0; e < 4; ++e) rope_pair<T>(kl[e], kh[e], cs[e], sn[e], p.rs);
                        Mma<T>::run(sacc, qa[2 * u], kl[0], kl[1]);
                        Mma<T>::run(sacc, qa[2 * u + 1], kl[2], kl[3]);
                        Mma<T>::run(sacc, qa[2 * u + 4], kh[0], kh[1]);
                        Mma<T>::run(sacc, qa[2 * u + 5], kh[2], kh[3]);
                    }
                    // the keys are rotated: hand the cos/sin stage back before the softmax and the P V product
                    __syncwarp();
                    if (lane_id == 0) mbar_arrive(&empty_cs[scs]);
                    // logits rounded to T (the reference's einsum output), masked past the valid keys
                    const int kk = key0 + 2 * tq;
#pragma unroll
                    for (int e = 0; e < 2 * kRowHalves; ++e) sacc[e] = (kk + (e & 1)) < nvalid ? rnd<T>(sacc[e]) : -INFINITY;
                    if (p.ema && !sink_tile) {
                        const int slot = row0 + kk;
#pragma unroll
                        for (int r = 0; r < kRowHalves; ++r) {
                            if (g + 8 * r < p.G) {
                                if (slot + 1 < p.S) {
                                    typename Pack<T>::T2 v = Pack<T>::from_f2(make_float2(sacc[2 * r], sacc[2 * r + 1]));
                                    *reinterpret_cast<typename Pack<T>::T2 *>(lrow[r] + slot) = v;
                                } else if (slot < p.S) {
                                    lrow[r][slot] = Elem<T>::from_f(sacc[2 * r]);
                                }
                            }
                        }
                    }
                    // online softmax over this warp's 8 keys; P^T (keys x heads) is the B operand of PV
                    uint32_t pb[kRowHalves];
                    float corr[kRowHalves];
                    bool rescale = false;
#pragma unroll
                    for (int r = 0; r < kRowHalves; ++r) {
                        float mx = fmaxf(sacc[2 * r], sacc[2 * r + 1]);
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                        const float m_new = fmaxf(m_run[r], mx);
                        float p0 = 0.f, p1 = 0.f;
                        corr[r] = 1.f;
                        if (m_new != -INFINITY) {
                            corr[r] = __expf(m_run[r] - m_new);
                            p0 = __expf(sacc[2 * r] - m_new);
                            p1 = __expf(sacc[2 * r + 1] - m_new);
                        }
                        m_run[r] = m_new;
                        l_run[r] = l_run[r] * corr[r] + (p0 + p1);
                        rescale |= corr[r] != 1.f;
                        pb[r] = Pack<T>::to_u(Pack<T>::from_f2(make_float2(p0, p1)));
                    }
                    if (__any_sync(0xffffffffu, rescale)) {  // the running max rarely moves
#pragma unroll
                        for (int nh = 0; nh < kRowHalves; ++nh) {
                            // this thread's out^T columns are heads 8 nh + 2 tq (+1); their factors sit in
                            // the lanes whose row g is that head
                            const float ca = __shfl_sync(0xffffffffu, corr[nh], (2 * tq) * 4);
                            const float cb = __shfl_sync(0xffffffffu, corr[nh], (2 * tq + 1) * 4);
#pragma unroll
                            for (int mt = 0; mt < 8; ++mt) {
                                ot[nh][mt][0] *= ca;
                                ot[nh][mt][1] *= cb;
                                ot[nh][mt][2] *= ca;
                                ot[nh][mt][3] *= cb;
                            }
                        }
                    }
                    // out^T (128 dims x heads) += V^T (128 x 8 keys) * P^T (8 keys x heads)
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
#pragma unroll
                        for (int cq = 0; cq < 2; ++cq) {
                            uint32_t v0, v1, v2, v3;
                            ldsm_x4_t(stage + kOffV + half * kSubBytes + choff[cq], v0, v1, v2, v3);
#pragma unroll
                            for (int nh = 0; nh < kRowHalves; ++nh) {
                                MmaK8<T>::run(ot[nh][4 * half + 2 * cq], v0, v1, pb[nh]);
                                MmaK8<T>::run(ot[nh][4 * half + 2 * cq + 1], v2, v3, pb[nh]);
                            }
                        }
                    }
                }
                else if (lane_id == 0) mbar_arrive(&empty_cs[scs]);   // a warp without valid keys in this tile
                __syncwarp();
                if (lane_id == 0) mbar_arrive(&empty[s]);
            }
            if (++ti == sc.tiles_per_lane) {
                ti = 0;
                ++lane;
            }
        }
        // a failed wait already raised the status flag; the warps then leave without the block-wide
        // merge (its barrier could otherwise wait for warps that left through another path)
        if (cur_lane >= 0 && !failed && *((volatile int *)p.status) == 0) flush(cur_lane);
    }
}

// ------------------------------------------------------------------------------ finish kernel
__device__ __forceinline__ float reduce_group(const float *v, int n, int how) {
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
    const int want = (n - 1) / 2;  // lower median
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

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// EMA pass over the cached slots of one lane, eight slots per thread and iteration:
//   p = T(exp(logit - m) / l),  e = T(p * (1-beta)),  red = max or mean over the group,
//   score = T(T(beta * score) + red)                       (cascade_attention.py:315-330)
// exp(x - m) / l is evaluated as exp2(x*log2e + c) with c = -m*log2e - log2(l).
template <typename T, bool kMax>
__device__ __forceinline__ void ema_pass_vec(const DecodeParams &p, const Schedule &sc, const T *lg, T *scr,
                                             const float *s_m, const float *s_linv, float w0, int tid) {
    using P = Pack<T>;
    constexpr float kLog2e = 1.4426950408889634f;
    const int nvec = p.S / 8;
    const int per_block = (nvec + p.finish_chunks - 1) / p.finish_chunks;
    const int v_end = min(nvec, (int)(blockIdx.x + 1) * per_block);
    float cg[8];
#pragma unroll
    for (int gh = 0; gh < 8; ++gh) cg[gh] = gh < p.G ? -s_m[gh] * kLog2e + __log2f(s_linv[gh]) : 0.f;
    const float inv_g = 1.f / (float)p.G;
    for (int v = blockIdx.x * per_block + tid; v < v_end; v += kFinishThreads) {
        const int slot0 = v * 8;
        uint4 sc4 = *reinterpret_cast<const uint4 *>(scr + slot0);
        uint4 l4[8];
        const bool any_valid = slot0 < sc.total;
        if (any_valid) {
#pragma unroll
            for (int gh = 0; gh < 8; ++gh)
                if (gh < p.G) l4[gh] = *reinterpret_cast<const uint4 *>(lg + (long long)gh * p.S + slot0);
        }
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = kMax ? -INFINITY : 0.f;
        if (any_valid) {
            if (kMax) {
                // max over the group: every step from the exponent to the weighted, rounded probability is
                // monotone (exp2, the two roundings, the product with the positive weight), so the largest
                // exponent of the group gives the group's largest value -- one exponential per slot
#pragma unroll
                for (int gh = 0; gh < 8; ++gh) {
                    if (gh < p.G) {
                        const uint32_t *lw = reinterpret_cast<const uint32_t *>(&l4[gh]);
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) {
                            const float2 l = P::to_f2(P::from_u(lw[jj]));
                            acc[2 * jj] = fmaxf(acc[2 * jj], fmaf(l.x, kLog2e, cg[gh]));
                            acc[2 * jj + 1] = fmaxf(acc[2 * jj + 1], fmaf(l.y, kLog2e, cg[gh]));
                        }
                    }
                }
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const float2 pr = P::to_f2(P::from_f2(make_float2(ex2_approx(acc[2 * jj]), ex2_approx(acc[2 * jj + 1]))));
                    const float2 e = P::to_f2(P::from_f2(make_float2(__fmul_rn(pr.x, w0), __fmul_rn(pr.y, w0))));
                    acc[2 * jj] = e.x;
                    acc[2 * jj + 1] = e.y;
                }
            } else {
#pragma unroll
                for (int gh = 0; gh < 8; ++gh) {
                    if (gh < p.G) {
                        const uint32_t *lw = reinterpret_cast<const uint32_t *>(&l4[gh]);
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) {
                            const float2 l = P::to_f2(P::from_u(lw[jj]));
                            const float2 pr = P::to_f2(P::from_f2(make_float2(ex2_approx(fmaf(l.x, kLog2e, cg[gh])),
                                                                              ex2_approx(fmaf(l.y, kLog2e, cg[gh])))));
                            const float2 e = P::to_f2(P::from_f2(make_float2(__fmul_rn(pr.x, w0), __fmul_rn(pr.y, w0))));
                            acc[2 * jj] += e.x;
                            acc[2 * jj + 1] += e.y;
                        }
                    }
                }
            }
        }
        uint32_t *sw = reinterpret_cast<uint32_t *>(&sc4);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            float2 red = make_float2(0.f, 0.f);
            if (slot0 + 2 * jj < sc.total) red.x = kMax ? acc[2 * jj] : acc[2 * jj] * inv_g;
            if (slot0 + 2 * jj + 1 < sc.total) red.y = kMax ? acc[2 * jj + 1] : acc[2 * jj + 1] * inv_g;
            red = P::to_f2(P::from_f2(red));
            const float2 old = P::to_f2(P::from_u(sw[jj]));
            const float2 dec = P::to_f2(P::from_f2(make_float2(__fmul_rn(old.x, p.beta_pow), __fmul_rn(old.y, p.beta_pow))));
            sw[jj] = P::to_u(P::from_f2(make_float2(__fadd_rn(dec.x, red.x), __fadd_rn(dec.y, red.y))));
        }
        *reinterpret_cast<uint4 *>(scr + slot0) = sc4;
    }
}

// kStatsOnly: a first, small launch of the same kernel under homogeneous_heads -- every lane leaves (max, 1/sum,
// new-token probability) of its heads in p.head_stats and returns, so that the real launch can reduce the scores
// of a slot over ALL heads of the sequence (cascade_attention.py:240-242), not only over its own KV group.
template <typename T, bool kStatsOnly>
__global__ void __launch_bounds__(kFinishThreads, 3) decode_finish_kernel(DecodeParams p) {
    __shared__ float s_m[kMaxG], s_linv[kMaxG], s_snew[kMaxG], s_pnew[kMaxG];
    __shared__ float s_hcg[kMaxHomogHeads], s_hpnew[kMaxHomogHeads];
    __shared__ int s_part[kMaxParts];
    __shared__ float s_w[kMaxG * kMaxParts];
    __shared__ long long s_stored[CKV_MAX_CASCADES], s_start[CKV_MAX_CASCADES], s_every[CKV_MAX_CASCADES];
    __shared__ long long s_new_stored[CKV_MAX_CASCADES], s_new_start[CKV_MAX_CASCADES];
    __shared__ long long s_new_sinks, s_new_total, s_tag[4];
    __shared__ int s_image_there;
    __shared__ int s_next_pos[kFinishThreads];
    __shared__ int s_is_last;
    const int lane = blockIdx.y;
    const int b = lane / p.KVH, kvh = lane % p.KVH;
    const int tid = threadIdx.x, warp = tid >> 5, lane_id = tid & 31;
    const Schedule sc = make_schedule(p);
    const T *rope = reinterpret_cast<const T *>(p.rope);
    const T *crow = rope + (sc.max_pos < p.rope_rows ? sc.max_pos : p.rope_rows - 1) * 128;
    const T *krow = reinterpret_cast<const T *>(p.knew) + b * p.ksb + kvh * p.ksh;
    const T *vrow = reinterpret_cast<const T *>(p.vnew) + b * p.ksb + kvh * p.ksh;

    // Blocks of a lane by role (blockIdx.x): [0, finish_chunks) merge the partials, write the output rows and run
    // the EMA pass; under the stride rule one further block inserts the token (nothing it touches depends on the
    // others); the last finish_img blocks rewrite the lane-invariant positions / masks and the next step's cos|sin
    // image.  Nothing on one role's path waits for another role: they meet only in the count that elects the
    // block which publishes the advanced counters.
    const int upd_base = p.finish_chunks, img_base = p.finish_chunks + p.finish_upd;
    const bool work_block = (int)blockIdx.x < upd_base;

    // the counters after this token: needed by whoever inserts the token (the old ones) and by whoever turns out
    // to publish (the new ones).  One warp fetches and advances them: in a work block a warp that has no head to
    // merge, while the others merge, so the fetch adds nothing to the block's critical path.
    auto counters_by_warp = [&]() {
        for (int i = lane_id; i < p.C; i += 32) {
            s_stored[i] = s_new_stored[i] = p.stored_tokens[i];
            s_start[i] = s_new_start[i] = p.start_indices[i];
            s_every[i] = p.every_n[i];
        }
        __syncwarp();
        if (lane_id == 0) {
            long long sinks = sc.sinks;
            advance_counters(s_new_stored, s_new_start, sinks, sc.seen, s_every, 1, p.NS, p.W, p.C, p.S, p.eager_fill);
            long long total = 0;
            for (int i = 0; i < p.C; ++i) total += s_new_stored[i];
            for (int i = 0; i < p.C; ++i)
                if (!CKV_COUNTERS_OK(s_new_stored[i], s_new_start[i], p.W)) s_new_stored[i] = s_new_start[i] = 0;
            s_new_sinks = sinks;
            s_new_total = total;
            const ImageTag t = make_image_tag(p, sc.seen + 1, sinks, s_new_stored, s_new_start);
            s_tag[0] = t.seen; s_tag[1] = t.counters; s_tag[2] = t.table; s_tag[3] = t.geometry;
            const volatile long long *tag = p.image_tag + 4 * ((sc.seen + 1) & 1);
            s_image_there = tag[0] == t.seen && tag[1] == t.counters && tag[2] == t.table && tag[3] == t.geometry;
        }
    };
    auto arrive_and_publish = [&]() {
        // every block that changed state counts itself once its writes are fenced; the last one of the grid
        // publishes the new counters
        __threadfence();
        __syncthreads();
        if (warp != 0) return;
        unsigned last = 0;
        const unsigned expected = gridDim.y * (unsigned)(p.finish_img + p.finish_upd + (p.ema ? 1 : p.finish_chunks));
        if (lane_id == 0) last = (atomicAdd(&p.sync[0], 1u) == expected - 1);
        last = __shfl_sync(0xffffffffu, last, 0);
        if (!last) return;
        __threadfence();
        // every lane has read the old counters and finished its insert: publish the new ones
        for (int i = lane_id; i < p.C; i += 32) {
            p.stored_tokens[i] = s_new_stored[i];
            p.start_indices[i] = s_new_start[i];
        }
        if (lane_id == 0) {
            if (s_new_sinks > sc.sinks) {
                p.sink_pos[sc.sinks] = sc.sinks;
                p.sink_mask[sc.sinks] = 0;
            }
            *p.stored_sinks = s_new_sinks;
            *p.seen = sc.seen + 1;
            // every image block has written its share of the next step's image (their fences precede the
            // count that elected this thread): say what it is valid for
            long long *tag = p.image_tag + 4 * ((sc.seen + 1) & 1);
            tag[1] = s_tag[1]; tag[2] = s_tag[2]; tag[3] = s_tag[3];
            __threadfence();
            tag[0] = s_tag[0];
        }
    };

    if (!kStatsOnly && p.update && !work_block) {
        if (warp == 0) counters_by_warp();
        __syncthreads();
    }
    if (!kStatsOnly && p.update && (int)blockIdx.x >= img_base) {
        // ---- image blocks: positions / masks from the advanced counters, every image block of the grid taking
        //      an equal share of the slots (nothing in this kernel reads them)
        {
            const int n_blocks = gridDim.y * p.finish_img, me = lane * p.finish_img + ((int)blockIdx.x - img_base);
            const int per_block = (p.S + n_blocks - 1) / n_blocks;
            const int s_begin = me * per_block, s_end = min(p.S, s_begin + per_block);
            const bool rewrite = sc.seen + 1 > p.NS;
            for (int t = s_begin + tid; t < s_end; t += kFinishThreads) {
                const int i = t / p.W, j = t % p.W;
                const int stored_i = (int)s_new_stored[i];                  // counters are at most W
                if (j < stored_i) p.mask[t] = 0;
                const long long ub = s_new_total - (long long)i * p.W;
                const int seg = stored_i < p.W ? stored_i : p.W;
                if (rewrite && ub > 0 && seg > 0) p.pos[t] = (long long)((j + seg - (int)s_new_start[i]) % seg) + ub - seg;
            }
            // the cos|sin image of the NEXT step (positions after this token), unless an earlier call of this
            // step -- another layer sharing the workspace -- has written it already.  256 slots at a time: a
            // thread works out one slot's next position, then the block copies the 256 table rows with 16
            // independent 16-byte loads per thread.
            if (!s_image_there) {
                const long long seen_next = sc.seen + 1;
                const long long shift = seen_next > p.NS ? p.NS : 0;
                const uint4 *rope = reinterpret_cast<const uint4 *>(p.rope);
                uint4 *img = image_of(p, seen_next) + (long long)p.sink_rows_pad * 16;
                for (int base = s_begin; base < s_end; base += kFinishThreads) {
                    const int t = base + tid;
                    long long pos = 0;
                    if (t < s_end && t < s_new_total) {
                        pos = p.pos[t];
                        if (rewrite) {
                            const int i = t / p.W, j = t % p.W;
                            const int stored_i = (int)s_new_stored[i];
                            const long long ub = s_new_total - (long long)i * p.W;
                            const int seg = stored_i < p.W ? stored_i : p.W;
                            if (seg > 0 && ub > 0) pos = (long long)((j + seg - (int)s_new_start[i]) % seg) + ub - seg;
                        }
                        pos += shift;
                    }
                    s_next_pos[tid] = (int)(pos < 0 ? 0 : (pos >= p.rope_rows ? p.rope_rows - 1 : pos));
                    __syncthreads();
                    const int n_here = min(kFinishThreads, s_end - base);
#pragma unroll
                    for (int r = 0; r < 16; ++r) {
                        const int idx = r * kFinishThreads + tid, slot = idx >> 4, c = idx & 15;
                        if (slot < n_here) img[(long long)(base + slot) * 16 + c] = rope[(long long)s_next_pos[slot] * 16 + c];
                    }
                    __syncthreads();
                }
                if (me == 0) {      // the sink rows: sink i sits at position i
                    uint4 *simg = image_of(p, seen_next);
                    for (int idx = tid; idx < p.sink_rows_pad * 16; idx += kFinishThreads) {
                        const int row = idx >> 4, c = idx & 15;
                        const long long pos = row < s_new_sinks ? row : 0;
                        simg[idx] = rope[pos * 16 + c];
                    }
                }
            }
        }
        arrive_and_publish();
        return;
    }
    if (!kStatsOnly && p.update && p.finish_upd && (int)blockIdx.x == upd_base) {
        // ---- stride rule: the token goes in at once
        if (warp == 0) {
            if (p.C <= kOneTokenMaxCascades) update_lane_one_token(p.upd, lane, s_stored, s_start, s_every, sc.sinks, sc.seen, 0u);
            else update_lane_walk(p.upd, lane, s_stored, s_start, s_every);
        }
        arrive_and_publish();
        return;
    }
    if (!work_block) return;

    // 1. which of the stream kernel's partials belong to this lane: CTAs whose tile range meets the lane's.
    //    Partial i comes from CTA cta_lo + i; CTAs with an empty tile range wrote nothing.  Worked out once
    //    per block (the range arithmetic is 64-bit divisions) and kept in shared memory.
    const long long a_tile = (long long)lane * sc.tiles_per_lane, b_tile = a_tile + sc.tiles_per_lane;
    int cta_lo = 0, cta_hi = -1;
    if (sc.tiles_per_lane > 0) {
        cta_lo = (int)((a_tile * p.stream_grid) / sc.n_tiles);
        while (cta_lo > 0 && cta_first_tile(cta_lo, sc.n_tiles, p.stream_grid) > a_tile) --cta_lo;
        while (cta_lo + 1 < p.stream_grid && cta_first_tile(cta_lo + 1, sc.n_tiles, p.stream_grid) <= a_tile) ++cta_lo;
        cta_hi = cta_lo;
        while (cta_hi + 1 < p.stream_grid && cta_first_tile(cta_hi + 1, sc.n_tiles, p.stream_grid) < b_tile) ++cta_hi;
    }
    const int n_parts = min(cta_hi - cta_lo + 1, kMaxParts);
    for (int i = tid; i < n_parts; i += kFinishThreads) {
        const int c = cta_lo + i;
        const bool wrote = cta_first_tile(c, sc.n_tiles, p.stream_grid) < cta_first_tile(c + 1, sc.n_tiles, p.stream_grid);
        s_part[i] = wrote ? c + lane : -1;
    }
    __syncthreads();

    // 2. one warp per head: the partials' (max, sum) are fetched first, the new token's own logit (both
    //    operands rotated at max_pos and scaled) is worked out while they travel, then everything is merged
    if (!kStatsOnly && p.update && warp == kFinishThreads / 32 - 1) counters_by_warp();
    constexpr int kPartsPerLane = (kMaxParts + 31) / 32;
    for (int gh = warp; gh < p.G; gh += kFinishThreads / 32) {
        float pm[kPartsPerLane], pl[kPartsPerLane];
#pragma unroll
        for (int j = 0; j < kPartsPerLane; ++j) {
            const int i = lane_id + 32 * j;
            pm[j] = -INFINITY;
            pl[j] = 0.f;
            if (i < n_parts && s_part[i] >= 0) {
                const float *pr = p.partials + ((long long)s_part[i] * p.G + gh) * kPartialStride;
                pm[j] = pr[0];
                pl[j] = pr[1];
            }
        }
        const T *qrow = reinterpret_cast<const T *>(p.q) + b * p.qsb + (long long)(kvh * p.G + gh) * p.qsh;
        float part = 0.f;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int i = lane_id + 32 * e;
            const float c = Elem<T>::to_f(crow[i]), sn = Elem<T>::to_f(crow[64 + i]);
            const float ql = Elem<T>::to_f(qrow[i]), qh = Elem<T>::to_f(qrow[i + 64]);
            const float kl = Elem<T>::to_f(krow[i]), kh = Elem<T>::to_f(krow[i + 64]);
            const float qrl = rnd<T>(__fmul_rn(rnd<T>(__fadd_rn(rnd<T>(__fmul_rn(ql, c)), rnd<T>(__fmul_rn(-qh, sn)))), p.rs));
            const float qrh = rnd<T>(__fmul_rn(rnd<T>(__fadd_rn(rnd<T>(__fmul_rn(qh, c)), rnd<T>(__fmul_rn(ql, sn)))), p.rs));
            const float krl = rnd<T>(__fmul_rn(rnd<T>(__fadd_rn(rnd<T>(__fmul_rn(kl, c)), rnd<T>(__fmul_rn(-kh, sn)))), p.rs));
            const float krh = rnd<T>(__fmul_rn(rnd<T>(__fadd_rn(rnd<T>(__fmul_rn(kh, c)), rnd<T>(__fmul_rn(kl, sn)))), p.rs));
            part = fmaf(qrl, krl, part);
            part = fmaf(qrh, krh, part);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
        const float snew = rnd<T>(part);
        float m = snew;
#pragma unroll
        for (int j = 0; j < kPartsPerLane; ++j) m = fmaxf(m, pm[j]);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        float l = 0.f;
#pragma unroll
        for (int j = 0; j < kPartsPerLane; ++j) {
            const float w = pm[j] == -INFINITY ? 0.f : __expf(pm[j] - m);
            l += pl[j] * w;
            if (lane_id + 32 * j < n_parts) s_w[gh * kMaxParts + lane_id + 32 * j] = w;   // the partial's weight in the output
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
        l += __expf(snew - m);
        if (lane_id == 0) {
            s_snew[gh] = snew;
            s_m[gh] = m;
            s_linv[gh] = 1.f / l;
            s_pnew[gh] = __expf(snew - m) / l;
        }
    }
    __syncthreads();

    if (kStatsOnly) {
        if (tid < p.G) {
            float *hs = p.head_stats + ((long long)b * p.H + kvh * p.G + tid) * 4;
            hs[0] = s_m[tid];
            hs[1] = s_linv[tid];
            hs[2] = s_pnew[tid];
        }
        return;
    }
    if (p.homog && p.update && p.ema) {
        // exponent shift and new-token probability of every head of the sequence (left by the first launch)
        for (int h = tid; h < p.H; h += kFinishThreads) {
            const float *hs = p.head_stats + ((long long)b * p.H + h) * 4;
            s_hcg[h] = -hs[0] * 1.4426950408889634f + __log2f(hs[1]);
            s_hpnew[h] = hs[2];
        }
        __syncthreads();
    }

    // 3. output rows, shared out among the lane's blocks
    {
        const int n_out = p.G * 128, per_out = (n_out + p.finish_chunks - 1) / p.finish_chunks;
        const int o_end = min(n_out, (int)(blockIdx.x + 1) * per_out);
        // the highest threads take the output rows: with a short EMA share they are the ones that have fewer
        // vectors of the EMA pass below
        for (int idx = blockIdx.x * per_out + (kFinishThreads - 1 - tid); idx < o_end; idx += kFinishThreads) {
            const int gh = idx >> 7, d = idx & 127;
            float acc = __expf(s_snew[gh] - s_m[gh]) * Elem<T>::to_f(vrow[d]);
#pragma unroll 4
            for (int i = 0; i < n_parts; ++i) {
                const float w = s_w[gh * kMaxParts + i];
                if (w != 0.f) acc = fmaf(p.partials[((long long)s_part[i] * p.G + gh) * kPartialStride + 2 + d], w, acc);
            }
            T *orow = reinterpret_cast<T *>(p.out) + b * p.osb + (long long)(kvh * p.G + gh) * p.osh;
            orow[d] = Elem<T>::from_f(acc * s_linv[gh]);
        }
    }
    if (!p.update) return;

    // 4. EMA scores of this block's slots:  score = T(T(beta*score) + reduce_g T(T(p_g) * (1-beta)))
    if (p.ema) {
        const float w0 = p.ema_w_cache[0];
        const T *lg = reinterpret_cast<const T *>(p.logits) + ((long long)b * p.H + kvh * p.G) * p.S;
        T *scr = reinterpret_cast<T *>(p.score_cache) + (long long)lane * p.S;
        if (p.homog) {
            // every KV head of the sequence computes the same reduction over all H heads and applies it to its own
            // score row: H / G times the logit reads of the per-group rule, no exchange between blocks
            const T *lgb = reinterpret_cast<const T *>(p.logits) + (long long)b * p.H * p.S;
            const int per_block = (p.S + p.finish_chunks - 1) / p.finish_chunks;
            const int s_end = min(p.S, (int)(blockIdx.x + 1) * per_block);
            constexpr float kL2e = 1.4426950408889634f;
            for (int slot = blockIdx.x * per_block + tid; slot < s_end; slot += kFinishThreads) {
                float red = 0.f;
                if (slot < sc.total) {
                    float e[kMaxHomogHeads];
#pragma unroll 4
                    for (int h = 0; h < p.H; ++h) {
                        const float pr = rnd<T>(ex2_approx(fmaf(Elem<T>::to_f(lgb[(long long)h * p.S + slot]), kL2e, s_hcg[h])));
                        e[h] = rnd<T>(__fmul_rn(pr, w0));
                    }
                    red = rnd<T>(reduce_group(e, p.H, p.head_reduction));
                }
                const float decayed = rnd<T>(__fmul_rn(Elem<T>::to_f(scr[slot]), p.beta_pow));
                scr[slot] = Elem<T>::from_f(__fadd_rn(decayed, red));
            }
        } else if (p.S % 8 == 0 && p.head_reduction != CKV_REDUCE_MEDIAN && p.G <= 8) {
            if (p.head_reduction == CKV_REDUCE_MAX) ema_pass_vec<T, true>(p, sc, lg, scr, s_m, s_linv, w0, tid);
            else ema_pass_vec<T, false>(p, sc, lg, scr, s_m, s_linv, w0, tid);
        } else {
            const int per_block = (p.S + p.finish_chunks - 1) / p.finish_chunks;
            const int s_end = min(p.S, (int)(blockIdx.x + 1) * per_block);
            for (int slot = blockIdx.x * per_block + tid; slot < s_end; slot += kFinishThreads) {
                float red = 0.f;
                if (slot < sc.total) {
                    float e[kMaxG];
                    for (int gh = 0; gh < p.G; ++gh) {
                        const float pr = rnd<T>(__expf(Elem<T>::to_f(lg[(long long)gh * p.S + slot]) - s_m[gh]) * s_linv[gh]);
                        e[gh] = rnd<T>(__fmul_rn(pr, w0));
                    }
                    red = rnd<T>(reduce_group(e, p.G, p.head_reduction));
                }
                const float decayed = rnd<T>(__fmul_rn(Elem<T>::to_f(scr[slot]), p.beta_pow));
                scr[slot] = Elem<T>::from_f(__fadd_rn(decayed, red));
            }
        }
    }

    if (p.ema) {
        // the last work block of the lane inserts the token: the scores of every slot must be final
        __threadfence();
        __syncthreads();
        if (tid == 0) s_is_last = (atomicAdd(&p.sync[1 + lane], 1u) == (unsigned)(p.finish_chunks - 1));
        __syncthreads();
        if (!s_is_last) return;
        __threadfence();
        if (warp == 0) {
            unsigned int new_score = 0;
            {
                float e[kMaxHomogHeads];
                const float w1 = Elem<T>::to_f(reinterpret_cast<const T *>(p.ema_w_new)[0]);
                const int n_red = p.homog ? p.H : p.G;
                const float *pn = p.homog ? s_hpnew : s_pnew;
                for (int gh = 0; gh < n_red; ++gh) e[gh] = rnd<T>(__fmul_rn(rnd<T>(pn[gh]), w1));
                const T red = Elem<T>::from_f(rnd<T>(reduce_group(e, n_red, p.head_reduction)));
                new_score = (unsigned int)*reinterpret_cast<const unsigned short *>(&red);
                if (lane_id == 0) reinterpret_cast<T *>(p.new_scores)[lane] = red;
            }
            __syncwarp();
            if (p.C <= kOneTokenMaxCascades) update_lane_one_token(p.upd, lane, s_stored, s_start, s_every, sc.sinks, sc.seen, new_score);
            else update_lane_walk(p.upd, lane, s_stored, s_start, s_every);
        }
    }
    arrive_and_publish();
}

// ------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// [rows, 128] 16-bit row-major tensor, boxes of 64 rows x 64 elements (128 bytes), 128-byte swizzle.
int make_rows_map(CUtensorMap *tm, const void *base, uint64_t rows, int dtype) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(CKV_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[2] = {128, rows};
    const cuuint64_t strides[1] = {256};
    const cuuint32_t box[2] = {64, (cuuint32_t)kTile};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(tm, dtype == CKV_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                          const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(CKV_E_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return CKV_OK;
}

// The six maps of a decode call describe the same tensors step after step: keep the last few encodings per
// host thread (a map depends only on base address, row count and element type) and copy instead of encoding.
int cached_rows_map(CUtensorMap *tm, const void *base, uint64_t rows, int dtype) {
    struct Entry {
        const void *base;
        uint64_t rows;
        int dtype;
        CUtensorMap map;
    };
    constexpr int kEntries = 32;
    static thread_local Entry entries[kEntries];
    static thread_local int n_entries = 0, next = 0;
    for (int i = 0; i < n_entries; ++i) {
        const Entry &e = entries[i];
        if (e.base == base && e.rows == rows && e.dtype == dtype) {
            *tm = e.map;
            return CKV_OK;
        }
    }
    const int rc = make_rows_map(tm, base, rows, dtype);
    if (rc != CKV_OK) return rc;
    Entry &e = entries[next];
    e.base = base; e.rows = rows; e.dtype = dtype; e.map = *tm;
    next = (next + 1) % kEntries;
    if (n_entries < kEntries) ++n_entries;
    return CKV_OK;
}

size_t up256(size_t x) { return (x + 255) & ~(size_t)255; }

struct DecodeScratch {
    size_t status, sync, image_tag, head_stats, logits, partials, new_scores, rope_slots, image_bytes, total;
};

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
    }
    return n;
}

int sink_rows_padded(const Dims &d) { return ((d.NS + kTile - 1) / kTile) * kTile; }

DecodeScratch decode_scratch(const Dims &d) {
    DecodeScratch s;
    const size_t lanes = (size_t)d.B * d.KVH;
    size_t off = 0;
    s.status = off; off += 256;
    s.sync = off; off += up256((1 + lanes) * 4);
    s.image_tag = off; off += 256;
    s.head_stats = off; off += up256((size_t)d.B * d.H * 4 * sizeof(float));
    s.logits = off; off += up256((size_t)d.B * d.H * d.S * 2);
    s.partials = off; off += up256((size_t)(sm_count() + lanes) * d.G * kPartialStride * 4);
    s.new_scores = off; off += up256(lanes * 2);
    off = (off + 1023) & ~(size_t)1023;
    s.image_bytes = ((size_t)(sink_rows_padded(d) + d.S + kTile) * 256 + 1023) & ~(size_t)1023;
    s.rope_slots = off; off += 2 * s.image_bytes;
    s.total = off;
    return s;
}

}  // namespace

bool decode_tuned_supported(const Dims &d, int n_tokens) {
    return n_tokens == 1 && (d.dtype == CKV_BF16 || d.dtype == CKV_F16) && d.D == 128 && d.G <= kMaxG &&
           (!d.homogeneous || d.H <= kMaxHomogHeads) && d.S % 2 == 0 && d.NS >= 1;
}

size_t decode_workspace_bytes(const Dims &d) { return decode_scratch(d).total; }

int launch_decode_tuned(const Dims &d, const ckv_layer_state *st, const void *q, int64_t qsb, int64_t qsh,
                        const void *key, const void *value, int64_t ksb, int64_t ksh, const void *rope,
                        int64_t rope_rows, const float *ema_w_cache, const void *ema_w_new, void *out, int64_t osb,
                        int64_t osh, void *workspace, size_t workspace_bytes, int flags, cudaStream_t stream,
                        ProfileHook *hook) {
    const DecodeScratch s = decode_scratch(d);
    if (!workspace || workspace_bytes < s.total)
        return fail(CKV_E_WORKSPACE, "workspace of %zu bytes, need %zu", workspace_bytes, s.total);
    if (rope_rows <= (int64_t)d.NS + d.S + 1)
        return fail(CKV_E_ARG, "rope table has %lld rows, need more than %d", (long long)rope_rows, d.NS + d.S + 1);
    const bool update = (flags & CKV_ATTN_UPDATE) != 0;
    const bool ema = update && d.admission == CKV_ADMIT_EMA;
    if (ema && (!ema_w_cache || !ema_w_new)) return fail(CKV_E_ARG, "EMA rule needs ema_w_cache and ema_w_new");
    if (((uintptr_t)q | (uintptr_t)out) % 4 != 0 || (qsb % 2) || (qsh % 2))
        return fail(CKV_E_ARG, "q rows must be 4-byte aligned");
    if (((uintptr_t)key | (uintptr_t)value | (uintptr_t)rope) % 16 != 0 || (ksb * 2) % 16 || (ksh * 2) % 16)
        return fail(CKV_E_ARG, "key/value/rope rows must be 16-byte aligned");
    if (((uintptr_t)st->key_cache | (uintptr_t)st->value_cache | (uintptr_t)st->sink_keys |
         (uintptr_t)st->sink_values) % 16 != 0)
        return fail(CKV_E_ARG, "cache tensors must be 16-byte aligned");

    static bool attr_set[64] = {};
    if (first_use_on_this_device(attr_set)) {
        CKV_CUDA_CHECK(cudaFuncSetAttribute(decode_stream_kernel<__nv_bfloat16, 1>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamSmem));
        CKV_CUDA_CHECK(cudaFuncSetAttribute(decode_stream_kernel<__nv_bfloat16, 2>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamSmem));
        CKV_CUDA_CHECK(cudaFuncSetAttribute(decode_stream_kernel<__half, 1>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamSmem));
        CKV_CUDA_CHECK(cudaFuncSetAttribute(decode_stream_kernel<__half, 2>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamSmem));
    }
    const uint64_t lanes = (uint64_t)d.B * d.KVH;
    CUtensorMap tmK, tmV, tmSK, tmSV, tmR0, tmR1;
    int rc;
    if ((rc = cached_rows_map(&tmK, st->key_cache, lanes * d.S, d.dtype)) != CKV_OK) return rc;
    if ((rc = cached_rows_map(&tmV, st->value_cache, lanes * d.S, d.dtype)) != CKV_OK) return rc;
    if ((rc = cached_rows_map(&tmSK, st->sink_keys, lanes * d.NS, d.dtype)) != CKV_OK) return rc;
    if ((rc = cached_rows_map(&tmSV, st->sink_values, lanes * d.NS, d.dtype)) != CKV_OK) return rc;
    if ((rc = cached_rows_map(&tmR0, (uint8_t *)workspace + s.rope_slots, (uint64_t)sink_rows_padded(d) + d.S, d.dtype)) != CKV_OK)
        return rc;
    if ((rc = cached_rows_map(&tmR1, (uint8_t *)workspace + s.rope_slots + s.image_bytes,
                            (uint64_t)sink_rows_padded(d) + d.S, d.dtype)) != CKV_OK)
        return rc;

    uint8_t *ws = (uint8_t *)workspace;
    DecodeParams p;
    p.q = q; p.qsb = qsb; p.qsh = qsh;
    p.knew = key; p.vnew = value; p.ksb = ksb; p.ksh = ksh;
    p.out = out; p.osb = osb; p.osh = osh;
    p.rope = rope; p.rope_rows = rope_rows;
    p.ema_w_cache = ema_w_cache; p.ema_w_new = ema_w_new;
    p.score_cache = st->score_cache;
    p.pos = (long long *)st->pos; p.sink_pos = (long long *)st->sink_pos;
    p.stored_tokens = (long long *)st->stored_tokens; p.start_indices = (long long *)st->start_indices;
    p.stored_sinks = (long long *)st->stored_sinks; p.seen = (long long *)st->seen_tokens;
    p.every_n = (const long long *)st->every_n;
    p.mask = st->mask; p.sink_mask = st->sink_mask;
    p.status = (int *)(ws + s.status);
    p.sync = (unsigned int *)(ws + s.sync);
    p.logits = ws + s.logits;
    p.partials = (float *)(ws + s.partials);
    p.new_scores = ws + s.new_scores;
    p.rope_slots = ws + s.rope_slots;
    p.image_bytes = (long long)s.image_bytes;
    p.image_tag = (long long *)(ws + s.image_tag);
    p.head_stats = (float *)(ws + s.head_stats);
    p.homog = d.homogeneous ? 1 : 0;
    p.sink_rows_pad = sink_rows_padded(d);
    p.B = d.B; p.KVH = d.KVH; p.H = d.H; p.G = d.G; p.NS = d.NS; p.W = d.W; p.C = d.C; p.S = d.S;
    p.ema = ema; p.update = update; p.head_reduction = d.head_reduction; p.eager_fill = d.eager_fill;
    p.dtype = d.dtype;
    p.stream_grid = sm_count() < kMaxParts ? sm_count() : kMaxParts;
    // Blocks per lane in the finish kernel: `chunks` work blocks (merge, output, EMA pass; one is enough without
    // the EMA pass), one block that inserts the token under the stride rule, `img` blocks for the lane-invariant
    // state -- about one image block per SM over the whole grid, the work blocks filling the rest of one wave of
    // three blocks per SM.
    int chunks = 1, upd = 0, img = 0;
    if (update) {
        img = (int)((uint64_t)sm_count() / lanes);
        img = img < 1 ? 1 : (img > 32 ? 32 : img);
        if (ema) {
            chunks = (int)((3 * (uint64_t)sm_count()) / lanes) - img;
            chunks = chunks < 1 ? 1 : (chunks > 64 ? 64 : chunks);
        } else {
            upd = 1;
        }
    }
    p.finish_chunks = chunks; p.finish_upd = upd; p.finish_img = img;
    p.rs = (float)sqrt(1.0 / sqrt((double)d.D));
    p.beta_pow = (float)d.beta;
    UpdateParams &u = p.upd;
    u.key = (const uint8_t *)key; u.val = (const uint8_t *)value;
    u.ksb = ksb * 2; u.ksh = ksh * 2; u.kst = 0;
    u.scr = ema ? (const uint8_t *)p.new_scores : nullptr;
    u.ssb = (long long)d.KVH * 2; u.ssh = 2; u.sst = 0;
    u.sink_k = (uint8_t *)st->sink_keys; u.sink_v = (uint8_t *)st->sink_values;
    u.cache_k = (uint8_t *)st->key_cache; u.cache_v = (uint8_t *)st->value_cache;
    u.cache_s = (uint8_t *)st->score_cache;
    u.og_pos = (long long *)st->og_pos;
    u.stored_tokens = (const long long *)st->stored_tokens; u.start_indices = (const long long *)st->start_indices;
    u.stored_sinks = (const long long *)st->stored_sinks; u.seen = (const long long *)st->seen_tokens;
    u.every_n = (const long long *)st->every_n;
    u.KVH = d.KVH; u.K = 1; u.NS = d.NS; u.W = d.W; u.C = d.C; u.S = d.S;
    u.row_bytes = 256; u.esz = 2; u.dtype = d.dtype; u.eager_fill = d.eager_fill;

    {
        const long long work = (long long)(p.sink_rows_pad + d.S) * 16;
        // Two blocks per SM: in steady state the kernel only compares the tag and returns, and a small grid returns
        // sooner (5.4 -> ~3 us); the full rewrite after a chunk or a reset takes a few more grid-stride rounds.
        int blocks = (int)((work + 255) / 256);
        blocks = blocks > 2 * sm_count() ? 2 * sm_count() : blocks;
        if (hook) hook->before(stream, "rope_slots_kernel");
        rope_slots_kernel<<<blocks, 256, 0, stream>>>(p);
        if (hook) hook->after(stream);
        CKV_CUDA_CHECK(cudaGetLastError());
    }
    if (hook) hook->before(stream, "decode_stream_kernel");
    const bool hi = d.G > 8;
    if (d.dtype == CKV_BF16) {
        if (hi) decode_stream_kernel<__nv_bfloat16, 2><<<p.stream_grid, kStreamThreads, kStreamSmem, stream>>>(tmK, tmV, tmSK, tmSV, tmR0, tmR1, p);
        else decode_stream_kernel<__nv_bfloat16, 1><<<p.stream_grid, kStreamThreads, kStreamSmem, stream>>>(tmK, tmV, tmSK, tmSV, tmR0, tmR1, p);
    } else {
        if (hi) decode_stream_kernel<__half, 2><<<p.stream_grid, kStreamThreads, kStreamSmem, stream>>>(tmK, tmV, tmSK, tmSV, tmR0, tmR1, p);
        else decode_stream_kernel<__half, 1><<<p.stream_grid, kStreamThreads, kStreamSmem, stream>>>(tmK, tmV, tmSK, tmSV, tmR0, tmR1, p);
    }
    if (hook) hook->after(stream);
    CKV_CUDA_CHECK(cudaGetLastError());
    const dim3 grid(chunks + upd + img, (unsigned)lanes);
    const bool two_launches = p.homog && ema;
    if (two_launches) {   // homogeneous heads: every lane first publishes its heads' statistics
        const dim3 sgrid(1, (unsigned)lanes);
        if (d.dtype == CKV_BF16) decode_finish_kernel<__nv_bfloat16, true><<<sgrid, kFinishThreads, 0, stream>>>(p);
        else decode_finish_kernel<__half, true><<<sgrid, kFinishThreads, 0, stream>>>(p);
        CKV_CUDA_CHECK(cudaGetLastError());
    }
    if (hook) hook->before(stream, "decode_finish_kernel");
    if (d.dtype == CKV_BF16) decode_finish_kernel<__nv_bfloat16, false><<<grid, kFinishThreads, 0, stream>>>(p);
    else decode_finish_kernel<__half, false><<<grid, kFinishThreads, 0, stream>>>(p);
    if (hook) hook->after(stream);
    CKV_CUDA_CHECK(cudaGetLastError());
    note_launches(two_launches ? 4 : 3);
    return CKV_OK;
}

int launch_decode_wait_selftest(int *status, cudaStream_t stream) {
    decode_wait_selftest_kernel<<<1, 32, 0, stream>>>(status);
    CKV_CUDA_CHECK(cudaGetLastError());
    return CKV_OK;
}

#ifdef CKV_BOUNDS
int read_bounds_status_decode(int *out) { return read_bounds_status_of_this_unit(out); }
#endif

}  // namespace ckv
