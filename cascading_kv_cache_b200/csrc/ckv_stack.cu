// The two element-wise operators between the dense layers of the decoder stack that surrounds the attention in
// the end-to-end configuration, each as one kernel instead of a chain of framework kernels:
//
//   ckv_add_rmsnorm : s = T(x + residual);  y = T(w * T(s * rsqrt(mean(s^2) + eps)))
//                     -- the residual add of the decoder layer followed by its RMSNorm
//                        (cascade/models/llama/modeling_llama.py:113-127, :745-770): fp32 variance, the
//                        normalised row rounded to T before the weight is applied, as the reference does
//   ckv_silu_mul    : y = T(T(silu(gate)) * up)      -- the SwiGLU gate (modeling_llama.py:282-313)
//
// Both are bandwidth-bound one-pass kernels over 16-bit rows: 16-byte loads, one block per row for the norm
// (the row stays in shared memory between the two sweeps), a grid-stride loop for the gate.
#include "ckv_common.cuh"

namespace ckv {

namespace {

constexpr int kNormThreads = 256;

template <typename T> struct Pair;
template <> struct Pair<__nv_bfloat16> {
    static __device__ __forceinline__ float2 to_f2(uint32_t u) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&u)); }
    static __device__ __forceinline__ uint32_t from_f2(float2 f) {
        __nv_bfloat162 v = __float22bfloat162_rn(f);
        return *reinterpret_cast<uint32_t *>(&v);
    }
};
template <> struct Pair<__half> {
    static __device__ __forceinline__ float2 to_f2(uint32_t u) { return __half22float2(*reinterpret_cast<__half2 *>(&u)); }
    static __device__ __forceinline__ uint32_t from_f2(float2 f) {
        __half2 v = __float22half2_rn(f);
        return *reinterpret_cast<uint32_t *>(&v);
    }
};

template <typename T>
__global__ void __launch_bounds__(kNormThreads)
add_rmsnorm_kernel(const uint4 *x, const uint4 *residual, const uint4 *weight, uint4 *normed, uint4 *sum_out,
                   int hidden8, float inv_hidden, float eps) {
    extern __shared__ uint4 s_row[];                 // the summed row, hidden8 vectors of 8 elements
    __shared__ float s_part[kNormThreads / 32];
    const long long row = blockIdx.x;
    const uint4 *xr = x + row * hidden8;
    const uint4 *rr = residual ? residual + row * hidden8 : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden8; i += kNormThreads) {
        uint4 a = xr[i];
        uint32_t *aw = reinterpret_cast<uint32_t *>(&a);
        if (rr) {
            const uint4 b = rr[i];
            const uint32_t *bw = reinterpret_cast<const uint32_t *>(&b);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 u = Pair<T>::to_f2(aw[j]), v = Pair<T>::to_f2(bw[j]);
                aw[j] = Pair<T>::from_f2(make_float2(__fadd_rn(u.x, v.x), __fadd_rn(u.y, v.y)));
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 u = Pair<T>::to_f2(aw[j]);
            ss = fmaf(u.x, u.x, ss);
            ss = fmaf(u.y, u.y, ss);
        }
        s_row[i] = a;
        if (sum_out) sum_out[row * hidden8 + i] = a;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kNormThreads / 32; ++w) tot += s_part[w];
    const float rs = rsqrtf(__fadd_rn(__fmul_rn(tot, inv_hidden), eps));
    for (int i = threadIdx.x; i < hidden8; i += kNormThreads) {
        const uint4 a = s_row[i], w = weight[i];       // each thread reads back what it wrote
        const uint32_t *aw = reinterpret_cast<const uint32_t *>(&a), *ww = reinterpret_cast<const uint32_t *>(&w);
        uint4 y;
        uint32_t *yw = reinterpret_cast<uint32_t *>(&y);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 u = Pair<T>::to_f2(aw[j]), g = Pair<T>::to_f2(ww[j]);
            const float2 t = Pair<T>::to_f2(Pair<T>::from_f2(make_float2(__fmul_rn(u.x, rs), __fmul_rn(u.y, rs))));
            yw[j] = Pair<T>::from_f2(make_float2(__fmul_rn(g.x, t.x), __fmul_rn(g.y, t.y)));
        }
        normed[row * hidden8 + i] = y;
    }
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(256)
silu_mul_kernel(const uint4 *gate, const uint4 *up, uint4 *out, long long rows, int cols8, long long ld_gate8,
                long long ld_up8) {
    const long long n = rows * cols8;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long r = idx / cols8;
        const int c = (int)(idx - r * cols8);
        const uint4 g = gate[r * ld_gate8 + c], u = up[r * ld_up8 + c];
        const uint32_t *gw = reinterpret_cast<const uint32_t *>(&g), *uw = reinterpret_cast<const uint32_t *>(&u);
        uint4 y;
        uint32_t *yw = reinterpret_cast<uint32_t *>(&y);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 a = Pair<T>::to_f2(gw[j]), b = Pair<T>::to_f2(uw[j]);
            const float2 s = Pair<T>::to_f2(Pair<T>::from_f2(make_float2(silu_f(a.x), silu_f(a.y))));
            yw[j] = Pair<T>::from_f2(make_float2(__fmul_rn(s.x, b.x), __fmul_rn(s.y, b.y)));
        }
        out[idx] = y;
    }
}

bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

}  // namespace ckv

extern "C" int ckv_add_rmsnorm(const void *x, const void *residual, const void *weight, void *normed, void *sum_out,
                               int64_t rows, int32_t hidden, double eps, int32_t dtype, void *stream) {
    using namespace ckv;
    if (!x || !weight || !normed) return fail(CKV_E_ARG, "ckv_add_rmsnorm: x, weight and normed are required");
    if (dtype != CKV_BF16 && dtype != CKV_F16) return fail(CKV_E_UNSUPPORTED, "ckv_add_rmsnorm: 16-bit rows only");
    if (rows < 0 || hidden <= 0 || hidden % 8 != 0 || hidden > 65536)
        return fail(CKV_E_ARG, "ckv_add_rmsnorm: hidden (%d) must be a multiple of 8, at most 65536", hidden);
    if (!aligned16(x) || !aligned16(weight) || !aligned16(normed) || (residual && !aligned16(residual)) ||
        (sum_out && !aligned16(sum_out)))
        return fail(CKV_E_ARG, "ckv_add_rmsnorm: rows must be 16-byte aligned");
    if (rows == 0) return CKV_OK;
    if (rows > 0x7fffffffLL) return fail(CKV_E_ARG, "ckv_add_rmsnorm: too many rows");
    const int hidden8 = hidden / 8;
    const size_t smem = (size_t)hidden * 2;
    cudaStream_t s = (cudaStream_t)stream;
    static bool attr_set[64] = {};
    if (first_use_on_this_device(attr_set)) {
        CKV_CUDA_CHECK(cudaFuncSetAttribute(add_rmsnorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536 * 2));
        CKV_CUDA_CHECK(cudaFuncSetAttribute(add_rmsnorm_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536 * 2));
    }
    const float inv = 1.0f / (float)hidden;
    if (dtype == CKV_BF16)
        add_rmsnorm_kernel<__nv_bfloat16><<<(unsigned)rows, kNormThreads, smem, s>>>(
            (const uint4 *)x, (const uint4 *)residual, (const uint4 *)weight, (uint4 *)normed, (uint4 *)sum_out, hidden8, inv, (float)eps);
    else
        add_rmsnorm_kernel<__half><<<(unsigned)rows, kNormThreads, smem, s>>>(
            (const uint4 *)x, (const uint4 *)residual, (const uint4 *)weight, (uint4 *)normed, (uint4 *)sum_out, hidden8, inv, (float)eps);
    CKV_CUDA_CHECK(cudaGetLastError());
    return CKV_OK;
}

extern "C" int ckv_silu_mul(const void *gate, const void *up, void *out, int64_t rows, int32_t cols, int64_t ld_gate,
                            int64_t ld_up, int32_t dtype, void *stream) {
    using namespace ckv;
    if (!gate || !up || !out) return fail(CKV_E_ARG, "ckv_silu_mul: null pointer");
    if (dtype != CKV_BF16 && dtype != CKV_F16) return fail(CKV_E_UNSUPPORTED, "ckv_silu_mul: 16-bit rows only");
    if (rows < 0 || cols <= 0 || cols % 8 != 0 || ld_gate % 8 != 0 || ld_up % 8 != 0 || ld_gate < cols || ld_up < cols)
        return fail(CKV_E_ARG, "ckv_silu_mul: cols and row strides must be multiples of 8 elements");
    if (!aligned16(gate) || !aligned16(up) || !aligned16(out)) return fail(CKV_E_ARG, "ckv_silu_mul: rows must be 16-byte aligned");
    if (rows == 0) return CKV_OK;
    const long long n = rows * (cols / 8);
    long long blocks = (n + 255) / 256;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (blocks > 8LL * sms) blocks = 8LL * sms;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CKV_BF16)
        silu_mul_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>((const uint4 *)gate, (const uint4 *)up, (uint4 *)out, rows,
                                                                        cols / 8, ld_gate / 8, ld_up / 8);
    else
        silu_mul_kernel<__half><<<(unsigned)blocks, 256, 0, s>>>((const uint4 *)gate, (const uint4 *)up, (uint4 *)out, rows, cols / 8,
                                                                 ld_gate / 8, ld_up / 8);
    CKV_CUDA_CHECK(cudaGetLastError());
    return CKV_OK;
}
