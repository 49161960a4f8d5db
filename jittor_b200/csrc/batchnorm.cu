// Global-batch BatchNorm pieces for NCHW tensors (python/jittor/nn.py:671-683):
//   bn_stats -- per-channel sum(x), sum(x*x) in ONE pass over x, written unnormalised into a 2*C float
//               buffer so that ranks of a batch-sharded job can all-reduce it as one message;
//   bn_apply -- y = [relu](x*w + b) with w = gamma/sqrt(var+eps), b = beta - mean*w, one read one write.
// Both are HBM-bound; 128-bit accesses, planes (n, c) are distributed over CTAs.
#include "common.cuh"

namespace b200jt {

template <typename T> struct IO;
template <> struct IO<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float* o) { float4 v = *reinterpret_cast<const float4*>(p); o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w; }
    static __device__ __forceinline__ void store(float* p, const float* o) { __stcs(reinterpret_cast<float4*>(p), make_float4(o[0], o[1], o[2], o[3])); }
    static __device__ __forceinline__ float ld(const float* p) { return *p; }
    static __device__ __forceinline__ void st(float* p, float v) { *p = v; }
};
template <> struct IO<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* o) {
        uint4 v = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; i++) { float2 f = __bfloat1622float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* o) {
        uint4 v; __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
        __stcs(reinterpret_cast<uint4*>(p), v);
    }
    static __device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void st(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }
};

// grid = (planes_per_channel_chunks, C): CTA (j, c) folds the planes n = j, j+gridDim.x, ... of channel c
// and adds its two partial sums to stats with one atomicAdd pair.
template <typename T>
__global__ void __launch_bounds__(256)
bn_stats_kernel(const T* __restrict__ x, float* __restrict__ stats, int N_, int C, int64_t HW) {
    constexpr int V = IO<T>::N;
    const int c = blockIdx.y;
    float s1 = 0.f, s2 = 0.f;
    const bool vec = (HW % V == 0) && ((uintptr_t)x % 16 == 0);
    for (int n = blockIdx.x; n < N_; n += gridDim.x) {
        const T* p = x + ((int64_t)n * C + c) * HW;
        if (vec) {
            for (int64_t i = threadIdx.x * V; i < HW; i += (int64_t)blockDim.x * V) {
                float v[V]; IO<T>::load(p + i, v);
#pragma unroll
                for (int e = 0; e < V; e++) { s1 += v[e]; s2 += v[e] * v[e]; }
            }
        } else {
            for (int64_t i = threadIdx.x; i < HW; i += blockDim.x) { float v = IO<T>::ld(p + i); s1 += v; s2 += v * v; }
        }
    }
    __shared__ float sm1[8], sm2[8];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) { s1 += __shfl_xor_sync(0xffffffffu, s1, d); s2 += __shfl_xor_sync(0xffffffffu, s2, d); }
    if ((threadIdx.x & 31) == 0) { sm1[threadIdx.x >> 5] = s1; sm2[threadIdx.x >> 5] = s2; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float a = 0.f, b = 0.f;
        for (int i = 0; i < 8; i++) { a += sm1[i]; b += sm2[i]; }
        atomicAdd(stats + c, a);
        atomicAdd(stats + C + c, b);
    }
}

// TX / TY: element types of x and y (the reference's dtype rules make bfloat16 x * float32 w a float32 result
// unless amp flags keep 16 bit, so both combinations occur). Every CTA first derives the per-channel scale and shift
// into shared memory, then the whole tensor is walked as one stream of 16-byte vectors (one division per vector
// finds the channel), so small planes do not leave lanes idle.
template <typename TX, typename TY>
__global__ void __launch_bounds__(256)
bn_apply_kernel(const TX* __restrict__ x, TY* __restrict__ y, const float* __restrict__ stats, float rcount,
                const float* __restrict__ gamma, const float* __restrict__ beta, float eps, int relu,
                int64_t planes, int C, int64_t HW,
                float* __restrict__ running_mean, float* __restrict__ running_var, float momentum) {
    extern __shared__ float ws_[];                 // [2][C]: scale, shift
    float* sw = ws_; float* sb = ws_ + C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float mean = stats[c] * rcount;
        const float var = fmaxf(stats[C + c] * rcount - mean * mean, 0.f);
        const float w = (gamma ? gamma[c] : 1.f) / sqrtf(var + eps);
        sw[c] = w; sb[c] = (beta ? beta[c] : 0.f) - mean * w;
        // running += (batch - running) * momentum (python/jittor/nn.py:684-688), done once, by the first CTA
        if (running_mean && blockIdx.x == 0) {
            running_mean[c] += (mean - running_mean[c]) * momentum;
            running_var[c] += (var - running_var[c]) * momentum;
        }
    }
    __syncthreads();
    constexpr int V = IO<TX>::N > IO<TY>::N ? IO<TX>::N : IO<TY>::N;     // elements per thread step
    const bool vec = (HW % V == 0) && ((uintptr_t)x % 16 == 0) && ((uintptr_t)y % 16 == 0);
    if (vec) {
        const int64_t vpp = HW / V, nvec = planes * vpp;
        for (int64_t v = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * blockDim.x) {
            const int c = (int)((v / vpp) % C);
            const float w = sw[c], b = sb[c];
            const int64_t i = v * V;
            float f[V];
#pragma unroll
            for (int k = 0; k < V / IO<TX>::N; k++) IO<TX>::load(x + i + k * IO<TX>::N, f + k * IO<TX>::N);
#pragma unroll
            for (int e = 0; e < V; e++) { float o = f[e] * w + b; f[e] = relu ? fmaxf(o, 0.f) : o; }
#pragma unroll
            for (int k = 0; k < V / IO<TY>::N; k++) IO<TY>::store(y + i + k * IO<TY>::N, f + k * IO<TY>::N);
        }
    } else {
        const int64_t n = planes * HW;
        for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
            const int c = (int)((i / HW) % C);
            float o = IO<TX>::ld(x + i) * sw[c] + sb[c];
            IO<TY>::st(y + i, relu ? fmaxf(o, 0.f) : o);
        }
    }
}

static int nchw(const b200jt_tensor* x, int* N_, int* C, int64_t* HW) {
    B200JT_CHECK_ARG(valid_tensor(x) && x->ndim >= 2, "x must be [N, C, ...]");
    B200JT_CHECK_ARG(x->dtype == B200JT_FLOAT32 || x->dtype == B200JT_BFLOAT16, "x must be float32 or bfloat16");
    *N_ = (int)x->shape[0]; *C = (int)x->shape[1]; *HW = 1;
    for (int d = 2; d < x->ndim; d++) *HW *= x->shape[d];
    return 0;
}

}  // namespace b200jt

using namespace b200jt;

extern "C" int b200jt_bn_stats(const b200jt_tensor* x, float* stats, void* stream) {
    int N_, C; int64_t HW;
    int rc = nchw(x, &N_, &C, &HW);
    if (rc) return rc;
    B200JT_CHECK_ARG(stats != nullptr, "stats is NULL");
    cudaStream_t st = (cudaStream_t)stream;
    B200JT_CUDA(cudaMemsetAsync(stats, 0, sizeof(float) * 2 * C, st));
    if (numel(x) == 0) return 0;
    // about 8 CTAs per SM in total, at most one per plane
    int per_c = (8 * kNumSMs + C - 1) / C;
    if (per_c > N_) per_c = N_;
    if (per_c < 1) per_c = 1;
    dim3 grid(per_c, C);
    if (x->dtype == B200JT_FLOAT32) bn_stats_kernel<float><<<grid, 256, 0, st>>>((const float*)x->ptr, stats, N_, C, HW);
    else bn_stats_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x->ptr, stats, N_, C, HW);
    B200JT_LAUNCH_CHECK();
    return 0;
}

extern "C" int b200jt_bn_apply(const b200jt_tensor* x, const float* stats, double count, const float* gamma, const float* beta,
                               double eps, int relu, const b200jt_tensor* y,
                               float* running_mean, float* running_var, double momentum, void* stream) {
    int N_, C; int64_t HW;
    int rc = nchw(x, &N_, &C, &HW);
    if (rc) return rc;
    B200JT_CHECK_ARG(valid_tensor(y) && numel(y) == numel(x) && (y->dtype == B200JT_FLOAT32 || y->dtype == B200JT_BFLOAT16),
                     "y must have x's size and be float32 or bfloat16");
    B200JT_CHECK_ARG(stats != nullptr && count > 0, "stats is NULL or count <= 0");
    B200JT_CHECK_ARG((running_mean == nullptr) == (running_var == nullptr), "running_mean and running_var go together");
    if (numel(x) == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t planes = (int64_t)N_ * C;
    B200JT_CHECK_ARG(C <= 6144, "at most 6144 channels");
    unsigned grid = grid_for(numel(x) / 8 + 1, 256);
    const size_t smem = sizeof(float) * 2 * C;
    const float rc_ = (float)(1.0 / count);
#define B200JT_BN(TX, TY) bn_apply_kernel<TX, TY><<<grid, 256, smem, st>>>((const TX*)x->ptr, (TY*)y->ptr, stats, rc_, gamma, beta, (float)eps, relu, planes, C, HW, running_mean, running_var, (float)momentum)
    if (x->dtype == B200JT_FLOAT32) { if (y->dtype == B200JT_FLOAT32) B200JT_BN(float, float); else B200JT_BN(float, __nv_bfloat16); }
    else { if (y->dtype == B200JT_FLOAT32) B200JT_BN(__nv_bfloat16, float); else B200JT_BN(__nv_bfloat16, __nv_bfloat16); }
#undef B200JT_BN
    B200JT_LAUNCH_CHECK();
    return 0;
}
