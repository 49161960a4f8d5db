// Fused row softmax / log-softmax and row LayerNorm over the last axis: one read and one write of
// the [rows, cols] tensor (the reference's meta-op form reads x three times, python/jittor/nn.py:527-535,778-787).
//
//   reg kernel  -- the row lives in registers: CTA of 256 threads (or one warp for short rows), 128-bit
//                  loads, warp-shuffle tree + one shared-memory hop, 128-bit stores. HBM-bound: 1R + 1W.
//   cluster kernel -- rows too long for one CTA's registers (above 8192 float32 / 16384 bfloat16 columns, up to 8x
//                  that): a thread-block cluster of 2, 4 or 8 CTAs holds the row, every CTA reduces its slice and the
//                  slices' partial results are exchanged through distributed shared memory. Still 1R + 1W.
//   pass kernel -- any cols / alignment: three sweeps by one CTA per row (re-reads hit L2).
// IO dtype float32 or bfloat16; all math in float32.
#include "common.cuh"
#include <algorithm>
#include <cfloat>
#include <cooperative_groups.h>

namespace b200jt {

enum RowOp : int { ROW_SOFTMAX = 0, ROW_LOG_SOFTMAX = 1, ROW_LAYERNORM = 2 };

template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float* out) {
        float4 v = __ldcs(reinterpret_cast<const float4*>(p)); out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* in) {
        __stcs(reinterpret_cast<float4*>(p), make_float4(in[0], in[1], in[2], in[3]));
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* out) {
        uint4 v = __ldcs(reinterpret_cast<const uint4*>(p));
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; i++) { float2 f = __bfloat1622float2(h[i]); out[2 * i] = f.x; out[2 * i + 1] = f.y; }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* in) {
        uint4 v; __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
        __stcs(reinterpret_cast<uint4*>(p), v);
    }
};

template <typename T> __device__ __forceinline__ float ld1(const T* p);
template <> __device__ __forceinline__ float ld1<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld1<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void st1(T* p, float v);
template <> __device__ __forceinline__ void st1<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void st1<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

// Reduction over the GROUP threads that share a row: a warp (GROUP == 32) or the whole CTA.
template <int GROUP, bool IS_MAX>
__device__ __forceinline__ float group_reduce(float v, float* sm) {
    v = IS_MAX ? warp_max(v) : warp_sum(v);
    if constexpr (GROUP == 32) return v;
    else {
        constexpr int W = GROUP / 32;
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        __syncthreads();                      // sm may still be read from the previous reduction
        if (lane == 0) sm[warp] = v;
        __syncthreads();
        float t = lane < W ? sm[lane] : (IS_MAX ? -FLT_MAX : 0.f);
        return IS_MAX ? warp_max(t) : warp_sum(t);
    }
}

template <int N>
__device__ __forceinline__ void load_gb(const float* __restrict__ gamma, const float* __restrict__ beta, int c, float* g, float* b) {
#pragma unroll
    for (int q = 0; q < N / 4; q++) {
        const float4 g4 = gamma ? __ldg(reinterpret_cast<const float4*>(gamma + c + q * 4)) : make_float4(1.f, 1.f, 1.f, 1.f);
        const float4 b4 = beta ? __ldg(reinterpret_cast<const float4*>(beta + c + q * 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
        g[q * 4] = g4.x; g[q * 4 + 1] = g4.y; g[q * 4 + 2] = g4.z; g[q * 4 + 3] = g4.w;
        b[q * 4] = b4.x; b[q * 4 + 1] = b4.y; b[q * 4 + 2] = b4.z; b[q * 4 + 3] = b4.w;
    }
}

// Sums (or maxima) of NV values per thread over the GROUP threads of a row with ONE shared-memory exchange
// (sm holds NV * 8 floats).
template <int GROUP, bool IS_MAX, int NV>
__device__ __forceinline__ void group_reduce_n(float (&v)[NV], float* sm) {
#pragma unroll
    for (int i = 0; i < NV; i++) v[i] = IS_MAX ? warp_max(v[i]) : warp_sum(v[i]);
    if constexpr (GROUP > 32) {
        constexpr int W = GROUP / 32;
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        __syncthreads();                      // sm may still be read from the previous reduction
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < NV; i++) sm[i * 8 + warp] = v[i];
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const float t = lane < W ? sm[i * 8 + lane] : (IS_MAX ? -FLT_MAX : 0.f);
            v[i] = IS_MAX ? warp_max(t) : warp_sum(t);
        }
    }
}

// GROUP threads per row, VPT 16-byte vectors per thread; requires cols % Vec16<T>::N == 0 and
// cols <= GROUP * VPT * N. RPI rows are taken per round (their reductions share the shared-memory exchanges).
template <typename T, int GROUP, int VPT, int OP>
__global__ void __launch_bounds__(256)
row_reg_kernel(const T* __restrict__ x, T* __restrict__ y, const float* __restrict__ gamma,
               const float* __restrict__ beta, int64_t rows, int cols, float eps) {
    constexpr int N = Vec16<T>::N;
    constexpr int ROWS_PER_CTA = 256 / GROUP;
    constexpr int RPI = 1;          // two rows per round were measured slower (fewer CTAs in flight outweigh the shared exchange)
    __shared__ float sm[32];
    const int g = threadIdx.x / GROUP, t = threadIdx.x % GROUP;
    const int nvec = cols / N;
    // a thread owns the same columns in every row it visits: keep their gamma / beta in registers when they fit
    constexpr bool CACHE_GB = (OP == ROW_LAYERNORM) && (VPT * N <= 16);
    float gm[CACHE_GB ? VPT : 1][N], bt[CACHE_GB ? VPT : 1][N];
    if constexpr (CACHE_GB) {
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int vi = t + k * GROUP;
            if (vi < nvec) load_gb<N>(gamma, beta, vi * N, gm[k], bt[k]);
        }
    }
    for (int64_t row0 = ((int64_t)blockIdx.x * ROWS_PER_CTA + g) * RPI; row0 < rows;
         row0 += (int64_t)gridDim.x * ROWS_PER_CTA * RPI) {
        float v[RPI][VPT][N];
        bool live[RPI];
#pragma unroll
        for (int r = 0; r < RPI; r++) {
            live[r] = row0 + r < rows;
            const T* xr = x + (row0 + r) * cols;
#pragma unroll
            for (int k = 0; k < VPT; k++) {
                const int vi = t + k * GROUP;
                if (vi < nvec && live[r]) Vec16<T>::load(xr + (int64_t)vi * N, v[r][k]);
                else {
#pragma unroll
                    for (int e = 0; e < N; e++) v[r][k][e] = (OP == ROW_LAYERNORM) ? 0.f : -FLT_MAX;
                }
            }
        }
        if constexpr (OP == ROW_LAYERNORM) {
            float s[2 * RPI];
#pragma unroll
            for (int r = 0; r < RPI; r++) {
                float s1 = 0.f, s2 = 0.f;
#pragma unroll
                for (int k = 0; k < VPT; k++)
#pragma unroll
                    for (int e = 0; e < N; e++) { s1 += v[r][k][e]; s2 += v[r][k][e] * v[r][k][e]; }
                s[2 * r] = s1; s[2 * r + 1] = s2;
            }
            group_reduce_n<GROUP, false, 2 * RPI>(s, sm);
            const float rc = 1.0f / (float)cols;
#pragma unroll
            for (int r = 0; r < RPI; r++) {
                if (!live[r]) continue;
                T* yr = y + (row0 + r) * cols;
                const float mean = s[2 * r] * rc, m2 = s[2 * r + 1] * rc;
                const float var = fmaxf(m2 - mean * mean, 0.f);
                const float rstd = 1.0f / sqrtf(var + eps);
#pragma unroll
                for (int k = 0; k < VPT; k++) {
                    const int vi = t + k * GROUP;
                    if (vi < nvec) {
                        float o[N];
                        if constexpr (CACHE_GB) {
#pragma unroll
                            for (int e = 0; e < N; e++) { const float w = gm[k][e] * rstd; o[e] = v[r][k][e] * w + (bt[k][e] - mean * w); }
                        } else {
                            float g1[N], b1[N];
                            load_gb<N>(gamma, beta, vi * N, g1, b1);
#pragma unroll
                            for (int e = 0; e < N; e++) { const float w = g1[e] * rstd; o[e] = v[r][k][e] * w + (b1[e] - mean * w); }
                        }
                        Vec16<T>::store(yr + (int64_t)vi * N, o);
                    }
                }
            }
        } else {
            float m[RPI];
#pragma unroll
            for (int r = 0; r < RPI; r++) {
                m[r] = -FLT_MAX;
#pragma unroll
                for (int k = 0; k < VPT; k++)
#pragma unroll
                    for (int e = 0; e < N; e++) m[r] = fmaxf(m[r], v[r][k][e]);
            }
            group_reduce_n<GROUP, true, RPI>(m, sm);
            float sum[RPI];
#pragma unroll
            for (int r = 0; r < RPI; r++) {
                sum[r] = 0.f;
#pragma unroll
                for (int k = 0; k < VPT; k++)
#pragma unroll
                    for (int e = 0; e < N; e++) {
                        if constexpr (OP == ROW_SOFTMAX) {
                            // exp(x - m) as ex2(x * log2e - m * log2e): one FMA and one ex2.approx per element (relative error
                            // ~1e-6 for arguments in [-88, 0]); the padding lanes hold -FLT_MAX and come out as exactly 0
                            const float ex = ex2_approx(fmaf(v[r][k][e], 1.4426950408889634f, -m[r] * 1.4426950408889634f));
                            sum[r] += ex;
                            v[r][k][e] = ex;
                        } else {
                            const float a = v[r][k][e] - m[r];
                            sum[r] += (t + k * GROUP < nvec) ? __expf(a) : 0.f;
                            v[r][k][e] = a;
                        }
                    }
            }
            group_reduce_n<GROUP, false, RPI>(sum, sm);
#pragma unroll
            for (int r = 0; r < RPI; r++) {
                if (!live[r]) continue;
                T* yr = y + (row0 + r) * cols;
                const float ls = logf(sum[r]), inv = 1.0f / sum[r];
#pragma unroll
                for (int k = 0; k < VPT; k++) {
                    const int vi = t + k * GROUP;
                    if (vi < nvec) {
                        float o[N];
#pragma unroll
                        for (int e = 0; e < N; e++) o[e] = (OP == ROW_SOFTMAX) ? v[r][k][e] * inv : v[r][k][e] - ls;
                        Vec16<T>::store(yr + (int64_t)vi * N, o);
                    }
                }
            }
        }
    }
}

// ---- rows held by a cluster -------------------------------------------------------------------------------------------
// CL CTAs of 256 threads share a row: CTA c of the cluster owns the vectors (c*256 + t) + k*256*CL, k < 8. A reduction is
// the CTA-wide one above followed by an exchange: thread 0 of every CTA publishes its CTA's value in its own shared
// memory, the cluster synchronises, and every thread reads the CL values through distributed shared memory and combines
// them in rank order (the same bits in every CTA). Four slots rotate, so a slot is rewritten only after four further
// cluster barriers; a last barrier keeps every CTA's shared memory alive until all its readers are done.
template <int CL, bool IS_MAX, int NV>
__device__ __forceinline__ void cluster_reduce_n(float (&v)[NV], float* sm, float* xch, int& slot) {
    namespace cg = cooperative_groups;
    group_reduce_n<256, IS_MAX, NV>(v, sm);
    cg::cluster_group cluster = cg::this_cluster();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int i = 0; i < NV; i++) xch[slot * 2 + i] = v[i];
    }
    cluster.sync();
#pragma unroll
    for (int i = 0; i < NV; i++) {
        float a = IS_MAX ? -FLT_MAX : 0.f;
#pragma unroll
        for (int c = 0; c < CL; c++) {
            const float p = cluster.map_shared_rank(xch, c)[slot * 2 + i];
            a = IS_MAX ? fmaxf(a, p) : a + p;
        }
        v[i] = a;
    }
    slot = (slot + 1) & 3;
}

template <typename T, int CL, int OP>
__global__ void __launch_bounds__(256)
row_cluster_kernel(const T* __restrict__ x, T* __restrict__ y, const float* __restrict__ gamma,
                   const float* __restrict__ beta, int64_t rows, int cols, float eps) {
    namespace cg = cooperative_groups;
    constexpr int N = Vec16<T>::N, VPT = 8;
    __shared__ float sm[32];
    __shared__ float xch[8];
    cg::cluster_group cluster = cg::this_cluster();
    const int crank = (int)cluster.block_rank(), t = threadIdx.x;
    const int nvec = cols / N;
    const int64_t n_clusters = gridDim.x / CL, cid = blockIdx.x / CL;
    int slot = 0;
    for (int64_t row = cid; row < rows; row += n_clusters) {                // the same trip count in every CTA of a cluster
        const T* xr = x + row * cols;
        T* yr = y + row * cols;
        float v[VPT][N];
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int vi = crank * 256 + t + k * 256 * CL;
            if (vi < nvec) Vec16<T>::load(xr + (int64_t)vi * N, v[k]);
            else {
#pragma unroll
                for (int e = 0; e < N; e++) v[k][e] = (OP == ROW_LAYERNORM) ? 0.f : -FLT_MAX;
            }
        }
        if constexpr (OP == ROW_LAYERNORM) {
            float s[2] = {0.f, 0.f};
#pragma unroll
            for (int k = 0; k < VPT; k++)
#pragma unroll
                for (int e = 0; e < N; e++) { s[0] += v[k][e]; s[1] += v[k][e] * v[k][e]; }
            cluster_reduce_n<CL, false, 2>(s, sm, xch, slot);
            const float rc = 1.0f / (float)cols;
            const float mean = s[0] * rc, m2 = s[1] * rc;
            const float var = fmaxf(m2 - mean * mean, 0.f);
            const float rstd = 1.0f / sqrtf(var + eps);
#pragma unroll
            for (int k = 0; k < VPT; k++) {
                const int vi = crank * 256 + t + k * 256 * CL;
                if (vi < nvec) {
                    float o[N], g1[N], b1[N];
                    load_gb<N>(gamma, beta, vi * N, g1, b1);
#pragma unroll
                    for (int e = 0; e < N; e++) { const float w = g1[e] * rstd; o[e] = v[k][e] * w + (b1[e] - mean * w); }
                    Vec16<T>::store(yr + (int64_t)vi * N, o);
                }
            }
        } else {
            float m[1] = {-FLT_MAX};
#pragma unroll
            for (int k = 0; k < VPT; k++)
#pragma unroll
                for (int e = 0; e < N; e++) m[0] = fmaxf(m[0], v[k][e]);
            cluster_reduce_n<CL, true, 1>(m, sm, xch, slot);
            float sum[1] = {0.f};
#pragma unroll
            for (int k = 0; k < VPT; k++)
#pragma unroll
                for (int e = 0; e < N; e++) {
                    if constexpr (OP == ROW_SOFTMAX) {
                        const float ex = ex2_approx(fmaf(v[k][e], 1.4426950408889634f, -m[0] * 1.4426950408889634f));
                        sum[0] += ex;
                        v[k][e] = ex;
                    } else {
                        const float a = v[k][e] - m[0];
                        sum[0] += (crank * 256 + t + k * 256 * CL < nvec) ? __expf(a) : 0.f;
                        v[k][e] = a;
                    }
                }
            cluster_reduce_n<CL, false, 1>(sum, sm, xch, slot);
            const float ls = logf(sum[0]), inv = 1.0f / sum[0];
#pragma unroll
            for (int k = 0; k < VPT; k++) {
                const int vi = crank * 256 + t + k * 256 * CL;
                if (vi < nvec) {
                    float o[N];
#pragma unroll
                    for (int e = 0; e < N; e++) o[e] = (OP == ROW_SOFTMAX) ? v[k][e] * inv : v[k][e] - ls;
                    Vec16<T>::store(yr + (int64_t)vi * N, o);
                }
            }
        }
    }
    cluster.sync();                     // nobody leaves while its shared memory may still be read
}

template <typename T, int CL, int OP>
static cudaError_t launch_cluster(const T* x, T* y, const float* gamma, const float* beta, int64_t rows, int cols, float eps,
                                  cudaStream_t st) {
    const int64_t fit = std::max<int64_t>(1, (int64_t)(kNumSMs - sm_reserve()) * 2 / CL);      // clusters resident at once
    const unsigned clusters = (unsigned)std::min<int64_t>(rows, fit);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(clusters * CL);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CL; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, row_cluster_kernel<T, CL, OP>, x, y, gamma, beta, rows, cols, eps);
}

// Any cols: one CTA per row, three sweeps.
template <typename T, int OP>
__global__ void __launch_bounds__(256)
row_pass_kernel(const T* __restrict__ x, T* __restrict__ y, const float* __restrict__ gamma,
                const float* __restrict__ beta, int64_t rows, int64_t cols, float eps) {
    __shared__ float sm[8];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + row * cols;
        T* yr = y + row * cols;
        if constexpr (OP == ROW_LAYERNORM) {
            float s1 = 0.f, s2 = 0.f;
            for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) { float a = ld1<T>(xr + c); s1 += a; s2 += a * a; }
            s1 = group_reduce<256, false>(s1, sm);
            s2 = group_reduce<256, false>(s2, sm);
            const float rc = 1.0f / (float)cols;
            const float mean = s1 * rc, m2 = s2 * rc;
            const float var = fmaxf(m2 - mean * mean, 0.f);
            for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
                const float w = (gamma ? gamma[c] : 1.f) / sqrtf(var + eps);
                const float b = (beta ? beta[c] : 0.f) - mean * w;
                st1<T>(yr + c, ld1<T>(xr + c) * w + b);
            }
        } else {
            float m = -FLT_MAX;
            for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, ld1<T>(xr + c));
            m = group_reduce<256, true>(m, sm);
            float s = 0.f;
            for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) s += expf(ld1<T>(xr + c) - m);
            s = group_reduce<256, false>(s, sm);
            const float ls = logf(s);
            for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
                const float a = ld1<T>(xr + c) - m;
                st1<T>(yr + c, OP == ROW_SOFTMAX ? expf(a) / s : a - ls);
            }
        }
        __syncthreads();
    }
}

// B200JT_ROW_CLUSTER=0 sends long rows to the three-sweep kernel instead (for comparison)
static bool cluster_rows_enabled() {
    const char* e = getenv("B200JT_ROW_CLUSTER");
    return !(e && e[0] == '0');
}

template <typename T, int OP>
static int launch_rows(const T* x, T* y, const float* gamma, const float* beta, int64_t rows, int64_t cols,
                       float eps, cudaStream_t st) {
    constexpr int N = Vec16<T>::N;
    const bool vec_ok = cols % N == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)y % 16 == 0);
    const int64_t nvec = cols / N;
#define B200JT_ROW(GROUP, VPT)                                                                      \
    do { const int rpc = 256 / GROUP;                                                               \
         int64_t ctas = (rows + rpc - 1) / rpc;                                                     \
         unsigned grid = (unsigned)(ctas < (int64_t)kNumSMs * 16 ? ctas : (int64_t)kNumSMs * 16);   \
         row_reg_kernel<T, GROUP, VPT, OP><<<grid, 256, 0, st>>>(x, y, gamma, beta, rows, (int)cols, eps); } while (0)
    if (vec_ok && nvec <= 32 * 8) {
        if (nvec <= 32) B200JT_ROW(32, 1);
        else if (nvec <= 64) B200JT_ROW(32, 2);
        else if (nvec <= 128) B200JT_ROW(32, 4);
        else B200JT_ROW(32, 8);
    } else if (vec_ok && nvec <= 256 * 8) {
        if (nvec <= 256) B200JT_ROW(256, 1);
        else if (nvec <= 512) B200JT_ROW(256, 2);
        else if (nvec <= 1024) B200JT_ROW(256, 4);
        else B200JT_ROW(256, 8);
    } else if (vec_ok && nvec <= 256 * 8 * 8 && rows > 0 && cluster_rows_enabled()) {
        // a cluster of 2 / 4 / 8 CTAs per row
        cudaError_t e;
        if (nvec <= 256 * 8 * 2) e = launch_cluster<T, 2, OP>(x, y, gamma, beta, rows, (int)cols, eps, st);
        else if (nvec <= 256 * 8 * 4) e = launch_cluster<T, 4, OP>(x, y, gamma, beta, rows, (int)cols, eps, st);
        else e = launch_cluster<T, 8, OP>(x, y, gamma, beta, rows, (int)cols, eps, st);
        B200JT_CUDA(e);
    } else {
        unsigned grid = (unsigned)(rows < (int64_t)kNumSMs * 16 ? rows : (int64_t)kNumSMs * 16);
        row_pass_kernel<T, OP><<<grid, 256, 0, st>>>(x, y, gamma, beta, rows, cols, eps);
    }
#undef B200JT_ROW
    B200JT_LAUNCH_CHECK();
    return 0;
}


// ---- softmax backward ----------------------------------------------------------------------------------------------
// dx = y * (dy - sum(y * dy))   for y = softmax(x),      dx = dy - exp(y) * sum(dy)   for y = log_softmax(x),
// the two reductions of the reference's hand-written backward (python/jittor/other/code_softmax.py:109-147). The row of y
// and of dy live in registers: one read of each, one write of dx.
template <typename T, int GROUP, int VPT, bool LOG>
__global__ void __launch_bounds__(256)
softmax_bwd_reg_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx, int64_t rows, int cols) {
    constexpr int N = Vec16<T>::N;
    constexpr int ROWS_PER_CTA = 256 / GROUP;
    __shared__ float sm[32];
    const int g = threadIdx.x / GROUP, t = threadIdx.x % GROUP;
    const int nvec = cols / N;
    for (int64_t row = (int64_t)blockIdx.x * ROWS_PER_CTA + g; ; row += (int64_t)gridDim.x * ROWS_PER_CTA) {
        // the CTA-wide reduction has a barrier inside: rows are taken in rounds the whole CTA goes through together
        const int64_t round0 = row - g;
        if (round0 >= rows) break;
        const bool live = row < rows;
        float a[VPT][N], b[VPT][N];
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int vi = t + k * GROUP;
            if (live && vi < nvec) {
                Vec16<T>::load(y + row * cols + (int64_t)vi * N, a[k]);
                Vec16<T>::load(dy + row * cols + (int64_t)vi * N, b[k]);
#pragma unroll
                for (int e = 0; e < N; e++) s += LOG ? b[k][e] : a[k][e] * b[k][e];
            }
        }
        s = group_reduce<GROUP, false>(s, sm);
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int vi = t + k * GROUP;
            if (live && vi < nvec) {
                float o[N];
#pragma unroll
                for (int e = 0; e < N; e++) o[e] = LOG ? b[k][e] - expf(a[k][e]) * s : a[k][e] * (b[k][e] - s);
                Vec16<T>::store(dx + row * cols + (int64_t)vi * N, o);
            }
        }
    }
}

// any cols / alignment: two sweeps by one CTA per row
template <typename T, bool LOG>
__global__ void __launch_bounds__(256)
softmax_bwd_pass_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx, int64_t rows, int64_t cols) {
    __shared__ float sm[32];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* yr = y + row * cols; const T* dr = dy + row * cols; T* xr = dx + row * cols;
        float s = 0.f;
        for (int64_t c = threadIdx.x; c < cols; c += 256) s += LOG ? ld1<T>(dr + c) : ld1<T>(yr + c) * ld1<T>(dr + c);
        s = group_reduce<256, false>(s, sm);
        for (int64_t c = threadIdx.x; c < cols; c += 256) {
            const float a = ld1<T>(yr + c), b = ld1<T>(dr + c);
            st1<T>(xr + c, LOG ? b - expf(a) * s : a * (b - s));
        }
    }
}

template <typename T, bool LOG>
static int launch_softmax_bwd(const T* y, const T* dy, T* dx, int64_t rows, int64_t cols, cudaStream_t st) {
    constexpr int N = Vec16<T>::N;
    const bool vec_ok = cols % N == 0 && ((uintptr_t)y % 16 == 0) && ((uintptr_t)dy % 16 == 0) && ((uintptr_t)dx % 16 == 0);
    const int64_t nvec = cols / N;
#define B200JT_SB(GROUP, VPT)                                                                       \
    do { const int rpc = 256 / GROUP;                                                               \
         int64_t ctas = (rows + rpc - 1) / rpc;                                                     \
         unsigned grid = (unsigned)(ctas < (int64_t)kNumSMs * 16 ? ctas : (int64_t)kNumSMs * 16);   \
         softmax_bwd_reg_kernel<T, GROUP, VPT, LOG><<<grid, 256, 0, st>>>(y, dy, dx, rows, (int)cols); } while (0)
    if (vec_ok && nvec <= 32 * 4) {
        if (nvec <= 32) B200JT_SB(32, 1);
        else if (nvec <= 64) B200JT_SB(32, 2);
        else B200JT_SB(32, 4);
    } else if (vec_ok && nvec <= 256 * 4) {
        if (nvec <= 256) B200JT_SB(256, 1);
        else if (nvec <= 512) B200JT_SB(256, 2);
        else B200JT_SB(256, 4);
    } else {
        unsigned grid = (unsigned)(rows < (int64_t)kNumSMs * 16 ? rows : (int64_t)kNumSMs * 16);
        softmax_bwd_pass_kernel<T, LOG><<<grid, 256, 0, st>>>(y, dy, dx, rows, cols);
    }
#undef B200JT_SB
    B200JT_LAUNCH_CHECK();
    return 0;
}

static int rows_cols(const b200jt_tensor* x, const b200jt_tensor* y, int64_t* rows, int64_t* cols) {
    B200JT_CHECK_ARG(valid_tensor(x) && valid_tensor(y), "invalid tensor descriptor");
    B200JT_CHECK_ARG(x->dtype == y->dtype && (x->dtype == B200JT_FLOAT32 || x->dtype == B200JT_BFLOAT16),
                     "x and y must both be float32 or bfloat16");
    B200JT_CHECK_ARG(numel(x) == numel(y), "x and y differ in size");
    *cols = x->shape[x->ndim - 1];
    *rows = *cols ? numel(x) / *cols : 0;
    return 0;
}

}  // namespace b200jt

using namespace b200jt;

extern "C" int b200jt_softmax(const b200jt_tensor* x, const b200jt_tensor* y, int log, void* stream) {
    int64_t rows, cols;
    int rc = rows_cols(x, y, &rows, &cols);
    if (rc) return rc;
    if (rows == 0 || cols == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (x->dtype == B200JT_FLOAT32) {
        return log ? launch_rows<float, ROW_LOG_SOFTMAX>((const float*)x->ptr, (float*)y->ptr, nullptr, nullptr, rows, cols, 0.f, st)
                   : launch_rows<float, ROW_SOFTMAX>((const float*)x->ptr, (float*)y->ptr, nullptr, nullptr, rows, cols, 0.f, st);
    }
    return log ? launch_rows<__nv_bfloat16, ROW_LOG_SOFTMAX>((const __nv_bfloat16*)x->ptr, (__nv_bfloat16*)y->ptr, nullptr, nullptr, rows, cols, 0.f, st)
               : launch_rows<__nv_bfloat16, ROW_SOFTMAX>((const __nv_bfloat16*)x->ptr, (__nv_bfloat16*)y->ptr, nullptr, nullptr, rows, cols, 0.f, st);
}

extern "C" int b200jt_softmax_backward(const b200jt_tensor* y, const b200jt_tensor* dy, const b200jt_tensor* dx, int log, void* stream) {
    int64_t rows, cols;
    int rc = rows_cols(y, dx, &rows, &cols);
    if (rc) return rc;
    B200JT_CHECK_ARG(valid_tensor(dy) && dy->dtype == y->dtype && numel(dy) == numel(y), "dy must have y's dtype and size");
    if (rows == 0 || cols == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (y->dtype == B200JT_FLOAT32) {
        return log ? launch_softmax_bwd<float, true>((const float*)y->ptr, (const float*)dy->ptr, (float*)dx->ptr, rows, cols, st)
                   : launch_softmax_bwd<float, false>((const float*)y->ptr, (const float*)dy->ptr, (float*)dx->ptr, rows, cols, st);
    }
    using B = __nv_bfloat16;
    return log ? launch_softmax_bwd<B, true>((const B*)y->ptr, (const B*)dy->ptr, (B*)dx->ptr, rows, cols, st)
               : launch_softmax_bwd<B, false>((const B*)y->ptr, (const B*)dy->ptr, (B*)dx->ptr, rows, cols, st);
}

extern "C" int b200jt_layer_norm(const b200jt_tensor* x, const b200jt_tensor* gamma, const b200jt_tensor* beta,
                                 const b200jt_tensor* y, double eps, void* stream) {
    int64_t rows, cols;
    int rc = rows_cols(x, y, &rows, &cols);
    if (rc) return rc;
    const float* g = nullptr; const float* b = nullptr;
    if (gamma) {
        B200JT_CHECK_ARG(valid_tensor(gamma) && gamma->dtype == B200JT_FLOAT32 && numel(gamma) == cols, "gamma must be float32 [cols]");
        g = (const float*)gamma->ptr;
    }
    if (beta) {
        B200JT_CHECK_ARG(valid_tensor(beta) && beta->dtype == B200JT_FLOAT32 && numel(beta) == cols, "beta must be float32 [cols]");
        b = (const float*)beta->ptr;
    }
    if (rows == 0 || cols == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (x->dtype == B200JT_FLOAT32)
        return launch_rows<float, ROW_LAYERNORM>((const float*)x->ptr, (float*)y->ptr, g, b, rows, cols, (float)eps, st);
    return launch_rows<__nv_bfloat16, ROW_LAYERNORM>((const __nv_bfloat16*)x->ptr, (__nv_bfloat16*)y->ptr, g, b, rows, cols, (float)eps, st);
}
