// CUDA-core contraction used where the result must match fp32 arithmetic to 1e-5 (float32 inputs) or the
// shape does not fit the tcgen05 tiles: broadcast-multiply-sum matmul and the reindex-lowered conv2d as an
// implicit GEMM (M = N*OH*OW pixels, N = Cout, K = Cin*KH*KW), both with fp32 accumulation in ascending k,
// the order of the reference's fused loop nest (python/jittor/nn.py:1009-1017: sum over [Cin, Kh, Kw]).
// 64x64x16 tiles, 256 threads, 4x4 outputs per thread, operands staged in shared memory.
#include "gemm_simt.cuh"

namespace b200jt {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

struct MatmulLoader {
    int64_t a_sm, a_sk, b_sk, b_sn, c_sm;
    template <typename T> __device__ __forceinline__ float A(const T* a, int64_t m, int64_t k) const { return to_f<T>(a[m * a_sm + k * a_sk]); }
    template <typename T> __device__ __forceinline__ float B(const T* b, int64_t k, int64_t n) const { return to_f<T>(b[k * b_sk + n * b_sn]); }
    __device__ __forceinline__ int64_t C(int64_t m, int64_t n) const { return m * c_sm + n; }
};

struct ConvLoader {
    int C_, H, W, Co, KH, KW, OH, OW, sh, sw, ph, pw, dh, dw;
    template <typename T> __device__ __forceinline__ float A(const T* x, int64_t m, int64_t k) const {
        const int ow = (int)(m % OW); int64_t t = m / OW;
        const int oh = (int)(t % OH); const int64_t n = t / OH;
        const int kw = (int)(k % KW); int t2 = (int)(k / KW);
        const int kh = t2 % KH; const int c = t2 / KH;
        const int ih = oh * sh - ph + kh * dh, iw = ow * sw - pw + kw * dw;
        if (ih < 0 || ih >= H || iw < 0 || iw >= W) return 0.f;
        return to_f<T>(x[((n * C_ + c) * H + ih) * (int64_t)W + iw]);
    }
    template <typename T> __device__ __forceinline__ float B(const T* w, int64_t k, int64_t n) const {
        return to_f<T>(w[n * ((int64_t)C_ * KH * KW) + k]);
    }
    __device__ __forceinline__ int64_t C(int64_t m, int64_t n) const {
        const int64_t pix = m % ((int64_t)OH * OW), img = m / ((int64_t)OH * OW);
        return (img * Co + n) * ((int64_t)OH * OW) + pix;
    }
};

template <typename T, typename L>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ c,
                 int64_t M, int64_t N, int64_t K, const L ld) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;            // 16 x 16 threads, 4 x 4 outputs each
    const int64_t m0 = (int64_t)blockIdx.x * BM, n0 = (int64_t)blockIdx.y * BN;
    float acc[4][4] = {};
    for (int64_t k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            // A tile: consecutive threads walk m (the contiguous axis of NCHW pixels)
            const int e = tid + i * 256;
            const int mm = e % BM, kk = e / BM;
            const int64_t m = m0 + mm, k = k0 + kk;
            As[kk][mm] = (m < M && k < K) ? ld.template A<T>(a, m, k) : 0.f;
            const int nn = e % BN, kb = e / BN;
            const int64_t n = n0 + nn, k2 = k0 + kb;
            Bs[kb][nn] = (n < N && k2 < K) ? ld.template B<T>(b, k2, n) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { av[i] = As[kk][ty * 4 + i]; bv[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int64_t m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int64_t n = n0 + tx * 4 + j;
            if (n < N) c[ld.C(m, n)] = from_f<T>(acc[i][j]);
        }
    }
}

int matmul_simt(const void* a, const void* b, void* c, int dtype, int64_t M, int64_t N, int64_t K,
                bool trans_a, bool trans_b, cudaStream_t st) {
    MatmulLoader L;
    L.a_sm = trans_a ? 1 : K; L.a_sk = trans_a ? M : 1;
    L.b_sk = trans_b ? 1 : N; L.b_sn = trans_b ? K : 1;
    L.c_sm = N;
    dim3 grid((unsigned)((M + BM - 1) / BM), (unsigned)((N + BN - 1) / BN));
    if (dtype == B200JT_FLOAT32)
        gemm_simt_kernel<float, MatmulLoader><<<grid, 256, 0, st>>>((const float*)a, (const float*)b, (float*)c, M, N, K, L);
    else
        gemm_simt_kernel<__nv_bfloat16, MatmulLoader><<<grid, 256, 0, st>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)c, M, N, K, L);
    B200JT_LAUNCH_CHECK();
    return 0;
}

int conv2d_simt(const void* x, const void* w, void* y, int dtype, const ConvShape& s, cudaStream_t st) {
    ConvLoader L{s.C, s.H, s.W, s.Co, s.KH, s.KW, s.OH, s.OW, s.sh, s.sw, s.ph, s.pw, s.dh, s.dw};
    const int64_t M = (int64_t)s.N * s.OH * s.OW, N = s.Co, K = (int64_t)s.C * s.KH * s.KW;
    dim3 grid((unsigned)((M + BM - 1) / BM), (unsigned)((N + BN - 1) / BN));
    if (dtype == B200JT_FLOAT32)
        gemm_simt_kernel<float, ConvLoader><<<grid, 256, 0, st>>>((const float*)x, (const float*)w, (float*)y, M, N, K, L);
    else
        gemm_simt_kernel<__nv_bfloat16, ConvLoader><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, M, N, K, L);
    B200JT_LAUNCH_CHECK();
    return 0;
}

}  // namespace b200jt
