// CUDA-core contraction used where the result must match fp32 arithmetic to 1e-5 (float32 inputs) or the
// shape does not fit the tcgen05 tiles: broadcast-multiply-sum matmul and the reindex-lowered conv2d as an
// implicit GEMM (M = N*OH*OW pixels, N = Cout, K = Cin*KH*KW), both with fp32 accumulation in ascending k,
// the order of the reference's fused loop nest (python/jittor/nn.py:1009-1017: sum over [Cin, Kh, Kw]).
// 64x64x16 tiles, 256 threads, 4x4 outputs per thread, operands staged in shared memory.
#include "gemm_simt.cuh"

#include <algorithm>

namespace b200jt {

constexpr int BK = 16;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

// A loader describes the two operands as functions A(m, k), B(k, n) and the output offset C(m, n). The part of the
// address that depends only on the row m is computed once per thread (Row) because a thread stages the same rows of
// the A tile in every k step.
struct MatmulLoader {
    static constexpr bool kTable = false;
    int64_t a_sm, a_sk, b_sk, b_sn, c_sm;
    struct Row { int64_t off; };
    __device__ __forceinline__ Row row(int64_t m) const { return Row{m * a_sm}; }
    template <typename T> __device__ __forceinline__ float A(const T* a, const Row& r, int64_t k) const { return to_f<T>(a[r.off + k * a_sk]); }
    template <typename T> __device__ __forceinline__ float B(const T* b, int64_t k, int64_t n) const { return to_f<T>(b[k * b_sk + n * b_sn]); }
    __device__ __forceinline__ int64_t C(int64_t m, int64_t n) const { return m * c_sm + n; }
    __device__ __forceinline__ int64_t a_group(int) const { return 0; }
    __device__ __forceinline__ int64_t b_group(int) const { return 0; }
    __device__ __forceinline__ int64_t c_group(int) const { return 0; }
};

// Strided-batched matmul: blockIdx.z is the batch index; a batch stride of 0 shares that operand between all products.
struct BatchedMatmulLoader : MatmulLoader {
    int64_t a_bs, b_bs, c_bs;
    __device__ __forceinline__ int64_t a_group(int g) const { return (int64_t)g * a_bs; }
    __device__ __forceinline__ int64_t b_group(int g) const { return (int64_t)g * b_bs; }
    __device__ __forceinline__ int64_t c_group(int g) const { return (int64_t)g * c_bs; }
};

// Grouped convolution: blockIdx.z is the group; C_ / Co are the channels of ONE group, Ct / CoT those of the tensors.
struct ConvLoader {
    int C_, Ct, H, W, Co, CoT, KH, KW, OH, OW, sh, sw, ph, pw, dh, dw;
    struct Row { int64_t base; int ih0, iw0; };          // image base offset and top-left input coordinate of the window
    __device__ __forceinline__ Row row(int64_t m) const {
        const int ow = (int)(m % OW); const int64_t t = m / OW;
        const int oh = (int)(t % OH); const int64_t n = t / OH;
        return Row{n * Ct * (int64_t)H * W, oh * sh - ph, ow * sw - pw};
    }
    template <typename T> __device__ __forceinline__ float A(const T* x, const Row& r, int64_t k) const {
        const int k32 = (int)k;                                         // K = C*KH*KW of one group: always below 2^31
        const int kw = k32 % KW; const int t2 = k32 / KW;
        const int kh = t2 % KH; const int c = t2 / KH;
        const int ih = r.ih0 + kh * dh, iw = r.iw0 + kw * dw;
        if (ih < 0 || ih >= H || iw < 0 || iw >= W) return 0.f;
        return to_f<T>(x[r.base + ((int64_t)c * H + ih) * W + iw]);
    }
    // The part of A's address that depends only on k, computed once per CTA and k by the deep-staging kernel.
    static constexpr bool kTable = true;
    struct KEntry { int plane; short dih, diw; };                       // c*H*W (a group's planes stay below 2^31 elements), kh*dh, kw*dw
    __device__ __forceinline__ KEntry kentry(int k) const {
        const int kw = k % KW; const int t2 = k / KW;
        const int kh = t2 % KH; const int c = t2 / KH;
        return KEntry{c * H * W, (short)(kh * dh), (short)(kw * dw)};
    }
    template <typename T> __device__ __forceinline__ float A_tab(const T* x, const Row& r, const KEntry& e) const {
        const int ih = r.ih0 + e.dih, iw = r.iw0 + e.diw;
        if ((unsigned)ih >= (unsigned)H || (unsigned)iw >= (unsigned)W) return 0.f;
        return to_f<T>(x[r.base + e.plane + ih * W + iw]);
    }
    template <typename T> __device__ __forceinline__ float B(const T* w, int64_t k, int64_t n) const {
        return to_f<T>(w[n * ((int64_t)C_ * KH * KW) + k]);
    }
    __device__ __forceinline__ int64_t C(int64_t m, int64_t n) const {
        const int64_t pix = m % ((int64_t)OH * OW), img = m / ((int64_t)OH * OW);
        return (img * CoT + n) * ((int64_t)OH * OW) + pix;
    }
    __device__ __forceinline__ int64_t a_group(int g) const { return (int64_t)g * C_ * H * W; }
    __device__ __forceinline__ int64_t b_group(int g) const { return (int64_t)g * Co * ((int64_t)C_ * KH * KW); }
    __device__ __forceinline__ int64_t c_group(int g) const { return (int64_t)g * Co * ((int64_t)OH * OW); }
};

// Transposed convolution in gather form: y[n,o,ho,wo] = sum over (i,kh,kw) of x[n,i,(ho+ph-kh*dh)/sh,(wo+pw-kw*dw)/sw] *
// w[i,o,kh,kw] wherever the divisions are exact and in range (the scatter of python/jittor/nn.py:1437-1449 read from
// the output side). M = N*OH*OW output pixels, N = out channels of a group, K = (in channels of a group)*KH*KW.
struct ConvTLoader {
    static constexpr bool kTable = false;
    int Ci, CiT, H, W, Co, CoT, KH, KW, OH, OW, sh, sw, ph, pw, dh, dw;   // H, W: input extent; OH, OW: output extent
    struct Row { int64_t base; int oh, ow; };
    __device__ __forceinline__ Row row(int64_t m) const {
        const int ow = (int)(m % OW); const int64_t t = m / OW;
        const int oh = (int)(t % OH); const int64_t n = t / OH;
        return Row{n * CiT * (int64_t)H * W, oh + ph, ow + pw};
    }
    template <typename T> __device__ __forceinline__ float A(const T* x, const Row& r, int64_t k) const {
        const int kw = (int)(k % KW); const int t2 = (int)(k / KW);
        const int kh = t2 % KH; const int c = t2 / KH;
        const int a = r.oh - kh * dh, b = r.ow - kw * dw;
        if (a < 0 || b < 0 || a % sh || b % sw) return 0.f;
        const int ih = a / sh, iw = b / sw;
        if (ih >= H || iw >= W) return 0.f;
        return to_f<T>(x[r.base + ((int64_t)c * H + ih) * W + iw]);
    }
    template <typename T> __device__ __forceinline__ float B(const T* w, int64_t k, int64_t n) const {
        const int64_t taps = (int64_t)KH * KW;
        const int64_t c = k / taps, tap = k - c * taps;
        return to_f<T>(w[(c * Co + n) * taps + tap]);                  // w[i][o within group][kh][kw]
    }
    __device__ __forceinline__ int64_t C(int64_t m, int64_t n) const {
        const int64_t pix = m % ((int64_t)OH * OW), img = m / ((int64_t)OH * OW);
        return (img * CoT + n) * ((int64_t)OH * OW) + pix;
    }
    __device__ __forceinline__ int64_t a_group(int g) const { return (int64_t)g * Ci * H * W; }
    __device__ __forceinline__ int64_t b_group(int g) const { return (int64_t)g * Ci * Co * ((int64_t)KH * KW); }
    __device__ __forceinline__ int64_t c_group(int g) const { return (int64_t)g * Co * ((int64_t)OH * OW); }
};

// Weight gradient of the convolution: dw[o,c,kh,kw] = sum over (n,oh,ow) of dy[n,o,oh,ow] * x[n,c,oh*sh-ph+kh*dh,ow*sw-pw+kw*dw]
// (the reduce over [0,3,4] of reindex(x) * broadcast(dy) that the reduce / broadcast gradient rules produce).
// M = Cout, N = Cin*KH*KW, K = batch*OH*OW, accumulated in ascending k.
struct ConvWgradLoader {
    static constexpr bool kTable = false;
    int Ci, H, W, Co, KH, KW, OH, OW, sh, sw, ph, pw, dh, dw;
    struct Row { int64_t off; };
    __device__ __forceinline__ Row row(int64_t m) const { return Row{m * (int64_t)OH * OW}; }
    template <typename T> __device__ __forceinline__ float A(const T* dy, const Row& r, int64_t k) const {
        const int64_t pix = k % ((int64_t)OH * OW), n = k / ((int64_t)OH * OW);
        return to_f<T>(dy[n * Co * (int64_t)OH * OW + r.off + pix]);
    }
    template <typename T> __device__ __forceinline__ float B(const T* x, int64_t k, int64_t n2) const {
        const int ow = (int)(k % OW); const int64_t t = k / OW;
        const int oh = (int)(t % OH); const int64_t img = t / OH;
        const int kw = (int)(n2 % KW); const int t2 = (int)(n2 / KW);
        const int kh = t2 % KH; const int c = t2 / KH;
        const int ih = oh * sh - ph + kh * dh, iw = ow * sw - pw + kw * dw;
        if (ih < 0 || ih >= H || iw < 0 || iw >= W) return 0.f;
        return to_f<T>(x[((img * Ci + c) * H + ih) * (int64_t)W + iw]);
    }
    __device__ __forceinline__ int64_t C(int64_t m, int64_t n2) const { return m * ((int64_t)Ci * KH * KW) + n2; }
    __device__ __forceinline__ int64_t a_group(int) const { return 0; }
    __device__ __forceinline__ int64_t b_group(int) const { return 0; }
    __device__ __forceinline__ int64_t c_group(int) const { return 0; }
};

// TM x TN output tile per CTA of 256 threads (16 x 16), (TM/16) x (TN/16) outputs per thread.
template <typename T, typename L, int TM, int TN>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ c,
                 int64_t M, int64_t N, int64_t K, const L ld) {
    constexpr int RM = TM / 16, RN = TN / 16;
    constexpr int LA = TM * BK / 256, LB = TN * BK / 256;         // staged elements per thread
    a += ld.a_group(blockIdx.z); b += ld.b_group(blockIdx.z); c += ld.c_group(blockIdx.z);
    __shared__ float As[BK][TM + 4];
    __shared__ float Bs[BK][TN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int64_t m0 = (int64_t)blockIdx.x * TM, n0 = (int64_t)blockIdx.y * TN;
    // consecutive threads walk m (the contiguous axis of NCHW pixels); a thread keeps its row across k steps
    const int a_mm = tid % TM, a_k0 = tid / TM;
    const int64_t a_m = m0 + a_mm;
    const typename L::Row arow = ld.row(a_m < M ? a_m : 0);
    const int b_nn = tid % TN, b_k0 = tid / TN;
    float acc[RM][RN] = {};
    for (int64_t k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < LA; i++) {
            const int kk = a_k0 + i * (256 / TM);
            const int64_t k = k0 + kk;
            As[kk][a_mm] = (a_m < M && k < K) ? ld.template A<T>(a, arow, k) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < LB; i++) {
            const int kb = b_k0 + i * (256 / TN);
            const int64_t n = n0 + b_nn, k2 = k0 + kb;
            Bs[kb][b_nn] = (n < N && k2 < K) ? ld.template B<T>(b, k2, n) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float av[RM], bv[RN];
#pragma unroll
            for (int i = 0; i < RM; i++) av[i] = As[kk][ty * RM + i];
#pragma unroll
            for (int j = 0; j < RN; j++) bv[j] = Bs[kk][tx * RN + j];
#pragma unroll
            for (int i = 0; i < RM; i++)
#pragma unroll
                for (int j = 0; j < RN; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < RM; i++) {
        const int64_t m = m0 + ty * RM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < RN; j++) {
            const int64_t n = n0 + tx * RN + j;
            if (n < N) c[ld.C(m, n)] = from_f<T>(acc[i][j]);
        }
    }
}

// Small problems (fewer tiles than two waves of CTAs) are bound by the latency of the k loop above, not by its arithmetic:
// every 16-deep step costs a trip to memory and two barriers. This form stages KC = 320 k values of both operands at
// once -- each thread issues its loads in batches of 8 per operand before it stores any of them, so a CTA pays a few
// memory latencies per 320 k instead of one per 16 -- and then runs the same ascending-k FMA sequence over the staged
// slab (same bits as the kernel above).
constexpr int KC = 320;

template <typename L, bool HAS> struct KTab { struct Entry { int unused; }; };
template <typename L> struct KTab<L, true> { using Entry = typename L::KEntry; };

template <typename T, typename L, int TM, int TN>
__global__ void __launch_bounds__(256)
gemm_simt_deep_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ c,
                      int64_t M, int64_t N, int64_t K, const L ld) {
    // PIX (the convolution forward): A and C are contiguous along m (pixels), B along k (a filter's taps). Then threads
    // walk m when they stage A and store C, walk k when they stage B (kept n-major in shared memory), and in the FMA
    // loop tx picks the rows and ty the columns, so every global access is coalesced and every shared access is either
    // conflict-free or a broadcast. Otherwise (matmul: C contiguous along n) tx picks the columns.
    constexpr bool PIX = L::kTable;
    constexpr int RM = TM / 16, RN = TN / 16, PA = TM + 4, PB = PIX ? KC + 4 : TN + 4;
    constexpr int KA = 256 / TM, KB = 256 / TN;                    // k values staged per pass of the CTA
    constexpr int U = 8;
    extern __shared__ float deep_smem[];
    float* As = deep_smem;                                          // [KC][PA]
    float* Bs = deep_smem + KC * PA;                                // [KC][PB], or for PIX [TN][PB] with PB = KC + 4
    a += ld.a_group(blockIdx.z); b += ld.b_group(blockIdx.z); c += ld.c_group(blockIdx.z);
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int64_t m0 = (int64_t)blockIdx.x * TM, n0 = (int64_t)blockIdx.y * TN;
    const int a_mm = tid % TM, a_k0 = tid / TM;
    const int64_t a_m = m0 + a_mm;
    const typename L::Row arow = ld.row(a_m < M ? a_m : 0);
    const int b_nn = tid % TN, b_k0 = tid / TN;
    const int64_t b_n = n0 + b_nn;
    float acc[RM][RN] = {};
    [[maybe_unused]] __shared__ typename KTab<L, L::kTable>::Entry ktab[L::kTable ? KC : 1];
    for (int64_t k0 = 0; k0 < K; k0 += KC) {
        const int kc = (int)(K - k0 < KC ? K - k0 : KC);
        if constexpr (L::kTable) {
            // the divisions that split k into (channel, kh, kw) are done once per k and CTA, not once per staged element
            for (int kk = tid; kk < kc; kk += 256) ktab[kk] = ld.kentry((int)k0 + kk);
            __syncthreads();
        }
        if constexpr (PIX) {
            for (int base = 0; base < kc; base += U * KA) {
                float r[U];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int kk = base + a_k0 + u * KA;
                    r[u] = (a_m < M && kk < kc) ? ld.template A_tab<T>(a, arow, ktab[kk]) : 0.f;
                }
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int kk = base + a_k0 + u * KA;
                    if (kk < kc) As[kk * PA + a_mm] = r[u];
                }
            }
            // B: a warp takes one filter row at a time and walks its taps
            const int lane = tid % 32, wid = tid / 32;
            for (int nn = wid; nn < TN; nn += 8) {
                const int64_t n = n0 + nn;
                for (int base = 0; base < kc; base += U * 32) {
                    float r[U];
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        const int kk = base + lane + u * 32;
                        r[u] = (n < N && kk < kc) ? ld.template B<T>(b, k0 + kk, n) : 0.f;
                    }
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        const int kk = base + lane + u * 32;
                        if (kk < kc) Bs[nn * PB + kk] = r[u];
                    }
                }
            }
        } else {
            for (int base = 0; base < kc; base += U * KA) {
                float r[U];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int kk = base + a_k0 + u * KA;
                    r[u] = (a_m < M && kk < kc) ? ld.template A<T>(a, arow, k0 + kk) : 0.f;
                }
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int kk = base + a_k0 + u * KA;
                    if (kk < kc) As[kk * PA + a_mm] = r[u];
                }
            }
            for (int base = 0; base < kc; base += U * KB) {
                float r[U];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int kk = base + b_k0 + u * KB;
                    r[u] = (b_n < N && kk < kc) ? ld.template B<T>(b, k0 + kk, b_n) : 0.f;
                }
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int kk = base + b_k0 + u * KB;
                    if (kk < kc) Bs[kk * PB + b_nn] = r[u];
                }
            }
        }
        __syncthreads();
        // rows / columns of this thread inside the tile
        const int rm = (PIX ? tx : ty) * RM, rn = (PIX ? ty : tx) * RN;
#pragma unroll 4
        for (int kk = 0; kk < kc; kk++) {
            float av[RM], bv[RN];
#pragma unroll
            for (int i = 0; i < RM; i++) av[i] = As[kk * PA + rm + i];
#pragma unroll
            for (int j = 0; j < RN; j++) bv[j] = PIX ? Bs[(rn + j) * PB + kk] : Bs[kk * PB + rn + j];
#pragma unroll
            for (int i = 0; i < RM; i++)
#pragma unroll
                for (int j = 0; j < RN; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
    const int rm = (PIX ? tx : ty) * RM, rn = (PIX ? ty : tx) * RN;
#pragma unroll
    for (int i = 0; i < RM; i++) {
        const int64_t m = m0 + rm + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < RN; j++) {
            const int64_t n = n0 + rn + j;
            if (n < N) c[ld.C(m, n)] = from_f<T>(acc[i][j]);
        }
    }
}

// 64x64 tiles when they fill the machine; small problems take 32x32 tiles (more CTAs in flight) with the deep staging.
template <typename T, typename L>
static void launch_simt(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K, const L& ld, cudaStream_t st,
                        int groups = 1) {
    const int64_t big = ((M + 63) / 64) * ((N + 63) / 64) * groups;
    if (big >= 2 * kNumSMs && N > 32) {
        dim3 grid((unsigned)((M + 63) / 64), (unsigned)((N + 63) / 64), (unsigned)groups);
        gemm_simt_kernel<T, L, 64, 64><<<grid, 256, 0, st>>>((const T*)a, (const T*)b, (T*)c, M, N, K, ld);
    } else {
        dim3 grid((unsigned)((M + 31) / 32), (unsigned)((N + 31) / 32), (unsigned)groups);
        constexpr int smem = (KC * (32 + 4) + (L::kTable ? 32 * (KC + 4) : KC * (32 + 4))) * (int)sizeof(float);
        static const cudaError_t attr = cudaFuncSetAttribute(gemm_simt_deep_kernel<T, L, 32, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (attr == cudaSuccess && K >= 64)
            gemm_simt_deep_kernel<T, L, 32, 32><<<grid, 256, smem, st>>>((const T*)a, (const T*)b, (T*)c, M, N, K, ld);
        else
            gemm_simt_kernel<T, L, 32, 32><<<grid, 256, 0, st>>>((const T*)a, (const T*)b, (T*)c, M, N, K, ld);
    }
}

int matmul_simt(const void* a, const void* b, void* c, int dtype, int64_t M, int64_t N, int64_t K,
                bool trans_a, bool trans_b, cudaStream_t st) {
    MatmulLoader L;
    L.a_sm = trans_a ? 1 : K; L.a_sk = trans_a ? M : 1;
    L.b_sk = trans_b ? 1 : N; L.b_sn = trans_b ? K : 1;
    L.c_sm = N;
    if (dtype == B200JT_FLOAT32) launch_simt<float, MatmulLoader>(a, b, c, M, N, K, L, st);
    else launch_simt<__nv_bfloat16, MatmulLoader>(a, b, c, M, N, K, L, st);
    B200JT_LAUNCH_CHECK();
    return 0;
}

int batched_matmul_simt(const void* a, const void* b, void* c, int dtype, int64_t batch, int64_t a_batch, int64_t b_batch,
                        int64_t M, int64_t N, int64_t K, bool trans_a, bool trans_b, cudaStream_t st) {
    BatchedMatmulLoader L;
    L.a_sm = trans_a ? 1 : K; L.a_sk = trans_a ? M : 1;
    L.b_sk = trans_b ? 1 : N; L.b_sn = trans_b ? K : 1;
    L.c_sm = N;
    L.a_bs = a_batch > 1 ? M * K : 0; L.b_bs = b_batch > 1 ? K * N : 0; L.c_bs = M * N;
    const size_t es = dtype == B200JT_FLOAT32 ? 4 : 2;
    for (int64_t b0 = 0; b0 < batch; b0 += 32768) {                 // grid.z is limited to 65535
        const int g = (int)std::min<int64_t>(32768, batch - b0);
        const char* ap = (const char*)a + (size_t)(b0 * L.a_bs) * es;
        const char* bp = (const char*)b + (size_t)(b0 * L.b_bs) * es;
        char* cp = (char*)c + (size_t)(b0 * L.c_bs) * es;
        if (dtype == B200JT_FLOAT32) launch_simt<float, BatchedMatmulLoader>(ap, bp, cp, M, N, K, L, st, g);
        else launch_simt<__nv_bfloat16, BatchedMatmulLoader>(ap, bp, cp, M, N, K, L, st, g);
    }
    B200JT_LAUNCH_CHECK();
    return 0;
}

int conv2d_simt(const void* x, const void* w, void* y, int dtype, const ConvShape& s, cudaStream_t st) {
    const int G = s.groups > 0 ? s.groups : 1;
    ConvLoader L{s.C / G, s.C, s.H, s.W, s.Co / G, s.Co, s.KH, s.KW, s.OH, s.OW, s.sh, s.sw, s.ph, s.pw, s.dh, s.dw};
    const int64_t M = (int64_t)s.N * s.OH * s.OW, N = s.Co / G, K = (int64_t)(s.C / G) * s.KH * s.KW;
    if (dtype == B200JT_FLOAT32) launch_simt<float, ConvLoader>(x, w, y, M, N, K, L, st, G);
    else launch_simt<__nv_bfloat16, ConvLoader>(x, w, y, M, N, K, L, st, G);
    B200JT_LAUNCH_CHECK();
    return 0;
}

// s: C/H/W describe the INPUT x, Co/OH/OW the OUTPUT y of the transposed convolution.
int conv2d_transpose_simt(const void* x, const void* w, void* y, int dtype, const ConvShape& s, cudaStream_t st) {
    const int G = s.groups > 0 ? s.groups : 1;
    ConvTLoader L{s.C / G, s.C, s.H, s.W, s.Co / G, s.Co, s.KH, s.KW, s.OH, s.OW, s.sh, s.sw, s.ph, s.pw, s.dh, s.dw};
    const int64_t M = (int64_t)s.N * s.OH * s.OW, N = s.Co / G, K = (int64_t)(s.C / G) * s.KH * s.KW;
    if (dtype == B200JT_FLOAT32) launch_simt<float, ConvTLoader>(x, w, y, M, N, K, L, st, G);
    else launch_simt<__nv_bfloat16, ConvTLoader>(x, w, y, M, N, K, L, st, G);
    B200JT_LAUNCH_CHECK();
    return 0;
}

// dw = wgrad(x, dy); s describes the forward convolution (C = in channels, Co = out channels, OH/OW = dy's extent).
int conv2d_backward_w_simt(const void* x, const void* dy, void* dw, int dtype, const ConvShape& s, cudaStream_t st) {
    ConvWgradLoader L{s.C, s.H, s.W, s.Co, s.KH, s.KW, s.OH, s.OW, s.sh, s.sw, s.ph, s.pw, s.dh, s.dw};
    const int64_t M = s.Co, N = (int64_t)s.C * s.KH * s.KW, K = (int64_t)s.N * s.OH * s.OW;
    if (dtype == B200JT_FLOAT32) launch_simt<float, ConvWgradLoader>(dy, x, dw, M, N, K, L, st);
    else launch_simt<__nv_bfloat16, ConvWgradLoader>(dy, x, dw, M, N, K, L, st);
    B200JT_LAUNCH_CHECK();
    return 0;
}

}  // namespace b200jt
