// 2-D pooling, forward and backward: the kernels `Pool.execute` builds with jt.code in the reference
// (python/jittor/pool.py:54-95 forward body, :96-118 backward body) as fixed sm_100a kernels.
//
// Window of output (oh, ow): rows [oh*sh - ph, oh*sh - ph + kh) x columns [ow*sw - pw, ow*sw - pw + kw), clipped to the
// input (padding is never read). maximum / minimum fold the clipped window starting from the op's init value; mean
// divides the clipped sum by kh*kw (count_include_pad) or by the clipped area.
// Backward: the reference scatters with atomicAdd, one thread per window; for maximum / minimum only the FIRST element
// of the window (row-major scan) that equals the pooled value receives the gradient. Here every INPUT element gathers
// from the windows that contain it instead (at most ceil(kh/sh) * ceil(kw/sw) of them), re-deriving "am I the first
// match" by scanning the part of the window that precedes it: no atomics, no zero fill, deterministic.
#include "atomic_ops.cuh"

namespace b200jt {
namespace pool {

struct Geo {
    int N, C, H, W, OH, OW, kh, kw, sh, sw, ph, pw;
    int count_include_pad;
};

template <typename T> struct AccOf { using type = float; };
template <> struct AccOf<double> { using type = double; };

template <typename T> __device__ __forceinline__ typename AccOf<T>::type ld(const T* p) { return (typename AccOf<T>::type)(*p); }
template <> __device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <> __device__ __forceinline__ float ld<__half>(const __half* p) { return __half2float(*p); }
template <typename T, typename A> __device__ __forceinline__ T cvt(A v) { return (T)v; }
template <> __device__ __forceinline__ __nv_bfloat16 cvt<__nv_bfloat16, float>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half cvt<__half, float>(float v) { return __float2half(v); }

// OP: 0 maximum, 1 minimum, 2 mean. KS: 0 = window and stride read from the geometry record, else a compile-time
// (kernel, stride) pair code so that the window arithmetic folds to constants for the common layers:
// 1: 2x2 stride 2, 2: 3x3 stride 2, 3: 3x3 stride 1.
template <int KS> struct Win {
    __device__ __forceinline__ static int kh(const Geo& g) { return KS == 1 ? 2 : KS >= 2 ? 3 : g.kh; }
    __device__ __forceinline__ static int kw(const Geo& g) { return KS == 1 ? 2 : KS >= 2 ? 3 : g.kw; }
    __device__ __forceinline__ static int sh(const Geo& g) { return KS == 1 || KS == 2 ? 2 : KS == 3 ? 1 : g.sh; }
    __device__ __forceinline__ static int sw(const Geo& g) { return KS == 1 || KS == 2 ? 2 : KS == 3 ? 1 : g.sw; }
};

// Thread layout of both kernels: blockDim (32, 8) covers 32 columns x 8 rows of one image plane, blockIdx.z walks the
// N*C planes (grid-stride), so no division is needed to find a thread's coordinates.
template <typename T, int OP, int KS>
__global__ void __launch_bounds__(256) pool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int32_t* __restrict__ indices,
                                                       Geo g, T init) {
    using A = typename AccOf<T>::type;
    using Wn = Win<KS>;
    const int ow = blockIdx.x * 32 + threadIdx.x, oh = blockIdx.y * 8 + threadIdx.y;
    if (ow >= g.OW || oh >= g.OH) return;
    int p0 = oh * Wn::sh(g) - g.ph, q0 = ow * Wn::sw(g) - g.pw;
    const int p1 = min(p0 + Wn::kh(g), g.H), q1 = min(q0 + Wn::kw(g), g.W);
    p0 = max(p0, 0); q0 = max(q0, 0);
    const int64_t planes = (int64_t)g.N * g.C;
    for (int64_t nc = blockIdx.z; nc < planes; nc += gridDim.z) {
        const T* xp = x + nc * (int64_t)g.H * g.W;
        const int64_t o = (nc * g.OH + oh) * g.OW + ow;
        if (KS != 0) {
            // compile-time window: all loads of PL planes are issued before the first use (a rolled loop would wait
            // for every element in turn; one plane alone leaves too few bytes in flight), out-of-range taps predicated
            constexpr int KH = KS == 1 ? 2 : 3, KW = KH, PL = 4;
            const int pb = oh * Wn::sh(g) - g.ph, qb = ow * Wn::sw(g) - g.pw;
            A vals[PL][KH * KW];
            bool ok[KH * KW];
#pragma unroll
            for (int a = 0; a < KH; a++)
#pragma unroll
                for (int b = 0; b < KW; b++)
                    ok[a * KW + b] = (unsigned)(pb + a) < (unsigned)g.H && (unsigned)(qb + b) < (unsigned)g.W;
#pragma unroll
            for (int u = 0; u < PL; u++) {
                const int64_t pl = nc + (int64_t)u * gridDim.z;
                const T* xu = x + pl * (int64_t)g.H * g.W;
#pragma unroll
                for (int t = 0; t < KH * KW; t++)
                    vals[u][t] = (ok[t] && pl < planes) ? ld<T>(xu + (int64_t)(pb + t / KW) * g.W + qb + t % KW) : (A)0;
            }
#pragma unroll
            for (int u = 0; u < PL; u++) {
                const int64_t pl = nc + (int64_t)u * gridDim.z;
                if (pl >= planes) break;
                const int64_t ou = (pl * g.OH + oh) * g.OW + ow;
                if (OP == 2) {
                    A acc = 0;
#pragma unroll
                    for (int t = 0; t < KH * KW; t++) acc += vals[u][t];
                    const int count = g.count_include_pad ? KH * KW : (p1 - p0) * (q1 - q0);
                    y[ou] = cvt<T, A>(acc / (A)count);
                } else {
                    A best = ld<T>(&init);
                    int tap = -1;
#pragma unroll
                    for (int t = 0; t < KH * KW; t++)
                        if (ok[t] && (OP == 0 ? best < vals[u][t] : vals[u][t] < best)) { best = vals[u][t]; tap = t; }
                    y[ou] = cvt<T, A>(best);
                    if (indices) indices[ou] = tap < 0 ? -1 : (pb + tap / KW) * g.W + qb + tap % KW;
                }
            }
            nc += (int64_t)(PL - 1) * gridDim.z;
            continue;
        }
        if (OP == 2) {
            A acc = 0;
            for (int p = p0; p < p1; p++)
                for (int q = q0; q < q1; q++) acc += ld<T>(xp + (int64_t)p * g.W + q);
            const int count = g.count_include_pad ? Wn::kh(g) * Wn::kw(g) : (p1 - p0) * (q1 - q0);
            y[o] = cvt<T, A>(acc / (A)count);
        } else {
            A best = ld<T>(&init);
            int where = -1;
            for (int p = p0; p < p1; p++)
                for (int q = q0; q < q1; q++) {
                    const A v = ld<T>(xp + (int64_t)p * g.W + q);
                    // a strict comparison keeps the first extreme element, as the reference's index variant does
                    if (OP == 0 ? best < v : v < best) { best = v; where = p * g.W + q; }
                }
            y[o] = cvt<T, A>(best);
            if (indices) indices[o] = where;
        }
    }
}

template <typename T, int OP, int KS>
__global__ void __launch_bounds__(256) pool_bwd_kernel(const T* __restrict__ x, const T* __restrict__ y, const T* __restrict__ dy,
                                                       T* __restrict__ dx, Geo g) {
    using A = typename AccOf<T>::type;
    using Wn = Win<KS>;
    const int q = blockIdx.x * 32 + threadIdx.x, p = blockIdx.y * 8 + threadIdx.y;
    if (q >= g.W || p >= g.H) return;
    const int kh = Wn::kh(g), kw = Wn::kw(g), sh = Wn::sh(g), sw = Wn::sw(g);
    // windows containing row p: oh*sh - ph <= p < oh*sh - ph + kh
    const int oh_lo = max(0, (p + g.ph - kh + sh) / sh), oh_hi = min(g.OH - 1, (p + g.ph) / sh);
    const int ow_lo = max(0, (q + g.pw - kw + sw) / sw), ow_hi = min(g.OW - 1, (q + g.pw) / sw);
    const int64_t planes = (int64_t)g.N * g.C;
    for (int64_t nc = blockIdx.z; nc < planes; nc += gridDim.z) {
        const T* xp = x + nc * (int64_t)g.H * g.W;
        const T* yp = y + nc * (int64_t)g.OH * g.OW;
        const T* dp = dy + nc * (int64_t)g.OH * g.OW;
        const A mine = ld<T>(xp + (int64_t)p * g.W + q);
        A acc = 0;
        if (KS != 0) {
            // at most NW x NW windows contain this element; their pooled values and gradients are fetched up front
            constexpr int NW = KS == 1 ? 1 : KS == 2 ? 2 : 3;
            A yv[NW * NW], dv[NW * NW];
            bool in[NW * NW];
#pragma unroll
            for (int a = 0; a < NW; a++)
#pragma unroll
                for (int b = 0; b < NW; b++) {
                    const int oh = oh_lo + a, ow = ow_lo + b;
                    in[a * NW + b] = oh <= oh_hi && ow <= ow_hi;
                    const int64_t o = (int64_t)oh * g.OW + ow;
                    yv[a * NW + b] = in[a * NW + b] && OP != 2 ? ld<T>(yp + o) : (A)0;
                    dv[a * NW + b] = in[a * NW + b] ? ld<T>(dp + o) : (A)0;
                }
#pragma unroll
            for (int a = 0; a < NW; a++)
#pragma unroll
                for (int b = 0; b < NW; b++) {
                    if (!in[a * NW + b]) continue;
                    const int oh = oh_lo + a, ow = ow_lo + b;
                    int p0 = oh * sh - g.ph, q0 = ow * sw - g.pw;
                    const int p1 = min(p0 + kh, g.H), q1 = min(q0 + kw, g.W);
                    p0 = max(p0, 0); q0 = max(q0, 0);
                    if (OP == 2) {
                        const int count = g.count_include_pad ? kh * kw : (p1 - p0) * (q1 - q0);
                        acc += dv[a * NW + b] / (A)count;
                    } else {
                        if (!(mine == yv[a * NW + b])) continue;
                        bool first = true;
                        for (int pp = p0; pp <= p && first; pp++) {
                            const int qe = pp == p ? q : q1;
                            for (int qq = q0; qq < qe; qq++)
                                if (ld<T>(xp + (int64_t)pp * g.W + qq) == mine) { first = false; break; }
                        }
                        if (first) acc += dv[a * NW + b];
                    }
                }
            dx[(nc * g.H + p) * (int64_t)g.W + q] = cvt<T, A>(acc);
            continue;
        }
        for (int oh = oh_lo; oh <= oh_hi; oh++) {
            int p0 = oh * sh - g.ph;
            const int p1 = min(p0 + kh, g.H);
            p0 = max(p0, 0);
            if (p < p0 || p >= p1) continue;
            for (int ow = ow_lo; ow <= ow_hi; ow++) {
                int q0 = ow * sw - g.pw;
                const int q1 = min(q0 + kw, g.W);
                q0 = max(q0, 0);
                if (q < q0 || q >= q1) continue;
                if (OP == 2) {
                    const int count = g.count_include_pad ? kh * kw : (p1 - p0) * (q1 - q0);
                    acc += ld<T>(dp + (int64_t)oh * g.OW + ow) / (A)count;
                } else {
                    const A v = ld<T>(yp + (int64_t)oh * g.OW + ow);
                    if (!(mine == v)) continue;
                    bool first = true;
                    for (int pp = p0; pp <= p && first; pp++) {
                        const int qe = pp == p ? q : q1;
                        for (int qq = q0; qq < qe; qq++)
                            if (ld<T>(xp + (int64_t)pp * g.W + qq) == v) { first = false; break; }
                    }
                    if (first) acc += ld<T>(dp + (int64_t)oh * g.OW + ow);
                }
            }
        }
        dx[(nc * g.H + p) * (int64_t)g.W + q] = cvt<T, A>(acc);
    }
}

// Backward of maximum / minimum from the forward's index map: input element (p, q) receives dy of every window whose
// recorded first extreme element it is. No comparison of values, no scan, and x is not read at all.
template <typename T, int KS>
__global__ void __launch_bounds__(256) pool_bwd_indices_kernel(const int32_t* __restrict__ idx, const T* __restrict__ dy,
                                                               T* __restrict__ dx, Geo g) {
    using A = typename AccOf<T>::type;
    using Wn = Win<KS>;
    const int q = blockIdx.x * 32 + threadIdx.x, p = blockIdx.y * 8 + threadIdx.y;
    if (q >= g.W || p >= g.H) return;
    const int kh = Wn::kh(g), kw = Wn::kw(g), sh = Wn::sh(g), sw = Wn::sw(g);
    const int oh_lo = max(0, (p + g.ph - kh + sh) / sh), oh_hi = min(g.OH - 1, (p + g.ph) / sh);
    const int ow_lo = max(0, (q + g.pw - kw + sw) / sw), ow_hi = min(g.OW - 1, (q + g.pw) / sw);
    const int me = p * g.W + q;
    const int64_t planes = (int64_t)g.N * g.C;
    constexpr int PL = 4;
    for (int64_t nc = blockIdx.z; nc < planes; nc += (int64_t)PL * gridDim.z) {
        A acc[PL];
#pragma unroll
        for (int u = 0; u < PL; u++) acc[u] = 0;
        if (KS != 0) {
            constexpr int NW = KS == 1 ? 1 : KS == 2 ? 2 : 3;
            int iv[PL][NW * NW];
            A dv[PL][NW * NW];
#pragma unroll
            for (int u = 0; u < PL; u++) {
                const int64_t pl = nc + (int64_t)u * gridDim.z;
#pragma unroll
                for (int a = 0; a < NW; a++)
#pragma unroll
                    for (int b = 0; b < NW; b++) {
                        const int oh = oh_lo + a, ow = ow_lo + b;
                        const bool in = oh <= oh_hi && ow <= ow_hi && pl < planes;
                        const int64_t o = (pl * g.OH + oh) * g.OW + ow;
                        iv[u][a * NW + b] = in ? idx[o] : -2;
                        dv[u][a * NW + b] = in ? ld<T>(dy + o) : (A)0;
                    }
            }
#pragma unroll
            for (int u = 0; u < PL; u++)
#pragma unroll
                for (int t = 0; t < NW * NW; t++) if (iv[u][t] == me) acc[u] += dv[u][t];
        } else {
            for (int u = 0; u < PL; u++) {
                const int64_t pl = nc + (int64_t)u * gridDim.z;
                if (pl >= planes) break;
                for (int oh = oh_lo; oh <= oh_hi; oh++)
                    for (int ow = ow_lo; ow <= ow_hi; ow++) {
                        const int64_t o = (pl * g.OH + oh) * g.OW + ow;
                        if (idx[o] == me) acc[u] += ld<T>(dy + o);
                    }
            }
        }
#pragma unroll
        for (int u = 0; u < PL; u++) {
            const int64_t pl = nc + (int64_t)u * gridDim.z;
            if (pl < planes) dx[(pl * g.H + p) * (int64_t)g.W + q] = cvt<T, A>(acc[u]);
        }
    }
}

// Backward from the index map for stride-2 windows of edge <= 3: a thread owns a 2 x 2 block of input elements. The
// windows that can contain any of them form at most a 2 x 2 set, whose indices and gradients are fetched once; an
// element receives a window's gradient exactly when the window's index names it (no range test is needed: a window
// cannot name an element outside itself).
template <typename T, int KS>
__global__ void __launch_bounds__(256) pool_bwd_indices_s2_kernel(const int32_t* __restrict__ idx, const T* __restrict__ dy,
                                                                  T* __restrict__ dx, Geo g) {
    using A = typename AccOf<T>::type;
    constexpr int K = KS == 1 ? 2 : 3, PL = 2;
    const int q0 = (blockIdx.x * 32 + threadIdx.x) * 2, p0 = (blockIdx.y * 8 + threadIdx.y) * 2;
    if (q0 >= g.W || p0 >= g.H) return;
    const int oh0 = max(0, (p0 + g.ph - K + 2) / 2), ow0 = max(0, (q0 + g.pw - K + 2) / 2);
    const bool r1 = oh0 + 1 < g.OH, c1 = ow0 + 1 < g.OW;
    const bool has_p1 = p0 + 1 < g.H, has_q1 = q0 + 1 < g.W;
    const int me00 = p0 * g.W + q0;
    const int64_t planes = (int64_t)g.N * g.C, oplane = (int64_t)g.OH * g.OW, iplane = (int64_t)g.H * g.W;
    const int64_t obase = (int64_t)oh0 * g.OW + ow0;
    const bool pair_store = (g.W % 2 == 0) && has_q1 && sizeof(T) == 4 && (reinterpret_cast<uintptr_t>(dx) & 7) == 0;
    for (int64_t nc = blockIdx.z; nc < planes; nc += (int64_t)PL * gridDim.z) {
        int iv[PL][4];
        A dv[PL][4];
#pragma unroll
        for (int u = 0; u < PL; u++) {
            const int64_t pl = nc + (int64_t)u * gridDim.z;
            const bool live = pl < planes;
            const int32_t* ip = idx + pl * oplane + obase;
            const T* dp = dy + pl * oplane + obase;
            iv[u][0] = live ? ip[0] : -2;                     dv[u][0] = live ? ld<T>(dp) : (A)0;
            iv[u][1] = live && c1 ? ip[1] : -2;               dv[u][1] = live && c1 ? ld<T>(dp + 1) : (A)0;
            iv[u][2] = live && r1 ? ip[g.OW] : -2;            dv[u][2] = live && r1 ? ld<T>(dp + g.OW) : (A)0;
            iv[u][3] = live && r1 && c1 ? ip[g.OW + 1] : -2;  dv[u][3] = live && r1 && c1 ? ld<T>(dp + g.OW + 1) : (A)0;
        }
#pragma unroll
        for (int u = 0; u < PL; u++) {
            const int64_t pl = nc + (int64_t)u * gridDim.z;
            if (pl >= planes) break;
            A acc[4] = {0, 0, 0, 0};                           // (p0,q0) (p0,q0+1) (p0+1,q0) (p0+1,q0+1)
#pragma unroll
            for (int t = 0; t < 4; t++) {
                const int d = iv[u][t] - me00;
                acc[0] += d == 0 ? dv[u][t] : (A)0;
                acc[1] += d == 1 ? dv[u][t] : (A)0;
                acc[2] += d == g.W ? dv[u][t] : (A)0;
                acc[3] += d == g.W + 1 ? dv[u][t] : (A)0;
            }
            T* out = dx + pl * iplane + me00;
            if (pair_store) {
                float2 a = make_float2((float)acc[0], (float)acc[1]);
                *reinterpret_cast<float2*>(out) = a;
                if (has_p1) { float2 b = make_float2((float)acc[2], (float)acc[3]); *reinterpret_cast<float2*>(out + g.W) = b; }
            } else {
                out[0] = cvt<T, A>(acc[0]);
                if (has_q1) out[1] = cvt<T, A>(acc[1]);
                if (has_p1) { out[g.W] = cvt<T, A>(acc[2]); if (has_q1) out[g.W + 1] = cvt<T, A>(acc[3]); }
            }
        }
    }
}

// Forward for stride-2 windows of edge <= 3 with padding 0 or 1 on rows of a multiple of 4 elements: a thread produces
// two horizontally adjacent outputs from ONE 16-byte load per input row plus the two neighbouring elements, instead of
// 2 x K strided 4-byte loads per row.
template <int OP, int KS>
__global__ void __launch_bounds__(256) pool_fwd_s2_kernel(const float* __restrict__ x, float* __restrict__ y, int32_t* __restrict__ indices,
                                                          Geo g, float init) {
    constexpr int K = KS == 1 ? 2 : 3, PL = 2;
    const int ow0 = (blockIdx.x * 32 + threadIdx.x) * 2, oh = blockIdx.y * 8 + threadIdx.y;
    if (ow0 >= g.OW || oh >= g.OH) return;
    const int pb = oh * 2 - g.ph, c0 = ow0 * 2;                 // first window row; column of the aligned 16-byte load
    const bool two = ow0 + 1 < g.OW;
    bool rok[K];
#pragma unroll
    for (int a = 0; a < K; a++) rok[a] = (unsigned)(pb + a) < (unsigned)g.H;
    const bool left = c0 - 1 >= 0, mid = c0 + 3 < g.W, right = c0 + 4 < g.W;   // W % 4 == 0: the vector is all in or all out
    const float pad = OP == 2 ? 0.f : init;
    const int64_t planes = (int64_t)g.N * g.C, iplane = (int64_t)g.H * g.W;
    for (int64_t nc = blockIdx.z; nc < planes; nc += (int64_t)PL * gridDim.z) {
        float v[PL][K][6];                                      // columns c0-1 .. c0+4
#pragma unroll
        for (int u = 0; u < PL; u++) {
            const int64_t pl = nc + (int64_t)u * gridDim.z;
            const float* xu = x + pl * iplane + (int64_t)pb * g.W + c0;
#pragma unroll
            for (int a = 0; a < K; a++) {
                const bool ok = rok[a] && pl < planes;
                const float* row = xu + (int64_t)a * g.W;
                const float4 m = ok && mid ? *reinterpret_cast<const float4*>(row) : make_float4(pad, pad, pad, pad);
                v[u][a][0] = ok && left ? row[-1] : pad;
                v[u][a][1] = m.x; v[u][a][2] = m.y; v[u][a][3] = m.z; v[u][a][4] = m.w;
                v[u][a][5] = ok && right ? row[4] : pad;
            }
        }
#pragma unroll
        for (int u = 0; u < PL; u++) {
            const int64_t pl = nc + (int64_t)u * gridDim.z;
            if (pl >= planes) break;
#pragma unroll
            for (int j = 0; j < 2; j++) {
                if (j == 1 && !two) break;
                const int ow = ow0 + j;
                const int qb = ow * 2 - g.pw;                   // first window column; slot of tap b is 2j - pw + b + 1
                float best = pad, acc = 0.f;
                int tap = -1;
#pragma unroll
                for (int a = 0; a < K; a++)
#pragma unroll
                    for (int b = 0; b < K; b++) {
                        const float val = g.pw ? v[u][a][2 * j + b] : v[u][a][2 * j + b + 1];
                        const bool in = rok[a] && (unsigned)(qb + b) < (unsigned)g.W;
                        if (OP == 2) acc += in ? val : 0.f;
                        else if (in && (OP == 0 ? best < val : val < best)) { best = val; tap = a * K + b; }
                    }
                const int64_t o = (pl * g.OH + oh) * g.OW + ow;
                if (OP == 2) {
                    const int p1 = min(pb + K, g.H), q1 = min(qb + K, g.W);
                    const int count = g.count_include_pad ? K * K : (p1 - max(pb, 0)) * (q1 - max(qb, 0));
                    y[o] = acc / (float)count;
                } else {
                    y[o] = best;
                    if (indices) indices[o] = tap < 0 ? -1 : (pb + tap / K) * g.W + qb + tap % K;
                }
            }
        }
    }
}

static int window_code(const Geo& g) {
    if (g.kh == 2 && g.kw == 2 && g.sh == 2 && g.sw == 2) return 1;
    if (g.kh == 3 && g.kw == 3 && g.sh == 2 && g.sw == 2) return 2;
    if (g.kh == 3 && g.kw == 3 && g.sh == 1 && g.sw == 1) return 3;
    return 0;
}

static dim3 plane_grid(int w, int h, int64_t planes) {
    const unsigned gx = (unsigned)((w + 31) / 32), gy = (unsigned)((h + 7) / 8);
    // enough plane slices to fill the machine a few times over, each block then strides over the remaining planes
    const int64_t want = ((int64_t)kNumSMs * 16 + (int64_t)gx * gy - 1) / ((int64_t)gx * gy);
    const unsigned gz = (unsigned)std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(planes, 65535), want));
    return dim3(gx, gy, gz);
}

static int parse(const b200jt_tensor* x, const b200jt_tensor* y, const char* op, int kh, int kw, int sh, int sw, int ph, int pw,
                 int count_include_pad, Geo* g, int* opc) {
    B200JT_CHECK_ARG(valid_tensor(x) && valid_tensor(y) && x->ndim == 4 && y->ndim == 4, "pool2d takes NCHW tensors");
    B200JT_CHECK_ARG(x->dtype == y->dtype, "x and y must have the same dtype");
    B200JT_CHECK_ARG(kh > 0 && kw > 0, "kernel_size must be greater than zero");
    B200JT_CHECK_ARG(sh > 0 && sw > 0, "stride must be greater than zero");
    B200JT_CHECK_ARG(ph >= 0 && pw >= 0, "padding must be non-negative");
    B200JT_CHECK_ARG(x->shape[0] == y->shape[0] && x->shape[1] == y->shape[1], "batch / channel mismatch between x and y");
    B200JT_CHECK_ARG(op != nullptr, "op is null");
    *opc = !strcmp(op, "maximum") ? 0 : !strcmp(op, "minimum") ? 1 : !strcmp(op, "mean") ? 2 : -1;
    B200JT_CHECK_ARG(*opc >= 0, std::string("pool2d op must be maximum, minimum or mean, got '") + op + "'");
    for (int d = 0; d < 4; d++)
        B200JT_CHECK_ARG(x->shape[d] < (1LL << 31) && y->shape[d] < (1LL << 31), "dimension too large");
    g->N = (int)x->shape[0]; g->C = (int)x->shape[1]; g->H = (int)x->shape[2]; g->W = (int)x->shape[3];
    g->OH = (int)y->shape[2]; g->OW = (int)y->shape[3];
    g->kh = kh; g->kw = kw; g->sh = sh; g->sw = sw; g->ph = ph; g->pw = pw; g->count_include_pad = count_include_pad;
    return 0;
}

template <typename T, int OP>
static void launch_fwd(const T* xp, T* yp, int32_t* indices, const Geo& g, T init, cudaStream_t st) {
    const dim3 grid = plane_grid(g.OW, g.OH, (int64_t)g.N * g.C), block(32, 8);
    if constexpr (sizeof(T) == 4) {
        const int code = window_code(g);
        if ((code == 1 || code == 2) && g.W % 4 == 0 && (g.pw == 0 || g.pw == 1) && ((uintptr_t)xp & 15) == 0) {
            const dim3 grid2 = plane_grid((g.OW + 1) / 2, g.OH, ((int64_t)g.N * g.C + 1) / 2);
            if (code == 1) pool_fwd_s2_kernel<OP, 1><<<grid2, block, 0, st>>>((const float*)xp, (float*)yp, indices, g, (float)init);
            else pool_fwd_s2_kernel<OP, 2><<<grid2, block, 0, st>>>((const float*)xp, (float*)yp, indices, g, (float)init);
            return;
        }
    }
    switch (window_code(g)) {
        case 1: pool_fwd_kernel<T, OP, 1><<<grid, block, 0, st>>>(xp, yp, indices, g, init); break;
        case 2: pool_fwd_kernel<T, OP, 2><<<grid, block, 0, st>>>(xp, yp, indices, g, init); break;
        case 3: pool_fwd_kernel<T, OP, 3><<<grid, block, 0, st>>>(xp, yp, indices, g, init); break;
        default: pool_fwd_kernel<T, OP, 0><<<grid, block, 0, st>>>(xp, yp, indices, g, init);
    }
}

template <typename T, int OP>
static void launch_bwd(const T* xp, const T* yp, const T* dp, T* op, const Geo& g, cudaStream_t st) {
    const dim3 grid = plane_grid(g.W, g.H, (int64_t)g.N * g.C), block(32, 8);
    switch (window_code(g)) {
        case 1: pool_bwd_kernel<T, OP, 1><<<grid, block, 0, st>>>(xp, yp, dp, op, g); break;
        case 2: pool_bwd_kernel<T, OP, 2><<<grid, block, 0, st>>>(xp, yp, dp, op, g); break;
        case 3: pool_bwd_kernel<T, OP, 3><<<grid, block, 0, st>>>(xp, yp, dp, op, g); break;
        default: pool_bwd_kernel<T, OP, 0><<<grid, block, 0, st>>>(xp, yp, dp, op, g);
    }
}

template <typename T>
static int run_bwd_indices(const int32_t* idx, const b200jt_tensor* dy, const b200jt_tensor* dx, const Geo& g, cudaStream_t st) {
    if (numel(dx) == 0) return 0;
    const int64_t planes = (int64_t)g.N * g.C;
    const dim3 grid = plane_grid(g.W, g.H, (planes + 3) / 4), block(32, 8);
    const dim3 grid2 = plane_grid((g.W + 1) / 2, (g.H + 1) / 2, (planes + 1) / 2);
    const T* dp = (const T*)dy->ptr; T* op = (T*)dx->ptr;
    switch (window_code(g)) {
        case 1: pool_bwd_indices_s2_kernel<T, 1><<<grid2, block, 0, st>>>(idx, dp, op, g); break;
        case 2: pool_bwd_indices_s2_kernel<T, 2><<<grid2, block, 0, st>>>(idx, dp, op, g); break;
        case 3: pool_bwd_indices_kernel<T, 3><<<grid, block, 0, st>>>(idx, dp, op, g); break;
        default: pool_bwd_indices_kernel<T, 0><<<grid, block, 0, st>>>(idx, dp, op, g);
    }
    B200JT_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int run_fwd(const b200jt_tensor* x, const b200jt_tensor* y, int32_t* indices, const Geo& g, int opc, cudaStream_t st) {
    if (numel(y) == 0) return 0;
    const T* xp = (const T*)x->ptr; T* yp = (T*)y->ptr;
    if (opc == 0) launch_fwd<T, 0>(xp, yp, indices, g, init_value<T>(OP_MAX), st);
    else if (opc == 1) launch_fwd<T, 1>(xp, yp, indices, g, init_value<T>(OP_MIN), st);
    else launch_fwd<T, 2>(xp, yp, indices, g, init_value<T>(OP_ADD), st);
    B200JT_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int run_bwd(const b200jt_tensor* x, const b200jt_tensor* y, const b200jt_tensor* dy, const b200jt_tensor* dx,
                   const Geo& g, int opc, cudaStream_t st) {
    if (numel(x) == 0) return 0;
    const T *xp = (const T*)x->ptr, *yp = (const T*)y->ptr, *dp = (const T*)dy->ptr; T* op = (T*)dx->ptr;
    if (opc == 0) launch_bwd<T, 0>(xp, yp, dp, op, g, st);
    else if (opc == 1) launch_bwd<T, 1>(xp, yp, dp, op, g, st);
    else launch_bwd<T, 2>(xp, yp, dp, op, g, st);
    B200JT_LAUNCH_CHECK();
    return 0;
}

}  // namespace pool
}  // namespace b200jt

using namespace b200jt;

extern "C" int b200jt_pool2d(const b200jt_tensor* x, const b200jt_tensor* y, int32_t* indices, const char* op,
                             int kh, int kw, int sh, int sw, int ph, int pw, int count_include_pad, void* stream) {
    pool::Geo g; int opc;
    if (int rc = pool::parse(x, y, op, kh, kw, sh, sw, ph, pw, count_include_pad, &g, &opc)) return rc;
    B200JT_CHECK_ARG(!indices || opc != 2, "indices are only produced for maximum and minimum");
    cudaStream_t st = (cudaStream_t)stream;
    switch (x->dtype) {
        case B200JT_FLOAT32: return pool::run_fwd<float>(x, y, indices, g, opc, st);
        case B200JT_FLOAT64: return pool::run_fwd<double>(x, y, indices, g, opc, st);
        case B200JT_BFLOAT16: return pool::run_fwd<__nv_bfloat16>(x, y, indices, g, opc, st);
        case B200JT_FLOAT16: return pool::run_fwd<__half>(x, y, indices, g, opc, st);
    }
    return fail(-1, "b200jt_pool2d: dtype must be float32, float64, float16 or bfloat16");
}

extern "C" int b200jt_pool2d_backward(const b200jt_tensor* x, const b200jt_tensor* y, const b200jt_tensor* dy,
                                      const b200jt_tensor* dx, const char* op,
                                      int kh, int kw, int sh, int sw, int ph, int pw, int count_include_pad, void* stream) {
    pool::Geo g; int opc;
    if (int rc = pool::parse(x, y, op, kh, kw, sh, sw, ph, pw, count_include_pad, &g, &opc)) return rc;
    B200JT_CHECK_ARG(valid_tensor(dy) && valid_tensor(dx) && dy->ndim == 4 && dx->ndim == 4 &&
                     dy->dtype == x->dtype && dx->dtype == x->dtype, "dy, dx must be NCHW tensors of x's dtype");
    for (int d = 0; d < 4; d++)
        B200JT_CHECK_ARG(dy->shape[d] == y->shape[d] && dx->shape[d] == x->shape[d], "dy must have y's shape and dx x's shape");
    cudaStream_t st = (cudaStream_t)stream;
    switch (x->dtype) {
        case B200JT_FLOAT32: return pool::run_bwd<float>(x, y, dy, dx, g, opc, st);
        case B200JT_FLOAT64: return pool::run_bwd<double>(x, y, dy, dx, g, opc, st);
        case B200JT_BFLOAT16: return pool::run_bwd<__nv_bfloat16>(x, y, dy, dx, g, opc, st);
        case B200JT_FLOAT16: return pool::run_bwd<__half>(x, y, dy, dx, g, opc, st);
    }
    return fail(-1, "b200jt_pool2d_backward: dtype must be float32, float64, float16 or bfloat16");
}

extern "C" int b200jt_pool2d_backward_indices(const b200jt_tensor* x, const b200jt_tensor* y, const int32_t* indices,
                                              const b200jt_tensor* dy, const b200jt_tensor* dx,
                                              int kh, int kw, int sh, int sw, int ph, int pw, void* stream) {
    pool::Geo g; int opc;
    if (int rc = pool::parse(x, y, "maximum", kh, kw, sh, sw, ph, pw, 1, &g, &opc)) return rc;
    B200JT_CHECK_ARG(indices != nullptr, "indices is null");
    B200JT_CHECK_ARG(valid_tensor(dy) && valid_tensor(dx) && dy->ndim == 4 && dx->ndim == 4 &&
                     dy->dtype == x->dtype && dx->dtype == x->dtype, "dy, dx must be NCHW tensors of x's dtype");
    for (int d = 0; d < 4; d++)
        B200JT_CHECK_ARG(dy->shape[d] == y->shape[d] && dx->shape[d] == x->shape[d], "dy must have y's shape and dx x's shape");
    B200JT_CHECK_ARG((int64_t)g.H * g.W < (1LL << 31), "plane too large for int32 indices");
    cudaStream_t st = (cudaStream_t)stream;
    switch (x->dtype) {
        case B200JT_FLOAT32: return pool::run_bwd_indices<float>(indices, dy, dx, g, st);
        case B200JT_FLOAT64: return pool::run_bwd_indices<double>(indices, dy, dx, g, st);
        case B200JT_BFLOAT16: return pool::run_bwd_indices<__nv_bfloat16>(indices, dy, dx, g, st);
        case B200JT_FLOAT16: return pool::run_bwd_indices<__half>(indices, dy, dx, g, st);
    }
    return fail(-1, "b200jt_pool2d_backward_indices: dtype must be float32, float64, float16 or bfloat16");
}
