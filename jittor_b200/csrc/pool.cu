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
                    int where = -1;
#pragma unroll
                    for (int t = 0; t < KH * KW; t++)
                        if (ok[t] && (OP == 0 ? best < vals[u][t] : vals[u][t] < best)) { best = vals[u][t]; where = (pb + t / KW) * g.W + qb + t % KW; }
                    y[ou] = cvt<T, A>(best);
                    if (indices) indices[ou] = where;
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
    const dim3 grid = plane_grid(g.W, g.H, ((int64_t)g.N * g.C + 3) / 4), block(32, 8);
    const T* dp = (const T*)dy->ptr; T* op = (T*)dx->ptr;
    switch (window_code(g)) {
        case 1: pool_bwd_indices_kernel<T, 1><<<grid, block, 0, st>>>(idx, dp, op, g); break;
        case 2: pool_bwd_indices_kernel<T, 2><<<grid, block, 0, st>>>(idx, dp, op, g); break;
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
