// reindex: y[i] = overflow(i) ? fill : x[index(i)]  (gather; a pure data movement, bit-exact).
//
// Two kernels:
//   * affine  -- every index is c0 + sum coef*i: one thread produces VEC consecutive outputs of the
//                innermost loop axis, coordinates are unflattened once per thread and advanced
//                incrementally; stores are VEC*elem-size wide (up to 128 bit) and coalesced.
//   * generic -- the bytecode of index_program.cuh interpreted per element (div/mod, conditions,
//                @eK loads).
// The output write stream dominates traffic (the gather source is usually much smaller and L2
// resident), so both kernels are organised around coalesced output stores.
#include "index_program.cuh"

namespace b200jt {

struct AffineArgs {
    int32_t ndim_loop, ndim_x;
    int64_t loop_shape[kMaxDims];
    int64_t x_shape[kMaxDims];
    int64_t c0[kMaxDims];
    int64_t coef[kMaxDims][kMaxDims];
};

// I = index type (32-bit arithmetic when every tensor is below 2^31 elements, as the reference's index_t).
// NL / NX are compile-time upper bounds of the two ranks: all loops over axes are fully unrolled to them (with
// uniform guards for the actual ranks) so that the coordinate arrays stay in registers.
template <typename T, typename I, int VEC, int NL, int NX>
__global__ void __launch_bounds__(256)
reindex_affine_kernel(const T* __restrict__ x, T* __restrict__ y, const __grid_constant__ AffineArgs A,
                      int64_t n_vec, T fill) {
    using U = typename std::conditional<sizeof(I) == 4, uint32_t, uint64_t>::type;
    const int nl = A.ndim_loop, nx = A.ndim_x;
    for (int64_t v = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; v < n_vec;
         v += (int64_t)gridDim.x * blockDim.x) {
        // vectors never straddle rows: the host picks VEC | innermost extent
        const int64_t flat = v * VEC;
        I iv[NL];
        U r = (U)flat;
#pragma unroll
        for (int d = NL - 1; d >= 0; d--) {
            iv[d] = 0;
            if (d < nl) { const U s = (U)A.loop_shape[d]; const U q = r / s; iv[d] = (I)(r - q * s); r = q; }
        }
        I xid[NX], xinner[NX], xs[NX];
#pragma unroll
        for (int d = 0; d < NX; d++) {
            xid[d] = 0; xinner[d] = 0; xs[d] = 1;
            if (d < nx) {
                I a = (I)A.c0[d];
#pragma unroll
                for (int j = 0; j < NL; j++)
                    if (j < nl) a += (I)A.coef[d][j] * iv[j];
                xid[d] = a; xinner[d] = (I)A.coef[d][nl - 1]; xs[d] = (I)A.x_shape[d];
            }
        }
        __align__(16) T out[VEC];
#pragma unroll
        for (int e = 0; e < VEC; e++) {
            bool over = false;
            int64_t off = 0;
#pragma unroll
            for (int d = 0; d < NX; d++) {
                if (d < nx) {
                    const I id = xid[d] + xinner[d] * (I)e;
                    over |= (id < 0) | (id >= xs[d]);
                    off = off * xs[d] + id;
                }
            }
            out[e] = over ? fill : x[off];
        }
        if (VEC == 1) y[flat] = out[0];
        else {
            if (VEC * sizeof(T) == 16) *reinterpret_cast<uint4*>(y + flat) = *reinterpret_cast<uint4*>(out);
            else if (VEC * sizeof(T) == 8) *reinterpret_cast<uint2*>(y + flat) = *reinterpret_cast<uint2*>(out);
            else if (VEC * sizeof(T) == 4) *reinterpret_cast<uint32_t*>(y + flat) = *reinterpret_cast<uint32_t*>(out);
            else if (VEC * sizeof(T) == 2) *reinterpret_cast<uint16_t*>(y + flat) = *reinterpret_cast<uint16_t*>(out);
            else {
#pragma unroll
                for (int e = 0; e < VEC; e++) y[flat + e] = out[e];
            }
        }
    }
}

template <typename T, int VEC>
static void launch_affine(const T* xp, T* yp, const AffineArgs& A, int64_t nv, T fill, bool small, cudaStream_t st) {
    const unsigned grid = grid_for(nv, 256);
    const int nl = A.ndim_loop, nx = A.ndim_x;
#define B200JT_AFF(NL, NX) reindex_affine_kernel<T, int32_t, VEC, NL, NX><<<grid, 256, 0, st>>>(xp, yp, A, nv, fill)
    if (!small) { reindex_affine_kernel<T, int64_t, VEC, kMaxDims, kMaxDims><<<grid, 256, 0, st>>>(xp, yp, A, nv, fill); return; }
    if (nl <= 2) { if (nx <= 2) B200JT_AFF(2, 2); else if (nx <= 4) B200JT_AFF(2, 4); else B200JT_AFF(2, kMaxDims); }
    else if (nl <= 4) { if (nx <= 2) B200JT_AFF(4, 2); else if (nx <= 4) B200JT_AFF(4, 4); else B200JT_AFF(4, kMaxDims); }
    else if (nl <= 8) { if (nx <= 2) B200JT_AFF(8, 2); else if (nx <= 4) B200JT_AFF(8, 4); else B200JT_AFF(8, kMaxDims); }
    else { if (nx <= 4) B200JT_AFF(kMaxDims, 4); else B200JT_AFF(kMaxDims, kMaxDims); }
#undef B200JT_AFF
}

template <typename T, typename I>
__global__ void __launch_bounds__(256)
reindex_generic_kernel(const T* __restrict__ x, T* __restrict__ y, const __grid_constant__ IndexProgram P,
                       int64_t n, T fill) {
    const int nl = P.ndim_loop, nx = P.ndim_x;
    for (int64_t flat = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; flat < n;
         flat += (int64_t)gridDim.x * blockDim.x) {
        I iv[kMaxDims];
        int64_t r = flat;
#pragma unroll 1
        for (int d = nl - 1; d >= 0; d--) { int64_t s = P.loop_shape[d]; iv[d] = (I)(r % s); r /= s; }
        I xid[kMaxDims];
        bool over = eval_index_program<I>(P, iv, xid);
        T v = fill;
        if (!over) {
            int64_t off = 0;
            for (int d = 0; d < nx; d++) off = off * P.x_shape[d] + (int64_t)xid[d];
            v = x[off];
        }
        y[flat] = v;
    }
}

template <typename T>
static T make_fill(double v, int dtype) {
    // Tx(overflow_value) with C conversion rules (reindex_op.cc:138)
    T out;
    switch (dtype) {
        case B200JT_BOOL: { uint8_t b = v != 0; memcpy(&out, &b, sizeof(T)); break; }
        case B200JT_INT8: { int8_t b = (int8_t)(int64_t)v; memcpy(&out, &b, sizeof(T)); break; }
        case B200JT_UINT8: { uint8_t b = (uint8_t)(int64_t)v; memcpy(&out, &b, sizeof(T)); break; }
        case B200JT_INT16: { int16_t b = (int16_t)(int64_t)v; memcpy(&out, &b, sizeof(T)); break; }
        case B200JT_INT32: { int32_t b = (int32_t)(int64_t)v; memcpy(&out, &b, sizeof(T)); break; }
        case B200JT_INT64: { int64_t b = (int64_t)v; memcpy(&out, &b, sizeof(T)); break; }
        case B200JT_FLOAT16: { __half b = __float2half((float)v); memcpy(&out, &b, sizeof(T)); break; }
        case B200JT_BFLOAT16: { __nv_bfloat16 b = __float2bfloat16((float)v); memcpy(&out, &b, sizeof(T)); break; }
        case B200JT_FLOAT32: { float b = (float)v; memcpy(&out, &b, sizeof(T)); break; }
        default: { double b = v; memcpy(&out, &b, sizeof(T)); break; }
    }
    return out;
}

template <typename T>
static int launch_reindex(const b200jt_tensor* x, const b200jt_tensor* y, const IndexProgram& P,
                          double overflow_value, cudaStream_t st) {
    const int64_t n = numel(y);
    const T fill = make_fill<T>(overflow_value, x->dtype);
    const bool small = numel(x) < (1LL << 31) && n < (1LL << 31);
    const T* xp = (const T*)x->ptr;
    T* yp = (T*)y->ptr;
    if (P.is_affine && numel(x) > 0) {
        AffineArgs A;
        memset(&A, 0, sizeof(A));
        A.ndim_loop = P.ndim_loop; A.ndim_x = P.ndim_x;
        memcpy(A.loop_shape, P.loop_shape, sizeof(A.loop_shape));
        memcpy(A.x_shape, P.x_shape, sizeof(A.x_shape));
        memcpy(A.c0, P.c0, sizeof(A.c0));
        memcpy(A.coef, P.coef, sizeof(A.coef));
        const int64_t inner = P.loop_shape[P.ndim_loop - 1];
        // one 16-byte (8-byte for 1-byte elements) output vector per thread when rows and alignment allow it
        constexpr int VMAX = 16 / sizeof(T) > 8 ? 8 : 16 / sizeof(T);
        const bool vec_ok = VMAX > 1 && inner % VMAX == 0 && ((uintptr_t)yp % (VMAX * sizeof(T))) == 0;
        if (vec_ok) launch_affine<T, VMAX>(xp, yp, A, n / VMAX, fill, small, st);
        else launch_affine<T, 1>(xp, yp, A, n, fill, small, st);
    } else {
        unsigned grid = grid_for(n, 256);
        if (small) reindex_generic_kernel<T, int32_t><<<grid, 256, 0, st>>>(xp, yp, P, n, fill);
        else       reindex_generic_kernel<T, int64_t><<<grid, 256, 0, st>>>(xp, yp, P, n, fill);
    }
    B200JT_LAUNCH_CHECK();
    return 0;
}

}  // namespace b200jt

using namespace b200jt;

extern "C" int b200jt_reindex(const b200jt_tensor* x, const b200jt_tensor* y,
                              const char* const* indexes, int n_indexes, double overflow_value,
                              const char* const* overflow_conditions, int n_conditions,
                              const b200jt_tensor* extras, int n_extras, void* stream) {
    B200JT_CHECK_ARG(valid_tensor(x) && valid_tensor(y), "invalid tensor descriptor");
    B200JT_CHECK_ARG(x->dtype == y->dtype, "x and y must have the same dtype");
    B200JT_CHECK_ARG(n_indexes == x->ndim, "Number of x's shape and indexes should be the same.");
    B200JT_CHECK_ARG(n_extras >= 0 && n_extras <= B200JT_MAX_EXTRAS, "too many extras");
    for (int k = 0; k < n_extras; k++) B200JT_CHECK_ARG(valid_tensor(&extras[k]), "invalid extras descriptor");
    if (numel(y) == 0) return 0;
    IndexProgram P;
    std::string err;
    if (!compile_index_program(y->shape, y->ndim, x->shape, x->ndim, indexes, n_indexes,
                               overflow_conditions, n_conditions, extras, n_extras, &P, &err))
        return fail(-2, "b200jt_reindex: " + err);
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype_size(x->dtype)) {
        case 1: return launch_reindex<uint8_t>(x, y, P, overflow_value, st);
        case 2: return launch_reindex<uint16_t>(x, y, P, overflow_value, st);
        case 4: return launch_reindex<uint32_t>(x, y, P, overflow_value, st);
        default: return launch_reindex<uint64_t>(x, y, P, overflow_value, st);
    }
}
