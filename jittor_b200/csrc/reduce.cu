// reduce: y = fold(op) of x over the axes of reduce_mask (python/jittor/src/ops/reduce_op.cc:374-399).
//
// The host first canonicalises the shape (drops size-1 axes, merges neighbours with the same
// kept/reduced status), then picks:
//   row kernel -- innermost axis reduced and long: one CTA per output, threads stride the reduced
//                 index space with the contiguous axis innermost (coalesced), warp-shuffle tree then one
//                 shared-memory hop per warp;
//   col kernel -- innermost axis kept (or short reductions): one thread per output, neighbouring
//                 threads read neighbouring addresses, serial fold over the reduced space.
// Few outputs with long reductions are split S ways into a workspace of partials that a second launch
// folds in fixed order (deterministic; no atomics).
// Accumulation is in the class of the output dtype: float32 -> float, float64 -> double, integers -> int64
// (truncated on store, which equals wrap-around arithmetic of the narrower type).
// `mean` accumulates x * rcount element by element (python/jittor/src/type/common_op_type.cc:141).
#include "atomic_ops.cuh"

namespace b200jt {

struct ReduceArgs {
    int32_t nk, nr;
    int64_t kshape[kMaxDims], kstride[kMaxDims];
    int64_t rshape[kMaxDims], rstride[kMaxDims];
    int64_t n_out, n_red;
    int32_t split;
    int64_t chunk;          // reduced elements per split
    double rcount;
};

template <typename C>
__device__ __forceinline__ C reduce_combine(int op, C a, C b) {
    if constexpr (std::is_integral<C>::value) {
        if (op == OP_BAND || op == OP_BOR || op == OP_BXOR) return apply_bitop_c<C>(op, a, b);
    }
    return apply_op_c<C>(op == OP_MEAN ? OP_ADD : op, a, b);
}

template <typename C>
__device__ __forceinline__ C reduce_init(int op, int ydt) {
    // initial value expressed in the accumulation class, limits taken from the OUTPUT dtype
    switch (op) {
        case OP_MUL: case OP_LAND: return (C)1;
        case OP_BAND: return (C)(-1);
        case OP_MAX:
            if (ydt == B200JT_FLOAT32) return (C)(-FLT_MAX);
            if (ydt == B200JT_FLOAT64) return (C)(-DBL_MAX);
            if (ydt == B200JT_INT32) return (C)INT32_MIN;
            if (ydt == B200JT_INT64) return (C)INT64_MIN;
            if (ydt == B200JT_INT16) return (C)INT16_MIN;
            if (ydt == B200JT_INT8) return (C)INT8_MIN;
            if (ydt == B200JT_FLOAT16) return (C)(-65504.0);
            if (ydt == B200JT_BFLOAT16) return (C)(-3.3895313892515355e38);
            return (C)0;
        case OP_MIN:
            if (ydt == B200JT_FLOAT32) return (C)(FLT_MAX);
            if (ydt == B200JT_FLOAT64) return (C)(DBL_MAX);
            if (ydt == B200JT_INT32) return (C)INT32_MAX;
            if (ydt == B200JT_INT64) return (C)INT64_MAX;
            if (ydt == B200JT_INT16) return (C)INT16_MAX;
            if (ydt == B200JT_INT8) return (C)INT8_MAX;
            if (ydt == B200JT_UINT8) return (C)UINT8_MAX;
            if (ydt == B200JT_FLOAT16) return (C)(65504.0);
            if (ydt == B200JT_BFLOAT16) return (C)(3.3895313892515355e38);
            return (C)1;
    }
    return (C)0;
}

__device__ __forceinline__ int64_t kept_offset(const ReduceArgs& A, int64_t o) {
    int64_t off = 0;
#pragma unroll 1
    for (int d = A.nk - 1; d >= 0; d--) { int64_t s = A.kshape[d]; off += (o % s) * A.kstride[d]; o /= s; }
    return off;
}
template <typename C>
__device__ __forceinline__ C shfl_down_c(C v, int delta) {
    if constexpr (sizeof(C) == 8) {
        long long b; memcpy(&b, &v, 8);
        b = __shfl_down_sync(0xffffffffu, b, delta);
        C r; memcpy(&r, &b, 8); return r;
    } else {
        return __shfl_down_sync(0xffffffffu, v, delta);
    }
}

// Typed element access: TX = void selects the run-time dtype switch, otherwise a plain typed load.
template <typename TX, typename C>
__device__ __forceinline__ C load_x(const void* x, int xdt, int64_t off) {
    if constexpr (std::is_same<TX, void>::value) return load_as<C>(x, xdt, off);
    else if constexpr (std::is_same<TX, __nv_bfloat16>::value) return (C)__bfloat162float(((const __nv_bfloat16*)x)[off]);
    else return (C)((const TX*)x)[off];
}

// One CTA per (output, split). out: y (final, dtype ydt) when !to_partial, else partial[o*split + s] in class C.
// The reduced index space is walked as (outer reduced axes) x (innermost reduced axis): threads stride the
// innermost axis (contiguous when its stride is 1 -> coalesced, 16-byte loads for float32), the outer axes are
// decomposed once per sweep.
// OPK >= 0 fixes the op at compile time (the switches in reduce_combine fold away); OPK < 0 takes it at run time.
template <typename TX, typename C, int OPK>
__global__ void __launch_bounds__(256)
reduce_row_kernel(const void* __restrict__ x, int xdt, void* __restrict__ out, int ydt,
                  const __grid_constant__ ReduceArgs A, int op_rt, bool to_partial) {
    const int op = OPK >= 0 ? OPK : op_rt;
    __shared__ C warp_acc[8];
    const C rcount = (C)A.rcount;
    const int64_t n_work = A.n_out * A.split;
    const int64_t inner = A.rshape[A.nr - 1], istride = A.rstride[A.nr - 1];
    for (int64_t w = blockIdx.x; w < n_work; w += gridDim.x) {
        const int64_t o = w / A.split;
        const int s = (int)(w % A.split);
        const int64_t base = kept_offset(A, o);
        const int64_t r0 = s * A.chunk;
        const int64_t r1 = r0 + A.chunk < A.n_red ? r0 + A.chunk : A.n_red;
        C acc = reduce_init<C>(op, ydt);
        // [r0, r1) in units of the flattened reduced space; split into sweeps over the innermost axis
        int64_t r = r0;
        while (r < r1) {
            const int64_t outer = r / inner, i0 = r - outer * inner;
            const int64_t i1 = (r1 - r) < (inner - i0) ? i0 + (r1 - r) : inner;
            int64_t obase = base;
            if (A.nr > 1) {
                int64_t q = outer;
#pragma unroll 1
                for (int d = A.nr - 2; d >= 0; d--) { const int64_t sh = A.rshape[d]; obase += (q % sh) * A.rstride[d]; q /= sh; }
            }
            bool done = false;
            if constexpr (std::is_same<TX, float>::value && std::is_same<C, float>::value) {
                const float* p = (const float*)x + obase + i0;
                if (istride == 1 && (((uintptr_t)p) & 15) == 0 && ((i1 - i0) & 3) == 0) {
                    const int64_t nv = (i1 - i0) >> 2;
                    // four independent 16-byte loads in flight per thread
                    for (int64_t v0 = threadIdx.x; v0 < nv; v0 += 4 * blockDim.x) {
                        float4 f[4];
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const int64_t v = v0 + u * blockDim.x;
                            const float idv = reduce_init<float>(op == OP_MEAN ? OP_ADD : op, B200JT_FLOAT32);
                            f[u] = v < nv ? __ldcs(reinterpret_cast<const float4*>(p) + v) : make_float4(idv, idv, idv, idv);
                            if (op == OP_MEAN && v >= nv) f[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                        }
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            float e0 = f[u].x, e1 = f[u].y, e2 = f[u].z, e3 = f[u].w;
                            if (op == OP_MEAN) { e0 *= rcount; e1 *= rcount; e2 *= rcount; e3 *= rcount; }
                            acc = reduce_combine<C>(op, reduce_combine<C>(op, reduce_combine<C>(op, reduce_combine<C>(op, acc, e0), e1), e2), e3);
                        }
                    }
                    done = true;
                }
            }
            if (!done) {
                for (int64_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
                    C v = load_x<TX, C>(x, xdt, obase + i * istride);
                    if (op == OP_MEAN) v = v * rcount;
                    acc = reduce_combine<C>(op, acc, v);
                }
            }
            r += i1 - i0;
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) acc = reduce_combine<C>(op, acc, shfl_down_c<C>(acc, d));
        if ((threadIdx.x & 31) == 0) warp_acc[threadIdx.x >> 5] = acc;
        __syncthreads();
        if (threadIdx.x == 0) {
            C t = warp_acc[0];
            for (int i = 1; i < (int)(blockDim.x >> 5); i++) t = reduce_combine<C>(op, t, warp_acc[i]);
            if (to_partial) ((C*)out)[w] = t; else store_as<C>(out, ydt, o, t);
        }
        __syncthreads();
    }
}

// One thread per (output, split); neighbouring threads own neighbouring outputs, so with the innermost axis kept
// every step of the serial fold is a coalesced row read. The reduced coordinates advance like an odometer (no
// division in the loop); four independent accumulators hide the load latency. Partials are laid out [split][n_out].
template <typename TX, typename C, int OPK>
__global__ void __launch_bounds__(256)
reduce_col_kernel(const void* __restrict__ x, int xdt, void* __restrict__ out, int ydt,
                  const __grid_constant__ ReduceArgs A, int op_rt, bool to_partial) {
    const int op = OPK >= 0 ? OPK : op_rt;
    const C rcount = (C)A.rcount;
    const int s = blockIdx.y;
    const int64_t r0 = s * A.chunk;
    const int64_t r1 = r0 + A.chunk < A.n_red ? r0 + A.chunk : A.n_red;
    const int nr = A.nr;
    for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < A.n_out; o += (int64_t)gridDim.x * blockDim.x) {
        const int64_t base = kept_offset(A, o);
        C acc0 = reduce_init<C>(op, ydt), acc1 = acc0, acc2 = acc0, acc3 = acc0;
        if (nr == 1) {
            const int64_t st = A.rstride[0];
            int64_t r = r0;
            for (; r + 8 <= r1; r += 8) {
                C v[8];
#pragma unroll
                for (int u = 0; u < 8; u++) v[u] = load_x<TX, C>(x, xdt, base + (r + u) * st);
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    if (op == OP_MEAN) v[u] *= rcount;
                    if ((u & 3) == 0) acc0 = reduce_combine<C>(op, acc0, v[u]);
                    else if ((u & 3) == 1) acc1 = reduce_combine<C>(op, acc1, v[u]);
                    else if ((u & 3) == 2) acc2 = reduce_combine<C>(op, acc2, v[u]);
                    else acc3 = reduce_combine<C>(op, acc3, v[u]);
                }
            }
            for (; r < r1; r++) {
                C v = load_x<TX, C>(x, xdt, base + r * st);
                if (op == OP_MEAN) v *= rcount;
                acc0 = reduce_combine<C>(op, acc0, v);
            }
        } else {
            int64_t idx[kMaxDims];
            int64_t off = base, q = r0;
#pragma unroll 1
            for (int d = nr - 1; d >= 0; d--) { const int64_t sh = A.rshape[d]; idx[d] = q % sh; q /= sh; off += idx[d] * A.rstride[d]; }
            for (int64_t r = r0; r < r1; r++) {
                C v = load_x<TX, C>(x, xdt, off);
                if (op == OP_MEAN) v *= rcount;
                acc0 = reduce_combine<C>(op, acc0, v);
#pragma unroll 1
                for (int d = nr - 1; d >= 0; d--) {
                    off += A.rstride[d];
                    if (++idx[d] < A.rshape[d]) break;
                    off -= A.rstride[d] * A.rshape[d];
                    idx[d] = 0;
                }
            }
        }
        const C acc = reduce_combine<C>(op, reduce_combine<C>(op, acc0, acc1), reduce_combine<C>(op, acc2, acc3));
        if (to_partial) ((C*)out)[(int64_t)s * A.n_out + o] = acc; else store_as<C>(out, ydt, o, acc);
    }
}

struct ReducePlan {
    ReduceArgs A;
    bool row = false;
    int cls = 0;          // 0 float, 1 double, 2 int64
    size_t workspace = 0;
};

static int class_of(int ydt) { return ydt == B200JT_FLOAT64 ? 1 : (dtype_is_float(ydt) ? 0 : 2); }
static int class_dtype(int cls) { return cls == 0 ? B200JT_FLOAT32 : cls == 1 ? B200JT_FLOAT64 : B200JT_INT64; }

static ReducePlan make_plan(const b200jt_tensor* x, const b200jt_tensor* y, uint32_t mask) {
    ReducePlan P; memset(&P.A, 0, sizeof(P.A));
    ReduceArgs& A = P.A;
    // canonical dims, outer -> inner
    int64_t shape[kMaxDims], stride[kMaxDims]; bool red[kMaxDims]; int n = 0;
    int64_t st = 1;
    int64_t xs[kMaxDims];
    for (int d = x->ndim - 1; d >= 0; d--) { xs[d] = st; st *= x->shape[d]; }
    for (int d = 0; d < x->ndim; d++) {
        if (x->shape[d] == 1) continue;
        bool r = mask >> d & 1;
        if (n && red[n - 1] == r) { shape[n - 1] *= x->shape[d]; stride[n - 1] = xs[d]; }
        else { shape[n] = x->shape[d]; stride[n] = xs[d]; red[n] = r; n++; }
    }
    A.n_out = 1; A.n_red = 1;
    for (int i = 0; i < n; i++) {
        if (red[i]) { A.rshape[A.nr] = shape[i]; A.rstride[A.nr] = stride[i]; A.nr++; A.n_red *= shape[i]; }
        else { A.kshape[A.nk] = shape[i]; A.kstride[A.nk] = stride[i]; A.nk++; A.n_out *= shape[i]; }
    }
    if (A.nr == 0) { A.nr = 1; A.rshape[0] = 1; A.rstride[0] = 0; }
    A.rcount = numel(x) ? (double)numel(y) / (double)numel(x) : 0.0;
    P.cls = class_of(y->dtype);
    const bool inner_reduced = n > 0 && red[n - 1];
    P.row = inner_reduced && A.n_red >= 256;
    A.split = 1; A.chunk = A.n_red;
    const int64_t target = 8LL * kNumSMs;
    if (P.row) {
        if (A.n_out < target && A.n_red >= 16384) {
            int64_t s = (target + A.n_out - 1) / A.n_out;
            int64_t smax = A.n_red / 4096;
            if (s > smax) s = smax;
            if (s > 1) { A.split = (int)s; A.chunk = (A.n_red + s - 1) / s; }
        }
    } else {
        const int64_t ctas = (A.n_out + 255) / 256;
        if (ctas < target && A.n_red >= 1024) {
            int64_t s = (target + ctas - 1) / ctas;
            int64_t smax = A.n_red / 256;
            if (s > smax) s = smax;
            if (s > 1024) s = 1024;
            if (s > 1) { A.split = (int)s; A.chunk = (A.n_red + s - 1) / s; }
        }
    }
    if (A.split > 1) P.workspace = (size_t)A.n_out * A.split * 8;
    return P;
}

template <typename TX, typename C, int OPK>
static void launch_stage_op(const void* xp, int xdt, void* out, int ydt, const ReduceArgs& A, int op, bool part, bool row,
                            cudaStream_t st) {
    if (row) {
        int64_t work = A.n_out * A.split;
        unsigned grid = (unsigned)(work < (int64_t)kNumSMs * 16 ? work : (int64_t)kNumSMs * 16);
        reduce_row_kernel<TX, C, OPK><<<grid, 256, 0, st>>>(xp, xdt, out, ydt, A, op, part);
    } else {
        dim3 grid(grid_for(A.n_out, 256), A.split);
        reduce_col_kernel<TX, C, OPK><<<grid, 256, 0, st>>>(xp, xdt, out, ydt, A, op, part);
    }
}

template <typename TX, typename C>
static void launch_stage(const void* xp, int xdt, void* out, int ydt, const ReduceArgs& A, int op, bool part, bool row,
                         cudaStream_t st) {
    // the common ops of typed inputs get a compile-time op; everything else shares the run-time variant
    if constexpr (!std::is_same<TX, void>::value) {
        switch (op) {
            case OP_ADD: return launch_stage_op<TX, C, OP_ADD>(xp, xdt, out, ydt, A, op, part, row, st);
            case OP_MEAN: return launch_stage_op<TX, C, OP_MEAN>(xp, xdt, out, ydt, A, op, part, row, st);
            case OP_MAX: return launch_stage_op<TX, C, OP_MAX>(xp, xdt, out, ydt, A, op, part, row, st);
            case OP_MIN: return launch_stage_op<TX, C, OP_MIN>(xp, xdt, out, ydt, A, op, part, row, st);
        }
    }
    launch_stage_op<TX, C, -1>(xp, xdt, out, ydt, A, op, part, row, st);
}

template <typename C>
static int run_class(const b200jt_tensor* x, const b200jt_tensor* y, int op, const ReducePlan& P, void* ws, cudaStream_t st) {
    const ReduceArgs& A = P.A;
    const bool part = A.split > 1;
    void* out1 = part ? ws : y->ptr;
    // typed loads for the common input dtypes of each accumulation class, run-time switch otherwise
    if (std::is_same<C, float>::value && x->dtype == B200JT_FLOAT32) launch_stage<float, C>(x->ptr, x->dtype, out1, y->dtype, A, op, part, P.row, st);
    else if (std::is_same<C, float>::value && x->dtype == B200JT_BFLOAT16) launch_stage<__nv_bfloat16, C>(x->ptr, x->dtype, out1, y->dtype, A, op, part, P.row, st);
    else if (std::is_same<C, int64_t>::value && x->dtype == B200JT_INT32) launch_stage<int32_t, C>(x->ptr, x->dtype, out1, y->dtype, A, op, part, P.row, st);
    else if (std::is_same<C, double>::value && x->dtype == B200JT_FLOAT64) launch_stage<double, C>(x->ptr, x->dtype, out1, y->dtype, A, op, part, P.row, st);
    else launch_stage<void, C>(x->ptr, x->dtype, out1, y->dtype, A, op, part, P.row, st);
    B200JT_LAUNCH_CHECK();
    if (!part) return 0;
    // second stage over the partials (already scaled for mean)
    ReduceArgs B; memset(&B, 0, sizeof(B));
    B.nk = 1; B.nr = 1; B.n_out = A.n_out; B.n_red = A.split; B.split = 1; B.chunk = A.split; B.rcount = 1.0;
    B.kshape[0] = A.n_out; B.rshape[0] = A.split;
    const int op2 = op == OP_MEAN ? OP_ADD : op;
    const int cdt = class_dtype(P.cls);
    if (P.row) { B.kstride[0] = A.split; B.rstride[0] = 1; }
    else       { B.kstride[0] = 1; B.rstride[0] = A.n_out; }
    launch_stage<C, C>(ws, cdt, y->ptr, y->dtype, B, op2, false, false, st);
    B200JT_LAUNCH_CHECK();
    return 0;
}

static int check_args(const b200jt_tensor* x, const b200jt_tensor* y, const char* op, uint32_t mask, int* opc) {
    B200JT_CHECK_ARG(valid_tensor(x) && valid_tensor(y), "invalid tensor descriptor");
    B200JT_CHECK_ARG(x->ndim == y->ndim, "reduce: y must be passed with x's rank");
    for (int d = 0; d < x->ndim; d++)
        B200JT_CHECK_ARG(y->shape[d] == ((mask >> d & 1) ? 1 : x->shape[d]), "reduce: y shape does not match reduce_mask");
    *opc = binary_op_from_name(op);
    bool ok = *opc == OP_ADD || *opc == OP_MEAN || *opc == OP_MUL || *opc == OP_MAX || *opc == OP_MIN ||
              *opc == OP_LAND || *opc == OP_LOR || *opc == OP_LXOR ||
              ((*opc == OP_BAND || *opc == OP_BOR || *opc == OP_BXOR) && !dtype_is_float(y->dtype));
    B200JT_CHECK_ARG(ok, std::string("unsupported reduce op '") + op + "'");
    return 0;
}

}  // namespace b200jt

using namespace b200jt;

extern "C" size_t b200jt_reduce_workspace(const b200jt_tensor* x, const b200jt_tensor* y, const char* op, uint32_t reduce_mask) {
    int opc;
    if (check_args(x, y, op, reduce_mask, &opc)) return 0;
    return make_plan(x, y, reduce_mask).workspace;
}

extern "C" int b200jt_reduce(const b200jt_tensor* x, const b200jt_tensor* y, const char* op, uint32_t reduce_mask,
                             void* workspace, size_t workspace_bytes, void* stream) {
    int opc;
    int rc = check_args(x, y, op, reduce_mask, &opc);
    if (rc) return rc;
    if (numel(y) == 0) return 0;
    ReducePlan P = make_plan(x, y, reduce_mask);
    if (numel(x) == 0) { P.A.n_red = 0; P.A.chunk = 0; P.A.split = 1; P.workspace = 0; P.row = false; }
    B200JT_CHECK_ARG(workspace_bytes >= P.workspace && (P.workspace == 0 || workspace),
                     "workspace too small: need " + std::to_string(P.workspace) + " bytes");
    cudaStream_t st = (cudaStream_t)stream;
    switch (P.cls) {
        case 0: return run_class<float>(x, y, opc, P, workspace, st);
        case 1: return run_class<double>(x, y, opc, P, workspace, st);
        default: return run_class<int64_t>(x, y, opc, P, workspace, st);
    }
}
