// Element-wise ops with the broadcast_to the reference inserts fused in (python/jittor/src/ops/binary_op.cc:435-441):
// operands are addressed with stride 0 on their size-1 axes, nothing is materialised.
// Arithmetic follows python/jittor/src/type/common_op_type.cc:82-152: operands are promoted to the compute class
// of the output dtype (float32 / float64 / int64), the result is converted with C rules.
#include "atomic_ops.cuh"

namespace b200jt {

struct BcastArgs {
    int32_t ndim;
    int64_t zshape[kMaxDims];
    int64_t xstride[kMaxDims];   // 0 on broadcast axes
    int64_t ystride[kMaxDims];
    int64_t cstride[kMaxDims];
};

enum UnaryCode : int {
    U_CAST = 0, U_NEG, U_ABS, U_LNOT, U_BNOT, U_LOG, U_EXP, U_SQRT, U_ROUND, U_FLOOR, U_CEIL,
    U_SIN, U_ASIN, U_SINH, U_ASINH, U_TAN, U_ATAN, U_TANH, U_ATANH, U_COS, U_ACOS, U_COSH, U_ACOSH,
    U_SIGMOID, U_ERF, U_ERFINV, U_INVALID
};

template <typename C>
__device__ __forceinline__ C binary_compute(int op, C a, C b) {
    switch (op) {
        case OP_ADD: return a + b;
        case OP_SUB: return a - b;
        case OP_MUL: return a * b;
        case OP_DIV: case OP_FLOORDIV:
            if constexpr (std::is_integral<C>::value) return b != 0 ? a / b : 0; else return a / b;
        case OP_MOD:
            if constexpr (std::is_integral<C>::value) return b != 0 ? a % b : 0;
            else return a - floor(a / b) * b;
        case OP_POW:
            if constexpr (std::is_integral<C>::value) return (C)pow((double)a, (double)b);
            else return pow(a, b);
        case OP_MAX: return a > b ? a : b;
        case OP_MIN: return b < a ? b : a;
        case OP_LT: return (C)(a < b);
        case OP_LE: return (C)(a <= b);
        case OP_GT: return (C)(a > b);
        case OP_GE: return (C)(a >= b);
        case OP_EQ: return (C)(a == b);
        case OP_NE: return (C)(a != b);
        case OP_LAND: return (C)((a != 0) && (b != 0));
        case OP_LOR: return (C)((a != 0) || (b != 0));
        case OP_LXOR: return (C)((a != 0) != (b != 0));
        case OP_BAND: if constexpr (std::is_integral<C>::value) return a & b; else return a;
        case OP_BOR:  if constexpr (std::is_integral<C>::value) return a | b; else return a;
        case OP_BXOR: if constexpr (std::is_integral<C>::value) return a ^ b; else return a;
        case OP_SHL:  if constexpr (std::is_integral<C>::value) return a << b; else return a;
        case OP_SHR:  if constexpr (std::is_integral<C>::value) return a >> b; else return a;
    }
    return a;
}

template <typename C>
__device__ __forceinline__ C unary_compute(int op, C a, bool f32_out) {
    if constexpr (std::is_integral<C>::value) {
        switch (op) {
            case U_NEG: return -a;
            case U_ABS: return a < 0 ? -a : a;
            case U_LNOT: return (C)(a == 0);
            case U_BNOT: return ~a;
        }
        return a;
    } else {
        switch (op) {
            case U_NEG: return -a;
            case U_ABS: return fabs(a);
            case U_LNOT: return (C)(a == 0);
            case U_LOG: return log(a);
            case U_EXP: return exp(a);
            case U_SQRT: return sqrt(a);
            case U_ROUND: return round(a);
            case U_FLOOR: return floor(a);
            case U_CEIL: return ceil(a);
            case U_SIN: return sin(a);
            case U_ASIN: return asin(a);
            case U_SINH: return sinh(a);
            case U_ASINH: return asinh(a);
            case U_TAN: return tan(a);
            case U_ATAN: return atan(a);
            case U_TANH: return tanh(a);
            case U_ATANH: return atanh(a);
            case U_COS: return cos(a);
            case U_ACOS: return acos(a);
            case U_COSH: return cosh(a);
            case U_ACOSH: return acosh(a);
            case U_SIGMOID: { C lim = f32_out ? (C)30 : (C)300; C t = -a < lim ? -a : lim; return (C)1 / ((C)1 + exp(t)); }
            case U_ERF: return erf(a);
            case U_ERFINV: return erfinv(a);
        }
        return a;
    }
}

// flat index of z -> strided offsets of up to three operands
__device__ __forceinline__ void bcast_offsets(const BcastArgs& A, int64_t flat, int64_t& xo, int64_t& yo, int64_t& co) {
    xo = yo = co = 0;
#pragma unroll 1
    for (int d = A.ndim - 1; d >= 0; d--) {
        int64_t s = A.zshape[d];
        int64_t i = flat % s; flat /= s;
        xo += i * A.xstride[d]; yo += i * A.ystride[d]; co += i * A.cstride[d];
    }
}

template <typename C>
__global__ void __launch_bounds__(256)
binary_kernel(const void* __restrict__ x, int xdt, const void* __restrict__ y, int ydt,
              void* __restrict__ z, int zdt, const __grid_constant__ BcastArgs A, int64_t n, int op, bool same_shape) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t xo = i, yo = i, co;
        if (!same_shape) bcast_offsets(A, i, xo, yo, co);
        C a = load_as<C>(x, xdt, xo), b = load_as<C>(y, ydt, yo);
        store_as<C>(z, zdt, i, binary_compute<C>(op, a, b));
    }
}

template <typename C>
__global__ void __launch_bounds__(256)
unary_kernel(const void* __restrict__ x, int xdt, void* __restrict__ y, int ydt, int64_t n, int op) {
    const bool f32_out = ydt != B200JT_FLOAT64;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        C a = load_as<C>(x, xdt, i);
        if (op == U_CAST && ydt == B200JT_BOOL) { ((uint8_t*)y)[i] = a != 0; continue; }
        store_as<C>(y, ydt, i, unary_compute<C>(op, a, f32_out));
    }
}

template <typename C>
__global__ void __launch_bounds__(256)
ternary_kernel(const void* __restrict__ c, int cdt, const void* __restrict__ x, int xdt, const void* __restrict__ y, int ydt,
               void* __restrict__ z, int zdt, const __grid_constant__ BcastArgs A, int64_t n, bool same_shape) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t xo = i, yo = i, co = i;
        if (!same_shape) bcast_offsets(A, i, xo, yo, co);
        bool cond = load_as<double>(c, cdt, co) != 0;
        store_as<C>(z, zdt, i, cond ? load_as<C>(x, xdt, xo) : load_as<C>(y, ydt, yo));
    }
}

// ---- fast paths: float32 / bfloat16, op known at compile time, 16-byte accesses --------------------------------
// Operand modes of y relative to z (x is always full; non-commutative ops get SWAP when the roles are exchanged):
//   FULL   same shape                        SCALAR one element
//   SUFFIX y is z's trailing block (bias over rows): index = i mod numel(y)
//   PREFIX y has z's leading axes and size-1 trailing axes (per-row scalar): index = i / (numel(z) / numel(y))
enum BMode : int { B_FULL = 0, B_SCALAR, B_SUFFIX, B_PREFIX };

template <typename T> struct V16;
template <> struct V16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void ld(const float* p, float* o) { float4 v = *reinterpret_cast<const float4*>(p); o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w; }
    static __device__ __forceinline__ void st(float* p, const float* o) { *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]); }
    static __device__ __forceinline__ float ld1(const float* p) { return *p; }
};
template <> struct V16<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void ld(const __nv_bfloat16* p, float* o) {
        uint4 v = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; i++) { float2 f = __bfloat1622float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
    }
    static __device__ __forceinline__ void st(__nv_bfloat16* p, const float* o) {
        uint4 v; __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = v;
    }
    static __device__ __forceinline__ float ld1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
};

template <typename T, int OP, int MODE, bool SWAP>
__global__ void __launch_bounds__(256)
binary_fast_kernel(const T* __restrict__ x, const T* __restrict__ y, T* __restrict__ z, uint32_t n_vec, uint32_t ydiv) {
    constexpr int N = V16<T>::N;
    for (uint32_t v = blockIdx.x * blockDim.x + threadIdx.x; v < n_vec; v += gridDim.x * blockDim.x) {
        float a[N], b[N], r[N];
        V16<T>::ld(x + (size_t)v * N, a);
        if (MODE == B_FULL) V16<T>::ld(y + (size_t)v * N, b);
        else if (MODE == B_SUFFIX) V16<T>::ld(y + (size_t)(v % ydiv) * N, b);          // ydiv = numel(y) / N
        else {
            const float s = V16<T>::ld1(y + (MODE == B_SCALAR ? 0u : v / ydiv));       // ydiv = inner / N
#pragma unroll
            for (int e = 0; e < N; e++) b[e] = s;
        }
#pragma unroll
        for (int e = 0; e < N; e++) r[e] = SWAP ? binary_compute<float>(OP, b[e], a[e]) : binary_compute<float>(OP, a[e], b[e]);
        V16<T>::st(z + (size_t)v * N, r);
    }
}

template <typename TI, typename TO, int OP>
__global__ void __launch_bounds__(256)
unary_fast_kernel(const TI* __restrict__ x, TO* __restrict__ y, uint32_t n8) {
    // 8 elements per thread: two 16-byte vectors of float32 or one of bfloat16
    for (uint32_t v = blockIdx.x * blockDim.x + threadIdx.x; v < n8; v += gridDim.x * blockDim.x) {
        float a[8];
#pragma unroll
        for (int k = 0; k < 8 / V16<TI>::N; k++) V16<TI>::ld(x + (size_t)v * 8 + k * V16<TI>::N, a + k * V16<TI>::N);
#pragma unroll
        for (int e = 0; e < 8; e++) a[e] = unary_compute<float>(OP, a[e], true);
#pragma unroll
        for (int k = 0; k < 8 / V16<TO>::N; k++) V16<TO>::st(y + (size_t)v * 8 + k * V16<TO>::N, a + k * V16<TO>::N);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
broadcast_kernel(const T* __restrict__ x, T* __restrict__ z, const __grid_constant__ BcastArgs A, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t xo, yo, co;
        bcast_offsets(A, i, xo, yo, co);
        z[i] = x[xo];
    }
}

// Broadcast over ONE contiguous group of axes: z[o][m][i] = x[o][i] (a scalar: O = I = 1; a row vector stretched over rows:
// O = 1; a per-row value stretched along the row: I = 1). 16-byte stores, no per-axis index arithmetic.
//   INNER: I * sizeof(T) is a multiple of 16 -- both sides move as uint4, z4[(o*M + m)*I4 + i4] = x4[o*I4 + i4];
//  !INNER: I == 1 and M * sizeof(T) is a multiple of 16 -- a 16-byte vector of z lies inside one o and repeats x[o].
template <typename T, bool INNER>
__global__ void __launch_bounds__(256)
broadcast_group_kernel(const T* __restrict__ x, uint4* __restrict__ z4, int64_t nvec, int64_t M, int64_t I4) {
    constexpr int PER = 16 / sizeof(T);
    for (int64_t v = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * blockDim.x) {
        if (INNER) {
            const int64_t t = v / I4, i4 = v - t * I4;
            z4[v] = __ldg(reinterpret_cast<const uint4*>(x) + (t / M) * I4 + i4);
        } else {
            const T val = __ldg(x + v / (M / PER));
            __align__(16) T rep[PER];
#pragma unroll
            for (int e = 0; e < PER; e++) rep[e] = val;
            z4[v] = *reinterpret_cast<const uint4*>(rep);
        }
    }
}

// Splits z's axes as outer x (one contiguous run of broadcast axes) x inner; false if the broadcast axes (extent > 1) are
// not one run. Axes of extent 1 belong to whichever side they touch.
static bool broadcast_group(const b200jt_tensor* z, uint32_t mask, int64_t* O, int64_t* M, int64_t* I) {
    int first = -1, last = -1;
    for (int d = 0; d < z->ndim; d++)
        if ((mask >> d & 1) && z->shape[d] != 1) { if (first < 0) first = d; last = d; }
    if (first < 0) return false;                               // nothing is stretched: a plain copy, left to the general kernel
    *O = *M = *I = 1;
    for (int d = 0; d < z->ndim; d++) {
        if (d < first) *O *= z->shape[d];
        else if (d > last) *I *= z->shape[d];
        else if ((mask >> d & 1) || z->shape[d] == 1) *M *= z->shape[d];
        else return false;                                     // a kept axis between two stretched ones
    }
    return true;
}

template <typename T>
static bool launch_broadcast_group(const b200jt_tensor* x, const b200jt_tensor* z, uint32_t mask, cudaStream_t st) {
    int64_t O, M, I;
    if (!broadcast_group(z, mask, &O, &M, &I)) return false;
    if (((uintptr_t)z->ptr & 15) != 0) return false;
    constexpr int PER = 16 / sizeof(T);
    const int64_t nvec = O * M * I / PER;
    if (I % PER == 0 && ((uintptr_t)x->ptr & 15) == 0) {
        broadcast_group_kernel<T, true><<<grid_for(nvec, 256), 256, 0, st>>>((const T*)x->ptr, (uint4*)z->ptr, nvec, M, I / PER);
        return true;
    }
    if (I == 1 && M % PER == 0) {
        broadcast_group_kernel<T, false><<<grid_for(nvec, 256), 256, 0, st>>>((const T*)x->ptr, (uint4*)z->ptr, nvec, M, 1);
        return true;
    }
    return false;
}

static bool fill_strides(const b200jt_tensor* t, const b200jt_tensor* z, int64_t* stride, bool* same) {
    if (t->ndim != z->ndim) return false;
    int64_t st = 1;
    for (int d = z->ndim - 1; d >= 0; d--) {
        if (t->shape[d] == z->shape[d]) stride[d] = st;
        else if (t->shape[d] == 1) { stride[d] = 0; *same = false; }
        else return false;
        st *= t->shape[d];
    }
    return true;
}

static UnaryCode unary_from_name(const char* n) {
    static const struct { const char* name; UnaryCode code; } tab[] = {
        {"negative", U_NEG}, {"abs", U_ABS}, {"logical_not", U_LNOT}, {"bitwise_not", U_BNOT}, {"log", U_LOG},
        {"exp", U_EXP}, {"sqrt", U_SQRT}, {"round", U_ROUND}, {"floor", U_FLOOR}, {"ceil", U_CEIL},
        {"round_int", U_ROUND}, {"floor_int", U_FLOOR}, {"ceil_int", U_CEIL}, {"sin", U_SIN}, {"asin", U_ASIN},
        {"sinh", U_SINH}, {"asinh", U_ASINH}, {"tan", U_TAN}, {"atan", U_ATAN}, {"tanh", U_TANH}, {"atanh", U_ATANH},
        {"cos", U_COS}, {"acos", U_ACOS}, {"cosh", U_COSH}, {"acosh", U_ACOSH}, {"sigmoid", U_SIGMOID},
        {"erf", U_ERF}, {"erfinv", U_ERFINV}, {"cast", U_CAST}};
    for (auto& e : tab) if (strcmp(e.name, n) == 0) return e.code;
    if (dtype_from_name(n) >= 0) return U_CAST;
    return U_INVALID;
}

// compute class: 0 = float32, 1 = float64, 2 = int64
static int compute_class(int a, int b) {
    if (a == B200JT_FLOAT64 || b == B200JT_FLOAT64) return 1;
    if (dtype_is_float(a) || dtype_is_float(b)) return 0;
    return 2;
}

// classification of an operand against z for the fast path
static int bcast_mode(const b200jt_tensor* t, const b200jt_tensor* z, int64_t* div, int vecn) {
    const int64_t nt = numel(t), nz = numel(z);
    if (nt == nz) { *div = 1; return B_FULL; }
    if (nt == 1) { *div = 1; return B_SCALAR; }
    // suffix: leading axes of t are 1, the rest equal z
    int d = 0;
    while (d < z->ndim && t->shape[d] == 1) d++;
    bool suffix = true;
    for (int k = d; k < z->ndim; k++) suffix &= t->shape[k] == z->shape[k];
    if (suffix && nt % vecn == 0) { *div = nt / vecn; return B_SUFFIX; }
    // prefix: trailing axes of t are 1, the leading ones equal z
    int e = z->ndim;
    while (e > 0 && t->shape[e - 1] == 1) e--;
    bool prefix = true;
    for (int k = 0; k < e; k++) prefix &= t->shape[k] == z->shape[k];
    const int64_t inner = nz / nt;
    if (prefix && inner % vecn == 0) { *div = inner / vecn; return B_PREFIX; }
    return -1;
}

template <typename T, int OP>
static bool launch_binary_fast(const void* x, const void* y, void* z, int mode, bool swap, uint32_t n_vec, uint32_t div, cudaStream_t st) {
    const unsigned grid = grid_for(n_vec, 256);
#define B200JT_BF(M, S) binary_fast_kernel<T, OP, M, S><<<grid, 256, 0, st>>>((const T*)x, (const T*)y, (T*)z, n_vec, div)
    switch (mode) {
        case B_FULL: if (swap) B200JT_BF(B_FULL, true); else B200JT_BF(B_FULL, false); break;
        case B_SCALAR: if (swap) B200JT_BF(B_SCALAR, true); else B200JT_BF(B_SCALAR, false); break;
        case B_SUFFIX: if (swap) B200JT_BF(B_SUFFIX, true); else B200JT_BF(B_SUFFIX, false); break;
        case B_PREFIX: if (swap) B200JT_BF(B_PREFIX, true); else B200JT_BF(B_PREFIX, false); break;
        default: return false;
    }
#undef B200JT_BF
    return true;
}

template <typename T>
static bool binary_fast(int op, const void* x, const void* y, void* z, int mode, bool swap, uint32_t n_vec, uint32_t div, cudaStream_t st) {
    switch (op) {
        case OP_ADD: return launch_binary_fast<T, OP_ADD>(x, y, z, mode, swap, n_vec, div, st);
        case OP_SUB: return launch_binary_fast<T, OP_SUB>(x, y, z, mode, swap, n_vec, div, st);
        case OP_MUL: return launch_binary_fast<T, OP_MUL>(x, y, z, mode, swap, n_vec, div, st);
        case OP_DIV: return launch_binary_fast<T, OP_DIV>(x, y, z, mode, swap, n_vec, div, st);
        case OP_MAX: return launch_binary_fast<T, OP_MAX>(x, y, z, mode, swap, n_vec, div, st);
        case OP_MIN: return launch_binary_fast<T, OP_MIN>(x, y, z, mode, swap, n_vec, div, st);
    }
    return false;
}

// Returns true if the fast path took the call.
static bool try_binary_fast(const b200jt_tensor* x, const b200jt_tensor* y, const b200jt_tensor* z, int op, cudaStream_t st) {
    const int dt = z->dtype;
    if ((dt != B200JT_FLOAT32 && dt != B200JT_BFLOAT16) || x->dtype != dt || y->dtype != dt) return false;
    const int vecn = dt == B200JT_FLOAT32 ? 4 : 8;
    const int64_t n = numel(z);
    if (n % vecn != 0 || n / vecn >= (1LL << 32)) return false;
    if ((((uintptr_t)x->ptr | (uintptr_t)y->ptr | (uintptr_t)z->ptr) & 15) != 0) return false;
    const b200jt_tensor* full = x; const b200jt_tensor* other = y; bool swap = false;
    if (numel(x) != n) { full = y; other = x; swap = true; }
    if (numel(full) != n) return false;
    int64_t div = 1;
    const int mode = bcast_mode(other, z, &div, vecn);
    if (mode < 0 || div >= (1LL << 32)) return false;
    if (dt == B200JT_FLOAT32) return binary_fast<float>(op, full->ptr, other->ptr, z->ptr, mode, swap, (uint32_t)(n / vecn), (uint32_t)div, st);
    return binary_fast<__nv_bfloat16>(op, full->ptr, other->ptr, z->ptr, mode, swap, (uint32_t)(n / vecn), (uint32_t)div, st);
}

template <typename TI, typename TO>
static bool unary_fast(int uc, const void* x, void* y, uint32_t n8, cudaStream_t st) {
    const unsigned grid = grid_for(n8, 256);
#define B200JT_UF(OP) case OP: unary_fast_kernel<TI, TO, OP><<<grid, 256, 0, st>>>((const TI*)x, (TO*)y, n8); return true
    switch (uc) {
        B200JT_UF(U_CAST); B200JT_UF(U_NEG); B200JT_UF(U_ABS); B200JT_UF(U_EXP); B200JT_UF(U_LOG); B200JT_UF(U_SQRT);
        B200JT_UF(U_TANH); B200JT_UF(U_SIGMOID);
    }
#undef B200JT_UF
    return false;
}

static bool try_unary_fast(const b200jt_tensor* x, const b200jt_tensor* y, int uc, cudaStream_t st) {
    const bool xf = x->dtype == B200JT_FLOAT32, xb = x->dtype == B200JT_BFLOAT16;
    const bool yf = y->dtype == B200JT_FLOAT32, yb = y->dtype == B200JT_BFLOAT16;
    const int64_t n = numel(x);
    if (!(xf || xb) || !(yf || yb) || n % 8 != 0 || n / 8 >= (1LL << 32)) return false;
    if ((((uintptr_t)x->ptr | (uintptr_t)y->ptr) & 15) != 0) return false;
    const uint32_t n8 = (uint32_t)(n / 8);
    if (xf && yf) return unary_fast<float, float>(uc, x->ptr, y->ptr, n8, st);
    if (xf && yb) return unary_fast<float, __nv_bfloat16>(uc, x->ptr, y->ptr, n8, st);
    if (xb && yf) return unary_fast<__nv_bfloat16, float>(uc, x->ptr, y->ptr, n8, st);
    return unary_fast<__nv_bfloat16, __nv_bfloat16>(uc, x->ptr, y->ptr, n8, st);
}

}  // namespace b200jt

using namespace b200jt;

extern "C" int b200jt_binary(const b200jt_tensor* x, const b200jt_tensor* y, const b200jt_tensor* z, const char* op, void* stream) {
    B200JT_CHECK_ARG(valid_tensor(x) && valid_tensor(y) && valid_tensor(z), "invalid tensor descriptor");
    OpCode oc = binary_op_from_name(op);
    B200JT_CHECK_ARG(oc != OP_INVALID && oc != OP_MEAN && oc != OP_VOID, std::string("unknown binary op '") + op + "'");
    BcastArgs A; memset(&A, 0, sizeof(A));
    A.ndim = z->ndim;
    bool same = true;
    for (int d = 0; d < z->ndim; d++) A.zshape[d] = z->shape[d];
    B200JT_CHECK_ARG(fill_strides(x, z, A.xstride, &same) && fill_strides(y, z, A.ystride, &same),
                     "Shape not match, x:" + shape_str(x) + " y:" + shape_str(y) + " z:" + shape_str(z));
    const int64_t n = numel(z);
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    // comparisons / logical ops compute in the promoted input class; the rest in the output class
    const bool cmp = z->dtype == B200JT_BOOL;
    int cc = cmp ? compute_class(x->dtype, y->dtype) : compute_class(z->dtype, z->dtype);
    if (!cmp && oc == OP_POW && cc == 2) cc = 2;
    const unsigned grid = grid_for(n, 256);
    if (try_binary_fast(x, y, z, oc, st)) {
        // float32 / bfloat16 with a compile-time op and 16-byte accesses
    } else if (cc == 0) binary_kernel<float><<<grid, 256, 0, st>>>(x->ptr, x->dtype, y->ptr, y->dtype, z->ptr, z->dtype, A, n, oc, same);
    else if (cc == 1)   binary_kernel<double><<<grid, 256, 0, st>>>(x->ptr, x->dtype, y->ptr, y->dtype, z->ptr, z->dtype, A, n, oc, same);
    else                binary_kernel<int64_t><<<grid, 256, 0, st>>>(x->ptr, x->dtype, y->ptr, y->dtype, z->ptr, z->dtype, A, n, oc, same);
    B200JT_LAUNCH_CHECK();
    return 0;
}

extern "C" int b200jt_unary(const b200jt_tensor* x, const b200jt_tensor* y, const char* op, void* stream) {
    B200JT_CHECK_ARG(valid_tensor(x) && valid_tensor(y), "invalid tensor descriptor");
    B200JT_CHECK_ARG(numel(x) == numel(y), "unary: x and y differ in size");
    UnaryCode uc = unary_from_name(op);
    B200JT_CHECK_ARG(uc != U_INVALID, std::string("unknown unary op '") + op + "'");
    const int64_t n = numel(x);
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    // float ops on integer inputs compute in the output's float class; casts compute in the input class
    int cc = uc == U_CAST ? compute_class(x->dtype, x->dtype)
                          : (dtype_is_float(y->dtype) ? compute_class(y->dtype, y->dtype) : compute_class(x->dtype, x->dtype));
    const unsigned grid = grid_for(n, 256);
    if (try_unary_fast(x, y, uc, st)) { B200JT_LAUNCH_CHECK(); return 0; }
    if (cc == 0)      unary_kernel<float><<<grid, 256, 0, st>>>(x->ptr, x->dtype, y->ptr, y->dtype, n, uc);
    else if (cc == 1) unary_kernel<double><<<grid, 256, 0, st>>>(x->ptr, x->dtype, y->ptr, y->dtype, n, uc);
    else              unary_kernel<int64_t><<<grid, 256, 0, st>>>(x->ptr, x->dtype, y->ptr, y->dtype, n, uc);
    B200JT_LAUNCH_CHECK();
    return 0;
}

extern "C" int b200jt_ternary(const b200jt_tensor* cond, const b200jt_tensor* x, const b200jt_tensor* y,
                              const b200jt_tensor* z, void* stream) {
    B200JT_CHECK_ARG(valid_tensor(cond) && valid_tensor(x) && valid_tensor(y) && valid_tensor(z), "invalid tensor descriptor");
    BcastArgs A; memset(&A, 0, sizeof(A));
    A.ndim = z->ndim;
    bool same = true;
    for (int d = 0; d < z->ndim; d++) A.zshape[d] = z->shape[d];
    B200JT_CHECK_ARG(fill_strides(x, z, A.xstride, &same) && fill_strides(y, z, A.ystride, &same) &&
                     fill_strides(cond, z, A.cstride, &same), "ternary: shapes do not match");
    const int64_t n = numel(z);
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const int cc = compute_class(z->dtype, z->dtype);
    const unsigned grid = grid_for(n, 256);
    if (cc == 0)      ternary_kernel<float><<<grid, 256, 0, st>>>(cond->ptr, cond->dtype, x->ptr, x->dtype, y->ptr, y->dtype, z->ptr, z->dtype, A, n, same);
    else if (cc == 1) ternary_kernel<double><<<grid, 256, 0, st>>>(cond->ptr, cond->dtype, x->ptr, x->dtype, y->ptr, y->dtype, z->ptr, z->dtype, A, n, same);
    else              ternary_kernel<int64_t><<<grid, 256, 0, st>>>(cond->ptr, cond->dtype, x->ptr, x->dtype, y->ptr, y->dtype, z->ptr, z->dtype, A, n, same);
    B200JT_LAUNCH_CHECK();
    return 0;
}

extern "C" int b200jt_broadcast_to(const b200jt_tensor* x, const b200jt_tensor* z, uint32_t bcast_mask, void* stream) {
    B200JT_CHECK_ARG(valid_tensor(x) && valid_tensor(z), "invalid tensor descriptor");
    B200JT_CHECK_ARG(x->dtype == z->dtype && x->ndim == z->ndim, "broadcast_to: x must have z's dtype and rank");
    BcastArgs A; memset(&A, 0, sizeof(A));
    A.ndim = z->ndim;
    int64_t st_ = 1;
    for (int d = z->ndim - 1; d >= 0; d--) {
        A.zshape[d] = z->shape[d];
        if (bcast_mask >> d & 1) {
            B200JT_CHECK_ARG(x->shape[d] == 1, "broadcast_to: x must have size 1 on broadcast axes");
            A.xstride[d] = 0;
        } else {
            B200JT_CHECK_ARG(x->shape[d] == z->shape[d], "Shape not match " + shape_str(x) + " " + shape_str(z));
            A.xstride[d] = st_;
        }
        st_ *= x->shape[d];
    }
    const int64_t n = numel(z);
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    bool done = false;
    switch (dtype_size(x->dtype)) {
        case 1: done = launch_broadcast_group<uint8_t>(x, z, bcast_mask, st); break;
        case 2: done = launch_broadcast_group<uint16_t>(x, z, bcast_mask, st); break;
        case 4: done = launch_broadcast_group<uint32_t>(x, z, bcast_mask, st); break;
        default: done = launch_broadcast_group<uint64_t>(x, z, bcast_mask, st);
    }
    if (done) { B200JT_LAUNCH_CHECK(); return 0; }
    const unsigned grid = grid_for(n, 256);
    switch (dtype_size(x->dtype)) {
        case 1: broadcast_kernel<uint8_t><<<grid, 256, 0, st>>>((const uint8_t*)x->ptr, (uint8_t*)z->ptr, A, n); break;
        case 2: broadcast_kernel<uint16_t><<<grid, 256, 0, st>>>((const uint16_t*)x->ptr, (uint16_t*)z->ptr, A, n); break;
        case 4: broadcast_kernel<uint32_t><<<grid, 256, 0, st>>>((const uint32_t*)x->ptr, (uint32_t*)z->ptr, A, n); break;
        default: broadcast_kernel<uint64_t><<<grid, 256, 0, st>>>((const uint64_t*)x->ptr, (uint64_t*)z->ptr, A, n);
    }
    B200JT_LAUNCH_CHECK();
    return 0;
}
