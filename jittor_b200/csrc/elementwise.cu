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

// float32 fast path: contiguous, same shape, 128-bit accesses
__global__ void __launch_bounds__(256)
binary_f32_vec_kernel(const float4* __restrict__ x, const float4* __restrict__ y, float4* __restrict__ z, int64_t n4, int op) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        float4 a = x[i], b = y[i], r;
        r.x = binary_compute<float>(op, a.x, b.x); r.y = binary_compute<float>(op, a.y, b.y);
        r.z = binary_compute<float>(op, a.z, b.z); r.w = binary_compute<float>(op, a.w, b.w);
        z[i] = r;
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

template <typename T>
__global__ void __launch_bounds__(256)
broadcast_kernel(const T* __restrict__ x, T* __restrict__ z, const __grid_constant__ BcastArgs A, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t xo, yo, co;
        bcast_offsets(A, i, xo, yo, co);
        z[i] = x[xo];
    }
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
    if (same && cc == 0 && x->dtype == B200JT_FLOAT32 && y->dtype == B200JT_FLOAT32 && z->dtype == B200JT_FLOAT32 &&
        n % 4 == 0 && ((uintptr_t)x->ptr | (uintptr_t)y->ptr | (uintptr_t)z->ptr) % 16 == 0) {
        binary_f32_vec_kernel<<<grid_for(n / 4, 256), 256, 0, st>>>((const float4*)x->ptr, (const float4*)y->ptr, (float4*)z->ptr, n / 4, oc);
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
