// Scalar semantics of the reduce-class ops and their atomic forms.
// Table followed: python/jittor/src/type/common_op_type.cc:117-151 (CPU column: init_maximum is
// numeric lowest(), not -inf). Float max/min use native integer atomics on the IEEE bit pattern
// (sign-split trick) instead of the reference's encode/decode passes
// (python/jittor/src/misc/cuda_atomic.h:16-60), which removes its separate fix-up kernel.
#pragma once
#include "common.cuh"
#include <cfloat>
#include <climits>

namespace b200jt {

// element types used by the templates (bool is stored as uint8 and handled by the logical ops)
template <typename T> struct TypeInfo;
#define B200JT_TI(T, CODE, ISF) template <> struct TypeInfo<T> { static constexpr int code = CODE; static constexpr bool is_float = ISF; };
B200JT_TI(int8_t, B200JT_INT8, false) B200JT_TI(uint8_t, B200JT_UINT8, false) B200JT_TI(int16_t, B200JT_INT16, false)
B200JT_TI(int32_t, B200JT_INT32, false) B200JT_TI(int64_t, B200JT_INT64, false) B200JT_TI(__half, B200JT_FLOAT16, true)
B200JT_TI(__nv_bfloat16, B200JT_BFLOAT16, true) B200JT_TI(float, B200JT_FLOAT32, true) B200JT_TI(double, B200JT_FLOAT64, true)
#undef B200JT_TI

template <typename T> struct Compute { using type = T; };
template <> struct Compute<__half> { using type = float; };
template <> struct Compute<__nv_bfloat16> { using type = float; };

template <typename T> __host__ __device__ inline typename Compute<T>::type to_compute(T v) { return v; }
template <> __host__ __device__ inline float to_compute<__half>(__half v) { return __half2float(v); }
template <> __host__ __device__ inline float to_compute<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __host__ __device__ inline T from_compute(typename Compute<T>::type v) { return (T)v; }
template <> __host__ __device__ inline __half from_compute<__half>(float v) { return __float2half(v); }
template <> __host__ __device__ inline __nv_bfloat16 from_compute<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

template <typename C> __host__ __device__ inline C lowest_of();
template <typename C> __host__ __device__ inline C highest_of();
#define B200JT_LIM(C, LO, HI) template <> __host__ __device__ inline C lowest_of<C>() { return LO; } \
                              template <> __host__ __device__ inline C highest_of<C>() { return HI; }
B200JT_LIM(int8_t, INT8_MIN, INT8_MAX) B200JT_LIM(uint8_t, 0, UINT8_MAX) B200JT_LIM(int16_t, INT16_MIN, INT16_MAX)
B200JT_LIM(int32_t, INT32_MIN, INT32_MAX) B200JT_LIM(int64_t, INT64_MIN, INT64_MAX)
B200JT_LIM(float, -FLT_MAX, FLT_MAX) B200JT_LIM(double, -DBL_MAX, DBL_MAX)
#undef B200JT_LIM

// init_<op>. `is_bool`: the tensor dtype is bool (stored in uint8).
template <typename T>
__host__ __device__ inline T init_value(int op, bool is_bool = false) {
    using C = typename Compute<T>::type;
    switch (op) {
        case OP_MUL: case OP_LAND: return from_compute<T>((C)1);
        case OP_BAND: return is_bool ? from_compute<T>((C)1) : from_compute<T>((C)(-1));
        case OP_MAX: {
            if (is_bool) return from_compute<T>((C)0);
            // half types: lowest finite value of the storage type
            if (TypeInfo<T>::code == B200JT_FLOAT16) return from_compute<T>((C)(-65504.0f));
            if (TypeInfo<T>::code == B200JT_BFLOAT16) return from_compute<T>((C)(-3.3895313892515355e38f));
            return from_compute<T>(lowest_of<C>());
        }
        case OP_MIN: {
            if (is_bool) return from_compute<T>((C)1);
            if (TypeInfo<T>::code == B200JT_FLOAT16) return from_compute<T>((C)(65504.0f));
            if (TypeInfo<T>::code == B200JT_BFLOAT16) return from_compute<T>((C)(3.3895313892515355e38f));
            return from_compute<T>(highest_of<C>());
        }
        default: return from_compute<T>((C)0);     // add, mean, void, bitwise_or/xor, logical_or/xor
    }
}

template <typename C>
__host__ __device__ inline C apply_op_c(int op, C a, C b) {
    switch (op) {
        case OP_ADD: return a + b;
        case OP_MUL: return a * b;
        case OP_MAX: return a > b ? a : b;       // std::max(a, b)
        case OP_MIN: return b < a ? b : a;       // std::min(a, b)
        case OP_LAND: return (C)((a != (C)0) && (b != (C)0));
        case OP_LOR: return (C)((a != (C)0) || (b != (C)0));
        case OP_LXOR: return (C)((a != (C)0) != (b != (C)0));
        case OP_VOID: return b;
        default: return a;
    }
}
template <typename C>
__host__ __device__ inline C apply_bitop_c(int op, C a, C b) {
    switch (op) {
        case OP_BAND: return a & b;
        case OP_BOR: return a | b;
        case OP_BXOR: return a ^ b;
        default: return a;
    }
}
template <typename T>
__host__ __device__ inline T apply_op(int op, T a, T b) {
    using C = typename Compute<T>::type;
    if constexpr (!TypeInfo<T>::is_float) {
        if (op == OP_BAND || op == OP_BOR || op == OP_BXOR) return apply_bitop_c<T>(op, a, b);
    }
    return from_compute<T>(apply_op_c<C>(op, to_compute<T>(a), to_compute<T>(b)));
}

#ifdef __CUDACC__
// ---- CAS fallbacks -------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void atomic_cas_apply(T* addr, T v, int op) {
    if constexpr (sizeof(T) == 8) {
        unsigned long long* p = (unsigned long long*)addr;
        unsigned long long old = *p, assumed;
        do {
            assumed = old;
            T cur; memcpy(&cur, &assumed, 8);
            T nv = apply_op<T>(op, cur, v);
            unsigned long long nb; memcpy(&nb, &nv, 8);
            if (nb == assumed) return;
            old = atomicCAS(p, assumed, nb);
        } while (old != assumed);
    } else if constexpr (sizeof(T) == 4) {
        unsigned* p = (unsigned*)addr;
        unsigned old = *p, assumed;
        do {
            assumed = old;
            T cur; memcpy(&cur, &assumed, 4);
            T nv = apply_op<T>(op, cur, v);
            unsigned nb; memcpy(&nb, &nv, 4);
            if (nb == assumed) return;
            old = atomicCAS(p, assumed, nb);
        } while (old != assumed);
    } else {
        // 1- and 2-byte elements: CAS on the aligned 32-bit word that contains them
        uintptr_t a = (uintptr_t)addr;
        unsigned* p = (unsigned*)(a & ~(uintptr_t)3);
        const unsigned shift = (unsigned)(a & 3) * 8;
        const unsigned mask = (sizeof(T) == 1 ? 0xffu : 0xffffu) << shift;
        unsigned old = *p, assumed;
        do {
            assumed = old;
            unsigned field = (assumed & mask) >> shift;
            T cur; memcpy(&cur, &field, sizeof(T));
            T nv = apply_op<T>(op, cur, v);
            unsigned nf = 0; memcpy(&nf, &nv, sizeof(T));
            unsigned nb = (assumed & ~mask) | (nf << shift);
            if (nb == assumed) return;
            old = atomicCAS(p, assumed, nb);
        } while (old != assumed);
    }
}

// x[addr] = op(x[addr], v), atomically; native red/atom instructions where sm_100 has them.
template <typename T>
__device__ __forceinline__ void atomic_apply(T* addr, T v, int op) {
    if constexpr (std::is_same<T, int32_t>::value) {
        switch (op) {
            case OP_ADD: atomicAdd(addr, v); return;
            case OP_MAX: atomicMax(addr, v); return;
            case OP_MIN: atomicMin(addr, v); return;
            case OP_BAND: atomicAnd(addr, v); return;
            case OP_BOR: atomicOr(addr, v); return;
            case OP_BXOR: atomicXor(addr, v); return;
        }
    } else if constexpr (std::is_same<T, int64_t>::value) {
        switch (op) {
            case OP_ADD: atomicAdd((unsigned long long*)addr, (unsigned long long)v); return;
            case OP_MAX: atomicMax((long long*)addr, (long long)v); return;
            case OP_MIN: atomicMin((long long*)addr, (long long)v); return;
            case OP_BAND: atomicAnd((unsigned long long*)addr, (unsigned long long)v); return;
            case OP_BOR: atomicOr((unsigned long long*)addr, (unsigned long long)v); return;
            case OP_BXOR: atomicXor((unsigned long long*)addr, (unsigned long long)v); return;
        }
    } else if constexpr (std::is_same<T, float>::value) {
        switch (op) {
            case OP_ADD: atomicAdd(addr, v); return;
            // IEEE order == signed-int order for v >= 0 and reversed unsigned order for v < 0
            case OP_MAX:
                if (v != v) break;
                if (!signbit(v)) atomicMax((int*)addr, __float_as_int(v)); else atomicMin((unsigned*)addr, __float_as_uint(v));
                return;
            case OP_MIN:
                if (v != v) break;
                if (!signbit(v)) atomicMin((int*)addr, __float_as_int(v)); else atomicMax((unsigned*)addr, __float_as_uint(v));
                return;
        }
    } else if constexpr (std::is_same<T, double>::value) {
        switch (op) {
            case OP_ADD: atomicAdd(addr, v); return;
            case OP_MAX:
                if (v != v) break;
                if (!signbit(v)) atomicMax((long long*)addr, __double_as_longlong(v));
                else atomicMin((unsigned long long*)addr, (unsigned long long)__double_as_longlong(v));
                return;
            case OP_MIN:
                if (v != v) break;
                if (!signbit(v)) atomicMin((long long*)addr, __double_as_longlong(v));
                else atomicMax((unsigned long long*)addr, (unsigned long long)__double_as_longlong(v));
                return;
        }
    } else if constexpr (std::is_same<T, __nv_bfloat16>::value || std::is_same<T, __half>::value) {
        if (op == OP_ADD) { atomicAdd(addr, v); return; }
    }
    if (op == OP_VOID) { *addr = v; return; }
    atomic_cas_apply<T>(addr, v, op);
}
#endif

}  // namespace b200jt
