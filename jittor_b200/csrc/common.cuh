// Shared declarations of the sm_100a kernel library: error plumbing, dtype helpers, launch sizing.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <string>

#include "../../include/b200jt.h"

namespace b200jt {

constexpr int kNumSMs = 148;            // B200: 2 dies x 74 SMs; grids are sized in multiples of this
constexpr int kMaxDims = B200JT_MAX_DIMS;

// ---- error plumbing: no exception crosses the C ABI ---------------------------------------------
void set_error(const std::string& msg);
int  fail(int code, const std::string& msg);

#define B200JT_CHECK_ARG(cond, msg)                                             \
    do { if (!(cond)) return ::b200jt::fail(-1, std::string(__func__) + ": " + (msg)); } while (0)

#define B200JT_CUDA(expr)                                                        \
    do { cudaError_t e_ = (expr); if (e_ != cudaSuccess)                         \
        return ::b200jt::fail((int)e_, std::string(__func__) + ": " #expr ": " + cudaGetErrorString(e_)); } while (0)

#define B200JT_LAUNCH_CHECK()  B200JT_CUDA(cudaGetLastError())

// ---- dtype helpers -----------------------------------------------------------------------------
__host__ __device__ inline int dtype_size(int dt) {
    switch (dt) {
        case B200JT_BOOL: case B200JT_INT8: case B200JT_UINT8: return 1;
        case B200JT_INT16: case B200JT_FLOAT16: case B200JT_BFLOAT16: return 2;
        case B200JT_INT32: case B200JT_FLOAT32: return 4;
        case B200JT_INT64: case B200JT_FLOAT64: return 8;
    }
    return 0;
}
__host__ __device__ inline bool dtype_is_float(int dt) {
    return dt == B200JT_FLOAT16 || dt == B200JT_BFLOAT16 || dt == B200JT_FLOAT32 || dt == B200JT_FLOAT64;
}
const char* dtype_name(int dt);
int dtype_from_name(const char* name);      // -1 if `name` is not a dtype

inline int64_t numel(const b200jt_tensor* t) {
    int64_t n = 1;
    for (int i = 0; i < t->ndim; i++) n *= t->shape[i];
    return n;
}
inline bool valid_tensor(const b200jt_tensor* t) {
    if (!t || t->ndim < 1 || t->ndim > kMaxDims || dtype_size(t->dtype) == 0) return false;
    for (int i = 0; i < t->ndim; i++) if (t->shape[i] < 0) return false;
    return numel(t) == 0 || t->ptr != nullptr;
}
std::string shape_str(const b200jt_tensor* t);

// Load element `i` of a buffer of runtime dtype as T (device side).
template <typename T>
__device__ __forceinline__ T load_as(const void* p, int dt, int64_t i) {
    switch (dt) {
        case B200JT_BOOL:     return (T)(((const uint8_t*)p)[i] != 0);
        case B200JT_INT8:     return (T)((const int8_t*)p)[i];
        case B200JT_UINT8:    return (T)((const uint8_t*)p)[i];
        case B200JT_INT16:    return (T)((const int16_t*)p)[i];
        case B200JT_INT32:    return (T)((const int32_t*)p)[i];
        case B200JT_INT64:    return (T)((const int64_t*)p)[i];
        case B200JT_FLOAT16:  return (T)__half2float(((const __half*)p)[i]);
        case B200JT_BFLOAT16: return (T)__bfloat162float(((const __nv_bfloat16*)p)[i]);
        case B200JT_FLOAT32:  return (T)((const float*)p)[i];
        case B200JT_FLOAT64:  return (T)((const double*)p)[i];
    }
    return T(0);
}
// Store v (of compute type T) into element i of a buffer of runtime dtype, with C conversion rules.
template <typename T>
__device__ __forceinline__ void store_as(void* p, int dt, int64_t i, T v) {
    switch (dt) {
        case B200JT_BOOL:     ((uint8_t*)p)[i] = (v != T(0)); break;
        case B200JT_INT8:     ((int8_t*)p)[i] = (int8_t)(int64_t)v; break;
        case B200JT_UINT8:    ((uint8_t*)p)[i] = (uint8_t)(int64_t)v; break;
        case B200JT_INT16:    ((int16_t*)p)[i] = (int16_t)(int64_t)v; break;
        case B200JT_INT32:    ((int32_t*)p)[i] = (int32_t)(int64_t)v; break;
        case B200JT_INT64:    ((int64_t*)p)[i] = (int64_t)v; break;
        case B200JT_FLOAT16:  ((__half*)p)[i] = __float2half((float)v); break;
        case B200JT_BFLOAT16: ((__nv_bfloat16*)p)[i] = __float2bfloat16((float)v); break;
        case B200JT_FLOAT32:  ((float*)p)[i] = (float)v; break;
        case B200JT_FLOAT64:  ((double*)p)[i] = (double)v; break;
    }
}

// ---- launch sizing -----------------------------------------------------------------------------
// Grid for a grid-stride loop over `work` threads: enough CTAs to cover it, capped at a whole number
// of waves over the 148 SMs.
// SMs the grids leave free for a collective that runs beside them on another stream (0 unless a host asked for it with
// b200jt_set_sm_reserve): the persistent kernels size themselves as if the GPU had kNumSMs - sm_reserve() SMs.
int sm_reserve();

inline unsigned grid_for(int64_t work, int block, int ctas_per_sm = 8) {
    int64_t need = (work + block - 1) / block;
    int64_t cap = (int64_t)(kNumSMs - sm_reserve()) * ctas_per_sm;
    if (need < 1) need = 1;
    return (unsigned)(need < cap ? need : cap);
}

// ---- reduce / binary op codes shared by several kernels -----------------------------------------
enum OpCode : int {
    OP_ADD = 0, OP_SUB, OP_MUL, OP_DIV, OP_FLOORDIV, OP_MOD, OP_POW, OP_MAX, OP_MIN,
    OP_LT, OP_LE, OP_GT, OP_GE, OP_EQ, OP_NE,
    OP_LAND, OP_LOR, OP_LXOR, OP_BAND, OP_BOR, OP_BXOR, OP_SHL, OP_SHR,
    OP_MEAN, OP_VOID, OP_INVALID
};
OpCode binary_op_from_name(const char* name);

}  // namespace b200jt
