// Program format and kernel argument block of the fused element-wise chains, shared by the interpreter kernels
// (fused_chain.cu) and the run-time specialiser (chain_jit.cu).
#pragma once
#include "common.cuh"

namespace b200jt {
namespace chain {

constexpr int kMaxInputs = 8;
constexpr int kMaxCode = 160;
constexpr int kMaxRowVals = 8;
constexpr int kTmp = 6;
constexpr int VEC = 8;

// word = op | sub << 4 | operand kind << 10 | operand index << 13 | swap << 21 | result dtype << 24
enum ChainOp : int {
    CH_OPERAND = 0,     // second operand of the SELECT before it
    CH_LOAD, CH_UNARY, CH_BINARY, CH_SELECT, CH_TSTORE,
    CH_ROW_REDUCE = 8,  // sub = reduce op, index = slot : ends a chain, one sweep
    CH_ROW_MAP,         // index = slot              : ends a chain evaluated once per row
    CH_STORE,           // ends a chain, one sweep, writes the output
    CH_STORE_ROW        // index = slot              : out[row] = rowval[slot]
};
enum OperandKind : int { K_NONE = 0, K_INPUT, K_CONST /* the float32 in the next word */, K_ROWVAL, K_TMP };

__host__ __device__ __forceinline__ int w_op(int32_t w) { return w & 15; }
__host__ __device__ __forceinline__ int w_sub(int32_t w) { return (w >> 4) & 63; }
__host__ __device__ __forceinline__ int w_kind(int32_t w) { return (w >> 10) & 7; }
__host__ __device__ __forceinline__ int w_index(int32_t w) { return (w >> 13) & 255; }
__host__ __device__ __forceinline__ int w_swap(int32_t w) { return (w >> 21) & 1; }
__host__ __device__ __forceinline__ int w_rdt(int32_t w) { return (w >> 24) & 255; }

// unary codes of elementwise.cu (kept in the same order)
enum UnaryCode : int {
    U_CAST = 0, U_NEG, U_ABS, U_LNOT, U_BNOT, U_LOG, U_EXP, U_SQRT, U_ROUND, U_FLOOR, U_CEIL,
    U_SIN, U_ASIN, U_SINH, U_ASINH, U_TAN, U_ATAN, U_TANH, U_ATANH, U_COS, U_ACOS, U_COSH, U_ACOSH,
    U_SIGMOID, U_ERF, U_ERFINV, U_INVALID
};

// How an input is addressed from (row, col):
enum InMode : int {
    IN_FULL = 0,        // same shape as the full space: offset row*cols + col
    IN_SCALAR,          // one element
    IN_COL,             // constant over the rows, complete along the row (bias): offset col
    IN_ROW,             // constant along the row: one offset per row, from the row index and the strides of the row axes
    IN_GENERAL          // broadcast over arbitrary axes: strides per merged axis of the full space
};

struct Input {
    const void* ptr;
    int32_t dtype, mode;
    int32_t vec_ok;                     // 16-byte aligned base and row pitch: vector loads allowed (FULL / COL)
    int32_t nd;                         // GENERAL: merged axes of the full space; ROW: merged row axes; innermost last
    int64_t shape[kMaxDims], stride[kMaxDims];
};

struct Program {
    int32_t n_inputs, n_code;
    Input in[kMaxInputs];
    int32_t code[kMaxCode];
    void* out;
    int32_t out_dtype, out_vec_ok;
    int64_t rows, cols;
};

// Launches a kernel specialised for Q's program and input classes, compiling it on first use. Returns 0 when the
// kernel was launched, kJitUnavailable when there is no specialised kernel (the caller runs the interpreter), any other
// value is an error code with the message set.
constexpr int kJitUnavailable = -1000;
int jit_launch(const Program& Q, bool pure_map, bool flat, cudaStream_t st);
// While a thread's t_dry_run is set, jit_launch only generates and compiles: the source, the compiler's log and whether
// it compiled are left there and nothing is launched.
struct DryRun { std::string source, log; bool compiled = false; };
extern thread_local DryRun* t_dry_run;
// The CUDA source jit_launch compiles for Q.
std::string jit_source(const Program& Q, bool pure_map, bool flat);

}  // namespace chain
}  // namespace b200jt
