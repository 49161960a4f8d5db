// Fused element-wise chains around a row reduce: the general form of what the reference's FusedOp produces when it
// stitches unary / binary / ternary ops, broadcasts and reduces into one loop nest
// (python/jittor/src/fused_op.cc:41-118, python/jittor/src/op_compiler.cc:839-1045; cases
// python/jittor/test/test_fused_op.py:144-176). There the fused source is generated and compiled per graph; here the
// graph arrives as a small postfix program that ONE ahead-of-time kernel interprets, so any chain costs one launch and
// its intermediates never reach memory.
//
// A program is a list of statements over the "full" index space [rows, cols] (cols = the trailing axes a reduce folds,
// or any split of the tensor if there is no reduce):
//   ROW_REDUCE j, op   rowval[j] = fold over the row of <chain>           one sweep over the row
//   ROW_MAP j          rowval[j] = <chain over row values / per-row inputs / constants>
//   STORE              out[row, col] = <chain>                            one sweep, the output write
//   STORE_ROW j        out[row] = rowval[j]
// A chain is code for an accumulator machine: LOAD o (acc = o), UNARY u (acc = u(acc)), BINARY b, o (acc = acc b o, or
// o b acc with the swap bit), SELECT o1, o2 (acc = acc ? o1 : o2), TSTORE t (tmp[t] = acc), where an operand o is an
// input, a constant, a row value or one of six temporaries. The accumulator and the temporaries are fixed registers,
// so an instruction is dispatched on its op code only. All arithmetic is the float32 compute class of the element-wise
// kernels (elementwise.cu), and every op's result is rounded to the dtype the reference's inference gives that node
// (float32 / bfloat16 / float16 / bool), so a fused chain returns the same bits as the same ops run one by one.
//
// Kernel: a group of G threads (a warp, or a CTA of 256) owns a row at a time; every statement that sweeps the row
// re-reads its inputs, which after the first sweep come from L1/L2 (a row is a few KB), so DRAM sees one read of each
// input and one write of the output. A thread evaluates 8 consecutive elements per interpreted instruction (one 16- or
// 32-byte access per operand), which amortises the decode.
#include "atomic_ops.cuh"

#include "fused_chain.cuh"

namespace b200jt {
namespace chain {

__device__ __forceinline__ float round_to(float v, int dt) {
    switch (dt) {
        case B200JT_BFLOAT16: return __bfloat162float(__float2bfloat16(v));
        case B200JT_FLOAT16: return __half2float(__float2half(v));
        case B200JT_BOOL: return v != 0.f ? 1.f : 0.f;
        default: return v;
    }
}

__device__ __forceinline__ float binary_f(int op, float a, float b) {
    switch (op) {
        case OP_ADD: return a + b;
        case OP_SUB: return a - b;
        case OP_MUL: return a * b;
        case OP_DIV: case OP_FLOORDIV: return a / b;
        case OP_MOD: return a - floorf(a / b) * b;
        case OP_POW: return powf(a, b);
        case OP_MAX: return a > b ? a : b;
        case OP_MIN: return b < a ? b : a;
        case OP_LT: return (float)(a < b);
        case OP_LE: return (float)(a <= b);
        case OP_GT: return (float)(a > b);
        case OP_GE: return (float)(a >= b);
        case OP_EQ: return (float)(a == b);
        case OP_NE: return (float)(a != b);
        case OP_LAND: return (float)((a != 0) && (b != 0));
        case OP_LOR: return (float)((a != 0) || (b != 0));
        case OP_LXOR: return (float)((a != 0) != (b != 0));
    }
    return a;
}

__device__ __forceinline__ float unary_f(int op, float a) {
    switch (op) {
        case U_NEG: return -a;
        case U_ABS: return fabsf(a);
        case U_LNOT: return (float)(a == 0);
        case U_LOG: return logf(a);
        case U_EXP: return expf(a);
        case U_SQRT: return sqrtf(a);
        case U_ROUND: return roundf(a);
        case U_FLOOR: return floorf(a);
        case U_CEIL: return ceilf(a);
        case U_SIN: return sinf(a);
        case U_ASIN: return asinf(a);
        case U_SINH: return sinhf(a);
        case U_ASINH: return asinhf(a);
        case U_TAN: return tanf(a);
        case U_ATAN: return atanf(a);
        case U_TANH: return tanhf(a);
        case U_ATANH: return atanhf(a);
        case U_COS: return cosf(a);
        case U_ACOS: return acosf(a);
        case U_COSH: return coshf(a);
        case U_ACOSH: return acoshf(a);
        case U_SIGMOID: { const float t = -a < 30.f ? -a : 30.f; return 1.f / (1.f + expf(t)); }
        case U_ERF: return erff(a);
        case U_ERFINV: return erfinvf(a);
    }
    return a;           // U_CAST: the rounding to the result dtype is the cast
}

// VEC consecutive elements of input k starting at (row, col); `n` of them are inside the row.
__device__ __forceinline__ int64_t row_offset(const Input& I, int64_t row) {
    int64_t off = 0;
    for (int d = I.nd - 1; d >= 0; d--) { off += (row % I.shape[d]) * I.stride[d]; row /= I.shape[d]; }
    return off;
}

__device__ __forceinline__ void load_input(const Input& I, int64_t row, int64_t col, int64_t cols, int n, float* o) {
    switch (I.mode) {
        case IN_SCALAR: {
            const float v = load_as<float>(I.ptr, I.dtype, 0);
#pragma unroll
            for (int e = 0; e < VEC; e++) o[e] = v;
            return;
        }
        case IN_ROW: {
            const float v = load_as<float>(I.ptr, I.dtype, row_offset(I, row));
#pragma unroll
            for (int e = 0; e < VEC; e++) o[e] = v;
            return;
        }
        case IN_FULL: case IN_COL: {
            const int64_t off = (I.mode == IN_FULL ? row * cols : 0) + col;
            if (I.vec_ok && n == VEC) {
                if (I.dtype == B200JT_FLOAT32) {
                    const float4 a = __ldg(reinterpret_cast<const float4*>((const float*)I.ptr + off));
                    const float4 b = __ldg(reinterpret_cast<const float4*>((const float*)I.ptr + off) + 1);
                    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
                    return;
                }
                if (I.dtype == B200JT_BFLOAT16) {
                    const uint4 v = __ldg(reinterpret_cast<const uint4*>((const __nv_bfloat16*)I.ptr + off));
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
                    for (int i = 0; i < 4; i++) { const float2 f = __bfloat1622float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
                    return;
                }
            }
#pragma unroll
            for (int e = 0; e < VEC; e++) o[e] = e < n ? load_as<float>(I.ptr, I.dtype, off + e) : 0.f;
            return;
        }
        default: {
            // general broadcast: decompose the flat index of the first element, then step like an odometer
            int64_t idx[kMaxDims];
            int64_t r = row * cols + col, off = 0;
            for (int d = I.nd - 1; d >= 0; d--) { idx[d] = r % I.shape[d]; r /= I.shape[d]; off += idx[d] * I.stride[d]; }
            // fully unrolled: a loop that indexes o[] with a run-time counter would put the caller's register array
            // (and with it every operand of the chain) into local memory
#pragma unroll
            for (int e = 0; e < VEC; e++) {
                o[e] = e < n ? load_as<float>(I.ptr, I.dtype, off) : 0.f;
                for (int d = I.nd - 1; d >= 0; d--) {
                    off += I.stride[d];
                    if (++idx[d] < I.shape[d]) break;
                    off -= I.stride[d] * I.shape[d]; idx[d] = 0;
                }
            }
        }
    }
}

__device__ __forceinline__ void store_vec(void* out, int out_dtype, int out_vec_ok, int64_t off, int n, const float* v) {
    if (out_vec_ok && n == VEC) {
        if (out_dtype == B200JT_FLOAT32) {
            float4* p = reinterpret_cast<float4*>((float*)out + off);
            __stcs(p, make_float4(v[0], v[1], v[2], v[3]));
            __stcs(p + 1, make_float4(v[4], v[5], v[6], v[7]));
            return;
        }
        if (out_dtype == B200JT_BFLOAT16) {
            uint4 u; __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
            for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            __stcs(reinterpret_cast<uint4*>((__nv_bfloat16*)out + off), u);
            return;
        }
    }
#pragma unroll
    for (int e = 0; e < VEC; e++)
        if (e < n) store_as<float>(out, out_dtype, off + e, v[e]);
}
__device__ __forceinline__ void store_output(const Program& P, int64_t off, int n, const float* v) {
    store_vec(P.out, P.out_dtype, P.out_vec_ok, off, n, v);
}

// ---- the interpreter -------------------------------------------------------------------------------------------
__device__ __noinline__ void rare_unary(int op, float* v) {
#pragma unroll 1
    for (int e = 0; e < VEC; e++) v[e] = unary_f(op, v[e]);
}
__device__ __noinline__ void rare_binary(int op, float* a, const float* b) {
#pragma unroll 1
    for (int e = 0; e < VEC; e++) a[e] = binary_f(op, a[e], b[e]);
}

__device__ __forceinline__ void apply_unary(int sub, float (&acc)[VEC]) {
    switch (sub) {
        case U_CAST: break;
#define B200JT_U(CODE, EXPR) case CODE: _Pragma("unroll") for (int e = 0; e < VEC; e++) { const float v = acc[e]; acc[e] = (EXPR); } break
        B200JT_U(U_NEG, -v);
        B200JT_U(U_ABS, fabsf(v));
        B200JT_U(U_LNOT, (float)(v == 0));
        B200JT_U(U_LOG, logf(v));
        B200JT_U(U_EXP, expf(v));
        B200JT_U(U_SQRT, sqrtf(v));
        B200JT_U(U_TANH, tanhf(v));
        B200JT_U(U_SIGMOID, 1.f / (1.f + expf(-v < 30.f ? -v : 30.f)));
#undef B200JT_U
        default: {
            // through a copy: handing `acc` itself to a function that is not inlined would pin the accumulator in local
            // memory for the whole kernel
            float buf[VEC];
#pragma unroll
            for (int e = 0; e < VEC; e++) buf[e] = acc[e];
            rare_unary(sub, buf);
#pragma unroll
            for (int e = 0; e < VEC; e++) acc[e] = buf[e];
        }
    }
}

// acc = acc (sub) o, or o (sub) acc with swap
__device__ __forceinline__ void apply_binary(int sub, int swap, float (&acc)[VEC], float (&o)[VEC]) {
    if (swap) {
#pragma unroll
        for (int e = 0; e < VEC; e++) { const float t = acc[e]; acc[e] = o[e]; o[e] = t; }
    }
    switch (sub) {
#define B200JT_B(CODE, EXPR) case CODE: _Pragma("unroll") for (int e = 0; e < VEC; e++) { const float p = acc[e], q = o[e]; acc[e] = (EXPR); } break
        B200JT_B(OP_ADD, p + q);
        B200JT_B(OP_SUB, p - q);
        B200JT_B(OP_MUL, p * q);
        B200JT_B(OP_DIV, p / q);
        B200JT_B(OP_MAX, p > q ? p : q);
        B200JT_B(OP_MIN, q < p ? q : p);
        B200JT_B(OP_LT, (float)(p < q));
        B200JT_B(OP_LE, (float)(p <= q));
        B200JT_B(OP_GT, (float)(p > q));
        B200JT_B(OP_GE, (float)(p >= q));
        B200JT_B(OP_EQ, (float)(p == q));
        B200JT_B(OP_NE, (float)(p != q));
#undef B200JT_B
        default: {
            float ba[VEC], bo[VEC];
#pragma unroll
            for (int e = 0; e < VEC; e++) { ba[e] = acc[e]; bo[e] = o[e]; }
            rare_binary(sub, ba, bo);
#pragma unroll
            for (int e = 0; e < VEC; e++) acc[e] = ba[e];
        }
    }
}

constexpr int kPre = 4;
static_assert(kPre == 4, "the operand select below is written out for this size");         // input operands of a chain whose loads are issued before the chain is interpreted

// Operand of word w into o[]; advances pc over an inline constant.
__device__ __forceinline__ void fetch(const Program& P, int32_t w, int& pc, int64_t row, int64_t col, int n, const float* rowval,
                                      const float (&tmp)[kTmp][VEC], const float (&pre)[kPre][VEC], int n_pre, int& used, float (&o)[VEC]) {
    const int kind = w_kind(w), idx = w_index(w);
    if (kind == K_INPUT) {
        if (used < n_pre) {
#pragma unroll
            for (int e = 0; e < VEC; e++) o[e] = used == 0 ? pre[0][e] : used == 1 ? pre[1][e] : used == 2 ? pre[2][e] : pre[3][e];
            used++;
        } else load_input(P.in[idx], row, col, P.cols, n, o);
        return;
    }
    if (kind == K_TMP) {
#pragma unroll
        for (int e = 0; e < VEC; e++) {
            float r = tmp[0][e];                      // selects on the value: no address depends on idx
#pragma unroll
            for (int t = 1; t < kTmp; t++) r = idx == t ? tmp[t][e] : r;
            o[e] = r;
        }
        return;
    }
    const float c = kind == K_CONST ? __int_as_float(P.code[++pc]) : rowval[idx];
#pragma unroll
    for (int e = 0; e < VEC; e++) o[e] = c;
}

// Runs the chain that starts at code[pc] for VEC elements; returns the pc of the statement word that ends it and leaves
// the chain's value in `acc`.
__device__ __forceinline__ int eval_chain(const Program& P, int pc, int64_t row, int64_t col, int n, const float* rowval, float (&acc)[VEC]) {
    // initialised on purpose: a conditional store into an undefined value lets the compiler drop the condition, and
    // then every TSTORE would write all temporaries
    float tmp[kTmp][VEC] = {};
    // The loads of the chain's first input operands are issued together, before any of them is used: the interpreter
    // consumes operands one instruction at a time, and without this every input would cost its own trip to memory.
    float pre[kPre][VEC] = {};
    int n_pre = 0, used = 0;
    for (int q = pc; n_pre < kPre; q++) {
        const int32_t w = P.code[q];
        if (w_op(w) >= CH_ROW_REDUCE) break;
        const int kind = w_kind(w);
        if (kind == K_CONST) q++;
        else if (kind == K_INPUT) {
#pragma unroll
            float t[VEC];
            load_input(P.in[w_index(w)], row, col, P.cols, n, t);
#pragma unroll
            for (int k = 0; k < kPre; k++) {
                const bool hit = k == n_pre;
#pragma unroll
                for (int e = 0; e < VEC; e++) pre[k][e] = hit ? t[e] : pre[k][e];
            }
            n_pre++;
        }
    }
    for (;; pc++) {
        const int32_t w = P.code[pc];
        const int op = w_op(w);
        if (op >= CH_ROW_REDUCE) break;
        const int sub = w_sub(w), rdt = w_rdt(w);
        if (op == CH_TSTORE) {
            const int idx = w_index(w);
#pragma unroll
            for (int t = 0; t < kTmp; t++) {
                // a select on the value, not a store under a condition: stores under conditions on t are merged by the
                // compiler into one store at a computed address, and that puts the array in local memory
                const bool hit = t == idx;
#pragma unroll
                for (int e = 0; e < VEC; e++) tmp[t][e] = hit ? acc[e] : tmp[t][e];
            }
            continue;
        }
        if (op == CH_UNARY) {
            apply_unary(sub, acc);
        } else {
            float o[VEC];
            fetch(P, w, pc, row, col, n, rowval, tmp, pre, n_pre, used, o);
            if (op == CH_LOAD) {
#pragma unroll
                for (int e = 0; e < VEC; e++) acc[e] = o[e];
            } else if (op == CH_BINARY) {
                apply_binary(sub, w_swap(w), acc, o);
            } else {                    // CH_SELECT: acc ? o : o2, the second operand is described by the next word
                float o2[VEC];
                const int32_t w2 = P.code[++pc];
                fetch(P, w2, pc, row, col, n, rowval, tmp, pre, n_pre, used, o2);
#pragma unroll
                for (int e = 0; e < VEC; e++) acc[e] = acc[e] != 0.f ? o[e] : o2[e];
            }
        }
        if (rdt != B200JT_FLOAT32) {
#pragma unroll
            for (int e = 0; e < VEC; e++) acc[e] = round_to(acc[e], rdt);
        }
    }
    return pc;
}

__device__ __forceinline__ float fold(int rop, float a, float b) {
    switch (rop) {
        case OP_MAX: return a > b ? a : b;
        case OP_MIN: return b < a ? b : a;
        case OP_MUL: return a * b;
        default: return a + b;          // add, mean
    }
}
__device__ __forceinline__ float fold_init(int rop) {
    switch (rop) {
        case OP_MAX: return -FLT_MAX;
        case OP_MIN: return FLT_MAX;
        case OP_MUL: return 1.f;
        default: return 0.f;
    }
}

// Pure map (the program is one chain ending in STORE): work items are 8-element vectors of the full space.
__global__ void __launch_bounds__(256, 2)
chain_map_kernel(const __grid_constant__ Program P) {
    const int64_t vpr = (P.cols + VEC - 1) / VEC, items = P.rows * vpr;
    const bool small = items < (1LL << 31);
    for (int64_t it = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; it < items; it += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = small ? (int64_t)((uint32_t)it / (uint32_t)vpr) : it / vpr, col = (it - row * vpr) * VEC;
        const int n = (int)min((int64_t)VEC, P.cols - col);
        float v[VEC];
        eval_chain(P, 0, row, col, n, nullptr, v);
        store_output(P, row * P.cols + col, n, v);
    }
}

// G threads per row (32: a warp, shuffles only; 256: the whole CTA, one shared-memory hop).
template <int G>
__global__ void __launch_bounds__(256, 2)
chain_rows_kernel(const __grid_constant__ Program P) {
    __shared__ float xch[8];
    constexpr int GROUPS = 256 / G;
    const int g = threadIdx.x / G, t = threadIdx.x % G;
    const int64_t n_groups = (int64_t)gridDim.x * GROUPS;
    const float rcols = 1.f / (float)P.cols;
    // uniform trip count per CTA so that __syncthreads inside the loop is legal for G == 256
    for (int64_t row = (int64_t)blockIdx.x * GROUPS + g; row < P.rows; row += n_groups) {
        float rowval[kMaxRowVals];
        int pc = 0;
        while (pc < P.n_code) {
            // find the statement that ends the chain starting at pc (statement words are >= CH_ROW_REDUCE)
            int end = pc;
            while (w_op(P.code[end]) < CH_ROW_REDUCE) end += (w_kind(P.code[end]) == K_CONST) ? 2 : 1;
            const int32_t w = P.code[end];
            const int sop = w_op(w), a = w_index(w), rdt = w_rdt(w);
            if (sop == CH_STORE_ROW) {
                if (t == 0) store_as<float>(P.out, P.out_dtype, row, rowval[a]);
            } else {
                // one loop for the three kinds of statement, so that the interpreter is instantiated once: a per-row map
                // is a single evaluation at column 0 by every thread of the group
                const bool row_map = sop == CH_ROW_MAP;
                const int rop = w_sub(w);
                float acc = fold_init(rop);
                const int64_t col_end = row_map ? 1 : P.cols;
                for (int64_t col = row_map ? 0 : (int64_t)t * VEC; col < col_end; col += (int64_t)G * VEC) {
                    const int n = (int)min((int64_t)VEC, col_end - col);
                    float v[VEC];
                    eval_chain(P, pc, row, col, n, rowval, v);
                    if (sop == CH_STORE) store_output(P, row * P.cols + col, n, v);
                    else if (row_map) acc = v[0];
                    else if (rop == OP_MEAN) {
#pragma unroll
                        for (int e = 0; e < VEC; e++) if (e < n) acc += v[e] * rcols;
                    } else {
#pragma unroll
                        for (int e = 0; e < VEC; e++) if (e < n) acc = fold(rop, acc, v[e]);
                    }
                }
                if (row_map) rowval[a] = acc;
                else if (sop == CH_ROW_REDUCE) {
#pragma unroll
                    for (int d = 16; d > 0; d >>= 1) acc = fold(rop, acc, __shfl_xor_sync(0xffffffffu, acc, d));
                    if (G == 256) {
                        __syncthreads();                       // xch free again
                        if ((threadIdx.x & 31) == 0) xch[threadIdx.x >> 5] = acc;
                        __syncthreads();
                        acc = xch[0];
#pragma unroll
                        for (int k = 1; k < 8; k++) acc = fold(rop, acc, xch[k]);
                    }
                    rowval[a] = round_to(acc, rdt);
                }
            }
            pc = end + 1;
        }
    }
}

}  // namespace chain
}  // namespace b200jt

using namespace b200jt;

/* One launch for a fused chain. inputs: n_inputs tensors, each given with the rank of `full_shape` (size 1 on the axes
 * it is broadcast over); the last `row_axes` axes of full_shape form a row (the axes the program's reduces fold; 0 if
 * there is none); code: the postfix program described at the top of this file; out: the element-wise result
 * (full_shape) or, for a program ending in STORE_ROW, one value per row. */
extern "C" int b200jt_fused_chain(const b200jt_tensor* inputs, int n_inputs, const int64_t* full_shape, int ndim, int row_axes,
                                  const int32_t* code, int n_code, const b200jt_tensor* out, void* stream) {
    using namespace chain;
    B200JT_CHECK_ARG(n_inputs >= 0 && n_inputs <= kMaxInputs, "at most 8 inputs");
    B200JT_CHECK_ARG(code && n_code > 0 && n_code <= kMaxCode, "program too long");
    B200JT_CHECK_ARG(ndim >= 1 && ndim <= kMaxDims && row_axes >= 0 && row_axes <= ndim, "bad shape");
    B200JT_CHECK_ARG(valid_tensor(out), "invalid output descriptor");
    Program Q; memset(&Q, 0, sizeof(Q));
    bool has_row_stmt = false, store_row = false;
    // validate the program: operand indices, the accumulator holds a value where one is used, statement structure
    {
        bool have_acc = false;
        auto operand_ok = [&](int32_t w, int& pc) -> bool {
            const int kind = w_kind(w), idx = w_index(w);
            if (kind == K_INPUT) return idx < n_inputs;
            if (kind == K_CONST) return ++pc < n_code;
            if (kind == K_ROWVAL) return idx < kMaxRowVals;
            if (kind == K_TMP) return idx < kTmp;
            return false;
        };
        for (int pc = 0; pc < n_code; pc++) {
            const int32_t w = code[pc];
            const int op = w_op(w), idx = w_index(w);
            switch (op) {
                case CH_LOAD: B200JT_CHECK_ARG(operand_ok(w, pc), "bad operand"); have_acc = true; break;
                case CH_UNARY: B200JT_CHECK_ARG(have_acc && w_sub(w) < U_INVALID, "bad unary"); break;
                case CH_BINARY: B200JT_CHECK_ARG(have_acc && operand_ok(w, pc), "bad binary"); break;
                case CH_SELECT: {
                    B200JT_CHECK_ARG(have_acc && operand_ok(w, pc) && pc + 1 < n_code, "bad select");
                    const int32_t w2 = code[++pc];
                    B200JT_CHECK_ARG(w_op(w2) == CH_OPERAND && operand_ok(w2, pc), "select needs a second operand word");
                    break;
                }
                case CH_TSTORE: B200JT_CHECK_ARG(have_acc && idx < kTmp, "bad temporary"); break;
                case CH_ROW_REDUCE: B200JT_CHECK_ARG(have_acc && idx < kMaxRowVals, "bad row reduce"); have_acc = false; has_row_stmt = true; break;
                case CH_ROW_MAP: B200JT_CHECK_ARG(have_acc && idx < kMaxRowVals, "bad row map"); have_acc = false; has_row_stmt = true; break;
                case CH_STORE: B200JT_CHECK_ARG(have_acc && pc == n_code - 1, "STORE must end the program"); have_acc = false; break;
                case CH_STORE_ROW: B200JT_CHECK_ARG(!have_acc && idx < kMaxRowVals && pc == n_code - 1, "STORE_ROW must end the program"); store_row = true; break;
                default: return fail(-1, "b200jt_fused_chain: unknown instruction");
            }
        }
        const int last = w_op(code[n_code - 1]);
        B200JT_CHECK_ARG(last == CH_STORE || last == CH_STORE_ROW, "the program must end in STORE or STORE_ROW");
    }
    for (int d = 0; d < ndim; d++) B200JT_CHECK_ARG(full_shape[d] >= 0, "negative extent");
    for (int k = 0; k < n_inputs; k++) {
        const b200jt_tensor* t = &inputs[k];
        B200JT_CHECK_ARG(valid_tensor(t) && t->ndim == ndim, "every input must be given with the rank of full_shape");
        for (int d = 0; d < ndim; d++)
            B200JT_CHECK_ARG(t->shape[d] == full_shape[d] || t->shape[d] == 1, "Shape not match " + shape_str(t));
    }
    const bool pure_map = !has_row_stmt && !store_row;
    // How an input relates to a split of the axes into `ra` trailing row axes (cols) and the rest (rows).
    auto classify = [&](const b200jt_tensor* t, int ra) {
        if (numel(t) == 1) return (int)IN_SCALAR;
        bool dep_rows = false, dep_cols = false, full_rows = true, full_cols = true;
        for (int d = 0; d < ndim; d++) {
            if (full_shape[d] == 1) continue;
            const bool bc = t->shape[d] == 1;
            if (d < ndim - ra) { if (bc) full_rows = false; else dep_rows = true; }
            else { if (bc) full_cols = false; else dep_cols = true; }
        }
        if (full_rows && full_cols) return (int)IN_FULL;
        if (!dep_rows && full_cols) return (int)IN_COL;
        if (!dep_cols) return (int)IN_ROW;
        return (int)IN_GENERAL;
    };
    if (pure_map) {
        // any split is legal: take the one with the longest rows (up to 64 Ki elements) that leaves no input in the
        // general form, preferring rows that are whole vectors
        int best = -1; int best_score = -1;
        for (int ra = 0; ra <= ndim; ra++) {
            int64_t c = 1;
            for (int d = ndim - ra; d < ndim; d++) c *= full_shape[d];
            if (c > (1 << 16) && ra > 1) break;
            int general = 0;
            for (int k = 0; k < n_inputs; k++) general += classify(&inputs[k], ra) == IN_GENERAL;
            const int score = (general == 0 ? 4 : 0) + (c % VEC == 0 ? 2 : 0) + (c >= 64 ? 1 : 0);
            if (score >= best_score) { best_score = score; best = ra; }
        }
        row_axes = best < 0 ? 0 : best;
    }
    int64_t rows = 1, cols = 1;
    for (int d = 0; d < ndim; d++) (d < ndim - row_axes ? rows : cols) *= full_shape[d];
    B200JT_CHECK_ARG(numel(out) == (store_row ? rows : rows * cols), "out has the wrong size " + shape_str(out));
    if (numel(out) == 0) return 0;
    bool all_flat = true;
    for (int k = 0; k < n_inputs; k++) { const int m = classify(&inputs[k], row_axes); all_flat &= (m == IN_FULL || m == IN_SCALAR); }
    if (pure_map && all_flat) {
        // nothing depends on the position inside the tensor: one flat index space cut into rows of whole vectors
        const int64_t n = rows * cols;
        cols = n % 2048 == 0 ? 2048 : n;
        rows = n / cols;
    }
    Q.rows = rows; Q.cols = cols;
    Q.n_inputs = n_inputs; Q.n_code = n_code;
    memcpy(Q.code, code, sizeof(int32_t) * n_code);
    Q.out = out->ptr; Q.out_dtype = out->dtype;
    Q.out_vec_ok = ((uintptr_t)out->ptr % 32 == 0) && cols % VEC == 0;
    for (int k = 0; k < n_inputs; k++) {
        const b200jt_tensor* t = &inputs[k];
        Input& I = Q.in[k];
        I.ptr = t->ptr; I.dtype = t->dtype;
        I.mode = classify(t, row_axes);
        const int es = dtype_size(t->dtype);
        const bool aligned = ((uintptr_t)t->ptr % 32 == 0) || (es == 2 && (uintptr_t)t->ptr % 16 == 0);
        I.vec_ok = (I.mode == IN_FULL || I.mode == IN_COL) && aligned && cols % VEC == 0;
        if (I.mode == IN_ROW || I.mode == IN_GENERAL) {
            // merged axes (of the row axes only for ROW): neighbours the input walks contiguously or ignores together
            const int lim = I.mode == IN_ROW ? ndim - row_axes : ndim;
            int64_t tstride[kMaxDims]; int64_t ts = 1;
            for (int d = ndim - 1; d >= 0; d--) { tstride[d] = (t->shape[d] == 1 && full_shape[d] != 1) ? 0 : ts; ts *= t->shape[d]; }
            int nd = 0;
            for (int d = 0; d < lim; d++) {
                if (full_shape[d] == 1) continue;
                if (nd && ((I.stride[nd - 1] == 0 && tstride[d] == 0) ||
                           (tstride[d] != 0 && I.stride[nd - 1] == tstride[d] * full_shape[d]))) {
                    I.shape[nd - 1] *= full_shape[d]; I.stride[nd - 1] = tstride[d];
                } else { I.shape[nd] = full_shape[d]; I.stride[nd] = tstride[d]; nd++; }
            }
            if (nd == 0) { I.shape[0] = 1; I.stride[0] = 0; nd = 1; }
            I.nd = nd;
        }
    }
    cudaStream_t st = (cudaStream_t)stream;
    // a kernel compiled for exactly this program, when the run-time compiler is there; the interpreter otherwise
    {
        const int r = chain::jit_launch(Q, pure_map, pure_map && all_flat, st);
        if (r != chain::kJitUnavailable) return r;
    }
    if (pure_map) {
        const int64_t items = Q.rows * ((Q.cols + VEC - 1) / VEC);
        chain::chain_map_kernel<<<grid_for(items, 256), 256, 0, st>>>(Q);
    } else if (Q.cols <= 1024) {          // a warp per row for short rows, a CTA per row otherwise
        const unsigned grid = grid_for((Q.rows + 7) / 8 * 256, 256);
        chain::chain_rows_kernel<32><<<grid, 256, 0, st>>>(Q);
    } else {
        const unsigned grid = grid_for(Q.rows * 256, 256);
        chain::chain_rows_kernel<256><<<grid, 256, 0, st>>>(Q);
    }
    B200JT_LAUNCH_CHECK();
    return 0;
}
