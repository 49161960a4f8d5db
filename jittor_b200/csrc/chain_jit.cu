// Run-time specialiser of the fused element-wise chains: the program that the interpreter kernels of fused_chain.cu
// would decode per element is instead written out once as straight-line CUDA source, compiled for sm_100a with NVRTC
// and kept in a per-process cache, so the steady state is one launch of a kernel in which every op code, operand kind,
// dtype, broadcast class and vector width is a compile-time fact. The reference does the same at a larger scale (its
// FusedOp emits a loop nest per graph and compiles it, python/jittor/src/fused_op.cc:140-247,
// python/jittor/src/op_compiler.cc:839-1045); here only the body of a fixed kernel skeleton is generated.
//
// What is specialised on (the cache key): the program words, and per input its class (full / scalar / column / row /
// general broadcast), dtype, vector alignment and merged rank; the output dtype and alignment; map or rows kernel and the
// group width; whether the row length is a whole number of 8-element vectors. Shapes, strides and pointers stay kernel
// arguments, so a chain compiled for one size serves all sizes of the same classes.
//
// Arithmetic: float32 throughout, every op rounded to its node's dtype, +, - and * through __fadd_rn / __fsub_rn /
// __fmul_rn so that the compiler cannot contract a multiply of one op with the add of the next -- a fused chain returns
// the bits of the same ops run one by one, exactly like the interpreter.
//
// NVRTC (jit.cu) is opened with dlopen on first use; without it (or with B200JT_CHAIN_JIT=0) jit_launch reports "not available"
// and the caller runs the interpreter kernels. B200JT_CHAIN_JIT=2 turns a failed compilation into an error.
#include "fused_chain.cuh"
#include "jit.cuh"

namespace b200jt {
namespace chain {
namespace {

// ---- source generation ------------------------------------------------------------------------------------------
const char* kPrelude = R"SRC(
typedef long long i64;
typedef unsigned short u16;
typedef unsigned char u8;
#define FOR8 _Pragma("unroll") for (int e = 0; e < VEC; e++)
#define FLT_MAX 3.402823466e+38f
struct Input { const void* ptr; int dtype, mode, vec_ok, nd; i64 shape[MAXD], stride[MAXD]; };
struct Program { int n_inputs, n_code; Input in[MAXIN]; int code[MAXCODE]; void* out; int out_dtype, out_vec_ok; i64 rows, cols; };
static_assert(sizeof(Program) == PROGRAM_BYTES, "argument block differs from the host's");

__device__ __forceinline__ float bf2f(u16 b) { return __uint_as_float(((unsigned)b) << 16); }
__device__ __forceinline__ u16 f2bf(float f) { u16 r; asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f)); return r; }
__device__ __forceinline__ float h2f(u16 h) { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h)); return f; }
__device__ __forceinline__ u16 f2h(float f) { u16 r; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(r) : "f"(f)); return r; }

// dtype codes: 0 bool, 1 int8, 2 int16, 3 int32, 4 int64, 5 uint8, 6 float16, 7 bfloat16, 8 float32, 9 float64
template <int DT> __device__ __forceinline__ float rnd(float v) {
    if (DT == 7) return bf2f(f2bf(v));
    if (DT == 6) return h2f(f2h(v));
    if (DT == 0) return v != 0.f ? 1.f : 0.f;
    return v;
}
template <int DT> __device__ __forceinline__ float ld1(const void* p, i64 i) {
    if (DT == 0) return (float)(__ldg((const u8*)p + i) != 0);
    if (DT == 1) return (float)__ldg((const signed char*)p + i);
    if (DT == 5) return (float)__ldg((const u8*)p + i);
    if (DT == 2) return (float)__ldg((const short*)p + i);
    if (DT == 3) return (float)__ldg((const int*)p + i);
    if (DT == 4) return (float)__ldg((const i64*)p + i);
    if (DT == 6) return h2f(__ldg((const u16*)p + i));
    if (DT == 7) return bf2f(__ldg((const u16*)p + i));
    if (DT == 8) return __ldg((const float*)p + i);
    if (DT == 9) return (float)__ldg((const double*)p + i);
    return 0.f;
}
template <int DT> __device__ __forceinline__ void st1(void* p, i64 i, float v) {
    if (DT == 0) ((u8*)p)[i] = (v != 0.f);
    if (DT == 1) ((signed char*)p)[i] = (signed char)(i64)v;
    if (DT == 5) ((u8*)p)[i] = (u8)(i64)v;
    if (DT == 2) ((short*)p)[i] = (short)(i64)v;
    if (DT == 3) ((int*)p)[i] = (int)(i64)v;
    if (DT == 4) ((i64*)p)[i] = (i64)v;
    if (DT == 6) ((u16*)p)[i] = f2h(v);
    if (DT == 7) ((u16*)p)[i] = f2bf(v);
    if (DT == 8) ((float*)p)[i] = v;
    if (DT == 9) ((double*)p)[i] = (double)v;
}

template <int ND> __device__ __forceinline__ i64 row_offset(const Input& I, i64 row) {
    i64 off = 0;
#pragma unroll
    for (int d = ND - 1; d >= 0; d--) { off += (row % I.shape[d]) * I.stride[d]; row /= I.shape[d]; }
    return off;
}

// VEC consecutive elements starting at flat offset `off`; WHOLE: all VEC are inside the row
template <int DT, int VOK, int WHOLE> __device__ __forceinline__ void ld_vec(const void* p, i64 off, int n, float (&o)[VEC]) {
    if (VOK && (WHOLE || n == VEC)) {
        if (DT == 8) {                  // 16 bytes per access: one (VEC 4) or two (VEC 8)
#pragma unroll
            for (int h = 0; h < VEC / 4; h++) {
                const float4 a = __ldg((const float4*)((const float*)p + off) + h);
                o[4 * h] = a.x; o[4 * h + 1] = a.y; o[4 * h + 2] = a.z; o[4 * h + 3] = a.w;
            }
            return;
        }
        if (DT == 7 || DT == 6) {       // 16 bytes (VEC 8) or 8 bytes (VEC 4)
            unsigned w[VEC / 2];
            if (VEC == 8) { const uint4 v = __ldg((const uint4*)((const u16*)p + off)); w[0] = v.x; w[1] = v.y; w[VEC / 2 - 2] = v.z; w[VEC / 2 - 1] = v.w; }
            else { const uint2 v = __ldg((const uint2*)((const u16*)p + off)); w[0] = v.x; w[1] = v.y; }
#pragma unroll
            for (int i = 0; i < VEC / 2; i++) {
                const u16 lo = (u16)(w[i] & 0xffffu), hi = (u16)(w[i] >> 16);
                o[2 * i] = DT == 7 ? bf2f(lo) : h2f(lo);
                o[2 * i + 1] = DT == 7 ? bf2f(hi) : h2f(hi);
            }
            return;
        }
    }
    FOR8 o[e] = (WHOLE || e < n) ? ld1<DT>(p, off + e) : 0.f;
}

// general broadcast: decompose the flat index of the first element, then step like an odometer
template <int DT, int ND, int WHOLE> __device__ __forceinline__ void ld_general(const Input& I, i64 flat, int n, float (&o)[VEC]) {
    i64 idx[ND];
    i64 off = 0;
#pragma unroll
    for (int d = ND - 1; d >= 0; d--) { idx[d] = flat % I.shape[d]; flat /= I.shape[d]; off += idx[d] * I.stride[d]; }
    FOR8 {
        o[e] = (WHOLE || e < n) ? ld1<DT>(I.ptr, off) : 0.f;
        bool carry = true;
#pragma unroll
        for (int d = ND - 1; d >= 0; d--) {
            if (carry) {
                off += I.stride[d];
                if (++idx[d] < I.shape[d]) carry = false;
                else { off -= I.stride[d] * I.shape[d]; idx[d] = 0; }
            }
        }
    }
}

template <int DT, int VOK, int WHOLE> __device__ __forceinline__ void st_vec(void* p, i64 off, int n, const float (&v)[VEC]) {
    if (VOK && (WHOLE || n == VEC)) {
        if (DT == 8) {
#pragma unroll
            for (int h = 0; h < VEC / 4; h++)
                __stcs((float4*)((float*)p + off) + h, make_float4(v[4 * h], v[4 * h + 1], v[4 * h + 2], v[4 * h + 3]));
            return;
        }
        if (DT == 7 || DT == 6) {
            unsigned w[VEC / 2];
#pragma unroll
            for (int i = 0; i < VEC / 2; i++) {
                const u16 lo = DT == 7 ? f2bf(v[2 * i]) : f2h(v[2 * i]), hi = DT == 7 ? f2bf(v[2 * i + 1]) : f2h(v[2 * i + 1]);
                w[i] = (unsigned)lo | ((unsigned)hi << 16);
            }
            if (VEC == 8) __stcs((uint4*)((u16*)p + off), make_uint4(w[0], w[1], w[VEC / 2 - 2], w[VEC / 2 - 1]));
            else __stcs((uint2*)((u16*)p + off), make_uint2(w[0], w[1]));
            return;
        }
    }
    FOR8 if (WHOLE || e < n) st1<DT>(p, off + e, v[e]);
}
)SRC";

struct Gen {
    const Program& Q;
    bool map, flat, whole;
    int G;
    int V;                              // elements per thread and step: 4 when every streamed tensor has 4-byte elements, else 8
    int variant;                        // map: 1 = a thread keeps its columns and walks the rows; rows: vectors of a row a thread keeps in registers (0: none)
    std::string s;
    bool held[kMaxInputs] = {};         // inputs whose vector is already in registers when a chain starts (not loaded by it)
    int cur_j = -1;                     // rows kernel with kept rows: which of the thread's vectors the chain works on

    void add(const std::string& t) { s += t; }
    static std::string num(long long v) { return std::to_string(v); }

    const Input& in(int k) const { return Q.in[k]; }
    bool per_element(int k) const { const int m = in(k).mode; return m == IN_FULL || m == IN_COL || m == IN_GENERAL; }

    static const char* unary_expr(int u) {
        switch (u) {
            case U_NEG: return "-v";
            case U_ABS: return "fabsf(v)";
            case U_LNOT: return "(float)(v == 0)";
            case U_LOG: return "logf(v)";
            case U_EXP: return "expf(v)";
            case U_SQRT: return "sqrtf(v)";
            case U_ROUND: return "roundf(v)";
            case U_FLOOR: return "floorf(v)";
            case U_CEIL: return "ceilf(v)";
            case U_SIN: return "sinf(v)";
            case U_ASIN: return "asinf(v)";
            case U_SINH: return "sinhf(v)";
            case U_ASINH: return "asinhf(v)";
            case U_TAN: return "tanf(v)";
            case U_ATAN: return "atanf(v)";
            case U_TANH: return "tanhf(v)";
            case U_ATANH: return "atanhf(v)";
            case U_COS: return "cosf(v)";
            case U_ACOS: return "acosf(v)";
            case U_COSH: return "coshf(v)";
            case U_ACOSH: return "acoshf(v)";
            case U_SIGMOID: return "1.f / (1.f + expf(-v < 30.f ? -v : 30.f))";
            case U_ERF: return "erff(v)";
            case U_ERFINV: return "erfinvf(v)";
        }
        return "v";         // cast: the rounding to the result dtype is the cast
    }
    static const char* binary_expr(int b) {
        switch (b) {
            case OP_ADD: return "__fadd_rn(p, q)";
            case OP_SUB: return "__fsub_rn(p, q)";
            case OP_MUL: return "__fmul_rn(p, q)";
            case OP_DIV: case OP_FLOORDIV: return "p / q";
            case OP_MOD: return "p - floorf(p / q) * q";
            case OP_POW: return "powf(p, q)";
            case OP_MAX: return "p > q ? p : q";
            case OP_MIN: return "q < p ? q : p";
            case OP_LT: return "(float)(p < q)";
            case OP_LE: return "(float)(p <= q)";
            case OP_GT: return "(float)(p > q)";
            case OP_GE: return "(float)(p >= q)";
            case OP_EQ: return "(float)(p == q)";
            case OP_NE: return "(float)(p != q)";
            case OP_LAND: return "(float)((p != 0) && (q != 0))";
            case OP_LOR: return "(float)((p != 0) || (q != 0))";
            case OP_LXOR: return "(float)((p != 0) != (q != 0))";
        }
        return "p";
    }
    static const char* fold_expr(int r) {
        switch (r) {
            case OP_MAX: return "a > b ? a : b";
            case OP_MIN: return "b < a ? b : a";
            case OP_MUL: return "a * b";
        }
        return "a + b";
    }
    static const char* fold_init(int r) {
        switch (r) {
            case OP_MAX: return "-FLT_MAX";
            case OP_MIN: return "FLT_MAX";
            case OP_MUL: return "1.f";
        }
        return "0.f";
    }

    // operand of word w as an expression in the element index e; advances pc over an inline constant
    std::string operand(int32_t w, int& pc) {
        const int kind = w_kind(w), idx = w_index(w);
        switch (kind) {
            case K_INPUT:
                if (in(idx).mode == IN_SCALAR) return "s" + num(idx);
                if (in(idx).mode == IN_ROW) return "r" + num(idx);
                if (held[idx] && cur_j >= 0) return "x" + num(idx) + "_" + num(cur_j) + "[e]";
                return "i" + num(idx) + "[e]";
            case K_CONST: return "c" + num(++pc);      // the value stays an argument: one kernel for every constant
            case K_ROWVAL: return "rv" + num(idx);
            default: return "t" + num(idx) + "[e]";
        }
    }

    // the load of input k at (row, col) into float i<k>[VEC]
    void load(int k, const std::string& ind, const std::string& dst = "", bool declare = true) {
        const Input& I = in(k);
        const std::string K = num(k), W = whole ? "1" : "0", D = dst.empty() ? "i" + K : dst;
        if (declare) add(ind + "float " + D + "[VEC];\n");
        if (I.mode == IN_GENERAL)
            add(ind + "ld_general<" + num(I.dtype) + ", " + num(I.nd) + ", " + W + ">(P.in[" + K + "], " + (flat ? "off" : "row * cols + col") + ", n, " + D + ");\n");
        else
            add(ind + "ld_vec<" + num(I.dtype) + ", " + num(I.vec_ok ? 1 : 0) + ", " + W + ">(P.in[" + K + "].ptr, " +
                (I.mode == IN_FULL ? (flat ? "off" : "row * cols + col") : "col") + ", n, " + D + ");\n");
    }

    // the chain that starts at code[pc]: leaves its value in acc[] and returns the pc of the statement word that ends it
    int chain(int pc, const std::string& ind) {
        // every per-element input of the chain is loaded once, before the arithmetic
        bool seen[kMaxInputs] = {};
        bool tmp_used[kTmp] = {};
        for (int q = pc;; q++) {
            const int32_t w = Q.code[q];
            if (w_op(w) >= CH_ROW_REDUCE) break;
            const int kind = w_kind(w), idx = w_index(w);
            if (w_op(w) == CH_TSTORE) { tmp_used[idx] = true; continue; }
            if (kind == K_CONST) q++;
            else if (kind == K_INPUT && per_element(idx) && !seen[idx]) { seen[idx] = true; if (!held[idx]) load(idx, ind); }
            else if (kind == K_TMP) tmp_used[idx] = true;
        }
        for (int t = 0; t < kTmp; t++)
            if (tmp_used[t]) add(ind + "float t" + num(t) + "[VEC];\n");
        add(ind + "float acc[VEC];\n");
        for (;; pc++) {
            const int32_t w = Q.code[pc];
            const int op = w_op(w);
            if (op >= CH_ROW_REDUCE) break;
            const int sub = w_sub(w), rdt = w_rdt(w);
            if (op == CH_TSTORE) { add(ind + "FOR8 t" + num(w_index(w)) + "[e] = acc[e];\n"); continue; }
            if (op == CH_UNARY) {
                if (sub != U_CAST) add(ind + "FOR8 { const float v = acc[e]; acc[e] = " + unary_expr(sub) + "; }\n");
            } else if (op == CH_LOAD) {
                add(ind + "FOR8 acc[e] = " + operand(w, pc) + ";\n");
            } else if (op == CH_BINARY) {
                const std::string o = operand(w, pc);
                if (w_swap(w)) add(ind + "FOR8 { const float p = " + o + ", q = acc[e]; acc[e] = " + binary_expr(sub) + "; }\n");
                else add(ind + "FOR8 { const float p = acc[e], q = " + o + "; acc[e] = " + binary_expr(sub) + "; }\n");
            } else {        // CH_SELECT: the second operand is described by the next word
                const std::string o1 = operand(w, pc);
                const int32_t w2 = Q.code[++pc];
                const std::string o2 = operand(w2, pc);
                add(ind + "FOR8 acc[e] = acc[e] != 0.f ? " + o1 + " : " + o2 + ";\n");
            }
            if (rdt == B200JT_BFLOAT16 || rdt == B200JT_FLOAT16 || rdt == B200JT_BOOL)
                add(ind + "FOR8 acc[e] = rnd<" + num(rdt) + ">(acc[e]);\n");
        }
        return pc;
    }

    void scalars() {
        for (int pc = 0; pc < Q.n_code; pc++) {
            const int32_t w = Q.code[pc];
            if (w_kind(w) == K_CONST && (w_op(w) < CH_TSTORE)) { pc++; add("    const float c" + num(pc) + " = __int_as_float(P.code[" + num(pc) + "]);\n"); }
        }
        for (int k = 0; k < Q.n_inputs; k++)
            if (in(k).mode == IN_SCALAR) add("    const float s" + num(k) + " = ld1<" + num(in(k).dtype) + ">(P.in[" + num(k) + "].ptr, 0);\n");
    }
    void row_inputs(const std::string& ind) {
        for (int k = 0; k < Q.n_inputs; k++)
            if (in(k).mode == IN_ROW)
                add(ind + "const float r" + num(k) + " = ld1<" + num(in(k).dtype) + ">(P.in[" + num(k) + "].ptr, row_offset<" + num(in(k).nd) + ">(P.in[" + num(k) + "], row));\n");
    }
    std::string store(const std::string& off) {
        return "st_vec<" + num(Q.out_dtype) + ", " + num(Q.out_vec_ok ? 1 : 0) + ", " + (whole ? "1" : "0") + ">(P.out, " + off + ", n, acc);\n";
    }

    void header() {
        add("#define MAXD " + num(kMaxDims) + "\n#define MAXIN " + num(kMaxInputs) + "\n#define MAXCODE " + num(kMaxCode) +
            "\n#define PROGRAM_BYTES " + num((long long)sizeof(Program)) + "\n#define VEC " + num(V) + "\n");
        add(kPrelude);
    }

    void gen_map() {
        header();
        add("extern \"C\" __global__ void __launch_bounds__(256) chain_jit_map_kernel(const __grid_constant__ Program P) {\n");
        add("    const i64 cols = P.cols;\n");
        scalars();
        if (flat) {
            // no input depends on the position inside the tensor: one flat index space
            add("    const i64 total = P.rows * cols, items = (total + VEC - 1) / VEC;\n");
            add("    for (i64 it = blockIdx.x * (i64)blockDim.x + threadIdx.x; it < items; it += (i64)gridDim.x * blockDim.x) {\n");
            add("        const i64 off = it * VEC;\n");
            add(std::string("        const int n = ") + (whole ? "VEC" : "(total - off < VEC ? (int)(total - off) : VEC)") + ";\n");
            chain(0, "        ");
            add("        " + store("off"));
            add("    }\n}\n");
            return;
        }
        if (variant == 1) {
            // inputs that are constant over the rows (bias, scale): a thread keeps its 8 columns, loads those inputs once
            // and walks down the rows, so the loop has no division and only the full-shape inputs touch memory
            add("    const i64 vpr = (cols + VEC - 1) / VEC;\n");
            add("    const i64 cv = (i64)blockIdx.x * blockDim.x + threadIdx.x;\n");
            add("    if (cv >= vpr) return;\n");
            add("    const i64 col = cv * VEC;\n");
            add(std::string("    const int n = ") + (whole ? "VEC" : "(cols - col < VEC ? (int)(cols - col) : VEC)") + ";\n");
            for (int k = 0; k < Q.n_inputs; k++)
                if (in(k).mode == IN_COL) { load(k, "    "); held[k] = true; }
            add("    for (i64 row = (i64)blockIdx.y * blockDim.y + threadIdx.y; row < P.rows; row += (i64)gridDim.y * blockDim.y) {\n");
            row_inputs("        ");
            chain(0, "        ");
            add("        " + store("row * cols + col"));
            add("    }\n}\n");
            return;
        }
        add("    const i64 vpr = (cols + VEC - 1) / VEC, items = P.rows * vpr;\n");
        add("    const bool small = items < (1LL << 31);\n");
        add("    for (i64 it = blockIdx.x * (i64)blockDim.x + threadIdx.x; it < items; it += (i64)gridDim.x * blockDim.x) {\n");
        add("        const i64 row = small ? (i64)((unsigned)it / (unsigned)vpr) : it / vpr, col = (it - row * vpr) * VEC;\n");
        add(std::string("        const int n = ") + (whole ? "VEC" : "(cols - col < VEC ? (int)(cols - col) : VEC)") + ";\n");
        row_inputs("        ");
        chain(0, "        ");
        add("        " + store("row * cols + col"));
        add("    }\n}\n");
    }

    void gen_rows() {
        header();
        add("extern \"C\" __global__ void __launch_bounds__(256) chain_jit_rows_kernel(const __grid_constant__ Program P) {\n");
        add("    constexpr int G = " + num(G) + ", GROUPS = 256 / G;\n");
        add("    __shared__ float xch[8];\n");
        add("    const i64 cols = P.cols;\n");
        add("    const int g = threadIdx.x / G, t = threadIdx.x % G;\n");
        add("    const i64 n_groups = (i64)gridDim.x * GROUPS;\n");
        add("    const float rcols = 1.f / (float)cols;\n");
        scalars();
        // the trip count is the same for every thread of a CTA, so the barriers inside the loop are legal for G == 256
        // rows short enough to keep: every full-shape or column input of a sweep is read once per row (column inputs once per
        // thread) into registers, and the later sweeps work from there instead of going back to L1 / L2
        bool swept[kMaxInputs] = {};
        if (variant > 0) {
            for (int pc = 0; pc < Q.n_code;) {
                int end = pc;
                while (w_op(Q.code[end]) < CH_ROW_REDUCE) end += (w_kind(Q.code[end]) == K_CONST) ? 2 : 1;
                const int sop = w_op(Q.code[end]);
                if (sop == CH_ROW_REDUCE || sop == CH_STORE)
                    for (int q = pc; q < end; q++) {
                        const int32_t w = Q.code[q];
                        if (w_kind(w) == K_CONST) { q++; continue; }
                        if (w_op(w) != CH_TSTORE && w_kind(w) == K_INPUT && (in(w_index(w)).mode == IN_FULL || in(w_index(w)).mode == IN_COL)) swept[w_index(w)] = true;
                    }
                pc = end + 1;
            }
        }
        auto keep = [&](int mode, const std::string& ind) {
            for (int k = 0; k < Q.n_inputs; k++)
                if (swept[k] && in(k).mode == mode)
                    for (int j = 0; j < variant; j++) {
                        const std::string D = "x" + num(k) + "_" + num(j);
                        add(ind + "float " + D + "[VEC];\n");
                        add(ind + "{ const i64 col = ((i64)t + " + num(j) + " * G) * VEC; if (col < cols) { " +
                            std::string("const int n = ") + (whole ? "VEC" : "(cols - col < VEC ? (int)(cols - col) : VEC)") + ";\n");
                        load(k, ind + "    ", D, false);
                        add(ind + "} else { FOR8 " + D + "[e] = 0.f; } }\n");
                        held[k] = true;
                    }
        };
        keep(IN_COL, "    ");
        add("    for (i64 row = (i64)blockIdx.x * GROUPS + g; row < P.rows; row += n_groups) {\n");
        row_inputs("        ");
        keep(IN_FULL, "        ");
        bool rv_used[kMaxRowVals] = {};
        for (int pc = 0; pc < Q.n_code; pc++) {
            const int32_t w = Q.code[pc];
            if (w_op(w) >= CH_ROW_REDUCE && w_op(w) != CH_STORE) rv_used[w_index(w)] = true;
            else if (w_kind(w) == K_ROWVAL) rv_used[w_index(w)] = true;
            if (w_op(w) < CH_ROW_REDUCE && w_kind(w) == K_CONST) pc++;
        }
        for (int j = 0; j < kMaxRowVals; j++)
            if (rv_used[j]) add("        float rv" + num(j) + " = 0.f;\n");
        int pc = 0;
        while (pc < Q.n_code) {
            int end = pc;
            while (w_op(Q.code[end]) < CH_ROW_REDUCE) end += (w_kind(Q.code[end]) == K_CONST) ? 2 : 1;
            const int32_t w = Q.code[end];
            const int sop = w_op(w), a = w_index(w), rdt = w_rdt(w), rop = w_sub(w);
            if (sop == CH_STORE_ROW) {
                add("        if (t == 0) st1<" + num(Q.out_dtype) + ">(P.out, row, rv" + num(a) + ");\n");
            } else if (sop == CH_ROW_MAP) {
                // evaluated once per row by every thread of the group, at column 0
                add("        {\n            const i64 col = 0; const int n = 1;\n");
                const bool w0 = whole; whole = false;
                bool h0[kMaxInputs];
                for (int k = 0; k < kMaxInputs; k++) { h0[k] = held[k]; held[k] = false; }
                chain(pc, "            ");
                for (int k = 0; k < kMaxInputs; k++) held[k] = h0[k];
                whole = w0;
                add("            rv" + num(a) + " = acc[0];\n        }\n");
            } else {
                add("        {\n");
                if (sop == CH_ROW_REDUCE) add(std::string("            float racc = ") + fold_init(rop) + ";\n");
                // with kept rows the sweep is written out per vector of the thread (same order as the loop, same bits)
                for (int j = 0; j < (variant > 0 ? variant : 1); j++) {
                    if (variant > 0) {
                        cur_j = j;
                        add("            { const i64 col = ((i64)t + " + num(j) + " * G) * VEC; if (col < cols) {\n");
                    } else add("            for (i64 col = (i64)t * VEC; col < cols; col += (i64)G * VEC) {\n");
                    add(std::string("                const int n = ") + (whole ? "VEC" : "(cols - col < VEC ? (int)(cols - col) : VEC)") + ";\n");
                    chain(pc, "                ");
                    if (sop == CH_STORE) add("                " + store("row * cols + col"));
                    else if (rop == OP_MEAN) add(std::string("                FOR8 if (") + (whole ? "true" : "e < n") + ") racc = fmaf(acc[e], rcols, racc);\n");
                    else add(std::string("                FOR8 if (") + (whole ? "true" : "e < n") + ") { const float a = racc, b = acc[e]; racc = " + fold_expr(rop) + "; }\n");
                    add(variant > 0 ? "            } }\n" : "            }\n");
                }
                cur_j = -1;
                if (sop == CH_ROW_REDUCE) {
                    add(std::string("#pragma unroll\n            for (int d = 16; d > 0; d >>= 1) { const float a = racc, b = __shfl_xor_sync(0xffffffffu, racc, d); racc = ") + fold_expr(rop) + "; }\n");
                    if (G == 256) {
                        add("            __syncthreads();\n            if ((threadIdx.x & 31) == 0) xch[threadIdx.x >> 5] = racc;\n            __syncthreads();\n");
                        add("            racc = xch[0];\n");
                        add(std::string("#pragma unroll\n            for (int k = 1; k < 8; k++) { const float a = racc, b = xch[k]; racc = ") + fold_expr(rop) + "; }\n");
                    }
                    add("            rv" + num(a) + " = rnd<" + num(rdt) + ">(racc);\n");
                }
                add("        }\n");
            }
            pc = end + 1;
        }
        add("    }\n}\n");
    }
};

// The form of the kernel a program gets; everything here is part of the cache key.
struct Form { int V, G, variant; bool whole; };

std::string make_key(const Program& Q, bool map, bool flat, const Form& f) {
    std::string k;
    k.reserve(64 + 4 * Q.n_code);
    const int32_t head[10] = {Q.n_inputs, Q.n_code, Q.out_dtype, Q.out_vec_ok, map, flat, f.whole, f.G, f.variant, f.V};
    k.append((const char*)head, sizeof head);
    for (int pc = 0; pc < Q.n_code; pc++) {
        const int32_t w = Q.code[pc];
        k.append((const char*)&w, 4);
        if (w_kind(w) == K_CONST && w_op(w) < CH_TSTORE) { const int32_t zero = 0; k.append((const char*)&zero, 4); pc++; }
    }
    for (int i = 0; i < Q.n_inputs; i++) {
        const int32_t v[4] = {Q.in[i].dtype, Q.in[i].mode, Q.in[i].vec_ok, (Q.in[i].mode == IN_ROW || Q.in[i].mode == IN_GENERAL) ? Q.in[i].nd : 0};
        k.append((const char*)v, sizeof v);
    }
    return k;
}

int jit_mode() {
    const char* e = getenv("B200JT_CHAIN_JIT");
    return e ? atoi(e) : 1;
}

}  // namespace

static Form pick_form(const Program& Q, bool pure_map, bool flat) {
    Form f;
    // 16 bytes per thread and access: 4 elements when every tensor that is streamed has 4-byte elements, else 8
    bool narrow = dtype_size(Q.out_dtype) < 4;
    for (int k = 0; k < Q.n_inputs; k++)
        if (Q.in[k].mode == IN_FULL || Q.in[k].mode == IN_COL || Q.in[k].mode == IN_GENERAL) narrow |= dtype_size(Q.in[k].dtype) < 4;
    f.V = narrow ? 8 : 4;
    f.whole = flat ? (Q.rows * Q.cols) % f.V == 0 : Q.cols % f.V == 0;
    f.G = Q.cols <= 128 * f.V ? 32 : 256;
    if (pure_map) {
        // column-keeping map: some input is constant over the rows and the rows are long enough to fill a CTA's x extent
        bool col_input = false;
        for (int k = 0; k < Q.n_inputs; k++) col_input |= Q.in[k].mode == IN_COL;
        f.variant = (!flat && col_input && Q.cols >= 8 * f.V && Q.rows >= 64) ? 1 : 0;
        f.G = 0;
        return f;
    }
    // rows kernel: keep the row when all kept vectors of a thread fit in 64 registers
    const int64_t per_thread = (Q.cols + (int64_t)f.G * f.V - 1) / ((int64_t)f.G * f.V);
    int inputs = 0;
    for (int k = 0; k < Q.n_inputs; k++) inputs += Q.in[k].mode == IN_FULL || Q.in[k].mode == IN_COL;
    f.variant = (per_thread >= 1 && inputs > 0 && per_thread * inputs * f.V <= 64) ? (int)per_thread : 0;
    return f;
}

// Vector accesses need the base and every row start on a multiple of the access size.
static void set_vector_flags(Program& Q, bool flat, int V) {
    auto ok = [&](const void* p, int dt, bool per_row) {
        const int es = dtype_size(dt);
        if (es != 4 && es != 2) return false;
        const uintptr_t access = (uintptr_t)std::min(16, V * es);
        if ((uintptr_t)p % access != 0) return false;
        return flat || !per_row || Q.cols % V == 0 || Q.rows == 1;
    };
    for (int k = 0; k < Q.n_inputs; k++) {
        Input& I = Q.in[k];
        I.vec_ok = (I.mode == IN_FULL && ok(I.ptr, I.dtype, true)) || (I.mode == IN_COL && ok(I.ptr, I.dtype, false) && Q.cols % V == 0);
    }
    Q.out_vec_ok = ok(Q.out, Q.out_dtype, true);
}

static std::string source_for(const Program& Q, bool pure_map, bool flat, const Form& f) {
    Gen g{Q, pure_map, flat, f.whole, f.G ? f.G : 256, f.V, f.variant, {}};
    if (pure_map) g.gen_map(); else g.gen_rows();
    return g.s;
}

// The CUDA source that jit_launch would compile for Q (for tests and for reading).
std::string jit_source(const Program& Q0, bool pure_map, bool flat) {
    Program Q = Q0;
    const Form f = pick_form(Q, pure_map, flat);
    set_vector_flags(Q, flat, f.V);
    return source_for(Q, pure_map, flat, f);
}

thread_local DryRun* t_dry_run = nullptr;

int jit_launch(const Program& Q0, bool pure_map, bool flat, cudaStream_t st) {
    Program Q = Q0;
    const Form f = pick_form(Q, pure_map, flat);
    set_vector_flags(Q, flat, f.V);
    if (t_dry_run) {
        // generate and compile only; nothing is loaded or launched, so this works without a GPU
        t_dry_run->source = source_for(Q, pure_map, flat, f);
        t_dry_run->compiled = jit::compile_only(t_dry_run->source, &t_dry_run->log);
        return 0;
    }
    const int mode = jit_mode();
    if (mode == 0) return kJitUnavailable;
    std::string why;
    if (!jit::available(&why)) return mode == 2 ? fail(-1, "b200jt_fused_chain: run-time compiler unavailable: " + why) : kJitUnavailable;
    std::string log;
    const cudaKernel_t kernel = jit::get_kernel("chain:" + make_key(Q, pure_map, flat, f), [&] { return source_for(Q, pure_map, flat, f); },
                                                pure_map ? "chain_jit_map_kernel" : "chain_jit_rows_kernel", &log);
    if (!kernel) return mode == 2 ? fail(-1, "b200jt_fused_chain: compiling the chain failed: " + log) : kJitUnavailable;
    dim3 grid(1), block(256);
    const int V = f.V;
    if (pure_map && f.variant == 1) {
        // x: the column vectors of a row (a power of two up to 256 wide), y: rows; about 8 CTAs per SM in all
        const int64_t vpr = (Q.cols + V - 1) / V;
        int bx = 8;
        while (bx < 256 && bx < vpr) bx *= 2;
        block = dim3(bx, 256 / bx);
        const int64_t gx = (vpr + bx - 1) / bx, row_ctas = (Q.rows + block.y - 1) / block.y;
        const int64_t cap = std::max<int64_t>(1, (int64_t)grid_for(INT64_MAX / 512, 256) / gx);
        grid = dim3((unsigned)gx, (unsigned)std::min<int64_t>(std::min(row_ctas, cap), 65535));
    } else if (pure_map) {
        const int64_t items = flat ? (Q.rows * Q.cols + V - 1) / V : Q.rows * ((Q.cols + V - 1) / V);
        grid = dim3(grid_for(items, 256));
    } else if (f.G == 32) grid = dim3(grid_for((Q.rows + 7) / 8 * 256, 256));
    else grid = dim3(grid_for(Q.rows * 256, 256));
    void* args[] = {(void*)&Q};
    B200JT_CUDA(cudaLaunchKernel((const void*)kernel, grid, block, args, 0, st));
    return 0;
}

}  // namespace chain
}  // namespace b200jt

using namespace b200jt;

/* The CUDA source the run-time specialiser generates for a call of b200jt_fused_chain with the same arguments, without
 * launching anything: the pointers in the descriptors are only looked at for their alignment. Copies at most cap bytes
 * (NUL-terminated) into src, stores the full length in *needed, and sets *compiled to 1 if NVRTC accepted the source
 * for sm_100a (0 with the compiler's log in b200jt_last_error() otherwise). Needs no GPU. */
extern "C" int b200jt_fused_chain_source(const b200jt_tensor* inputs, int n_inputs, const int64_t* full_shape, int ndim, int row_axes,
                                         const int32_t* code, int n_code, const b200jt_tensor* out, char* src, int64_t cap,
                                         int64_t* needed, int* compiled) {
    chain::DryRun dry;
    chain::t_dry_run = &dry;
    const int rc = b200jt_fused_chain(inputs, n_inputs, full_shape, ndim, row_axes, code, n_code, out, nullptr);
    chain::t_dry_run = nullptr;
    if (rc != 0) return rc;
    if (needed) *needed = (int64_t)dry.source.size();
    if (src && cap > 0) {
        const size_t n = std::min((size_t)cap - 1, dry.source.size());
        memcpy(src, dry.source.data(), n); src[n] = 0;
    }
    if (compiled) *compiled = dry.compiled ? 1 : 0;
    if (!dry.compiled) set_error("b200jt_fused_chain_source: " + dry.log);
    return 0;
}

/* Counters of the run-time specialiser since the process started: kernels compiled, launches served from the cache,
 * compilations that failed (those chains run through the interpreter kernels). Any pointer may be NULL. */
extern "C" int b200jt_chain_jit_stats(int* compiled, int* hits, int* failed) {
    jit::stats(compiled, hits, failed);
    return 0;
}
