// Index programs: the reference pastes the `indexes` / `overflow_conditions` strings of reindex and
// reindex_reduce into generated C++ (python/jittor/src/ops/reindex_op.cc:131-137). Here the same
// strings are compiled once on the host into (a) a postfix bytecode that a generic kernel interprets
// per element, and (b) where every index is affine in i0..in, a coefficient table for the fast kernels.
#pragma once
#include "common.cuh"
#include <vector>

namespace b200jt {

enum IxOp : int {
    IX_CONST = 0,   // push imm24 (sign-extended)
    IX_CONST64,     // push the next two words (lo, hi)
    IX_LOOPVAR,     // push i<imm>
    IX_ADD, IX_SUB, IX_MUL, IX_DIV, IX_MOD, IX_NEG, IX_LNOT, IX_BNOT,
    IX_LT, IX_LE, IX_GT, IX_GE, IX_EQ, IX_NE, IX_LAND, IX_LOR, IX_BAND, IX_BOR, IX_BXOR, IX_SHL, IX_SHR,
    IX_SELECT,      // pop c, b, a -> a ? b : c   (stack order: cond, then, else)
    IX_LOAD_EXT,    // imm = k | nargs<<8 : pop nargs subscripts, push (index_t) extras[k][...]
    IX_STORE_XID,   // imm = d : pop -> xid[d]
    IX_STORE_COND   // pop -> overflow |= (v != 0)
};

constexpr int kMaxCode = 192;
constexpr int kIxStack = 16;

struct ExtraDesc {
    const void* ptr;
    int32_t dtype;
    int32_t ndim;
    int64_t shape[kMaxDims];
};

// Passed to kernels by value (__grid_constant__).
struct IndexProgram {
    int32_t ndim_loop;                 // rank of the iterated tensor (i0..in)
    int32_t ndim_x;                    // rank of the indexed tensor
    int64_t loop_shape[kMaxDims];
    int64_t x_shape[kMaxDims];
    int32_t n_code;
    int32_t n_extras;
    int32_t code[kMaxCode];
    ExtraDesc extras[B200JT_MAX_EXTRAS];
    // affine form: xid[d] = c0[d] + sum_j coef[d][j] * i_j, no user conditions, no extras
    int32_t is_affine;
    int64_t coef[kMaxDims][kMaxDims];
    int64_t c0[kMaxDims];
    // "direct scatter/gather": one indexed dim, index = @e0(i0..in) with identity subscripts and
    // extras[0] shaped like the loop tensor (x[e0[i]] <- y[i])
    int32_t is_direct_extra;
    // "inner run": the last inner_dims loop axes map one-to-one onto the last inner_dims axes of x (index = that loop
    // variable, equal extents) and nothing else reads them, so inner_elems consecutive loop elements address
    // inner_elems consecutive x elements and the program only has to be evaluated once per run
    int32_t inner_dims;
    int64_t inner_elems;
};

// Compiles the strings. Returns false and sets `err` on a syntax error (the reference rejects the
// same inputs when its generated source fails to compile).
bool compile_index_program(const int64_t* loop_shape, int ndim_loop, const int64_t* x_shape, int ndim_x,
                           const char* const* indexes, int n_indexes,
                           const char* const* conds, int n_conds,
                           const b200jt_tensor* extras, int n_extras,
                           IndexProgram* out, std::string* err);

#ifdef __CUDACC__
// Evaluates the program for loop coordinates `iv`; writes xid[0..ndim_x) and returns the overflow flag
// (out-of-range index or a user condition that is true).
template <typename I>
__device__ __forceinline__ bool eval_index_program(const IndexProgram& P, const I* iv, I* xid) {
    I st[kIxStack];
    int sp = 0;
    bool over = false;
    for (int pc = 0; pc < P.n_code; pc++) {
        int32_t w = P.code[pc];
        int op = w & 0xff;
        int imm = w >> 8;
        switch (op) {
            case IX_CONST: st[sp++] = (I)imm; break;
            case IX_CONST64: {
                uint64_t lo = (uint32_t)P.code[pc + 1], hi = (uint32_t)P.code[pc + 2];
                st[sp++] = (I)(int64_t)(lo | (hi << 32)); pc += 2; break;
            }
            case IX_LOOPVAR: st[sp++] = iv[imm]; break;
            case IX_NEG: st[sp - 1] = -st[sp - 1]; break;
            case IX_LNOT: st[sp - 1] = (I)(st[sp - 1] == 0); break;
            case IX_BNOT: st[sp - 1] = ~st[sp - 1]; break;
            case IX_SELECT: {
                I c = st[--sp], b = st[--sp]; st[sp - 1] = st[sp - 1] != 0 ? b : c; break;
            }
            case IX_LOAD_EXT: {
                int k = imm & 0xff, na = imm >> 8;
                const ExtraDesc& e = P.extras[k];
                int64_t flat = 0;
                for (int a = 0; a < na; a++) flat = flat * e.shape[a] + (int64_t)st[sp - na + a];
                sp -= na;
                I v;
                if (e.dtype == B200JT_INT32) v = (I)((const int32_t*)e.ptr)[flat];
                else if (e.dtype == B200JT_INT64) v = (I)((const int64_t*)e.ptr)[flat];
                else v = (I)load_as<double>(e.ptr, e.dtype, flat);
                st[sp++] = v; break;
            }
            case IX_STORE_XID: {
                I v = st[--sp]; xid[imm] = v;
                over |= (v < 0) | (v >= (I)P.x_shape[imm]); break;
            }
            case IX_STORE_COND: over |= (st[--sp] != 0); break;
            default: {
                I b = st[--sp], a = st[sp - 1], r = 0;
                switch (op) {
                    case IX_ADD: r = a + b; break;
                    case IX_SUB: r = a - b; break;
                    case IX_MUL: r = a * b; break;
                    case IX_DIV: r = b != 0 ? a / b : 0; break;
                    case IX_MOD: r = b != 0 ? a % b : 0; break;
                    case IX_LT: r = a < b; break;
                    case IX_LE: r = a <= b; break;
                    case IX_GT: r = a > b; break;
                    case IX_GE: r = a >= b; break;
                    case IX_EQ: r = a == b; break;
                    case IX_NE: r = a != b; break;
                    case IX_LAND: r = (a != 0) && (b != 0); break;
                    case IX_LOR: r = (a != 0) || (b != 0); break;
                    case IX_BAND: r = a & b; break;
                    case IX_BOR: r = a | b; break;
                    case IX_BXOR: r = a ^ b; break;
                    case IX_SHL: r = a << b; break;
                    case IX_SHR: r = a >> b; break;
                }
                st[sp - 1] = r;
            }
        }
    }
    return over;
}
#endif

}  // namespace b200jt
