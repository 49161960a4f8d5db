// Host-side compiler of reindex index strings into IndexProgram (see index_program.cuh).
// Grammar: C integer expressions -- literals, i0..i9, <name>shape<k>/<name>stride<k> symbols,
// @eK(e, ...) loads, unary - + ! ~, binary * / % + - << >> < <= > >= == != & ^ | && ||, ?:, parentheses.
// `//` is rejected, as in the reference (python/jittor/src/opt/pass/loop_var_analyze_pass.cc:298-309).
#include "index_program.cuh"

#include <cctype>
#include <cstdlib>
#include <map>

namespace b200jt {
namespace {

struct Affine {               // value = c + sum coef[j]*i_j   (valid only if ok)
    bool ok = true;
    int64_t c = 0;
    int64_t coef[kMaxDims] = {0};
    bool is_const() const { for (int j = 0; j < kMaxDims; j++) if (coef[j]) return false; return ok; }
};

struct Compiler {
    const char* s;
    size_t pos = 0;
    std::string err;
    std::vector<int32_t> code;
    std::vector<Affine> aff;          // symbolic stack mirroring the runtime stack
    int depth = 0, max_depth = 0;
    std::map<std::string, int64_t> syms;
    int ndim_loop = 0, n_extras = 0;
    const b200jt_tensor* extras = nullptr;
    bool used_extra = false;
    // direct-extra detection: the expression is exactly @e0(i0,..,in)
    bool direct_candidate = false;

    bool fail(const std::string& m) { if (err.empty()) err = m + " in \"" + s + "\""; return false; }
    void skip() { while (s[pos] && isspace((unsigned char)s[pos])) pos++; }
    bool peek(const char* t) { skip(); return strncmp(s + pos, t, strlen(t)) == 0; }
    bool accept(const char* t) { if (peek(t)) { pos += strlen(t); return true; } return false; }

    void emit(int op, int imm = 0) { code.push_back((op & 0xff) | (imm << 8)); }
    void push_aff(const Affine& a) { aff.push_back(a); depth++; if (depth > max_depth) max_depth = depth; }
    Affine pop_aff() { Affine a = aff.back(); aff.pop_back(); depth--; return a; }

    void emit_const(int64_t v) {
        if (v >= -(1 << 22) && v < (1 << 22)) emit(IX_CONST, (int)v);
        else { emit(IX_CONST64); code.push_back((int32_t)(uint32_t)(v & 0xffffffffu)); code.push_back((int32_t)(uint32_t)((uint64_t)v >> 32)); }
        Affine a; a.c = v; push_aff(a);
    }

    void binop(int op) {
        Affine b = pop_aff(), a = pop_aff(), r;
        emit(op);
        r.ok = false;
        if (a.ok && b.ok) {
            if (op == IX_ADD || op == IX_SUB) {
                r.ok = true; int sg = op == IX_ADD ? 1 : -1;
                r.c = a.c + sg * b.c;
                for (int j = 0; j < kMaxDims; j++) r.coef[j] = a.coef[j] + sg * b.coef[j];
            } else if (op == IX_MUL && (a.is_const() || b.is_const())) {
                const Affine& k = a.is_const() ? a : b; const Affine& v = a.is_const() ? b : a;
                r.ok = true; r.c = v.c * k.c;
                for (int j = 0; j < kMaxDims; j++) r.coef[j] = v.coef[j] * k.c;
            } else if (a.is_const() && b.is_const()) {
                // constant folding of the remaining operators keeps e.g. "i0*(4/2)" affine
                int64_t x = a.c, y = b.c, v = 0; bool ok = true;
                switch (op) {
                    case IX_DIV: if (y) v = x / y; else ok = false; break;
                    case IX_MOD: if (y) v = x % y; else ok = false; break;
                    case IX_SHL: v = x << y; break;
                    case IX_SHR: v = x >> y; break;
                    default: ok = false;
                }
                if (ok) { r = Affine(); r.c = v; }
            }
        }
        push_aff(r);
    }

    bool expr() { return ternary(); }

    bool ternary() {
        if (!lor()) return false;
        if (accept("?")) {
            if (!ternary()) return false;
            skip(); if (!accept(":")) return fail("expected ':'");
            if (!ternary()) return false;
            emit(IX_SELECT); pop_aff(); pop_aff(); pop_aff(); Affine r; r.ok = false; push_aff(r);
        }
        return true;
    }
    bool lor()  { if (!land()) return false; while (peek("||")) { pos += 2; if (!land()) return false; binop(IX_LOR); } return true; }
    bool land() { if (!bor()) return false;  while (peek("&&")) { pos += 2; if (!bor()) return false; binop(IX_LAND); } return true; }
    bool bor()  { if (!bxor()) return false; while (peek("|") && !peek("||")) { pos += 1; if (!bxor()) return false; binop(IX_BOR); } return true; }
    bool bxor() { if (!band()) return false; while (peek("^")) { pos += 1; if (!band()) return false; binop(IX_BXOR); } return true; }
    bool band() { if (!eq()) return false;   while (peek("&") && !peek("&&")) { pos += 1; if (!eq()) return false; binop(IX_BAND); } return true; }
    bool eq() {
        if (!rel()) return false;
        for (;;) {
            if (peek("==")) { pos += 2; if (!rel()) return false; binop(IX_EQ); }
            else if (peek("!=")) { pos += 2; if (!rel()) return false; binop(IX_NE); }
            else return true;
        }
    }
    bool rel() {
        if (!shift()) return false;
        for (;;) {
            if (peek("<=")) { pos += 2; if (!shift()) return false; binop(IX_LE); }
            else if (peek(">=")) { pos += 2; if (!shift()) return false; binop(IX_GE); }
            else if (peek("<") && !peek("<<")) { pos += 1; if (!shift()) return false; binop(IX_LT); }
            else if (peek(">") && !peek(">>")) { pos += 1; if (!shift()) return false; binop(IX_GT); }
            else return true;
        }
    }
    bool shift() {
        if (!add()) return false;
        for (;;) {
            if (peek("<<")) { pos += 2; if (!add()) return false; binop(IX_SHL); }
            else if (peek(">>")) { pos += 2; if (!add()) return false; binop(IX_SHR); }
            else return true;
        }
    }
    bool add() {
        if (!mul()) return false;
        for (;;) {
            if (peek("+")) { pos += 1; if (!mul()) return false; binop(IX_ADD); }
            else if (peek("-")) { pos += 1; if (!mul()) return false; binop(IX_SUB); }
            else return true;
        }
    }
    bool mul() {
        if (!unary()) return false;
        for (;;) {
            if (peek("//")) return fail("'//' is not an operator of the index language");
            if (peek("*")) { pos += 1; if (!unary()) return false; binop(IX_MUL); }
            else if (peek("/")) { pos += 1; if (!unary()) return false; binop(IX_DIV); }
            else if (peek("%")) { pos += 1; if (!unary()) return false; binop(IX_MOD); }
            else return true;
        }
    }
    bool unary() {
        skip();
        if (accept("-")) {
            if (!unary()) return false;
            emit(IX_NEG); Affine a = pop_aff();
            if (a.ok) { a.c = -a.c; for (int j = 0; j < kMaxDims; j++) a.coef[j] = -a.coef[j]; }
            push_aff(a); return true;
        }
        if (accept("+")) return unary();
        if (accept("!")) { if (!unary()) return false; emit(IX_LNOT); pop_aff(); Affine r; r.ok = false; push_aff(r); return true; }
        if (accept("~")) { if (!unary()) return false; emit(IX_BNOT); pop_aff(); Affine r; r.ok = false; push_aff(r); return true; }
        return atom();
    }
    bool atom() {
        skip();
        char c = s[pos];
        if (isdigit((unsigned char)c)) {
            char* end; long long v = strtoll(s + pos, &end, 0); pos = end - s;
            emit_const(v); return true;
        }
        if (c == '(') {
            pos++; if (!expr()) return false; skip();
            if (!accept(")")) return fail("expected ')'");
            return true;
        }
        if (c == '@') {
            if (s[pos + 1] != 'e' || !isdigit((unsigned char)s[pos + 2])) return fail("expected @e<k>(...)");
            pos += 2; int k = 0;
            while (isdigit((unsigned char)s[pos])) k = k * 10 + (s[pos++] - '0');
            if (k >= n_extras) return fail("@e" + std::to_string(k) + " but only " + std::to_string(n_extras) + " extras");
            skip(); if (!accept("(")) return fail("expected '(' after @e<k>");
            int na = 0; bool identity = true;
            size_t code_before = code.size();
            for (;;) {
                size_t c0 = code.size();
                if (!expr()) return false;
                // identity subscript a == i_a ?
                if (!(code.size() == c0 + 1 && code[c0] == ((IX_LOOPVAR & 0xff) | (na << 8)))) identity = false;
                na++; skip();
                if (accept(",")) continue;
                if (accept(")")) break;
                return fail("expected ',' or ')'");
            }
            if (na != extras[k].ndim) return fail("@e" + std::to_string(k) + " takes " + std::to_string(extras[k].ndim) + " subscripts");
            for (int a = 0; a < na; a++) pop_aff();
            emit(IX_LOAD_EXT, k | (na << 8));
            Affine r; r.ok = false; push_aff(r);
            used_extra = true;
            direct_candidate = (code_before == 0 && k == 0 && identity && na == ndim_loop);
            return true;
        }
        if (isalpha((unsigned char)c) || c == '_') {
            size_t b = pos;
            while (isalnum((unsigned char)s[pos]) || s[pos] == '_') pos++;
            std::string name(s + b, pos - b);
            if (name.size() >= 2 && name[0] == 'i' && isdigit((unsigned char)name[1]) &&
                name.find_first_not_of("0123456789", 1) == std::string::npos) {
                int d = atoi(name.c_str() + 1);
                if (d >= ndim_loop) return fail("loop variable " + name + " out of range");
                emit(IX_LOOPVAR, d);
                Affine a; a.coef[d] = 1; push_aff(a); return true;
            }
            auto it = syms.find(name);
            if (it == syms.end()) return fail("unknown symbol '" + name + "'");
            emit_const(it->second); return true;
        }
        return fail(std::string("unexpected character '") + (c ? c : '$') + "'");
    }

    bool compile_one(const char* text, Affine* out) {
        s = text; pos = 0; depth = 0; aff.clear();
        size_t before = code.size();
        direct_candidate = false;
        bool whole_is_load = false;
        if (!expr()) return false;
        skip();
        if (s[pos]) return fail("trailing characters");
        // a lone @e0(i0..in): the last word is the LOAD_EXT and nothing precedes the subscripts
        whole_is_load = direct_candidate && before == 0 && (code.back() & 0xff) == IX_LOAD_EXT &&
                        code.size() == (size_t)ndim_loop + 1;
        direct_candidate = whole_is_load;
        *out = pop_aff();
        return true;
    }
};

void add_shape_syms(std::map<std::string, int64_t>& m, const std::string& prefix, const int64_t* shape, int nd) {
    int64_t st = 1;
    for (int d = nd - 1; d >= 0; d--) {
        m[prefix + "shape" + std::to_string(d)] = shape[d];
        m[prefix + "stride" + std::to_string(d)] = st;
        st *= shape[d];
    }
}

}  // namespace

bool compile_index_program(const int64_t* loop_shape, int ndim_loop, const int64_t* x_shape, int ndim_x,
                           const char* const* indexes, int n_indexes,
                           const char* const* conds, int n_conds,
                           const b200jt_tensor* extras, int n_extras,
                           IndexProgram* P, std::string* err) {
    memset(P, 0, sizeof(*P));
    P->ndim_loop = ndim_loop; P->ndim_x = ndim_x; P->n_extras = n_extras;
    for (int d = 0; d < ndim_loop; d++) P->loop_shape[d] = loop_shape[d];
    for (int d = 0; d < ndim_x; d++) P->x_shape[d] = x_shape[d];
    for (int k = 0; k < n_extras; k++) {
        P->extras[k].ptr = extras[k].ptr; P->extras[k].dtype = extras[k].dtype; P->extras[k].ndim = extras[k].ndim;
        for (int d = 0; d < extras[k].ndim; d++) P->extras[k].shape[d] = extras[k].shape[d];
    }
    Compiler C;
    C.ndim_loop = ndim_loop; C.n_extras = n_extras; C.extras = extras;
    // In reindex the indexed tensor is x and the loop tensor y; in reindex_reduce the loop tensor is y
    // and the indexed one x as well (reindex_reduce_op.cc:104-114), so the symbol names coincide.
    add_shape_syms(C.syms, "x", x_shape, ndim_x);
    add_shape_syms(C.syms, "y", loop_shape, ndim_loop);
    for (int k = 0; k < n_extras; k++)
        add_shape_syms(C.syms, "extras" + std::to_string(k), extras[k].shape, extras[k].ndim);

    bool affine = (n_conds == 0);
    bool direct = (n_indexes == 1 && n_conds == 0 && n_extras >= 1);
    std::vector<size_t> seg_begin, seg_end;          // code range of every expression (indexes, then conditions)
    for (int d = 0; d < n_indexes; d++) {
        Affine a;
        seg_begin.push_back(C.code.size());
        if (!C.compile_one(indexes[d], &a)) { *err = C.err; return false; }
        seg_end.push_back(C.code.size());
        if (d == 0 && !C.direct_candidate) direct = false;
        C.emit(IX_STORE_XID, d);
        if (a.ok) { P->c0[d] = a.c; for (int j = 0; j < kMaxDims; j++) P->coef[d][j] = a.coef[j]; }
        else affine = false;
    }
    for (int k = 0; k < n_conds; k++) {
        Affine a;
        seg_begin.push_back(C.code.size());
        if (!C.compile_one(conds[k], &a)) { *err = C.err; return false; }
        seg_end.push_back(C.code.size());
        C.emit(IX_STORE_COND);
    }
    if (C.max_depth > kIxStack) { *err = "index expression too deep"; return false; }
    if ((int)C.code.size() > kMaxCode) { *err = "index expressions too long"; return false; }
    P->n_code = (int)C.code.size();
    for (int i = 0; i < P->n_code; i++) P->code[i] = C.code[i];
    P->is_affine = affine && !C.used_extra;
    if (direct) {
        const b200jt_tensor& e = extras[0];
        direct = e.ndim == ndim_loop;
        for (int d = 0; direct && d < ndim_loop; d++) direct = e.shape[d] == loop_shape[d];
    }
    P->is_direct_extra = direct;
    // inner run: count, per loop variable, the expressions that read it
    {
        std::vector<int> readers(kMaxDims, 0);
        auto reads = [&](size_t e, int j) {
            for (size_t pc = seg_begin[e]; pc < seg_end[e]; pc++) {
                const int op = C.code[pc] & 0xff;
                if (op == IX_CONST64) { pc += 2; continue; }
                if (op == IX_LOOPVAR && (C.code[pc] >> 8) == j) return true;
            }
            return false;
        };
        for (size_t e = 0; e < seg_begin.size(); e++)
            for (int j = 0; j < ndim_loop; j++) if (reads(e, j)) readers[j]++;
        int k = 0; int64_t run = 1;
        while (k < ndim_loop && k < ndim_x) {
            const int j = ndim_loop - 1 - k, d = ndim_x - 1 - k;
            const bool identity = seg_end[d] - seg_begin[d] == 1 && (C.code[seg_begin[d]] & 0xff) == IX_LOOPVAR &&
                                  (C.code[seg_begin[d]] >> 8) == j;
            if (!identity || readers[j] != 1 || loop_shape[j] != x_shape[d]) break;
            run *= loop_shape[j];
            k++;
        }
        P->inner_dims = k;
        P->inner_elems = run;
    }
    return true;
}

}  // namespace b200jt

extern "C" int b200jt_index_affine(const int64_t* loop_shape, int ndim_loop, const int64_t* x_shape, int ndim_x,
                                   const char* const* indexes, int n_indexes, int64_t* coef, int64_t* c0) {
    using namespace b200jt;
    B200JT_CHECK_ARG(ndim_loop >= 1 && ndim_loop <= kMaxDims && ndim_x >= 1 && ndim_x <= kMaxDims && n_indexes == ndim_x,
                     "bad ranks");
    IndexProgram P;
    std::string err;
    if (!compile_index_program(loop_shape, ndim_loop, x_shape, ndim_x, indexes, n_indexes, nullptr, 0, nullptr, 0, &P, &err))
        return fail(-2, "b200jt_index_affine: " + err);
    if (!P.is_affine) return 0;
    for (int d = 0; d < ndim_x; d++) {
        c0[d] = P.c0[d];
        for (int j = 0; j < kMaxDims; j++) coef[d * kMaxDims + j] = P.coef[d][j];
    }
    return 1;
}
