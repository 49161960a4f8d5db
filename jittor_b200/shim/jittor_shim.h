// The slice of the reference's core headers (op.h, var.h, misc/nano_string.h, misc/nano_vector.h, jit_key.h) that a
// custom op written in the documented form needs (python/jittor/test/test_custom_op.py:12-58): a `struct XxxOp : Op`
// with `Var*` members, a constructor that calls create_output, jit_prepare with add_jit_define, and a jit_run that reads
// shapes and raw pointers. compile_custom_ops builds user sources against this header instead of the reference's core.
#pragma once
#include <cstdint>
#include <cstring>
#include <initializer_list>
#include <string>
#include <vector>

namespace jittor {

typedef int8_t int8; typedef int16_t int16; typedef int32_t int32; typedef int64_t int64;
typedef uint8_t uint8; typedef uint16_t uint16; typedef uint32_t uint32; typedef uint64_t uint64;
typedef float float32; typedef double float64; typedef uint32_t uint;
#ifndef index_t
typedef int32_t index_t;
#endif
using std::string; using std::vector;

// dtype / op names (python/jittor/src/misc/nano_string.h)
struct NanoString {
    int id;
    constexpr NanoString(int i = 0) : id(i) {}
    NanoString(const char* s) : id(0) { for (int i = 0; i < count(); i++) if (!strcmp(s, names()[i])) id = i; }
    NanoString(const std::string& s) : NanoString(s.c_str()) {}
    static int count() { return 11; }
    static const char* const* names() {
        static const char* n[] = {"void", "bool", "int8", "int16", "int32", "int64", "uint8", "float16", "bfloat16", "float32", "float64"};
        return n;
    }
    const char* to_cstring() const { return names()[id]; }
    int dsize() const { static const int s[] = {0, 1, 1, 2, 4, 8, 1, 2, 2, 4, 8}; return s[id]; }
    bool is_float() const { return id >= 7; }
    bool is_int() const { return id >= 2 && id <= 6; }
    bool operator==(const NanoString& o) const { return id == o.id; }
    bool operator!=(const NanoString& o) const { return id != o.id; }
};
constexpr NanoString ns_void(0), ns_bool(1), ns_int8(2), ns_int16(3), ns_int32(4), ns_int64(5), ns_uint8(6), ns_float16(7),
    ns_bfloat16(8), ns_float32(9), ns_float64(10);

// shapes (python/jittor/src/misc/nano_vector.h: at most 10 dims)
struct NanoVector {
    int64 v[10]; int n;
    NanoVector() : n(0) {}
    NanoVector(std::initializer_list<int64> l) : n(0) { for (int64 x : l) push_back(x); }
    void push_back(int64 x) { if (n < 10) v[n++] = x; }
    int size() const { return n; }
    int64 operator[](int i) const { return v[i < 0 ? i + n : i]; }
    int64 at(int i) const { return (*this)[i]; }
    int64 back() const { return v[n - 1]; }
    const int64* begin() const { return v; }
    const int64* end() const { return v + n; }
    bool operator==(const NanoVector& o) const { if (n != o.n) return false; for (int i = 0; i < n; i++) if (v[i] != o.v[i]) return false; return true; }
};

struct Var {
    void* mem_ptr = nullptr;
    NanoVector shape;
    NanoString dtype_;
    int64 num = 0, size = 0;
    NanoString dtype() const { return dtype_; }
    template <class T> T* ptr() const { return (T*)mem_ptr; }
    int64 numel() const { return num; }
    void set_shape(NanoVector s) { shape = s; num = 1; for (int64 d : s) num *= d; size = num * dtype_.dsize(); }
};

// jit key: the defines jit_prepare adds become -D options of the JIT compilation (python/jittor/src/jit_key.h:285-325)
struct JK { std::string defines; };
inline void add_jit_define(JK& jk, const std::string& key, NanoString val) { jk.defines += key + "=" + val.to_cstring() + ";"; }
inline void add_jit_define(JK& jk, const std::string& key, const std::string& val) { jk.defines += key + "=" + val + ";"; }
inline void add_jit_define(JK& jk, const std::string& key, const char* val) { jk.defines += key + "=" + val + ";"; }
inline void add_jit_define(JK& jk, const std::string& key, long long val) { jk.defines += key + "=" + std::to_string(val) + ";"; }
inline void add_jit_define(JK& jk, const std::string& key, int val) { jk.defines += key + "=" + std::to_string(val) + ";"; }
inline void add_jit_define(JK& jk, const std::string& key, long val) { jk.defines += key + "=" + std::to_string(val) + ";"; }
inline void add_jit_define(JK& jk, const std::string& key, bool val) { jk.defines += key + "=" + (val ? "1" : "0") + ";"; }
template <class I, class V> inline void add_jit_define(JK& jk, const std::string& key, const I& i, const V& val) { add_jit_define(jk, key + std::to_string(i), val); }

struct NodeFlags { enum Flags { _cpu = 1, _cuda = 2, _forwarded = 4 }; int bits = 0; void set(int f, int v = 1) { if (v) bits |= f; else bits &= ~f; } bool get(int f) const { return bits & f; } };
enum OpType { other = 0, element = 1, broadcast = 2, reduce = 3 };

struct Op {
    std::vector<Var*> inputs_, outputs_;
    NodeFlags flags;
    virtual ~Op() { for (Var* v : outputs_) delete v; }
    Var* create_output(NanoVector shape, NanoString dtype) {
        Var* v = new Var();
        v->dtype_ = dtype; v->set_shape(shape);
        outputs_.push_back(v);
        return v;
    }
    void set_type(OpType) {}
    virtual void infer_shape() {}
    virtual void jit_prepare(JK&) {}
    virtual void jit_run() {}
    virtual const char* name() const = 0;
    const std::vector<Var*>& inputs() const { return inputs_; }
    const std::vector<Var*>& outputs() const { return outputs_; }
};

// Outside the JIT compilation the op declares jit_prepare (and gets an empty jit_run); inside it declares jit_run, the
// same split as python/jittor/src/op.h:67-71.
#define DECLARE_jit_run void jit_prepare(JK& jk) override; void jit_run() override;

#define CHECK(cond) if (!(cond)) throw std::runtime_error(std::string("Check failed: ") + #cond)
#define ASSERT(cond) CHECK(cond)

}  // namespace jittor
#include <stdexcept>
