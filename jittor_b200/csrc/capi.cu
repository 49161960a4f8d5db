// Error plumbing, dtype/op name tables and version query of the C ABI.
#include "common.cuh"

#include <atomic>

namespace b200jt {

static thread_local std::string g_last_error;

void set_error(const std::string& msg) { g_last_error = msg; }
int fail(int code, const std::string& msg) { g_last_error = msg; return code; }

static const char* kDtypeNames[] = {"bool", "int8", "int16", "int32", "int64", "uint8",
                                    "float16", "bfloat16", "float32", "float64"};

const char* dtype_name(int dt) { return dt >= 0 && dt <= B200JT_FLOAT64 ? kDtypeNames[dt] : "?"; }
int dtype_from_name(const char* name) {
    for (int i = 0; i <= B200JT_FLOAT64; i++) if (strcmp(name, kDtypeNames[i]) == 0) return i;
    return -1;
}

std::string shape_str(const b200jt_tensor* t) {
    std::string s = "[";
    for (int i = 0; i < t->ndim; i++) s += std::to_string(t->shape[i]) + ",";
    return s + "]";
}

OpCode binary_op_from_name(const char* n) {
    static const struct { const char* name; OpCode code; } tab[] = {
        {"add", OP_ADD}, {"subtract", OP_SUB}, {"multiply", OP_MUL}, {"divide", OP_DIV}, {"floor_divide", OP_FLOORDIV},
        {"mod", OP_MOD}, {"pow", OP_POW}, {"maximum", OP_MAX}, {"minimum", OP_MIN}, {"less", OP_LT}, {"less_equal", OP_LE},
        {"greater", OP_GT}, {"greater_equal", OP_GE}, {"equal", OP_EQ}, {"not_equal", OP_NE}, {"logical_and", OP_LAND},
        {"logical_or", OP_LOR}, {"logical_xor", OP_LXOR}, {"bitwise_and", OP_BAND}, {"bitwise_or", OP_BOR},
        {"bitwise_xor", OP_BXOR}, {"left_shift", OP_SHL}, {"right_shift", OP_SHR}, {"mean", OP_MEAN}, {"void", OP_VOID}};
    for (auto& e : tab) if (strcmp(e.name, n) == 0) return e.code;
    return OP_INVALID;
}

static std::atomic<int> g_sm_reserve{0};
int sm_reserve() { return g_sm_reserve.load(std::memory_order_relaxed); }

}  // namespace b200jt

extern "C" int b200jt_set_sm_reserve(int sms) {
    B200JT_CHECK_ARG(sms >= 0 && sms <= 64, "sms must be 0..64");
    b200jt::g_sm_reserve.store(sms);
    return 0;
}

extern "C" const char* b200jt_last_error(void) { return b200jt::g_last_error.c_str(); }
extern "C" int b200jt_version(void) { return 100; }
