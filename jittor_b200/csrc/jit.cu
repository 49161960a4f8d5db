// NVRTC through dlopen and the per-process kernel cache (see jit.cuh).
#include "jit.cuh"

#include <dlfcn.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace b200jt {
namespace jit {
namespace {

struct Nvrtc {
    typedef struct _nvrtcProgram* Prog;
    int (*create)(Prog*, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
    int (*compile)(Prog, int, const char* const*) = nullptr;
    int (*cubin_size)(Prog, size_t*) = nullptr;
    int (*cubin)(Prog, char*) = nullptr;
    int (*log_size)(Prog, size_t*) = nullptr;
    int (*log)(Prog, char*) = nullptr;
    int (*destroy)(Prog*) = nullptr;
    int (*version)(int*, int*) = nullptr;
    bool ok = false;
    std::string why;
};

const Nvrtc& nvrtc() {
    static Nvrtc N = [] {
        Nvrtc n;
        void* h = nullptr;
        for (const char* name : {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12"}) {
            h = dlopen(name, RTLD_NOW | RTLD_LOCAL);
            if (h) break;
        }
        if (!h) { n.why = "libnvrtc.so.12 not found"; return n; }
        auto sym = [&](const char* s) { void* p = dlsym(h, s); if (!p) n.why = std::string("missing symbol ") + s; return p; };
        n.create = (decltype(n.create))sym("nvrtcCreateProgram");
        n.compile = (decltype(n.compile))sym("nvrtcCompileProgram");
        n.cubin_size = (decltype(n.cubin_size))sym("nvrtcGetCUBINSize");
        n.cubin = (decltype(n.cubin))sym("nvrtcGetCUBIN");
        n.log_size = (decltype(n.log_size))sym("nvrtcGetProgramLogSize");
        n.log = (decltype(n.log))sym("nvrtcGetProgramLog");
        n.destroy = (decltype(n.destroy))sym("nvrtcDestroyProgram");
        n.version = (decltype(n.version))sym("nvrtcVersion");
        n.ok = n.why.empty();
        return n;
    }();
    return N;
}

struct Compiled { cudaLibrary_t lib = nullptr; cudaKernel_t kernel = nullptr; std::string log; };

std::mutex g_mu;
std::unordered_map<std::string, Compiled> g_cache;
std::atomic<int> g_compiled{0}, g_hits{0}, g_failed{0};

bool compile_cubin(const std::string& src, std::vector<char>& cubin, std::string& log) {
    const Nvrtc& N = nvrtc();
    if (!N.ok) { log = N.why; return false; }
    Nvrtc::Prog prog = nullptr;
    if (N.create(&prog, src.c_str(), "b200jt_jit.cu", 0, nullptr, nullptr) != 0) { log = "nvrtcCreateProgram failed"; return false; }
    const char* opts[] = {"--gpu-architecture=sm_100a", "-std=c++17", "-lineinfo"};
    const int rc = N.compile(prog, 3, opts);
    size_t ls = 0;
    if (N.log_size(prog, &ls) == 0 && ls > 1) { log.resize(ls); N.log(prog, &log[0]); }
    if (rc != 0) { N.destroy(&prog); return false; }
    size_t cs = 0;
    if (N.cubin_size(prog, &cs) != 0 || cs == 0) { N.destroy(&prog); log += " (no cubin)"; return false; }
    cubin.resize(cs);
    N.cubin(prog, cubin.data());
    N.destroy(&prog);
    return true;
}

// ---- cubins on disk ----------------------------------------------------------------------------------------------
// Compiled kernels are kept under $B200JT_CACHE_DIR (default ~/.cache/b200jt; empty or "0" switches the disk cache off),
// one file per source, named by a hash of the source text, the compiler's version and the target -- what the reference's
// ~/.cache/jittor does for its generated ops. A file is written under a temporary name and renamed, so concurrent
// processes never read a partial cubin; a file that fails to load is ignored and overwritten.
std::string cache_dir() {
    static const std::string dir = [] {
        const char* e = getenv("B200JT_CACHE_DIR");
        std::string d;
        if (e) { d = e; if (d.empty() || d == "0") return std::string(); }
        else {
            const char* home = getenv("HOME");
            if (!home || !*home) return std::string();
            d = std::string(home) + "/.cache";
            mkdir(d.c_str(), 0755);
            d += "/b200jt";
        }
        mkdir(d.c_str(), 0755);
        struct stat st;
        return (stat(d.c_str(), &st) == 0 && S_ISDIR(st.st_mode)) ? d : std::string();
    }();
    return dir;
}

std::string cache_file(const std::string& src) {
    const std::string dir = cache_dir();
    if (dir.empty()) return std::string();
    uint64_t h1 = 1469598103934665603ull, h2 = 0x9e3779b97f4a7c15ull;         // two independent 64-bit FNV-style hashes
    auto mix = [&](const std::string& t) {
        for (unsigned char c : t) { h1 = (h1 ^ c) * 1099511628211ull; h2 = (h2 + c) * 0x100000001b3ull ^ (h2 >> 29); }
    };
    int major = 0, minor = 0;
    if (nvrtc().ok && nvrtc().version) nvrtc().version(&major, &minor);
    mix(src); mix("|sm_100a|nvrtc" + std::to_string(major) + "." + std::to_string(minor));
    char name[64];
    snprintf(name, sizeof name, "/%016llx%016llx.cubin", (unsigned long long)h1, (unsigned long long)h2);
    return dir + name;
}

bool read_file(const std::string& path, std::vector<char>& out) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return false;
    fseek(f, 0, SEEK_END);
    const long n = ftell(f);
    fseek(f, 0, SEEK_SET);
    bool ok = n > 0;
    if (ok) { out.resize((size_t)n); ok = fread(out.data(), 1, (size_t)n, f) == (size_t)n; }
    fclose(f);
    return ok;
}

void write_file(const std::string& path, const std::vector<char>& data) {
    const std::string tmp = path + "." + std::to_string((long long)getpid()) + ".tmp";
    FILE* f = fopen(tmp.c_str(), "wb");
    if (!f) return;
    const bool ok = fwrite(data.data(), 1, data.size(), f) == data.size();
    fclose(f);
    if (!ok || rename(tmp.c_str(), path.c_str()) != 0) unlink(tmp.c_str());
}

std::atomic<int> g_disk_hits{0};

}  // namespace

bool available(std::string* why) {
    const Nvrtc& N = nvrtc();
    if (!N.ok && why) *why = N.why;
    return N.ok;
}

bool compile_only(const std::string& src, std::string* log) {
    std::vector<char> cubin;
    std::string l;
    const bool ok = compile_cubin(src, cubin, l);
    if (log) *log = l;
    return ok;
}

cudaKernel_t get_kernel(const std::string& key, const std::function<std::string()>& make_source, const char* entry, std::string* log) {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_cache.find(key);
    if (it != g_cache.end()) {
        g_hits++;
        if (!it->second.kernel && log) *log = it->second.log;
        return it->second.kernel;
    }
    Compiled c;
    std::vector<char> cubin;
    const std::string src = make_source();
    const std::string file = cache_file(src);
    auto load = [&]() {
        cudaError_t e = cudaLibraryLoadData(&c.lib, cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
        if (e == cudaSuccess) e = cudaLibraryGetKernel(&c.kernel, c.lib, entry);
        if (e != cudaSuccess) { c.log += std::string(" loading the compiled kernel: ") + cudaGetErrorString(e); (void)cudaGetLastError(); c.kernel = nullptr; }
        return c.kernel != nullptr;
    };
    if (!file.empty() && read_file(file, cubin) && load()) g_disk_hits++;
    else {
        c = Compiled();
        if (compile_cubin(src, cubin, c.log) && load() && !file.empty()) write_file(file, cubin);
    }
    if (c.kernel) g_compiled++; else { g_failed++; if (log) *log = c.log; }
    g_cache.emplace(key, c);
    return c.kernel;
}

void stats(int* compiled, int* hits, int* failed) {
    if (compiled) *compiled = g_compiled.load();
    if (hits) *hits = g_hits.load();
    if (failed) *failed = g_failed.load();
}

}  // namespace jit
}  // namespace b200jt
