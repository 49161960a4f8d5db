// Affine reindex (gathers whose every index is an affine function of the output coordinates: padding, windows of a
// convolution, slices, shifts, broadcasts) as a kernel compiled for ONE op instance: shapes, coefficients and offsets are
// literals, so the split of the flat output index is divisions by constants, zero coefficients vanish, range checks are
// emitted only for the axes that can actually leave the tensor, and the step from one element of a 16-byte output vector
// to the next is an odometer over constants. This is what the reference gets from compiling its reindex op with the
// index expressions pasted into the loop nest (python/jittor/src/ops/reindex_op.cc:93-109). The ahead-of-time kernels
// of reindex.cu do the same work with the shapes and coefficients as run-time arguments and are several times slower on
// high-rank windows (the [4,32,32,32] -> [4,64,32,32,32,3,3] conv window: 7 divisions and 28 multiply-adds per element).
//
// A shape-specialised kernel costs a compilation (~0.1 s), so an op instance is compiled when it is seen for the second
// time and has at least 2^16 outputs; until then, and without NVRTC, the ahead-of-time kernels run.
// B200JT_REINDEX_JIT = 0: never, 1 (default): as described, 2: compile at first sight and fail loudly.
#include "jit.cuh"
#include "reindex_jit.cuh"

#include <mutex>
#include <unordered_map>

namespace b200jt {
namespace {

std::string num(long long v) { return std::to_string(v); }

// elem: bytes per element (1, 2, 4, 8); vec: elements per 16-byte (8-byte for 1-byte elements) output vector, or 1
std::string make_source(const ReindexAffine& A, int elem, int vec) {
    const int nl = A.ndim_loop, nx = A.ndim_x;
    const char* T = elem == 1 ? "unsigned char" : elem == 2 ? "unsigned short" : elem == 4 ? "unsigned int" : "unsigned long long";
    const char* VT = vec * elem == 16 ? "uint4" : vec * elem == 8 ? "uint2" : vec * elem == 4 ? "unsigned int" : vec * elem == 2 ? "unsigned short" : nullptr;
    long long n = 1;
    for (int j = 0; j < nl; j++) n *= A.loop_shape[j];
    std::string s;
    s += "typedef " + std::string(T) + " T;\n";
    s += "extern \"C\" __global__ void __launch_bounds__(256) reindex_jit_kernel(const T* __restrict__ x, T* __restrict__ y, T fill) {\n";
    s += "    const unsigned n_vec = " + num(n / vec) + "u;\n";
    s += "    for (unsigned v = blockIdx.x * 256u + threadIdx.x; v < n_vec; v += gridDim.x * 256u) {\n";
    s += "        unsigned r = v * " + num(vec) + "u;\n";
    // loop coordinates, innermost first (axes of extent 1 are constant 0)
    for (int j = nl - 1; j >= 0; j--) {
        if (A.loop_shape[j] == 1) { s += "        int i" + num(j) + " = 0;\n"; continue; }
        if (j == 0) s += "        int i0 = (int)r;\n";
        else s += "        int i" + num(j) + " = (int)(r % " + num(A.loop_shape[j]) + "u); r /= " + num(A.loop_shape[j]) + "u;\n";
    }
    // source coordinates; which of them can leave [0, extent)
    bool check[kMaxDims] = {};
    for (int d = 0; d < nx; d++) {
        long long lo = A.c0[d], hi = A.c0[d];
        std::string e = num(A.c0[d]);
        for (int j = 0; j < nl; j++) {
            const long long c = A.coef[d][j];
            if (c == 0 || A.loop_shape[j] == 1) continue;
            e += " + " + num(c) + " * i" + num(j);
            const long long span = c * (A.loop_shape[j] - 1);
            if (span < 0) lo += span; else hi += span;
        }
        check[d] = lo < 0 || hi >= A.x_shape[d];
        s += "        int a" + num(d) + " = " + e + ";\n";
    }
    if (vec > 1) s += "        __align__(16) T out[" + num(vec) + "];\n";
    s += "#pragma unroll\n        for (int e = 0; e < " + num(vec) + "; e++) {\n";
    std::string over, off;
    for (int d = 0; d < nx; d++) {
        if (check[d]) over += (over.empty() ? "" : " | ") + std::string("((unsigned)a") + num(d) + " >= " + num(A.x_shape[d]) + "u)";
        off = d == 0 ? "a0" : "(" + off + ") * " + num(A.x_shape[d]) + " + a" + num(d);
    }
    const std::string dst = vec > 1 ? "out[e]" : "y[v]";
    if (over.empty()) s += "            " + dst + " = __ldg(x + (" + off + "));\n";
    else s += "            " + dst + " = (" + over + ") ? fill : __ldg(x + (" + off + "));\n";
    if (vec > 1) {
        // odometer step to the next output element: the innermost axis advances, carries ripple outwards; a vector never
        // crosses the end of the tensor, so the carry chain needs no terminator
        s += "            if (e + 1 < " + num(vec) + ") {\n";
        std::string ind = "                ";
        int open = 0;
        for (int j = nl - 1; j >= 0; j--) {
            if (A.loop_shape[j] == 1) continue;
            s += ind + "i" + num(j) + "++;";
            for (int d = 0; d < nx; d++)
                if (A.coef[d][j] != 0) s += " a" + num(d) + " += " + num(A.coef[d][j]) + ";";
            s += "\n";
            // a vector of `vec` elements that divides the innermost extent never carries
            if (j == nl - 1 && A.loop_shape[j] % vec == 0) break;
            bool outer = false;
            for (int q = j - 1; q >= 0; q--) outer |= A.loop_shape[q] != 1;
            if (!outer) break;
            s += ind + "if (i" + num(j) + " == " + num(A.loop_shape[j]) + ") {\n";
            open++;
            ind += "    ";
            s += ind + "i" + num(j) + " = 0;";
            for (int d = 0; d < nx; d++)
                if (A.coef[d][j] != 0) s += " a" + num(d) + " -= " + num(A.coef[d][j] * A.loop_shape[j]) + ";";
            s += "\n";
        }
        for (; open > 0; open--) { ind.resize(ind.size() - 4); s += ind + "}\n"; }
        s += "            }\n";
    }
    s += "        }\n";
    if (vec > 1) s += "        *reinterpret_cast<" + std::string(VT) + "*>(y + (size_t)v * " + num(vec) + ") = *reinterpret_cast<" + std::string(VT) + "*>(out);\n";
    s += "    }\n}\n";
    return s;
}

// Ragged trailing axes (a 3x3 window at the end of a conv-window reindex): a thread takes a TILE of consecutive outputs
// that covers the small trailing axes completely plus k steps of the axis before them, chosen so that the tile is a whole
// number of 16-byte vectors. Inside the tile every trailing coordinate is a literal, so the code is straight-line: one
// decomposition per tile, loads of the same source element are merged by the compiler (a 3x3 window moved over 4 columns
// reads 18 elements for 36 outputs). The tiles of a warp go through shared memory and leave as coalesced 16-byte
// stores. Returns "" when no such tile exists.
bool pick_tile(const ReindexAffine& A, int elem, int vec, int* j0_out, int* k_out, int* tile_out) {
    const int nl = A.ndim_loop;
    if (vec <= 1) return false;
    const int cap = elem == 8 ? 23 : 47;               // 256 threads x (tile + 1) elements of staging stay below 48 KB
    long long inner = 1;
    int j0 = nl - 1;                                   // first axis that is only partly inside the tile
    while (j0 >= 0 && inner * A.loop_shape[j0] <= cap / 2) { inner *= A.loop_shape[j0]; j0--; }
    if (j0 == nl - 1 || j0 < 0) return false;          // the innermost axis alone is long: the vector form has no carries to lose
    int k = 0;
    for (int c = 1; c * inner <= cap; c++)
        if (A.loop_shape[j0] % c == 0 && (c * inner) % vec == 0) { k = c; break; }
    if (k == 0) return false;
    *j0_out = j0; *k_out = k; *tile_out = (int)(k * inner);
    return true;
}

std::string make_source_tiled(const ReindexAffine& A, int elem, int vec) {
    const int nl = A.ndim_loop, nx = A.ndim_x;
    int j0 = 0, k = 0, tile = 0;
    if (!pick_tile(A, elem, vec, &j0, &k, &tile)) return "";
    long long n = 1;
    for (int j = 0; j < nl; j++) n *= A.loop_shape[j];
    const char* T = elem == 1 ? "unsigned char" : elem == 2 ? "unsigned short" : elem == 4 ? "unsigned int" : "unsigned long long";
    const char* VT = vec * elem == 16 ? "uint4" : "uint2";
    std::string s;
    s += "typedef " + std::string(T) + " T;\n";
    s += "extern \"C\" __global__ void __launch_bounds__(256) reindex_jit_kernel(const T* __restrict__ x, T* __restrict__ y, T fill) {\n";
    s += "    const unsigned n_tiles = " + num(n / tile) + "u;\n";
    s += "    constexpr unsigned TILE = " + num(tile) + ", PITCH = TILE + 1, VEC = " + num(vec) + ";\n";
    s += "    __shared__ T stage[8][32 * PITCH];\n";
    s += "    const unsigned lane = threadIdx.x & 31u, w = threadIdx.x >> 5;\n";
    s += "    T* mine = &stage[w][lane * PITCH];\n";
    s += "    for (unsigned t0 = (blockIdx.x * 8u + w) * 32u; t0 < n_tiles; t0 += gridDim.x * 256u) {\n";
    s += "        const unsigned t = t0 + lane;\n";
    s += "        if (t < n_tiles) {\n";
    s += "        unsigned r = t;\n";
    // outer coordinates; axis j0 advances k per tile
    const long long steps = A.loop_shape[j0] / k;
    if (j0 == 0) s += "        const int i0 = (int)r * " + num(k) + ";\n";
    else s += "        const int i" + num(j0) + " = (int)(r % " + num(steps) + "u) * " + num(k) + "; r /= " + num(steps) + "u;\n";
    for (int j = j0 - 1; j >= 0; j--) {
        if (A.loop_shape[j] == 1) { s += "        const int i" + num(j) + " = 0;\n"; continue; }
        if (j == 0) s += "        const int i0 = (int)r;\n";
        else s += "        const int i" + num(j) + " = (int)(r % " + num(A.loop_shape[j]) + "u); r /= " + num(A.loop_shape[j]) + "u;\n";
    }
    // source coordinates of the tile's first element, and which of them can leave the tensor
    bool check[kMaxDims] = {};
    long long xstride[kMaxDims];
    { long long st = 1; for (int d = nx - 1; d >= 0; d--) { xstride[d] = st; st *= A.x_shape[d]; } }
    std::string base_off;
    for (int d = 0; d < nx; d++) {
        long long lo = A.c0[d], hi = A.c0[d];
        std::string e = num(A.c0[d]);
        for (int j = 0; j < nl; j++) {
            const long long c = A.coef[d][j];
            if (c == 0 || A.loop_shape[j] == 1) continue;
            if (j <= j0) e += " + " + num(c) + " * i" + num(j);
            const long long span = c * (A.loop_shape[j] - 1);
            if (span < 0) lo += span; else hi += span;
        }
        check[d] = lo < 0 || hi >= A.x_shape[d];
        s += "        const int a" + num(d) + " = " + e + ";\n";
        base_off += (d ? " + " : "") + std::string("a") + num(d) + " * " + num(xstride[d]);
    }
    s += "        const T* xb = x + (" + base_off + ");\n";
    for (int e = 0; e < tile; e++) {
        // literal coordinates of element e inside the tile: trailing axes j0+1.., then the step of axis j0
        long long rem = e;
        long long lit[kMaxDims] = {};
        for (int j = nl - 1; j > j0; j--) { lit[j] = rem % A.loop_shape[j]; rem /= A.loop_shape[j]; }
        lit[j0] = rem;
        long long off = 0;
        std::string over;
        for (int d = 0; d < nx; d++) {
            long long cd = 0;
            for (int j = j0; j < nl; j++) cd += A.coef[d][j] * lit[j];
            off += cd * xstride[d];
            if (check[d]) over += (over.empty() ? "" : " | ") + std::string("((unsigned)(a") + num(d) + " + " + num(cd) + ") >= " + num(A.x_shape[d]) + "u)";
        }
        if (over.empty()) s += "        mine[" + num(e) + "] = __ldg(xb + " + num(off) + ");\n";
        else s += "        mine[" + num(e) + "] = (" + over + ") ? fill : __ldg(xb + " + num(off) + ");\n";
    }
    // the warp's 32 tiles are consecutive in y: written out together, 16 bytes per lane and instruction, fully coalesced
    // (a thread storing its own 36 elements would touch 9 different 128-byte lines per instruction across the warp)
    s += "        }\n        __syncwarp();\n";
    s += "        const unsigned total = (n_tiles - t0 < 32u ? n_tiles - t0 : 32u) * TILE;\n";
    s += "        T* dst = y + (size_t)t0 * TILE;\n";
    s += "        for (unsigned q = lane * VEC; q < total; q += 32u * VEC) {\n";
    s += "            __align__(16) T v[VEC];\n";
    s += "#pragma unroll\n            for (unsigned c = 0; c < VEC; c++) { const unsigned L = q + c; v[c] = stage[w][(L / TILE) * PITCH + (L % TILE)]; }\n";
    s += "            *reinterpret_cast<" + std::string(VT) + "*>(dst + q) = *reinterpret_cast<" + std::string(VT) + "*>(v);\n";
    s += "        }\n        __syncwarp();\n";
    s += "    }\n}\n";
    return s;
}

// Outputs one thread produces, and the source for an op instance.
int outputs_per_thread(const ReindexAffine& A, int elem, int vec) {
    int j0, k, tile;
    return pick_tile(A, elem, vec, &j0, &k, &tile) ? tile : vec;
}
std::string pick_source(const ReindexAffine& A, int elem, int vec) {
    const std::string s = make_source_tiled(A, elem, vec);
    return s.empty() ? make_source(A, elem, vec) : s;
}

std::string make_key(const ReindexAffine& A, int elem, int vec) {
    std::string k = "reindex:";
    const int32_t head[4] = {elem, vec, A.ndim_loop, A.ndim_x};
    k.append((const char*)head, sizeof head);
    k.append((const char*)A.loop_shape, sizeof(int64_t) * A.ndim_loop);
    k.append((const char*)A.x_shape, sizeof(int64_t) * A.ndim_x);
    k.append((const char*)A.c0, sizeof(int64_t) * A.ndim_x);
    for (int d = 0; d < A.ndim_x; d++) k.append((const char*)A.coef[d], sizeof(int64_t) * A.ndim_loop);
    return k;
}

std::mutex g_seen_mu;
std::unordered_map<std::string, int> g_seen;

thread_local ReindexDryRun* t_dry = nullptr;

}  // namespace

void reindex_jit_dry_run(ReindexDryRun* d) { t_dry = d; }
bool reindex_jit_dry_running() { return t_dry != nullptr; }

int reindex_jit_launch(const ReindexAffine& A, int elem, int vec, const void* x, void* y, uint64_t fill_bits, cudaStream_t st) {
    if (t_dry) {
        t_dry->source = pick_source(A, elem, vec);
        t_dry->compiled = jit::compile_only(t_dry->source, &t_dry->log);
        return 0;
    }
    const char* env = getenv("B200JT_REINDEX_JIT");
    const int mode = env ? atoi(env) : 1;
    if (mode == 0) return kReindexJitUnavailable;
    long long n = 1;
    for (int j = 0; j < A.ndim_loop; j++) n *= A.loop_shape[j];
    if (mode == 1 && n < (1 << 16)) return kReindexJitUnavailable;
    std::string why;
    if (!jit::available(&why)) return mode == 2 ? fail(-1, "b200jt_reindex: run-time compiler unavailable: " + why) : kReindexJitUnavailable;
    const std::string key = make_key(A, elem, vec);
    if (mode == 1) {
        std::lock_guard<std::mutex> lock(g_seen_mu);
        if (++g_seen[key] < 2) return kReindexJitUnavailable;         // first sight: not worth a compilation yet
    }
    std::string log;
    const cudaKernel_t kernel = jit::get_kernel(key, [&] { return pick_source(A, elem, vec); }, "reindex_jit_kernel", &log);
    if (!kernel) return mode == 2 ? fail(-1, "b200jt_reindex: compiling the reindex failed: " + log) : kReindexJitUnavailable;
    void* args[] = {(void*)&x, (void*)&y, (void*)&fill_bits};
    B200JT_CUDA(cudaLaunchKernel((const void*)kernel, dim3(grid_for(n / outputs_per_thread(A, elem, vec), 256)), dim3(256), args, 0, st));
    return 0;
}

}  // namespace b200jt
