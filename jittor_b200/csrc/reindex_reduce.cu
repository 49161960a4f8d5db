// reindex_reduce: x[:] = init(op); for every element i of y, unless it overflows: x[index(i)] = op(x[index(i)], y[i]).
//
// Paths, chosen on the host from the compiled index program:
//   injective  -- affine index map that never sends two y elements to one x element (e.g. the 2x2 pool
//                 backward): plain stores after the init fill, no atomics.
//   privatised -- one indexed dim addressed through @e0(i0..in) ("scatter") and few bins: every CTA
//                 accumulates into replicated shared-memory bins (replicas spread same-address
//                 conflicts of skewed inputs over banks), writes one partial row to a workspace and a
//                 second kernel folds the rows in fixed order -- deterministic for floating point.
//   direct     -- same scatter form, many bins: 128-bit loads of values and indices, one red.global per
//                 element (the bins live in L2).
//   generic    -- bytecode-interpreted index, one atomic per element.
#include "atomic_ops.cuh"

#include <type_traits>
#include "index_program.cuh"

#include <algorithm>

namespace b200jt {

constexpr int kPrivThreads = 1024;
constexpr int kPrivMaxSmemBytes = 160 * 1024;
constexpr int64_t kPrivMaxBinBytes = 32 * 1024;     // bins*sizeof(T) up to which the privatised path is used
constexpr int kPrivGrid = kNumSMs;                  // one CTA per SM (dynamic smem limits residency to 1)

template <typename T>
__global__ void __launch_bounds__(256) fill_kernel(T* __restrict__ x, int64_t n, T v) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        x[i] = v;
}

template <typename T, typename I>
__global__ void __launch_bounds__(256)
rr_generic_kernel(const T* __restrict__ y, T* __restrict__ x, const __grid_constant__ IndexProgram P,
                  int64_t n, int op) {
    const int nl = P.ndim_loop, nx = P.ndim_x;
    for (int64_t flat = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; flat < n;
         flat += (int64_t)gridDim.x * blockDim.x) {
        I iv[kMaxDims];
        int64_t r = flat;
#pragma unroll 1
        for (int d = nl - 1; d >= 0; d--) { int64_t s = P.loop_shape[d]; iv[d] = (I)(r % s); r /= s; }
        I xid[kMaxDims];
        if (eval_index_program<I>(P, iv, xid)) continue;
        int64_t off = 0;
        for (int d = 0; d < nx; d++) off = off * P.x_shape[d] + (int64_t)xid[d];
        atomic_apply<T>(x + off, y[flat], op);
    }
}

// Row form of the generic kernel: the program is evaluated once per run of `inner` consecutive y elements, which land
// on `inner` consecutive x elements (x[idx[i], :] op= y[i, :]). A warp takes 32 runs at a time: every lane interprets
// the program for one of them, the offsets go round by shuffle and the whole warp applies each run.
template <typename T, typename I>
__global__ void __launch_bounds__(256)
rr_rows_kernel(const T* __restrict__ y, T* __restrict__ x, const __grid_constant__ IndexProgram P,
               int64_t rows, int64_t inner, int op) {
    const int nl = P.ndim_loop - P.inner_dims, nx = P.ndim_x;
    const int lane = threadIdx.x & 31;
    const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t row0 = warp * 32; row0 < rows; row0 += nwarps * 32) {
        const int64_t row = row0 + lane;
        long long off = -1;                                   // -1: index outside x, the run is skipped
        if (row < rows) {
            I iv[kMaxDims];
            int64_t r = row;
            for (int d = P.ndim_loop - 1; d >= nl; d--) iv[d] = 0;
#pragma unroll 1
            for (int d = nl - 1; d >= 0; d--) { int64_t s = P.loop_shape[d]; iv[d] = (I)(r % s); r /= s; }
            I xid[kMaxDims];
            if (!eval_index_program<I>(P, iv, xid)) {
                off = 0;
                for (int d = 0; d < nx; d++) off = off * P.x_shape[d] + (long long)xid[d];
            }
        }
        const int active = (int)min((int64_t)32, rows - row0);
        if constexpr (std::is_same<T, float>::value) {
            // float add on short aligned runs (a 64-float row is 16 vectors): the warp covers 32 / nv runs per access, one
            // 16-byte vector reduction per lane instead of four scalar ones, four runs' loads in flight
            const int64_t nv = inner / 4;
            if (op == OP_ADD && inner % 4 == 0 && nv <= 32 && (32 % nv) == 0 && (((uintptr_t)x | (uintptr_t)y) & 15) == 0) {
                const int per = 32 / (int)nv, sub = lane / (int)nv, li = lane % (int)nv;
                constexpr int U = 4;
                for (int k0 = 0; k0 < active; k0 += per * U) {
                    float4 v[U];
                    long long o[U];
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        const int k = k0 + u * per + sub;
                        o[u] = __shfl_sync(0xffffffffu, off, k & 31);
                        if (k >= active) o[u] = -1;
                        if (o[u] >= 0) v[u] = reinterpret_cast<const float4*>(y + (row0 + k) * inner)[li];
                    }
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        if (o[u] < 0) continue;
                        float* dst = x + o[u] + li * 4;
                        if (o[u] % 4 == 0)
                            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v[u].x), "f"(v[u].y), "f"(v[u].z), "f"(v[u].w) : "memory");
                        else { atomicAdd(dst, v[u].x); atomicAdd(dst + 1, v[u].y); atomicAdd(dst + 2, v[u].z); atomicAdd(dst + 3, v[u].w); }
                    }
                }
                continue;
            }
        }
        for (int k = 0; k < active; k++) {
            const long long o = __shfl_sync(0xffffffffu, off, k);
            if (o < 0) continue;
            const T* src = y + (row0 + k) * inner;
            for (int64_t i = lane; i < inner; i += 32) atomic_apply<T>(x + o + i, src[i], op);
        }
    }
}

// ---- injective affine map: x[A.i + c] = op(init, y[i]) with plain stores -----------------------------
// One thread takes 4 consecutive y elements (one 128-bit load for 4-byte types), advances the loop
// coordinates like an odometer and pairs neighbouring x offsets into 8/16-byte stores.
struct RRAffineArgs {
    int32_t ndim_loop, ndim_x;
    int64_t loop_shape[kMaxDims];
    int64_t x_shape[kMaxDims];
    int64_t coef[kMaxDims][kMaxDims];
    int64_t c0[kMaxDims];
    int32_t check_bounds;          // 0 when the host proved every index in range
};

template <typename T>
__global__ void __launch_bounds__(256)
rr_affine_kernel(const T* __restrict__ y, T* __restrict__ x, const __grid_constant__ RRAffineArgs A,
                 int64_t n, int op, T init) {
    constexpr int VEC = 4;
    const int nl = A.ndim_loop, nx = A.ndim_x;
    const int64_t n_vec = (n + VEC - 1) / VEC;
    const bool aligned = ((uintptr_t)y % (VEC * sizeof(T))) == 0;
    for (int64_t v = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; v < n_vec; v += (int64_t)gridDim.x * blockDim.x) {
        const int64_t flat = v * VEC;
        const int cnt = (int)(n - flat < VEC ? n - flat : VEC);
        __align__(16) T val[VEC];
        if (cnt == VEC && aligned && sizeof(T) * VEC == 16) *reinterpret_cast<uint4*>(val) = __ldcs(reinterpret_cast<const uint4*>(y + flat));
        else for (int e = 0; e < cnt; e++) val[e] = y[flat + e];
        int64_t iv[kMaxDims];
        int64_t r = flat;
#pragma unroll 1
        for (int d = nl - 1; d >= 0; d--) { int64_t s = A.loop_shape[d]; iv[d] = r % s; r /= s; }
        int64_t off[VEC];
        bool ok[VEC];
#pragma unroll
        for (int e = 0; e < VEC; e++) {
            int64_t o = 0; bool over = false;
#pragma unroll 1
            for (int d = 0; d < nx; d++) {
                int64_t id = A.c0[d];
                for (int j = 0; j < nl; j++) id += A.coef[d][j] * iv[j];
                if (A.check_bounds) over |= (id < 0) | (id >= A.x_shape[d]);
                o = o * A.x_shape[d] + id;
            }
            off[e] = o; ok[e] = !over && e < cnt;
            // odometer step
#pragma unroll 1
            for (int d = nl - 1; d >= 0; d--) { if (++iv[d] < A.loop_shape[d]) break; iv[d] = 0; }
        }
#pragma unroll
        for (int e = 0; e < VEC; e++) val[e] = apply_op<T>(op, init, val[e]);
        if constexpr (sizeof(T) == 4) {
            const bool all = ok[0] & ok[1] & ok[2] & ok[3];
            if (all && off[1] == off[0] + 1 && off[2] == off[0] + 2 && off[3] == off[0] + 3 && (((uintptr_t)(x + off[0])) & 15) == 0) {
                *reinterpret_cast<uint4*>(x + off[0]) = *reinterpret_cast<uint4*>(val);
                continue;
            }
            if (all && off[1] == off[0] + 1 && off[3] == off[2] + 1 && (((uintptr_t)(x + off[0])) & 7) == 0 && (((uintptr_t)(x + off[2])) & 7) == 0) {
                *reinterpret_cast<uint2*>(x + off[0]) = *reinterpret_cast<uint2*>(val);
                *reinterpret_cast<uint2*>(x + off[2]) = *reinterpret_cast<uint2*>(val + 2);
                continue;
            }
        }
#pragma unroll
        for (int e = 0; e < VEC; e++) if (ok[e]) x[off[e]] = val[e];
    }
}

// Fast form of the injective path when every index is provably in range: the x offset is one linear
// function of the (merged) loop coordinates, off = c + sum_j F[j]*i_j. A thread owns 4 consecutive y
// elements whose x offsets are off + delta[0..3] with a host-computed constant delta table (the 4 elements
// stay inside the trailing loop axes), so the only index arithmetic is one 32-bit div/mod per outer axis.
struct RRFlatArgs {
    int32_t nd;                    // outer (merged) axes
    uint32_t shape[kMaxDims];
    int64_t F[kMaxDims];
    int64_t c;
    int64_t delta[4];
    int32_t store_mode;            // 0 scalar, 1 two 8-byte stores, 2 one 16-byte store
};

template <typename T>
__global__ void __launch_bounds__(256)
rr_flat_kernel(const T* __restrict__ y, T* __restrict__ x, const __grid_constant__ RRFlatArgs A,
               uint32_t n_vec, int op, T init) {
    static_assert(sizeof(T) == 4, "4-byte elements");
    for (uint32_t v = blockIdx.x * blockDim.x + threadIdx.x; v < n_vec; v += gridDim.x * blockDim.x) {
        uint4 raw = __ldcs(reinterpret_cast<const uint4*>(y) + v);
        T val[4]; memcpy(val, &raw, 16);
        uint32_t r = v;
        int64_t off = A.c;
#pragma unroll 1
        for (int d = A.nd - 1; d >= 0; d--) {
            const uint32_t s = A.shape[d];
            const uint32_t q = r / s;
            off += A.F[d] * (int64_t)(r - q * s);
            r = q;
        }
#pragma unroll
        for (int e = 0; e < 4; e++) val[e] = apply_op<T>(op, init, val[e]);
        if (A.store_mode == 2) {
            memcpy(&raw, val, 16);
            __stcs(reinterpret_cast<uint4*>(x + off + A.delta[0]), raw);
        } else if (A.store_mode == 1) {
            uint2 lo, hi; memcpy(&lo, val, 8); memcpy(&hi, val + 2, 8);
            __stcs(reinterpret_cast<uint2*>(x + off + A.delta[0]), lo);
            __stcs(reinterpret_cast<uint2*>(x + off + A.delta[2]), hi);
        } else {
#pragma unroll
            for (int e = 0; e < 4; e++) x[off + A.delta[e]] = val[e];
        }
    }
}

// ---- scatter through an index array: x[e0[i]] = op(x[e0[i]], y[i]) ----------------------------------
// Loads are issued UNROLL vectors ahead so that enough bytes are in flight per SM to cover HBM latency.
// f(bin, value, valid) is called by all 32 lanes of a warp together (valid == false on lanes past the end), so
// that warp-collective code may run inside it.
template <typename T, typename E, int VEC, int UNROLL, typename F>
__device__ __forceinline__ void for_each_pair(const T* __restrict__ y, const E* __restrict__ idx, int64_t n, F&& f) {
    const int64_t n_vec = n / VEC;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int lane = threadIdx.x & 31;
    for (int64_t w0 = blockIdx.x * (int64_t)blockDim.x + (threadIdx.x - lane); w0 < n_vec; w0 += stride * UNROLL) {
        const int64_t v0 = w0 + lane;
        __align__(16) T val[UNROLL][VEC];
        __align__(16) E ind[UNROLL][VEC];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int64_t v = v0 + u * stride;
            if (v < n_vec) {
                if constexpr (VEC * sizeof(T) == 16) *reinterpret_cast<uint4*>(val[u]) = __ldcs(reinterpret_cast<const uint4*>(y) + v);
                else {
#pragma unroll
                    for (int e = 0; e < VEC; e++) val[u][e] = y[v * VEC + e];
                }
                if constexpr (VEC * sizeof(E) == 16) *reinterpret_cast<uint4*>(ind[u]) = __ldcs(reinterpret_cast<const uint4*>(idx) + v);
                else if constexpr (VEC * sizeof(E) == 32) {
                    *reinterpret_cast<uint4*>(ind[u]) = __ldcs(reinterpret_cast<const uint4*>(idx) + 2 * v);
                    *reinterpret_cast<uint4*>(ind[u] + VEC / 2) = __ldcs(reinterpret_cast<const uint4*>(idx) + 2 * v + 1);
                } else {
#pragma unroll
                    for (int e = 0; e < VEC; e++) ind[u][e] = idx[v * VEC + e];
                }
            } else {
#pragma unroll
                for (int e = 0; e < VEC; e++) { ind[u][e] = (E)-1; val[u][e] = T(); }
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            if (w0 + u * stride < n_vec) {                       // warp-uniform
                const bool valid = v0 + u * stride < n_vec;
#pragma unroll
                for (int e = 0; e < VEC; e++) f((int64_t)ind[u][e], val[u][e], valid);
            }
        }
    }
    for (int64_t w = n_vec * VEC + blockIdx.x * (int64_t)blockDim.x + (threadIdx.x - lane); w < n; w += stride) {
        const int64_t i = w + lane;
        const bool valid = i < n;
        f(valid ? (int64_t)idx[i] : (int64_t)-1, valid ? y[i] : T(), valid);
    }
}

// Many bins: the bins live in L2 and every element costs one red.global. A per-CTA direct-mapped
// shared-memory cache (slot = bin mod SLOTS, claimed by the first bin that arrives) absorbs the hot
// head of skewed index distributions, whose same-address atomics would otherwise serialise in L2; the cache is
// flushed with one atomic per used slot.
constexpr int kCacheThreads = 1024;
constexpr int kCacheSlots = 4096;

template <typename T, typename E, int VEC>
__global__ void __launch_bounds__(kCacheThreads, 2)
rr_direct_cached_kernel(const T* __restrict__ y, const E* __restrict__ idx, T* __restrict__ x,
                        int64_t n, int64_t bins, int op, T init) {
    __shared__ int32_t tag[kCacheSlots];
    __shared__ T acc[kCacheSlots];
    for (int i = threadIdx.x; i < kCacheSlots; i += blockDim.x) { tag[i] = -1; acc[i] = init; }
    __syncthreads();
    for_each_pair<T, E, VEC, 2>(y, idx, n, [&](int64_t b, T v, bool valid) {
        if (!valid || b < 0 || b >= bins) return;
        const int s = (int)(b & (kCacheSlots - 1));
        int32_t t = *reinterpret_cast<volatile int32_t*>(tag + s);
        if (t == -1) { t = atomicCAS(tag + s, -1, (int32_t)b); if (t == -1) t = (int32_t)b; }
        if (t == (int32_t)b) atomic_apply<T>(acc + s, v, op);
        else atomic_apply<T>(x + b, v, op);
    });
    __syncthreads();
    for (int i = threadIdx.x; i < kCacheSlots; i += blockDim.x) {
        const int32_t t = tag[i];
        if (t >= 0) atomic_apply<T>(x + t, acc[i], op);
    }
}

// Plain variant (2^31 bins or more, or element types without a cache specialisation).
template <typename T, typename E, int VEC>
__global__ void __launch_bounds__(256)
rr_direct_kernel(const T* __restrict__ y, const E* __restrict__ idx, T* __restrict__ x,
                 int64_t n, int64_t bins, int op) {
    for_each_pair<T, E, VEC, 2>(y, idx, n, [&](int64_t b, T v, bool valid) {
        if (valid && b >= 0 && b < bins) atomic_apply<T>(x + b, v, op);
    });
}

// ---- privatised scatter, few bins ------------------------------------------------------------------
// smem layout: R replicas of `bins` elements at a stride of bins+1 (so that the replicas of one bin sit in
// different banks); lane l of a warp updates replica (l % R), which spreads the same-bin lanes of skewed inputs.
//
// Hot bins (float add): a float add in shared memory is a compare-and-swap loop, and lanes of one warp that meet in one
// bin retry one after the other -- measured 35 G/s on one address against 560 G/s on spread addresses -- so skewed inputs
// (Zipf: a few bins take a third of the elements) ran at half the speed of uniform ones. Each CTA therefore looks at the
// first vector of indices of each of its threads (4096 indices of the elements it is about to process), finds the kHot
// most frequent bins (if any holds more than 1 % of the sample) and keeps those bins' sums in registers: an element of a
// hot bin costs a compare and a predicated add, no atomic. The registers are combined per warp and enter the replicas
// with one atomic per warp and hot bin.
constexpr int kHot = 4;

template <typename T, typename E, int VEC>
__global__ void __launch_bounds__(kPrivThreads, 1)
rr_privatised_kernel(const T* __restrict__ y, const E* __restrict__ idx, T* __restrict__ partial,
                     int64_t n, int bins, int replicas, int op, bool is_bool, bool allow_hot) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* sm = reinterpret_cast<T*>(smem_raw);
    const int rstride = bins + 1;
    const T init = init_value<T>(op, is_bool);
    __shared__ int hot_bin[kHot];
    __shared__ unsigned warp_best[kPrivThreads / 32];
    constexpr bool kHotPath = std::is_same<T, float>::value && VEC > 1;
    bool use_hot = false;
    if (kHotPath && allow_hot && op == OP_ADD && bins < 8192 && n / VEC >= (int64_t)gridDim.x * blockDim.x * 8) {
        // histogram of the sample in the (not yet initialised) replica area
        int* hist = reinterpret_cast<int*>(smem_raw);
        for (int i = threadIdx.x; i < bins; i += blockDim.x) hist[i] = 0;
        __syncthreads();
        {
            const E* p = idx + (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) * VEC;      // inside the array: n / VEC >= threads * 8
#pragma unroll
            for (int e = 0; e < VEC; e++) {
                const int64_t b = (int64_t)p[e];
                if (b >= 0 && b < bins) atomicAdd(hist + b, 1);
            }
        }
        __syncthreads();
        const unsigned threshold = (unsigned)(blockDim.x * VEC) / 100u;                       // 1 % of the sample
        if (threadIdx.x < kHot) hot_bin[threadIdx.x] = -2;
        for (int k = 0; k < kHot; k++) {
            unsigned best = 0;                                                                // count << 13 | bin
            for (int i = threadIdx.x; i < bins; i += blockDim.x) best = max(best, ((unsigned)hist[i] << 13) | (unsigned)i);
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, d));
            if ((threadIdx.x & 31) == 0) warp_best[threadIdx.x >> 5] = best;
            __syncthreads();
            unsigned b2 = warp_best[threadIdx.x & 31];                                        // 32 warps: every warp folds the 32 maxima
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) b2 = max(b2, __shfl_xor_sync(0xffffffffu, b2, d));
            const bool hot = (b2 >> 13) > threshold;                                          // the same in every thread
            if (!hot) break;                                                                  // uniform inputs leave after one look
            if (threadIdx.x == 0) { hot_bin[k] = (int)(b2 & 8191u); hist[b2 & 8191u] = 0; }
            __syncthreads();
        }
        __syncthreads();
        use_hot = hot_bin[0] >= 0;                                                            // the same for the whole CTA
        __syncthreads();
    }
    for (int i = threadIdx.x; i < rstride * replicas; i += blockDim.x) sm[i] = init;
    __syncthreads();
    T* mine = sm + (threadIdx.x % replicas) * rstride;
    if constexpr (kHotPath) {
        // one loop for both cases (with no hot bin the compares never hit): two copies of the unrolled loop in one kernel
        // cost the plain case 15 % through the register allocation they share
        float hacc[kHot];
#pragma unroll
        for (int k = 0; k < kHot; k++) hacc[k] = 0.f;
        int hb[kHot];
#pragma unroll
        for (int k = 0; k < kHot; k++) hb[k] = use_hot ? hot_bin[k] : -2;
        for_each_pair<T, E, VEC, 4>(y, idx, n, [&](int64_t b, T v, bool valid) {
            const int bi = (int)b;
            bool hit = false;
#pragma unroll
            for (int k = 0; k < kHot; k++) {
                const bool m = bi == hb[k];
                hacc[k] += m ? (float)v : 0.f;
                hit |= m;
            }
            if (!hit && valid && b >= 0 && b < bins) atomic_apply<T>(mine + b, v, op);
        });
        if (use_hot) {
#pragma unroll
            for (int k = 0; k < kHot; k++) {
                float a = hacc[k];
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) a += __shfl_down_sync(0xffffffffu, a, d);
                if ((threadIdx.x & 31) == 0 && hb[k] >= 0) atomic_apply<T>(mine + hb[k], (T)a, op);
            }
        }
    } else {
        for_each_pair<T, E, VEC, 4>(y, idx, n, [&](int64_t b, T v, bool valid) {
            if (valid && b >= 0 && b < bins) atomic_apply<T>(mine + b, v, op);
        });
    }
    __syncthreads();
    // fold the replicas in fixed order and publish this CTA's row
    for (int b = threadIdx.x; b < bins; b += blockDim.x) {
        T acc = sm[b];
        for (int r = 1; r < replicas; r++) acc = apply_op<T>(op, acc, sm[r * rstride + b]);
        partial[(int64_t)blockIdx.x * bins + b] = acc;
    }
}

// Folds the per-CTA rows into x in a fixed order (deterministic): a CTA owns 32 bins, its 8 warps take the rows
// r = w, w+8, ... (coalesced 128-byte reads), then warp 0 combines the 8 partial sums in warp order.
template <typename T>
__global__ void __launch_bounds__(256)
rr_fold_partials_kernel(const T* __restrict__ partial, T* __restrict__ x, int bins, int rows, int op, bool is_bool) {
    __shared__ T part[8][33];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    for (int b0 = blockIdx.x * 32; b0 < bins; b0 += gridDim.x * 32) {
        const int b = b0 + lane;
        T acc = init_value<T>(op, is_bool);
        if (b < bins)
            for (int r = w; r < rows; r += 8) acc = apply_op<T>(op, acc, partial[(int64_t)r * bins + b]);
        part[w][lane] = acc;
        __syncthreads();
        if (w == 0 && b < bins) {
            T t = part[0][lane];
#pragma unroll
            for (int k = 1; k < 8; k++) t = apply_op<T>(op, t, part[k][lane]);
            x[b] = t;
        }
        __syncthreads();
    }
}

// ---- host side -----------------------------------------------------------------------------------
struct RRPlan {
    enum Path { GENERIC, INJECTIVE, DIRECT, PRIVATISED } path = GENERIC;
    int replicas = 1;
    size_t workspace = 0;
    size_t smem = 0;
    bool in_range = false;      // injective path: every index of every y element is inside x
    bool covers_all = false;    // ... and every x element is written: the init fill is skipped
};

static bool affine_injective(const IndexProgram& P) {
    if (!P.is_affine) return false;
    // flat coefficient of every loop axis
    int64_t xs[kMaxDims]; int64_t st = 1;
    for (int d = P.ndim_x - 1; d >= 0; d--) { xs[d] = st; st *= P.x_shape[d]; }
    std::vector<std::pair<int64_t, int64_t>> terms;   // (|F_j|, n_j - 1)
    for (int j = 0; j < P.ndim_loop; j++) {
        if (P.loop_shape[j] <= 1) continue;
        int64_t F = 0;
        for (int d = 0; d < P.ndim_x; d++) F += P.coef[d][j] * xs[d];
        if (F == 0) return false;
        terms.push_back({F < 0 ? -F : F, P.loop_shape[j] - 1});
    }
    std::sort(terms.begin(), terms.end());
    int64_t reach = 0;            // max offset reachable with the smaller terms
    for (auto& t : terms) {
        if (t.first <= reach) return false;
        reach += t.first * t.second;
    }
    return true;
}

static bool op_supported(int op, int dtype) {
    switch (op) {
        case OP_ADD: case OP_MUL: case OP_MAX: case OP_MIN: case OP_VOID: return true;
        case OP_BAND: case OP_BOR: case OP_BXOR: return !dtype_is_float(dtype);
        case OP_LAND: case OP_LOR: case OP_LXOR: return true;
    }
    return false;
}

static RRPlan make_plan(const b200jt_tensor* y, const b200jt_tensor* x, int op, const IndexProgram& P) {
    RRPlan plan;
    const int es = dtype_size(x->dtype);
    const int64_t bins = numel(x);
    if (op != OP_VOID && affine_injective(P)) {
        plan.path = RRPlan::INJECTIVE;
        plan.in_range = true;
        for (int d = 0; d < P.ndim_x; d++) {
            int64_t lo = P.c0[d], hi = P.c0[d];
            for (int j = 0; j < P.ndim_loop; j++) {
                const int64_t span = P.coef[d][j] * (P.loop_shape[j] - 1);
                if (span < 0) lo += span; else hi += span;
            }
            if (lo < 0 || hi >= P.x_shape[d]) plan.in_range = false;
        }
        plan.covers_all = plan.in_range && numel(y) == bins;
        return plan;
    }
    if (P.is_direct_extra && op != OP_VOID &&
        (P.extras[0].dtype == B200JT_INT32 || P.extras[0].dtype == B200JT_INT64) && es >= 4) {
        if (bins * es <= kPrivMaxBinBytes && numel(y) >= (1 << 16)) {
            plan.path = RRPlan::PRIVATISED;
            int r = (int)(kPrivMaxSmemBytes / ((bins + 1) * es));
            plan.replicas = r >= 8 ? 8 : r >= 4 ? 4 : r >= 2 ? 2 : 1;
            plan.smem = (size_t)plan.replicas * (bins + 1) * es;
            plan.workspace = (size_t)kPrivGrid * bins * es;
        } else {
            plan.path = RRPlan::DIRECT;
        }
    }
    return plan;
}

// Builds the flat-offset description used by rr_flat_kernel; false if 4 consecutive y elements can leave the
// trailing axes (then the odometer kernel is used).
static bool make_flat_args(const IndexProgram& P, uintptr_t xbase, size_t es, RRFlatArgs* A) {
    memset(A, 0, sizeof(*A));
    int64_t xs[kMaxDims]; int64_t st = 1;
    for (int d = P.ndim_x - 1; d >= 0; d--) { xs[d] = st; st *= P.x_shape[d]; }
    int64_t F[kMaxDims], shp[kMaxDims]; int n = 0;
    A->c = 0;
    for (int d = 0; d < P.ndim_x; d++) A->c += P.c0[d] * xs[d];
    for (int j = 0; j < P.ndim_loop; j++) {
        int64_t f = 0;
        for (int d = 0; d < P.ndim_x; d++) f += P.coef[d][j] * xs[d];
        if (P.loop_shape[j] == 1) continue;
        if (n && F[n - 1] == f * P.loop_shape[j]) { shp[n - 1] *= P.loop_shape[j]; F[n - 1] = f; }   // merge
        else { F[n] = f; shp[n] = P.loop_shape[j]; n++; }
    }
    if (n == 0) return false;
    // fold trailing axes until their product is a multiple of 4 elements
    int64_t prod = 1; int t = n;
    while (t > 0 && prod % 4 != 0) { t--; prod *= shp[t]; }
    if (prod % 4 != 0) return false;
    if (t == n - 1) {
        // the inner axis alone holds whole vectors
        for (int e = 0; e < 4; e++) A->delta[e] = e * F[n - 1];
        shp[n - 1] /= 4; F[n - 1] *= 4;
        t = n;
    } else {
        if (prod != 4) return false;             // the vector must cover the folded axes exactly
        for (int e = 0; e < 4; e++) {
            int64_t r = e, off = 0;
            for (int j = n - 1; j >= t; j--) { off += (r % shp[j]) * F[j]; r /= shp[j]; }
            A->delta[e] = off;
        }
    }
    A->nd = 0;
    for (int j = 0; j < t; j++) {
        if (shp[j] == 1) continue;
        if (shp[j] >= (1LL << 32)) return false;
        A->shape[A->nd] = (uint32_t)shp[j]; A->F[A->nd] = F[j]; A->nd++;
    }
    // store mode: alignment must hold for every vector -> every F and c + delta must keep it
    auto aligned_all = [&](int64_t first, int bytes) {
        const int64_t k = bytes / (int64_t)es;
        if ((xbase % bytes) != 0 || ((A->c + first) % k) != 0) return false;
        for (int j = 0; j < A->nd; j++) if (A->F[j] % k != 0) return false;
        return true;
    };
    const int64_t* d = A->delta;
    if (d[1] == d[0] + 1 && d[2] == d[0] + 2 && d[3] == d[0] + 3 && aligned_all(d[0], 16)) A->store_mode = 2;
    else if (d[1] == d[0] + 1 && d[3] == d[2] + 1 && aligned_all(d[0], 8) && aligned_all(d[2], 8)) A->store_mode = 1;
    else A->store_mode = 0;
    return true;
}

template <typename T>
static int run_typed(const b200jt_tensor* y, const b200jt_tensor* x, int op, const IndexProgram& P,
                     const RRPlan& plan, void* workspace, cudaStream_t st) {
    const int64_t n = numel(y), bins = numel(x);
    const bool is_bool = x->dtype == B200JT_BOOL;
    const T* yp = (const T*)y->ptr;
    T* xp = (T*)x->ptr;
    if (plan.path == RRPlan::PRIVATISED) {
        T* partial = (T*)workspace;
        const bool e64 = P.extras[0].dtype == B200JT_INT64;
        constexpr int VEC = 16 / sizeof(T);
        const bool aligned = ((uintptr_t)yp % 16 == 0) && ((uintptr_t)P.extras[0].ptr % 16 == 0);
        const int priv_grid = kPrivGrid - sm_reserve();         // rows of `partial` actually written and folded
        const char* hot_env = getenv("B200JT_RR_HOT");
        const bool allow_hot = !(hot_env && hot_env[0] == '0');
        // the shared-memory opt-in is set once per instantiation, not on every launch
#define B200JT_PRIV(E, V)                                                                                      \
        do { auto k = rr_privatised_kernel<T, E, V>;                                                            \
             static const cudaError_t attr_ = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrivMaxSmemBytes); \
             B200JT_CUDA(attr_);                                                                                  \
             k<<<priv_grid, kPrivThreads, plan.smem, st>>>(yp, (const E*)P.extras[0].ptr, partial, n, (int)bins,   \
                                                           plan.replicas, op, is_bool, allow_hot); } while (0)
        if (e64) { if (aligned) B200JT_PRIV(int64_t, VEC); else B200JT_PRIV(int64_t, 1); }
        else     { if (aligned) B200JT_PRIV(int32_t, VEC); else B200JT_PRIV(int32_t, 1); }
#undef B200JT_PRIV
        B200JT_LAUNCH_CHECK();
        rr_fold_partials_kernel<T><<<grid_for((bins + 31) / 32 * 256, 256), 256, 0, st>>>(partial, xp, (int)bins, priv_grid, op, is_bool);
        B200JT_LAUNCH_CHECK();
        return 0;
    }
    if (op != OP_VOID && bins > 0 && !(plan.path == RRPlan::INJECTIVE && plan.covers_all)) {
        fill_kernel<T><<<grid_for(bins, 256), 256, 0, st>>>(xp, bins, init_value<T>(op, is_bool));
        B200JT_LAUNCH_CHECK();
    }
    if (n == 0 || bins == 0) return 0;
    if (plan.path == RRPlan::INJECTIVE && plan.in_range && sizeof(T) == 4 && n % 4 == 0 && n / 4 < (1LL << 32) &&
        ((uintptr_t)yp % 16) == 0) {
        RRFlatArgs FA;
        if (make_flat_args(P, (uintptr_t)xp, sizeof(T), &FA)) {
            if constexpr (sizeof(T) == 4) {
                rr_flat_kernel<T><<<grid_for(n / 4, 256), 256, 0, st>>>(yp, xp, FA, (uint32_t)(n / 4), op, init_value<T>(op, is_bool));
                B200JT_LAUNCH_CHECK();
                return 0;
            }
        }
    }
    if (plan.path == RRPlan::INJECTIVE) {
        RRAffineArgs A; memset(&A, 0, sizeof(A));
        A.ndim_loop = P.ndim_loop; A.ndim_x = P.ndim_x;
        memcpy(A.loop_shape, P.loop_shape, sizeof(A.loop_shape));
        memcpy(A.x_shape, P.x_shape, sizeof(A.x_shape));
        memcpy(A.coef, P.coef, sizeof(A.coef));
        memcpy(A.c0, P.c0, sizeof(A.c0));
        A.check_bounds = plan.in_range ? 0 : 1;
        rr_affine_kernel<T><<<grid_for((n + 3) / 4, 256), 256, 0, st>>>(yp, xp, A, n, op, init_value<T>(op, is_bool));
        B200JT_LAUNCH_CHECK();
        return 0;
    }
    if (plan.path == RRPlan::DIRECT) {
        const bool e64 = P.extras[0].dtype == B200JT_INT64;
        constexpr int VEC = 16 / sizeof(T);
        const bool aligned = ((uintptr_t)yp % 16 == 0) && ((uintptr_t)P.extras[0].ptr % 16 == 0);
        if constexpr (sizeof(T) == 4 || sizeof(T) == 8) {
            if (bins < (1LL << 31)) {
                const T init = init_value<T>(op, is_bool);
                // two CTAs are resident per SM; three waves of them balance the tail better than one (0.117 -> 0.114 ms
                // uniform, 0.103 -> 0.097 ms Zipf for 2^24 -> 2^20); B200JT_RR_DIRECT_CTAS overrides the CTAs per SM
                const char* gm_ = getenv("B200JT_RR_DIRECT_CTAS");
                const int per_sm = gm_ ? std::max(1, std::min(16, atoi(gm_))) : 6;
                const unsigned grid = (unsigned)per_sm * (kNumSMs - sm_reserve());
                if (e64) {
                    if (aligned) rr_direct_cached_kernel<T, int64_t, VEC><<<grid, kCacheThreads, 0, st>>>(yp, (const int64_t*)P.extras[0].ptr, xp, n, bins, op, init);
                    else rr_direct_cached_kernel<T, int64_t, 1><<<grid, kCacheThreads, 0, st>>>(yp, (const int64_t*)P.extras[0].ptr, xp, n, bins, op, init);
                } else {
                    if (aligned) rr_direct_cached_kernel<T, int32_t, VEC><<<grid, kCacheThreads, 0, st>>>(yp, (const int32_t*)P.extras[0].ptr, xp, n, bins, op, init);
                    else rr_direct_cached_kernel<T, int32_t, 1><<<grid, kCacheThreads, 0, st>>>(yp, (const int32_t*)P.extras[0].ptr, xp, n, bins, op, init);
                }
                B200JT_LAUNCH_CHECK();
                return 0;
            }
        }
        const unsigned grid = grid_for(n / VEC + 1, 256);
        if (e64) {
            if (aligned) rr_direct_kernel<T, int64_t, VEC><<<grid, 256, 0, st>>>(yp, (const int64_t*)P.extras[0].ptr, xp, n, bins, op);
            else rr_direct_kernel<T, int64_t, 1><<<grid, 256, 0, st>>>(yp, (const int64_t*)P.extras[0].ptr, xp, n, bins, op);
        } else {
            if (aligned) rr_direct_kernel<T, int32_t, VEC><<<grid, 256, 0, st>>>(yp, (const int32_t*)P.extras[0].ptr, xp, n, bins, op);
            else rr_direct_kernel<T, int32_t, 1><<<grid, 256, 0, st>>>(yp, (const int32_t*)P.extras[0].ptr, xp, n, bins, op);
        }
        B200JT_LAUNCH_CHECK();
        return 0;
    }
    const bool small = n < (1LL << 31) && bins < (1LL << 31);
    if (P.inner_dims > 0 && P.inner_elems * (int64_t)sizeof(T) >= 64) {
        const int64_t rows = n / P.inner_elems;
        const unsigned rgrid = grid_for(rows, 256);
        if (small) rr_rows_kernel<T, int32_t><<<rgrid, 256, 0, st>>>(yp, xp, P, rows, P.inner_elems, op);
        else       rr_rows_kernel<T, int64_t><<<rgrid, 256, 0, st>>>(yp, xp, P, rows, P.inner_elems, op);
        B200JT_LAUNCH_CHECK();
        return 0;
    }
    const unsigned grid = grid_for(n, 256);
    if (small) rr_generic_kernel<T, int32_t><<<grid, 256, 0, st>>>(yp, xp, P, n, op);
    else       rr_generic_kernel<T, int64_t><<<grid, 256, 0, st>>>(yp, xp, P, n, op);
    B200JT_LAUNCH_CHECK();
    return 0;
}

static int prepare(const b200jt_tensor* y, const b200jt_tensor* x, const char* op_name,
                   const char* const* indexes, int n_indexes, const char* const* conds, int n_conds,
                   const b200jt_tensor* extras, int n_extras, IndexProgram* P, int* op, RRPlan* plan) {
    B200JT_CHECK_ARG(valid_tensor(x) && valid_tensor(y), "invalid tensor descriptor");
    B200JT_CHECK_ARG(x->dtype == y->dtype, "x and y must have the same dtype");
    B200JT_CHECK_ARG(n_indexes == x->ndim, "Number of shape and indexes should be the same.");
    B200JT_CHECK_ARG(n_extras >= 0 && n_extras <= B200JT_MAX_EXTRAS, "too many extras");
    for (int k = 0; k < n_extras; k++) B200JT_CHECK_ARG(valid_tensor(&extras[k]), "invalid extras descriptor");
    *op = strcmp(op_name, "void") == 0 ? OP_VOID : binary_op_from_name(op_name);
    B200JT_CHECK_ARG(*op != OP_INVALID && *op != OP_MEAN && op_supported(*op, x->dtype),
                     std::string("unsupported reindex_reduce op '") + op_name + "' for " + dtype_name(x->dtype));
    std::string err;
    if (!compile_index_program(y->shape, y->ndim, x->shape, x->ndim, indexes, n_indexes, conds, n_conds,
                               extras, n_extras, P, &err))
        return fail(-2, "b200jt_reindex_reduce: " + err);
    *plan = make_plan(y, x, *op, *P);
    return 0;
}

}  // namespace b200jt

using namespace b200jt;

extern "C" size_t b200jt_reindex_reduce_workspace(const b200jt_tensor* y, const b200jt_tensor* x, const char* op,
                                                  const char* const* indexes, int n_indexes,
                                                  const char* const* overflow_conditions, int n_conditions,
                                                  const b200jt_tensor* extras, int n_extras) {
    IndexProgram P; int opc; RRPlan plan;
    if (prepare(y, x, op, indexes, n_indexes, overflow_conditions, n_conditions, extras, n_extras, &P, &opc, &plan) != 0)
        return 0;
    return plan.workspace;
}

extern "C" int b200jt_reindex_reduce(const b200jt_tensor* y, const b200jt_tensor* x, const char* op,
                                     const char* const* indexes, int n_indexes,
                                     const char* const* overflow_conditions, int n_conditions,
                                     const b200jt_tensor* extras, int n_extras,
                                     void* workspace, size_t workspace_bytes, void* stream) {
    IndexProgram P; int opc; RRPlan plan;
    int rc = prepare(y, x, op, indexes, n_indexes, overflow_conditions, n_conditions, extras, n_extras, &P, &opc, &plan);
    if (rc) return rc;
    B200JT_CHECK_ARG(workspace_bytes >= plan.workspace && (plan.workspace == 0 || workspace),
                     "workspace too small: need " + std::to_string(plan.workspace) + " bytes");
    cudaStream_t st = (cudaStream_t)stream;
    switch (x->dtype) {
        case B200JT_BOOL: case B200JT_UINT8: return run_typed<uint8_t>(y, x, opc, P, plan, workspace, st);
        case B200JT_INT8: return run_typed<int8_t>(y, x, opc, P, plan, workspace, st);
        case B200JT_INT16: return run_typed<int16_t>(y, x, opc, P, plan, workspace, st);
        case B200JT_INT32: return run_typed<int32_t>(y, x, opc, P, plan, workspace, st);
        case B200JT_INT64: return run_typed<int64_t>(y, x, opc, P, plan, workspace, st);
        case B200JT_FLOAT16: return run_typed<__half>(y, x, opc, P, plan, workspace, st);
        case B200JT_BFLOAT16: return run_typed<__nv_bfloat16>(y, x, opc, P, plan, workspace, st);
        case B200JT_FLOAT32: return run_typed<float>(y, x, opc, P, plan, workspace, st);
        case B200JT_FLOAT64: return run_typed<double>(y, x, opc, P, plan, workspace, st);
    }
    return fail(-1, "b200jt_reindex_reduce: unsupported dtype");
}

// ---- setitem: accumulate into a copy of x instead of into the op's identity -------------------------------
// out = x; for every element i of data: out[index(i)] = op(out[index(i)], data[i]); op "void" assigns. This is the
// loop of SetitemOp::jit_run (python/jittor/src/ops/setitem_op.cc:312-366): the copy, then one read-modify-write per
// element of the sliced region. Elements whose index falls outside out are skipped (the reference does not check).
// "add" (and the other ops with an atomic form) are exact under duplicate indices; "void" keeps one of the
// duplicates, as on the reference's CUDA path.
extern "C" int b200jt_setitem(const b200jt_tensor* x, const b200jt_tensor* data, const b200jt_tensor* out, const char* op,
                              const char* const* indexes, int n_indexes,
                              const b200jt_tensor* extras, int n_extras, void* stream) {
    B200JT_CHECK_ARG(valid_tensor(x) && valid_tensor(out) && valid_tensor(data), "invalid tensor descriptor");
    B200JT_CHECK_ARG(x->dtype == out->dtype && x->ndim == out->ndim, "x and out must have the same dtype and shape");
    for (int d = 0; d < x->ndim; d++) B200JT_CHECK_ARG(x->shape[d] == out->shape[d], "x and out must have the same shape");
    IndexProgram P; int opc; RRPlan plan;
    int rc = prepare(data, out, op, indexes, n_indexes, nullptr, 0, extras, n_extras, &P, &opc, &plan);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t bins = numel(out);
    if (bins == 0) return 0;
    if (x->ptr != out->ptr)
        B200JT_CUDA(cudaMemcpyAsync(out->ptr, x->ptr, (size_t)bins * dtype_size(x->dtype), cudaMemcpyDeviceToDevice, st));
    const int64_t n = numel(data);
    if (n == 0) return 0;
    const bool small = n < (1LL << 31) && bins < (1LL << 31);
    const unsigned grid = grid_for(n, 256);
    const bool by_rows = P.inner_dims > 0 && P.inner_elems * dtype_size(out->dtype) >= 64;
    const int64_t rows = by_rows ? n / P.inner_elems : 0;
    const unsigned rgrid = grid_for(rows, 256);
#define B200JT_SETITEM(T)                                                                                        \
    do { if (by_rows) {                                                                                          \
             if (small) rr_rows_kernel<T, int32_t><<<rgrid, 256, 0, st>>>((const T*)data->ptr, (T*)out->ptr, P, rows, P.inner_elems, opc); \
             else       rr_rows_kernel<T, int64_t><<<rgrid, 256, 0, st>>>((const T*)data->ptr, (T*)out->ptr, P, rows, P.inner_elems, opc); \
         } else if (small) rr_generic_kernel<T, int32_t><<<grid, 256, 0, st>>>((const T*)data->ptr, (T*)out->ptr, P, n, opc);  \
         else              rr_generic_kernel<T, int64_t><<<grid, 256, 0, st>>>((const T*)data->ptr, (T*)out->ptr, P, n, opc);  \
    } while (0)
    switch (out->dtype) {
        case B200JT_BOOL: case B200JT_UINT8: B200JT_SETITEM(uint8_t); break;
        case B200JT_INT8: B200JT_SETITEM(int8_t); break;
        case B200JT_INT16: B200JT_SETITEM(int16_t); break;
        case B200JT_INT32: B200JT_SETITEM(int32_t); break;
        case B200JT_INT64: B200JT_SETITEM(int64_t); break;
        case B200JT_FLOAT16: B200JT_SETITEM(__half); break;
        case B200JT_BFLOAT16: B200JT_SETITEM(__nv_bfloat16); break;
        case B200JT_FLOAT32: B200JT_SETITEM(float); break;
        case B200JT_FLOAT64: B200JT_SETITEM(double); break;
        default: return fail(-1, "b200jt_setitem: unsupported dtype");
    }
#undef B200JT_SETITEM
    B200JT_LAUNCH_CHECK();
    return 0;
}

// ---- allocation-free variant ----------------------------------------------------------------------
// Some callers cannot hand over a workspace because they are not allowed to allocate device memory at
// the point of the call: code running inside a memory-pool callback, a real-time loop whose allocator is
// frozen after start-up, or a host runtime that gives a plugin no allocation hook at all. For them the
// scratch rows of the privatised scatter live in a fixed array inside the library image. Every GPU that
// loads the library carries these 4 MiB until the process exits.
namespace b200jt {

constexpr size_t kStaticScratchBytes = 4u << 20;
static __device__ __align__(256) unsigned char g_rr_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_scratch_addr[kMaxDevices] = {};

// The array's name is only a host-side handle; the kernels need its device address, which is looked up once per
// device (with that device current) and cached.
static int static_scratch_ptr(void** out) {
    int dev = 0;
    B200JT_CUDA(cudaGetDevice(&dev));
    B200JT_CHECK_ARG(dev >= 0 && dev < kMaxDevices, "device ordinal out of range");
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        B200JT_CUDA(cudaGetSymbolAddress(&p, g_rr_static_scratch));
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return 0;
}

}  // namespace b200jt

extern "C" size_t b200jt_reindex_reduce_noalloc_max_scratch(void) { return b200jt::kStaticScratchBytes; }

extern "C" int b200jt_reindex_reduce_noalloc(const b200jt_tensor* y, const b200jt_tensor* x, const char* op,
                                             const char* const* indexes, int n_indexes,
                                             const char* const* overflow_conditions, int n_conditions,
                                             const b200jt_tensor* extras, int n_extras, void* stream) {
    IndexProgram P; int opc; RRPlan plan;
    int rc = prepare(y, x, op, indexes, n_indexes, overflow_conditions, n_conditions, extras, n_extras, &P, &opc, &plan);
    if (rc) return rc;
    if (plan.workspace > kStaticScratchBytes)
        return fail(-3, "b200jt_reindex_reduce_noalloc: this scatter needs " + std::to_string(plan.workspace) +
                        " bytes of scratch, the built-in array holds " + std::to_string(kStaticScratchBytes) +
                        "; use b200jt_reindex_reduce with a caller workspace");
    void* scratch = nullptr;
    rc = static_scratch_ptr(&scratch);
    if (rc) return rc;
    return b200jt_reindex_reduce(y, x, op, indexes, n_indexes, overflow_conditions, n_conditions, extras, n_extras,
                                 scratch, kStaticScratchBytes, stream);
}
