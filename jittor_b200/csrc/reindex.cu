// reindex: y[i] = overflow(i) ? fill : x[index(i)]  (gather; a pure data movement, bit-exact).
//
// Two kernels:
//   * affine  -- every index is c0 + sum coef*i: one thread produces VEC consecutive outputs of the
//                innermost loop axis, coordinates are unflattened once per thread and advanced
//                incrementally; stores are VEC*elem-size wide (up to 128 bit) and coalesced.
//   * generic -- the bytecode of index_program.cuh interpreted per element (div/mod, conditions,
//                @eK loads).
// The output write stream dominates traffic (the gather source is usually much smaller and L2
// resident), so both kernels are organised around coalesced output stores.
#include "index_program.cuh"
#include "reindex_jit.cuh"

namespace b200jt {

using AffineArgs = ReindexAffine;

// I = index type (32-bit arithmetic when every tensor is below 2^31 elements, as the reference's index_t).
// NL / NX are compile-time upper bounds of the two ranks: all loops over axes are fully unrolled to them (with
// uniform guards for the actual ranks) so that the coordinate arrays stay in registers.
template <typename T, typename I, int VEC, int NL, int NX>
__global__ void __launch_bounds__(256)
reindex_affine_kernel(const T* __restrict__ x, T* __restrict__ y, const __grid_constant__ AffineArgs A,
                      int64_t n_vec, T fill) {
    using U = typename std::conditional<sizeof(I) == 4, uint32_t, uint64_t>::type;
    const int nl = A.ndim_loop, nx = A.ndim_x;
    for (int64_t v = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; v < n_vec;
         v += (int64_t)gridDim.x * blockDim.x) {
        // vectors never straddle rows: the host picks VEC | innermost extent
        const int64_t flat = v * VEC;
        I iv[NL];
        U r = (U)flat;
#pragma unroll
        for (int d = NL - 1; d >= 0; d--) {
            iv[d] = 0;
            if (d < nl) { const U s = (U)A.loop_shape[d]; const U q = r / s; iv[d] = (I)(r - q * s); r = q; }
        }
        I xid[NX], xinner[NX], xs[NX];
#pragma unroll
        for (int d = 0; d < NX; d++) {
            xid[d] = 0; xinner[d] = 0; xs[d] = 1;
            if (d < nx) {
                I a = (I)A.c0[d];
#pragma unroll
                for (int j = 0; j < NL; j++)
                    if (j < nl) a += (I)A.coef[d][j] * iv[j];
                xid[d] = a; xinner[d] = (I)A.coef[d][nl - 1]; xs[d] = (I)A.x_shape[d];
            }
        }
        __align__(16) T out[VEC];
        // x offset and validity are linear in the position e inside the vector: off(e) = off0 + e*dflat, and every
        // index stays in range on an interval of e
        I off0 = 0, dflat = 0;
        int lo = 0, hi = VEC - 1;
        bool slow = false;
#pragma unroll
        for (int d = 0; d < NX; d++) {
            if (d < nx) {
                off0 = off0 * xs[d] + xid[d];
                dflat = dflat * xs[d] + xinner[d];
                if (xinner[d] == 0) { if (xid[d] < 0 || xid[d] >= xs[d]) hi = -1; }
                else if (xinner[d] == 1) { lo = max(lo, (int)min((I)VEC, -xid[d])); hi = min(hi, (int)max((I)-1, xs[d] - 1 - xid[d])); }
                else slow = true;
            }
        }
        if (!slow) {
#pragma unroll
            for (int e = 0; e < VEC; e++) out[e] = (e >= lo && e <= hi) ? x[off0 + (I)e * dflat] : fill;
        } else {
#pragma unroll
            for (int e = 0; e < VEC; e++) {
                bool over = false;
#pragma unroll
                for (int d = 0; d < NX; d++)
                    if (d < nx) { const I id = xid[d] + xinner[d] * (I)e; over |= (id < 0) | (id >= xs[d]); }
                out[e] = over ? fill : x[off0 + (I)e * dflat];
            }
        }
        if (VEC == 1) y[flat] = out[0];
        else {
            if (VEC * sizeof(T) == 16) *reinterpret_cast<uint4*>(y + flat) = *reinterpret_cast<uint4*>(out);
            else if (VEC * sizeof(T) == 8) *reinterpret_cast<uint2*>(y + flat) = *reinterpret_cast<uint2*>(out);
            else if (VEC * sizeof(T) == 4) *reinterpret_cast<uint32_t*>(y + flat) = *reinterpret_cast<uint32_t*>(out);
            else if (VEC * sizeof(T) == 2) *reinterpret_cast<uint16_t*>(y + flat) = *reinterpret_cast<uint16_t*>(out);
            else {
#pragma unroll
                for (int e = 0; e < VEC; e++) y[flat + e] = out[e];
            }
        }
    }
}

// Rows whose length is not a multiple of the vector (e.g. the 3x3 inner axes of a conv window): a thread still
// produces VEC consecutive flat outputs and one wide store, advancing the loop coordinates like an odometer.
template <typename T, int VEC, int NL, int NX>
__global__ void __launch_bounds__(256)
reindex_affine_flat_kernel(const T* __restrict__ x, T* __restrict__ y, const __grid_constant__ AffineArgs A,
                           uint32_t n_vec, T fill) {
    const int nl = A.ndim_loop, nx = A.ndim_x;
    for (uint32_t v = blockIdx.x * blockDim.x + threadIdx.x; v < n_vec; v += gridDim.x * blockDim.x) {
        const uint32_t flat = v * VEC;
        int iv[NL];
        uint32_t r = flat;
#pragma unroll
        for (int d = NL - 1; d >= 0; d--) {
            iv[d] = 0;
            if (d < nl) { const uint32_t s = (uint32_t)A.loop_shape[d]; const uint32_t q = r / s; iv[d] = (int)(r - q * s); r = q; }
        }
        __align__(16) T out[VEC];
#pragma unroll
        for (int e = 0; e < VEC; e++) {
            int off = 0; bool over = false;
#pragma unroll
            for (int d = 0; d < NX; d++) {
                if (d < nx) {
                    int a = (int)A.c0[d];
#pragma unroll
                    for (int j = 0; j < NL; j++) if (j < nl) a += (int)A.coef[d][j] * iv[j];
                    over |= (a < 0) | (a >= (int)A.x_shape[d]);
                    off = off * (int)A.x_shape[d] + a;
                }
            }
            out[e] = over ? fill : x[off];
            // odometer step
            bool carry = true;
#pragma unroll
            for (int d = NL - 1; d >= 0; d--) {
                if (d < nl && carry) { if (++iv[d] < (int)A.loop_shape[d]) carry = false; else iv[d] = 0; }
            }
        }
        if (VEC * sizeof(T) == 16) *reinterpret_cast<uint4*>(y + flat) = *reinterpret_cast<uint4*>(out);
        else *reinterpret_cast<uint2*>(y + flat) = *reinterpret_cast<uint2*>(out);
    }
}

template <typename T, int VEC>
static void launch_affine(const T* xp, T* yp, const AffineArgs& A, int64_t nv, T fill, bool small, cudaStream_t st) {
    const unsigned grid = grid_for(nv, 256);
    const int nl = A.ndim_loop, nx = A.ndim_x;
#define B200JT_AFF(NL, NX) reindex_affine_kernel<T, int32_t, VEC, NL, NX><<<grid, 256, 0, st>>>(xp, yp, A, nv, fill)
    if (!small) { reindex_affine_kernel<T, int64_t, VEC, kMaxDims, kMaxDims><<<grid, 256, 0, st>>>(xp, yp, A, nv, fill); return; }
    if (nl <= 2) { if (nx <= 2) B200JT_AFF(2, 2); else if (nx <= 4) B200JT_AFF(2, 4); else B200JT_AFF(2, kMaxDims); }
    else if (nl <= 4) { if (nx <= 2) B200JT_AFF(4, 2); else if (nx <= 4) B200JT_AFF(4, 4); else B200JT_AFF(4, kMaxDims); }
    else if (nl <= 8) { if (nx <= 2) B200JT_AFF(8, 2); else if (nx <= 4) B200JT_AFF(8, 4); else B200JT_AFF(8, kMaxDims); }
    else { if (nx <= 4) B200JT_AFF(kMaxDims, 4); else B200JT_AFF(kMaxDims, kMaxDims); }
#undef B200JT_AFF
}

template <typename T, typename I>
__global__ void __launch_bounds__(256)
reindex_generic_kernel(const T* __restrict__ x, T* __restrict__ y, const __grid_constant__ IndexProgram P,
                       int64_t n, T fill) {
    const int nl = P.ndim_loop, nx = P.ndim_x;
    for (int64_t flat = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; flat < n;
         flat += (int64_t)gridDim.x * blockDim.x) {
        I iv[kMaxDims];
        int64_t r = flat;
#pragma unroll 1
        for (int d = nl - 1; d >= 0; d--) { int64_t s = P.loop_shape[d]; iv[d] = (I)(r % s); r /= s; }
        I xid[kMaxDims];
        bool over = eval_index_program<I>(P, iv, xid);
        T v = fill;
        if (!over) {
            int64_t off = 0;
            for (int d = 0; d < nx; d++) off = off * P.x_shape[d] + (int64_t)xid[d];
            v = x[off];
        }
        y[flat] = v;
    }
}

// ---- row gather: the index program is evaluated once per run of `inner` consecutive elements ----------------------
// (x[idx[i], :] style gathers: embedding look-ups, getitem with an index Var on a leading axis). A warp takes 32 runs
// at a time: every lane interprets the program for ONE of them, then the offsets are passed around with shuffles and
// the whole warp copies each run, 16 bytes per lane when aligned.
template <typename T, typename I>
__global__ void __launch_bounds__(256)
reindex_rows_kernel(const T* __restrict__ x, T* __restrict__ y, const __grid_constant__ IndexProgram P,
                    int64_t rows, int64_t inner, T fill) {
    const int nl = P.ndim_loop - P.inner_dims, nx = P.ndim_x;
    const int lane = threadIdx.x & 31;
    const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    constexpr int V = 16 / sizeof(T);
    const bool vec_shape = inner % V == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    uint4 f;
    {
        T* fp = reinterpret_cast<T*>(&f);
#pragma unroll
        for (int e = 0; e < V; e++) fp[e] = fill;
    }
    for (int64_t row0 = warp * 32; row0 < rows; row0 += nwarps * 32) {
        const int64_t row = row0 + lane;
        long long off = -1;                                   // -1: overflow (fill), else element offset of the run in x
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
        const int64_t nv = inner / V;                       // 16-byte vectors per run
        if (vec_shape && nv <= 32 && (32 % nv) == 0) {
            // short runs (an embedding row of 64 floats is 16 vectors): the warp copies 32 / nv runs per access and keeps eight
            // accesses in flight, instead of one run per access with half of the lanes idle
            const int per = 32 / (int)nv, sub = lane / (int)nv, li = lane % (int)nv;
            constexpr int U = 8;
            for (int k0 = 0; k0 < active; k0 += per * U) {
                uint4 v[U];
                long long o[U];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int k = k0 + u * per + sub;
                    o[u] = __shfl_sync(0xffffffffu, off, k & 31);
                    if (k < active) {
                        if (o[u] >= 0 && o[u] % V == 0) v[u] = reinterpret_cast<const uint4*>(x + o[u])[li];
                        else if (o[u] < 0) v[u] = f;
                        else {                              // a run that starts off a 16-byte boundary: element by element
                            T* t = reinterpret_cast<T*>(&v[u]);
#pragma unroll
                            for (int e = 0; e < V; e++) t[e] = x[o[u] + (long long)li * V + e];
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int k = k0 + u * per + sub;
                    if (k < active) reinterpret_cast<uint4*>(y + (row0 + k) * inner)[li] = v[u];
                }
            }
            continue;
        }
        for (int k = 0; k < active; k++) {
            const long long o = __shfl_sync(0xffffffffu, off, k);
            T* dst = y + (row0 + k) * inner;
            if (vec_shape && (o < 0 || o % V == 0)) {
                const uint4* src = reinterpret_cast<const uint4*>(x + (o < 0 ? 0 : o));
                for (int64_t i = lane; i < inner / V; i += 32) reinterpret_cast<uint4*>(dst)[i] = o < 0 ? f : src[i];
            } else {
                for (int64_t i = lane; i < inner; i += 32) dst[i] = o < 0 ? fill : x[o + i];
            }
        }
    }
}

// ---- pure axis permutations (what jt.transpose lowers to) ------------------------------------------------------
// y[.., a, .., b] = x[.., b, .., a]: x is contiguous along loop axis q, y along the last loop axis. 32 x 32 tiles go
// through shared memory so that both the reads and the writes are coalesced; the other axes are a batch.
struct PermArgs {
    int32_t nbatch_dims;
    int64_t bshape[kMaxDims], bxstride[kMaxDims], bystride[kMaxDims];
    int64_t A, B;                 // extents of loop axis q and of the last loop axis
    int64_t x_sb, y_sa;           // x stride along the last loop axis, y stride along axis q
    int64_t tiles_a, tiles_b, batch;
};

template <typename T>
__global__ void __launch_bounds__(256)
reindex_permute_kernel(const T* __restrict__ x, T* __restrict__ y, const __grid_constant__ PermArgs P) {
    __shared__ T tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;      // 32 x 8
    const int64_t total = P.tiles_a * P.tiles_b * P.batch;
    for (int64_t t = blockIdx.x; t < total; t += gridDim.x) {
        const int64_t ta = t % P.tiles_a; int64_t r = t / P.tiles_a;
        const int64_t tb = r % P.tiles_b; r /= P.tiles_b;
        int64_t xb = 0, yb = 0;
#pragma unroll 1
        for (int d = P.nbatch_dims - 1; d >= 0; d--) { const int64_t i = r % P.bshape[d]; r /= P.bshape[d]; xb += i * P.bxstride[d]; yb += i * P.bystride[d]; }
        const int64_t a0 = ta * 32, b0 = tb * 32;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int64_t b = b0 + ty + k * 8, a = a0 + tx;
            if (a < P.A && b < P.B) tile[ty + k * 8][tx] = x[xb + b * P.x_sb + a];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int64_t a = a0 + ty + k * 8, b = b0 + tx;
            if (a < P.A && b < P.B) y[yb + a * P.y_sa + b] = tile[tx][ty + k * 8];
        }
        __syncthreads();
    }
}

// 4-byte elements with every extent, stride and base a multiple of 4 elements: 64 x 64 tiles, 16-byte global accesses on
// both sides (the 32 x 32 kernel moves 4 bytes per lane). Pitch 65 keeps the transposing shared-memory accesses at most
// 2-way conflicted.
__global__ void __launch_bounds__(256)
reindex_permute_vec4_kernel(const uint32_t* __restrict__ x, uint32_t* __restrict__ y, const __grid_constant__ PermArgs P) {
    __shared__ uint32_t tile[64][65];
    const int c4 = threadIdx.x & 15, r0 = threadIdx.x >> 4;     // 16 vectors per 64-element row, 16 rows per pass
    const int64_t tiles_a = (P.A + 63) / 64, tiles_b = (P.B + 63) / 64;
    const int64_t total = tiles_a * tiles_b * P.batch;
    for (int64_t t = blockIdx.x; t < total; t += gridDim.x) {
        const int64_t ta = t % tiles_a; int64_t r = t / tiles_a;
        const int64_t tb = r % tiles_b; r /= tiles_b;
        int64_t xb = 0, yb = 0;
#pragma unroll 1
        for (int d = P.nbatch_dims - 1; d >= 0; d--) { const int64_t i = r % P.bshape[d]; r /= P.bshape[d]; xb += i * P.bxstride[d]; yb += i * P.bystride[d]; }
        const int64_t a0 = ta * 64, b0 = tb * 64;
        uint4 v[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int64_t b = b0 + r0 + k * 16, a = a0 + c4 * 4;
            v[k] = (a < P.A && b < P.B) ? __ldcs(reinterpret_cast<const uint4*>(x + xb + b * P.x_sb + a)) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {
            uint32_t* row = &tile[r0 + k * 16][c4 * 4];
            row[0] = v[k].x; row[1] = v[k].y; row[2] = v[k].z; row[3] = v[k].w;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int ar = r0 + k * 16;                         // output row = input column
            const int64_t a = a0 + ar, b = b0 + c4 * 4;
            if (a < P.A && b < P.B) {
                uint4 o;
                o.x = tile[c4 * 4 + 0][ar]; o.y = tile[c4 * 4 + 1][ar]; o.z = tile[c4 * 4 + 2][ar]; o.w = tile[c4 * 4 + 3][ar];
                __stcs(reinterpret_cast<uint4*>(y + yb + a * P.y_sa + b), o);
            }
        }
        __syncthreads();
    }
}

static bool perm_vec4_ok(const PermArgs& P, const void* x, const void* y) {
    if (P.A % 4 || P.B % 4 || P.x_sb % 4 || P.y_sa % 4 || ((uintptr_t)x & 15) || ((uintptr_t)y & 15)) return false;
    for (int d = 0; d < P.nbatch_dims; d++) if (P.bxstride[d] % 4 || P.bystride[d] % 4) return false;
    return P.A >= 64 && P.B >= 64;
}

// Fills P if the program is a pure permutation whose contiguous axes differ; false otherwise.
static bool make_perm_args(const IndexProgram& Q, PermArgs* P) {
    const int n = Q.ndim_loop;
    if (!Q.is_affine || Q.ndim_x != n || n < 2) return false;
    int var_of[kMaxDims]; bool used[kMaxDims] = {false};
    for (int d = 0; d < n; d++) {
        if (Q.c0[d] != 0) return false;
        int j1 = -1;
        for (int j = 0; j < n; j++) {
            if (Q.coef[d][j] == 0) continue;
            if (Q.coef[d][j] != 1 || j1 >= 0) return false;
            j1 = j;
        }
        if (j1 < 0 || used[j1] || Q.x_shape[d] != Q.loop_shape[j1]) return false;
        used[j1] = true; var_of[d] = j1;
    }
    const int q = var_of[n - 1];
    if (q == n - 1) return false;                       // same contiguous axis: the affine kernel is already coalesced
    int64_t xs[kMaxDims], ys[kMaxDims]; int64_t st = 1;
    for (int d = n - 1; d >= 0; d--) { xs[d] = st; st *= Q.x_shape[d]; }
    st = 1;
    for (int d = n - 1; d >= 0; d--) { ys[d] = st; st *= Q.loop_shape[d]; }
    int64_t xstride_of_var[kMaxDims];
    for (int d = 0; d < n; d++) xstride_of_var[var_of[d]] = xs[d];
    memset(P, 0, sizeof(*P));
    P->A = Q.loop_shape[q]; P->B = Q.loop_shape[n - 1];
    P->x_sb = xstride_of_var[n - 1]; P->y_sa = ys[q];
    P->batch = 1;
    for (int j = 0; j < n - 1; j++) {
        if (j == q || Q.loop_shape[j] == 1) continue;
        P->bshape[P->nbatch_dims] = Q.loop_shape[j]; P->bxstride[P->nbatch_dims] = xstride_of_var[j];
        P->bystride[P->nbatch_dims] = ys[j]; P->nbatch_dims++; P->batch *= Q.loop_shape[j];
    }
    P->tiles_a = (P->A + 31) / 32; P->tiles_b = (P->B + 31) / 32;
    return true;
}

template <typename T>
static T make_fill(double v, int dtype) {
    // Tx(overflow_value) with C conversion rules (reindex_op.cc:138)
    T out;
    switch (dtype) {
        case B200JT_BOOL: { uint8_t b = v != 0; memcpy(&out, &b, sizeof(T)); break; }
        case B200JT_INT8: { int8_t b = (int8_t)(int64_t)v; memcpy(&out, &b, sizeof(T)); break; }
        case B200JT_UINT8: { uint8_t b = (uint8_t)(int64_t)v; memcpy(&out, &b, sizeof(T)); break; }
        case B200JT_INT16: { int16_t b = (int16_t)(int64_t)v; memcpy(&out, &b, sizeof(T)); break; }
        case B200JT_INT32: { int32_t b = (int32_t)(int64_t)v; memcpy(&out, &b, sizeof(T)); break; }
        case B200JT_INT64: { int64_t b = (int64_t)v; memcpy(&out, &b, sizeof(T)); break; }
        case B200JT_FLOAT16: { __half b = __float2half((float)v); memcpy(&out, &b, sizeof(T)); break; }
        case B200JT_BFLOAT16: { __nv_bfloat16 b = __float2bfloat16((float)v); memcpy(&out, &b, sizeof(T)); break; }
        case B200JT_FLOAT32: { float b = (float)v; memcpy(&out, &b, sizeof(T)); break; }
        default: { double b = v; memcpy(&out, &b, sizeof(T)); break; }
    }
    return out;
}

template <typename T>
static int launch_reindex(const b200jt_tensor* x, const b200jt_tensor* y, const IndexProgram& P,
                          double overflow_value, cudaStream_t st) {
    const int64_t n = numel(y);
    const T fill = make_fill<T>(overflow_value, x->dtype);
    const bool small = numel(x) < (1LL << 31) && n < (1LL << 31);
    const T* xp = (const T*)x->ptr;
    T* yp = (T*)y->ptr;
    const bool dry = reindex_jit_dry_running();          // source generation only: nothing may be launched
    if (dry && !(P.is_affine && numel(x) > 0 && small)) return 0;
    PermArgs PA;
    if (!dry && numel(x) > 0 && make_perm_args(P, &PA)) {
        if (sizeof(T) == 4 && perm_vec4_ok(PA, xp, yp)) {
            const int64_t total = ((PA.A + 63) / 64) * ((PA.B + 63) / 64) * PA.batch;
            const unsigned grid = (unsigned)(total < (int64_t)kNumSMs * 16 ? total : (int64_t)kNumSMs * 16);
            reindex_permute_vec4_kernel<<<grid, 256, 0, st>>>((const uint32_t*)xp, (uint32_t*)yp, PA);
            B200JT_LAUNCH_CHECK();
            return 0;
        }
        const int64_t total = PA.tiles_a * PA.tiles_b * PA.batch;
        const unsigned grid = (unsigned)(total < (int64_t)kNumSMs * 32 ? total : (int64_t)kNumSMs * 32);
        reindex_permute_kernel<T><<<grid, 256, 0, st>>>(xp, yp, PA);
        B200JT_LAUNCH_CHECK();
        return 0;
    }
    if (P.is_affine && numel(x) > 0) {
        AffineArgs A;
        memset(&A, 0, sizeof(A));
        A.ndim_loop = P.ndim_loop; A.ndim_x = P.ndim_x;
        memcpy(A.loop_shape, P.loop_shape, sizeof(A.loop_shape));
        memcpy(A.x_shape, P.x_shape, sizeof(A.x_shape));
        memcpy(A.c0, P.c0, sizeof(A.c0));
        memcpy(A.coef, P.coef, sizeof(A.coef));
        const int64_t inner = P.loop_shape[P.ndim_loop - 1];
        // one 16-byte (8-byte for 1-byte elements) output vector per thread when rows and alignment allow it
        constexpr int VMAX = 16 / sizeof(T) > 8 ? 8 : 16 / sizeof(T);
        const bool vec_ok = VMAX > 1 && inner % VMAX == 0 && ((uintptr_t)yp % (VMAX * sizeof(T))) == 0;
        const bool flat_ok = VMAX > 1 && small && n % VMAX == 0 && ((uintptr_t)yp % (VMAX * sizeof(T))) == 0 &&
                             P.ndim_loop <= 8 && P.ndim_x <= 4;
        if (small) {
            // a kernel compiled for this very op instance, when it has been seen before (reindex_jit.cu)
            const int v = (VMAX > 1 && n % VMAX == 0 && ((uintptr_t)yp % (VMAX * sizeof(T))) == 0) ? VMAX : 1;
            uint64_t fill_bits = 0;
            memcpy(&fill_bits, &fill, sizeof(T));
            const int r = reindex_jit_launch(A, (int)sizeof(T), v, xp, yp, fill_bits, st);
            if (r != kReindexJitUnavailable) return r;
        }
        if (vec_ok) launch_affine<T, VMAX>(xp, yp, A, n / VMAX, fill, small, st);
        else if (flat_ok) {
            const uint32_t nv = (uint32_t)(n / VMAX);
            reindex_affine_flat_kernel<T, VMAX, 8, 4><<<grid_for(nv, 256), 256, 0, st>>>(xp, yp, A, nv, fill);
        } else launch_affine<T, 1>(xp, yp, A, n, fill, small, st);
    } else if (P.inner_dims > 0 && P.inner_elems * (int64_t)sizeof(T) >= 64 && numel(x) > 0) {
        const int64_t rows = n / P.inner_elems;
        const unsigned grid = grid_for(rows, 256);
        if (small) reindex_rows_kernel<T, int32_t><<<grid, 256, 0, st>>>(xp, yp, P, rows, P.inner_elems, fill);
        else       reindex_rows_kernel<T, int64_t><<<grid, 256, 0, st>>>(xp, yp, P, rows, P.inner_elems, fill);
    } else {
        unsigned grid = grid_for(n, 256);
        if (small) reindex_generic_kernel<T, int32_t><<<grid, 256, 0, st>>>(xp, yp, P, n, fill);
        else       reindex_generic_kernel<T, int64_t><<<grid, 256, 0, st>>>(xp, yp, P, n, fill);
    }
    B200JT_LAUNCH_CHECK();
    return 0;
}

}  // namespace b200jt

using namespace b200jt;

extern "C" int b200jt_reindex(const b200jt_tensor* x, const b200jt_tensor* y,
                              const char* const* indexes, int n_indexes, double overflow_value,
                              const char* const* overflow_conditions, int n_conditions,
                              const b200jt_tensor* extras, int n_extras, void* stream) {
    B200JT_CHECK_ARG(valid_tensor(x) && valid_tensor(y), "invalid tensor descriptor");
    B200JT_CHECK_ARG(x->dtype == y->dtype, "x and y must have the same dtype");
    B200JT_CHECK_ARG(n_indexes == x->ndim, "Number of x's shape and indexes should be the same.");
    B200JT_CHECK_ARG(n_extras >= 0 && n_extras <= B200JT_MAX_EXTRAS, "too many extras");
    for (int k = 0; k < n_extras; k++) B200JT_CHECK_ARG(valid_tensor(&extras[k]), "invalid extras descriptor");
    if (numel(y) == 0) return 0;
    IndexProgram P;
    std::string err;
    if (!compile_index_program(y->shape, y->ndim, x->shape, x->ndim, indexes, n_indexes,
                               overflow_conditions, n_conditions, extras, n_extras, &P, &err))
        return fail(-2, "b200jt_reindex: " + err);
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype_size(x->dtype)) {
        case 1: return launch_reindex<uint8_t>(x, y, P, overflow_value, st);
        case 2: return launch_reindex<uint16_t>(x, y, P, overflow_value, st);
        case 4: return launch_reindex<uint32_t>(x, y, P, overflow_value, st);
        default: return launch_reindex<uint64_t>(x, y, P, overflow_value, st);
    }
}

/* The CUDA source the library compiles for this reindex once it has seen it twice (affine index expressions, tensors
 * below 2^31 elements), without launching anything; the pointers are only looked at for their alignment, no GPU is
 * needed. Copies at most cap bytes, NUL-terminated, into src (may be NULL), stores the full length in *needed (0 when
 * the op is not of the compiled kind) and sets *compiled to 1 if NVRTC accepted the source for sm_100a. */
extern "C" int b200jt_reindex_source(const b200jt_tensor* x, const b200jt_tensor* y, const char* const* indexes, int n_indexes,
                                     double overflow_value, const char* const* overflow_conditions, int n_conditions,
                                     const b200jt_tensor* extras, int n_extras, char* src, int64_t cap, int64_t* needed,
                                     int* compiled) {
    ReindexDryRun dry;
    reindex_jit_dry_run(&dry);
    const int rc = b200jt_reindex(x, y, indexes, n_indexes, overflow_value, overflow_conditions, n_conditions, extras, n_extras, nullptr);
    reindex_jit_dry_run(nullptr);
    if (rc != 0) return rc;
    if (needed) *needed = (int64_t)dry.source.size();
    if (src && cap > 0) {
        const size_t n = std::min((size_t)cap - 1, dry.source.size());
        memcpy(src, dry.source.data(), n); src[n] = 0;
    }
    if (compiled) *compiled = dry.compiled ? 1 : 0;
    if (!dry.source.empty() && !dry.compiled) set_error("b200jt_reindex_source: " + dry.log);
    return 0;
}
