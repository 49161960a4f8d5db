// Reindex-lowered conv2d (python/jittor/nn.py:1009-1017) as an implicit GEMM on tcgen05: bf16 in, fp32 accumulate in TMEM.
//
// The reference never materialises the 7-D window tensor; its relay is cudnnConvolutionForward
// (python/jittor/extern/cuda/cudnn/ops/cudnn_conv_op.cc:293). Here:
//   GEMM view   M = N*OH*OW output pixels, N = Cout, K = KH*KW*Cin, walked tap by tap in 64-channel blocks;
//   layout      x is first copied NCHW -> NHWC (channels innermost) and w OIHW -> [tap][Cout][Cin], so that both
//               operands are K-major and every TMA box starts at a channel offset that is a multiple of 64 (the
//               16-byte start rule); the spatial shift of a tap is carried by the H/W box coordinates, which may be
//               negative or past the edge -- TMA zero-fills, which is exactly the reindex overflow value 0;
//   tile        128 pixels (two 8x8 spatial patches, each one 4-D TMA box of 64 rows x 128 B) x 256 output channels;
//   pipeline    same persistent warp-specialised ring as the GEMM (TMA warp, MMA warp, 4 epilogue warps, TMEM
//               double buffering); strides 1..4 through the traversal stride of the x tensor map;
//   epilogue    tcgen05.ld -> bf16 -> y in NCHW; optionally per-channel sum / sum of squares of the stored values
//               (the two reduce.mean of BatchNorm, python/jittor/nn.py:674-675) accumulated per CTA in shared memory
//               and flushed with one atomicAdd per channel.
#include "gemm_simt.cuh"
#include "tc_common.cuh"

#include <mutex>

namespace b200jt {
namespace tcconv {

using namespace tc;

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int PATCH = 8;                            // spatial patch edge: 8 x 8 = 64 pixels = half a tile
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STATS_MAX_CO = 512;                   // widest layer whose statistics the epilogue can keep per CTA
constexpr int STATS_BYTES = 2 * STATS_MAX_CO * 4;
constexpr int OUT_STAGE_BYTES = 2 * 64 * 64 * 2;      // TMA-store staging: 2 patches x 64 channels x 64 pixels
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + STATS_BYTES + OUT_STAGE_BYTES;
constexpr int THREADS = 192;
constexpr double kNarrowTilePenalty = 1.5;         // measured cost per FLOP of 128-wide tiles relative to 256-wide ones (1.37 ms vs 0.92 ms)

struct ConvArgs {
    int N, C, H, W, Co, KH, KW, OH, OW, sh, sw, ph, pw, dh, dw;
    int tiles_h, tiles_w;            // patches per image
    int64_t patches;                 // N * tiles_h * tiles_w
    int tiles_m, tiles_n;
};

__device__ __forceinline__ void patch_coords(const ConvArgs& A, int64_t q, int& n, int& h0, int& w0) {
    const int per_img = A.tiles_h * A.tiles_w;
    n = (int)(q / per_img);
    const int r = (int)(q - (int64_t)n * per_img);
    h0 = (r / A.tiles_w) * PATCH;
    w0 = (r % A.tiles_w) * PATCH;
}

// OUT == 1: the epilogue stages 64 channels x 128 pixels of bf16 in shared memory ([patch][channel][8x8]) and writes
// them to y (NCHW) with two 4-D TMA box stores; edges are clipped by the tensor map. Needs OW % 8 == 0 (16-byte row
// pitch); otherwise (OUT == 0) the lanes store their values directly. OUT == 2: y is NHWC ("acdb"), a lane stores the 32
// consecutive channels of its pixel as four 16-byte vectors.
// BN_T: output channels per tile (256, or 128 when that fills the last wave of the persistent grid better; the
// shared-memory ring keeps the 256-channel stage size either way).
template <int OUT, int BN_T>
__global__ void __launch_bounds__(THREADS, 1)
conv_bf16_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_y,
                 __nv_bfloat16* __restrict__ y, float* __restrict__ stats, const __grid_constant__ ConvArgs A) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* acc_full = bars + 2 * STAGES;
    uint64_t* acc_empty = bars + 2 * STAGES + 2;
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    float* sstat = (float*)(smem + STAGES * STAGE_BYTES + 256);      // [2][STATS_MAX_CO] per-CTA channel sums
    unsigned char* stage_out = smem + STAGES * STAGE_BYTES + 256 + STATS_BYTES;   // [2 patches][64 ch][64 px] bf16
    constexpr bool TMA_OUT = OUT == 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total = A.tiles_m * A.tiles_n;
    const int cblocks = (A.C + BK - 1) / BK;
    const int k_blocks = A.KH * A.KW * cblocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        for (int b = 0; b < 2; b++) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = threadIdx.x; i < 2 * STATS_MAX_CO; i += blockDim.x) sstat[i] = 0.f;
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                const int tm = t / A.tiles_n, tn = t - tm * A.tiles_n;
                int n0, h0, w0, n1, h1, w1;
                patch_coords(A, 2 * (int64_t)tm, n0, h0, w0);
                patch_coords(A, 2 * (int64_t)tm + 1, n1, h1, w1);       // past the last patch: n1 >= N, zero-filled
                for (int kb = 0; kb < k_blocks; kb++) {
                    const int tap = kb / cblocks, cb = kb - tap * cblocks;
                    const int kh = tap / A.KW, kw = tap - kh * A.KW;
                    const int dy = kh * A.dh - A.ph, dx = kw * A.dw - A.pw;
                    if (!(ok = mbar_wait(empty + stage, phase ^ 1, abort_flag, 11))) break;
                    unsigned char* sa = smem + stage * STAGE_BYTES;
                    mbar_expect_tx(full + stage, A_BYTES + BN_T * BK * 2);
                    // a box covers 8 x 8 OUTPUT pixels: with stride s the tensor map steps s input elements per box element
                    tma_load_4d(sa, &map_x, full + stage, cb * BK, w0 * A.sw + dx, h0 * A.sh + dy, n0);
                    tma_load_4d(sa + A_BYTES / 2, &map_x, full + stage, cb * BK, w1 * A.sw + dx, h1 * A.sh + dy, n1);
                    tma_load_2d(sa + A_BYTES, &map_w, full + stage, cb * BK, tap * A.Co + tn * BN_T);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                for (int s = 0; s < STAGES; s++)
                    for (uint32_t i = 0; i < 4096 && !mbar_try(full + s, 0) && !mbar_try(full + s, 1); i++) __nanosleep(64);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN_T);
            int stage = 0; uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x, it++) {
                const int buf = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!(ok = mbar_wait(acc_empty + buf, acc_phase ^ 1, abort_flag, 12))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = 0; kb < k_blocks; kb++) {
                    if (!(ok = mbar_wait(full + stage, phase, abort_flag, 13))) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
                    const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) umma_f16(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    umma_commit(empty + stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit(acc_full + buf);
            }
        }
    } else {
        const int quad = warp & 3;
        int it = 0;
        bool ok = true;
        const int64_t plane = (int64_t)A.OH * A.OW;
        for (int t = blockIdx.x; t < total && ok; t += gridDim.x, it++) {
            const int tm = t / A.tiles_n, tn = t - tm * A.tiles_n;
            const int buf = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            ok = mbar_wait(acc_full + buf, acc_phase, abort_flag, 14);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // this lane's pixel: row r of the tile = patch (r / 64), position (r % 64) = hh*8 + ww
            const int r = quad * 32 + lane;
            const int64_t q = 2 * (int64_t)tm + (r >> 6);
            int n, h0, w0;
            patch_coords(A, q, n, h0, w0);
            const int oh = h0 + ((r & 63) >> 3), ow = w0 + (r & 7);
            const bool valid = q < A.patches && oh < A.OH && ow < A.OW;
            __nv_bfloat16* yp = y + ((int64_t)n * A.Co) * plane + (int64_t)oh * A.OW + ow;
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BN;
            const bool issuer = threadIdx.x == 64;          // first epilogue thread drives the TMA stores
#pragma unroll 1
            for (int ch = 0; ch < BN_T / 32; ch++) {
                const int co0 = tn * BN_T + ch * 32;
                if (TMA_OUT && (ch & 1) == 0) {
                    // staging buffer free again? (the previous round's stores must have read it)
                    if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                }
                uint32_t v[32];
                tmem_ld32(taddr + ch * 32, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                float f[32];
                if (TMA_OUT) {
                    __nv_bfloat16* sp = reinterpret_cast<__nv_bfloat16*>(stage_out) + (r >> 6) * (64 * 64) + (ch & 1) * (32 * 64) + (r & 63);
#pragma unroll
                    for (int e = 0; e < 32; e++) {
                        const __nv_bfloat16 b = __float2bfloat16(__uint_as_float(v[e]));
                        sp[e * 64] = b;
                        f[e] = (valid && co0 + e < A.Co) ? __bfloat162float(b) : 0.f;
                    }
                } else if (OUT == 2) {
                    // NHWC: this lane's pixel, channels co0 .. co0 + 31 are contiguous
                    __align__(16) __nv_bfloat16 row[32];
#pragma unroll
                    for (int e = 0; e < 32; e++) {
                        row[e] = __float2bfloat16(__uint_as_float(v[e]));
                        f[e] = (valid && co0 + e < A.Co) ? __bfloat162float(row[e]) : 0.f;
                    }
                    if (valid) {
                        __nv_bfloat16* yq = y + (((int64_t)n * A.OH + oh) * A.OW + ow) * A.Co + co0;
                        if (co0 + 32 <= A.Co && (A.Co & 7) == 0) {
#pragma unroll
                            for (int q = 0; q < 4; q++) reinterpret_cast<uint4*>(yq)[q] = reinterpret_cast<const uint4*>(row)[q];
                        } else {
#pragma unroll
                            for (int e = 0; e < 32; e++) if (co0 + e < A.Co) yq[e] = row[e];
                        }
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 32; e++) {
                        const __nv_bfloat16 b = __float2bfloat16(__uint_as_float(v[e]));
                        const bool st = valid && co0 + e < A.Co;
                        if (st) yp[(int64_t)(co0 + e) * plane] = b;
                        f[e] = st ? __bfloat162float(b) : 0.f;      // statistics of the value as stored
                    }
                }
                if (stats) {
                    // lanes are 32 pixels, f[] 32 channels: halving exchange leaves lane L with the sum of channel L
                    float g[32];
#pragma unroll
                    for (int e = 0; e < 32; e++) g[e] = f[e] * f[e];
#pragma unroll
                    for (int s = 16; s > 0; s >>= 1) {
                        const bool up = (lane & s) != 0;
#pragma unroll
                        for (int i = 0; i < s; i++) {
                            const float keep = up ? f[i + s] : f[i], send = up ? f[i] : f[i + s];
                            f[i] = keep + __shfl_xor_sync(0xffffffffu, send, s);
                            const float keep2 = up ? g[i + s] : g[i], send2 = up ? g[i] : g[i + s];
                            g[i] = keep2 + __shfl_xor_sync(0xffffffffu, send2, s);
                        }
                    }
                    if (co0 + lane < A.Co) {
                        atomicAdd(sstat + co0 + lane, f[0]);
                        atomicAdd(sstat + STATS_MAX_CO + co0 + lane, g[0]);
                    }
                }
                if (TMA_OUT && (ch & 1) == 1) {
                    // 64 channels staged: make the writes visible to the async proxy, then two box stores
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (issuer) {
                        const int cbase = tn * BN_T + (ch - 1) * 32;
#pragma unroll
                        for (int pp = 0; pp < 2; pp++) {
                            const int64_t qq = 2 * (int64_t)tm + pp;
                            if (qq < A.patches && cbase < A.Co) {
                                int nn, hh0, ww0;
                                patch_coords(A, qq, nn, hh0, ww0);
                                asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                                             ::"l"(&map_y), "r"(smem_u32(stage_out + pp * (64 * 64 * 2))), "r"(ww0), "r"(hh0), "r"(cbase), "r"(nn) : "memory");
                            }
                        }
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + buf);
        }
        if (TMA_OUT && threadIdx.x == 64) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (stats) {
        for (int i = threadIdx.x; i < A.Co; i += blockDim.x) {
            atomicAdd(stats + i, sstat[i]);
            atomicAdd(stats + A.Co + i, sstat[STATS_MAX_CO + i]);
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

// ---- layout passes -----------------------------------------------------------------------------------------
// in[b][R][Cn] -> out[b][Cn][R] (bf16), 64x64 tiles, 16-byte global accesses on both sides. The tile is kept as
// 32-bit pairs with an odd pitch (33 words) so that the column reads of the second phase spread over the banks.
// Block (0,0,0) also zeroes `zero[0..n_zero)`. The first wz slices (blockIdx.z < wz) of the same grid re-order the weights instead (w[Co][C][taps] -> wt[taps][Co][C]), so
// that both layout passes of a convolution are one launch.
__global__ void __launch_bounds__(256)
transpose_bf16_batched_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int R, int Cn, int wz,
                              const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ wt, int Co, int C, int taps,
                              float* __restrict__ zero, int n_zero, int w_ohwi) {
    __shared__ __nv_bfloat16 tile[64][66];
    if (zero && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0)       // the statistics the conv epilogue adds into
        for (int i = threadIdx.x; i < n_zero; i += blockDim.x) zero[i] = 0.f;
    if ((int)blockIdx.z < wz) {
        const int64_t n = (int64_t)Co * C * taps;
        const int64_t nblk = (int64_t)gridDim.x * gridDim.y * wz;
        const int64_t blk = ((int64_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
        for (int64_t i = blk * blockDim.x + threadIdx.x; i < n; i += nblk * blockDim.x) {
            const int c = (int)(i % C); const int64_t t2 = i / C;
            const int co = (int)(t2 % Co); const int tap = (int)(t2 / Co);
            wt[i] = w_ohwi ? w[((int64_t)co * taps + tap) * C + c] : w[((int64_t)co * C + c) * taps + tap];
        }
        return;
    }
    const int64_t boff = (int64_t)((int)blockIdx.z - wz) * R * Cn;
    const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    const int j = threadIdx.x & 7, i = threadIdx.x >> 3;          // 8 chunks of 8 elements x 32 rows
    const bool vec_in = (Cn % 8 == 0), vec_out = (R % 8 == 0);
#pragma unroll
    for (int p = 0; p < 2; p++) {
        const int r = r0 + i + p * 32, c = c0 + j * 8;
        __align__(16) __nv_bfloat16 v[8];
        if (r < R && vec_in && c + 8 <= Cn) *reinterpret_cast<uint4*>(v) = __ldcs(reinterpret_cast<const uint4*>(in + boff + (int64_t)r * Cn + c));
        else {
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = (r < R && c + e < Cn) ? in[boff + (int64_t)r * Cn + c + e] : __float2bfloat16(0.f);
        }
        uint32_t* row = reinterpret_cast<uint32_t*>(&tile[i + p * 32][0]);
#pragma unroll
        for (int e = 0; e < 4; e++) row[j * 4 + e] = reinterpret_cast<const uint32_t*>(v)[e];
    }
    __syncthreads();
#pragma unroll
    for (int p = 0; p < 2; p++) {
        const int c = c0 + i + p * 32, r = r0 + j * 8;           // output row = input column
        if (c >= Cn) continue;
        __align__(16) __nv_bfloat16 v[8];
#pragma unroll
        for (int e = 0; e < 8; e++) v[e] = tile[j * 8 + e][i + p * 32];
        if (vec_out && r + 8 <= R) __stcs(reinterpret_cast<uint4*>(out + boff + (int64_t)c * R + r), *reinterpret_cast<uint4*>(v));
        else {
            for (int e = 0; e < 8 && r + e < R; e++) out[boff + (int64_t)c * R + r + e] = v[e];
        }
    }
}

static bool make_map_x(CUtensorMap* map, const void* base, const ConvShape& s) {
    auto fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[4] = {(cuuint64_t)s.C, (cuuint64_t)s.W, (cuuint64_t)s.H, (cuuint64_t)s.N};
    cuuint64_t strides[3] = {(cuuint64_t)s.C * 2, (cuuint64_t)s.W * s.C * 2, (cuuint64_t)s.H * s.W * s.C * 2};
    // strided convolution: the traversal stride of the map skips input pixels, so that a box still delivers 8 x 8 window
    // origins; the box extent counts tensor elements, i.e. 8 * stride per axis (at most 8 * 8 = 64 <= 256)
    cuuint32_t box[4] = {(cuuint32_t)BK, (cuuint32_t)(PATCH * s.sw), (cuuint32_t)(PATCH * s.sh), 1};
    cuuint32_t estr[4] = {1, (cuuint32_t)s.sw, (cuuint32_t)s.sh, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
static bool make_map_w(CUtensorMap* map, const void* base, const ConvShape& s, int bn) {
    auto fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)s.C, (cuuint64_t)s.Co * s.KH * s.KW};
    cuuint64_t strides[1] = {(cuuint64_t)s.C * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)bn};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool make_map_y(CUtensorMap* map, const void* base, const ConvShape& s) {
    auto fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[4] = {(cuuint64_t)s.OW, (cuuint64_t)s.OH, (cuuint64_t)s.Co, (cuuint64_t)s.N};
    cuuint64_t strides[3] = {(cuuint64_t)s.OW * 2, (cuuint64_t)s.OH * s.OW * 2, (cuuint64_t)s.Co * s.OH * s.OW * 2};
    cuuint32_t box[4] = {PATCH, PATCH, 64, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tcconv

bool conv2d_tc_supported(const ConvShape& s, const void* x, const void* w, const void* y) {
    return s.sh >= 1 && s.sh <= 4 && s.sw >= 1 && s.sw <= 4 && s.C % 8 == 0 && s.C >= 64 && s.Co >= 64 && s.H >= 8 && s.W >= 8 &&
           (int64_t)s.N * s.OH * s.OW >= 1024 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 2 == 0) &&
           ((uintptr_t)y % 2 == 0) && tc::encode_fn() != nullptr;
}

size_t conv2d_tc_workspace(const ConvShape& s) {
    const size_t xb = ((size_t)s.N * s.H * s.W * s.C * 2 + 1023) & ~(size_t)1023;
    const size_t wb = ((size_t)s.Co * s.C * s.KH * s.KW * 2 + 1023) & ~(size_t)1023;
    return xb + wb + 1024;
}

int conv2d_tc(const void* x, const void* w, void* y, float* stats, const ConvShape& s, void* workspace, cudaStream_t st,
              const ConvLayout& lay) {
    using namespace tcconv;
    unsigned char* ws = (unsigned char*)(((uintptr_t)workspace + 1023) & ~(uintptr_t)1023);
    // NHWC ("acdb") activations are what the kernel reads: no staging pass for x then
    __nv_bfloat16* xt = lay.x_nhwc ? (__nv_bfloat16*)const_cast<void*>(x) : (__nv_bfloat16*)ws;
    __nv_bfloat16* wt = (__nv_bfloat16*)(ws + (((size_t)s.N * s.H * s.W * s.C * 2 + 1023) & ~(size_t)1023));
    const int HW = s.H * s.W;
    {   // x[N][C][HW] -> xt[N][HW][C], and the weights tap-major, in one launch
        const int64_t nw = (int64_t)s.Co * s.C * s.KH * s.KW;
        const unsigned gx = (unsigned)((HW + 63) / 64), gy = (unsigned)((s.C + 63) / 64);
        const int64_t per_slice = (int64_t)gx * gy * 256;
        const unsigned wz = (unsigned)std::min<int64_t>(32, std::max<int64_t>(1, (nw + per_slice - 1) / per_slice));
        dim3 g(gx, gy, (lay.x_nhwc ? 0u : (unsigned)s.N) + wz);          // the first wz slices re-order the weights
        float* zero = (stats && s.Co <= STATS_MAX_CO) ? stats : nullptr;   // zeroed here instead of by a memset node
        transpose_bf16_batched_kernel<<<g, 256, 0, st>>>((const __nv_bfloat16*)x, xt, s.C, HW, (int)wz,
                                                          (const __nv_bfloat16*)w, wt, s.Co, s.C, s.KH * s.KW, zero, 2 * s.Co, lay.w_ohwi ? 1 : 0);
        B200JT_LAUNCH_CHECK();
    }
    ConvArgs A;
    A.N = s.N; A.C = s.C; A.H = s.H; A.W = s.W; A.Co = s.Co; A.KH = s.KH; A.KW = s.KW; A.OH = s.OH; A.OW = s.OW;
    A.sh = s.sh; A.sw = s.sw; A.ph = s.ph; A.pw = s.pw; A.dh = s.dh; A.dw = s.dw;
    A.tiles_h = (s.OH + PATCH - 1) / PATCH; A.tiles_w = (s.OW + PATCH - 1) / PATCH;
    A.patches = (int64_t)s.N * A.tiles_h * A.tiles_w;
    A.tiles_m = (int)((A.patches + 1) / 2);
    // Tile width: the grid is persistent with a static round-robin, so its time is ceil(tiles / SMs) rounds. 128-wide
    // tiles do a little worse per FLOP (more operand bytes per MMA) but halve the granularity of the last round.
    auto rounds = [&](int bn) { const int64_t t = (int64_t)A.tiles_m * ((s.Co + bn - 1) / bn); return (double)((t + kNumSMs - 1) / kNumSMs) * bn; };
    const char* bn_env = getenv("B200JT_CONV_BN");          // read on every call: tests force each variant in turn
    const int forced_bn = bn_env ? atoi(bn_env) : 0;
    const int bn = forced_bn == 128 || forced_bn == 256 ? forced_bn : (rounds(128) * kNarrowTilePenalty < rounds(256) ? 128 : 256);
    A.tiles_n = (s.Co + bn - 1) / bn;
    CUtensorMap mx, mw;
    if (!make_map_x(&mx, xt, s) || !make_map_w(&mw, wt, s, bn)) return fail(-4, "conv2d: cuTensorMapEncodeTiled failed");
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        const void* kernels[] = {(const void*)conv_bf16_kernel<1, 256>, (const void*)conv_bf16_kernel<0, 256>,
                                 (const void*)conv_bf16_kernel<1, 128>, (const void*)conv_bf16_kernel<0, 128>,
                                 (const void*)conv_bf16_kernel<2, 256>, (const void*)conv_bf16_kernel<2, 128>};
        for (const void* k : kernels)
            if (attr_err == cudaSuccess) attr_err = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    });
    B200JT_CUDA(attr_err);
    // TMA stores need a 16-byte aligned base and row pitch
    const bool tma_out = !lay.y_nhwc && (s.OW % 8 == 0) && ((uintptr_t)y % 16 == 0);
    CUtensorMap my = mx;
    if (tma_out && !make_map_y(&my, y, s)) return fail(-4, "conv2d: cuTensorMapEncodeTiled failed (y)");
    float* fused = (stats && s.Co <= STATS_MAX_CO) ? stats : nullptr;
    const int total = A.tiles_m * A.tiles_n;
    const int grid = total < kNumSMs ? total : kNumSMs;
    auto kern = bn == 256 ? (lay.y_nhwc ? conv_bf16_kernel<2, 256> : tma_out ? conv_bf16_kernel<1, 256> : conv_bf16_kernel<0, 256>)
                          : (lay.y_nhwc ? conv_bf16_kernel<2, 128> : tma_out ? conv_bf16_kernel<1, 128> : conv_bf16_kernel<0, 128>);
    kern<<<grid, THREADS, SMEM_BYTES, st>>>(mx, mw, my, (__nv_bfloat16*)y, fused, A);
    B200JT_LAUNCH_CHECK();
    return fused ? 1 : 0;      // 1: statistics were produced by the epilogue
}

// ---- weight gradient ---------------------------------------------------------------------------------------
// dw[o,c,kh,kw] = sum over (n,oh,ow) of dy[n,o,oh,ow] * x[n,c,oh*stride-pad+kh*dil, ow*stride-pad+kw*dil]: the reduce.add
// over (batch, rows, columns) of reindex(x) * broadcast(dy) that ConvTuner relays to cudnnConvolutionBackwardFilter
// (python/jittor/extern/cuda/cudnn/ops/cudnn_conv_backward_w_op.cc:292). As a GEMM per filter tap:
//   D[c, o] = sum over pixels of X_tap[pixel, c] * DY[pixel, o],     M = Cin (128 per CTA), N = Cout (256), K = N*OH*OW.
// x and dy are first copied to NHWC, so a 4-D TMA box of 8 x 8 output pixels x 64 channels lands as 64 rows of 128 B with
// the channel axis contiguous: both operands are MN-major (their own axis contiguous, K = pixel strided), and the same box
// geometry as the forward kernel carries the tap's shift and the stride in its coordinates. One CTA owns one
// (tap, 128 input channels, 256 output channels) accumulator in TMEM and walks a contiguous range of pixel patches; the
// K axis is split over `splits` CTAs per accumulator to fill the GPU, each writing fp32 partial sums that a second kernel
// adds in split order (deterministic) and stores as bf16 in OIHW order.
namespace tcwgrad {

using namespace tc;

constexpr int BM = 128, PIX = 64, PATCH = 8, THREADS = 192;
constexpr int CHUNK_BYTES = PIX * 64 * 2;                    // one box: 64 pixels x 64 channels of bf16
// TAPS filter taps per CTA share the dy tile of a stage (their x tiles differ by the tap's shift): with two taps a stage is
// 2 * 16 KB of x + 32 KB of dy for twice the MMAs, i.e. two thirds of the operand bytes per FLOP -- the feed from L2 into
// shared memory is what bounds the one-tap form. Two accumulators fill the 512 TMEM columns; three 64 KB stages.
template <int TAPS> struct Ring {
    static constexpr int STAGES = TAPS == 2 ? 3 : 4;
    static constexpr int MAX_STAGE_BYTES = (TAPS * (BM / 64) + 256 / 64) * CHUNK_BYTES;
    static constexpr int SMEM_BYTES = STAGES * MAX_STAGE_BYTES + 1024 + 256;
};

struct WgradArgs {
    int N, C, H, W, Co, KH, KW, OH, OW, sh, sw, ph, pw, dh, dw;
    int tiles_h, tiles_w;            // patches per image
    int64_t patches;                 // N * tiles_h * tiles_w: the K axis in units of 64 pixels
    int tiles_m, tiles_n, splits, groups;      // groups: ceil(taps / TAPS) tap groups
};

template <int BN_T, int TAPS>
__global__ void __launch_bounds__(THREADS, 1)
wgrad_bf16_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_dy,
                  float* __restrict__ part, const __grid_constant__ WgradArgs A) {
    constexpr int STAGES = Ring<TAPS>::STAGES, MAX_STAGE_BYTES = Ring<TAPS>::MAX_STAGE_BYTES;
    constexpr int XBOX = BM / 64, YBOX = BN_T / 64;           // boxes per tap of x, boxes of dy
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + STAGES * MAX_STAGE_BYTES);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* acc_full = bars + 2 * STAGES;
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int taps = A.KH * A.KW;
    const int base = A.groups * A.tiles_m * A.tiles_n;
    const int split = blockIdx.x / base;
    int tile = blockIdx.x - split * base;
    const int group = tile % A.groups; tile /= A.groups;
    const int tn = tile % A.tiles_n, tm = tile / A.tiles_n;
    const int tap0 = group * TAPS;
    const int ntap = min(TAPS, taps - tap0);                 // the last group of an odd tap count holds one tap
    const int64_t p0 = A.patches * split / A.splits, p1 = A.patches * (split + 1) / A.splits;
    const int k_blocks = (int)(p1 - p0);                     // >= 1: the host keeps splits <= patches

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(TAPS * BN_T) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // The whole warp walks the patches; lane 0 waits for the slot and announces the bytes, then every lane that owns a box
        // issues it: chunk j of a stage belongs to lane j -- x chunks of tap 0, x chunks of tap 1, then the dy chunks.
        const bool is_x = lane < TAPS * XBOX;
        const int t = is_x ? lane / XBOX : 0;                 // which of this CTA's taps the lane's x box serves
        const int tap = min(tap0 + t, taps - 1);
        const int kh = tap / A.KW, kw = tap - kh * A.KW;
        const int per_img = A.tiles_h * A.tiles_w;
        int n = (int)(p0 / per_img);
        const int r0 = (int)(p0 - (int64_t)n * per_img);
        int th = r0 / A.tiles_w, tw = r0 - th * A.tiles_w;
        const bool owns = is_x ? t < ntap : lane < TAPS * XBOX + YBOX;
        const CUtensorMap* map = is_x ? &map_x : &map_dy;
        const int c0 = is_x ? tm * BM + (lane - t * XBOX) * 64 : tn * BN_T + (lane - TAPS * XBOX) * 64;
        const int sw = is_x ? A.sw : 1, sh = is_x ? A.sh : 1;
        const int ox = is_x ? kw * A.dw - A.pw : 0, oy = is_x ? kh * A.dh - A.ph : 0;
        const uint32_t stage_bytes = (uint32_t)(ntap * XBOX + YBOX) * CHUNK_BYTES;
        int stage = 0; uint32_t phase = 0;
        bool ok = true;
        for (int kb = 0; kb < k_blocks; kb++) {
            if (lane == 0) {
                ok = mbar_wait(empty + stage, phase ^ 1, abort_flag, 21);
                if (ok) mbar_expect_tx(full + stage, stage_bytes);
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            // pixels past the edge of x (padding, ragged patches) and channels past C / Co are zero-filled by TMA
            if (owns)
                tma_load_4d(smem + stage * MAX_STAGE_BYTES + lane * CHUNK_BYTES, map, full + stage, c0,
                            tw * PATCH * sw + ox, th * PATCH * sh + oy, n);
            if (++tw == A.tiles_w) { tw = 0; if (++th == A.tiles_h) { th = 0; n++; } }
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok && lane == 0) {
            for (int s = 0; s < STAGES; s++)
                for (uint32_t i = 0; i < 4096 && !mbar_try(full + s, 0) && !mbar_try(full + s, 1); i++) __nanosleep(64);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN_T, true) | (1u << 15);      // A and B both MN-major
            constexpr int KSTEP = (UMMA_K * 128) / 16;                                // 16 pixel rows of 128 B, in 16-byte units
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int kb = 0; kb < k_blocks; kb++) {
                if (!(ok = mbar_wait(full + stage, phase, abort_flag, 22))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t sa = smem_u32(smem + stage * MAX_STAGE_BYTES);
                const uint64_t db = make_smem_desc_mn(sa + TAPS * XBOX * CHUNK_BYTES, CHUNK_BYTES, 1024);
#pragma unroll
                for (int t = 0; t < TAPS; t++) {
                    if (t < ntap) {
                        const uint64_t da = make_smem_desc_mn(sa + t * XBOX * CHUNK_BYTES, CHUNK_BYTES, 1024);
#pragma unroll
                        for (int k = 0; k < PIX / UMMA_K; k++)
                            umma_f16(tmem_base + t * BN_T, da + KSTEP * k, db + KSTEP * k, idesc, (kb | k) != 0);
                    }
                }
                umma_commit(empty + stage);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
            if (ok) umma_commit(acc_full);
        }
    } else {
        const int quad = warp & 3;
        bool ok = mbar_wait(acc_full, 0, abort_flag, 23);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int c = tm * BM + quad * 32 + lane;                        // TMEM lane = input channel
            const bool vec = (A.Co & 3) == 0;
            for (int t = 0; t < ntap; t++) {
                const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + t * BN_T;
                float* prow = part + (((int64_t)split * taps + tap0 + t) * A.C + c) * A.Co;
#pragma unroll 1
                for (int ch = 0; ch < BN_T / 32; ch++) {
                    uint32_t v[32];
                    tmem_ld32(taddr + ch * 32, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    const int o0 = tn * BN_T + ch * 32;
                    if (c < A.C && o0 < A.Co) {
                        if (vec && o0 + 32 <= A.Co) {
#pragma unroll
                            for (int q = 0; q < 8; q++)
                                *reinterpret_cast<uint4*>(prow + o0 + q * 4) = make_uint4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
                        } else {
#pragma unroll
                            for (int e = 0; e < 32; e++) if (o0 + e < A.Co) prow[o0 + e] = __uint_as_float(v[e]);
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(TAPS * BN_T) : "memory");
    }
}

// dw[o][c][tap] (or [o][tap][c] for the "ohwi" layout) = sum over splits (ascending) of part[split][tap][c][o], rounded to bf16 once.
__global__ void __launch_bounds__(256)
wgrad_fold_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ dw, int splits, int taps, int C, int Co, int ohwi) {
    const int64_t n = (int64_t)taps * C * Co;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int o = (int)(i % Co); const int64_t t = i / Co;
        const int c = (int)(t % C); const int tap = (int)(t / C);
        float acc = 0.f;
        for (int s = 0; s < splits; s++) acc += part[(int64_t)s * n + i];
        dw[ohwi ? ((int64_t)o * taps + tap) * C + c : ((int64_t)o * C + c) * taps + tap] = __float2bfloat16(acc);
    }
}

// NHWC tensor [N][H][W][C] as a 4-D map whose box is 64 channels x (8 * sw) x (8 * sh) x 1 with traversal strides
// (1, sw, sh, 1): 64 pixels x 128 B in shared memory.
static bool make_map_nhwc(CUtensorMap* map, const void* base, int N, int H, int W, int C, int sh, int sw) {
    auto fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
    cuuint64_t strides[3] = {(cuuint64_t)C * 2, (cuuint64_t)W * C * 2, (cuuint64_t)H * W * C * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)(PATCH * sw), (cuuint32_t)(PATCH * sh), 1};
    cuuint32_t estr[4] = {1, (cuuint32_t)sw, (cuuint32_t)sh, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct Plan { int bn, taps_per_cta, groups, tiles_m, tiles_n, splits; int64_t patches; size_t xb, dyb, pb; };

static Plan plan_for(const ConvShape& s) {
    Plan p;
    const int taps = s.KH * s.KW;
    const char* env = getenv("B200JT_WGRAD_TAPS");           // 1 forces one tap per CTA (tests run both forms)
    p.bn = s.Co <= 128 ? 128 : 256;
    p.taps_per_cta = (taps >= 2 && !(env && atoi(env) == 1)) ? 2 : 1;
    p.groups = (taps + p.taps_per_cta - 1) / p.taps_per_cta;
    p.tiles_m = (s.C + BM - 1) / BM;
    p.tiles_n = (s.Co + p.bn - 1) / p.bn;
    p.patches = (int64_t)s.N * ((s.OH + PATCH - 1) / PATCH) * ((s.OW + PATCH - 1) / PATCH);
    // fill the GPU once when the accumulators alone do not; every split keeps at least 16 patches (1024 pixels) of K
    auto splits_for = [&](int64_t groups) {
        const int64_t base = groups * p.tiles_m * p.tiles_n;
        return std::max<int64_t>(1, std::min<int64_t>(base >= kNumSMs ? 1 : kNumSMs / base, p.patches / 16));
    };
    p.splits = (int)splits_for(p.groups);
    p.xb = ((size_t)s.N * s.H * s.W * s.C * 2 + 1023) & ~(size_t)1023;
    p.dyb = ((size_t)s.N * s.OH * s.OW * s.Co * 2 + 1023) & ~(size_t)1023;
    // the partial sums are sized for whichever form splits K more finely, so the workspace query does not depend on the switch
    const int64_t most = std::max(splits_for(taps), splits_for((taps + 1) / 2));
    p.pb = ((size_t)most * taps * s.C * s.Co * 4 + 1023) & ~(size_t)1023;
    return p;
}

}  // namespace tcwgrad

bool conv2d_wgrad_tc_supported(const ConvShape& s, const void* x, const void* dy, const void* dw) {
    const int64_t taps = (int64_t)s.KH * s.KW;
    return s.groups == 1 && s.sh >= 1 && s.sh <= 4 && s.sw >= 1 && s.sw <= 4 && s.C % 8 == 0 && s.Co % 8 == 0 && s.C >= 64 &&
           s.Co >= 64 && s.H >= 8 * s.sh && s.W >= 8 * s.sw && s.OH >= 8 && s.OW >= 8 && (int64_t)s.N * s.OH * s.OW >= 4096 &&
           taps * ((s.C + 127) / 128) * ((s.Co + 255) / 256) <= (1 << 20) &&
           ((uintptr_t)x % 16 == 0) && ((uintptr_t)dy % 16 == 0) && ((uintptr_t)dw % 2 == 0) && tc::encode_fn() != nullptr;
}

size_t conv2d_wgrad_tc_workspace(const ConvShape& s) {
    const tcwgrad::Plan p = tcwgrad::plan_for(s);
    return p.xb + p.dyb + p.pb + 1024;
}

int conv2d_wgrad_tc(const void* x, const void* dy, void* dw, const ConvShape& s, void* workspace, cudaStream_t st,
                    const ConvLayout& lay) {
    using namespace tcwgrad;
    const Plan p = plan_for(s);
    unsigned char* ws = (unsigned char*)(((uintptr_t)workspace + 1023) & ~(uintptr_t)1023);
    // channels-last ("acdb") x / dy are what the kernel reads: no copy on that side (lay.y_nhwc describes dy)
    __nv_bfloat16* xt = lay.x_nhwc ? (__nv_bfloat16*)const_cast<void*>(x) : (__nv_bfloat16*)ws;
    __nv_bfloat16* dyt = lay.y_nhwc ? (__nv_bfloat16*)const_cast<void*>(dy) : (__nv_bfloat16*)(ws + p.xb);
    float* part = (float*)(ws + p.xb + p.dyb);
    const int HW = s.H * s.W, OHW = s.OH * s.OW;
    if (!lay.x_nhwc) {   // x[N][C][HW] -> [N][HW][C]
        dim3 gx((unsigned)((HW + 63) / 64), (unsigned)((s.C + 63) / 64), (unsigned)s.N);
        tcconv::transpose_bf16_batched_kernel<<<gx, 256, 0, st>>>((const __nv_bfloat16*)x, xt, s.C, HW, 0, nullptr, nullptr, 0, 0, 0, nullptr, 0, 0);
        B200JT_LAUNCH_CHECK();
    }
    if (!lay.y_nhwc) {   // dy[N][Co][OH*OW] -> [N][OH*OW][Co]
        dim3 gy((unsigned)((OHW + 63) / 64), (unsigned)((s.Co + 63) / 64), (unsigned)s.N);
        tcconv::transpose_bf16_batched_kernel<<<gy, 256, 0, st>>>((const __nv_bfloat16*)dy, dyt, s.Co, OHW, 0, nullptr, nullptr, 0, 0, 0, nullptr, 0, 0);
        B200JT_LAUNCH_CHECK();
    }
    WgradArgs A;
    A.N = s.N; A.C = s.C; A.H = s.H; A.W = s.W; A.Co = s.Co; A.KH = s.KH; A.KW = s.KW; A.OH = s.OH; A.OW = s.OW;
    A.sh = s.sh; A.sw = s.sw; A.ph = s.ph; A.pw = s.pw; A.dh = s.dh; A.dw = s.dw;
    A.tiles_h = (s.OH + PATCH - 1) / PATCH; A.tiles_w = (s.OW + PATCH - 1) / PATCH;
    A.patches = p.patches; A.tiles_m = p.tiles_m; A.tiles_n = p.tiles_n; A.splits = p.splits; A.groups = p.groups;
    CUtensorMap mx, mdy;
    if (!make_map_nhwc(&mx, xt, s.N, s.H, s.W, s.C, s.sh, s.sw) || !make_map_nhwc(&mdy, dyt, s.N, s.OH, s.OW, s.Co, 1, 1))
        return fail(-4, "conv2d_backward_w: cuTensorMapEncodeTiled failed");
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        const std::pair<const void*, int> kernels[] = {
            {(const void*)wgrad_bf16_kernel<256, 1>, Ring<1>::SMEM_BYTES}, {(const void*)wgrad_bf16_kernel<128, 1>, Ring<1>::SMEM_BYTES},
            {(const void*)wgrad_bf16_kernel<256, 2>, Ring<2>::SMEM_BYTES}, {(const void*)wgrad_bf16_kernel<128, 2>, Ring<2>::SMEM_BYTES}};
        for (auto& k : kernels)
            if (attr_err == cudaSuccess) attr_err = cudaFuncSetAttribute(k.first, cudaFuncAttributeMaxDynamicSharedMemorySize, k.second);
    });
    B200JT_CUDA(attr_err);
    const int taps = s.KH * s.KW;
    const unsigned grid = (unsigned)((int64_t)p.groups * p.tiles_m * p.tiles_n * p.splits);
    if (p.taps_per_cta == 2) {
        if (p.bn == 256) wgrad_bf16_kernel<256, 2><<<grid, THREADS, Ring<2>::SMEM_BYTES, st>>>(mx, mdy, part, A);
        else wgrad_bf16_kernel<128, 2><<<grid, THREADS, Ring<2>::SMEM_BYTES, st>>>(mx, mdy, part, A);
    } else {
        if (p.bn == 256) wgrad_bf16_kernel<256, 1><<<grid, THREADS, Ring<1>::SMEM_BYTES, st>>>(mx, mdy, part, A);
        else wgrad_bf16_kernel<128, 1><<<grid, THREADS, Ring<1>::SMEM_BYTES, st>>>(mx, mdy, part, A);
    }
    B200JT_LAUNCH_CHECK();
    const int64_t n = (int64_t)taps * s.C * s.Co;
    wgrad_fold_kernel<<<grid_for(n, 256), 256, 0, st>>>(part, (__nv_bfloat16*)dw, p.splits, taps, s.C, s.Co, lay.w_ohwi ? 1 : 0);
    B200JT_LAUNCH_CHECK();
    return 0;
}

int tcconv_status_fetch_and_clear() { return tc::status_fetch_and_clear(); }

}  // namespace b200jt
