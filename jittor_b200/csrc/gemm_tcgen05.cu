// bf16 GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] . Bt[N,K]^T, fp32 accumulation in TMEM.
//
// The broadcast-multiply-sum matmul of the reference (python/jittor/nn.py:157-159) is a dense contraction; its
// relay is cublasGemmEx (python/jittor/extern/cuda/cublas/ops/cublas_matmul_op.cc:117-123). Here it is one
// persistent, warp-specialised kernel:
//   warp 0     TMA producer: cp.async.bulk.tensor 2-D loads of 128x64 (A) and 256x64 (Bt) bf16 tiles, 128-byte
//              swizzle, into a 4-stage shared-memory ring (192 KB), completion on mbarriers;
//   warp 1     MMA issuer: one lane issues tcgen05.mma.cta_group::1.kind::f16 (M=128, N=256, K=16) on shared-memory
//              descriptors; accumulators live in TMEM, 2 x 256 columns so the next tile starts while the previous
//              one is drained; tcgen05.commit releases ring slots / publishes accumulators;
//   warps 2-5  epilogue: tcgen05.ld (32 lanes x 32 columns), fp32 -> bf16, 16-byte global stores.
// Tiles are scheduled statically (tile = blockIdx.x + i*gridDim.x) in groups of 8 tile-rows for L2 reuse; one CTA
// per SM. Ragged M/N/K edges rely on TMA zero fill and masked stores. No cluster launch and no multicast.
// Every mbarrier wait is bounded: on expiry the CTA records a status word, stops issuing, drains and frees TMEM.
#include "gemm_simt.cuh"
#include "tc_common.cuh"

#include <algorithm>
#include <mutex>

namespace b200jt {

namespace tc {

constexpr int BM = 128, BN = 256, BK = 64;          // one MMA tile; BK * 2 B = 128 B = swizzle width
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
constexpr int THREADS = 192;                        // 6 warps

// MT = number of 128-row MMA tiles a CTA stacks per output tile. MT = 2 re-uses every Bt stage for two MMAs
// (64 KB of operands per 8.4 MFLOP instead of 48 KB per 4.2 MFLOP), so the same 192 KB ring covers 1.5x more time
// of tensor work -- enough to hide an HBM miss -- at the price of a single TMEM accumulator set (512 columns).
template <int MT> struct Cfg {
    static constexpr int STAGES = MT == 1 ? 4 : 3;
    static constexpr int STAGE_BYTES = MT * A_BYTES + B_BYTES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
    static constexpr int NBUF = 2 / MT;             // accumulator sets in the 512 TMEM columns
};

struct Tiles {
    int tiles_m, tiles_n, total, G;                          // G: tile-rows per group (L2 reuse of the Bt tiles)
    __device__ __forceinline__ void coords(int t, int& m, int& n) const {
        const int per_group = G * tiles_n;
        const int g = t / per_group, r = t - g * per_group;
        const int rows = min(G, tiles_m - g * G);
        m = g * G + r % rows;
        n = r / rows;
    }
};

// BMN: B is given as [K, N] (N contiguous) and used as an MN-major operand -- four 64 x 64 TMA boxes per stage -- instead
// of being transposed into K-major form by a separate pass.
// BATCH: the maps are 3-D ([batch][rows][cols]) and the tile index runs over batch x tiles; an operand whose batch
// extent is 1 is shared by all products (its batch coordinate stays 0). This is the strided-batched product the
// reference relays to cublasGemmStridedBatchedEx (python/jittor/extern/cuda/cublas/ops/cublas_batched_matmul_op.cc:160).
template <int MT, bool BMN, bool BATCH = false>
__global__ void __launch_bounds__(THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 __nv_bfloat16* __restrict__ c, int M, int N, int K, int group, uint32_t b_lbo, uint32_t b_sbo,
                 int batch = 1, int a_batched = 0, int b_batched = 0) {
    constexpr int STAGES = Cfg<MT>::STAGES, STAGE_BYTES = Cfg<MT>::STAGE_BYTES, NBUF = Cfg<MT>::NBUF;
    extern __shared__ unsigned char smem_raw[];
    // operand tiles need 1024-byte alignment for the 128-byte swizzle
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + STAGES * STAGE_BYTES);
    uint64_t* full = bars;                 // [STAGES] TMA -> MMA
    uint64_t* empty = bars + STAGES;       // [STAGES] MMA -> TMA
    uint64_t* acc_full = bars + 2 * STAGES;      // [2] MMA -> epilogue
    uint64_t* acc_empty = bars + 2 * STAGES + 2; // [2] epilogue -> MMA
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    Tiles T;
    T.tiles_m = (M + MT * BM - 1) / (MT * BM); T.tiles_n = (N + BN - 1) / BN; T.total = T.tiles_m * T.tiles_n; T.G = group;
    const int k_blocks = (K + BK - 1) / BK;
    const int per_batch = T.total;
    const int all_tiles = BATCH ? per_batch * batch : per_batch;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        for (int b = 0; b < NBUF; b++) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // all 512 TMEM columns: two 128 x 256 fp32 accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < all_tiles && ok; t += gridDim.x) {
                const int bi = BATCH ? t / per_batch : 0;
                int tm, tn; T.coords(BATCH ? t - bi * per_batch : t, tm, tn);
                const int ba = a_batched ? bi : 0, bb = b_batched ? bi : 0;
                for (int kb = 0; kb < k_blocks; kb++) {
                    if (!(ok = mbar_wait(empty + stage, phase ^ 1, abort_flag, 1))) break;
                    unsigned char* sa = smem + stage * STAGE_BYTES;
                    mbar_expect_tx(full + stage, STAGE_BYTES);
#pragma unroll
                    for (int j = 0; j < MT; j++) {
                        if (BATCH) tma_load_3d(sa + j * A_BYTES, &map_a, full + stage, kb * BK, (tm * MT + j) * BM, ba);
                        else tma_load_2d(sa + j * A_BYTES, &map_a, full + stage, kb * BK, (tm * MT + j) * BM);
                    }
                    if (BMN) {
#pragma unroll
                        for (int cch = 0; cch < BN / 64; cch++) {
                            if (BATCH) tma_load_3d(sa + MT * A_BYTES + cch * (64 * BK * 2), &map_b, full + stage, tn * BN + cch * 64, kb * BK, bb);
                            else tma_load_2d(sa + MT * A_BYTES + cch * (64 * BK * 2), &map_b, full + stage, tn * BN + cch * 64, kb * BK);
                        }
                    } else {
                        if (BATCH) tma_load_3d(sa + MT * A_BYTES, &map_b, full + stage, kb * BK, tn * BN, bb);
                        else tma_load_2d(sa + MT * A_BYTES, &map_b, full + stage, kb * BK, tn * BN);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                // give copies that are already in flight a bounded chance to land before the CTA goes away
                for (int s = 0; s < STAGES; s++)
                    for (uint32_t i = 0; i < 4096 && !mbar_try(full + s, 0) && !mbar_try(full + s, 1); i++) __nanosleep(64);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN, BMN);
            int stage = 0; uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < all_tiles && ok; t += gridDim.x, it++) {
                const int buf = it % NBUF;
                const uint32_t acc_phase = (it / NBUF) & 1;
                if (!(ok = mbar_wait(acc_empty + buf, acc_phase ^ 1, abort_flag, 2))) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + buf * (MT * BN);
                for (int kb = 0; kb < k_blocks; kb++) {
                    if (!(ok = mbar_wait(full + stage, phase, abort_flag, 3))) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
                    const uint64_t db = BMN ? make_smem_desc_mn(sa + MT * A_BYTES, b_lbo, b_sbo) : make_smem_desc(sa + MT * A_BYTES);
                    // advancing K by 16: K-major +32 B inside the swizzled row (+2 units of 16 B); MN-major 16 rows of 128 B
                    constexpr int B_KSTEP = BMN ? (UMMA_K * 128) / 16 : 2;
#pragma unroll
                    for (int j = 0; j < MT; j++) {
                        const uint64_t da = make_smem_desc(sa + j * A_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; k++)
                            umma_f16(tmem_d + j * BN, da + 2 * k, db + B_KSTEP * k, idesc, (kb | k) != 0);
                    }
                    umma_commit(empty + stage);                 // slot reusable once these MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit(acc_full + buf);             // accumulator complete
            }
        }
    } else {
        // ---------------- epilogue: warps 2..5 own TMEM lane quadrants (warp % 4) ----------------
        const int quad = warp & 3;
        int it = 0;
        bool ok = true;
        const bool vec_ok = (N % 8 == 0) && (((uintptr_t)c & 15) == 0);
        for (int t = blockIdx.x; t < all_tiles && ok; t += gridDim.x, it++) {
            const int bi = BATCH ? t / per_batch : 0;
            int tm, tn; T.coords(BATCH ? t - bi * per_batch : t, tm, tn);
            const int buf = it % NBUF;
            const uint32_t acc_phase = (it / NBUF) & 1;
            ok = mbar_wait(acc_full + buf, acc_phase, abort_flag, 4);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int j = 0; j < MT; j++) {
            const int row = (tm * MT + j) * BM + quad * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * (MT * BN) + j * BN;
            __nv_bfloat16* crow = c + ((int64_t)bi * M + row) * N + (int64_t)tn * BN;
#pragma unroll 1
            for (int ch = 0; ch < BN / 32; ch++) {
                uint32_t r[32];
                tmem_ld32(taddr + ch * 32, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const int col0 = tn * BN + ch * 32;
                if (row < M && col0 < N) {
                    if (vec_ok && col0 + 32 <= N) {
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            uint4 v;
                            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
                            for (int e = 0; e < 4; e++)
                                h[e] = __floats2bfloat162_rn(__uint_as_float(r[q * 8 + 2 * e]), __uint_as_float(r[q * 8 + 2 * e + 1]));
                            *reinterpret_cast<uint4*>(crow + ch * 32 + q * 8) = v;
                        }
                    } else {
                        for (int e = 0; e < 32 && col0 + e < N; e++) crow[ch * 32 + e] = __float2bfloat16(__uint_as_float(r[e]));
                    }
                }
            }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + buf);
        }
    }
    // ---------------- teardown ----------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

// ---- bf16 transpose: out[c, r] = in[r, c] (used to bring an operand into K-major form) -------------------
__global__ void __launch_bounds__(256)
transpose_bf16_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int R, int Cn) {
    __shared__ __nv_bfloat16 tile[64][66];
    const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;          // 32 x 8
    for (int i = ty; i < 64; i += 8) {
        const int r = r0 + i;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int cc = c0 + tx * 2 + j;
            tile[i][tx * 2 + j] = (r < R && cc < Cn) ? in[(int64_t)r * Cn + cc] : __float2bfloat16(0.f);
        }
    }
    __syncthreads();
    for (int i = ty; i < 64; i += 8) {
        const int cc = c0 + i;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int r = r0 + tx * 2 + j;
            if (cc < Cn && r < R) out[(int64_t)cc * R + r] = tile[tx * 2 + j][i];
        }
    }
}

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
    });
    return fn;
}

// 2-D bf16 row-major [rows, cols] with a {BK, box_rows} box and 128-byte swizzle
static bool make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int box_rows) {
    auto fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// 3-D bf16 [batch][rows][cols] with a {BK, box_rows, 1} box: one box has the shared-memory layout of the 2-D form
static bool make_map_3d(CUtensorMap* map, const void* base, int64_t batch, int64_t rows, int64_t cols, int box_rows) {
    auto fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
    cuuint64_t strides[2] = {(cuuint64_t)cols * 2, (cuuint64_t)rows * cols * 2};
    cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace tc

bool matmul_tc_supported(int64_t M, int64_t N, int64_t K, const void* a, const void* b, const void* c) {
    // TMA: 16-byte aligned bases and row pitches (K % 8); tiny problems stay on the CUDA-core kernel
    return K % 8 == 0 && K >= 64 && M >= 128 && N >= 64 && M < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31) &&
           ((uintptr_t)a % 16 == 0) && ((uintptr_t)b % 16 == 0) && ((uintptr_t)c % 2 == 0) && tc::encode_fn() != nullptr;
}

static bool b_mn_direct(int64_t N, bool trans_b) {
    const char* e = getenv("B200JT_GEMM_BMN");
    return !trans_b && N % 8 == 0 && !(e && atoi(e) == 0);
}

size_t matmul_tc_workspace(int64_t M, int64_t N, int64_t K, bool trans_a, bool trans_b) {
    // A that is not K-major is transposed into the workspace first; B [K, N] is consumed directly as an MN-major operand
    size_t bytes = 0;
    if (trans_a) bytes += (size_t)M * K * 2;
    if (!trans_b && !b_mn_direct(N, trans_b)) bytes += (size_t)N * K * 2;
    return bytes;
}

int matmul_tc(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K, bool trans_a, bool trans_b,
              void* workspace, cudaStream_t st) {
    using namespace tc;
    const __nv_bfloat16* ak = (const __nv_bfloat16*)a;      // [M, K]
    const __nv_bfloat16* bk = (const __nv_bfloat16*)b;      // [N, K]
    unsigned char* ws = (unsigned char*)workspace;
    if (trans_a) {   // a is [K, M]
        dim3 g((unsigned)((M + 63) / 64), (unsigned)((K + 63) / 64));
        transpose_bf16_kernel<<<g, 256, 0, st>>>((const __nv_bfloat16*)a, (__nv_bfloat16*)ws, (int)K, (int)M);
        ak = (const __nv_bfloat16*)ws; ws += (size_t)M * K * 2;
    }
    const bool bmn = b_mn_direct(N, trans_b);
    if (!trans_b && !bmn) {  // b is [K, N]
        dim3 g((unsigned)((N + 63) / 64), (unsigned)((K + 63) / 64));
        transpose_bf16_kernel<<<g, 256, 0, st>>>((const __nv_bfloat16*)b, (__nv_bfloat16*)ws, (int)K, (int)N);
        bk = (const __nv_bfloat16*)ws;
    }
    B200JT_LAUNCH_CHECK();
    CUtensorMap ma, mb;
    // K-major operands: boxes of 64 K-elements x rows; MN-major B: boxes of 64 N-elements x 64 K-rows of b[K, N]
    if (!make_map(&ma, ak, M, K, BM) || !(bmn ? make_map(&mb, b, K, N, 64) : make_map(&mb, bk, N, K, BN)))
        return fail(-4, "matmul: cuTensorMapEncodeTiled failed");
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(gemm_bf16_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<1>::SMEM_BYTES);
        if (attr_err == cudaSuccess) attr_err = cudaFuncSetAttribute(gemm_bf16_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<2>::SMEM_BYTES);
        if (attr_err == cudaSuccess) attr_err = cudaFuncSetAttribute(gemm_bf16_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<1>::SMEM_BYTES);
        if (attr_err == cudaSuccess) attr_err = cudaFuncSetAttribute(gemm_bf16_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<2>::SMEM_BYTES);
    });
    B200JT_CUDA(attr_err);
    // 256-row tiles when they still fill the machine for several waves, 128-row tiles otherwise
    const int64_t tiles2 = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
    const char* genv = getenv("B200JT_GEMM_G");
    const int group = genv ? atoi(genv) : 8;
    const char* force = getenv("B200JT_GEMM_MT");
    const bool two = force ? atoi(force) == 2 : tiles2 >= 4 * kNumSMs;
    // MN-major B: 64-column chunks are 8 KB apart (leading offset), 8-row groups along K 1 KB apart (stride offset)
    const uint32_t lbo = 64 * BK * 2, sbo = 1024;
    const int64_t tiles1 = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = (int)std::min<int64_t>(two ? tiles2 : tiles1, kNumSMs);
#define B200JT_GEMM(MT_, BMN_) gemm_bf16_kernel<MT_, BMN_><<<grid, THREADS, Cfg<MT_>::SMEM_BYTES, st>>>( \
        ma, mb, (__nv_bfloat16*)c, (int)M, (int)N, (int)K, group, lbo, sbo)
    if (two) { if (bmn) B200JT_GEMM(2, true); else B200JT_GEMM(2, false); }
    else     { if (bmn) B200JT_GEMM(1, true); else B200JT_GEMM(1, false); }
#undef B200JT_GEMM
    B200JT_LAUNCH_CHECK();
    return 0;
}

// One launch for `batch` products c[i] = a[i or 0] . b[i or 0] (a [.., M, K] K-major; b [.., K, N] consumed MN-major, or
// [.., N, K] when trans_b). The caller has checked batched_matmul_tc_supported.
bool batched_matmul_tc_supported(int64_t batch, int64_t M, int64_t N, int64_t K, bool trans_a, bool trans_b,
                                 const void* a, const void* b, const void* c) {
    if (trans_a || !matmul_tc_supported(M, N, K, a, b, c) || batch >= (1LL << 31)) return false;
    if ((M * K) % 8 != 0 || (N * K) % 8 != 0) return false;            // 16-byte batch pitch of the tensor maps
    return trans_b || b_mn_direct(N, trans_b);
}

int batched_matmul_tc(const void* a, const void* b, void* c, int64_t batch, int64_t a_batch, int64_t b_batch,
                      int64_t M, int64_t N, int64_t K, bool trans_b, cudaStream_t st) {
    using namespace tc;
    const bool bmn = !trans_b;
    CUtensorMap ma, mb;
    if (!make_map_3d(&ma, a, a_batch, M, K, BM) ||
        !(bmn ? make_map_3d(&mb, b, b_batch, K, N, 64) : make_map_3d(&mb, b, b_batch, N, K, BN)))
        return fail(-4, "batched matmul: cuTensorMapEncodeTiled failed");
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(gemm_bf16_kernel<1, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<1>::SMEM_BYTES);
        if (attr_err == cudaSuccess) attr_err = cudaFuncSetAttribute(gemm_bf16_kernel<2, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<2>::SMEM_BYTES);
        if (attr_err == cudaSuccess) attr_err = cudaFuncSetAttribute(gemm_bf16_kernel<1, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<1>::SMEM_BYTES);
        if (attr_err == cudaSuccess) attr_err = cudaFuncSetAttribute(gemm_bf16_kernel<2, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<2>::SMEM_BYTES);
    });
    B200JT_CUDA(attr_err);
    const int64_t tiles2 = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN) * batch;
    const int64_t tiles1 = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * batch;
    if (tiles1 >= (1LL << 31)) return fail(-1, "batched matmul: too many tiles");
    const bool two = tiles2 >= 4 * kNumSMs && M > BM;
    const uint32_t lbo = 64 * BK * 2, sbo = 1024;
    const int grid = (int)std::min<int64_t>(two ? tiles2 : tiles1, kNumSMs);
#define B200JT_BGEMM(MT_, BMN_) gemm_bf16_kernel<MT_, BMN_, true><<<grid, THREADS, Cfg<MT_>::SMEM_BYTES, st>>>( \
        ma, mb, (__nv_bfloat16*)c, (int)M, (int)N, (int)K, 8, lbo, sbo, (int)batch, a_batch > 1 ? 1 : 0, b_batch > 1 ? 1 : 0)
    if (two) { if (bmn) B200JT_BGEMM(2, true); else B200JT_BGEMM(2, false); }
    else     { if (bmn) B200JT_BGEMM(1, true); else B200JT_BGEMM(1, false); }
#undef B200JT_BGEMM
    B200JT_LAUNCH_CHECK();
    return 0;
}

int tc_status_fetch_and_clear() { return tc::status_fetch_and_clear(); }

}  // namespace b200jt
