// All-reduce across the GPUs of one node as ONE kernel per rank over NVLink peer mappings: the role of the relay
// NcclAllReduceOp::jit_run (python/jittor/extern/cuda/nccl/ops/nccl_all_reduce_op.cc:46-58) for the message sizes of
// this path (batch-norm statistics, scatter outputs), where a ring/tree collective is latency-bound.
//
// Every rank owns one `segment` of device memory, exported to the other ranks as a CUDA IPC handle:
//     [ flags : kMaxBlocks x kMaxRanks u32 ][ epochs : kMaxBlocks u32 ][ in[0] | in[1] | out[0] | out[1] : data_bytes (+ pad) each ]
// Block b of rank r only ever talks to block b of the other ranks:
//   small messages (one shot, while (world-1) * bytes <= 4 MiB):  copy its chunk of src into in[parity] of its own segment, flag every peer, wait for
//       every peer's flag, then sum that chunk over the ranks' segments IN RANK ORDER (so all ranks get the same
//       bits) straight into dst;
//   large messages (two shot):  rank r PUSHES its chunk of slice s from src into slot r of rank s's in[parity] (posted
//       writes), flag round, then rank r sums the world slots of slice r from its own memory and writes the result
//       into out[parity] of EVERY rank, a second flag round, and each rank copies out[parity] into dst.
// Flags carry a per-block epoch that only grows (kept in device memory, so a captured launch can be replayed; every
// call advances the epochs of all blocks, used or not, so all blocks of all ranks agree on the call count);
// in/out alternate between two halves by call parity, which is what lets the one-shot form skip a closing flag
// round: a peer can only overwrite half p again two calls later, after it has seen this rank enter the next call.
// Every wait is bounded by wall time (%globaltimer); a wait that runs out records status 5, the block stops taking
// part and the kernel returns, leaving the context usable. No multicast objects are involved: plain peer loads
// and stores only.
#include "common.cuh"

#include <vector>

namespace b200jt {
namespace peer {

constexpr int kMaxRanks = 8;
constexpr int kMaxBlocks = 128;
constexpr int kThreads = 512;
constexpr size_t kFlagBytes = (size_t)kMaxBlocks * kMaxRanks * 4;
constexpr size_t kEpochBytes = (size_t)kMaxBlocks * 4;
constexpr size_t kHeaderBytes = 8192;                       // flags + epochs, padded so the data halves stay 256-B aligned
static_assert(kFlagBytes + kEpochBytes <= kHeaderBytes, "header too small");
constexpr size_t kHalfPad = 256;
constexpr size_t kOneShotMaxRemoteBytes = 4 << 20;      // one shot while a rank reads at most this much from its peers

static __device__ int g_status = 0;

struct DevComm {                    // one per (emulated) rank, passed to the kernel by value
    unsigned char* seg[kMaxRanks];  // every rank's segment as mapped into THIS process
    int rank, world;
    unsigned long long data_bytes;  // capacity of each of the four data halves
    unsigned long long wait_ns;     // bound of one wait
};

struct Launch {                     // by-value kernel argument; entry blockIdx.y is the rank this block plays
    DevComm comm[kMaxRanks];
    const void* src[kMaxRanks];
    void* dst[kMaxRanks];
};

__device__ __forceinline__ uint32_t* flag_of(unsigned char* seg, int block, int from) {
    return reinterpret_cast<uint32_t*>(seg) + block * kMaxRanks + from;
}
__device__ __forceinline__ uint32_t* epoch_of(unsigned char* seg, int block) {
    return reinterpret_cast<uint32_t*>(seg + kFlagBytes) + block;
}
__device__ __forceinline__ unsigned char* half_of(unsigned char* seg, unsigned long long data_bytes, int which) {
    // which: 0,1 = in[parity], 2,3 = out[parity]; kHalfPad spare bytes per half: world slots of ceil(packs/world) packs
    return seg + kHeaderBytes + (size_t)which * (data_bytes + kHalfPad);
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One flag round of block `b`: tell every peer that this rank reached `value`, then wait until every peer did.
// The block's earlier writes are ordered before the flags by the barrier plus the release store of the flagging
// thread (release is cumulative over what that thread observed through the barrier); the peers' writes are ordered
// before this block's later reads by the acquire fence of the polling thread plus the closing barrier.
// Returns false for the whole block if a wait ran out.
__device__ bool flag_round(const DevComm& c, int b, uint32_t value, int* ok_smem) {
    __syncthreads();
    const int t = threadIdx.x;
    if (t < c.world && t != c.rank) {
        st_release_sys(flag_of(c.seg[t], b, c.rank), value);
        const uint32_t* mine = flag_of(c.seg[c.rank], b, t);
        uint32_t spins = 0;
        unsigned long long t0 = 0;
        while ((int32_t)(ld_relaxed_sys(mine) - value) < 0) {
            if (++spins > 512) {
                if (t0 == 0) t0 = global_ns();
                __nanosleep(spins > 8192 ? 200 : 20);
                if ((spins & 255) == 0 && global_ns() - t0 > c.wait_ns) {
                    *ok_smem = 0;
                    atomicCAS(&g_status, 0, 5);
                    break;
                }
            }
        }
        asm volatile("fence.acq_rel.sys;" ::: "memory");
    }
    __syncthreads();
    return *ok_smem != 0;
}

template <typename T> struct Acc { using type = T; };
template <> struct Acc<__nv_bfloat16> { using type = float; };
template <> struct Acc<__half> { using type = float; };

template <int OP, typename A> __device__ __forceinline__ A combine(A a, A b) {
    if (OP == 0) return a + b;
    if (OP == 1) return a > b ? a : b;
    return a < b ? a : b;
}

template <typename T, int V> struct alignas(16) Pack { T v[V]; };

// Segment halves are 256-byte aligned and padded to whole packs: always one 16-byte access. volatile: peers rewrite
// these addresses between calls and nothing of an earlier call may be reused.
template <typename T, int V> __device__ __forceinline__ Pack<T, V> load_seg(const T* p) {
    Pack<T, V> r;
    uint4 u;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(p) : "memory");
    memcpy(&r, &u, 16);
    return r;
}
template <typename T, int V> __device__ __forceinline__ void store_seg(T* p, const Pack<T, V>& r) {
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}
// Caller memory: 16-byte accesses when the pointer allows it and the pack is whole, else element by element.
template <typename T, int V> __device__ __forceinline__ Pack<T, V> load_user(const T* base, long long i, long long count, bool vec) {
    Pack<T, V> r;
    if (vec && (i + 1) * V <= count) {
        *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(base + i * V);
    } else {
#pragma unroll
        for (int e = 0; e < V; e++) r.v[e] = i * V + e < count ? base[i * V + e] : static_cast<T>(0.0f);
    }
    return r;
}
template <typename T, int V> __device__ __forceinline__ void store_user(T* base, long long i, long long count, bool vec, const Pack<T, V>& r) {
    if (vec && (i + 1) * V <= count) {
        *reinterpret_cast<uint4*>(base + i * V) = *reinterpret_cast<const uint4*>(&r);
    } else {
#pragma unroll
        for (int e = 0; e < V; e++) if (i * V + e < count) base[i * V + e] = r.v[e];
    }
}

// Sum (max, min) of `U` packs, kThreads apart starting at i, over the ranks' in[parity] halves: all loads are issued
// before the first use, so that a thread keeps U * world 16-byte NVLink reads in flight.
template <typename T, int V, int OP, int U>
__device__ __forceinline__ void reduce_over_ranks(const DevComm& c, int parity, int i, int hi, Pack<T, V> (&o)[U]) {
    using A = typename Acc<T>::type;
    Pack<T, V> p[kMaxRanks][U];
#pragma unroll
    for (int k = 0; k < kMaxRanks; k++) {
        if (k < c.world) {
            const T* base = reinterpret_cast<const T*>(half_of(c.seg[k], c.data_bytes, parity));
#pragma unroll
            for (int u = 0; u < U; u++)
                if (i + u * kThreads < hi) p[k][u] = load_seg<T, V>(base + (size_t)(i + u * kThreads) * V);
        }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
#pragma unroll
        for (int e = 0; e < V; e++) {
            A acc = (A)p[0][u].v[e];
#pragma unroll
            for (int k = 1; k < kMaxRanks; k++)
                if (k < c.world) acc = combine<OP, A>(acc, (A)p[k][u].v[e]);     // rank order: the same bits on every rank
            o[u].v[e] = (T)acc;
        }
    }
}

// The packs block b owns: chunk b (per packs) of each of `slices` slices, as one flat index space of slices*per entries.
struct BlockPacks {
    int slice, per, b, nv, slices;
    __device__ __forceinline__ int total() const { return slices * per; }
    __device__ __forceinline__ int at(int f) const {            // pack index, or -1 for padding
        const int s = f / per, j = f - s * per;
        const int i = s * slice + per * b + j;
        return (f < slices * per && i < min(nv, (s + 1) * slice)) ? i : -1;
    }
};

// The message is cut into 16-byte packs (nv of them, the last one possibly partial); which block handles which pack
// depends on the byte count only, so that all ranks agree whatever the alignment of their src/dst pointers.
// LIGHT: built for two CTAs per SM (64 registers), so that a CTA finds room on an SM that another kernel half fills; used
// when the call is capped to a few blocks to run beside other work (b200jt_peer_comm_set_max_blocks).
template <typename T, int OP, bool TWO_SHOT, bool LIGHT>
__global__ void __launch_bounds__(kThreads, LIGHT ? 2 : 1) peer_all_reduce_kernel(Launch L, long long count) {
    constexpr int V = 16 / (int)sizeof(T);
    // the light form has half the registers: fewer packs in flight per thread, twice the resident threads
    constexpr int UC = LIGHT ? 2 : 4;   // packs in flight per thread in the copies
    constexpr int UR = LIGHT ? 1 : 2;   // ... and per rank in the reduction
    __shared__ int ok;
    __shared__ DevComm c;
    if (threadIdx.x == 0) { c = L.comm[blockIdx.y]; ok = 1; }
    __syncthreads();
    const T* src = static_cast<const T*>(L.src[blockIdx.y]);
    T* dst = static_cast<T*>(L.dst[blockIdx.y]);
    const bool src_vec = (reinterpret_cast<uintptr_t>(src) & 15) == 0, dst_vec = (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
    const int nv = (int)((count + V - 1) / V);
    const int b = blockIdx.x, nb = gridDim.x, W = c.world, r = c.rank;
    uint32_t* epoch_ptr = epoch_of(c.seg[r], b);
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(epoch_ptr);
    const int parity = (epoch >> 1) & 1;
    T* in_own = reinterpret_cast<T*>(half_of(c.seg[r], c.data_bytes, parity));

    // slice s = packs [s*slice, (s+1)*slice) is reduced by rank s (two shot) or there is one slice every rank reduces
    BlockPacks mine;
    mine.slices = TWO_SHOT ? W : 1;
    mine.slice = TWO_SHOT ? (nv + W - 1) / W : nv;
    mine.per = (mine.slice + nb - 1) / nb;
    mine.b = b; mine.nv = nv;
    const int lo = (TWO_SHOT ? r * mine.slice : 0) + mine.per * b;
    const int hi = min(min(nv, (TWO_SHOT ? r + 1 : 1) * mine.slice), lo + mine.per);

    bool fine;
    if (!TWO_SHOT) {
        // 1. this block's packs of src -> in[parity] of the own segment
        for (int f0 = threadIdx.x; f0 < mine.total(); f0 += UC * kThreads) {
            int idx[UC];
            Pack<T, V> p[UC];
#pragma unroll
            for (int u = 0; u < UC; u++) {
                idx[u] = mine.at(f0 + u * kThreads);
                if (idx[u] >= 0) p[u] = load_user<T, V>(src, idx[u], count, src_vec);
            }
#pragma unroll
            for (int u = 0; u < UC; u++)
                if (idx[u] >= 0) store_seg<T, V>(in_own + (size_t)idx[u] * V, p[u]);
        }
        fine = flag_round(c, b, epoch + 1, &ok);
        // 2. reduce over the ranks straight into dst
        if (fine) {
            for (int i = lo + threadIdx.x; i < hi; i += UR * kThreads) {
                Pack<T, V> o[UR];
                reduce_over_ranks<T, V, OP, UR>(c, parity, i, hi, o);
#pragma unroll
                for (int u = 0; u < UR; u++)
                    if (i + u * kThreads < hi) store_user<T, V>(dst, i + u * kThreads, count, dst_vec, o[u]);
            }
        }
    } else {
        // 1. push: this block's chunk of slice s goes from src straight into slot r of rank s's in[parity] (posted NVLink
        //    writes; no local staging pass and no remote reads later)
        for (int f0 = threadIdx.x; f0 < mine.total(); f0 += UC * kThreads) {
            int idx[UC];
            Pack<T, V> p[UC];
#pragma unroll
            for (int u = 0; u < UC; u++) {
                idx[u] = mine.at(f0 + u * kThreads);
                if (idx[u] >= 0) p[u] = load_user<T, V>(src, idx[u], count, src_vec);
            }
#pragma unroll
            for (int u = 0; u < UC; u++) {
                if (idx[u] < 0) continue;
                const int s = idx[u] / mine.slice, j = idx[u] - s * mine.slice;
                T* slot = reinterpret_cast<T*>(half_of(c.seg[s], c.data_bytes, parity)) + ((size_t)r * mine.slice + j) * V;
                store_seg<T, V>(slot, p[u]);
            }
        }
        fine = flag_round(c, b, epoch + 1, &ok);
        // 2. reduce the W slots of the own slice (local reads, rank order) and write the result to every rank's out[parity]
        if (fine) {
            using A = typename Acc<T>::type;
            for (int i = lo + threadIdx.x; i < hi; i += UR * kThreads) {
                Pack<T, V> p[kMaxRanks][UR];
#pragma unroll
                for (int k = 0; k < kMaxRanks; k++)
                    if (k < W) {
#pragma unroll
                        for (int u = 0; u < UR; u++) {
                            const int iu = i + u * kThreads;
                            if (iu < hi) p[k][u] = load_seg<T, V>(in_own + ((size_t)k * mine.slice + (iu - r * mine.slice)) * V);
                        }
                    }
#pragma unroll
                for (int u = 0; u < UR; u++) {
                    const int iu = i + u * kThreads;
                    if (iu >= hi) continue;
                    Pack<T, V> o;
#pragma unroll
                    for (int e = 0; e < V; e++) {
                        A acc = (A)p[0][u].v[e];
#pragma unroll
                        for (int k = 1; k < kMaxRanks; k++)
                            if (k < W) acc = combine<OP, A>(acc, (A)p[k][u].v[e]);
                        o.v[e] = (T)acc;
                    }
#pragma unroll
                    for (int k = 0; k < kMaxRanks; k++)
                        if (k < W) store_seg<T, V>(reinterpret_cast<T*>(half_of(c.seg[k], c.data_bytes, 2 + parity)) + (size_t)iu * V, o);
                }
            }
        }
    }
    if (TWO_SHOT) {
        if (fine) fine = flag_round(c, b, epoch + 2, &ok);
        // 3. out[parity] of the own segment (filled by all ranks) -> dst
        if (fine) {
            const T* out_own = reinterpret_cast<const T*>(half_of(c.seg[r], c.data_bytes, 2 + parity));
            for (int f0 = threadIdx.x; f0 < mine.total(); f0 += UC * kThreads) {
                int idx[UC];
                Pack<T, V> p[UC];
#pragma unroll
                for (int u = 0; u < UC; u++) {
                    idx[u] = mine.at(f0 + u * kThreads);
                    if (idx[u] >= 0) p[u] = load_seg<T, V>(out_own + (size_t)idx[u] * V);
                }
#pragma unroll
                for (int u = 0; u < UC; u++)
                    if (idx[u] >= 0) store_user<T, V>(dst, idx[u], count, dst_vec, p[u]);
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) *epoch_ptr = epoch + 2;
    // Blocks this launch did not use keep step with the call count, so that a later, larger message finds the same
    // epoch -- hence the same staging half -- in every block (the block count follows the message size).
    if (b == 0)
        for (int i = nb + threadIdx.x; i < kMaxBlocks; i += kThreads) *epoch_of(c.seg[r], i) += 2;
}

struct Comm {
    int rank = 0, world = 1, device = 0;
    size_t data_bytes = 0;
    unsigned char* segs[kMaxRanks] = {};
    bool opened[kMaxRanks] = {};        // mapped through an IPC handle (to be closed), not owned
    bool owns_segment = false;
    int max_blocks = 0;                 // 0: no limit below kMaxBlocks (b200jt_peer_comm_set_max_blocks)
    DevComm dev{};                      // what the kernel receives
};

static size_t segment_bytes(size_t data_bytes) { return kHeaderBytes + 4 * (data_bytes + kHalfPad); }

static int upload(Comm* c, double wait_ms) {
    DevComm h{};
    for (int i = 0; i < c->world; i++) h.seg[i] = c->segs[i];
    h.rank = c->rank; h.world = c->world; h.data_bytes = c->data_bytes;
    h.wait_ns = (unsigned long long)(wait_ms * 1e6);
    c->dev = h;
    return 0;
}

template <typename T, int OP>
static int launch_t(const Launch& L, int ranks_in_grid, int world, int64_t count, int max_blocks, cudaStream_t st) {
    const size_t bytes = (size_t)count * sizeof(T);
    const long long nv = (long long)((bytes + 15) / 16);
    const bool two = bytes * (size_t)(world - 1) > kOneShotMaxRemoteBytes;
    const long long unit = two ? (nv + world - 1) / world : nv;             // packs one rank reduces
    // an emulated job keeps every rank's blocks co-resident: at most one block per SM over all ranks
    int cap = ranks_in_grid == 1 ? kMaxBlocks : std::max(1, std::min(kMaxBlocks, kNumSMs / ranks_in_grid));
    if (max_blocks > 0) cap = std::min(cap, max_blocks);
    const int blocks = (int)std::min<long long>(cap, std::max<long long>(1, (unit + kThreads - 1) / kThreads));
    dim3 grid(blocks, ranks_in_grid);
    void (*kern)(Launch, long long) = max_blocks > 0
        ? (two ? peer_all_reduce_kernel<T, OP, true, true> : peer_all_reduce_kernel<T, OP, false, true>)
        : (two ? peer_all_reduce_kernel<T, OP, true, false> : peer_all_reduce_kernel<T, OP, false, false>);
    if (ranks_in_grid == 1) {
        kern<<<grid, kThreads, 0, st>>>(L, (long long)count);
    } else {
        // all ranks of an emulated job in one grid: the blocks wait on one another, so they must be co-resident
        Launch l = L; long long n = count;
        void* args[] = {&l, &n};
        B200JT_CUDA(cudaLaunchCooperativeKernel((const void*)kern, grid, dim3(kThreads), args, 0, st));
    }
    B200JT_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch_op(const Launch& L, int ranks, int world, int64_t count, int op, int max_blocks, cudaStream_t st) {
    if (op == 0) return launch_t<T, 0>(L, ranks, world, count, max_blocks, st);
    if (op == 1) return launch_t<T, 1>(L, ranks, world, count, max_blocks, st);
    return launch_t<T, 2>(L, ranks, world, count, max_blocks, st);
}

static int launch(const Launch& L, int ranks, int world, int64_t count, int dtype, int op, int max_blocks, cudaStream_t st) {
    switch (dtype) {
        case B200JT_FLOAT32: return launch_op<float>(L, ranks, world, count, op, max_blocks, st);
        case B200JT_FLOAT64: return launch_op<double>(L, ranks, world, count, op, max_blocks, st);
        case B200JT_INT32: return launch_op<int32_t>(L, ranks, world, count, op, max_blocks, st);
        case B200JT_INT64: return launch_op<int64_t>(L, ranks, world, count, op, max_blocks, st);
        case B200JT_BFLOAT16: return launch_op<__nv_bfloat16>(L, ranks, world, count, op, max_blocks, st);
        case B200JT_FLOAT16: return launch_op<__half>(L, ranks, world, count, op, max_blocks, st);
    }
    return fail(-1, "b200jt_peer_all_reduce: dtype must be float32/64, int32/64, float16 or bfloat16");
}

static int op_code(const char* op) {
    if (!op) return -1;
    if (!strcmp(op, "add")) return 0;
    if (!strcmp(op, "maximum")) return 1;
    if (!strcmp(op, "minimum")) return 2;
    return -1;
}

int status_fetch_and_clear() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
    if (v) { int z = 0; cudaMemcpyToSymbol(g_status, &z, sizeof(int)); }
    return v;
}

}  // namespace peer
}  // namespace b200jt

using namespace b200jt;
using peer::Comm;

namespace b200jt { int peer_status_fetch_and_clear() { return peer::status_fetch_and_clear(); } }

extern "C" size_t b200jt_peer_segment_bytes(size_t data_bytes) { return peer::segment_bytes(data_bytes); }

extern "C" int b200jt_peer_segment_create(size_t data_bytes, void** segment, unsigned char* ipc_handle) {
    B200JT_CHECK_ARG(segment && ipc_handle && data_bytes > 0 && data_bytes % 256 == 0 && data_bytes <= ((size_t)1 << 30),
                     "data_bytes must be a positive multiple of 256, at most 1 GiB");
    void* p = nullptr;
    B200JT_CUDA(cudaMalloc(&p, peer::segment_bytes(data_bytes)));
    B200JT_CUDA(cudaMemset(p, 0, peer::segment_bytes(data_bytes)));
    B200JT_CUDA(cudaDeviceSynchronize());
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) == B200JT_IPC_HANDLE_BYTES, "IPC handle size");
    cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) { cudaFree(p); return fail((int)e, std::string("b200jt_peer_segment_create: cudaIpcGetMemHandle: ") + cudaGetErrorString(e)); }
    memcpy(ipc_handle, &h, sizeof(h));
    *segment = p;
    return 0;
}

extern "C" int b200jt_peer_segment_destroy(void* segment) {
    if (segment) B200JT_CUDA(cudaFree(segment));
    return 0;
}

extern "C" int b200jt_peer_comm_create(int rank, int world, void* own_segment, const unsigned char* ipc_handles,
                                       size_t data_bytes, double wait_ms, void** comm) {
    B200JT_CHECK_ARG(comm && own_segment && ipc_handles, "null argument");
    B200JT_CHECK_ARG(world >= 2 && world <= peer::kMaxRanks && rank >= 0 && rank < world, "world must be 2..8 and rank inside it");
    B200JT_CHECK_ARG(wait_ms > 0, "wait_ms must be positive");
    Comm* c = new Comm();
    c->rank = rank; c->world = world; c->data_bytes = data_bytes; c->owns_segment = true;
    cudaGetDevice(&c->device);
    c->segs[rank] = static_cast<unsigned char*>(own_segment);
    for (int i = 0; i < world; i++) {
        if (i == rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, ipc_handles + (size_t)i * B200JT_IPC_HANDLE_BYTES, sizeof(h));
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            for (int j = 0; j < i; j++) if (c->opened[j]) cudaIpcCloseMemHandle(c->segs[j]);
            delete c;
            return fail((int)e, std::string("b200jt_peer_comm_create: cudaIpcOpenMemHandle(rank ") + std::to_string(i) + "): " + cudaGetErrorString(e));
        }
        c->segs[i] = static_cast<unsigned char*>(p);
        c->opened[i] = true;
    }
    if (int rc = peer::upload(c, wait_ms)) { delete c; return rc; }
    *comm = c;
    return 0;
}

extern "C" int b200jt_peer_comm_create_local(int world, size_t data_bytes, double wait_ms, void** comms) {
    B200JT_CHECK_ARG(comms && world >= 2 && world <= peer::kMaxRanks, "world must be 2..8");
    B200JT_CHECK_ARG(data_bytes > 0 && data_bytes % 256 == 0 && data_bytes <= ((size_t)1 << 30) && wait_ms > 0,
                     "data_bytes must be a positive multiple of 256, at most 1 GiB; wait_ms positive");
    unsigned char* segs[peer::kMaxRanks] = {};
    for (int i = 0; i < world; i++) {
        B200JT_CUDA(cudaMalloc(&segs[i], peer::segment_bytes(data_bytes)));
        B200JT_CUDA(cudaMemset(segs[i], 0, peer::segment_bytes(data_bytes)));
    }
    for (int r = 0; r < world; r++) {
        Comm* c = new Comm();
        c->rank = r; c->world = world; c->data_bytes = data_bytes; c->owns_segment = true;
        cudaGetDevice(&c->device);
        for (int i = 0; i < world; i++) c->segs[i] = segs[i];
        if (int rc = peer::upload(c, wait_ms)) return rc;
        comms[r] = c;
    }
    B200JT_CUDA(cudaDeviceSynchronize());
    return 0;
}

extern "C" int b200jt_peer_comm_destroy(void* comm) {
    Comm* c = static_cast<Comm*>(comm);
    if (!c) return 0;
    cudaDeviceSynchronize();
    for (int i = 0; i < c->world; i++) if (c->opened[i]) cudaIpcCloseMemHandle(c->segs[i]);
    if (c->owns_segment && c->segs[c->rank]) cudaFree(c->segs[c->rank]);
    delete c;
    return 0;
}

extern "C" int b200jt_peer_comm_set_max_blocks(void* comm, int max_blocks) {
    B200JT_CHECK_ARG(comm && max_blocks >= 0 && max_blocks <= peer::kMaxBlocks, "max_blocks must be 0..128");
    static_cast<Comm*>(comm)->max_blocks = max_blocks;
    return 0;
}

extern "C" size_t b200jt_peer_max_bytes(const void* comm) { return comm ? static_cast<const Comm*>(comm)->data_bytes : 0; }

static int check_call(const Comm* c, const void* src, void* dst, int64_t count, int dtype, int op) {
    B200JT_CHECK_ARG(c && src && dst, "null argument");
    B200JT_CHECK_ARG(count > 0 && dtype_size(dtype) > 0, "count must be positive and dtype valid");
    B200JT_CHECK_ARG(op >= 0, "op must be add, maximum or minimum");
    B200JT_CHECK_ARG((size_t)count * dtype_size(dtype) <= c->data_bytes,
                     "message of " + std::to_string((size_t)count * dtype_size(dtype)) + " bytes exceeds the segment's " + std::to_string(c->data_bytes));
    return 0;
}

extern "C" int b200jt_peer_all_reduce(void* comm, const void* src, void* dst, int64_t count, int dtype, const char* op, void* stream) {
    const Comm* c = static_cast<const Comm*>(comm);
    const int opc = peer::op_code(op);
    if (int rc = check_call(c, src, dst, count, dtype, opc)) return rc;
    peer::Launch L{};
    L.comm[0] = c->dev; L.src[0] = src; L.dst[0] = dst;
    return peer::launch(L, 1, c->world, count, dtype, opc, c->max_blocks, (cudaStream_t)stream);
}

extern "C" int b200jt_peer_all_reduce_local(void* const* comms, int world, const void* const* srcs, void* const* dsts,
                                            int64_t count, int dtype, const char* op, void* stream) {
    B200JT_CHECK_ARG(comms && srcs && dsts && world >= 1 && world <= peer::kMaxRanks, "bad argument");
    const int opc = peer::op_code(op);
    peer::Launch L{};
    for (int r = 0; r < world; r++) {
        const Comm* c = static_cast<const Comm*>(comms[r]);
        if (int rc = check_call(c, srcs[r], dsts[r], count, dtype, opc)) return rc;
        L.comm[r] = c->dev; L.src[r] = srcs[r]; L.dst[r] = dsts[r];
        B200JT_CHECK_ARG(c->world == world && c->rank == r, "comms must be the ranks 0..world-1 of one local job, in order");
    }
    return peer::launch(L, world, world, count, dtype, opc, static_cast<const Comm*>(comms[0])->max_blocks, (cudaStream_t)stream);
}
