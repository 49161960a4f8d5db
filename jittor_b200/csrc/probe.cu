// Rate probes: what the atomic units behind the scatter kernels can do on this GPU, measured with one kernel each, so that
// the ceiling of a one-atomic-per-element scatter is a number next to its HBM fraction (bench.py prints them).
#include "common.cuh"

namespace b200jt {
namespace probe {

__device__ __forceinline__ uint32_t xorshift(uint32_t& s) { s ^= s << 13; s ^= s >> 17; s ^= s << 5; return s; }

// MODE 0: shared-memory atomicAdd(int), 1: shared-memory atomicAdd(float), 2: __match_any_sync
template <int MODE>
__global__ void __launch_bounds__(1024, 1) smem_rate_kernel(int iters, int words, int skewed, float* sink) {
    extern __shared__ int sm[];
    for (int i = threadIdx.x; i < words; i += blockDim.x) sm[i] = 0;
    __syncthreads();
    uint32_t s = threadIdx.x * 2654435761u + blockIdx.x * 40503u + 12345u;
    int acc = 0;
    for (int it = 0; it < iters; it++) {
        const uint32_t r = xorshift(s);
        int b = (int)(r % (uint32_t)words);
        if (skewed && (r >> 20) % 6 == 0) b = 7;              // about 16 % of the operations on one address
        if (MODE == 0) atomicAdd(&sm[b], 1);
        else if (MODE == 1) atomicAdd(reinterpret_cast<float*>(&sm[b]), 1.0f);
        else acc += __popc(__match_any_sync(0xffffffffu, b));
    }
    __syncthreads();
    if (threadIdx.x == 0) sink[blockIdx.x] = (float)sm[0] + (float)acc;
}

__global__ void __launch_bounds__(1024, 2) red_rate_kernel(int iters, uint32_t words, int* table) {
    uint32_t s = (threadIdx.x + blockIdx.x * blockDim.x) * 2654435761u + 99u;
    for (int it = 0; it < iters; it++) atomicAdd(&table[xorshift(s) % words], 1);
}

}  // namespace probe
}  // namespace b200jt

using namespace b200jt;

/* Operations per second (in 1e9/s) of: "red_global" -- red.global.add.u32 to random words of `table` (words of them),
 * 296 x 1024 threads; "smem_int" / "smem_float" -- shared-memory atomicAdd on 4096 words, 148 x 1024 threads;
 * "match_any" -- __match_any_sync. skewed != 0 sends about 16 % of the shared-memory operations to one address.
 * Synchronises the device; `scratch` must hold max(words * 4, 1024) bytes. */
extern "C" int b200jt_probe_rate(const char* what, int skewed, void* scratch, int64_t words, double* gops) {
    B200JT_CHECK_ARG(what && scratch && gops && words > 0 && words < (1LL << 31), "bad argument");
    cudaEvent_t e0, e1;
    B200JT_CUDA(cudaEventCreate(&e0));
    B200JT_CUDA(cudaEventCreate(&e1));
    double ops = 0;
    for (int rep = 0; rep < 2; rep++) {            // the second launch is the timed one
        B200JT_CUDA(cudaEventRecord(e0));
        if (!strcmp(what, "red_global")) {
            if (rep == 0) B200JT_CUDA(cudaMemset(scratch, 0, (size_t)words * 4));
            probe::red_rate_kernel<<<2 * kNumSMs, 1024>>>(64, (uint32_t)words, (int*)scratch);
            ops = 2.0 * kNumSMs * 1024 * 64;
        } else {
            const int iters = 256, w = 4096;
            if (!strcmp(what, "smem_int")) probe::smem_rate_kernel<0><<<kNumSMs, 1024, w * 4>>>(iters, w, skewed, (float*)scratch);
            else if (!strcmp(what, "smem_float")) probe::smem_rate_kernel<1><<<kNumSMs, 1024, w * 4>>>(iters, w, skewed, (float*)scratch);
            else if (!strcmp(what, "match_any")) probe::smem_rate_kernel<2><<<kNumSMs, 1024, w * 4>>>(iters, w, skewed, (float*)scratch);
            else return fail(-1, std::string("b200jt_probe_rate: unknown probe '") + what + "'");
            ops = (double)kNumSMs * 1024 * iters;
        }
        B200JT_CUDA(cudaEventRecord(e1));
        B200JT_CUDA(cudaEventSynchronize(e1));
    }
    B200JT_LAUNCH_CHECK();
    float ms = 0;
    B200JT_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    *gops = ops / (ms * 1e6);
    return 0;
}
