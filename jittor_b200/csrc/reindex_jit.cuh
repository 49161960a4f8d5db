// Affine reindex compiled per op instance (reindex_jit.cu).
#pragma once
#include "common.cuh"

namespace b200jt {

// x index d of output element (i_0 .. i_{ndim_loop-1}) = c0[d] + sum_j coef[d][j] * i_j
struct ReindexAffine {
    int32_t ndim_loop, ndim_x;
    int64_t loop_shape[kMaxDims];
    int64_t x_shape[kMaxDims];
    int64_t c0[kMaxDims];
    int64_t coef[kMaxDims][kMaxDims];
};

// Launches the kernel compiled for exactly this op instance (every tensor below 2^31 elements; `vec` output elements of
// `elem` bytes per thread: vec divides the output size and y is aligned to vec * elem). Returns 0 when it ran,
// kReindexJitUnavailable when the caller should run the ahead-of-time kernel, any other value is an error.
constexpr int kReindexJitUnavailable = -1000;
int reindex_jit_launch(const ReindexAffine& A, int elem, int vec, const void* x, void* y, uint64_t fill_bits, cudaStream_t st);

// While set for the calling thread, reindex_jit_launch only generates and compiles (no GPU needed).
struct ReindexDryRun { std::string source, log; bool compiled = false; };
void reindex_jit_dry_run(ReindexDryRun* d);
bool reindex_jit_dry_running();

}  // namespace b200jt
