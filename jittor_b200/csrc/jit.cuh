// Run-time compilation shared by the kernels that are specialised at first use (chain_jit.cu, reindex_jit.cu): NVRTC
// opened with dlopen, CUDA source -> sm_100a cubin -> cudaLibrary -> kernel handle, cached per process under a
// caller-chosen key.
#pragma once
#include "common.cuh"

#include <functional>

namespace b200jt {
namespace jit {

// NVRTC found and complete? `why` gets the reason when it is not.
bool available(std::string* why);
// The kernel `entry` of the source make_source() returns, compiled on the first request for `key` and served from the
// cache afterwards; nullptr when the compilation or the load failed (the failure is cached too; `log` gets the
// compiler's output).
cudaKernel_t get_kernel(const std::string& key, const std::function<std::string()>& make_source, const char* entry, std::string* log);
// Compile without loading (works without a GPU).
bool compile_only(const std::string& src, std::string* log);
// kernels compiled, requests served from the cache, failed compilations; any pointer may be null
void stats(int* compiled, int* hits, int* failed);

}  // namespace jit
}  // namespace b200jt
