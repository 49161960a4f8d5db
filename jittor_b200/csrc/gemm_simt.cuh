// Host entry points of the CUDA-core contraction kernels (gemm_simt.cu) and of the tcgen05 kernels.
#pragma once
#include "common.cuh"

namespace b200jt {

struct ConvShape {
    int N, C, H, W, Co, KH, KW, OH, OW, sh, sw, ph, pw, dh, dw;
    int groups = 1;
};
// Memory layouts other than the default NCHW / OIHW (tensor-core path only): x and y as NHWC ("acdb"), w as OHWI ("ohwi").
struct ConvLayout { bool x_nhwc = false, w_ohwi = false, y_nhwc = false; };

int matmul_simt(const void* a, const void* b, void* c, int dtype, int64_t M, int64_t N, int64_t K,
                bool trans_a, bool trans_b, cudaStream_t st);
int batched_matmul_simt(const void* a, const void* b, void* c, int dtype, int64_t batch, int64_t a_batch, int64_t b_batch,
                        int64_t M, int64_t N, int64_t K, bool trans_a, bool trans_b, cudaStream_t st);
// tcgen05 path (gemm_tcgen05.cu)
bool matmul_tc_supported(int64_t M, int64_t N, int64_t K, const void* a, const void* b, const void* c);
size_t matmul_tc_workspace(int64_t M, int64_t N, int64_t K, bool trans_a, bool trans_b);
int matmul_tc(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K, bool trans_a, bool trans_b,
              void* workspace, cudaStream_t st);
bool batched_matmul_tc_supported(int64_t batch, int64_t M, int64_t N, int64_t K, bool trans_a, bool trans_b,
                                 const void* a, const void* b, const void* c);
int batched_matmul_tc(const void* a, const void* b, void* c, int64_t batch, int64_t a_batch, int64_t b_batch,
                      int64_t M, int64_t N, int64_t K, bool trans_b, cudaStream_t st);
int tc_status_fetch_and_clear();

bool conv2d_tc_supported(const ConvShape& s, const void* x, const void* w, const void* y);
size_t conv2d_tc_workspace(const ConvShape& s);
// returns < 0 / > 1 on error, 0 on success, 1 on success with `stats` filled by the epilogue
int conv2d_tc(const void* x, const void* w, void* y, float* stats, const ConvShape& s, void* workspace, cudaStream_t st,
              const ConvLayout& lay = ConvLayout());
// weight gradient on tcgen05 (bf16, groups == 1): K = N*OH*OW pixels, split over CTAs, fp32 partial sums folded in a fixed order
bool conv2d_wgrad_tc_supported(const ConvShape& s, const void* x, const void* dy, const void* dw);
size_t conv2d_wgrad_tc_workspace(const ConvShape& s);
// lay: x_nhwc / y_nhwc say that x / dy are channels-last already (no copy), w_ohwi that dw is written [Co][KH][KW][C]
int conv2d_wgrad_tc(const void* x, const void* dy, void* dw, const ConvShape& s, void* workspace, cudaStream_t st,
                    const ConvLayout& lay = ConvLayout());
int tcconv_status_fetch_and_clear();
int peer_status_fetch_and_clear();          // peer_allreduce.cu

int conv2d_simt(const void* x, const void* w, void* y, int dtype, const ConvShape& s, cudaStream_t st);
int conv2d_backward_w_simt(const void* x, const void* dy, void* dw, int dtype, const ConvShape& s, cudaStream_t st);
int conv2d_transpose_simt(const void* x, const void* w, void* y, int dtype, const ConvShape& s, cudaStream_t st);

}  // namespace b200jt
