/*
 * C restatement of the reference's CPU loop nests for the benchmark workloads.
 *
 * TEST INFRASTRUCTURE ONLY: linked by the tests, the smoke check and the CPU-baseline / reference arm of the
 * benchmark, never by the shipped package. Parity pinned: tests/test_oracle_c.py checks every function here
 * against oracle/meta_ops_ref.py, which is itself pinned to outputs of the reference's CPU executor
 * (tests/golden).
 *
 * Each function is the loop nest the reference's JIT emits for the op on CPU (templates cited per function,
 * paths relative to the reference root), compiled like its kernels with -Ofast -fopenmp
 * (python/jittor/src/jit_compiler.cc:210-274). Loops are parallelised over the outermost independent axis
 * where the reference's `parallel` option would (python/jittor/src/opt/pass/parallel_pass.h); the scatter
 * loop stays serial, as it does in the reference (its read-modify-write is not parallelised on CPU).
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

/* ReindexReduceOp::jit_run with index "@e0(i0)", op add: python/jittor/src/ops/reindex_reduce_op.cc:116-130 */
void oracle_scatter_add_i32(const int32_t* y, const int32_t* e0, int64_t n, int32_t* x, int64_t bins) {
    for (int64_t i = 0; i < bins; i++) x[i] = 0;
    for (int64_t i = 0; i < n; i++) {
        int64_t xid = e0[i];
        if (xid < 0 || xid >= bins) continue;
        x[xid] = x[xid] + y[i];
    }
}

void oracle_scatter_add_f32(const float* y, const int32_t* e0, int64_t n, float* x, int64_t bins) {
    for (int64_t i = 0; i < bins; i++) x[i] = 0.f;
    for (int64_t i = 0; i < n; i++) {
        int64_t xid = e0[i];
        if (xid < 0 || xid >= bins) continue;
        x[xid] = x[xid] + y[i];
    }
}

/* ReindexReduceOp::jit_run, op add, indexes [i0, i1, i2*2+i4, i3*2+i5] on y[N,C,H,W,2,2] -> x[N,C,2H,2W]
 * (the 2x2 max-pool backward), same template :116-130 */
void oracle_pool2x2_bwd_f32(const float* y, float* x, int64_t N, int64_t C, int64_t H, int64_t W) {
    const int64_t XH = 2 * H, XW = 2 * W;
#pragma omp parallel for
    for (int64_t i = 0; i < N * C * XH * XW; i++) x[i] = 0.f;
#pragma omp parallel for collapse(2)
    for (int64_t i0 = 0; i0 < N; i0++)
        for (int64_t i1 = 0; i1 < C; i1++)
            for (int64_t i2 = 0; i2 < H; i2++)
                for (int64_t i3 = 0; i3 < W; i3++)
                    for (int64_t i4 = 0; i4 < 2; i4++)
                        for (int64_t i5 = 0; i5 < 2; i5++) {
                            int64_t yid = ((((i0 * C + i1) * H + i2) * W + i3) * 2 + i4) * 2 + i5;
                            int64_t xh = i2 * 2 + i4, xw = i3 * 2 + i5;
                            int64_t xid = ((i0 * C + i1) * XH + xh) * XW + xw;
                            x[xid] = x[xid] + y[yid];
                        }
}

/* softmax over the last axis in the reference's meta-op form, python/jittor/nn.py:533-534: three fused kernels
 * {reduce.maximum}, {subtract, exp, reduce.add}, {subtract, exp, divide} -- exp is recomputed, x is read three
 * times. Templates: python/jittor/src/ops/reduce_op.cc:374-399, binary_op.cc:563-570. */
void oracle_softmax_rows_f32(const float* x, float* y, int64_t rows, int64_t cols, int log_form) {
#pragma omp parallel for
    for (int64_t r = 0; r < rows; r++) {
        const float* xr = x + r * cols;
        float* yr = y + r * cols;
        float m = -FLT_MAX;
        for (int64_t c = 0; c < cols; c++) m = xr[c] > m ? xr[c] : m;
        float s = 0.f;
        for (int64_t c = 0; c < cols; c++) s = s + expf(xr[c] - m);
        if (log_form) {
            float ls = logf(s);
            for (int64_t c = 0; c < cols; c++) yr[c] = (xr[c] - m) - ls;
        } else {
            for (int64_t c = 0; c < cols; c++) yr[c] = expf(xr[c] - m) / s;
        }
    }
}

/* LayerNorm over the last axis, python/jittor/nn.py:781-787; mean accumulates x*rcount
 * (python/jittor/src/type/common_op_type.cc:141). gamma/beta may be NULL. */
void oracle_layernorm_rows_f32(const float* x, const float* gamma, const float* beta, float* y,
                               int64_t rows, int64_t cols, float eps) {
    const float rcount = (float)(1.0 / (double)cols);
#pragma omp parallel for
    for (int64_t r = 0; r < rows; r++) {
        const float* xr = x + r * cols;
        float* yr = y + r * cols;
        float mean = 0.f, m2 = 0.f;
        for (int64_t c = 0; c < cols; c++) { mean = mean + xr[c] * rcount; m2 = m2 + (xr[c] * xr[c]) * rcount; }
        float var = m2 - mean * mean;
        var = var > 0.f ? var : 0.f;
        const float sd = sqrtf(var + eps);
        for (int64_t c = 0; c < cols; c++) {
            float w = (gamma ? gamma[c] : 1.f) / sd;
            float b = (beta ? beta[c] : 0.f) - mean * w;
            yr[c] = xr[c] * w + b;
        }
    }
}

/* Broadcast-multiply-sum matmul, python/jittor/nn.py:157-159: c[i0,i2] = sum_i1 a[i0,i1]*b[i1,i2], loops in
 * the order of the product shape [n, m, k] (reduce_op.cc:386-394). */
void oracle_matmul_f32(const float* a, const float* b, float* c, int64_t n, int64_t m, int64_t k) {
#pragma omp parallel for
    for (int64_t i0 = 0; i0 < n; i0++) {
        float* cr = c + i0 * k;
        for (int64_t i2 = 0; i2 < k; i2++) cr[i2] = 0.f;
        for (int64_t i1 = 0; i1 < m; i1++) {
            const float av = a[i0 * m + i1];
            const float* br = b + i1 * k;
            for (int64_t i2 = 0; i2 < k; i2++) cr[i2] = cr[i2] + av * br[i2];
        }
    }
}

/* Reindex-lowered conv2d, python/jittor/nn.py:1009-1017: y[n,co,oh,ow] = sum_{c,kh,kw} x[n,c,oh*s-p+kh*d,ow*s-p+kw*d]
 * * w[co,c,kh,kw] with zero for out-of-range taps; the 7-deep nest in the order [N,Co,C,OH,OW,KH,KW]
 * (reindex_op.cc:131-138 for the window, reduce_op.cc:386-394 for the sum). */
void oracle_conv2d_f32(const float* x, const float* w, float* y, int64_t N, int64_t C, int64_t H, int64_t W,
                       int64_t Co, int64_t KH, int64_t KW, int64_t s, int64_t p, int64_t d) {
    const int64_t OH = (H + p * 2 - KH * d + d - 1) / s + 1, OW = (W + p * 2 - KW * d + d - 1) / s + 1;
#pragma omp parallel for collapse(2)
    for (int64_t n = 0; n < N; n++)
        for (int64_t co = 0; co < Co; co++) {
            float* yp = y + (n * Co + co) * OH * OW;
            for (int64_t i = 0; i < OH * OW; i++) yp[i] = 0.f;
            for (int64_t c = 0; c < C; c++)
                for (int64_t oh = 0; oh < OH; oh++)
                    for (int64_t ow = 0; ow < OW; ow++)
                        for (int64_t kh = 0; kh < KH; kh++)
                            for (int64_t kw = 0; kw < KW; kw++) {
                                int64_t ih = oh * s - p + kh * d, iw = ow * s - p + kw * d;
                                if (ih < 0 || ih >= H || iw < 0 || iw >= W) continue;
                                yp[oh * OW + ow] += x[((n * C + c) * H + ih) * W + iw] * w[((co * C + c) * KH + kh) * KW + kw];
                            }
        }
}

/* Weight gradient of the reindex-lowered conv2d as the gradient rules build it: the multiply's rule gives
 * reindex(x) * broadcast(dy) (binary_op.cc:491-550), the broadcast's rule sums it over the axes the weight was stretched
 * along, [N, OH, OW] of the 7-deep space (broadcast_to_op.cc:112-117, reduce_op.cc:386-394):
 * dw[co,c,kh,kw] = sum_{n,oh,ow} x[n,c,oh*s-p+kh*d,ow*s-p+kw*d] * dy[n,co,oh,ow], out-of-range taps contribute 0
 * (reindex_op.cc:131-138). ConvTuner relays this graph to the cuDNN filter gradient (conv_tuner.cc:375-397). */
void oracle_conv2d_backward_w_f32(const float* x, const float* dy, float* dw, int64_t N, int64_t C, int64_t H, int64_t W,
                                  int64_t Co, int64_t KH, int64_t KW, int64_t s, int64_t p, int64_t d) {
    const int64_t OH = (H + p * 2 - KH * d + d - 1) / s + 1, OW = (W + p * 2 - KW * d + d - 1) / s + 1;
#pragma omp parallel for collapse(2)
    for (int64_t co = 0; co < Co; co++)
        for (int64_t c = 0; c < C; c++) {
            float* wp = dw + (co * C + c) * KH * KW;
            for (int64_t i = 0; i < KH * KW; i++) wp[i] = 0.f;
            for (int64_t n = 0; n < N; n++)
                for (int64_t oh = 0; oh < OH; oh++)
                    for (int64_t ow = 0; ow < OW; ow++) {
                        const float g = dy[((n * Co + co) * OH + oh) * OW + ow];
                        for (int64_t kh = 0; kh < KH; kh++)
                            for (int64_t kw = 0; kw < KW; kw++) {
                                int64_t ih = oh * s - p + kh * d, iw = ow * s - p + kw * d;
                                if (ih < 0 || ih >= H || iw < 0 || iw >= W) continue;
                                wp[kh * KW + kw] += x[((n * C + c) * H + ih) * W + iw] * g;
                            }
                    }
        }
}

/* Per-channel mean / mean of squares over [0,2,3] then normalise (+ReLU), python/jittor/nn.py:674-683. */
void oracle_bn_relu_f32(const float* x, const float* gamma, const float* beta, float* y,
                        int64_t N, int64_t C, int64_t HW, float eps, int relu) {
    const float rcount = (float)(1.0 / (double)(N * HW));
#pragma omp parallel for
    for (int64_t c = 0; c < C; c++) {
        float mean = 0.f, m2 = 0.f;
        for (int64_t n = 0; n < N; n++) {
            const float* p = x + (n * C + c) * HW;
            for (int64_t i = 0; i < HW; i++) { mean += p[i] * rcount; m2 += (p[i] * p[i]) * rcount; }
        }
        float var = m2 - mean * mean;
        var = var > 0.f ? var : 0.f;
        const float wv = gamma[c] / sqrtf(var + eps), bv = beta[c] - mean * wv;
        for (int64_t n = 0; n < N; n++) {
            const float* p = x + (n * C + c) * HW;
            float* q = y + (n * C + c) * HW;
            for (int64_t i = 0; i < HW; i++) { float o = p[i] * wv + bv; q[i] = (relu && !(o > 0.f)) ? 0.f : o; }
        }
    }
}
