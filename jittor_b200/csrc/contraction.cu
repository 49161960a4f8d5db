// C entry points of the two contraction relays (matmul, conv2d): argument checks and the choice
// between the tcgen05 tensor-core kernels (bfloat16, tile-aligned shapes) and the CUDA-core kernels
// (float32, or shapes the tensor-core tiles do not cover).
#include "gemm_simt.cuh"

using namespace b200jt;

static bool matmul_dims(const b200jt_tensor* a, const b200jt_tensor* b, int trans_a, int trans_b, int64_t* M, int64_t* N, int64_t* K) {
    if (!valid_tensor(a) || !valid_tensor(b) || a->ndim != 2 || b->ndim != 2) return false;
    *M = trans_a ? a->shape[1] : a->shape[0]; *K = trans_a ? a->shape[0] : a->shape[1];
    *N = trans_b ? b->shape[0] : b->shape[1];
    return (trans_b ? b->shape[1] : b->shape[0]) == *K;
}

extern "C" size_t b200jt_matmul_workspace(const b200jt_tensor* a, const b200jt_tensor* b, const b200jt_tensor* c, int trans_a, int trans_b) {
    int64_t M, N, K;
    if (!matmul_dims(a, b, trans_a, trans_b, &M, &N, &K) || !valid_tensor(c)) return 0;
    if (a->dtype == B200JT_BFLOAT16 && matmul_tc_supported(M, N, K, a->ptr, b->ptr, c->ptr))
        return matmul_tc_workspace(M, N, K, trans_a != 0, trans_b != 0);
    return 0;
}

/* Status word of the tensor-core kernels: 0, or the code of the first bounded wait that expired since the last call
 * (1 producer, 2 accumulator hand-back, 3 operand arrival, 4 accumulator ready; 5: a peer's flag in the all-reduce kernel). Synchronises the device. */
extern "C" int b200jt_device_status(void) {
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    const int a = tc_status_fetch_and_clear(), b = tcconv_status_fetch_and_clear(), c = peer_status_fetch_and_clear();
    return a ? a : b ? b : c;
}

extern "C" int b200jt_matmul(const b200jt_tensor* a, const b200jt_tensor* b, const b200jt_tensor* c,
                             int trans_a, int trans_b, void* workspace, size_t workspace_bytes, void* stream) {
    B200JT_CHECK_ARG(valid_tensor(a) && valid_tensor(b) && valid_tensor(c), "invalid tensor descriptor");
    B200JT_CHECK_ARG(a->ndim == 2 && b->ndim == 2 && c->ndim == 2, "matmul takes 2-D tensors");
    B200JT_CHECK_ARG(a->dtype == b->dtype && a->dtype == c->dtype &&
                     (a->dtype == B200JT_FLOAT32 || a->dtype == B200JT_BFLOAT16), "a, b, c must all be float32 or bfloat16");
    const int64_t M = trans_a ? a->shape[1] : a->shape[0], K = trans_a ? a->shape[0] : a->shape[1];
    const int64_t Kb = trans_b ? b->shape[1] : b->shape[0], N = trans_b ? b->shape[0] : b->shape[1];
    B200JT_CHECK_ARG(K == Kb, "dimension not match, a:" + shape_str(a) + " b:" + shape_str(b));
    B200JT_CHECK_ARG(c->shape[0] == M && c->shape[1] == N, "c has the wrong shape " + shape_str(c));
    if (M == 0 || N == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (a->dtype == B200JT_BFLOAT16 && matmul_tc_supported(M, N, K, a->ptr, b->ptr, c->ptr)) {
        const size_t need = matmul_tc_workspace(M, N, K, trans_a != 0, trans_b != 0);
        B200JT_CHECK_ARG(workspace_bytes >= need && (need == 0 || workspace), "workspace too small: need " + std::to_string(need) + " bytes");
        return matmul_tc(a->ptr, b->ptr, c->ptr, M, N, K, trans_a != 0, trans_b != 0, workspace, st);
    }
    return matmul_simt(a->ptr, b->ptr, c->ptr, a->dtype, M, N, K, trans_a != 0, trans_b != 0, st);
}

// c[i] = op_a(a[i]) . op_b(b[i]) for i < batch; a: [Ba, ., .], b: [Bb, ., .], c: [batch, M, N] with Ba, Bb in {1, batch}
// (extent 1 shares the operand). One launch: tcgen05 for bfloat16 shapes its tiles cover, else the CUDA-core kernel with
// the batch in grid z.
extern "C" int b200jt_batched_matmul(const b200jt_tensor* a, const b200jt_tensor* b, const b200jt_tensor* c,
                                     int trans_a, int trans_b, void* stream) {
    B200JT_CHECK_ARG(valid_tensor(a) && valid_tensor(b) && valid_tensor(c), "invalid tensor descriptor");
    B200JT_CHECK_ARG(a->ndim == 3 && b->ndim == 3 && c->ndim == 3, "batched matmul takes 3-D tensors [batch, rows, cols]");
    B200JT_CHECK_ARG(a->dtype == b->dtype && a->dtype == c->dtype &&
                     (a->dtype == B200JT_FLOAT32 || a->dtype == B200JT_BFLOAT16), "a, b, c must all be float32 or bfloat16");
    const int64_t batch = c->shape[0];
    const int64_t M = trans_a ? a->shape[2] : a->shape[1], K = trans_a ? a->shape[1] : a->shape[2];
    const int64_t Kb = trans_b ? b->shape[2] : b->shape[1], N = trans_b ? b->shape[1] : b->shape[2];
    B200JT_CHECK_ARG(K == Kb, "dimension not match, a:" + shape_str(a) + " b:" + shape_str(b));
    B200JT_CHECK_ARG((a->shape[0] == batch || a->shape[0] == 1) && (b->shape[0] == batch || b->shape[0] == 1),
                     "batch extents must equal c's or be 1, a:" + shape_str(a) + " b:" + shape_str(b) + " c:" + shape_str(c));
    B200JT_CHECK_ARG(c->shape[1] == M && c->shape[2] == N, "c has the wrong shape " + shape_str(c));
    if (batch == 0 || M == 0 || N == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (a->dtype == B200JT_BFLOAT16 && batched_matmul_tc_supported(batch, M, N, K, trans_a != 0, trans_b != 0, a->ptr, b->ptr, c->ptr))
        return batched_matmul_tc(a->ptr, b->ptr, c->ptr, batch, a->shape[0], b->shape[0], M, N, K, trans_b != 0, st);
    return batched_matmul_simt(a->ptr, b->ptr, c->ptr, a->dtype, batch, a->shape[0], b->shape[0], M, N, K,
                               trans_a != 0, trans_b != 0, st);
}

static int conv_shape(const b200jt_tensor* x, const b200jt_tensor* w, const b200jt_tensor* y,
                      int sh, int sw, int ph, int pw, int dh, int dw, int groups, ConvShape* s) {
    B200JT_CHECK_ARG(valid_tensor(x) && valid_tensor(w) && valid_tensor(y), "invalid tensor descriptor");
    B200JT_CHECK_ARG(x->ndim == 4 && w->ndim == 4 && y->ndim == 4, "conv2d takes NCHW x, OIHW w, NCHW y");
    B200JT_CHECK_ARG(groups >= 1, "groups must be positive");
    B200JT_CHECK_ARG(x->dtype == w->dtype && x->dtype == y->dtype &&
                     (x->dtype == B200JT_FLOAT32 || x->dtype == B200JT_BFLOAT16), "x, w, y must all be float32 or bfloat16");
    B200JT_CHECK_ARG(sh > 0 && sw > 0 && dh > 0 && dw > 0 && ph >= 0 && pw >= 0, "bad stride/padding/dilation");
    s->N = (int)x->shape[0]; s->C = (int)x->shape[1]; s->H = (int)x->shape[2]; s->W = (int)x->shape[3];
    s->Co = (int)w->shape[0]; s->KH = (int)w->shape[2]; s->KW = (int)w->shape[3];
    B200JT_CHECK_ARG(s->C % groups == 0 && s->Co % groups == 0, "in_channels and out_channels must be divisible by groups");
    B200JT_CHECK_ARG(w->shape[1] == s->C / groups, "weight in-channels do not match x");
    s->groups = groups;
    // output extent, python/jittor/nn.py:1006-1007
    s->OH = (s->H + ph * 2 - s->KH * dh + dh - 1) / sh + 1;
    s->OW = (s->W + pw * 2 - s->KW * dw + dw - 1) / sw + 1;
    s->sh = sh; s->sw = sw; s->ph = ph; s->pw = pw; s->dh = dh; s->dw = dw;
    B200JT_CHECK_ARG(s->OH > 0 && s->OW > 0, "empty output");
    B200JT_CHECK_ARG(y->shape[0] == s->N && y->shape[1] == s->Co && y->shape[2] == s->OH && y->shape[3] == s->OW,
                     "y has the wrong shape " + shape_str(y));
    return 0;
}

// Layout strings of the reference's conv relays: a = batch / out channel, b = in channel, c/d = rows / columns.
// Returns the descriptors re-expressed as NCHW / OIHW shapes (the data stays where it is) and the layout flags.
static int conv_formats(const b200jt_tensor* x, const b200jt_tensor* w, const b200jt_tensor* y,
                        const char* xformat, const char* wformat, const char* yformat,
                        b200jt_tensor* xl, b200jt_tensor* wl, b200jt_tensor* yl, ConvLayout* lay) {
    B200JT_CHECK_ARG(valid_tensor(x) && valid_tensor(w) && valid_tensor(y) && x->ndim == 4 && w->ndim == 4 && y->ndim == 4,
                     "conv2d takes 4-d x, w, y");
    const std::string xf = xformat && *xformat ? xformat : "abcd", wf = wformat && *wformat ? wformat : "oihw";
    const std::string yf = yformat && *yformat ? yformat : xf;               // an empty yformat follows x, as in the reference
    B200JT_CHECK_ARG(xf == "abcd" || xf == "acdb", "xformat must be abcd or acdb, got " + xf);
    B200JT_CHECK_ARG(yf == "abcd" || yf == "acdb", "yformat must be abcd or acdb, got " + yf);
    B200JT_CHECK_ARG(wf == "oihw" || wf == "ohwi", "wformat must be oihw or ohwi, got " + wf);
    lay->x_nhwc = xf == "acdb"; lay->y_nhwc = yf == "acdb"; lay->w_ohwi = wf == "ohwi";
    auto to_nchw = [](const b200jt_tensor* t, bool last_is_channel, b200jt_tensor* o) {
        *o = *t;
        if (last_is_channel) { o->shape[1] = t->shape[3]; o->shape[2] = t->shape[1]; o->shape[3] = t->shape[2]; }
    };
    to_nchw(x, lay->x_nhwc, xl); to_nchw(w, lay->w_ohwi, wl); to_nchw(y, lay->y_nhwc, yl);
    return 0;
}

extern "C" size_t b200jt_conv2d_formats_workspace(const b200jt_tensor* x, const b200jt_tensor* w, const b200jt_tensor* y,
                                                  int sh, int sw, int ph, int pw, int dh, int dw,
                                                  const char* xformat, const char* wformat, const char* yformat) {
    b200jt_tensor xl, wl, yl; ConvLayout lay; ConvShape s;
    if (conv_formats(x, w, y, xformat, wformat, yformat, &xl, &wl, &yl, &lay)) return 0;
    if (conv_shape(&xl, &wl, &yl, sh, sw, ph, pw, dh, dw, 1, &s)) return 0;
    if (x->dtype == B200JT_BFLOAT16 && conv2d_tc_supported(s, x->ptr, w->ptr, y->ptr)) return conv2d_tc_workspace(s);
    return 0;
}

extern "C" int b200jt_conv2d_formats(const b200jt_tensor* x, const b200jt_tensor* w, const b200jt_tensor* y,
                                     int sh, int sw, int ph, int pw, int dh, int dw,
                                     const char* xformat, const char* wformat, const char* yformat,
                                     float* stats, void* workspace, size_t workspace_bytes, void* stream) {
    b200jt_tensor xl, wl, yl; ConvLayout lay; ConvShape s;
    int rc = conv_formats(x, w, y, xformat, wformat, yformat, &xl, &wl, &yl, &lay);
    if (rc) return rc;
    if (!lay.x_nhwc && !lay.w_ohwi && !lay.y_nhwc)
        return b200jt_conv2d(x, w, y, sh, sw, ph, pw, dh, dw, 1, stats, workspace, workspace_bytes, stream);
    rc = conv_shape(&xl, &wl, &yl, sh, sw, ph, pw, dh, dw, 1, &s);
    if (rc) return rc;
    if (numel(y) == 0) return 0;
    if (!(x->dtype == B200JT_BFLOAT16 && conv2d_tc_supported(s, x->ptr, w->ptr, y->ptr) && ((uintptr_t)y->ptr % 16 == 0)))
        return fail(-5, "b200jt_conv2d_formats: acdb / ohwi layouts run on the tensor-core kernel only (bfloat16, in channels a "
                        "multiple of 8 and >= 64, out channels >= 64, at least 1024 output pixels, 16-byte aligned tensors)");
    const size_t need = conv2d_tc_workspace(s);
    B200JT_CHECK_ARG(workspace_bytes >= need && workspace, "workspace too small: need " + std::to_string(need) + " bytes");
    rc = conv2d_tc(x->ptr, w->ptr, y->ptr, stats, s, workspace, (cudaStream_t)stream, lay);
    if (rc == 1) return 0;             // statistics came out of the conv epilogue
    if (rc) return rc;
    if (stats) {
        // wider than the epilogue keeps per CTA: statistics of the stored values by a separate pass are only built for NCHW
        return fail(-5, "b200jt_conv2d_formats: fused statistics need out channels <= 512 with an acdb output");
    }
    return 0;
}

extern "C" size_t b200jt_conv2d_backward_w_formats_workspace(const b200jt_tensor* x, const b200jt_tensor* dy, const b200jt_tensor* dw,
                                                             int sh, int sw, int ph, int pw, int dh, int dw_,
                                                             const char* xformat, const char* wformat, const char* yformat) {
    b200jt_tensor xl, wl, yl; ConvLayout lay; ConvShape s;
    if (conv_formats(x, dw, dy, xformat, wformat, yformat, &xl, &wl, &yl, &lay)) return 0;
    if (conv_shape(&xl, &wl, &yl, sh, sw, ph, pw, dh, dw_, 1, &s)) return 0;
    if (x->dtype == B200JT_BFLOAT16 && conv2d_wgrad_tc_supported(s, x->ptr, dy->ptr, dw->ptr)) return conv2d_wgrad_tc_workspace(s);
    return 0;
}

extern "C" int b200jt_conv2d_backward_w_formats(const b200jt_tensor* x, const b200jt_tensor* dy, const b200jt_tensor* dw,
                                                int sh, int sw, int ph, int pw, int dh, int dw_,
                                                const char* xformat, const char* wformat, const char* yformat,
                                                void* workspace, size_t workspace_bytes, void* stream) {
    b200jt_tensor xl, wl, yl; ConvLayout lay; ConvShape s;
    int rc = conv_formats(x, dw, dy, xformat, wformat, yformat, &xl, &wl, &yl, &lay);
    if (rc) return rc;
    if (!lay.x_nhwc && !lay.w_ohwi && !lay.y_nhwc)
        return b200jt_conv2d_backward_w_tc(x, dy, dw, sh, sw, ph, pw, dh, dw_, workspace, workspace_bytes, stream);
    rc = conv_shape(&xl, &wl, &yl, sh, sw, ph, pw, dh, dw_, 1, &s);
    if (rc) return rc;
    if (numel(dw) == 0) return 0;
    if (!(x->dtype == B200JT_BFLOAT16 && conv2d_wgrad_tc_supported(s, x->ptr, dy->ptr, dw->ptr)))
        return fail(-5, "b200jt_conv2d_backward_w_formats: acdb / ohwi layouts run on the tensor-core kernel only (bfloat16, in and "
                        "out channels multiples of 8 and >= 64, outputs of at least 8 x 8 per image and 4096 pixels in all, "
                        "16-byte aligned x and dy)");
    const size_t need = conv2d_wgrad_tc_workspace(s);
    B200JT_CHECK_ARG(workspace_bytes >= need && workspace, "workspace too small: need " + std::to_string(need) + " bytes");
    return conv2d_wgrad_tc(x->ptr, dy->ptr, dw->ptr, s, workspace, (cudaStream_t)stream, lay);
}

extern "C" size_t b200jt_conv2d_workspace(const b200jt_tensor* x, const b200jt_tensor* w, const b200jt_tensor* y,
                                          int sh, int sw, int ph, int pw, int dh, int dw, int groups) {
    ConvShape s;
    if (conv_shape(x, w, y, sh, sw, ph, pw, dh, dw, groups, &s)) return 0;
    if (groups == 1 && x->dtype == B200JT_BFLOAT16 && conv2d_tc_supported(s, x->ptr, w->ptr, y->ptr)) return conv2d_tc_workspace(s);
    return 0;
}

extern "C" int b200jt_conv2d(const b200jt_tensor* x, const b200jt_tensor* w, const b200jt_tensor* y,
                             int sh, int sw, int ph, int pw, int dh, int dw, int groups,
                             float* stats, void* workspace, size_t workspace_bytes, void* stream) {
    ConvShape s;
    int rc = conv_shape(x, w, y, sh, sw, ph, pw, dh, dw, groups, &s);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (numel(y) != 0) {
        if (groups == 1 && x->dtype == B200JT_BFLOAT16 && conv2d_tc_supported(s, x->ptr, w->ptr, y->ptr)) {
            const size_t need = conv2d_tc_workspace(s);
            B200JT_CHECK_ARG(workspace_bytes >= need && workspace, "workspace too small: need " + std::to_string(need) + " bytes");
            rc = conv2d_tc(x->ptr, w->ptr, y->ptr, stats, s, workspace, st);
            if (rc == 1) return 0;             // statistics came out of the conv epilogue
            if (rc) return rc;
        } else {
            rc = conv2d_simt(x->ptr, w->ptr, y->ptr, x->dtype, s, st);
            if (rc) return rc;
        }
    }
    if (stats) return b200jt_bn_stats(y, stats, stream);
    return 0;
}

extern "C" int b200jt_conv2d_transpose(const b200jt_tensor* x, const b200jt_tensor* w, const b200jt_tensor* y,
                                       int sh, int sw, int ph, int pw, int dh, int dw, int groups, void* stream) {
    B200JT_CHECK_ARG(valid_tensor(x) && valid_tensor(w) && valid_tensor(y), "invalid tensor descriptor");
    B200JT_CHECK_ARG(x->ndim == 4 && w->ndim == 4 && y->ndim == 4, "conv2d_transpose takes NCHW x, IOHW w, NCHW y");
    B200JT_CHECK_ARG(x->dtype == w->dtype && x->dtype == y->dtype &&
                     (x->dtype == B200JT_FLOAT32 || x->dtype == B200JT_BFLOAT16), "x, w, y must all be float32 or bfloat16");
    B200JT_CHECK_ARG(sh > 0 && sw > 0 && dh > 0 && dw > 0 && ph >= 0 && pw >= 0 && groups >= 1, "bad stride/padding/dilation/groups");
    ConvShape s;
    s.N = (int)x->shape[0]; s.C = (int)x->shape[1]; s.H = (int)x->shape[2]; s.W = (int)x->shape[3];
    s.KH = (int)w->shape[2]; s.KW = (int)w->shape[3];
    s.Co = (int)w->shape[1] * groups;
    B200JT_CHECK_ARG(w->shape[0] == s.C && s.C % groups == 0, "weight in-channels do not match x");
    s.OH = (int)y->shape[2]; s.OW = (int)y->shape[3];
    // the output extent is (H-1)*stride - 2*padding + dilation*(K-1) + 1 + output_padding with output_padding < max(stride, dilation)
    const int64_t oh0 = (int64_t)(s.H - 1) * sh - 2 * ph + (int64_t)(s.KH - 1) * dh + 1;
    const int64_t ow0 = (int64_t)(s.W - 1) * sw - 2 * pw + (int64_t)(s.KW - 1) * dw + 1;
    B200JT_CHECK_ARG(y->shape[0] == s.N && y->shape[1] == s.Co && s.OH >= oh0 && s.OH < oh0 + std::max(sh, dh) &&
                     s.OW >= ow0 && s.OW < ow0 + std::max(sw, dw), "y has the wrong shape " + shape_str(y));
    s.sh = sh; s.sw = sw; s.ph = ph; s.pw = pw; s.dh = dh; s.dw = dw; s.groups = groups;
    if (numel(y) == 0) return 0;
    return conv2d_transpose_simt(x->ptr, w->ptr, y->ptr, x->dtype, s, (cudaStream_t)stream);
}

extern "C" int b200jt_conv2d_backward_w(const b200jt_tensor* x, const b200jt_tensor* dy, const b200jt_tensor* dw,
                                        int sh, int sw, int ph, int pw, int dh, int dw_, void* stream) {
    ConvShape s;
    int rc = conv_shape(x, dw, dy, sh, sw, ph, pw, dh, dw_, 1, &s);        // same shape relations as the forward conv
    if (rc) return rc;
    if (numel(dw) == 0) return 0;
    if (numel(dy) == 0) return fail(-1, "b200jt_conv2d_backward_w: empty dy");
    return conv2d_backward_w_simt(x->ptr, dy->ptr, dw->ptr, x->dtype, s, (cudaStream_t)stream);
}

extern "C" size_t b200jt_conv2d_backward_w_workspace(const b200jt_tensor* x, const b200jt_tensor* dy, const b200jt_tensor* dw,
                                                     int sh, int sw, int ph, int pw, int dh, int dw_) {
    ConvShape s;
    if (conv_shape(x, dw, dy, sh, sw, ph, pw, dh, dw_, 1, &s)) return 0;
    if (x->dtype == B200JT_BFLOAT16 && conv2d_wgrad_tc_supported(s, x->ptr, dy->ptr, dw->ptr)) return conv2d_wgrad_tc_workspace(s);
    return 0;
}

extern "C" int b200jt_conv2d_backward_w_tc(const b200jt_tensor* x, const b200jt_tensor* dy, const b200jt_tensor* dw,
                                           int sh, int sw, int ph, int pw, int dh, int dw_,
                                           void* workspace, size_t workspace_bytes, void* stream) {
    ConvShape s;
    int rc = conv_shape(x, dw, dy, sh, sw, ph, pw, dh, dw_, 1, &s);        // same shape relations as the forward conv
    if (rc) return rc;
    if (numel(dw) == 0) return 0;
    if (numel(dy) == 0) return fail(-1, "b200jt_conv2d_backward_w_tc: empty dy");
    if (x->dtype == B200JT_BFLOAT16 && conv2d_wgrad_tc_supported(s, x->ptr, dy->ptr, dw->ptr)) {
        const size_t need = conv2d_wgrad_tc_workspace(s);
        B200JT_CHECK_ARG(workspace_bytes >= need && workspace, "workspace too small: need " + std::to_string(need) + " bytes");
        return conv2d_wgrad_tc(x->ptr, dy->ptr, dw->ptr, s, workspace, (cudaStream_t)stream);
    }
    return conv2d_backward_w_simt(x->ptr, dy->ptr, dw->ptr, x->dtype, s, (cudaStream_t)stream);
}
