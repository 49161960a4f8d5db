"""GPU parity of the tcgen05 implicit-GEMM convolution (csrc/conv_tcgen05.cu) against the CPU oracle.

The kernel has four instantiations (256- or 128-channel tiles x TMA-box or per-lane stores of y), zero-filled halo
boxes, a ragged last pair of 8x8 patches, ragged last channel blocks on both operands and an epilogue that also
produces the per-channel sum / sum of squares. Every case below is run through the C ABI with the tile width forced
to each value, compared with the oracle's loop nest (fp32 accumulation on bf16-rounded inputs, result rounded to
bf16, |d| <= 2e-2*|ref| + 2e-2*max|ref|), and its fused statistics are compared with float64 sums of the bf16 values
the kernel stored. The last tests run benchmark config 4 ([256,256,56,56] * [256,256,3,3]) exactly as stated.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import c_oracle as co
from tests.golden_cases import check

pytestmark = pytest.mark.gpu


def bf16_round(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).bfloat16().float().numpy()


def conv_capi(x, w, pad, dil, stats=True, force_bn=None, stride=1):
    """b200jt_conv2d on bf16 CUDA tensors; returns (y, stats or None, used the tensor-core path)."""
    from jittor_b200 import _capi as C
    N, Ci, H, W = x.shape
    Co, _, KH, KW = w.shape
    OH, OW = (H + 2 * pad - dil * (KH - 1) - 1) // stride + 1, (W + 2 * pad - dil * (KW - 1) - 1) // stride + 1
    y = torch.empty(N, Co, OH, OW, dtype=torch.bfloat16, device="cuda")
    st = torch.full((2 * Co,), 7.0, dtype=torch.float32, device="cuda") if stats else None   # the callee zeroes it
    args = (C.desc(x), C.desc(w), C.desc(y), stride, stride, pad, pad, dil, dil, 1)
    nbytes = C.lib.b200jt_conv2d_workspace(*args)
    ws = torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device="cuda")
    old = os.environ.get("B200JT_CONV_BN")
    if force_bn:
        os.environ["B200JT_CONV_BN"] = str(force_bn)
    try:
        rc = C.lib.b200jt_conv2d(*args, ctypes.c_void_p(st.data_ptr() if stats else 0), ctypes.c_void_p(ws.data_ptr()),
                                 nbytes, C.stream_ptr())
    finally:
        if force_bn:
            if old is None:
                del os.environ["B200JT_CONV_BN"]
            else:
                os.environ["B200JT_CONV_BN"] = old
    C.check(rc, "b200jt_conv2d")
    torch.cuda.synchronize()
    return y, st, nbytes > 0


def check_stats(y, st):
    """Fused statistics = sums of the values as stored (bf16), accumulated in fp32 by the kernel."""
    Co = y.shape[1]
    yd = y.double()
    s1, s2 = yd.sum((0, 2, 3)), (yd * yd).sum((0, 2, 3))
    got1, got2 = st[:Co].double(), st[Co:].double()
    cnt = y.numel() // Co
    # fp32 accumulation of cnt terms in tree / atomic order: error ~ 1e-6 * sum|y|
    tol1 = 1e-4 * yd.abs().sum((0, 2, 3)) + 1e-6
    assert bool(((got1 - s1).abs() <= tol1).all()), f"sum: max err {(got1 - s1).abs().max().item()}"
    assert bool(((got2 - s2).abs() <= 1e-4 * s2 + 1e-6).all()), f"sum of squares: max err {(got2 - s2).abs().max().item()}"
    assert cnt > 0


# (x shape, w shape, padding, dilation): chosen to reach every variant --
#   Co in {64,128,192,256,320,512}: one tile, several tiles, ragged last tile for both widths;
#   C in {64,72,96,128,200}: one or several 64-channel blocks, ragged last block;
#   OW in {14,16,19,20,24,28,56}: TMA-box stores (OW % 8 == 0) and per-lane stores, ragged patches;
#   1x1, 3x3, 5x5 windows, dilation 2, padding 0 / 1 / 2; odd numbers of patches (ragged last pair).
CASES = [
    ((4, 64, 16, 16), (64, 64, 3, 3), 1, 1),
    ((4, 128, 20, 20), (192, 128, 3, 3), 1, 1),
    ((4, 72, 23, 27), (96, 72, 5, 5), 0, 2),
    ((4, 64, 16, 16), (128, 64, 1, 1), 0, 1),
    ((4, 64, 16, 16), (256, 64, 3, 3), 1, 1),
    ((2, 200, 24, 24), (320, 200, 3, 3), 1, 1),
    ((2, 96, 28, 28), (64, 96, 3, 3), 1, 1),
    ((1, 64, 56, 56), (64, 64, 3, 3), 1, 1),
    ((8, 96, 14, 14), (64, 96, 3, 3), 1, 1),
    ((6, 64, 14, 14), (64, 64, 3, 3), 2, 1),
    ((3, 64, 24, 24), (512, 64, 3, 3), 1, 1),
    ((5, 136, 17, 19), (72, 136, 3, 3), 1, 1),
]


# (x shape, w shape, stride, padding, dilation): the same kernel with the x tensor map stepping `stride` input pixels per
# box element -- the 3x3 stride-2 and 1x1 stride-2 layers of a ResNet, odd extents, stride 3, stride with dilation
STRIDED = [
    ((4, 64, 32, 32), (64, 64, 3, 3), 2, 1, 1),
    ((8, 128, 28, 28), (192, 128, 3, 3), 2, 1, 1),
    ((4, 64, 33, 35), (64, 64, 1, 1), 2, 0, 1),
    ((6, 72, 40, 40), (96, 72, 5, 5), 3, 2, 1),
    ((3, 64, 45, 47), (64, 64, 3, 3), 2, 0, 2),
    ((2, 256, 56, 56), (256, 256, 3, 3), 2, 1, 1),
]


@pytest.mark.parametrize("xs,wshape,stride,pad,dil", STRIDED)
def test_conv_tc_strided_against_oracle(xs, wshape, stride, pad, dil):
    from jittor_b200 import _capi as C
    rng = np.random.default_rng(sum(xs) + sum(wshape) + stride + pad + dil)
    x = bf16_round(rng.normal(size=xs))
    w = bf16_round(rng.normal(size=wshape) * np.sqrt(2.0 / (wshape[1] * wshape[2] * wshape[3])))
    xt, wt = torch.from_numpy(x).bfloat16().cuda(), torch.from_numpy(w).bfloat16().cuda()
    y, st, used_tc = conv_capi(xt, wt, pad, dil, stats=True, stride=stride)
    assert used_tc, "case does not reach the tensor-core kernel"
    want = co.conv2d(x, w, stride, pad, dil)
    check(y.float().cpu().numpy(), bf16_round(want), False, rtol=2e-2)
    check_stats(y, st)
    assert C.lib.b200jt_device_status() == 0


@pytest.mark.parametrize("force_bn", [128, 256])
@pytest.mark.parametrize("xs,wshape,pad,dil", CASES)
def test_conv_tc_variants_against_oracle(xs, wshape, pad, dil, force_bn):
    from jittor_b200 import _capi as C
    rng = np.random.default_rng(sum(xs) + sum(wshape) + pad + dil)
    x = bf16_round(rng.normal(size=xs))
    w = bf16_round(rng.normal(size=wshape) * np.sqrt(2.0 / (wshape[1] * wshape[2] * wshape[3])))
    xt, wt = torch.from_numpy(x).bfloat16().cuda(), torch.from_numpy(w).bfloat16().cuda()
    y, st, used_tc = conv_capi(xt, wt, pad, dil, stats=True, force_bn=force_bn)
    assert used_tc, "case does not reach the tensor-core kernel"
    want = co.conv2d(x, w, 1, pad, dil)
    check(y.float().cpu().numpy(), bf16_round(want), False, rtol=2e-2)
    check_stats(y, st)
    assert C.lib.b200jt_device_status() == 0
    # without statistics the same values must come out (the epilogue takes another branch)
    y2, _, _ = conv_capi(xt, wt, pad, dil, stats=False, force_bn=force_bn)
    assert torch.equal(y2, y)


def test_conv_tc_statistics_beyond_the_epilogue_limit():
    """More output channels than the epilogue keeps per CTA: the statistics come from the separate pass."""
    rng = np.random.default_rng(5)
    x = bf16_round(rng.normal(size=(2, 64, 24, 24)))
    w = bf16_round(rng.normal(size=(576, 64, 1, 1)) * 0.1)
    xt, wt = torch.from_numpy(x).bfloat16().cuda(), torch.from_numpy(w).bfloat16().cuda()
    y, st, used_tc = conv_capi(xt, wt, 0, 1)
    assert used_tc
    check(y.float().cpu().numpy(), bf16_round(co.conv2d(x, w, 1, 0, 1)), False, rtol=2e-2)
    check_stats(y, st)


# ------------------------------------------------------------------------------------------------ config 4 at full size
C5 = dict(N=256, C=256, H=56, W=56, CO=256)


@pytest.fixture(scope="module")
def c5_data():
    g = torch.Generator("cuda").manual_seed(4)
    x = torch.randn(C5["N"], C5["C"], C5["H"], C5["W"], device="cuda", generator=g).bfloat16()
    w = (torch.randn(C5["CO"], C5["C"], 3, 3, device="cuda", generator=g) * (2 / (9 * C5["C"])) ** 0.5).bfloat16()
    return x, w


def _sampled_windows(x, pix):
    """x[n, :, oh-1:oh+2, ow-1:ow+2] with zero padding for every sampled pixel -> [P, C, 3, 3] float32 numpy."""
    xp = torch.nn.functional.pad(x, (1, 1, 1, 1))
    return torch.stack([xp[n, :, oh:oh + 3, ow:ow + 3] for n, oh, ow in pix]).float().cpu().numpy()


def test_config4_conv_full_size(c5_data):
    """[256,256,56,56] * [256,256,3,3] bf16 through nn.conv2d: 96 random output pixels x all 256 channels against the
    oracle's loop nest on the touched input windows, per-channel checksums of the whole tensor against a float32 torch
    convolution, the epilogue's statistics against float64 sums of the stored values, and no expired wait."""
    import jittor_b200 as jt
    from jittor_b200 import nn, _capi as C
    x, w = c5_data
    y = nn.conv2d(jt.array(x), jt.array(w), None, 1, 1, 1)
    assert y.dtype == "bfloat16" and list(y.shape) == [256, 256, 56, 56]
    yt = y.torch()
    assert C.lib.b200jt_device_status() == 0
    rng = np.random.default_rng(11)
    pix = [(int(rng.integers(256)), int(rng.integers(56)), int(rng.integers(56))) for _ in range(88)]
    pix += [(0, 0, 0), (255, 55, 55), (17, 0, 55), (101, 55, 0), (3, 7, 8), (200, 48, 47), (128, 8, 0), (64, 55, 23)]
    want = co.conv2d(_sampled_windows(x, pix), w.float().cpu().numpy(), 1, 0, 1)[:, :, 0, 0]        # [P, Co]
    got = torch.stack([yt[n, :, oh, ow] for n, oh, ow in pix]).float().cpu().numpy()
    check(got, bf16_round(want), False, rtol=2e-2)
    # whole tensor: per-(image-block, channel) sums against a float32 torch convolution, in slabs of 32 images
    for n0 in range(0, 256, 32):
        ref = torch.nn.functional.conv2d(x[n0:n0 + 32].float(), w.float(), padding=1)
        mine = yt[n0:n0 + 32].float()
        scale = ref.abs().max().item()
        assert (mine - ref).abs().max().item() <= 2e-2 * scale
        s_ref, s_mine = ref.double().sum((0, 2, 3)), mine.double().sum((0, 2, 3))
        assert bool(((s_ref - s_mine).abs() <= 4e-3 * ref.double().abs().sum((0, 2, 3))).all())
        del ref, mine
    # the C ABI with fused statistics on the same data
    y2, st, used_tc = conv_capi(x, w, 1, 1, stats=True)
    assert used_tc and torch.equal(y2, yt)
    check_stats(y2, st)
    assert C.lib.b200jt_device_status() == 0


def test_config4_conv_bn_relu_full_size(c5_data):
    """relu(bn(conv(x, w))) of config 4 in one plan (statistics from the conv epilogue, normalise + ReLU): the whole
    result against the same chain computed from the stored conv output in float32, and sampled pixels against the
    oracle's normalisation formula with float64 batch statistics."""
    import jittor_b200 as jt
    from jittor_b200 import nn, _capi as C
    x, w = c5_data
    xv, wv = jt.array(x), jt.array(w)
    yt = nn.conv2d(xv, wv, None, 1, 1, 1).torch()
    bn = nn.BatchNorm(256, is_train=True, sync=False)
    gam = torch.rand(256, device="cuda") + 0.5
    bet = torch.randn(256, device="cuda") * 0.1
    bn.weight.assign(jt.array(gam))
    bn.bias.assign(jt.array(bet))
    with jt.flag_scope(amp_reg=2):
        z = nn.relu(bn(nn.conv2d(xv, wv, None, 1, 1, 1)))
    assert z.dtype == "bfloat16"
    zt = z.torch()
    assert C.lib.b200jt_device_status() == 0
    yd = yt.double()
    mean = yd.mean((0, 2, 3))
    var = ((yd * yd).mean((0, 2, 3)) - mean * mean).clamp_min(0)
    del yd
    wgt = (gam.double() / torch.sqrt(var + 1e-5)).float()
    bias = (bet.double() - mean * wgt.double()).float()
    worst = 0.0
    for n0 in range(0, 256, 32):
        ref = torch.relu(yt[n0:n0 + 32].float() * wgt[None, :, None, None] + bias[None, :, None, None])
        d = (zt[n0:n0 + 32].float() - ref).abs()
        tol = 2e-2 * ref.abs() + 2e-2 * ref.abs().max()
        assert bool((d <= tol).all()), f"max err {d.max().item()}"
        worst = max(worst, d.max().item())
    # sampled pixels through the oracle: conv on the touched windows, then its normalisation with the batch statistics
    rng = np.random.default_rng(12)
    pix = [(int(rng.integers(256)), int(rng.integers(56)), int(rng.integers(56))) for _ in range(64)]
    conv = bf16_round(co.conv2d(_sampled_windows(x, pix), w.float().cpu().numpy(), 1, 0, 1)[:, :, 0, 0])
    want = np.maximum(conv * wgt.cpu().numpy()[None] + bias.cpu().numpy()[None], 0)
    got = torch.stack([zt[n, :, oh, ow] for n, oh, ow in pix]).float().cpu().numpy()
    check(got, bf16_round(want), False, rtol=2e-2)


# (x NCHW shape, w OIHW shape, stride, padding, xformat, wformat, yformat): NHWC ("acdb") activations are the kernel's own
# operand layout (no layout pass on that side), "ohwi" weights only change the re-ordering pass, an acdb output is written
# by the epilogue as 32 contiguous channels per pixel (vector stores, or element stores for a ragged last chunk)
LAYOUTS = [
    ((4, 64, 16, 16), (64, 64, 3, 3), 1, 1, "acdb", "oihw", "acdb"),
    ((4, 64, 16, 16), (64, 64, 3, 3), 1, 1, "acdb", "ohwi", "abcd"),
    ((4, 64, 16, 16), (64, 64, 3, 3), 1, 1, "abcd", "ohwi", "acdb"),
    ((2, 96, 28, 28), (192, 96, 3, 3), 1, 1, "acdb", "ohwi", ""),
    ((3, 128, 21, 19), (72, 128, 3, 3), 1, 1, "acdb", "oihw", "acdb"),
    ((8, 72, 28, 28), (100, 72, 5, 5), 2, 2, "acdb", "ohwi", "acdb"),
    ((2, 256, 28, 28), (320, 256, 1, 1), 1, 0, "acdb", "oihw", "acdb"),
]


@pytest.mark.parametrize("xs,wshape,stride,pad,xf,wf,yf", LAYOUTS)
def test_conv_layouts_of_the_relay_against_oracle(xs, wshape, stride, pad, xf, wf, yf):
    """cudnn_conv with the layout strings ConvTuner derives (python/jittor/src/opt/tuner/conv_tuner.cc:292-341)."""
    import jittor_b200 as jt
    from jittor_b200 import _capi as C
    rng = np.random.default_rng(sum(xs) + sum(wshape) + stride)
    x = bf16_round(rng.normal(size=xs))
    w = bf16_round(rng.normal(size=wshape) * np.sqrt(2.0 / (wshape[1] * wshape[2] * wshape[3])))
    want = bf16_round(co.conv2d(x, w, stride, pad, 1))
    xin = x if xf == "abcd" else np.ascontiguousarray(x.transpose(0, 2, 3, 1))
    win = w if wf == "oihw" else np.ascontiguousarray(w.transpose(0, 2, 3, 1))
    conv = jt.get_op_info("cudnn_conv").get_constructor()
    xv = jt.array(torch.from_numpy(xin).bfloat16())
    wv = jt.array(torch.from_numpy(win).bfloat16())
    y = conv(xv, wv, stride, stride, pad, pad, 1, 1, 1, xf, wf, yf)
    got = y.torch().float().cpu().numpy()
    if (yf or xf) == "acdb":
        assert list(got.shape) == [want.shape[0], want.shape[2], want.shape[3], want.shape[1]]
        got = got.transpose(0, 3, 1, 2)
    check(np.ascontiguousarray(got), want, False, rtol=2e-2)
    assert C.lib.b200jt_device_status() == 0


def test_conv_layouts_outside_the_tensor_core_path_are_refused():
    import jittor_b200 as jt
    from jittor_b200 import _capi as C
    conv = jt.get_op_info("cudnn_conv").get_constructor()
    x = jt.array(torch.randn(2, 8, 8, 16).bfloat16())            # 16 channels: not a tensor-core shape
    w = jt.array(torch.randn(32, 16, 3, 3).bfloat16())
    with pytest.raises(C.B200Error, match="tensor-core kernel only"):
        conv(x, w, 1, 1, 1, 1, 1, 1, 1, "acdb", "oihw", "acdb").sync()
    with pytest.raises(ValueError):
        conv(x, w, 1, 1, 1, 1, 1, 1, 1, "bacd", "oihw", "")


# (x shape, w shape, stride, padding, dilation, path): weight gradients of bf16 layers. "tc": the tensor-core weight-gradient
# kernel (K = pixels; outputs of at least 8 x 8 per image); "exchanged": the forward kernel on x and dy with batch and channel
# axes exchanged (needs a batch that can serve as the channel axis: a multiple of 8, at least 64).
WGRAD = [
    ((64, 128, 12, 12), (64, 128, 3, 3), 1, 1, 1, "tc"),            # one 128 x 128 accumulator per tap, 16 pixel ranges
    ((72, 256, 9, 11), (64, 256, 1, 1), 1, 0, 1, "tc"),             # 1 x 1 filter, ragged patches
    ((64, 128, 16, 16), (64, 128, 3, 3), 1, 2, 2, "tc"),            # dilation 2
    ((20, 192, 30, 34), (320, 192, 3, 3), 2, 1, 1, "tc"),           # stride 2; ragged channel tiles (128 + 64, 256 + 64)
    ((8, 256, 28, 28), (256, 256, 3, 3), 1, 1, 1, "tc"),            # the 256-wide tile, 18 accumulators x 8 ranges
    ((40, 72, 28, 32), (136, 72, 5, 5), 3, 2, 1, "tc"),             # stride 3, 5 x 5, channel counts that are only multiples of 8
    ((64, 128, 12, 12), (64, 128, 3, 3), 1, 1, 1, "exchanged"),
    ((64, 128, 14, 14), (96, 128, 3, 3), 2, 1, 1, "exchanged"),     # 7 x 7 output: below the dedicated kernel's patch size
    ((64, 128, 16, 16), (64, 128, 3, 3), 1, 2, 2, "exchanged"),
]


@pytest.mark.parametrize("xs,wshape,stride,pad,dil,path", WGRAD)
def test_weight_gradient_on_the_tensor_cores(xs, wshape, stride, pad, dil, path, monkeypatch):
    """Checked against the C restatement of the weight-gradient graph (oracle_conv2d_backward_w_f32, pinned to the reference's
    conv_wgrad fixtures), a float32 torch convolution's gradient and the CUDA-core weight-gradient kernel."""
    import jittor_b200 as jt
    from jittor_b200 import _capi as C, nn
    rng = np.random.default_rng(sum(xs) + sum(wshape) + stride + dil)
    x = bf16_round(rng.normal(size=xs))
    w = bf16_round(rng.normal(size=wshape) * 0.05)
    oh = (xs[2] + 2 * pad - dil * (wshape[2] - 1) - 1) // stride + 1
    ow = (xs[3] + 2 * pad - dil * (wshape[3] - 1) - 1) // stride + 1
    dy = bf16_round(rng.normal(size=(xs[0], wshape[0], oh, ow)) * 0.1)
    xv, wv, dyv = (jt.array(torch.from_numpy(a).bfloat16()) for a in (x, w, dy))
    geo = (stride, stride, pad, pad, dil, dil)
    applies = C.lib.b200jt_conv2d_backward_w_workspace(C.desc(xv.torch()), C.desc(dyv.torch()), C.desc(wv.torch()), *geo)
    if path == "tc":
        assert applies > 0, "case does not reach the tensor-core weight-gradient kernel"
    with jt.flag_scope(b200_wgrad_tc=1 if path == "tc" else 2):
        loss = (nn.conv2d(xv, wv, None, stride, pad, dil) * dyv).sum()
        got = jt.grad(loss, wv).torch().float().cpu().numpy()
        if path == "tc":                                       # one tap per CTA instead of two (K is then split differently: equal within rounding)
            monkeypatch.setenv("B200JT_WGRAD_TAPS", "1")
            loss1 = (nn.conv2d(xv, wv, None, stride, pad, dil) * dyv).sum()
            one_tap = jt.grad(loss1, wv).torch().float().cpu().numpy()
            monkeypatch.delenv("B200JT_WGRAD_TAPS")
            check(got, one_tap, False, rtol=2e-2)
    check(got, bf16_round(co.conv2d_backward_w(x, dy, wshape[2], wshape[3], stride, pad, dil)), False, rtol=2e-2)
    tw = torch.from_numpy(w).cuda().requires_grad_()
    ty = torch.nn.functional.conv2d(torch.from_numpy(x).cuda(), tw, None, stride, pad, dil)
    (ty * torch.from_numpy(dy).cuda()).sum().backward()
    check(got, bf16_round(tw.grad.cpu().numpy()), False, rtol=2e-2)
    with jt.flag_scope(b200_wgrad_tc=0):                       # the CUDA-core kernel agrees (fp32 sums, bf16 result)
        loss2 = (nn.conv2d(xv, wv, None, stride, pad, dil) * dyv).sum()
        simt = jt.grad(loss2, wv).torch().float().cpu().numpy()
    check(got, simt, False, rtol=2e-2)
    if path == "tc":                                           # partial sums are folded in a fixed order: results repeat
        with jt.flag_scope(b200_wgrad_tc=1):
            loss3 = (nn.conv2d(xv, wv, None, stride, pad, dil) * dyv).sum()
            again = jt.grad(loss3, wv).torch().float().cpu().numpy()
        assert np.array_equal(got, again)
    assert C.lib.b200jt_device_status() == 0


WGRAD_LAYOUTS = [
    ((20, 192, 30, 34), (320, 192, 3, 3), 2, 1, "acdb", "oihw", "acdb"),
    ((8, 256, 28, 28), (256, 256, 3, 3), 1, 1, "acdb", "ohwi", "acdb"),
    ((64, 128, 12, 12), (64, 128, 3, 3), 1, 1, "abcd", "ohwi", "acdb"),
    ((72, 256, 9, 11), (64, 256, 1, 1), 1, 0, "acdb", "oihw", "abcd"),
]


@pytest.mark.parametrize("xs,wshape,stride,pad,xf,wf,yf", WGRAD_LAYOUTS)
def test_weight_gradient_layouts_of_the_relay(xs, wshape, stride, pad, xf, wf, yf):
    """cudnn_conv_backward_w with the layout strings ConvTuner derives (python/jittor/src/opt/tuner/conv_tuner.cc:292-341,
    390-396): channels-last x / dy are read as they are, dw comes out in the asked order -- same bits as the abcd / oihw call."""
    import jittor_b200 as jt
    from jittor_b200 import _capi as C
    rng = np.random.default_rng(sum(xs) + sum(wshape) + stride)
    x = bf16_round(rng.normal(size=xs))
    oh = (xs[2] + 2 * pad - (wshape[2] - 1) - 1) // stride + 1
    ow = (xs[3] + 2 * pad - (wshape[3] - 1) - 1) // stride + 1
    dy = bf16_round(rng.normal(size=(xs[0], wshape[0], oh, ow)) * 0.1)
    relay = jt.get_op_info("cudnn_conv_backward_w").get_constructor()
    xv, dyv = jt.array(torch.from_numpy(x).bfloat16()), jt.array(torch.from_numpy(dy).bfloat16())
    want = relay(xv, dyv, wshape[2], wshape[3], stride, stride, pad, pad, 1, 1, 1).torch()
    xin = x if xf == "abcd" else np.ascontiguousarray(x.transpose(0, 2, 3, 1))
    dyin = dy if yf == "abcd" else np.ascontiguousarray(dy.transpose(0, 2, 3, 1))
    got = relay(jt.array(torch.from_numpy(xin).bfloat16()), jt.array(torch.from_numpy(dyin).bfloat16()),
                wshape[2], wshape[3], stride, stride, pad, pad, 1, 1, 1, xf, wf, yf).torch()
    if wf == "ohwi":
        assert list(got.shape) == [wshape[0], wshape[2], wshape[3], wshape[1]]
        got = got.permute(0, 3, 1, 2)
    assert torch.equal(got, want)
    tw = torch.zeros(wshape, device="cuda").requires_grad_()
    ty = torch.nn.functional.conv2d(torch.from_numpy(x).cuda(), tw, None, stride, pad, 1)
    (ty * torch.from_numpy(dy).cuda()).sum().backward()
    check(got.float().cpu().numpy(), bf16_round(tw.grad.cpu().numpy()), False, rtol=2e-2)
    assert C.lib.b200jt_device_status() == 0


def test_weight_gradient_layouts_are_refused_off_the_tensor_core_kernel():
    import jittor_b200 as jt
    from jittor_b200 import _capi as C
    relay = jt.get_op_info("cudnn_conv_backward_w").get_constructor()
    x = jt.array(torch.zeros(2, 8, 8, 16, device="cuda"))                 # float32, 16 channels: CUDA-core territory
    dy = jt.array(torch.zeros(2, 8, 8, 16, device="cuda"))
    with pytest.raises(C.B200Error):
        relay(x, dy, 3, 3, 1, 1, 1, 1, 1, 1, 1, "acdb", "oihw", "acdb").sync()
