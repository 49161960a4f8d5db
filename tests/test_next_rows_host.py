"""Host logic of the callers of the path, on placeholder Vars (no GPU): pooling shapes / checks and route selection,
grouped and transposed convolution graphs, conv gradient pattern recognition, optimiser bookkeeping."""
import pytest

import jittor_b200 as jt
from jittor_b200 import executor, nn, optim, pool


def test_pool_shapes_routes_and_errors():
    x = jt.Var([2, 3, 10, 11], "float32")
    y = pool.max_pool2d(x, 3, 2, 1)
    assert list(y.shape) == [2, 3, 5, 6] and y._op.kind == "custom" and y._op.attrs["name"] == "pool2d"
    y = pool.max_pool2d(x, 3, 2, 1, ceil_mode=True)
    assert list(y.shape) == [2, 3, 6, 6]
    # mean in floor mode stays the meta-operator lowering (python/jittor/pool.py:46-50,187-197); ceil mode uses the kernel
    y = pool.avg_pool2d(x, 2)
    assert list(y.shape) == [2, 3, 5, 5] and y._op.kind == "reduce" and y._op.inputs[0]._op.kind == "reindex"
    assert pool.avg_pool2d(x, 2, ceil_mode=True)._op.kind == "custom"
    y, idx = pool.max_pool2d(x, 2, return_indices=True)
    assert str(idx.dtype) == "int32" and list(idx.shape) == list(y.shape)
    with pytest.raises(RuntimeError, match="kernel_size"):
        pool.Pool(0)
    with pytest.raises(RuntimeError, match="stride"):
        pool.Pool(2, -1)
    with pytest.raises(RuntimeError, match="padding"):
        pool.Pool(2, 2, -1)
    with pytest.raises(RuntimeError, match="larger than kernel_size"):
        pool.max_pool2d(jt.Var([1, 1, 3, 3], "float32"), 3)
    saved = pool.pool_use_code_op
    try:
        pool.pool_use_code_op = False
        assert pool.max_pool2d(x, 3, 2, 1)._op.kind == "reduce"
    finally:
        pool.pool_use_code_op = saved
    # the pooling relay brings its own gradient
    g = jt.grad(pool.max_pool2d(x, 3, 2, 1), x)
    assert list(g.shape) == [2, 3, 10, 11] and g._op.attrs["name"] == "pool2d_backward"


def test_grouped_and_transposed_conv_graphs():
    x = jt.Var([2, 8, 9, 9], "float32")
    y = nn.conv2d(x, jt.Var([12, 2, 3, 3], "float32"), None, 2, 1, 1, groups=4)
    assert list(y.shape) == [2, 12, 5, 5] and y._op.kind == "reindex_reduce" and y._relay[0] == "conv2d" and y._relay[4] == 4
    plan = executor._make_plan(y)
    assert plan.leaves == [y._relay[1], y._relay[2]]
    y = nn.conv_transpose2d(x, jt.Var([8, 5, 3, 3], "float32"), None, 2, 1, 1)
    assert list(y.shape) == [2, 5, 18, 18] and y._relay[0] == "conv2d_transpose"
    y = nn.conv_transpose2d(x, jt.Var([8, 3, 4, 4], "float32"), jt.Var([6], "float32"), 2, 1, 0, groups=2)
    assert list(y.shape) == [2, 6, 18, 18] and y._op.kind == "binary"          # bias add on top of the relayed Var
    with pytest.raises(AssertionError, match="output padding"):
        nn.conv_transpose2d(x, jt.Var([8, 5, 3, 3], "float32"), None, 2, 1, 2)


def test_conv_gradient_graphs_are_recognised():
    x, w = jt.Var([4, 8, 10, 12], "float32"), jt.Var([16, 8, 3, 3], "float32")
    y = nn.conv2d(x, w, None, 2, 1, 1)
    dy = jt.Var(list(y.shape), "float32")
    dx, dw = jt.grad((y * dy).sum(), [x, w])
    p = executor._match_conv_dgrad(dx)
    assert p is not None and p.leaves[1] is w
    p = executor._match_conv_wgrad(dw)
    assert p is not None and p.leaves[0] is x
    # stride-1 bf16: the data gradient becomes a convolution with flipped, transposed weights (a reindex of w)
    xb, wb = jt.Var([4, 64, 16, 16], "bfloat16"), jt.Var([64, 64, 3, 3], "bfloat16")
    dxb, dwb = jt.grad(nn.conv2d(xb, wb, None, 1, 1, 1), [xb, wb])
    p = executor._match_conv_dgrad(dxb)
    assert p is not None and p.leaves[1]._op.kind == "reindex" and p.leaves[1]._op.attrs["indexes"] == ["i1", "i0", "2-i2", "2-i3"]
    assert executor._match_conv_wgrad(dwb._op.inputs[0]) is not None          # under the cast back to bfloat16
    # a different reduce mask is not a weight gradient
    assert executor._match_conv_wgrad(y) is None and executor._match_conv_dgrad(y) is None


def test_optimizer_bookkeeping_without_a_device():
    a, b = jt.Var([3], "float32"), jt.Var([2, 2], "float32").stop_grad()
    opt = optim.SGD([a, b], lr=0.1, momentum=0.9)
    assert len(opt.param_groups) == 1 and len(opt.param_groups[0]["values"]) == 2
    assert b.is_stop_grad() and not a.is_stop_grad()
    opt.add_param_group({"params": [jt.Var([5], "float32")], "lr": 0.01})
    assert len(opt.param_groups) == 2 and opt.param_groups[1]["lr"] == 0.01
    with pytest.raises(RuntimeError, match="not managed"):
        opt.find_grad(jt.Var([1], "float32"))
    with pytest.raises(AssertionError):
        optim.SGD([], lr=0.1)

    class Leaf(nn.Module):
        def __init__(self, n):
            self.weight, self.bias = jt.Var([n], "float32"), jt.Var([n], "float32")

    class Net(nn.Module):
        def __init__(self):
            self.first = Leaf(3)
            self.blocks = [Leaf(4), {"head": Leaf(2)}]
            self.shared = self.first.weight            # the same Var twice is one parameter

    assert len(Net().parameters()) == 6


def test_pooling_lowering_is_recognised():
    """reduce over [4,5] of the window reindex (python/jittor/pool.py:187-197, :419-432) becomes one pooling launch;
    maximum with padding is not relayed (the lowering reads padding as 0, the kernel clips the window)."""
    x = jt.Var([2, 3, 10, 12], "float32")
    assert executor._match_pool(pool.avg_pool2d(x, 2)) is not None
    assert executor._match_pool(pool.avg_pool2d(x, 3, 2, 1)) is not None
    assert executor._match_pool(pool.AdaptiveAvgPool2d(5)(x)) is not None
    assert executor._match_pool(pool.AdaptiveMaxPool2d((5, 3))(x)) is not None
    saved = pool.pool_use_code_op
    try:
        pool.pool_use_code_op = False
        assert executor._match_pool(pool.max_pool2d(x, 2, 2, 0)) is not None
        assert executor._match_pool(pool.max_pool2d(x, 3, 2, 1)) is None
    finally:
        pool.pool_use_code_op = saved
    assert executor._match_pool(x.reindex([2, 3, 5, 6, 2, 2], ["i0", "i1", "i2*2+i4", "i3*2+i5"]).sum([4, 5])) is None
    # 16-bit mean: cast(float32) -> reduce -> cast back (reduce_op.cc:260-266); the inner reduce is the relayed node
    bf = jt.Var([2, 3, 10, 12], "bfloat16")
    y = pool.avg_pool2d(bf, 2)
    assert str(y.dtype) == "bfloat16" and y._op.kind == "unary"
    assert executor._match_pool(y._op.inputs[0]) is not None


def test_conv2d_writes_its_graph_only_when_it_is_read():
    """nn.conv2d returns a Var that can be planned from its relay record; the four-op meta-operator graph appears when
    something reads the producer (jt.grad, a consumer's pattern match) and is the one the eager construction makes."""
    x, w = jt.Var([4, 32, 32, 32], "float32"), jt.Var([64, 32, 3, 3], "float32")
    y = nn.conv2d(x, w, None, 2, 1, 1)
    assert "_op" not in y.__dict__ and list(y.shape) == [4, 64, 16, 16] and y.dtype == "float32"
    p = executor._make_plan(y)
    assert p.leaves[0] is x and p.leaves[1] is w and "_op" not in y.__dict__          # planned without the graph
    op = y._op                                                                        # now it is written
    assert op.kind == "reduce" and op.attrs["reduce_mask"] == 0b1100100
    mul = op.inputs[0]
    assert mul._op.kind == "binary" and {i._op.kind for i in mul._op.inputs} == {"reindex", "broadcast_to"}
    assert y._op is op                                                                # once
    assert executor._match_conv(y) is not None                                        # the search finds the same operands
    for dtype in ("bfloat16", "float16"):
        for amp in (0, 2, 4, 16):
            with jt.flag_scope(amp_reg=amp):
                xb, wb = jt.Var([4, 64, 16, 16], dtype), jt.Var([64, 64, 3, 3], dtype)
                yb = nn.conv2d(xb, wb, None, 1, 1, 1)
                with jt.flag_scope(amp_reg=amp | 36):
                    eager = (xb.reindex([4, 64, 64, 16, 16, 3, 3], ["i0", "i2", "i3*1-1+i5*1", "i4*1-1+i6*1"])
                             * wb.broadcast([4, 64, 64, 16, 16, 3, 3], [0, 3, 4])).sum([2, 5, 6])
                assert str(yb.dtype) == str(eager.dtype) and yb._op.kind == eager._op.kind
