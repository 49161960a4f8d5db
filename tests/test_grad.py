"""Gradients through the meta-operators (the reference's per-op rules) -- graph structure on CPU, values on the GPU
against the reference-made fixtures and against torch autograd (float32 reference of the same expression)."""
import numpy as np
import pytest

import jittor_b200 as jt
from jittor_b200 import nn
from tests import golden_cases as G


def test_duality_of_the_meta_operators():
    x = jt.Var([3, 10], "float32")
    y = x.reindex([3, 14], ["i0", "i1-2"])
    g = jt.grad(y, x)
    assert g._op.kind == "reindex_reduce" and g._op.attrs["op"] == "add" and list(g.shape) == [3, 10]
    z = x.reindex_reduce("add", [3, 4], ["i0", "i1/3"])
    assert jt.grad(z, x)._op.kind == "reindex"
    b = x.broadcast([5, 3, 10], [0])
    gb = jt.grad(b, x)
    assert gb._op.kind == "reduce" and gb._op.attrs["op"] == "add" and list(gb.shape) == [3, 10]
    s = x.sum(1)
    assert jt.grad(s, x)._op.kind == "broadcast_to"
    w = jt.Var([10], "float32")
    gw = jt.grad((x * w).sum(), w)            # implicit broadcast of w is summed back over the rows
    assert list(gw.shape) == [10]
    assert list(jt.grad(x.sum(), jt.Var([2], "float32")).shape) == [2]        # unrelated target: zeros


def _case(name):
    c = [c for c in G.CASES if c["name"] == name][0]
    A = G.arrays()
    return [A[k] for k in c["inputs"]], A[c["out"]], c["args"]


@pytest.mark.gpu
def test_grads_match_reference_fixtures():
    (x, m), want, a = _case("grad_reindex")
    v = jt.array(x)
    got = jt.grad((v.reindex(a["shape"], a["indexes"]) * jt.array(m)).sum(), v).numpy()
    G.check(got, want, False)
    (x, m), want, a = _case("grad_reindex_reduce_add")
    v = jt.array(x)
    got = jt.grad((v.reindex_reduce("add", a["shape"], a["indexes"]) * jt.array(m)).sum(), v).numpy()
    G.check(got, want, False)
    (x, dy), want, _ = _case("maxpool2x2_bwd")
    v = jt.array(x)
    got = jt.grad((nn.max_pool2x2(v) * jt.array(dy)).sum(), v).numpy()
    G.check(got, want, False)


@pytest.mark.gpu
def test_grads_match_torch_autograd():
    import torch
    import torch.nn.functional as F
    rng = np.random.default_rng(3)

    def close(a, b, tol=1e-4):
        b = b.detach().cpu().numpy()
        assert np.abs(a - b).max() <= tol * (1 + np.abs(b).max()), np.abs(a - b).max()

    # conv2d: data and weight gradients
    x, w = rng.normal(size=(2, 3, 8, 8)).astype(np.float32), rng.normal(size=(4, 3, 3, 3)).astype(np.float32)
    m = rng.normal(size=(2, 4, 8, 8)).astype(np.float32)
    vx, vw = jt.array(x), jt.array(w)
    dx, dw = jt.grad((nn.conv2d(vx, vw, None, 1, 1, 1) * jt.array(m)).sum(), [vx, vw])
    tx, tw = torch.tensor(x, requires_grad=True), torch.tensor(w, requires_grad=True)
    (F.conv2d(tx, tw, padding=1) * torch.tensor(m)).sum().backward()
    close(dx.numpy(), tx.grad)
    close(dw.numpy(), tw.grad)
    # matmul, softmax, layer norm
    a, b = rng.normal(size=(9, 7)).astype(np.float32), rng.normal(size=(7, 5)).astype(np.float32)
    va, vb = jt.array(a), jt.array(b)
    mm = rng.normal(size=(9, 5)).astype(np.float32)
    da, db = jt.grad((nn.matmul(va, vb) * jt.array(mm)).sum(), [va, vb])
    ta, tb = torch.tensor(a, requires_grad=True), torch.tensor(b, requires_grad=True)
    ((ta @ tb) * torch.tensor(mm)).sum().backward()
    close(da.numpy(), ta.grad)
    close(db.numpy(), tb.grad)
    xs = rng.normal(size=(6, 33)).astype(np.float32)
    ms = rng.normal(size=(6, 33)).astype(np.float32)
    vs = jt.array(xs)
    ds = jt.grad((nn.softmax(vs, -1) * jt.array(ms)).sum(), vs)
    ts = torch.tensor(xs, requires_grad=True)
    (torch.softmax(ts, -1) * torch.tensor(ms)).sum().backward()
    close(ds.numpy(), ts.grad)
    g, bb = rng.normal(size=33).astype(np.float32), rng.normal(size=33).astype(np.float32)
    vg, vbb = jt.array(g), jt.array(bb)
    dl, dg = jt.grad((nn.layer_norm(vs, (33,), vg, vbb) * jt.array(ms)).sum(), [vs, vg])
    ts2, tg = torch.tensor(xs, requires_grad=True), torch.tensor(g, requires_grad=True)
    (F.layer_norm(ts2, (33,), tg, torch.tensor(bb)) * torch.tensor(ms)).sum().backward()
    close(dl.numpy(), ts2.grad, 1e-3)
    close(dg.numpy(), tg.grad, 1e-3)
