"""The allocation-free scatter entry point, called straight through the C ABI.

It exists for callers that cannot allocate device memory at call time (allocator callbacks, loops with a
frozen memory pool, plugin hosts without an allocation hook): its scratch is an array inside the library.
The test runs it twice in a row on the same inputs (the built-in array keeps what the previous call left in it)
and compares each result with the CPU oracle's scatter loop and with the regular entry point (caller-provided
workspace): bit-exact for int32, and the fp32 tolerance of the other parity tests
(|d| <= 1e-5*|ref| + 1e-5*max|ref|), because the order of shared-memory atomics is not fixed.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _scatter(C, fn_name, val, idx, bins, workspace=None):
    out = torch.empty(bins, dtype=val.dtype, device="cuda")
    idx_s, none_s = C.strings(["@e0(i0)"]), C.strings([])
    args = [C.desc(val), C.desc(out), b"add", idx_s, 1, none_s, 0, C.descs([idx]), 1]
    if fn_name == "b200jt_reindex_reduce":
        nbytes = C.lib.b200jt_reindex_reduce_workspace(*args)
        ws = torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device="cuda")
        args += [ctypes.c_void_p(ws.data_ptr()), nbytes]
    rc = getattr(C.lib, fn_name)(*args, C.stream_ptr())
    torch.cuda.synchronize()
    return rc, out


@pytest.mark.parametrize("dtype,bins", [(torch.float32, 4096), (torch.int32, 4096), (torch.float32, 1000), (torch.int32, 1 << 16)])
def test_noalloc_matches_workspace_entry_point_twice(dtype, bins):
    from jittor_b200 import _capi as C
    g = torch.Generator("cuda").manual_seed(bins)
    n = (1 << 20) + 3
    idx = torch.randint(0, bins, (n,), device="cuda", dtype=torch.int32, generator=g)
    val = (torch.randn(n, device="cuda", generator=g) if dtype == torch.float32
           else torch.randint(0, 100, (n,), device="cuda", dtype=torch.int32, generator=g))
    from oracle import c_oracle as co
    rc, want = _scatter(C, "b200jt_reindex_reduce", val, idx, bins)
    assert rc == 0, C.lib.b200jt_last_error()
    oracle = torch.from_numpy(co.scatter_add(val.cpu().numpy(), idx.cpu().numpy(), bins)).cuda()
    for _ in range(2):                                   # the scratch keeps the previous call's rows
        rc, got = _scatter(C, "b200jt_reindex_reduce_noalloc", val, idx, bins)
        assert rc == 0, C.lib.b200jt_last_error()
        for ref in (oracle, want):
            if dtype == torch.int32:
                assert torch.equal(got, ref)
            else:
                w = ref.double()
                tol = 1e-5 * w.abs() + 1e-5 * w.abs().max()
                assert bool(((got.double() - w).abs() <= tol).all())


def test_noalloc_rejects_scratch_beyond_the_builtin_array():
    from jittor_b200 import _capi as C
    bins = 8000                                          # 148 rows * 8000 * 4 B > 4 MiB
    n = 1 << 17
    idx = torch.randint(0, bins, (n,), device="cuda", dtype=torch.int32)
    val = torch.randn(n, device="cuda")
    assert 148 * bins * 4 > C.lib.b200jt_reindex_reduce_noalloc_max_scratch()
    rc, _ = _scatter(C, "b200jt_reindex_reduce_noalloc", val, idx, bins)
    assert rc == -3
    assert b"scratch" in C.lib.b200jt_last_error()
    rc, _ = _scatter(C, "b200jt_reindex_reduce", val, idx, bins)       # the regular entry point still serves it
    assert rc == 0
