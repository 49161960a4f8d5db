"""`jt.flags` and `jt.flag_scope` (python/jittor/__init__.py:138-160).

Only the flags that influence the meta-operator path are interpreted (`amp_reg`, `lazy_execution`);
the others the reference's callers commonly set (`use_cuda`, `enable_tuner`, `use_tensorcore`,
`compile_options`, ...) are accepted and stored so that code written for the reference runs unchanged.
"""
import os


class _Flags:
    _defaults = dict(use_cuda=1, amp_reg=0, amp_level=0, lazy_execution=1, enable_tuner=1, use_tensorcore=0,
                     try_use_32bit_index=1, compile_options={}, exclude_pass="", log_silent=0,
                     use_device_mpi=1,
                     b200_fuse_chains=1,        # 0: run element-wise chains op by op (the fused result has the same bits)
                     b200_wgrad_tc=1)           # weight gradients: 1 tensor-core kernel where it applies, 2 only the exchanged-axes
                                                # convolution, 0 always the CUDA-core kernel (fp32 sums in ascending order)

    def __init__(self):
        object.__setattr__(self, "_v", dict(self._defaults))
        for k, d in self._defaults.items():
            if k in os.environ and isinstance(d, int):
                self._v[k] = int(os.environ[k])

    def __getattr__(self, k):
        try:
            return self._v[k]
        except KeyError:
            raise AttributeError(f"unknown flag {k!r}")

    def __setattr__(self, k, v):
        self._v[k] = v


flags = _Flags()


class flag_scope:
    """Context manager that sets flags for the duration of a block and restores them afterwards."""

    def __init__(self, **kw):
        self.kw = kw

    def __enter__(self):
        self.saved = {k: flags._v.get(k) for k in self.kw}
        for k, v in self.kw.items():
            setattr(flags, k, v)
        return self

    def __exit__(self, *exc):
        for k, v in self.saved.items():
            setattr(flags, k, v)
        return False
