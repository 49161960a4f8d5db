"""Benchmark of the meta-operator hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c4|c5|meta|fused|next] [--impl reference]

One JSON line on stdout (rank 0). The default run measures c2 (the headline keys of the line) and then c1, c3, c4, c5 and
the meta / fused / next sets with the same method into "workloads"; --workload X measures X alone. Workloads are the benchmark configurations:
    c1            reindex-lowered conv2d fp32 [4,32,32,32] * [64,32,3,3], L2 flushed before every repetition    (GB/s and TFLOP/s)
    c2 (default)  reindex_reduce scatter: 2^24 int32 -> 2^20 bins and 2^24 fp32 -> 4096 bins, uniform and Zipf(1.1)
                  indices, plus the 2x2 max-pool backward [64,128,56,56,2,2] -> [64,128,112,112]      (GB/s, HBM)
    c3            fused row softmax and LayerNorm on [32768, 4096], fp32 and bf16 IO                  (GB/s, HBM)
    c4            broadcast-multiply-sum matmul, bf16: 8192^3 and 16384 x 4096 x 4096                 (TFLOP/s)
    c5            reindex conv2d bf16 [256,256,56,56] * [256,256,3,3] -> global BatchNorm statistics (one all-reduce
                  of 2*C floats) -> normalise + ReLU, batch-sharded over the ranks                     (TFLOP/s)
    meta          the meta-operators on their own on [32768,4096] fp32 (reindex pad / transpose / conv window, row and
                  column sum, broadcast add)                                                           (GB/s, HBM)
    fused         general element-wise chains as one compiled kernel each (x*w+b, relu(x+b), (a*b).sum(1),
                  centre-and-scale) and the softmax backward, [32768,4096] fp32                        (GB/s, HBM)
    next          callers of the path: 3x3 s2 max-pool forward / backward, getitem row gather, setitem scatter-add (GB/s)
One step = one pass over the parts of the workload. `value` is algorithmic work / CUDA-event time with inputs
resident in HBM (max over ranks); `e2e` is the same step through the public API from pinned host buffers including
host->device copies and the device->host read of the results. Every part works on more bytes than the 126 MB L2
and the parts rotate, so no L2 flush is issued (stated in `config`). `--impl reference` times the CPU restatement of the
reference's loop nests (oracle/meta_ops.c) on the host cores, on a bounded sample. With N > 1 (torchrun) c2-c4 give every
rank its own inputs (weak scaling; c2 all-reduces the scatter bins), c5 splits the batch (strong scaling).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def zipf_indices(rng, n, bins, s=1.1):
    """Inverse-CDF draw from the truncated Zipf(s) over bin ranks; rank -> bin by a fixed permutation."""
    p = np.arange(1, bins + 1, dtype=np.float64) ** (-s)
    cdf = np.cumsum(p / p.sum())
    rank = np.minimum(np.searchsorted(cdf, rng.random(n)), bins - 1)
    return rng.permutation(bins)[rank].astype(np.int32)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.stop = index, [], False
        self.t = threading.Thread(target=self.run, daemon=True)

    def run(self):
        while not self.stop:
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([f.strip() for f in out.split(",")])
            except Exception:
                pass
            time.sleep(0.05)

    def __enter__(self):
        self.t.start()
        return self

    def __exit__(self, *a):
        self.stop = True
        self.t.join(timeout=6)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        mhz = sorted(float(s[0]) for s in self.samples)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": float(self.samples[0][1]), "reasons": reasons,
                "samples": len(self.samples), "window": "timed region and untimed repeats of the same step"}


# =====================================================================================================
# Workloads. A workload knows its parts, the algorithmic work of each (bytes or FLOP), how to run a part on
# device-resident inputs or from pinned host buffers, and how to run a bounded sample of it on the CPU oracle.
# =====================================================================================================
class C1ConvF32:
    """Config 0: the reindex-lowered conv2d in fp32 at the size the reference's CPU path runs. 1.6 MB of operands: the
    whole problem sits in L2, so L2 is flushed (a 256 MB fill) before every timed repetition."""
    key, metric, unit, bound, dtype, scaling = "c1", "meta-op GB/s", "GB/s", "hbm", "f32", "weak"
    N, C, H, W, CO = 4, 32, 32, 32, 64
    description = ("config 0: reindex-lowered conv2d fp32 [4,32,32,32] * [64,32,3,3] s1 p1 "
                   "(reindex -> broadcast -> multiply -> sum over [Cin,Kh,Kw], recognised and run as one CUDA-core implicit GEMM)")
    kernel_of = {"conv-f32": "gemm_simt_deep_kernel<float, ConvLoader, 32, 32>"}
    launches = {"conv-f32": 1}
    flush_l2 = True
    FLOP = 2 * 4 * 64 * 32 * 32 * 32 * 9

    def work(self):
        return {"conv-f32": 4 * (self.N * self.C * self.H * self.W + self.CO * self.C * 9 + self.N * self.CO * self.H * self.W)}

    def host_inputs(self, seed):
        rng = np.random.default_rng(seed)
        x = rng.uniform(-1, 1, size=(self.N, self.C, self.H, self.W)).astype(np.float32)
        w = (rng.normal(size=(self.CO, self.C, 3, 3)) * 0.05).astype(np.float32)
        return x, w

    def setup(self, rank, world, jt, torch, multi):
        from jittor_b200 import nn
        self.jt, self.torch, self.nn = jt, torch, nn
        x, w = self.host_inputs(0 + rank)
        self.hx, self.hw = torch.from_numpy(x).pin_memory(), torch.from_numpy(w).pin_memory()
        self.x, self.w = jt.array(self.hx), jt.array(self.hw)
        self.out = torch.empty(self.N, self.CO, self.H, self.W).pin_memory()
        return ["conv-f32"]

    def run(self, name):
        return self.nn.conv2d(self.x, self.w, None, 1, 1, 1).sync()

    def run_e2e(self, name):
        x, w = self.jt.array(self.hx.cuda(non_blocking=True)), self.jt.array(self.hw.cuda(non_blocking=True))
        self.nn.conv2d(x, w, None, 1, 1, 1).fetch_into(self.out, stream=self.d2h_stream)

    def e2e_bytes(self, names):
        return (self.hx.numel() + self.hw.numel()) * 4, self.out.numel() * 4

    def extra(self, part_ms):
        return {"TFLOP/s": self.FLOP / part_ms["conv-f32"] / 1e9, "flop_per_step": self.FLOP, "launch_path": self.launch_path()}

    def launch_path(self, calls=300):
        """The public call WITHOUT a CUDA graph, back to back: wall-clock per call until the call returns (Python builds
        the four-op graph, plans it and launches) and until the GPU has finished all of them."""
        for _ in range(20):
            self.run("conv-f32")
        self.torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(calls):
            self.run("conv-f32")
        t1 = time.perf_counter()
        self.torch.cuda.synchronize()
        t2 = time.perf_counter()
        return {"calls": calls, "us_per_call_returned": (t1 - t0) / calls * 1e6, "us_per_call_finished": (t2 - t0) / calls * 1e6,
                "what": "nn.conv2d(x, w).sync() launched directly, no CUDA graph, no L2 flush between calls"}

    def verify(self, env):
        from oracle import c_oracle as co
        x, w = self.host_inputs(0 + env["rank"])
        got = self.run("conv-f32").numpy()
        want = co.conv2d(x, w, 1, 1, 1)
        return bool((np.abs(got - want) <= 1e-5 * np.abs(want) + 1e-5 * np.abs(want).max()).all())

    def cpu(self, names):
        from oracle import c_oracle as co
        x, w = self.host_inputs(0)
        reps, t0 = 20, time.perf_counter()
        for _ in range(reps):
            co.conv2d(x, w, 1, 1, 1)
        return self.work()["conv-f32"] * reps, time.perf_counter() - t0, f"full size, {reps} repetitions (OpenMP over image x channel)"


class C2Scatter:
    key, metric, unit, bound, dtype, scaling = "c2", "meta-op GB/s", "GB/s", "hbm", "int32/f32", "weak"
    N_VAL, BINS_A, BINS_B = 1 << 24, 1 << 20, 4096
    POOL_SHAPE = (64, 128, 56, 56, 2, 2)
    POOL_IDX = ["i0", "i1", "i2*2+i4", "i3*2+i5"]
    description = ("config 1: reindex_reduce scatter-add 2^24 -> 2^20 int32 and -> 4096 fp32 (uniform + Zipf 1.1 "
                   "indices) + 2x2 max-pool backward [64,128,112,112] fp32")
    kernel_of = {"a-uniform": "rr_direct_cached_kernel<int,int,4>", "a-zipf": "rr_direct_cached_kernel<int,int,4>",
                 "b-uniform": "rr_privatised_kernel<float,int,4>", "b-zipf": "rr_privatised_kernel<float,int,4>",
                 "pool-bwd": "rr_flat_kernel<float>"}
    launches = {"a-uniform": 2, "a-zipf": 2, "b-uniform": 2, "b-zipf": 2, "pool-bwd": 1}
    all_reduced = ("a-uniform", "a-zipf", "b-uniform", "b-zipf")     # parts whose output is summed over the ranks
    # DRAM bytes (read + written) of the main kernel per launch, from the ncu captures summarised under profiles/
    traffic = {"a-uniform": 144.5e6, "a-zipf": 147.3e6, "b-uniform": 137.6e6, "b-zipf": 137.7e6, "pool-bwd": 776.2e6}

    def work(self):
        pool = int(np.prod(self.POOL_SHAPE)) * 4
        n = self.N_VAL
        return {"a-uniform": n * 8 + self.BINS_A * 4, "a-zipf": n * 8 + self.BINS_A * 4,
                "b-uniform": n * 8 + self.BINS_B * 4, "b-zipf": n * 8 + self.BINS_B * 4, "pool-bwd": 2 * pool}

    def host_inputs(self, seed, pool_images=None):
        rng = np.random.default_rng(seed)       # seed = config index (+ rank)
        n = self.N_VAL
        vi = rng.integers(0, 100, size=n).astype(np.int32)
        vf = rng.normal(size=n).astype(np.float32)
        pshape = (pool_images or self.POOL_SHAPE[0],) + self.POOL_SHAPE[1:]
        # pool gradient: N(0,1) where the element is its window's arg-max, else 0 (what the max-reduce grad emits)
        g = rng.normal(size=pshape).astype(np.float32)
        keep = rng.integers(0, 4, size=pshape[:4])
        mask = np.zeros(pshape[:4] + (4,), dtype=bool)
        np.put_along_axis(mask, keep[..., None], True, axis=-1)
        g *= mask.reshape(pshape)
        return {"a-uniform": (vi, rng.integers(0, self.BINS_A, size=n).astype(np.int32), self.BINS_A),
                "a-zipf": (vi, zipf_indices(rng, n, self.BINS_A), self.BINS_A),
                "b-uniform": (vf, rng.integers(0, self.BINS_B, size=n).astype(np.int32), self.BINS_B),
                "b-zipf": (vf, zipf_indices(rng, n, self.BINS_B), self.BINS_B),
                "pool-bwd": (g, None, None)}

    def setup(self, rank, world, jt, torch, multi):
        self.jt, self.torch, self.multi = jt, torch, multi
        self.host = self.host_inputs(1 + rank)
        self.pinned = {k: tuple(torch.from_numpy(a).pin_memory() if a is not None else None for a in v[:2]) + (v[2],)
                       for k, v in self.host.items()}
        self.dev = {k: (jt.array(v[0]), jt.array(v[1]) if v[1] is not None else None, v[2])
                    for k, v in self.pinned.items()}
        sizes = {"a-uniform": self.BINS_A, "a-zipf": self.BINS_A, "b-uniform": self.BINS_B, "b-zipf": self.BINS_B,
                 "pool-bwd": int(np.prod(self.POOL_SHAPE))}
        self.out_host = {k: torch.empty(n, dtype=torch.int32 if k.startswith("a-") else torch.float32).pin_memory()
                         for k, n in sizes.items()}
        return list(self.dev)

    def _scatter(self, val, idx, bins):
        if idx is None:
            return val.reindex_reduce("add", list(self.POOL_SHAPE[:2]) + [112, 112], self.POOL_IDX)
        out = val.reindex_reduce("add", [bins], ["@e0(i0)"], extras=[idx])
        return out.mpi_all_reduce("add") if self.multi else out      # shared output across ranks

    def extra(self, part_ms):
        """The atomic units' measured rates beside the HBM fractions: a scatter that issues one red.global per element
        (parts a-*) cannot run faster than 2^24 / red_global; the fp32 parts lean on shared-memory float adds."""
        import ctypes
        C = self.jt._capi
        scratch = self.torch.empty(self.BINS_A, dtype=self.torch.int32, device="cuda")
        rates = {}
        for what, skew in (("red_global", 0), ("smem_int", 0), ("smem_int", 1), ("smem_float", 0), ("smem_float", 1), ("match_any", 0)):
            g = ctypes.c_double()
            C.check(C.lib.b200jt_probe_rate(what.encode(), skew, ctypes.c_void_p(scratch.data_ptr()), self.BINS_A, ctypes.byref(g)), "probe")
            rates[what + ("_skewed" if skew else "")] = round(g.value, 1)
        floor_ms = self.N_VAL / (rates["red_global"] * 1e9) * 1e3
        out = {"atomic_rates_gops": rates, "red_global_floor_ms": floor_ms}
        if "a-uniform" in part_ms:
            out["a_uniform_frac_of_atomic_ceiling"] = floor_ms / part_ms["a-uniform"]
        return out

    def step_context(self):
        """The bins' all-reduce of one part runs beside the scatter kernel of the next part (side stream, a few CTAs)."""
        from jittor_b200 import dist
        return dist.overlap_collectives()

    def run(self, name):
        return self._scatter(*self.dev[name]).sync()

    def run_step(self, names, overlap):
        """One step as the timed region runs it. N > 1: the four bins' all-reduces are held back while the scatter kernels
        run (no rank is tied to another in between) and issued together on the side stream when the last scatter has been
        launched, so that the exchange runs beside the pooling gradient, which needs no collective."""
        from jittor_b200 import dist
        if not (overlap and self.multi):
            return [self.run(nm) for nm in names]
        with dist.overlap_collectives(defer=True) as scope:
            keep = []
            for nm in names:
                if nm == "pool-bwd":
                    scope.flush()
                keep.append(self.run(nm))
            return keep

    def run_e2e(self, name):
        hv, hi, bins = self.pinned[name]
        v = self.jt.array(hv.cuda(non_blocking=True))
        i = self.jt.array(hi.cuda(non_blocking=True)) if hi is not None else None
        self._scatter(v, i, bins).fetch_into(self.out_host[name], stream=self.d2h_stream)

    def e2e_bytes(self, names):
        h2d = sum(a.numel() * a.element_size() for n in names for a in self.pinned[n][:2] if a is not None)
        return h2d, sum(self.out_host[n].numel() * 4 for n in names)

    def verify(self, env):
        """Untimed correctness witness. One GPU: the int32 bins equal the CPU oracle's. Several GPUs: the all-reduced bins
        equal the rank-ordered sum of the ranks' own bins (gathered with NCCL): bit-exact for both dtypes."""
        torch = self.torch
        ok = True
        for name in ("a-uniform", "b-zipf"):
            val, idx, bins = self.dev[name]
            local = val.reindex_reduce("add", [bins], ["@e0(i0)"], extras=[idx]).torch().clone()
            if not env["multi"]:
                if name.startswith("a-"):
                    from oracle import c_oracle as co
                    ok = ok and bool(np.array_equal(local.cpu().numpy(), co.scatter_add(self.host[name][0], self.host[name][1], bins)))
                continue
            tdist = env["tdist"]
            mine = self.jt.array(local).mpi_all_reduce("add").torch()
            everyone = [torch.empty_like(local) for _ in range(env["world"])]
            tdist.all_gather(everyone, local)
            want = everyone[0].clone()
            for t in everyone[1:]:
                want = want + t
            ok = ok and bool(torch.equal(mine, want))
            if name.startswith("a-"):               # the whole pipeline once more: scatter + all-reduce of integers is exact
                ok = ok and bool(torch.equal(self._scatter(val, idx, bins).torch(), want))
        return ok

    def cpu(self, names):
        from oracle import c_oracle as co
        host = getattr(self, "host", None) or self.host_inputs(1, 8)
        self.host = host
        work, done = self.work(), 0
        t0 = time.perf_counter()
        for nm in names:
            v, i, b = host[nm]
            if i is None:
                co.pool2x2_bwd(v[:8])
                done += work[nm] * 8 // self.POOL_SHAPE[0]
            else:
                co.scatter_add(v, i, b)
                done += work[nm]
        return done, time.perf_counter() - t0, ("scatter parts at full size + 8 of 64 pool-bwd images; the scatter loop is "
                                                "serial in the reference (1 core), pool-bwd uses OpenMP")


class C3Rows:
    key, metric, unit, bound, dtype, scaling = "c3", "meta-op GB/s", "GB/s", "hbm", "f32 (bf16 IO variants)", "weak"
    ROWS, COLS = 32768, 4096
    description = "config 2: fused row softmax and LayerNorm on [32768,4096], fp32 and bf16 IO with fp32 math"
    kernel_of = {k: "row_reg_kernel" for k in ("softmax-f32", "layernorm-f32", "softmax-bf16", "layernorm-bf16")}
    launches = {k: 1 for k in kernel_of}
    traffic = {"softmax-f32": 1023.4e6, "layernorm-f32": 1023.3e6, "softmax-bf16": 488.3e6, "layernorm-bf16": 488.1e6}

    def work(self):
        n = self.ROWS * self.COLS
        return {"softmax-f32": 8 * n, "layernorm-f32": 8 * n, "softmax-bf16": 4 * n, "layernorm-bf16": 4 * n}

    def setup(self, rank, world, jt, torch, multi):
        from jittor_b200 import nn
        self.jt, self.torch, self.nn = jt, torch, nn
        g = torch.Generator().manual_seed(2 + rank)
        x = torch.randn(self.ROWS, self.COLS, generator=g)
        self.h32 = x.pin_memory()
        self.h16 = x.bfloat16().pin_memory()
        # two device copies per dtype so that consecutive parts never reuse a buffer that is still in L2
        self.x32 = [jt.array(self.h32), jt.array(self.h32.clone())]
        self.x16 = [jt.array(self.h16), jt.array(self.h16.clone())]
        self.gamma = jt.array((1 + 0.02 * torch.randn(self.COLS, generator=g)))
        self.beta = jt.array(torch.zeros(self.COLS))
        self.o32 = torch.empty(self.ROWS, self.COLS).pin_memory()
        self.o16 = torch.empty(self.ROWS, self.COLS, dtype=torch.bfloat16).pin_memory()
        return list(self.kernel_of)

    def _op(self, name, x):
        if name.startswith("softmax"):
            return self.nn.softmax(x, -1)
        return self.nn.layer_norm(x, (self.COLS,), self.gamma, self.beta)

    def run(self, name):
        x = (self.x32 if name.endswith("f32") else self.x16)[0 if name.startswith("softmax") else 1]
        return self._op(name, x).sync()

    def run_e2e(self, name):
        f32 = name.endswith("f32")
        x = self.jt.array((self.h32 if f32 else self.h16).cuda(non_blocking=True))
        self._op(name, x).fetch_into(self.o32 if f32 else self.o16, stream=self.d2h_stream)

    def e2e_bytes(self, names):
        n = self.ROWS * self.COLS
        b = sum(4 * n if nm.endswith("f32") else 2 * n for nm in names)
        return b, b

    def verify(self, env):
        """Untimed correctness witness: 64 sampled rows of every part against the CPU oracle's row loops (fp32 1e-5 mixed;
        bf16 IO: inputs are the bf16 values, result compared after rounding, 2e-2 mixed)."""
        from oracle import c_oracle as co
        torch = self.torch
        pick = torch.randperm(self.ROWS, generator=torch.Generator().manual_seed(5))[:64]
        g, b = self.gamma.numpy(), self.beta.numpy()
        ok = True
        for name in self.kernel_of:
            f32 = name.endswith("f32")
            src = (self.h32 if f32 else self.h16)[pick].float().numpy()
            got = self.run(name).torch()[pick.cuda()].float().cpu().numpy()
            want = co.softmax_rows(src) if name.startswith("softmax") else co.layernorm_rows(src, g, b)
            if not f32:
                want = torch.from_numpy(want).bfloat16().float().numpy()
            rtol = 1e-5 if f32 else 2e-2
            ok = ok and bool((np.abs(got - want) <= rtol * np.abs(want) + rtol * np.abs(want).max()).all())
        return ok

    def cpu(self, names):
        from oracle import c_oracle as co
        rows = 2048
        x = np.random.default_rng(2).normal(size=(rows, self.COLS)).astype(np.float32)
        g, z = np.ones(self.COLS, np.float32), np.zeros(self.COLS, np.float32)
        done, t0 = 0, time.perf_counter()
        for nm in names:
            if nm.startswith("softmax"):
                co.softmax_rows(x)
            else:
                co.layernorm_rows(x, g, z)
            done += self.work()[nm] * rows // self.ROWS
        return done, time.perf_counter() - t0, f"{rows} of {self.ROWS} rows per part, fp32 math (OpenMP over rows)"


class C4Matmul:
    key, metric, unit, bound, dtype, scaling = "c4", "matmul TFLOP/s", "TFLOP/s", "tensor", "bf16 (fp32 accumulate)", "weak"
    SHAPES = {"8192x8192x8192": (8192, 8192, 8192), "16384x4096x4096": (16384, 4096, 4096)}
    description = "config 3: broadcast-multiply-sum matmul A[M,K] x B[K,N], bf16 inputs ~ N(0,1/K), fp32 accumulate"
    kernel_of = {k: "gemm_bf16_kernel (tcgen05)" for k in SHAPES}
    launches = {k: 1 for k in SHAPES}
    traffic = {"8192x8192x8192": 1011.8e6, "16384x4096x4096": 450.9e6}

    def work(self):
        return {k: 2 * m * n * kk for k, (m, n, kk) in self.SHAPES.items()}

    def setup(self, rank, world, jt, torch, multi):
        from jittor_b200 import nn
        self.jt, self.torch, self.nn = jt, torch, nn
        g = torch.Generator().manual_seed(3 + rank)
        self.hostab, self.dev, self.out = {}, {}, {}
        for k, (m, n, kk) in self.SHAPES.items():
            a = (torch.randn(m, kk, generator=g) / kk ** 0.5).bfloat16().pin_memory()
            b = (torch.randn(kk, n, generator=g) / kk ** 0.5).bfloat16().pin_memory()
            self.hostab[k] = (a, b)
            self.dev[k] = (jt.array(a), jt.array(b))
            self.out[k] = torch.empty(m, n, dtype=torch.bfloat16).pin_memory()
        return list(self.SHAPES)

    def run(self, name):
        a, b = self.dev[name]
        return self.nn.matmul(a, b).sync()

    def run_e2e(self, name):
        a, b = self.hostab[name]
        self.nn.matmul(self.jt.array(a.cuda(non_blocking=True)),
                       self.jt.array(b.cuda(non_blocking=True))).fetch_into(self.out[name], stream=self.d2h_stream)

    def e2e_bytes(self, names):
        return (sum(a.numel() * 2 + b.numel() * 2 for a, b in (self.hostab[n] for n in names)),
                sum(self.out[n].numel() * 2 for n in names))

    def verify(self, env):
        """Untimed correctness witness: 32 sampled rows of each product against the CPU oracle (fp32 accumulation on the
        bf16 inputs, result rounded to bf16, 2e-2 mixed)."""
        from oracle import c_oracle as co
        torch = self.torch
        ok = True
        for name, (m, n, kk) in self.SHAPES.items():
            a, b = self.hostab[name]
            pick = torch.randperm(m, generator=torch.Generator().manual_seed(6))[:32]
            want = torch.from_numpy(co.matmul(a[pick].float().numpy(), b.float().numpy())).bfloat16().float().numpy()
            got = self.run(name).torch()[pick.cuda()].float().cpu().numpy()
            ok = ok and bool((np.abs(got - want) <= 2e-2 * np.abs(want) + 2e-2 * np.abs(want).max()).all())
        return ok

    def cpu(self, names):
        from oracle import c_oracle as co
        rows, done, secs = 256, 0, 0.0
        rng = np.random.default_rng(3)
        for nm in names:
            m, n, kk = self.SHAPES[nm]
            a = rng.normal(size=(rows, kk)).astype(np.float32)
            b = rng.normal(size=(kk, n)).astype(np.float32)
            t1 = time.perf_counter()
            co.matmul(a, b)
            secs += time.perf_counter() - t1
            done += 2 * rows * n * kk
        return done, secs, f"a slab of {rows} rows of A per shape, fp32 (OpenMP over rows)"


class C5ConvBN:
    key, metric, unit, bound, dtype, scaling = "c5", "conv TFLOP/s", "TFLOP/s", "tensor", "bf16 (fp32 accumulate)", "strong"
    N, C, H, W, CO = 256, 256, 56, 56, 256
    description = ("config 4: reindex conv2d bf16 [256,256,56,56] * [256,256,3,3] s1 p1, then global BatchNorm statistics "
                   "(one all-reduce of 2*C fp32) and fused normalise+ReLU; batch split over the ranks; third part: the same "
                   "convolution through the relay with acdb (NHWC) activations in and out, the layout ConvTuner derives for "
                   "tensor-core kernels, which needs no layout pass; fourth part: the weight gradient of the same layer as "
                   "jt.grad builds it (reduce.add over batch and pixels of reindex(x) * broadcast(dy)), each rank over its own "
                   "images; fifth part: the same weight gradient through the relay with acdb x and dy")
    kernel_of = {"conv": "conv_bf16_kernel (tcgen05)", "conv-bn-relu": "conv_bf16_kernel (tcgen05)",
                 "conv-acdb": "conv_bf16_kernel (tcgen05)", "conv-wgrad": "wgrad_bf16_kernel (tcgen05)",
                 "conv-wgrad-acdb": "wgrad_bf16_kernel (tcgen05)"}
    launches = {"conv": 2, "conv-bn-relu": 3, "conv-acdb": 2, "conv-wgrad": 6, "conv-wgrad-acdb": 2}
    all_reduced = ("conv-bn-relu",)
    traffic = {"conv": 776.5e6, "conv-bn-relu": 776.5e6, "conv-acdb": 776.5e6, "conv-wgrad": 826.0e6, "conv-wgrad-acdb": 826.0e6}

    def work(self):
        f = 2 * self.N * self.H * self.W * self.CO * self.C * 9
        return {"conv": f, "conv-bn-relu": f, "conv-acdb": f, "conv-wgrad": f, "conv-wgrad-acdb": f}

    def setup(self, rank, world, jt, torch, multi):
        from jittor_b200 import nn
        self.jt, self.torch, self.nn, self.world = jt, torch, nn, world
        n = self.N // world
        g = torch.Generator().manual_seed(4 + rank)
        self.hx = torch.randn(n, self.C, self.H, self.W, generator=g).bfloat16().pin_memory()
        gw = torch.Generator().manual_seed(4)          # weights are replicated
        self.hw = (torch.randn(self.CO, self.C, 3, 3, generator=gw) * (2 / (9 * self.C)) ** 0.5).bfloat16().pin_memory()
        self.x, self.w = jt.array(self.hx), jt.array(self.hw)
        self.bn = nn.BatchNorm(self.CO, is_train=True, sync=True)
        self.bn.weight.sync()
        self.bn.bias.sync()
        self.out = torch.empty(n, self.CO, self.H, self.W, dtype=torch.bfloat16).pin_memory()
        self.hxn = self.hx.permute(0, 2, 3, 1).contiguous().pin_memory()          # the same images, NHWC
        self.xn = jt.array(self.hxn)
        self.relay = jt.get_op_info("cudnn_conv").get_constructor()
        gd = torch.Generator().manual_seed(40 + rank)
        self.hdy = (torch.randn(n, self.CO, self.H, self.W, generator=gd) * 0.1).bfloat16().pin_memory()
        self.dy = jt.array(self.hdy)
        self.hdw = torch.empty(self.CO, self.C, 3, 3, dtype=torch.bfloat16).pin_memory()
        self.hdyn = self.hdy.permute(0, 2, 3, 1).contiguous().pin_memory()        # the same gradient, NHWC
        self.dyn = jt.array(self.hdyn)
        self.relay_w = jt.get_op_info("cudnn_conv_backward_w").get_constructor()
        return ["conv", "conv-bn-relu", "conv-acdb", "conv-wgrad", "conv-wgrad-acdb"]

    def per_rank_work(self, name):
        return self.work()[name] // self.world

    def _op(self, name, x, w, dy=None):
        if name == "conv-acdb":
            return self.relay(x, w, 1, 1, 1, 1, 1, 1, 1, "acdb", "oihw", "acdb")
        if name == "conv-wgrad":
            return self.jt.grad((self.nn.conv2d(x, w, None, 1, 1, 1) * (self.dy if dy is None else dy)).sum(), w)
        if name == "conv-wgrad-acdb":
            return self.relay_w(x, self.dyn if dy is None else dy, 3, 3, 1, 1, 1, 1, 1, 1, 1, "acdb", "oihw", "acdb")
        y = self.nn.conv2d(x, w, None, 1, 1, 1)
        if name == "conv":
            return y
        with self.jt.flag_scope(amp_reg=2):            # keep 16-bit results: the activation is written as bf16
            return self.nn.relu(self.bn(y))

    def run(self, name):
        return self._op(name, self.xn if name.endswith("-acdb") else self.x, self.w).sync()

    def run_e2e(self, name):
        x = self.jt.array((self.hxn if name.endswith("-acdb") else self.hx).cuda(non_blocking=True))
        w = self.jt.array(self.hw.cuda(non_blocking=True))
        if name.startswith("conv-wgrad"):
            dy = self.jt.array((self.hdyn if name.endswith("-acdb") else self.hdy).cuda(non_blocking=True))
            self._op(name, x, w, dy).fetch_into(self.hdw, stream=self.d2h_stream)
            return
        out = self.out.view(self.hxn.shape[0], self.H, self.W, self.CO) if name == "conv-acdb" else self.out
        self._op(name, x, w).fetch_into(out, stream=self.d2h_stream)

    def e2e_bytes(self, names):
        fwd = sum(1 for n in names if not n.startswith("conv-wgrad"))
        bwd = len(names) - fwd
        return (len(names) * (self.hx.numel() + self.hw.numel()) * 2 + bwd * self.hdy.numel() * 2,
                fwd * self.out.numel() * 2 + bwd * self.hdw.numel() * 2)

    def verify(self, env):
        """Untimed correctness witness: relu(bn(conv)) on this rank's images against the same chain computed by torch from
        this rank's stored conv output and the statistics of the FULL batch (float64 sums over all ranks, gathered with
        NCCL) -- what the reference checks sync BatchNorm against (a single process fed the global batch)."""
        torch = self.torch
        y = self._op("conv", self.x, self.w).torch()
        z = self._op("conv-bn-relu", self.x, self.w).torch()
        yd = y.double()
        st = torch.stack([yd.sum((0, 2, 3)), (yd * yd).sum((0, 2, 3))])
        del yd
        if env["multi"]:
            env["tdist"].all_reduce(st)
        cnt = float(self.N * self.H * self.W)
        mean = st[0] / cnt
        var = (st[1] / cnt - mean * mean).clamp_min(0)
        wgt = (1.0 / torch.sqrt(var + 1e-5)).float()
        bias = (-mean * wgt.double()).float()
        ok = bool(torch.equal(self._op("conv-acdb", self.xn, self.w).torch()[:8], y[:8].permute(0, 2, 3, 1)))   # same sums, other store
        for n0 in range(0, y.shape[0], 16):
            ref = torch.relu(y[n0:n0 + 16].float() * wgt[None, :, None, None] + bias[None, :, None, None])
            d = (z[n0:n0 + 16].float() - ref).abs()
            ok = ok and bool((d <= 2e-2 * ref.abs() + 2e-2 * ref.abs().max()).all())
        del y, z
        # this rank's weight gradient against torch's float32 one over the same images
        dw = self._op("conv-wgrad", self.x, self.w).torch().float()
        ref = torch.nn.grad.conv2d_weight(self.x.torch().float(), list(self.hw.shape), self.dy.torch().float(), stride=1, padding=1)
        ok = ok and bool(((dw - ref).abs() <= 2e-2 * ref.abs() + 2e-2 * ref.abs().max()).all())
        ok = ok and bool(torch.equal(self._op("conv-wgrad-acdb", self.xn, self.w).torch().float(), dw))    # same sums, no copies
        return ok

    def cpu(self, names):
        from oracle import c_oracle as co
        imgs = 2
        rng = np.random.default_rng(4)
        x = rng.normal(size=(imgs, self.C, self.H, self.W)).astype(np.float32)
        w = (rng.normal(size=(self.CO, self.C, 3, 3)) * (2 / (9 * self.C)) ** 0.5).astype(np.float32)
        done, t0 = 0, time.perf_counter()
        dy = None
        for nm in names:
            if nm.startswith("conv-wgrad"):
                if dy is None:
                    dy = (rng.normal(size=(imgs, self.CO, self.H, self.W)) * 0.1).astype(np.float32)
                co.conv2d_backward_w(x, dy, 3, 3, 1, 1, 1)
                done += self.work()[nm] * imgs // self.N
                continue
            y = co.conv2d(x, w, 1, 1, 1)
            if nm == "conv-bn-relu":
                co.bn_relu(y, np.ones(self.CO, np.float32), np.zeros(self.CO, np.float32))
            done += self.work()[nm] * imgs // self.N
        return max(done, 1), time.perf_counter() - t0, f"{imgs} of {self.N} images per part, fp32 (OpenMP over image x channel; weight gradients over out x in channel)"


class MetaOps:
    """The four meta-operators on their own (not fused): what a chain costs when it is not one of the recognised forms."""
    key, metric, unit, bound, dtype, scaling = "meta", "meta-op GB/s", "GB/s", "hbm", "f32", "weak"
    ROWS, COLS = 32768, 4096
    description = ("plain meta-operators on [32768,4096] fp32: reindex (pad by 2 columns; transpose), reduce (row sum, "
                   "column sum), broadcast fused into a binary add and on its own (a row stretched over all rows), and the conv-window "
                   "reindex of config 0 "
                   "([4,32,32,32] -> [4,64,32,32,32,3,3])")
    kernel_of = {"reindex-pad": "reindex_jit_kernel", "reindex-transpose": "reindex_permute_vec4_kernel",
                 "reindex-conv-window": "reindex_jit_kernel", "reduce-row-sum": "reduce_row_kernel",
                 "reduce-col-sum": "reduce_col_kernel", "broadcast-add": "binary_kernel",
                 "broadcast-rows": "broadcast_group_kernel"}
    launches = {"reindex-pad": 1, "reindex-transpose": 1, "reindex-conv-window": 1, "reduce-row-sum": 1,
                "reduce-col-sum": 2, "broadcast-add": 1, "broadcast-rows": 1}
    WIN = [4, 64, 32, 32, 32, 3, 3]

    def work(self):
        n = self.ROWS * self.COLS
        win = int(np.prod(self.WIN))
        return {"reindex-pad": 4 * n + 4 * self.ROWS * (self.COLS + 4), "reindex-transpose": 8 * n,
                "reindex-conv-window": 4 * win + 4 * 4 * 32 * 32 * 32, "reduce-row-sum": 4 * n + 4 * self.ROWS,
                "reduce-col-sum": 4 * n + 4 * self.COLS, "broadcast-add": 8 * n + 4 * self.COLS,
                "broadcast-rows": 4 * n + 4 * self.COLS}

    def setup(self, rank, world, jt, torch, multi):
        self.jt, self.torch = jt, torch
        g = torch.Generator().manual_seed(9 + rank)
        self.hx = torch.randn(self.ROWS, self.COLS, generator=g).pin_memory()
        self.x = [jt.array(self.hx), jt.array(self.hx.clone())]
        self.b = jt.array(torch.randn(self.COLS, generator=g))
        self.xs = jt.array(torch.rand(4, 32, 32, 32, generator=g))
        self.k = 0
        return list(self.kernel_of)

    def _op(self, name, x):
        if name == "reindex-pad":
            return x.reindex([self.ROWS, self.COLS + 4], ["i0", "i1-2"])
        if name == "reindex-transpose":
            return x.reindex([self.COLS, self.ROWS], ["i1", "i0"])
        if name == "reindex-conv-window":
            return self.xs.reindex(self.WIN, ["i0", "i2", "i3*1-1+i5*1", "i4*1-1+i6*1"])
        if name == "reduce-row-sum":
            return x.sum(1)
        if name == "reduce-col-sum":
            return x.sum(0)
        if name == "broadcast-rows":
            return self.b.broadcast([self.ROWS, self.COLS])
        return x + self.b

    def run(self, name):
        self.k += 1
        return self._op(name, self.x[self.k & 1]).sync()

    def run_e2e(self, name):
        x = self.jt.array(self.hx.cuda(non_blocking=True))
        self._op(name, x).sync()

    def e2e_bytes(self, names):
        return len(names) * self.hx.numel() * 4, 0

    def verify(self, env):
        """Untimed: every part at full size on the device, a band of it against the numpy oracle (bit-exact for the gathers)."""
        from oracle import meta_ops_ref as ref
        x = self.x[0]
        xh = x.torch()[:96].cpu().numpy()                           # the first rows decide the first rows / columns of each result
        ok = True
        got = self._op("reindex-pad", x).torch()[:96].cpu().numpy()
        ok = ok and bool(np.array_equal(got, ref.reindex(xh, [96, self.COLS + 4], ["i0", "i1-2"])))
        got = self._op("reindex-transpose", x).torch()[:, :96].cpu().numpy()
        ok = ok and bool(np.array_equal(got, xh.T))
        xs = self.xs.numpy()
        got = self._op("reindex-conv-window", x).numpy()
        ok = ok and bool(np.array_equal(got, ref.reindex(xs, self.WIN, ["i0", "i2", "i3*1-1+i5*1", "i4*1-1+i6*1"])))
        got = self._op("reduce-row-sum", x).torch()[:96].cpu().numpy()
        want = xh.astype(np.float64).sum(1)
        ok = ok and bool((np.abs(got - want) <= 1e-5 * np.abs(want) + 1e-5 * np.abs(want).max()).all())
        got = self._op("reduce-col-sum", x).numpy()
        want = x.torch().double().sum(0).cpu().numpy()
        ok = ok and bool((np.abs(got - want) <= 1e-5 * np.abs(want) + 1e-5 * np.abs(want).max()).all())
        got = self._op("broadcast-add", x).torch()[:96].cpu().numpy()
        ok = ok and bool(np.array_equal(got, xh + self.b.numpy()))
        got = self._op("broadcast-rows", x).torch()
        ok = ok and bool(self.torch.equal(got, self.b.torch()[None, :].expand(self.ROWS, self.COLS)))
        return ok

    def cpu(self, names):
        rows = 2048
        x = np.random.default_rng(9).normal(size=(rows, self.COLS)).astype(np.float32)
        from oracle import meta_ops_ref as ref
        done, t0 = 0, time.perf_counter()
        for nm in names:
            if nm == "reindex-pad":
                ref.reindex(x, [rows, self.COLS + 4], ["i0", "i1-2"])
            elif nm == "reindex-transpose":
                ref.reindex(x, [self.COLS, rows], ["i1", "i0"])
            elif nm == "reduce-row-sum":
                ref.reduce(x, "add", (1,))
            elif nm == "reduce-col-sum":
                ref.reduce(x, "add", (0,))
            elif nm == "broadcast-add":
                ref.binary(x, np.ones(self.COLS, np.float32), "add")
            elif nm == "broadcast-rows":
                ref.broadcast(np.ones(self.COLS, np.float32), [rows, self.COLS])
            else:
                continue
            done += self.work()[nm] * rows // self.ROWS
        return max(done, 1), time.perf_counter() - t0, f"{rows} of {self.ROWS} rows per part through the numpy oracle (1 core)"


class FusedChains:
    """Element-wise chains no named pattern covers, each run as ONE launch of a kernel compiled for it."""
    key, metric, unit, bound, dtype, scaling = "fused", "meta-op GB/s", "GB/s", "hbm", "f32", "weak"
    ROWS, COLS = 32768, 4096
    description = ("fused element-wise chains on [32768,4096] fp32, one launch of a kernel compiled for the chain each: x*w+b "
                   "(w, b per column), relu(x+bias), (a*b).sum(1), (x-mean)/sqrt(mean(x*x)+eps) (three row statements), the "
                   "gradient of LayerNorm w.r.t. x as jt.grad builds it (four row reduces), and the backward of nn.softmax "
                   "(its own kernel from y and dy)")
    kernel_of = {"scale-shift": "chain_jit_map_kernel", "relu-bias": "chain_jit_map_kernel", "mul-rowsum": "chain_jit_rows_kernel",
                 "centre-scale": "chain_jit_rows_kernel", "layernorm-bwd": "chain_jit_rows_kernel",
                 "softmax-bwd": "softmax_bwd_reg_kernel"}
    launches = {k: 1 for k in kernel_of}

    def work(self):
        n = self.ROWS * self.COLS * 4
        return {"scale-shift": 2 * n + 8 * self.COLS, "relu-bias": 2 * n + 4 * self.COLS, "mul-rowsum": 2 * n + 4 * self.ROWS,
                "centre-scale": 2 * n, "layernorm-bwd": 3 * n + 4 * self.COLS, "softmax-bwd": 3 * n}

    def setup(self, rank, world, jt, torch, multi):
        from jittor_b200 import nn
        self.jt, self.torch, self.nn = jt, torch, nn
        g = torch.Generator().manual_seed(13 + rank)
        self.hx = torch.randn(self.ROWS, self.COLS, generator=g).pin_memory()
        self.x = [jt.array(self.hx), jt.array(torch.randn(self.ROWS, self.COLS, generator=g)), jt.array(torch.randn(self.ROWS, self.COLS, generator=g))]
        self.w, self.b = jt.array(torch.randn(self.COLS, generator=g)), jt.array(torch.randn(self.COLS, generator=g))
        self.sm = [nn.softmax(v, -1).sync() for v in self.x]          # forward outputs the backward part starts from
        self.k = 0
        return list(self.kernel_of)

    def _op(self, name, x, y):
        if name == "scale-shift":
            return x * self.w + self.b
        if name == "relu-bias":
            return self.nn.relu(x + self.b)
        if name == "mul-rowsum":
            return (x * y).sum(1)
        if name == "centre-scale":
            return (x - x.mean(1, keepdims=True)) / ((x * x).mean(1, keepdims=True) + 1e-5).sqrt()
        if name == "layernorm-bwd":        # d LayerNorm / dx as jt.grad builds it from the per-op rules: four row reduces, one program
            return self.jt.grad((self.nn.layer_norm(x, (x.shape[-1],), self.w, self.b) * y).sum(), x)
        sm = next((s for v, s in zip(self.x, self.sm) if v is x), None)
        if sm is None:
            sm = self.nn.softmax(x, -1)
        return self.nn._softmax_backward(sm, y, False, self.COLS)       # what jt.grad emits for nn.softmax: dx from y and dy

    def run(self, name):
        self.k += 1
        return self._op(name, self.x[self.k % 3], self.x[(self.k + 1) % 3]).sync()

    def run_e2e(self, name):
        x = self.jt.array(self.hx.cuda(non_blocking=True))
        self._op(name, x, self.x[1]).sync()

    def e2e_bytes(self, names):
        return len(names) * self.hx.numel() * 4, 0

    def verify(self, env):
        from oracle import meta_ops_ref as ref
        x, y = self.x[0].torch()[:64].cpu().numpy(), self.x[1].torch()[:64].cpu().numpy()
        xv, yv = self.jt.array(x), self.jt.array(y)
        w, b = self.w.numpy(), self.b.numpy()
        ok = True
        for name in self.kernel_of:
            got = self._op(name, xv, yv).numpy()
            if name == "scale-shift":
                want = x * w + b
            elif name == "relu-bias":
                want = np.maximum(x + b, 0)
            elif name == "mul-rowsum":
                want = (x.astype(np.float64) * y).sum(1).astype(np.float32)
            elif name == "centre-scale":
                xd = x.astype(np.float64)
                want = ((xd - xd.mean(1, keepdims=True)) / np.sqrt((xd * xd).mean(1, keepdims=True) + 1e-5)).astype(np.float32)
            elif name == "layernorm-bwd":
                xd, dyg = x.astype(np.float64), y.astype(np.float64) * w
                rstd = 1 / np.sqrt(xd.var(1, keepdims=True) + 1e-5)
                xh = (xd - xd.mean(1, keepdims=True)) * rstd
                want = (rstd * (dyg - dyg.mean(1, keepdims=True) - xh * (dyg * xh).mean(1, keepdims=True))).astype(np.float32)
            else:
                sm = ref.softmax(x, -1).astype(np.float64)
                want = (sm * (y - (sm * y).sum(-1, keepdims=True))).astype(np.float32)
            ok = ok and bool((np.abs(got - want) <= 1e-4 * np.abs(want) + 1e-4 * np.abs(want).max()).all())
        return ok

    def cpu(self, names):
        rows = 1024
        rng = np.random.default_rng(13)
        x, y = rng.normal(size=(rows, self.COLS)).astype(np.float32), rng.normal(size=(rows, self.COLS)).astype(np.float32)
        w = np.ones(self.COLS, np.float32)
        from oracle import meta_ops_ref as ref
        done, t0 = 0, time.perf_counter()
        for nm in names:
            if nm == "scale-shift":
                ref.binary(ref.binary(x, w, "multiply"), w, "add")
            elif nm == "relu-bias":
                ref.ternary(ref.binary(ref.binary(x, w, "add"), np.float32(0), "greater"), x, np.float32(0))
            elif nm == "mul-rowsum":
                ref.reduce(ref.binary(x, y, "multiply"), "add", (1,))
            else:
                continue
            done += self.work()[nm] * rows // self.ROWS
        return max(done, 1), time.perf_counter() - t0, f"{rows} of {self.ROWS} rows per part, op by op through the numpy oracle (1 core)"


class NextOps:
    """The callers either side of the path: pooling kernels, getitem gather, setitem scatter-add."""
    key, metric, unit, bound, dtype, scaling = "next", "meta-op GB/s", "GB/s", "hbm", "f32", "weak"
    SHAPE = (64, 128, 112, 112)
    ROWS, COLS, PICK = 1 << 20, 64, 1 << 19
    description = ("callers of the path: 3x3 stride-2 pad-1 max-pool forward and backward on [64,128,112,112] fp32, "
                   "getitem x[idx] of 2^19 rows out of [2^20,64] fp32, setitem x[idx] += v on the same shapes")
    kernel_of = {"maxpool-fwd": "pool_fwd_s2_kernel", "maxpool-bwd": "pool_bwd_indices_s2_kernel",
                 "getitem-rows": "reindex_rows_kernel", "setitem-add-rows": "rr_rows_kernel (+ table copy)"}
    launches = {"maxpool-fwd": 1, "maxpool-bwd": 1, "getitem-rows": 1, "setitem-add-rows": 1}
    traffic = {"maxpool-fwd": 584.9e6, "maxpool-bwd": 566.8e6, "getitem-rows": 241.1e6, "setitem-add-rows": 365.8e6}

    def work(self):
        n = int(np.prod(self.SHAPE)) * 4
        o = self.SHAPE[0] * self.SHAPE[1] * 56 * 56 * 4
        rows = self.PICK * self.COLS * 4
        # backward: index map + output gradient in, input gradient out (x and y are not read by the index-based kernel)
        return {"maxpool-fwd": n + o, "maxpool-bwd": n + 2 * o, "getitem-rows": 2 * rows + self.PICK * 4,
                "setitem-add-rows": 2 * self.ROWS * self.COLS * 4 + 2 * rows + self.PICK * 4}

    def setup(self, rank, world, jt, torch, multi):
        from jittor_b200 import pool
        self.jt, self.torch, self.pool = jt, torch, pool
        g = torch.Generator().manual_seed(11 + rank)
        self.hx = torch.randn(*self.SHAPE, generator=g).pin_memory()
        self.x = jt.array(self.hx)
        self.y = pool.max_pool2d(self.x, 3, 2, 1).sync()
        self.dy = jt.array(torch.randn(self.SHAPE[0], self.SHAPE[1], 56, 56, generator=g))
        self.table = jt.array(torch.randn(self.ROWS, self.COLS, generator=g))
        self.idx = jt.array(torch.randperm(self.ROWS, generator=g)[:self.PICK].to(torch.int32))
        self.vals = jt.array(torch.randn(self.PICK, self.COLS, generator=g))
        return list(self.launches)

    def _op(self, name, x):
        if name == "maxpool-fwd":
            return self.pool.max_pool2d(x, 3, 2, 1)
        if name == "maxpool-bwd":
            return self.y._op.attrs["grad"](self.y, self.dy, 0)
        if name == "getitem-rows":
            return self.table[self.idx]
        return self.table.setitem((self.idx,), self.vals, "add")

    def run(self, name):
        return self._op(name, self.x).sync()

    def run_e2e(self, name):
        x = self.jt.array(self.hx.cuda(non_blocking=True))
        self._op(name, x).sync()

    def e2e_bytes(self, names):
        return len(names) * self.hx.numel() * 4, 0

    def verify(self, env):
        """Untimed: the four parts at full size on the device; two images of the pooling parts and the whole gather /
        scatter-add against the numpy oracle."""
        from oracle import meta_ops_ref as ref
        torch = self.torch
        xh = self.x.torch()[:2, :4].cpu().numpy()
        y = self._op("maxpool-fwd", self.x).torch()
        ok = bool(np.array_equal(y[:2, :4].cpu().numpy(), ref.pool2d(xh, 3, "maximum", 2, 1)))
        dyh = self.dy.torch()[:2, :4].cpu().numpy()
        dx = self._op("maxpool-bwd", self.x).torch()[:2, :4].cpu().numpy()
        want = ref.pool2d_backward(xh, dyh, 3, "maximum", 2, 1)
        ok = ok and bool((np.abs(dx - want) <= 1e-5 * np.abs(want) + 1e-5 * np.abs(want).max()).all())
        table, idx, vals = self.table.torch(), self.idx.torch().long(), self.vals.torch()
        ok = ok and bool(torch.equal(self._op("getitem-rows", self.x).torch(), table[idx]))
        want_t = table.clone()
        want_t[idx] += vals                                             # the picked rows are distinct (a permutation prefix)
        ok = ok and bool(torch.allclose(self._op("setitem-add-rows", self.x).torch(), want_t, rtol=1e-6, atol=1e-6))
        return ok

    def cpu(self, names):
        from oracle import meta_ops_ref as ref
        x = np.random.default_rng(11).normal(size=(2, 16, 112, 112)).astype(np.float32)
        done, t0 = 0, time.perf_counter()
        frac = x.size / float(np.prod(self.SHAPE))
        for nm in names:
            if nm == "maxpool-fwd":
                ref.pool2d(x, 3, "maximum", 2, 1)
            elif nm == "maxpool-bwd":
                ref.pool2d_backward(x, np.ones((2, 16, 56, 56), np.float32), 3, "maximum", 2, 1)
            else:
                continue
            done += self.work()[nm] * frac
        return max(done, 1), time.perf_counter() - t0, "2x16 of 64x128 images per pooling part through the numpy oracle (1 core)"


WORKLOADS = {w.key: w for w in (C1ConvF32, C2Scatter, C3Rows, C4Matmul, C5ConvBN, MetaOps, FusedChains, NextOps)}
HEADLINE = "c2"                               # the default run's top-level line; the other configs follow in "workloads"
CONFIGS = ("c1", "c3", "c4", "c5", "meta", "fused", "next")   # measured after the headline in the default run


def scale_of(unit):
    return 1e6 if unit == "GB/s" else 1e9          # work / ms -> GB/s (1e6) or TFLOP/s (1e9)


def cpu_value(wl, names, steps, warmup):
    """The reference's CPU implementation of the step (C restatement of its loop nests) on a bounded sample."""
    for _ in range(max(warmup, 0)):
        wl.cpu(names)
    done = secs = 0.0
    sample = ""
    for _ in range(steps):
        d, t, sample = wl.cpu(names)
        done, secs = done + d, secs + t
    return done / secs / (1e9 if wl.unit == "GB/s" else 1e12), secs / steps * 1e3, sample


def run_reference(args, rank, world):
    if rank != 0:
        return
    wl = WORKLOADS[args.workload]()
    names = [n for n in wl.work() if not args.parts or n in args.parts.split(",")]
    val, ms, sample = cpu_value(wl, names, args.steps, args.warmup)
    out = {
        "impl": "reference", "metric": wl.metric, "value": val, "unit": wl.unit, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": wl.scaling, "vs_baseline": None, "dtype": wl.dtype if wl.key == "c2" else "f32", "data": "synthetic",
        "config": {"workload": wl.description, "sample": sample},
        "cpu_baseline": {"value": val, "unit": wl.unit, "cores": os.cpu_count(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    if args.all and args.workload == HEADLINE and not args.parts:
        extra = {}
        for key in CONFIGS:
            w2 = WORKLOADS[key]()
            v2, ms2, sample2 = cpu_value(w2, list(w2.work()), min(args.steps, 3), min(args.warmup, 1))
            extra[key] = {"value": v2, "unit": w2.unit, "ms_per_step": ms2, "cores": os.cpu_count(), "kind": "port", "sample": sample2}
        out["workloads"] = extra
    print(json.dumps(out))


def percentile(sorted_vals, q):
    return sorted_vals[min(len(sorted_vals) - 1, int(q * len(sorted_vals)))]


def measure(wl, args, env, headline):
    """Times one workload on this rank's GPU and returns its record (max over ranks)."""
    torch, tdist, jt = env["torch"], env["tdist"], env["jt"]
    rank, world, multi, local = env["rank"], env["world"], env["multi"], env["local"]
    names = [n for n in wl.setup(rank, world, jt, torch, multi) if not args.parts or n in args.parts.split(",")]
    work = {n: wl.work()[n] for n in names}
    sc = scale_of(wl.unit)
    job_work = sum(work.values()) * (world if wl.scaling == "weak" else 1)
    steps = args.steps if headline else max(20, min(args.steps, 50))
    flush = None
    if getattr(wl, "flush_l2", False):
        flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        flush = flush_buf.zero_

    def barrier():
        if multi:
            tdist.barrier()
        torch.cuda.synchronize()

    import contextlib
    step_context = wl.step_context if (multi and hasattr(wl, "step_context") and args.overlap) else contextlib.nullcontext

    def run_step():
        """One step: the workload's own step runner when it has one (it places the collectives), else part after part."""
        if hasattr(wl, "run_step"):
            return wl.run_step(names, bool(args.overlap))
        with step_context():
            return [wl.run(nm) for nm in names]

    def step_direct():
        run_step()

    warm = max(args.warmup, 3)
    for _ in range(warm):
        step_direct()
    barrier()
    # (1) per-part times: direct launches with an event after every part
    psteps = min(steps, 10)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)] for _ in range(psteps)]
    barrier()
    for s in range(psteps):
        if flush:
            flush()
        ev[s][0].record()
        with step_context():
            for i, nm in enumerate(names):
                wl.run(nm)
                ev[s][i + 1].record()
    barrier()
    part_ms = {nm: sum(ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(psteps)) / psteps for i, nm in enumerate(names)}
    # (2) the timed region: K steps. One step (kernels and collectives of all parts) is captured into a CUDA graph and
    # replayed, so that the device is not waiting for the Python launch path; without --graph, or if capture fails, the
    # steps are launched directly.
    graph = None
    if args.graph:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step_direct()
            torch.cuda.current_stream().wait_stream(side)
            barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                keep = run_step()                            # noqa: F841  (outputs stay alive with the graph)
            graph.replay()
            barrier()
        except Exception as exc:                     # noqa: BLE001
            print(f"[bench] CUDA graph capture unavailable ({type(exc).__name__}: {exc}); launching directly", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
    step = graph.replay if graph is not None else step_direct
    clocks = ClockSampler(local)
    clocks.__enter__()
    barrier()
    if flush is None:
        e_beg, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e_beg.record()
        for s in range(steps):
            step()
        e_end.record()
        barrier()
        step_ms = e_beg.elapsed_time(e_end) / steps
    else:
        # inputs smaller than L2: every repetition is preceded by an L2 flush and timed by its own event pair
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for a, b in pairs:
            flush()
            a.record()
            step()
            b.record()
        barrier()
        step_ms = sum(a.elapsed_time(b) for a, b in pairs) / steps
    # (3) stability: further repetitions (the same count on every rank), each timed by its own event pair; the clocks are
    # sampled through the timed region and this window
    reps = max(args.stability, 0)
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    for k, (a, b) in enumerate(pairs):
        if flush:
            flush()
        a.record()
        step()
        b.record()
        if k % 64 == 63:
            torch.cuda.current_stream().synchronize()
    barrier()
    clocks.__exit__()
    rep_ms = sorted(a.elapsed_time(b) for a, b in pairs)
    # (4) per-part times once more, each part replayed from its own CUDA graph: the direct launches of (1) include the
    # Python launch path, which for small or graph-building parts (a conv of 25 us, a jt.grad chain) is longer than the kernel
    parts_timing = "direct launches, an event after every part"
    # (a part whose collective runs on the side stream is not captured on its own: its times stay those of (1))
    if graph is not None and not (multi and hasattr(wl, "run_step")):
        try:
            graphed = {}
            for nm in names:
                barrier()
                g1 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g1):
                    with step_context():
                        keep1 = wl.run(nm)                   # noqa: F841
                g1.replay()
                barrier()
                pp = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(psteps)]
                for a, b in pp:
                    if flush:
                        flush()
                    a.record()
                    g1.replay()
                    b.record()
                barrier()
                graphed[nm] = sum(a.elapsed_time(b) for a, b in pp) / psteps
                del g1, keep1
            part_ms = graphed
            parts_timing = "each part replayed from its own CUDA graph"
        except Exception as exc:                     # noqa: BLE001
            print(f"[bench] per-part graphs unavailable ({type(exc).__name__}: {exc}); keeping the direct per-part times", file=sys.stderr)
            torch.cuda.synchronize()
    status = jt._capi.lib.b200jt_device_status()

    # ---- end to end: pinned host -> device -> kernels -> pinned host ------------------------------------
    wl.d2h_stream = torch.cuda.Stream()          # results go back on their own stream: PCIe is full duplex

    def e2e_step():
        # steps pipeline: the read-back of one step overlaps the uploads of the next; everything is drained
        # (both streams synchronised) before the timed region closes
        with step_context():
            for nm in names:
                wl.run_e2e(nm)

    e2e_steps = (max(2, min(steps, 5)) if headline else 2) if args.e2e else 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.e2e:
        e2e_step()
    wl.d2h_stream.synchronize()
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.current_stream().wait_stream(wl.d2h_stream)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / max(e2e_steps, 1)
    h2d, d2h = wl.e2e_bytes(names)

    # ---- correctness witness (untimed) ----------------------------------------------------------------
    parity = None
    if args.verify and hasattr(wl, "verify") and not args.parts:
        try:
            parity = bool(wl.verify(env))
        except Exception as exc:                     # noqa: BLE001
            print(f"[bench] verify({wl.key}) raised {type(exc).__name__}: {exc}", file=sys.stderr)
            parity = False
        status = status or jt._capi.lib.b200jt_device_status()

    # ---- max over ranks ------------------------------------------------------------------------------
    p50, p10, p90 = (percentile(rep_ms, 0.5), percentile(rep_ms, 0.1), percentile(rep_ms, 0.9)) if rep_ms else (0.0, 0.0, 0.0)
    times = torch.tensor([step_ms, e2e_ms, p50, p10, p90] + [part_ms[n] for n in names], device="cuda", dtype=torch.float64)
    flags_ = torch.tensor([0 if parity is False else 1, 1 if status == 0 else 0], device="cuda", dtype=torch.int32)
    if multi:
        tdist.all_reduce(times, op=tdist.ReduceOp.MAX)
        tdist.all_reduce(flags_, op=tdist.ReduceOp.MIN)
    times = times.tolist()
    step_ms, e2e_ms, p50, p10, p90 = times[:5]
    part_ms = dict(zip(names, times[5:]))
    if parity is not None:
        parity = bool(flags_[0].item())
    if status == 0 and not bool(flags_[1].item()):
        status = -2                                  # another rank's status word was set
    if rank != 0:
        return None

    peaks = env["peaks"]
    if wl.bound == "hbm":
        peak, peak_src = (peaks["hbm_gbs"], "measured") if peaks else (6650.0, "fallback")
    else:
        peak, peak_src = (peaks["bf16_tflops"], "measured (burst)") if peaks else (1590.0, "fallback")
    per_rank = wl.per_rank_work if hasattr(wl, "per_rank_work") else (lambda n: work[n])
    parts = [{"part": n, "ms": part_ms[n], wl.unit: per_rank(n) / part_ms[n] / sc,
              "frac_of_peak": per_rank(n) / part_ms[n] / sc / peak, "kernel": wl.kernel_of[n]} for n in names]
    # the dominant kernel: largest summed time over the parts of one step
    by_kernel = {}
    for n in names:
        k = by_kernel.setdefault(wl.kernel_of[n], {"ms": 0.0, "work": 0, "parts": [], "launches": 0, "traffic": 0.0})
        k["ms"] += part_ms[n]
        k["work"] += per_rank(n)
        k["parts"].append(n)
        k["launches"] += 1
        t = getattr(wl, "traffic", {}).get(n)
        k["traffic"] = None if (t is None or k["traffic"] is None) else k["traffic"] + t
    dom_name = max(by_kernel, key=lambda k: by_kernel[k]["ms"])
    dom = by_kernel[dom_name]
    achieved = dom["work"] / dom["ms"] / sc
    per_rank_step = sum(per_rank(n) for n in names)
    peer_kernel = env["peer_kernel"]
    out = {
        "metric": wl.metric, "value": job_work / step_ms / sc, "unit": wl.unit, "n_gpus": world,
        "steps": steps, "warmup": warm, "ms_per_step": step_ms, "higher_is_better": True,
        "scaling": wl.scaling, "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": {"workload": wl.description, "algorithmic_work_per_step": job_work,
                   "l2": ("flushed (256 MB fill) before every timed repetition: the operands fit in L2" if flush else
                          "no flush: every part touches more than the 126 MB L2 and the parts rotate"),
                   "parallelism": f"dp{world}" if world > 1 else "1 GPU"},
        "clocks": clocks.summary(),
        "e2e": {"value": job_work / e2e_ms / sc if e2e_steps else None, "unit": wl.unit, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": steps * sum(wl.launches[n] + (1 if peer_kernel and n in getattr(wl, "all_reduced", ()) else 0)
                                    for n in names),
        "collective": None if not multi else ("peer-kernel (NVLink loads/stores, one launch per rank)" if peer_kernel else "nccl"),
        "collective_overlap": bool(multi and peer_kernel and hasattr(wl, "step_context") and args.overlap),
        "roofline": {"bound": wl.bound, "kernel": dom_name, "parts": dom["parts"], "achieved": achieved, "peak": peak,
                     "unit": wl.unit, "frac": achieved / peak, "peak_source": peak_src,
                     "traffic": (dom["traffic"] / dom["launches"]) if dom["traffic"] else None,
                     "step_frac": per_rank_step / step_ms / sc / peak,
                     "note": "dominant kernel = largest summed time over the parts of one step; achieved = algorithmic work "
                             "of those parts / their CUDA-event time (main kernel plus small helper launches); traffic = "
                             "DRAM bytes per launch from the ncu captures under profiles/; step_frac = whole step / peak"},
        "parts": parts,
        "stability": {"repetitions": reps, "ms_median": p50, "ms_p10": p10, "ms_p90": p90},
        "cuda_graph": graph is not None,
        "parts_timing": parts_timing,
        "device_status": status,
    }
    if parity is not None:
        out["parity_ok"] = parity
    if hasattr(wl, "extra"):
        out.update(wl.extra(part_ms))
    if args.cpu_baseline and world == 1:
        done, secs, sample = wl.cpu(names)
        out["cpu_baseline"] = {"value": done / secs / (1e9 if wl.unit == "GB/s" else 1e12), "unit": wl.unit,
                               "cores": os.cpu_count(), "kind": "port", "sample": sample}
    return out


def allreduce_latency(env):
    """`--workload allreduce` (N > 1): latency of the NVLink peer all-reduce kernel next to NCCL for the message sizes of the
    path, fp32 sum, 200 back-to-back calls between CUDA events, max over ranks. Prints one JSON line on rank 0."""
    torch, tdist, jt = env["torch"], env["tdist"], env["jt"]
    from jittor_b200 import dist
    pc = dist.peer_comm()

    def timeit(fn, n=200):
        for _ in range(10):
            fn()
        tdist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n * 1e3], device="cuda")
        tdist.all_reduce(t, op=tdist.ReduceOp.MAX)
        return t.item()

    rows = []
    for nbytes in (2048, 16384, 262144, 1 << 20, 4 << 20, 8 << 20):
        x = torch.ones(nbytes // 4, device="cuda")
        y, z = torch.empty_like(x), x.clone()
        tp = timeit(lambda: pc.all_reduce(x, y)) if pc and pc.usable(x) else None
        rows.append({"bytes": nbytes, "peer_us": tp, "nccl_us": timeit(lambda: tdist.all_reduce(z))})
    status = jt._capi.lib.b200jt_device_status()
    if env["rank"] == 0:
        print(json.dumps({"metric": "all-reduce latency", "unit": "us", "n_gpus": env["world"], "higher_is_better": False,
                          "peer_kernel": pc is not None, "device_status": status, "rows": rows}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--workload", default=HEADLINE, choices=sorted(WORKLOADS) + ["allreduce"])
    ap.add_argument("--all", type=int, default=1, help="default run: after the headline workload also measure c1, c3, c4, c5")
    ap.add_argument("--cpu-baseline", type=int, default=1)
    ap.add_argument("--parts", default="", help="comma-separated subset of the parts (profiling aid)")
    ap.add_argument("--e2e", type=int, default=1)
    ap.add_argument("--verify", type=int, default=1, help="untimed correctness witness after the timed regions")
    ap.add_argument("--stability", type=int, default=300, help="individually timed repetitions after the timed region")
    ap.add_argument("--overlap", type=int, default=1, help="N > 1: run a part's all-reduce beside the next part's kernel")
    ap.add_argument("--graph", type=int, default=1, help="replay the step from a CUDA graph in the timed region")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        return run_reference(args, rank, world)

    import gc

    import torch
    import torch.distributed as tdist

    import jittor_b200 as jt
    from jittor_b200 import dist

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init("nccl")
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    env = {"torch": torch, "tdist": tdist, "jt": jt, "rank": rank, "world": world, "local": local,
           "multi": dist.in_mpi(), "peer_kernel": dist.peer_comm() is not None,
           "peaks": json.load(open(peaks_path)) if os.path.exists(peaks_path) else None}
    if args.workload == "allreduce":
        return allreduce_latency(env)
    out = measure(WORKLOADS[args.workload](), args, env, True)
    if args.all and args.workload == HEADLINE and not args.parts:
        others = {}
        for key in CONFIGS:
            gc.collect()
            torch.cuda.empty_cache()
            rec = measure(WORKLOADS[key](), args, env, False)
            if rec is not None:
                others[key] = rec
        if out is not None:
            out["workloads"] = others
            out["gpu_launches_all_workloads"] = out["gpu_launches"] + sum(r["gpu_launches"] for r in others.values())
    if out is not None:
        print(json.dumps(out))


if __name__ == "__main__":
    main()
