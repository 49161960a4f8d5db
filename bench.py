"""Benchmark of the meta-operator hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c5] [--impl reference]

One JSON line on stdout (rank 0). The default workload is the reindex_reduce scatter configuration
(benchmark config 1): one step = one pass over its five parts
    a-uniform / a-zipf : 2^24 int32 values into 2^20 bins (op add, bit-exact)
    b-uniform / b-zipf : 2^24 fp32 values into 4096 bins
    pool-bwd           : 2x2 max-pool backward as reindex_reduce add, [64,128,56,56,2,2] -> [64,128,112,112] fp32
`value` is algorithmic GB/s with inputs resident in HBM, timed with CUDA events on the launching stream
(max over ranks); `e2e` is the same step through the public API from pinned host buffers including the
host->device copies and the device->host read of the results. Every part's input is larger than L2 and five
different inputs are touched between two uses of one buffer, so no L2 flush is needed (stated in `config`).
`--impl reference` times the CPU restatement of the reference's loop nests (oracle/meta_ops.c) on the host cores.
With N > 1 (torchrun) every rank processes its own inputs (weak scaling); the scatter parts all-reduce their bins
over NCCL, which is the reference's exchange step for a shared output.
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

N_VAL = 1 << 24
BINS_A = 1 << 20
BINS_B = 4096
POOL_SHAPE = (64, 128, 56, 56, 2, 2)
POOL_IDX = ["i0", "i1", "i2*2+i4", "i3*2+i5"]


def algorithmic_bytes():
    """inputs read once + outputs written once, intermediates free."""
    pool = int(np.prod(POOL_SHAPE)) * 4
    return {"a-uniform": N_VAL * 8 + BINS_A * 4, "a-zipf": N_VAL * 8 + BINS_A * 4,
            "b-uniform": N_VAL * 8 + BINS_B * 4, "b-zipf": N_VAL * 8 + BINS_B * 4, "pool-bwd": 2 * pool}


def zipf_indices(rng, n, bins, s=1.1):
    """Inverse-CDF draw from the truncated Zipf(s) over bin ranks; rank -> bin by a fixed permutation."""
    p = np.arange(1, bins + 1, dtype=np.float64) ** (-s)
    cdf = np.cumsum(p / p.sum())
    rank = np.minimum(np.searchsorted(cdf, rng.random(n)), bins - 1)
    return rng.permutation(bins)[rank].astype(np.int32)


def make_inputs(seed, pool_images=POOL_SHAPE[0]):
    rng = np.random.default_rng(seed)       # seed = config index (+ rank)
    vi = rng.integers(0, 100, size=N_VAL).astype(np.int32)
    vf = rng.normal(size=N_VAL).astype(np.float32)
    pshape = (pool_images,) + POOL_SHAPE[1:]
    # pool gradient: N(0,1) where the element is its window's arg-max, else 0 (what the max-reduce grad emits)
    g = rng.normal(size=pshape).astype(np.float32)
    keep = rng.integers(0, 4, size=pshape[:4])
    mask = np.zeros(pshape, dtype=bool).reshape(pshape[:4] + (4,))
    np.put_along_axis(mask, keep[..., None], True, axis=-1)
    g *= mask.reshape(pshape)
    return {
        "a-uniform": (vi, rng.integers(0, BINS_A, size=N_VAL).astype(np.int32), BINS_A),
        "a-zipf": (vi, zipf_indices(rng, N_VAL, BINS_A), BINS_A),
        "b-uniform": (vf, rng.integers(0, BINS_B, size=N_VAL).astype(np.int32), BINS_B),
        "b-zipf": (vf, zipf_indices(rng, N_VAL, BINS_B), BINS_B),
        "pool-bwd": (g, None, None),
    }


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
            time.sleep(0.1)

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
                "samples": len(self.samples)}


def run_reference(args, rank, world):
    """The reference's CPU implementation of the step (C restatement of its loop nests), bounded sample."""
    if rank != 0:
        return
    from oracle import c_oracle as co
    pool_images = 8                                    # bounded sample: 8 of the 64 images of the pool part
    inp = make_inputs(1, pool_images)
    ab = algorithmic_bytes()
    ab["pool-bwd"] = ab["pool-bwd"] * pool_images // POOL_SHAPE[0]
    total = sum(ab.values())

    def step():
        for name, (val, idx, bins) in inp.items():
            if idx is None:
                co.pool2x2_bwd(val)
            else:
                co.scatter_add(val, idx, bins)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = total / dt / 1e9
    sample = "the four scatter parts at full size + 8 of 64 images of pool-bwd, per step"
    print(json.dumps({
        "impl": "reference", "metric": "meta-op GB/s", "value": val, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int32/f32", "data": "synthetic",
        "config": {"workload": "config 1: reindex_reduce scatter-add (a,b x uniform,zipf) + pool-bwd", "sample": sample},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port", "sample": sample,
                         "note": "scatter loops are serial in the reference (1 core); pool-bwd uses OpenMP"},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--cpu-baseline", type=int, default=1)
    ap.add_argument("--parts", default="", help="comma-separated subset of the parts (profiling aid)")
    ap.add_argument("--e2e", type=int, default=1)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        return run_reference(args, rank, world)

    import torch
    import torch.distributed as tdist

    import jittor_b200 as jt
    from jittor_b200 import dist

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init("nccl")
    multi = dist.in_mpi()

    ab = algorithmic_bytes()
    total_bytes = sum(ab.values())
    host = make_inputs(1 + rank)
    pinned = {k: tuple(torch.from_numpy(a).pin_memory() if a is not None else None for a in v[:2]) + (v[2],)
              for k, v in host.items()}
    dev = {k: (jt.array(v[0]), jt.array(v[1]) if v[1] is not None else None, v[2]) for k, v in pinned.items()}
    names = [n for n in dev if not args.parts or n in args.parts.split(",")]
    ab = {n: ab[n] for n in names}
    total_bytes = sum(ab.values())

    def run_part(name, val, idx, bins):
        if idx is None:
            out = val.reindex_reduce("add", list(POOL_SHAPE[:2]) + [112, 112], POOL_IDX)
        else:
            out = val.reindex_reduce("add", [bins], ["@e0(i0)"], extras=[idx])
            if multi:
                out = out.mpi_all_reduce("add")      # shared output across ranks
        out.sync()
        return out

    def barrier():
        if multi:
            tdist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput ------------------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        for nm in names:
            run_part(nm, *dev[nm])
    barrier()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)] for _ in range(args.steps)]
    with ClockSampler(local) as clocks:
        barrier()
        for s in range(args.steps):
            ev[s][0].record()
            for i, nm in enumerate(names):
                run_part(nm, *dev[nm])
                ev[s][i + 1].record()
        barrier()
    step_ms = ev[0][0].elapsed_time(ev[-1][-1]) / args.steps
    part_ms = {nm: sum(ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(args.steps)) / args.steps
               for i, nm in enumerate(names)}

    # ---- end to end: pinned host -> device -> kernels -> host ----------------------------------------
    out_host = {nm: torch.empty(ab_out, dtype=(torch.int32 if nm.startswith("a-") else torch.float32)).pin_memory()
                for nm, ab_out in (("a-uniform", BINS_A), ("a-zipf", BINS_A), ("b-uniform", BINS_B), ("b-zipf", BINS_B),
                                   ("pool-bwd", int(np.prod(POOL_SHAPE))))}

    def e2e_step():
        for nm in names:
            hv, hi, bins = pinned[nm]
            v = jt.array(hv.cuda(non_blocking=True))
            i = jt.array(hi.cuda(non_blocking=True)) if hi is not None else None
            run_part(nm, v, i, bins).fetch_into(out_host[nm])
        torch.cuda.current_stream().synchronize()

    e2e_steps = max(2, min(args.steps, 5)) if args.e2e else 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.e2e:
        e2e_step()
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / max(e2e_steps, 1)
    h2d = sum(a.numel() * a.element_size() for n in names for a in pinned[n][:2] if a is not None)
    d2h = sum(out_host[n].numel() * 4 for n in names)

    # ---- max over ranks ------------------------------------------------------------------------------
    times = torch.tensor([step_ms, e2e_ms] + [part_ms[n] for n in names], device="cuda", dtype=torch.float64)
    if multi:
        tdist.all_reduce(times, op=tdist.ReduceOp.MAX)
    times = times.tolist()
    step_ms, e2e_ms = times[0], times[1]
    part_ms = dict(zip(names, times[2:]))
    if rank != 0:
        return

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = json.load(open(peaks_path))["hbm_gbs"], "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    parts = [{"part": n, "ms": part_ms[n], "GB/s": ab[n] / part_ms[n] / 1e6, "frac_of_hbm": ab[n] / part_ms[n] / 1e6 / peak}
             for n in names]
    dom = max(names, key=lambda n: part_ms[n])
    kernel_of = {"a-uniform": "rr_direct_kernel<int,int,4>", "a-zipf": "rr_direct_kernel<int,int,4>",
                 "b-uniform": "rr_privatised_kernel<float,int,4>", "b-zipf": "rr_privatised_kernel<float,int,4>",
                 "pool-bwd": "rr_affine_kernel<float>"}
    achieved = ab[dom] / part_ms[dom] / 1e6
    out = {
        "metric": "meta-op GB/s", "value": world * total_bytes / step_ms / 1e6, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int32/f32", "data": "synthetic",
        "config": {"workload": "config 1: reindex_reduce scatter-add 2^24 -> 2^20 int32 and -> 4096 fp32 "
                               "(uniform + Zipf 1.1 indices) + 2x2 max-pool backward [64,128,112,112] fp32",
                   "algorithmic_bytes_per_step": total_bytes,
                   "l2": "no flush: every part's input exceeds the 126 MB L2 and five inputs rotate",
                   "parallelism": f"dp{world} (per-rank inputs; NCCL all-reduce of the scatter bins)" if world > 1 else "1 GPU"},
        "clocks": clocks.summary(),
        "e2e": {"value": world * total_bytes / e2e_ms / 1e6, "unit": "GB/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": args.steps * sum(1 if n == "pool-bwd" else 2 for n in names),
        "roofline": {"bound": "hbm", "kernel": kernel_of[dom], "part": dom, "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src, "traffic": None,
                     "note": "achieved = algorithmic bytes of the part / CUDA-event time of the part "
                             "(its main kernel plus the init-fill or fold kernel)"},
        "parts": parts,
    }
    if args.cpu_baseline and world == 1:
        from oracle import c_oracle as co
        t0 = time.perf_counter()
        done = 0
        for nm in ("a-uniform", "a-zipf", "b-uniform", "b-zipf"):
            v, i, b = host[nm]
            co.scatter_add(v, i, b)
            done += ab[nm]
        co.pool2x2_bwd(host["pool-bwd"][0][:8])
        done += ab["pool-bwd"] * 8 // POOL_SHAPE[0]
        dt = time.perf_counter() - t0
        out["cpu_baseline"] = {"value": done / dt / 1e9, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
                               "sample": "one pass: the four scatter parts at full size + 8 of 64 pool-bwd images",
                               "note": "scatter loops are serial in the reference (1 core); pool-bwd uses OpenMP"}
    print(json.dumps(out))


if __name__ == "__main__":
    main()
