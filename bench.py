"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the hot path over one batch: the flash forward and the flash
backward (dQ, dK, dV of output.sum()) of the workload.  The default workload is the
configuration the headline metric is quoted on: B=8, H=8, Sq=Skv=2048, D=64, fp16,
checkerboard score_mod, no mask (examples/benchmark.py of the reference).  Inputs are
synthetic N(0,1) tensors from fixed seeds (K: 0, Q: 1, V: 2).

Every timed leg runs the K steps asked for and then keeps repeating blocks of K steps until it
has lasted half a second, so that the clock record has samples; `ms_per_step` is the mean over
all timed steps (`timed_steps`).  L2 is flushed between timed steps; times are CUDA events on
the launching stream, the maximum over ranks under torchrun.

Scaling (`value`) is weak: under torchrun every rank processes its own batch of 8 with the
global batch offset 8 * rank passed to the kernels, and there is no data-path collective.
With more than one rank the line also carries `strong`: the B4 H16 S8192 D128 attention-sink
problem cut over the ranks by batch x heads (flaxattention_b200.sharding), every rank timing
its shard.

The single JSON line carries the contract keys plus:
  roofline      the dominant kernel against the measured bf16 tensor peak (algorithmic FLOPs of
                the blocks it computes / its device time)
  kernels       device time of every kernel of a step (fa_profile_read) and achieved TFLOP/s
  fwd           forward-only numbers
  workloads     the causal+ALiBi and the attention-sink configurations (N=1)
  decode        split-KV decode GB/s (N=1)
  cpu_baseline  the CPU oracle (a port of the reference's dense path) timed on this box's
                host cores on a bounded sample
  e2e           the same step from pinned host buffers through flaxattention_b200.HostPipeline:
                host->device copies of q, k, v and device->host copies of out, dq, dk, dv
                inside the timing, overlapped with the kernels chunk by chunk
`--impl reference` times the CPU oracle alone (the reference itself needs JAX, which is not
installed); it is the one place besides cpu_baseline where bench.py runs code from oracle/.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

WORKLOADS = {
    # name: B, H, Sq, Skv, D, dtype, score_mod, mask
    "cfg2": dict(B=8, H=8, Sq=2048, Skv=2048, D=64, dtype="f16", score="checkerboard", mask=None),
    "cfg2_nomod": dict(B=8, H=8, Sq=2048, Skv=2048, D=64, dtype="f16", score=None, mask=None),
    "cfg3": dict(B=8, H=8, Sq=2048, Skv=2048, D=64, dtype="bf16", score="alibi", mask="causal"),
    "cfg4": dict(B=4, H=16, Sq=8192, Skv=8192, D=128, dtype="bf16", score=None, mask="sink"),
}
DECODE = dict(B=32, H=8, Skv=16384, D=64, dtype="f16")
DT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}
MIN_LEG_SECONDS = 0.5

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under
# profiles/, per workload and kernel.  The captures were taken on the B=2 case of each workload and are
# scaled to its full batch (x4 for B=8, x2 for B=4): the traffic grows with the batch.  Workloads and
# kernels without a capture are absent.
NCU_TRAFFIC = {
    "cfg2": {"fa_fwd_tc_kernel": 4 * 12.65e6, "fa_bwd_tc_kernel": 4 * 25.58e6},
    "cfg4": {"fa_fwd_tc_kernel": 2 * (248.4e6 + 49.8e6), "fa_bwd_tc_kernel": 2 * (649.6e6 + 360.2e6)},
}

# S x S x D products per computed block pair that count as algorithmic work of each kernel: the
# forward has two, the backward five (S, dP, dV, dK, dQ), however a kernel splits or recomputes them
PRODUCTS = {"fa_fwd_tc_kernel": 2, "fa_fwd_kernel": 2, "fa_bwd_tc_kernel": 5, "fa_bwd_dkdv_tc_kernel": 4,
            "fa_bwd_dq_tc_kernel": 1, "fa_bwd_dkdv_kernel": 4, "fa_bwd_dq_kernel": 1}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(tflops=p["bf16_tflops"], tflops_sustained=p["bf16_tflops_sustained"], hbm=p["hbm_gbs"],
                    source="measured")
    return dict(tflops=1590.0, tflops_sustained=1400.0, hbm=6650.0, source="fallback")


def mods_for(w):
    from flaxattention_b200.masks import causal_mask, generate_attention_sink
    from flaxattention_b200.mods import checkerboard, generate_alibi_bias

    score = {None: None, "checkerboard": checkerboard, "alibi": generate_alibi_bias(w["H"])}[w["score"]]
    mask = {None: None, "causal": causal_mask, "sink": generate_attention_sink(1024, 4)}[w["mask"]]
    return score, mask


def host_inputs(w, b_offset, pinned):
    """Seeded N(0,1) tensors; batch entry b of the global problem is generated on its own,
    so a shard does not depend on the number of ranks."""
    out = []
    for seed, S in ((1, w["Sq"]), (0, w["Skv"]), (2, w["Skv"])):
        t = torch.empty(w["B"], w["H"], S, w["D"], dtype=DT[w["dtype"]])
        if pinned:
            t = t.pin_memory()
        for b in range(w["B"]):
            g = np.random.Generator(np.random.Philox(key=[seed, b_offset + b]))
            t[b] = torch.from_numpy(g.standard_normal((w["H"], S, w["D"]), dtype=np.float32)).to(t.dtype)
        out.append(t)
    return out


def device_inputs(w, dev, seed=0):
    """N(0,1) tensors made on the device (for the legs whose inputs are resident anyway)."""
    g = torch.Generator(device=dev).manual_seed(seed)
    mk = lambda S: torch.randn(w["B"], w["H"], S, w["D"], generator=g, device=dev, dtype=torch.float32).to(DT[w["dtype"]])  # noqa: E731
    return mk(w["Sq"]), mk(w["Skv"]), mk(w["Skv"])


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU from a background thread through NVML
    while the timed region runs (reading only; nothing is set)."""

    def __init__(self, index, period_s=0.002):
        import threading

        self.samples, self.reasons, self.max_mhz, self.err = [], set(), None, None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # pragma: no cover - depends on the box
            self.err = f"NVML unavailable: {e}"
            return
        self._period = period_s
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self):
        nv = self._nv
        bits = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(
            nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                r = int(get_reasons(self._h))
                for name, bit in bits.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception as e:  # pragma: no cover
                self.err = str(e)
                break
            self._stop.wait(self._period)

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
        out = {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
               "samples": len(self.samples), "reasons": sorted(self.reasons)}
        if self.err:
            out["note"] = self.err
        return out


def cpu_oracle_step(w, sample_b, score, mask):
    """One forward + backward of the CPU oracle on `sample_b` batch entries; returns seconds."""
    from oracle.attention_oracle import attention_grads_oracle

    ws = dict(w, B=sample_b)
    q, k, v = host_inputs(ws, 0, pinned=False)
    dout = torch.ones(sample_b, w["H"], w["Sq"], w["D"])
    t0 = time.perf_counter()
    attention_grads_oracle(q, k, v, dout, score, mask)
    return time.perf_counter() - t0


def flops_fwd(w):
    """Dense-equivalent forward FLOPs: two S x S x D products."""
    return 4.0 * w["B"] * w["H"] * w["Sq"] * w["Skv"] * w["D"]


def run_reference(args, w, rank, world):
    """CPU arm: the oracle port of the reference's dense path on all host threads."""
    if rank != 0:
        return
    score, mask = mods_for(w)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sample_b = 1
    for _ in range(args.warmup):
        cpu_oracle_step(w, sample_b, score, mask)
    ts = [cpu_oracle_step(w, sample_b, score, mask) for _ in range(args.steps)]
    sec = sum(ts) / len(ts)
    fl = 3.5 * flops_fwd(dict(w, B=sample_b))
    val = fl / sec / 1e12
    sample = f"B={sample_b} of {w['B']} batch entries per step, all heads, fwd+bwd, fp32 dense oracle (torch CPU)"
    line = {
        "impl": "reference", "metric": "fwd+bwd attention TFLOP/s (dense-equivalent)", "value": val,
        "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, **{k: w[k] for k in ("B", "H", "Sq", "Skv", "D")},
                   "score_mod": w["score"], "mask": w["mask"], "sample": sample},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the reference needs JAX, which is not installed; this is the CPU oracle port of its dense path",
    }
    print(json.dumps(line), flush=True)


class Bench:
    """Timing helpers bound to one device and (under torchrun) one process group."""

    def __init__(self, dev, world, steps, warmup, leg_seconds=MIN_LEG_SECONDS):
        self.dev, self.world, self.steps, self.warmup, self.leg_seconds = dev, world, steps, warmup, leg_seconds
        self.flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        self.last_timed_steps = 0

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, x):
        if self.world == 1:
            return x
        import torch.distributed as dist
        t = torch.tensor([x], device=self.dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def timed(self, fn, steps=None, warmup=None, min_seconds=None, sync=True):
        """Mean milliseconds per step of fn: `steps` steps, then further blocks of `steps` until the
        leg has lasted `min_seconds`.  L2 is flushed before every step, outside the events."""
        steps = self.steps if steps is None else steps
        min_seconds = self.leg_seconds if min_seconds is None else min_seconds
        for _ in range(self.warmup if warmup is None else warmup):
            fn()
        if sync:
            self.barrier()
        total_ms, n = 0.0, 0
        t_start = time.perf_counter()
        while True:
            evs = []
            for _ in range(steps):
                self.flush_buf.fill_(1)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                evs.append((e0, e1))
            torch.cuda.synchronize()
            total_ms += sum(a.elapsed_time(b) for a, b in evs)
            n += steps
            if time.perf_counter() - t_start >= min_seconds or n >= 200 * steps:
                break
        if sync:
            self.barrier()
        self.last_timed_steps = n
        return total_ms / n


def computed_flops_fwd(w, bm):
    """Forward FLOPs of the blocks a BlockMask lists (dense-equivalent without one)."""
    if bm is None:
        return flops_fwd(w)
    blocks = bm.computed_blocks() * (w["B"] // bm.kv_indices.shape[0]) * (w["H"] // bm.kv_indices.shape[1])
    return 4.0 * w["D"] * bm.BLOCK_SIZE[0] * bm.BLOCK_SIZE[1] * blocks


def measure_workload(bench, w, q, k, v, b_off, h_off, bm, pk, steps, with_kernels=True, name=None):
    """Device-timed forward + backward of one workload with resident inputs: step time, forward
    time, per-kernel times (from the library's event records) and the roofline of the dominant one."""
    from flaxattention_b200 import _cabi
    from flaxattention_b200 import attention as A

    score, mask = mods_for(w)
    mask_mod = None if bm is None else bm.mask_mod
    dout = torch.ones(q.shape[0], q.shape[1], w["Sq"], w["D"], dtype=q.dtype, device=q.device)
    call = A._Call(q, k, v, score, mask_mod, bm, 1.0 / math.sqrt(w["D"]), "bhsd", b_off, h_off, {"flags": 0})

    def step():
        out, lse = A._forward(call, q, k, v)
        return A._backward(call, q, k, v, out, lse, dout)

    res = {"ms_per_step": bench.timed(step, steps), "timed_steps": bench.last_timed_steps}
    if not with_kernels:
        return res
    res["fwd_ms"] = bench.timed(lambda: A._forward(call, q, k, v), steps, 3, sync=False)
    # per-kernel device times: the library brackets each launch with events while profiling is on
    out, lse = A._forward(call, q, k, v)
    acc, n = {}, max(5, steps // 4)
    _cabi.profile_enable(True)
    try:
        for _ in range(n):
            bench.flush_buf.fill_(1)
            A._forward(call, q, k, v)
            recs = _cabi.profile_read()
            A._backward(call, q, k, v, out, lse, dout)
            recs += _cabi.profile_read()
            for kname, ms in recs:
                acc[kname] = acc.get(kname, 0.0) + ms
    finally:
        _cabi.profile_enable(False)
    shard = dict(w, B=q.shape[0], H=q.shape[1])
    fl_dense = flops_fwd(shard)
    fl_comp = computed_flops_fwd(shard, bm)
    kernels = {}
    for kname, ms in acc.items():
        ms /= n
        d = {"ms": ms}
        if kname in PRODUCTS:
            d["algorithmic_tflops"] = PRODUCTS[kname] * (fl_comp / 2.0) / (ms * 1e-3) / 1e12
            d["frac_of_measured_peak"] = d["algorithmic_tflops"] / pk["tflops"]
        kernels[kname] = d
    res["kernels"] = kernels
    res["launches_per_step"] = len(acc)
    dom = max((nm for nm in kernels if nm in PRODUCTS), key=lambda nm: kernels[nm]["ms"])
    ach = kernels[dom]["algorithmic_tflops"]
    res["roofline"] = {"bound": "tensor", "kernel": dom, "achieved": ach, "peak": pk["tflops"], "unit": "TFLOP/s",
                       "frac": ach / pk["tflops"], "peak_source": pk["source"] + " (bf16 cuBLAS burst)",
                       "frac_of_nominal_2250": ach / 2250.0, "traffic": NCU_TRAFFIC.get(name, {}).get(dom),
                       "flops": "S x S x D products of the computed blocks that the kernel owes (2 forward, 5 backward)"}
    t_fwd = res["fwd_ms"]
    res["fwd"] = {"ms": t_fwd, "tflops_dense_equivalent": fl_dense / (t_fwd * 1e-3) / 1e12,
                  "tflops_computed_blocks": fl_comp / (t_fwd * 1e-3) / 1e12,
                  "frac_of_measured_peak": fl_comp / (t_fwd * 1e-3) / 1e12 / pk["tflops"]}
    res["tflops_dense_equivalent"] = 3.5 * fl_dense / (res["ms_per_step"] * 1e-3) / 1e12
    res["tflops_computed_blocks"] = 3.5 * fl_comp / (res["ms_per_step"] * 1e-3) / 1e12
    if bm is not None:
        res["sparsity_pct"] = bm.sparsity()
    return res


def bind_rank_to_cores(rank_local, world_local):
    """Gives each local rank its own slice of the cores this process may run on, before it
    allocates (and first touches) its pinned buffers, so the ranks' staging memory and copy
    threads do not pile onto the same cores."""
    try:
        cpus = sorted(os.sched_getaffinity(0))
        per = len(cpus) // world_local
        if per >= 1:
            mine = cpus[rank_local * per:(rank_local + 1) * per]
            os.sched_setaffinity(0, mine)
            return f"{mine[0]}-{mine[-1]}"
    except (AttributeError, OSError):
        pass
    return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-extras", action="store_true", help="skip forward-only, decode, per-kernel and CPU legs")
    ap.add_argument("--leg-seconds", type=float, default=MIN_LEG_SECONDS,
                    help="minimum duration of a timed leg (0: exactly --steps steps, e.g. for a profiler's launch list)")
    ap.add_argument("--profile", default=None, choices=["fwd", "bwd", "decode", "decode64"],
                    help="small case for a profiler: a few launches of one kernel family, no JSON line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    w = WORKLOADS[args.workload]

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, w, rank, world)
        return
    if args.profile:
        run_profile_case(args, w)
        return

    import flaxattention_b200 as fa
    from flaxattention_b200.sharding import shard_for

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    cores = bind_rank_to_cores(local_rank, world) if world > 1 else None
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    bench = Bench(dev, world, args.steps, args.warmup, args.leg_seconds)
    pk = peaks()

    score, mask = mods_for(w)
    b_off = w["B"] * rank
    hq, hk, hv = host_inputs(w, b_off, pinned=True)
    q, k, v = hq.to(dev), hk.to(dev), hv.to(dev)
    bm = None
    if mask is not None:
        bm = fa.create_block_mask(mask, w["B"], w["H"], w["Sq"], w["Skv"], b_offset=b_off)

    # ---- headline: fwd + bwd, inputs resident in HBM -----------------------------------
    sampler = ClockSampler(local_rank) if rank == 0 else None
    head = measure_workload(bench, w, q, k, v, b_off, 0, bm, pk, args.steps, with_kernels=not args.no_extras,
                            name=args.workload)
    clocks = sampler.stop() if sampler else None
    ms = bench.max_over_ranks(head["ms_per_step"])
    fl_fwd = flops_fwd(w)
    value = 3.5 * fl_fwd * world / (ms * 1e-3) / 1e12

    # ---- e2e: pinned host buffers in and out, copies inside the timing -------------------
    pipe = fa.HostPipeline(w["B"], w["H"], w["H"], w["Sq"], w["Skv"], w["D"], dtype=DT[w["dtype"]], device=dev,
                           score_mod=score, block_mask=bm, b_offset=b_off)
    ho, hdq, hdk, hdv = (torch.empty_like(hq).pin_memory() for _ in range(4))
    ms_e2e = bench.max_over_ranks(bench.timed(lambda: pipe.step(hq, hk, hv, ho, hdq, hdk, hdv), max(3, args.steps // 2), 3))
    h2d, d2h = pipe.bytes_per_step()
    e2e = {"value": 3.5 * fl_fwd * world / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "timed_steps": bench.last_timed_steps,
           "api": f"flaxattention_b200.HostPipeline.step ({len(pipe.chunks)} chunks of batch entries, one CUDA graph)",
           "h2d_gbs_per_rank": h2d / (ms_e2e * 1e-3) / 1e9, "d2h_gbs_per_rank": d2h / (ms_e2e * 1e-3) / 1e9,
           "cores_of_rank0": cores}

    launches = head.get("launches_per_step", 4)
    line = {
        "metric": "fwd+bwd attention TFLOP/s (dense-equivalent)", "value": value, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "timed_steps": head["timed_steps"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": args.workload, **{k_: w[k_] for k_ in ("B", "H", "Sq", "Skv", "D")},
                   "score_mod": w["score"], "mask": w["mask"], "global_batch": w["B"] * world,
                   "parallelism": f"batch x heads shards, {world} rank(s), no collective",
                   "l2": "flushed between timed steps (256 MiB write)", "flops": "3.5 * 4*B*H*Sq*Skv*D per step",
                   "leg": f"each timed leg repeats its K steps until it has run for {args.leg_seconds} s"},
        "e2e": e2e, "gpu_launches": launches * head["timed_steps"], "clocks": clocks,
    }
    for key in ("kernels", "roofline", "fwd"):
        if key in head:
            line[key] = head[key]
    if bm is not None and "tflops_computed_blocks" in head:
        line["computed_blocks"] = {"fwd_bwd_tflops": head["tflops_computed_blocks"] * world, "sparsity_pct": head["sparsity_pct"]}
    del pipe, ho, hdq, hdk, hdv, q, k, v

    if not args.no_extras:
        if world > 1:
            line["strong"] = bench_strong(bench, fa, shard_for, rank, world, dev, pk, max(5, args.steps // 4))
        else:
            line["workloads"] = {}
            for name in ("cfg3", "cfg4"):
                if name == args.workload:
                    continue
                ww = WORKLOADS[name]
                qq, kk, vv = device_inputs(ww, dev)
                _, m2 = mods_for(ww)
                bm2 = fa.create_block_mask(m2, ww["B"], ww["H"], ww["Sq"], ww["Skv"])
                r = measure_workload(bench, ww, qq, kk, vv, 0, 0, bm2, pk, max(5, args.steps // 4), name=name)
                r["config"] = {k_: ww[k_] for k_ in ("B", "H", "Sq", "Skv", "D", "dtype", "score", "mask")}
                line["workloads"][name] = r
                del qq, kk, vv, bm2
            line["decode"] = bench_decode(fa, dev, bench, pk)
            cores_n = os.cpu_count() or 1
            torch.set_num_threads(cores_n)
            sb = 1
            cpu_oracle_step(w, sb, score, mask)
            ts = [cpu_oracle_step(w, sb, score, mask) for _ in range(5)]
            sec = sum(ts) / len(ts)
            line["cpu_baseline"] = {
                "value": 3.5 * flops_fwd(dict(w, B=sb)) / sec / 1e12, "unit": "TFLOP/s", "cores": cores_n,
                "kind": "port",
                "sample": f"B={sb} of {w['B']} batch entries, all heads, fwd+bwd, 5 repetitions, fp32 dense oracle"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def bench_strong(bench, fa, shard_for, rank, world, dev, pk, steps):
    """Strong scaling of fixed global problems cut by batch x heads (flaxattention_b200.sharding):
    the attention-sink configuration B4 H16 S8192 D128 (8 ranks: a 4 x 2 mesh, odd ranks start at
    head 8) and the default B8 H8 S2048 D64 one.  Every rank times its shard with the global
    offsets; value = global FLOPs of the computed blocks / the slowest rank's time.  Rank 0 then
    times the whole problem alone for the one-GPU reference of the same run."""
    out = {}
    for name in ("cfg4", "cfg2"):
        w = WORKLOADS[name]
        sh = shard_for(rank, world, w["B"], w["H"], w["H"])
        _, mask = mods_for(w)
        nb, nh = sh.b.stop - sh.b.start, sh.hq.stop - sh.hq.start
        q, k, v = device_inputs(dict(w, B=nb, H=nh), dev, seed=1 + rank)
        bm_global = fa.create_block_mask(mask, w["B"], w["H"], w["Sq"], w["Skv"]) if mask is not None else None
        bm = None if bm_global is None else bm_global.shard(sh.b, sh.hq)
        r = measure_workload_shard(bench, w, q, k, v, sh.b_offset, sh.h_offset, bm, steps)
        ms_n = bench.max_over_ranks(r)
        fl = 3.5 * computed_flops_fwd(w, bm_global)
        ent = {"mesh": list(sh.mesh), "shard": {"B": nb, "H": nh, "b_offset_of_last_rank": None},
               "ms_per_step": ms_n, "tflops_computed_blocks": fl / (ms_n * 1e-3) / 1e12,
               "tflops_dense_equivalent": 3.5 * flops_fwd(w) / (ms_n * 1e-3) / 1e12}
        last = shard_for(world - 1, world, w["B"], w["H"], w["H"])
        ent["shard"]["b_offset_of_last_rank"], ent["shard"]["h_offset_of_last_rank"] = last.b_offset, last.h_offset
        del q, k, v
        bench.barrier()
        if rank == 0:
            qq, kk, vv = device_inputs(w, dev)
            one = measure_workload_shard(bench, w, qq, kk, vv, 0, 0, bm_global, steps, sync=False)
            ent["one_gpu_ms_per_step"] = one
            ent["efficiency_vs_one_gpu"] = one / (world * ms_n)
            del qq, kk, vv
        bench.barrier()
        if name == "cfg2":
            ent["note"] = (f"a shard is B={nb} x H={nh}: {nb * nh * (w['Sq'] // 256)} forward CTAs and "
                           f"{nb * nh * (w['Skv'] // 128)} backward items (kv tiles) for 148 SMs")
        out[name] = ent
    return out


def measure_workload_shard(bench, w_global, q, k, v, b_off, h_off, bm, steps, sync=True):
    """Mean step time of one shard of `w_global` (mods are built from the global head count)."""
    from flaxattention_b200 import attention as A

    score, _ = mods_for(w_global)
    mask_mod = None if bm is None else bm.mask_mod
    dout = torch.ones_like(q)
    call = A._Call(q, k, v, score, mask_mod, bm, 1.0 / math.sqrt(w_global["D"]), "bhsd", b_off, h_off, {"flags": 0})

    def step():
        out, lse = A._forward(call, q, k, v)
        return A._backward(call, q, k, v, out, lse, dout)

    return bench.timed(step, steps, 3, sync=sync)


def run_profile_case(args, w):
    """A few launches of one kernel family on a reduced batch, for ncu (a capture replays every
    launch many times, so the case is kept small).  fwd / bwd: the workload with B=2;
    decode / decode64: B=8, H=8, Skv=16384, Sq=1 / 64 (K+V = 268 MB, larger than L2)."""
    import flaxattention_b200 as fa
    from flaxattention_b200 import attention as A
    from flaxattention_b200.masks import generate_causal_offset
    from flaxattention_b200.mods import generate_alibi_bias

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if args.profile in ("decode", "decode64"):
        sq = 1 if args.profile == "decode" else 64
        d = dict(DECODE, B=8)
        kk = torch.randn(d["B"], d["H"], d["Skv"], d["D"], device=dev, dtype=DT[d["dtype"]])
        vv = torch.randn_like(kk)
        qq = torch.randn(d["B"], d["H"], sq, d["D"], device=dev, dtype=kk.dtype)
        bm = fa.create_block_mask(generate_causal_offset(d["Skv"] - sq), d["B"], d["H"], sq, d["Skv"])
        for _ in range(4):
            fa.flax_attention_pallas(qq, kk, vv, score_mod=generate_alibi_bias(d["H"]), block_mask=bm)
        torch.cuda.synchronize()
        return
    ws = dict(w, B=2)
    score, mask = mods_for(ws)
    q, k, v = (t.to(dev) for t in host_inputs(ws, 0, pinned=False))
    bm = fa.create_block_mask(mask, ws["B"], ws["H"], ws["Sq"], ws["Skv"]) if mask is not None else None
    call = A._Call(q, k, v, score, None if bm is None else bm.mask_mod, bm, 1.0 / math.sqrt(ws["D"]), "bhsd", 0, 0, None)
    dout = torch.ones(ws["B"], ws["H"], ws["Sq"], ws["D"], dtype=q.dtype, device=dev)
    for _ in range(4):
        out, lse = A._forward(call, q, k, v)
        if args.profile == "bwd":
            A._backward(call, q, k, v, out, lse, dout)
    torch.cuda.synchronize()


def bench_decode(fa, dev, bench, pk):
    from flaxattention_b200.masks import generate_causal_offset
    from flaxattention_b200.mods import generate_alibi_bias

    d = DECODE
    res = {}
    kk = torch.randn(d["B"], d["H"], d["Skv"], d["D"], device=dev, dtype=DT[d["dtype"]])
    vv = torch.randn_like(kk)
    alibi = generate_alibi_bias(d["H"])
    for sq in (1, 16, 64):
        qq = torch.randn(d["B"], d["H"], sq, d["D"], device=dev, dtype=kk.dtype)
        bm = fa.create_block_mask(generate_causal_offset(d["Skv"] - sq), d["B"], d["H"], sq, d["Skv"])
        fn = lambda: fa.flax_attention_pallas(qq, kk, vv, score_mod=alibi, block_mask=bm)  # noqa: E731
        ms = bench.timed(fn, 20, 3, sync=False)
        nbytes = 2 * kk.numel() * 2 + 2 * qq.numel() * 2
        res[f"sq{sq}"] = {"ms": ms, "gbs": nbytes / (ms * 1e-3) / 1e9, "frac_of_measured_hbm": nbytes / (ms * 1e-3) / 1e9 / pk["hbm"]}
    return res


if __name__ == "__main__":
    main()
