"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the hot path over one batch: the flash forward and the flash
backward (dQ, dK, dV of output.sum()) of the workload.  The default workload is the
configuration the headline metric is quoted on: B=8, H=8, Sq=Skv=2048, D=64, fp16,
checkerboard score_mod, no mask (examples/benchmark.py of the reference).  Inputs are
synthetic N(0,1) tensors from fixed seeds (K: 0, Q: 1, V: 2).

Scaling is weak: under torchrun every rank processes its own batch of 8 with the global
batch offset 8 * rank passed to the kernels, and there is no data-path collective.

The single JSON line carries the contract keys plus:
  roofline      the dominant kernel against the measured bf16 tensor peak
  kernels       per-kernel device time and achieved TFLOP/s
  fwd / decode  forward-only TFLOP/s and split-KV decode GB/s (N=1)
  cpu_baseline  the CPU oracle (a port of the reference's dense path) timed on this box's
                host cores on a bounded sample
  e2e           the same step through the public API with pinned host buffers: host->device
                copies of q, k, v and device->host copies of out, dq, dk, dv inside the timing
`--impl reference` times the CPU oracle alone (the reference itself needs JAX, which is not
installed); it is the one place besides cpu_baseline where bench.py runs code from oracle/.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

WORKLOADS = {
    # name: B, H, Sq, Skv, D, dtype, score_mod, mask, block
    "cfg2": dict(B=8, H=8, Sq=2048, Skv=2048, D=64, dtype="f16", score="checkerboard", mask=None),
    "cfg2_nomod": dict(B=8, H=8, Sq=2048, Skv=2048, D=64, dtype="f16", score=None, mask=None),
    "cfg3": dict(B=8, H=8, Sq=2048, Skv=2048, D=64, dtype="bf16", score="alibi", mask="causal"),
    "cfg4": dict(B=4, H=16, Sq=8192, Skv=8192, D=128, dtype="bf16", score=None, mask="sink"),
}
DECODE = dict(B=32, H=8, Skv=16384, D=64, dtype="f16")
DT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}

# dram__bytes_read.sum + dram__bytes_write.sum per launch from ncu captures (profiles/); None = not captured
# (captured on the B=2 profile case and scaled by 4 to the B=8 workload: traffic grows with the batch)
NCU_TRAFFIC = {"fa_fwd_tc_kernel": 4 * 12.66e6, "fa_bwd_tc_kernel": 4 * 25.49e6, "fa_fwd_kernel": None, "fa_bwd_dkdv_kernel": None,
               "fa_bwd_dq_kernel": None}


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
        for b in range(w["B"]):
            g = np.random.Generator(np.random.Philox(key=[seed, b_offset + b]))
            t[b] = torch.from_numpy(g.standard_normal((w["H"], S, w["D"]), dtype=np.float32)).to(t.dtype)
        out.append(t.pin_memory() if pinned else t)
    return out


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-extras", action="store_true", help="skip forward-only, decode, per-kernel and CPU legs")
    ap.add_argument("--profile", default=None, choices=["fwd", "bwd", "decode"],
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
    from flaxattention_b200 import _cabi
    from flaxattention_b200 import attention as A

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    score, mask = mods_for(w)
    b_off = w["B"] * rank
    hq, hk, hv = host_inputs(w, b_off, pinned=True)
    q, k, v = hq.to(dev), hk.to(dev), hv.to(dev)
    bm = None
    if mask is not None:
        bm = fa.create_block_mask(mask, w["B"], w["H"], w["Sq"], w["Skv"], b_offset=b_off)
    dout = torch.ones(w["B"], w["H"], w["Sq"], w["D"], dtype=q.dtype, device=dev)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def flush_l2():
        flush_buf.fill_(1)

    mask_mod = None if bm is None else bm.mask_mod

    def make_call(flags=0):
        return A._Call(q, k, v, score, mask_mod, bm, 1.0 / math.sqrt(w["D"]), "bhsd", b_off, 0, {"flags": flags})

    call = make_call()

    def step_kernels():
        out, lse = A._forward(call, q, k, v)
        return A._backward(call, q, k, v, out, lse, dout)

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        evs = []
        for _ in range(steps):
            flush_l2()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            evs.append((e0, e1))
        barrier()
        return sum(a.elapsed_time(b) for a, b in evs) / steps  # ms per step

    # ---- headline: fwd + bwd, inputs resident in HBM -----------------------------------
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms = timed(step_kernels, args.steps, args.warmup)
    clocks = sampler.stop() if sampler else None
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    fl_fwd = flops_fwd(w)
    value = 3.5 * fl_fwd * world / (ms * 1e-3) / 1e12

    # ---- e2e: public API, pinned host buffers, copies inside the timing -----------------
    ho = [torch.empty_like(hq).pin_memory() for _ in range(4)]

    def step_e2e():
        qd = hq.to(dev, non_blocking=True).requires_grad_(True)
        kd = hk.to(dev, non_blocking=True).requires_grad_(True)
        vd = hv.to(dev, non_blocking=True).requires_grad_(True)
        out = fa.flax_attention_pallas(qd, kd, vd, score_mod=score, mask_mod=mask_mod, block_mask=bm, b_offset=b_off)
        out.backward(dout)
        ho[0].copy_(out.detach(), non_blocking=True)
        ho[1].copy_(qd.grad, non_blocking=True)
        ho[2].copy_(kd.grad, non_blocking=True)
        ho[3].copy_(vd.grad, non_blocking=True)

    ms_e2e = timed(step_e2e, max(3, args.steps // 2), 3)
    if world > 1:
        t = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = t.item()
    nbytes = hq.numel() * hq.element_size()
    e2e = {"value": 3.5 * fl_fwd * world / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
           "h2d_bytes_per_step": 3 * nbytes, "d2h_bytes_per_step": 4 * nbytes}

    line = {
        "metric": "fwd+bwd attention TFLOP/s (dense-equivalent)", "value": value, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": args.workload, **{k_: w[k_] for k_ in ("B", "H", "Sq", "Skv", "D")},
                   "score_mod": w["score"], "mask": w["mask"], "global_batch": w["B"] * world,
                   "parallelism": f"batch x heads shards, {world} rank(s), no collective",
                   "l2": "flushed between timed steps (256 MiB write)", "flops": "3.5 * 4*B*H*Sq*Skv*D per step"},
        "e2e": e2e, "gpu_launches": 4 * args.steps, "clocks": clocks,
    }

    # ---- per-kernel timing, roofline, forward-only, decode, CPU baseline (rank 0, N=1 legs) ----
    pk = peaks()
    if not args.no_extras:
        steps_k = max(5, args.steps // 2)
        out, lse = A._forward(call, q, k, v)
        t_fwd = timed(lambda: A._forward(call, q, k, v), steps_k, 3)
        # this workload runs the tcgen05 kernels: the forward, and a single-pass backward made
        # of fa_bwd_prep_kernel (row scalars; it also clears the dQ accumulator), fa_bwd_tc_kernel
        # and fa_dq_convert_kernel; the FA_FLAG_BWD_SKIP_* aids isolate them (run alone, the main
        # kernel is preceded by a memset of the accumulator instead)
        tc = w["D"] == 64 and w["dtype"] != "f32"
        fwd_name = "fa_fwd_tc_kernel" if tc else "fa_fwd_kernel"
        main_name, post_name = ("fa_bwd_tc_kernel", "fa_dq_convert_kernel") if tc else ("fa_bwd_dkdv_kernel", "fa_bwd_dq_kernel")
        pre_name = "fa_bwd_prep_kernel" if tc else "fa_delta_kernel"
        only = {
            main_name: _cabi.FLAG_BWD_SKIP_DELTA | _cabi.FLAG_BWD_SKIP_DQ,
            post_name: _cabi.FLAG_BWD_SKIP_DELTA | _cabi.FLAG_BWD_SKIP_DKDV,
            pre_name: _cabi.FLAG_BWD_SKIP_DKDV | _cabi.FLAG_BWD_SKIP_DQ,
        }
        A._backward(call, q, k, v, out, lse, dout)  # delta is in place for the partial runs
        unit = fl_fwd / 4.0  # one S x S x D product = 2*B*H*Sq*Skv*D
        alg = {fwd_name: 2 * unit, main_name: (5 if tc else 4) * unit, post_name: (0 if tc else 1) * unit,
               pre_name: 0.0}
        kernels = {fwd_name: {"ms": t_fwd}}
        for name, flags in only.items():
            c2 = make_call(flags)
            kernels[name] = {"ms": timed(lambda c2=c2: A._backward(c2, q, k, v, out, lse, dout), steps_k, 3)}
        for name, d in kernels.items():
            d["algorithmic_tflops"] = alg[name] / (d["ms"] * 1e-3) / 1e12 if alg[name] else None
        dom = max((n for n in kernels if alg[n]), key=lambda n: kernels[n]["ms"])
        ach = kernels[dom]["algorithmic_tflops"]
        line["kernels"] = kernels
        line["roofline"] = {"bound": "tensor", "kernel": dom, "achieved": ach, "peak": pk["tflops"], "unit": "TFLOP/s",
                            "frac": ach / pk["tflops"], "peak_source": pk["source"] + " (bf16 cuBLAS burst)",
                            "frac_of_nominal_2250": ach / 2250.0, "traffic": NCU_TRAFFIC.get(dom)}
        line["fwd"] = {"ms": t_fwd, "tflops": fl_fwd / (t_fwd * 1e-3) / 1e12,
                       "frac_of_measured_peak": fl_fwd / (t_fwd * 1e-3) / 1e12 / pk["tflops"]}
        if bm is not None:
            blocks = bm.computed_blocks() * (w["B"] // bm.kv_indices.shape[0]) * (w["H"] // bm.kv_indices.shape[1])
            comp = 4.0 * w["D"] * bm.BLOCK_SIZE[0] * bm.BLOCK_SIZE[1] * blocks
            line["computed_blocks"] = {"fwd_tflops": comp / (t_fwd * 1e-3) / 1e12,
                                       "fwd_bwd_tflops": 3.5 * comp * world / (ms * 1e-3) / 1e12,
                                       "sparsity_pct": bm.sparsity()}
        if world == 1:
            line["decode"] = bench_decode(fa, dev, timed, pk)
            if rank == 0:
                cores = os.cpu_count() or 1
                torch.set_num_threads(cores)
                sb = 1
                cpu_oracle_step(w, sb, score, mask)
                ts = [cpu_oracle_step(w, sb, score, mask) for _ in range(5)]
                sec = sum(ts) / len(ts)
                line["cpu_baseline"] = {
                    "value": 3.5 * flops_fwd(dict(w, B=sb)) / sec / 1e12, "unit": "TFLOP/s", "cores": cores,
                    "kind": "port",
                    "sample": f"B={sb} of {w['B']} batch entries, all heads, fwd+bwd, 5 repetitions, fp32 dense oracle"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_profile_case(args, w):
    """A few launches of one kernel family on a reduced batch, for ncu (a capture replays every
    launch many times, so the case is kept small).  fwd / bwd: the workload with B=2;
    decode: B=8, H=8, Skv=16384, Sq=1 (K+V = 268 MB, larger than L2)."""
    import flaxattention_b200 as fa
    from flaxattention_b200 import attention as A
    from flaxattention_b200.masks import generate_causal_offset
    from flaxattention_b200.mods import generate_alibi_bias

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if args.profile == "decode":
        d = dict(DECODE, B=8)
        kk = torch.randn(d["B"], d["H"], d["Skv"], d["D"], device=dev, dtype=DT[d["dtype"]])
        vv = torch.randn_like(kk)
        qq = torch.randn(d["B"], d["H"], 1, d["D"], device=dev, dtype=kk.dtype)
        bm = fa.create_block_mask(generate_causal_offset(d["Skv"] - 1), d["B"], d["H"], 1, d["Skv"])
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


def bench_decode(fa, dev, timed, pk):
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
        ms = timed(fn, 20, 3)
        nbytes = 2 * kk.numel() * 2 + 2 * qq.numel() * 2
        res[f"sq{sq}"] = {"ms": ms, "gbs": nbytes / (ms * 1e-3) / 1e9, "frac_of_measured_hbm": nbytes / (ms * 1e-3) / 1e9 / pk["hbm"]}
    return res


if __name__ == "__main__":
    main()
