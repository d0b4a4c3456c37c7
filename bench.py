"""Benchmark of the JVP flash-attention hot path (fused forward-dual + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline workload (default ``c2_bf16_causal``): bf16 causal self-attention B=4, H=16, L=2048, D=64, q,k,v ~
N(0,1), tangents ~ N(0,0.1^2), target ~ N(0,1), seeded synthetic data; one step = fwd_dual (primal + tangent)
followed by the backward of loss = mean((tO - target)^2) to q, k, v.  With N ranks every rank runs the whole
configuration on its own (batch x head) shard of a batch N times larger (no collective on the data path; weak
scaling), and ``value`` sums all ranks.

One JSON line is printed by rank 0.  ``value`` is device-resident throughput through the C ABI (CUDA events per
step, max over ranks, L2 flushed between steps); ``e2e`` is the same step through the public Python API with
pinned host inputs copied in and the loss read back every step.  Further keys of the same line:

  sustained          the same step back to back for seconds (no flush), with the clocks and power seen
  other_workloads    the other benchmark configurations (fp32 plumbing, fp16 key padding, fp32 bias + HVP, a shard
                     of the long-sequence one): ms through the C ABI and through the public API
  reference_triton   upstream's own Triton kernels timed in the same run on the same tensors (N = 1)
  c5_strong          the long-sequence configuration (B32 H16 L8192 D128, 512 (batch, head) units) split over the
                     ranks; results gathered over NCCL for verification only
  roofline, cpu_baseline   the dominant call against the measured tensor peak; upstream's CPU path on the host

``--impl reference`` times upstream's CPU path (torch.func.jvp over SDPA-MATH + autograd) on the host cores on a
bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "fwd_dual+bwd TFLOP/s (bf16 causal B4 H16 L2048 D64; algorithmic MMA flops)"
CPU_SAMPLE_HEADS = 8
DEFAULT_WORKLOAD = "c2_bf16_causal"
# DRAM bytes per call of the timed kernels from an ncu capture of this source tree, with the commit it was taken
# at; when the file is absent or describes another workload the roofline's traffic is null.
TRAFFIC_FILE = ROOT / "profiles" / "ncu_dram_traffic.json"


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm=d["hbm_gbs"], burst=d["bf16_tflops"], sustained=d["bf16_tflops_sustained"], src="measured")
    return dict(hbm=6650.0, burst=1590.0, sustained=1400.0, src="fallback")


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU with nvidia-smi while a timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
                pw.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


def _dist_env():
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


# ------------------------------------------------------------------------------------------------
# Upstream's CPU path (reference arm and cpu_baseline)
# ------------------------------------------------------------------------------------------------
def _cpu_reference(wname: str, steps: int, warmup: int):
    """Upstream's CPU path on a bounded sample: CPU_SAMPLE_HEADS (batch, head) slices of the workload."""
    from jvp_flash_attention_b200 import workloads
    from oracle import jvp_attention_oracle as orc

    spec = workloads.SPECS[wname]
    w = workloads.make_workload(wname, B=1, H=CPU_SAMPLE_HEADS)
    t = w.tensors
    n = t["q"].numel() * (spec[1] * spec[2]) // CPU_SAMPLE_HEADS  # loss normaliser of the full workload

    def loss_fn(o, to):
        return ((to.float() - t["target"].float()) ** 2).sum() / n

    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        orc.cpu_reference_step(t["q"], t["k"], t["v"], t["tq"], t["tk"], t["tv"], loss_fn, causal=w.causal,
                               dtype=torch.float32)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    fl = workloads.flops(w, ("fwd_dual", "bwd_to"))
    sec = sum(times) / len(times)
    return fl / sec / 1e12, sec, f"{CPU_SAMPLE_HEADS} of {spec[1] * spec[2]} (batch, head) slices, fp32, {len(times)} timed steps"


def run_reference(args, rank, world):
    if rank != 0:
        return
    steps = max(3, min(args.steps, 5))
    warm = 1 if args.warmup > 0 else 0
    torch.set_num_threads(max(1, os.cpu_count() or 1))  # torchrun pins OMP_NUM_THREADS=1; use every host core
    tf, sec, sample = _cpu_reference(args.workload, steps, warm)
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "path": "torch.func.jvp over SDPA-MATH + autograd on host cores",
                   "sample": sample, "host_cpus": os.cpu_count()},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# Timing helpers
# ------------------------------------------------------------------------------------------------
def _time_call(fn, reps, flush=None):
    """Mean ms of fn() with CUDA events, each repetition timed alone (L2 flushed first when a buffer is given).
    Two untimed calls come first: a kernel's first launch in a process includes loading its module."""
    fn()
    fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        if flush is not None:
            flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    return sum(ts) / len(ts)


def _time_loop(fn, warmup, iters):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


class CStep:
    """One fwd_dual + preprocess + backward step of a workload through the C ABI, every buffer preallocated.
    ``cot``: which cotangents the backward takes ('gt': of tO only, 'both': w1 for O and w2 for tO)."""

    def __init__(self, d, spec, scale, cot, dev):
        from jvp_flash_attention_b200 import _lib

        self.lib, self.d, self.spec, self.scale, self.cot = _lib, d, spec, scale, cot
        q = d["q"]
        B, H, L, D = q.shape
        self.o, self.to = torch.empty_like(q), torch.empty_like(q)
        self.lse = torch.empty(B, H, L, device=dev, dtype=torch.float32)
        self.mu = torch.empty_like(self.lse)
        self.stats = torch.empty(3, B, H, L, device=dev, dtype=torch.float32)
        self.dq, self.dk, self.dv = (torch.empty_like(q) for _ in range(3))
        self.go = d["w1"] if cot == "both" else None
        self.gto = d["w2"] if cot == "both" else torch.empty_like(q)
        single = D == 64 and q.dtype != torch.float32 and spec.kind in _lib.INDEX_MASKS
        self.acc = torch.empty(q.shape, device=dev, dtype=torch.float32) if single else None

    def fwd(self, impl=0):
        d = self.d
        self.lib.fwd(d["q"], d["k"], d["v"], d["tq"], d["tk"], d["tv"], self.o, self.to, self.lse, self.mu, self.spec,
                     self.scale, impl)

    def pre(self):
        self.lib.bwd_preprocess(self.o, self.to, self.go, self.gto, self.mu, self.stats[0], self.stats[1], self.stats[2])

    def bwd(self, impl=0, single_pass=True):
        d = self.d
        self.lib.bwd(d["q"], d["k"], d["v"], d["tq"], d["tk"], d["tv"], self.go, self.gto, self.lse, self.mu,
                     self.stats[0], self.stats[1], self.stats[2], self.dq, self.dk, self.dv, self.spec, self.scale,
                     impl, dq_accum=self.acc if single_pass else None)

    def step(self):
        self.fwd()
        self.pre()
        self.bwd()


def _mask_spec(w, d):
    from jvp_flash_attention_b200 import _lib

    if w.causal:
        return _lib.MaskSpec(_lib.MASK_CAUSAL)
    if w.mask_kind == "kvlen":
        return _lib.MaskSpec(_lib.MASK_KVLEN, d["kv_len"].to(torch.int32))
    if w.mask_kind == "bias":
        m = d["mask"]
        return _lib.MaskSpec(_lib.MASK_BIAS, m, m.stride(), _lib.DTYPE_ENUM[m.dtype])
    return _lib.MaskSpec(_lib.MASK_NONE)


# ------------------------------------------------------------------------------------------------
# Extra legs (rank 0, N = 1): the other configurations, upstream's Triton kernels
# ------------------------------------------------------------------------------------------------
def other_workloads(dev, peaks):
    """ms per step of the other benchmark configurations, device-resident through the C ABI and through the public
    API (tensors on the device, torch.func.jvp + autograd.grad), with the algorithmic MMA flops of each."""
    import jvp_flash_attention_b200.jvp_attention as ja
    from jvp_flash_attention_b200 import workloads

    out = {}
    cases = [("c1_fp32_plumbing", None), ("c3_fp16_keypad", None), ("c4_fp32_bias_hvp", None), ("c5_bf16_long", (0, 16))]
    for name, heads in cases:
        w = workloads.make_workload(name, heads=heads) if heads else workloads.make_workload(name)
        d = {k_: v_.to(dev) for k_, v_ in w.tensors.items() if isinstance(v_, torch.Tensor)}
        mask = d.get("mask")
        rec = {"shape": [w.B, w.H, w.L, w.D], "dtype": str(w.dtype).replace("torch.", "")}
        if heads:
            rec["shard"] = f"(batch, head) units {heads[0]}..{heads[1] - 1} of 512"
        iters = 20 if w.L <= 2048 else 5
        if w.loss == "hvp":
            # primal + tangent forward, then the Hessian-vector product d/dq <d/dq sum(O*w), v_dir> through the API
            stages = ("fwd_dual", "fwd", "bwd_o", "fwd_dual", "bwd_to")

            def api():
                torch.func.jvp(lambda q_, k_, v_: ja.JVPAttn.fwd_dual(q_, k_, v_, attn_mask=mask),
                               (d["q"], d["k"], d["v"]), (d["tq"], d["tk"], d["tv"]))
                q1 = d["q"].detach().requires_grad_()
                o1 = ja.attention(q1, d["k"], d["v"], attn_mask=mask)
                (g,) = torch.autograd.grad((o1 * d["w"]).sum(), q1, create_graph=True)
                (h,) = torch.autograd.grad((g * d["v_dir"]).sum(), q1)
                return h
        else:
            stages = ("fwd_dual", "bwd_both")
            if "w1" not in d:
                d["w1"], d["w2"] = torch.ones_like(d["q"]), torch.ones_like(d["q"])
            cs = CStep(d, _mask_spec(w, d), w.scale, "both", dev)
            rec["c_abi_ms"] = _time_loop(cs.step, 3, iters)
            rec["c_abi_fwd_dual_ms"] = _time_loop(cs.fwd, 2, iters)
            user_mask = None if w.causal else mask

            def api():
                a = [d[n].detach().requires_grad_() for n in ("q", "k", "v")]
                o, to = torch.func.jvp(
                    lambda q_, k_, v_: ja.JVPAttn.fwd_dual(q_, k_, v_, attn_mask=user_mask, causal=w.causal),
                    tuple(a), (d["tq"], d["tk"], d["tv"]))
                return torch.autograd.grad((o * d["w1"]).sum() + (to * d["w2"]).sum(), a)
        rec["api_ms"] = _time_loop(api, 3, iters)
        fl = workloads.flops(w, stages)
        best = min(rec.get("c_abi_ms", rec["api_ms"]), rec["api_ms"])
        rec["flops_per_step"] = fl
        rec["tflops"] = fl / (best * 1e-3) / 1e12
        rec["frac_of_bf16_burst_peak"] = rec["tflops"] / peaks["burst"]
        rec["stages"] = "+".join(stages)
        out[name] = rec
        del d
        torch.cuda.empty_cache()
    return out


def reference_triton(w, d, spec, scale):
    """Upstream's own Triton kernels (unmodified file under baseline/_ref, default keyword arguments first) on the
    headline tensors: ms per fwd_dual call and per backward through O, next to this library's kernels for the same
    two operations.  Returns {'unavailable': why} when the file is absent or no variant runs."""
    try:
        from baseline import upstream
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"loader: {e}"}
    if not upstream.available():
        return {"unavailable": "baseline/_ref/jvp_flash_attention/jvp_attention.py is absent"}
    from jvp_flash_attention_b200 import _lib

    try:
        mod = upstream.load()
        kw, errors = upstream.pick_kwargs(mod)
        if kw is None:
            return {"unavailable": "no upstream variant compiled and ran", "errors": errors}
        q, k, v, tq, tk, tv = (d[n] for n in ("q", "k", "v", "tq", "tk", "tv"))
        wgt = d["target"]
        res = {"kwargs_used": kw or "defaults (warp_specialize=True, USE_TMA=True)", "rejected": errors,
               "fwd_dual_ms": upstream.time_fwd_dual(mod, q, k, v, tq, tk, tv, causal=w.causal, **kw),
               "bwd_o_ms": upstream.time_bwd_o(mod, q, k, v, wgt, causal=w.causal, **kw)}
        # the same two operations here, through the C ABI
        B, H, L, D = q.shape
        o, to = torch.empty_like(q), torch.empty_like(q)
        lse = torch.empty(B, H, L, device=q.device, dtype=torch.float32)
        mu = torch.empty_like(lse)
        stats = torch.empty(3, B, H, L, device=q.device, dtype=torch.float32)
        dq, dk, dv = (torch.empty_like(q) for _ in range(3))
        acc = torch.empty(q.shape, device=q.device, dtype=torch.float32)
        res["ours_fwd_dual_ms"] = _time_loop(lambda: _lib.fwd(q, k, v, tq, tk, tv, o, to, lse, mu, spec, scale), 5, 50)

        def bwd_o():
            _lib.bwd_preprocess(o, None, wgt, None, None, stats[0], stats[1], stats[2])
            _lib.bwd(q, k, v, None, None, None, wgt, None, lse, None, stats[0], stats[1], stats[2], dq, dk, dv, spec, scale,
                     dq_accum=acc)

        res["ours_bwd_o_ms"] = _time_loop(bwd_o, 5, 20)
        o_r, to_r = upstream.fwd_dual(mod, q, k, v, tq, tk, tv, causal=w.causal, **kw)
        res["max_abs_diff_o"] = (o_r.float() - o.float()).abs().max().item()
        res["max_abs_diff_to"] = (to_r.float() - to.float()).abs().max().item()
        return res
    except Exception as e:  # noqa: BLE001  (a failing comparison leg must not take the bench line with it)
        return {"unavailable": f"{type(e).__name__}: {str(e).splitlines()[0][:200] if str(e) else ''}"}


# ------------------------------------------------------------------------------------------------
# Long-sequence configuration split over the ranks (strong scaling)
# ------------------------------------------------------------------------------------------------
def c5_strong(rank, world, dev, verify_oracle_heads):
    """B32 H16 L8192 D128 bf16: the 512 (batch, head) units are split contiguously over the ranks, each rank draws
    its own heads on its GPU (seeded per head) and runs fwd_dual + backward through both outputs.  Outside the
    timed region: per-head float64 checksums of all five results are gathered over NCCL (sharding.gather_heads),
    and each rank's first head travels to rank 0, which recomputes it with the other kernel family on its own GPU
    and checks the first ``verify_oracle_heads`` of them against the float64 oracle as well."""
    import torch.distributed as dist

    from jvp_flash_attention_b200 import _lib, sharding, workloads

    name = "c5_bf16_long"
    dtype, B, H, L, D = workloads.SPECS[name][:5]
    total = B * H
    lo, hi = workloads.shard_range(total, rank, world)
    n = hi - lo
    w = workloads.make_workload_on_device(name, (lo, hi), dev)
    cs = CStep(w.tensors, _lib.MaskSpec(_lib.MASK_NONE), w.scale, "both", dev)
    for _ in range(2):
        cs.step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    steps = 3
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        cs.step()
    e.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([s.elapsed_time(e) / steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = ms.item()

    # ---- verification, not timed ----
    outs = [cs.o, cs.to, cs.dq, cs.dk, cs.dv]
    sums = torch.stack([x[0].double().sum(dim=(-1, -2)) for x in outs], dim=1)  # (n_local, 5)
    all_sums = sharding.gather_heads(sums, total)
    first = torch.stack([x[0, 0] for x in outs])  # (5, L, D): results of this rank's first head
    if world > 1:
        parts = [torch.empty_like(first) for _ in range(world)]
        dist.all_gather(parts, first)
    else:
        parts = [first]
    rec = {"heads_total": total, "heads_per_rank": n, "shape_per_rank": [1, n, L, D], "ms_per_step": ms, "steps": steps,
           "stages": "fwd_dual+bwd_both", "gathered_over": "nccl" if world > 1 else "single rank"}
    wfull = workloads.Workload(name, dtype, B, H, L, D)
    fl = workloads.flops(wfull, ("fwd_dual", "bwd_both"))
    rec["flops_per_step_total"] = fl
    rec["tflops_total"] = fl / (ms * 1e-3) / 1e12
    del cs, w
    torch.cuda.empty_cache()
    if rank == 0:
        from oracle import jvp_attention_oracle as orc

        torch.set_num_threads(max(1, os.cpu_count() or 1))
        ver = {"checksums_finite": bool(torch.isfinite(all_sums).all().item()), "checksums_shape": list(all_sums.shape),
               "heads": []}
        for r in range(world):
            bh = workloads.shard_range(total, r, world)[0]
            one = workloads.make_workload_on_device(name, (bh, bh + 1), dev).tensors
            # the same head on this GPU with the register-tiled kernel family
            g = CStep(one, _lib.MaskSpec(_lib.MASK_NONE), D**-0.5, "both", dev)
            g.fwd(_lib.IMPL_GENERIC)
            g.pre()
            g.bwd(_lib.IMPL_GENERIC, single_pass=False)
            torch.cuda.synchronize()
            mine = [g.o, g.to, g.dq, g.dk, g.dv]
            h = {"rank": r, "head": bh,
                 "max_abs_diff_vs_other_kernel_family": [float((parts[r][i].float() - mine[i][0, 0].float()).abs().max())
                                                          for i in range(5)]}
            if r < verify_oracle_heads:
                c = {k_: v_.cpu() for k_, v_ in one.items()}
                refs = orc.grads_through_both(c["q"], c["k"], c["v"], c["tq"], c["tk"], c["tv"], c["w1"], c["w2"])
                h["max_abs_err_vs_fp64_oracle"] = [orc.max_abs_err(parts[r][i][None, None].cpu(), refs[i]) for i in range(5)]
                h["max_abs_ref"] = [float(x.abs().max()) for x in refs]
            ver["heads"].append(h)
        rec["verification"] = ver
    return rec


# ------------------------------------------------------------------------------------------------
# The headline run
# ------------------------------------------------------------------------------------------------
def run_ours(args, rank, world, local):
    import torch.distributed as dist

    import jvp_flash_attention_b200.jvp_attention as ja
    from jvp_flash_attention_b200 import _lib, workloads

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this library has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    peaks = _peaks()

    w = workloads.make_workload(args.workload)
    if w.loss != "mse_tangent":
        raise SystemExit("the headline step is defined for c2_bf16_causal; the other configurations are timed as extra legs")
    # every rank owns a full-size shard of an N-times larger batch: reseed per rank
    if world > 1:
        w.seed = w.seed + 1000 * rank
        gshift = torch.Generator().manual_seed(w.seed)
        for name in ("q", "k", "v"):
            w.tensors[name] = torch.randn(w.tensors[name].shape, generator=gshift).to(w.dtype)
    host = {k_: v_.contiguous().pin_memory() for k_, v_ in w.tensors.items() if k_ in
            ("q", "k", "v", "tq", "tk", "tv", "target")}
    d = {k_: v_.to(dev) for k_, v_ in host.items()}
    B, H, L, D = w.B, w.H, w.L, w.D
    scale = w.scale
    spec = _lib.MaskSpec(_lib.MASK_CAUSAL if w.causal else _lib.MASK_NONE)
    n_el = d["q"].numel()

    # ---- device-resident step through the C ABI, all buffers preallocated ----
    cs = CStep(d, spec, scale, "gt", dev)
    loss_buf = torch.empty((), device=dev, dtype=torch.float32)
    nrm = torch.empty((), device=dev, dtype=torch.float32)
    zero_c = torch.zeros((), device=dev, dtype=torch.float32)
    side = torch.cuda.Stream(dev)
    grad_ready, loss_ready = torch.cuda.Event(), torch.cuda.Event()
    # Kernels of this library per step, counted at the calls below: forward 1, preprocess 1, backward 2 (the single
    # pass and the conversion of dQ; its accumulation buffer is cleared by a memset, not a kernel).
    own_launches = {"jvpfa_fwd": 1, "jvpfa_bwd_preprocess": 1, "jvpfa_bwd": 2}
    torch_launches = 3

    one_c = torch.ones((), device=dev, dtype=d["q"].dtype)

    def k_loss():
        # loss = mean((tO - target)^2) and its gradient w.r.t. tO; user-side torch ops.  The backward needs only the
        # gradient g = 2 (tO - target) / n, which torch's own fused kernel for this loss writes in one pass; the loss
        # value, ||g||^2 n / 4 in fp32, is reduced from it on a second stream, and the step ends (join_loss) when both
        # are done.
        torch.ops.aten.mse_loss_backward.grad_input(one_c, cs.to, d["target"], 1, grad_input=cs.gto)  # 1 = mean
        grad_ready.record()
        with torch.cuda.stream(side):
            side.wait_event(grad_ready)
            torch.linalg.vector_norm(cs.gto, dtype=torch.float32, out=nrm)
            torch.addcmul(zero_c, nrm, nrm, value=n_el / 4.0, out=loss_buf)
            loss_ready.record(side)

    def join_loss():
        torch.cuda.current_stream().wait_event(loss_ready)

    def step():
        cs.fwd()
        k_loss()
        cs.pre()
        cs.bwd()
        join_loss()

    def k_loss_alone():
        k_loss()
        join_loss()

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        for s, e in evs:
            flush.zero_()
            s.record()
            fn()
            e.record()
        barrier()
        ts = [s.elapsed_time(e) for s, e in evs]
        return sum(ts) / len(ts)

    sampler = ClockSampler(local)  # runs through warm-up and the timed region (both under load)
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    # The step's launches (seven kernels and a memset on two streams, every buffer preallocated) are captured once in a
    # CUDA graph and the timed steps replay it: the same work, without the per-launch gaps.  --no-graph times the
    # launches as they are issued; the other figure of the two is reported beside the headline.
    run_step, launch_mode = step, "eager (one launch per kernel)"
    ms_other = timed(step, max(3, min(args.steps, 50)))  # before the capture; every rank times both
    if not args.no_graph:
        try:
            cap = torch.cuda.Stream(dev)
            cap.wait_stream(torch.cuda.current_stream())
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(cap):
                with torch.cuda.graph(graph, stream=cap):
                    step()
            torch.cuda.current_stream().wait_stream(cap)
            for _ in range(3):
                graph.replay()
            run_step, launch_mode = graph.replay, "one CUDA graph of the step's launches, replayed"
        except Exception as exc:  # capture is an optimisation of the launch path only
            launch_mode = f"eager (graph capture failed: {type(exc).__name__})"
            run_step = step
    ms = timed(run_step, args.steps)
    clocks = sampler.stop()

    # ---- per-call breakdown (each launch group timed alone, L2 flushed) ----
    reps = max(3, min(args.steps, 20))
    br = {"fwd_dual": _time_call(cs.fwd, reps, flush), "loss(torch)": _time_call(k_loss_alone, reps, flush),
          "bwd_preprocess": _time_call(cs.pre, reps, flush), "bwd": _time_call(cs.bwd, reps, flush),
          "bwd_two_launch_kernels": _time_call(lambda: cs.bwd(single_pass=False), reps, flush)}
    step()  # leave dq, dk, dv complete again

    # ---- the same step back to back for seconds: clocks and power as under a long-running job ----
    sustained = None
    if args.sustain_seconds > 0:
        n_iter = max(10, int(args.sustain_seconds * 1e3 / ms))
        s2 = ClockSampler(local)
        t_ms = _time_loop(run_step, 5, n_iter)
        c2 = s2.stop()
        sustained = {"ms_per_step": t_ms, "steps": n_iter,
                     "l2": "not flushed (the step's tensors, 200+ MiB, exceed the 126 MiB L2)",
                     "sm_mhz_median": c2.get("sm_mhz"), "power_w_max": c2.get("power_w_max"), "reasons": c2.get("reasons")}

    if args.skip_e2e:
        if rank == 0:
            print(json.dumps({"note": "--skip-e2e: profiling run, no bench line", "ms_per_step": ms,
                              "breakdown_ms": br, "sustained": sustained}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end through the public API, host buffers in, loss out ----
    copy_stream = torch.cuda.Stream(dev)
    bufs = [{k_: torch.empty_like(v_, device=dev) for k_, v_ in host.items()} for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def upload(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])
            for k_, v_ in host.items():
                bufs[slot][k_].copy_(v_, non_blocking=True)
            ready[slot].record(copy_stream)

    def api_step(slot):
        torch.cuda.current_stream().wait_event(ready[slot])
        b = bufs[slot]
        a = [b[n].detach().requires_grad_() for n in ("q", "k", "v")]
        _, to_ = torch.func.jvp(lambda q_, k_, v_: ja.JVPAttn.fwd_dual(q_, k_, v_, causal=w.causal), tuple(a),
                                (b["tq"], b["tk"], b["tv"]))
        loss = ((to_.float() - b["target"].float()) ** 2).mean()
        g = torch.autograd.grad(loss, a)
        consumed[slot].record()
        return loss, g

    e2e_steps = args.steps
    for c in consumed:
        c.record()
    upload(0)
    for i in range(3):  # warm-up of the API path
        upload((i + 1) % 2)
        loss, _ = api_step(i % 2)
        loss.item()
    barrier()
    s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall = time.perf_counter()
    s0.record()
    slot = 1  # slot 1 was uploaded by the last warm-up iteration
    for i in range(e2e_steps):
        upload(1 - slot)  # next step's inputs overlap this step's kernels (counted: inside the region)
        loss, _ = api_step(slot)
        loss_host = loss.item()  # device -> host read of the step result
        slot = 1 - slot
    e0.record()
    barrier()
    e2e_ms = s0.elapsed_time(e0) / e2e_steps
    e2e_wall_ms = (time.perf_counter() - t_wall) * 1e3 / e2e_steps
    h2d = sum(v_.numel() * v_.element_size() for v_ in host.values())

    # ---- reductions over ranks ----
    fl_step = workloads.flops(w, ("fwd_dual", "bwd_to"))
    vals = torch.tensor([ms, e2e_ms, sustained["ms_per_step"] if sustained else 0.0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    ms_max, e2e_max, sus_max = vals.tolist()
    value = world * fl_step / (ms_max * 1e-3) / 1e12
    e2e_val = world * fl_step / (e2e_max * 1e-3) / 1e12

    # ---- extra legs ----
    del bufs
    torch.cuda.empty_cache()
    strong = extras = triton = None
    if not args.no_extras:
        strong = c5_strong(rank, world, dev, args.verify_oracle_heads)
        if rank == 0 and world == 1:
            extras = other_workloads(dev, peaks)
            triton = reference_triton(w, d, spec, scale)

    if rank == 0:
        stage_flops = {"fwd_dual": workloads.flops(w, ("fwd_dual",)), "bwd": workloads.flops(w, ("bwd_to",))}
        dom = max(("fwd_dual", "bwd"), key=lambda n: br[n])
        ach = stage_flops[dom] / (br[dom] * 1e-3) / 1e12
        n_pairs = w.attended_pairs()
        mma = 2.0 * D * n_pairs  # flops of one L x L x D product over the attended pairs
        pre_bytes = 3 * n_el * 2 + 4 * B * H * L * 4
        kernels = [
            {"name": "fwd_tc5_pair64_kernel (fwd_dual)", "ms": br["fwd_dual"], "mma_executed": 6, "mma_algorithmic": 6},
            {"name": "bwd_tc5_fused64_kernel + dq_convert_kernel (dQ, dK, dV in one pass)", "ms": br["bwd"],
             "mma_executed": 10, "mma_algorithmic": 10},
            {"name": "bwd_tc5_d64_kernel x2 (two-launch backward; not part of the step)", "ms": br["bwd_two_launch_kernels"],
             "mma_executed": 15, "mma_algorithmic": 10},
            {"name": "pre_kernel (HBM bound)", "ms": br["bwd_preprocess"],
             "gbs": pre_bytes / (br["bwd_preprocess"] * 1e-3) / 1e9,
             "frac_of_hbm_peak": pre_bytes / (br["bwd_preprocess"] * 1e-3) / 1e9 / peaks["hbm"]},
        ]
        for kk in kernels[:3]:
            kk["tflops_executed"] = kk["mma_executed"] * mma / (kk["ms"] * 1e-3) / 1e12
            kk["frac_of_burst_peak"] = kk["tflops_executed"] / peaks["burst"]
        traffic, traffic_src = None, None
        if TRAFFIC_FILE.exists():
            t = json.loads(TRAFFIC_FILE.read_text())
            if t.get("workload") == args.workload and dom in t.get("dram_bytes_per_call", {}):
                traffic = t["dram_bytes_per_call"][dom]
                traffic_src = {"commit": t.get("commit"), "captured": t.get("captured"),
                               "kernels": t.get("kernels", {}).get(dom)}
        config = {"workload": args.workload, "B_per_gpu": B, "H": H, "L": L, "D": D, "causal": w.causal,
                  "global_batch": B * world, "sharding": f"(batch x head) shards, {world} rank(s), no collective",
                  "l2": "flushed between steps (256 MiB memset outside the per-step event pairs)",
                  "launch": launch_mode, "ms_per_step_launched_one_by_one": ms_other,
                  "flops_per_step_per_gpu": fl_step, "flop_model": "2*D*pairs*(6 fwd_dual + 10 bwd via tO)",
                  "pct_of_nominal_bf16_peak_2250": 100 * value / world / 2250.0,
                  "pct_of_measured_burst": 100 * value / world / peaks["burst"]}
        if sustained:
            tf_s = fl_step / (sus_max * 1e-3) / 1e12
            sustained = dict(sustained, ms_per_step_max_over_ranks=sus_max, tflops_per_gpu=tf_s,
                             pct_of_measured_sustained=100 * tf_s / peaks["sustained"])
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_max, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config,
            "clocks": clocks,
            "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e_max, "wall_ms_per_step": e2e_wall_ms,
                    "path": "torch.func.jvp(JVPAttn.fwd_dual) + autograd.grad; pinned host inputs, double-buffered H2D"},
            "gpu_launches": sum(own_launches.values()) * args.steps,
            "launches_per_step": {"library_kernels": own_launches, "torch_kernels_of_the_loss": torch_launches,
                                  "memsets": 1},
            "roofline": {"bound": "tensor",
                         "kernel": "jvpfa_fwd (fwd_tc5_pair64_kernel)" if dom == "fwd_dual" else
                         "jvpfa_bwd (bwd_tc5_fused64_kernel + dq_convert_kernel, timed as one call; 10 algorithmic "
                         "MMAs, 10 executed)",
                         "achieved": ach, "peak": peaks["burst"],
                         "unit": "TFLOP/s", "frac": ach / peaks["burst"],
                         "traffic": traffic, "traffic_source": traffic_src,
                         "peak_source": f"{peaks['src']} bf16 burst (kernel timed alone)",
                         "ms_per_launch": br[dom], "algorithmic_flops_per_launch": stage_flops[dom]},
            "breakdown_ms": br,
            "kernels": kernels,
            "sustained": sustained,
            "last_loss": loss_host,
        }
        if strong is not None:
            line["c5_strong"] = strong
        if extras is not None:
            line["other_workloads"] = extras
        if triton is not None:
            line["reference_triton"] = triton
        if world == 1 and not args.no_cpu_baseline:
            torch.set_num_threads(max(1, os.cpu_count() or 1))
            tf, sec, sample = _cpu_reference(args.workload, 3, 1)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": sample, "s_per_sample_step": sec}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--skip-e2e", action="store_true", help="stop after the device-resident part (profiling runs)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time the step's launches as issued, not a graph replay")
    ap.add_argument("--no-extras", action="store_true", help="skip the other configurations, the Triton leg and the C5 split")
    ap.add_argument("--sustain-seconds", type=float, default=3.0)
    ap.add_argument("--verify-oracle-heads", type=int, default=1,
                    help="how many ranks' sampled heads of the C5 split rank 0 checks against the float64 oracle")
    args = ap.parse_args()
    rank, world, local = _dist_env()
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local)


if __name__ == "__main__":
    main()
