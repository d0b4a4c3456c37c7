"""Benchmark of the JVP flash-attention hot path (fused forward-dual + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (default ``c2_bf16_causal``): bf16 causal self-attention B=4, H=16, L=2048, D=64, q,k,v ~
N(0,1), tangents ~ N(0,0.1^2), target ~ N(0,1), seeded synthetic data; one step = fwd_dual
(primal + tangent) followed by the backward of loss = mean((tO - target)^2) to q, k, v.
With N ranks every rank runs the whole configuration on its own (batch x head) shard of a batch
N times larger (no collective on the data path; weak scaling), and ``value`` sums all ranks.

One JSON line is printed by rank 0.  ``value`` is device-resident throughput through the C ABI
(CUDA events per step, max over ranks, L2 flushed between steps); ``e2e`` is the same step through
the public Python API with pinned host inputs copied in and the loss read back every step.
``--impl reference`` times upstream's CPU path (torch.func.jvp over SDPA-MATH + autograd) on the
host cores on a bounded sample of the same workload.
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
# DRAM bytes (read + write) per C-ABI call on the default workload, from one ncu --set full capture of each kernel
# (profiles/tc5_kernels_c2_bf16_causal.md): forward 147.8 + 15.7 MB; backward = own-keys launch 123.1 + 12.7 MB
# plus own-queries launch 148.4 + 10.1 MB.
NCU_DRAM_BYTES = {"fwd_dual": 163.5e6, "bwd": 294.3e6}


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm=d["hbm_gbs"], burst=d["bf16_tflops"], sustained=d["bf16_tflops_sustained"], src="measured")
    return dict(hbm=6650.0, burst=1590.0, sustained=1400.0, src="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
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
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def _dist_init(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


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
    steps = max(1, min(args.steps, 3))
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
    o, to = torch.empty_like(d["q"]), torch.empty_like(d["q"])
    lse = torch.empty(B, H, L, device=dev, dtype=torch.float32)
    mu = torch.empty_like(lse)
    stats = torch.empty(3, B, H, L, device=dev, dtype=torch.float32)
    dq, dk, dv = (torch.empty_like(d["q"]) for _ in range(3))
    gto = torch.empty_like(d["q"])
    loss_buf = torch.empty((), device=dev, dtype=torch.float32)

    def k_fwd():
        _lib.fwd(d["q"], d["k"], d["v"], d["tq"], d["tk"], d["tv"], o, to, lse, mu, spec, scale)

    diff = torch.empty_like(d["q"])

    nrm = torch.empty((), device=dev, dtype=torch.float32)
    zero_c = torch.zeros((), device=dev, dtype=torch.float32)

    side = torch.cuda.Stream(dev)
    diff_ready, loss_ready = torch.cuda.Event(), torch.cuda.Event()

    def k_loss():
        # loss = mean((tO - target)^2) and its gradient w.r.t. tO; user-side torch ops, kept in
        # the compute dtype so that they stay a small part of the step (four launches).  The backward
        # needs only the gradient: the loss value is reduced on a second stream next to it, and the
        # step ends (join_loss) when both are done.
        torch.sub(to, d["target"], out=diff)
        diff_ready.record()
        with torch.cuda.stream(side):
            side.wait_event(diff_ready)
            torch.linalg.vector_norm(diff, dtype=torch.float32, out=nrm)
            torch.addcmul(zero_c, nrm, nrm, value=1.0 / n_el, out=loss_buf)  # ||diff||^2 / n
            loss_ready.record(side)
        torch.mul(diff, 2.0 / n_el, out=gto)

    def join_loss():
        torch.cuda.current_stream().wait_event(loss_ready)

    def k_pre():
        _lib.bwd_preprocess(o, to, None, gto, mu, stats[0], stats[1], stats[2])

    def k_bwd():
        _lib.bwd(d["q"], d["k"], d["v"], d["tq"], d["tk"], d["tv"], None, gto, lse, mu, stats[0], stats[1], stats[2],
                 dq, dk, dv, spec, scale)

    def step():
        k_fwd()
        k_loss()
        k_pre()
        k_bwd()
        join_loss()

    def k_loss_alone():
        k_loss()
        join_loss()

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)  # runs through warm-up and the timed region (both under load)
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for s, e in evs:
        flush.zero_()
        s.record()
        step()
        e.record()
    barrier()
    clocks = sampler.stop()
    ms_list = [s.elapsed_time(e) for s, e in evs]
    ms = sum(ms_list) / len(ms_list)

    # ---- per-call breakdown (each launch group timed alone, L2 flushed) ----
    def time_call(fn, reps):
        ts = []
        for _ in range(reps):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        return sum(ts) / len(ts)

    def k_bwd_only(flag):
        def f():
            _lib.bwd(d["q"], d["k"], d["v"], d["tq"], d["tk"], d["tv"], None, gto, lse, mu, stats[0], stats[1],
                     stats[2], dq, dk, dv, spec, scale, _lib.IMPL_AUTO | flag)
        return f

    reps = max(3, min(args.steps, 20))
    br = {"fwd_dual": time_call(k_fwd, reps), "loss(torch)": time_call(k_loss_alone, reps),
          "bwd_preprocess": time_call(k_pre, reps), "bwd": time_call(k_bwd, reps),
          "bwd_dkdv_only": time_call(k_bwd_only(_lib.IMPL_ONLY_DKDV), reps),
          "bwd_dq_only": time_call(k_bwd_only(_lib.IMPL_ONLY_DQ), reps)}
    step()  # leave dq, dk, dv complete again

    # ---- end to end through the public API, host buffers in, loss out ----
    if args.skip_e2e:
        if rank == 0:
            print(json.dumps({"note": "--skip-e2e: profiling run, no bench line", "ms_per_step": ms,
                              "breakdown_ms": br}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
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
    vals = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    ms_max, e2e_max = vals.tolist()
    value = world * fl_step / (ms_max * 1e-3) / 1e12
    e2e_val = world * fl_step / (e2e_max * 1e-3) / 1e12

    if rank == 0:
        stage_flops = {"fwd_dual": workloads.flops(w, ("fwd_dual",)), "bwd": workloads.flops(w, ("bwd_to",))}
        dom = max(("fwd_dual", "bwd"), key=lambda n: br[n])
        ach = stage_flops[dom] / (br[dom] * 1e-3) / 1e12
        n_pairs = w.attended_pairs()
        mma = 2.0 * D * n_pairs  # flops of one L x L x D product over the attended pairs
        kernels = [
            {"name": "fwd_tc5_pair64_kernel (fwd_dual)", "ms": br["fwd_dual"], "mma_executed": 6, "mma_algorithmic": 6},
            {"name": "bwd_tc5_d64_kernel<own keys> (dK,dV)", "ms": br["bwd_dkdv_only"], "mma_executed": 8,
             "mma_algorithmic": None},
            {"name": "bwd_tc5_d64_kernel<own queries> (dQ)", "ms": br["bwd_dq_only"], "mma_executed": 7,
             "mma_algorithmic": None},
            {"name": "pre_kernel (HBM bound)", "ms": br["bwd_preprocess"],
             "gbs": (3 * n_el * 2 + 4 * B * H * L * 4) / (br["bwd_preprocess"] * 1e-3) / 1e9,
             "frac_of_hbm_peak": (3 * n_el * 2 + 4 * B * H * L * 4) / (br["bwd_preprocess"] * 1e-3) / 1e9 / peaks["hbm"]},
        ]
        for kk in kernels[:3]:
            kk["tflops_executed"] = kk["mma_executed"] * mma / (kk["ms"] * 1e-3) / 1e12
            kk["frac_of_burst_peak"] = kk["tflops_executed"] / peaks["burst"]
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_max, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "B_per_gpu": B, "H": H, "L": L, "D": D, "causal": w.causal,
                       "global_batch": B * world, "sharding": f"(batch x head) shards, {world} rank(s), no collective",
                       "l2": "flushed between steps (256 MiB memset outside the per-step event pairs)",
                       "flops_per_step_per_gpu": fl_step, "flop_model": "2*D*pairs*(6 fwd_dual + 10 bwd via tO)",
                       "pct_of_nominal_bf16_peak_2250": 100 * value / world / 2250.0,
                       "pct_of_measured_sustained": 100 * value / world / peaks["sustained"]},
            "clocks": clocks,
            "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e_max, "wall_ms_per_step": e2e_wall_ms,
                    "path": "torch.func.jvp(JVPAttn.fwd_dual) + autograd.grad; pinned host inputs, double-buffered H2D"},
            "gpu_launches": 4 * args.steps,
            "roofline": {"bound": "tensor",
                         "kernel": "jvpfa_fwd (fwd_tc5_pair64_kernel)" if dom == "fwd_dual" else
                         "jvpfa_bwd (bwd_tc5_d64_kernel own-keys + own-queries launches, timed as one call; "
                         "10 algorithmic MMAs, 15 executed because both launches recompute the score tiles)",
                         "achieved": ach, "peak": peaks["burst"],
                         "unit": "TFLOP/s", "frac": ach / peaks["burst"],
                         # dram__bytes_read.sum + dram__bytes_write.sum per call from the committed ncu capture of
                         # this same workload (profiles/tc5_kernels_c2_bf16_causal.md); algorithmic minimum 138 MB
                         "traffic": (NCU_DRAM_BYTES[dom] if args.workload == DEFAULT_WORKLOAD else None),
                         "peak_source": f"{peaks['src']} bf16 burst (kernel timed alone)",
                         "ms_per_launch": br[dom], "algorithmic_flops_per_launch": stage_flops[dom]},
            "breakdown_ms": br,
            "kernels": kernels,
            "last_loss": loss_host,
        }
        if world == 1 and not args.no_cpu_baseline:
            tf, sec, sample = _cpu_reference(args.workload, 1, 1)
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
    args = ap.parse_args()
    rank, world, local = _dist_init(args.gpus)
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local)


if __name__ == "__main__":
    main()
