"""Accuracy / speed harness over the reference's own grid, with its table layout.

The reference ships no pytest tests; it ships a script (tests/test_jvp_attention.py) that walks
sequence length x mask type x causal, compares `JVPAttn.fwd_dual` with SDPA-MATH in the working
dtype on the same GPU (forward-mode route and torch.func.jvp route; primal, tangent, loss, dq, dk,
dv) and times the fused forward against SDPA-MATH (test_jvp_attention.py:670-975; grid 211, 698-720;
shapes 225-227, 291; seeds 290-304, 331-340; tolerances 688-693; flop convention 49-83).  This
script does the same for this library so that the two sets of tables can be put side by side:

    python tests/harness.py --dtype bfloat16 [--json out.json] [--max-len 2048] [--fp32-precision tf32]

Same grid (L in 32..2048, mask in none/boolean/additive, causal on/off, causal+mask skipped: 28
cases), same shapes (B=2, 12 heads, D=64), same seeds and mask density (90 % masked, additive mask
in {0, -100}), same tolerances, same flop formula.  Differences, all deliberate: the timed closure
is also reported without the six clones and three make_dual calls that the reference times
(test_jvp_attention.py:772-779); a float mask is an additive bias as in SDPA; the loss also has a
term on the tangent output, whose gradient the reference cannot form.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

import torch
import torch.autograd.forward_ad as fwAD
import torch.nn.functional as F
from torch.nn.attention import SDPBackend, sdpa_kernel

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from jvp_flash_attention_b200.jvp_attention import JVPAttn, set_fp32_precision  # noqa: E402

MASK_CONST = -100.0
TOL = {torch.float16: 4e-3, torch.float32: 2.35e-2, torch.bfloat16: 3.2e-2}
SEQ_LENS = (32, 64, 128, 256, 512, 1024, 2048)


def reference_flops(B, H, L, D, causal):
    """The reference's convention: 2 * (4 B H L^2 D + 5 B H L^2), halved for causal."""
    f = 2.0 * (4.0 * B * H * L * L * D + 5.0 * B * H * L * L)
    return f / 2 if causal else f


def make_case(L, mask_type, dtype, dev, B=2, H=12, D=64):
    g = torch.Generator(device=dev).manual_seed(42)
    ts = [torch.randn(B, H, L, D, device=dev, dtype=dtype, generator=g) for _ in range(7)]
    q, tq, k, tk, v, tv, target = ts
    mask = None
    if mask_type != "none":
        gm = torch.Generator(device=dev).manual_seed(1042)
        keep = torch.rand(B, H, L, L, device=dev, generator=gm) > 0.9
        dead = ~keep.any(dim=-1, keepdim=True)  # a fully masked row gets 10 % of its keys back
        keep = keep | (dead & (torch.rand(B, H, L, L, device=dev, generator=gm) < 0.1))
        keep[..., 0] |= ~keep.any(dim=-1)
        mask = keep if mask_type == "boolean" else torch.where(keep, 0.0, MASK_CONST).to(dtype)
    return q, k, v, tq, tk, tv, target, mask


def sdpa_dual(q, k, v, tq, tk, tv, mask, causal):
    with sdpa_kernel(SDPBackend.MATH), fwAD.dual_level():
        out = F.scaled_dot_product_attention(fwAD.make_dual(q, tq), fwAD.make_dual(k, tk), fwAD.make_dual(v, tv),
                                             attn_mask=mask, is_causal=causal)
        p, t = fwAD.unpack_dual(out)
        return p, t


def ours_fwad(q, k, v, tq, tk, tv, mask, causal):
    with fwAD.dual_level():
        out = JVPAttn.fwd_dual(fwAD.make_dual(q, tq), fwAD.make_dual(k, tk), fwAD.make_dual(v, tv), attn_mask=mask,
                               causal=causal)
        p, t = fwAD.unpack_dual(out)
        return p, t


def ours_func(q, k, v, tq, tk, tv, mask, causal):
    return torch.func.jvp(lambda a, b, c: JVPAttn.fwd_dual(a, b, c, attn_mask=mask, causal=causal), (q, k, v), (tq, tk, tv))


def grads(fn, q, k, v, tq, tk, tv, target, mask, causal):
    a = [x.detach().clone().requires_grad_() for x in (q, k, v)]
    p, t = fn(*a, tq, tk, tv, mask, causal)
    loss = F.mse_loss(p.float(), target.float())
    g = torch.autograd.grad(loss, a)
    return p.detach(), t.detach(), loss.detach(), g


def timed(fn, iters=100, warmup=10):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(iters):
        fn()
    torch.cuda.synchronize()
    return (time.perf_counter() - t0) / iters * 1e3


def run(dtype, max_len, bench=True, min_len=0, masks=("none", "boolean", "additive")):
    dev = torch.device("cuda", 0)
    rows = []
    for L in [s for s in SEQ_LENS if min_len <= s <= max_len]:
        for mask_type in masks:
            for causal in (False, True):
                if causal and mask_type != "none":
                    continue
                q, k, v, tq, tk, tv, target, mask = make_case(L, mask_type, dtype, dev)
                rp, rt, rl, rg = grads(sdpa_dual, q, k, v, tq, tk, tv, target, mask, causal)
                err = {}
                for name, fn in (("fwad", ours_fwad), ("func", ours_func)):
                    p, t, l, g_ = grads(fn, q, k, v, tq, tk, tv, target, mask, causal)
                    e = {"primal": (p.float() - rp.float()).abs().max().item(),
                         "tangent": (t.float() - rt.float()).abs().max().item(),
                         "loss": (l - rl).abs().item(),
                         "dq": (g_[0].float() - rg[0].float()).abs().max().item(),
                         "dk": (g_[1].float() - rg[1].float()).abs().max().item(),
                         "dv": (g_[2].float() - rg[2].float()).abs().max().item()}
                    err[name] = e
                worst = max(max(e["primal"], e["tangent"]) for e in err.values())
                row = {"seq_len": L, "mask": mask_type, "causal": causal, "errors": err, "max_error": worst,
                       "tolerance": TOL[dtype], "pass": worst < TOL[dtype]}
                if bench:
                    ms_sdpa = timed(lambda: sdpa_dual(q, k, v, tq, tk, tv, mask, causal), iters=20, warmup=3)
                    ms_clone = timed(lambda: ours_fwad(q.clone(), k.clone(), v.clone(), tq.clone(), tk.clone(), tv.clone(),
                                                       mask, causal))
                    ms = timed(lambda: ours_fwad(q, k, v, tq, tk, tv, mask, causal))
                    fl = reference_flops(2, 12, L, 64, causal)
                    row.update({"sdpa_math_ms": ms_sdpa, "ms_with_clones": ms_clone, "ms": ms,
                                "tflops_reference_convention": fl / ms / 1e9,
                                "tflops_reference_convention_with_clones": fl / ms_clone / 1e9})
                rows.append(row)
                print(fmt(row), flush=True)
    return rows


def fmt(r):
    s = (f"L={r['seq_len']:5d} causal={str(r['causal']):5s} mask={r['mask']:8s} "
         f"max err {r['max_error']:.2e} (tol {r['tolerance']:.1e}) {'ok  ' if r['pass'] else 'FAIL'}")
    e = r["errors"]["func"]
    s += f" | loss {e['loss']:.1e} dq {e['dq']:.1e} dk {e['dk']:.1e} dv {e['dv']:.1e}"
    if "ms" in r:
        s += (f" | sdpa-math {r['sdpa_math_ms']:8.3f} ms, fwd_dual {r['ms']:.3f} ms ({r['ms_with_clones']:.3f} with clones), "
              f"{r['tflops_reference_convention']:.1f} TFLOP/s (reference convention)")
    return s


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dtype", default="bfloat16", choices=["float16", "bfloat16", "float32"])
    ap.add_argument("--max-len", type=int, default=2048)
    ap.add_argument("--min-len", type=int, default=0)
    ap.add_argument("--masks", default="none,boolean,additive", help="comma-separated subset of the grid's mask types")
    ap.add_argument("--no-benchmark-performance", action="store_true")
    ap.add_argument("--json", default=None)
    ap.add_argument("--fp32-precision", default="3xtf32", choices=["3xtf32", "tf32"],
                    help="float32 only: products as three TF32 MMAs (default) or as one, which is what the reference computes")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("the harness needs a CUDA device: this library has no CPU path")
    set_fp32_precision(args.fp32_precision)
    rows = run(getattr(torch, args.dtype), args.max_len, bench=not args.no_benchmark_performance, min_len=args.min_len,
               masks=tuple(args.masks.split(",")))
    n_ok = sum(r["pass"] for r in rows)
    print(f"{n_ok} of {len(rows)} cases within the reference's tolerance for {args.dtype}")
    if args.json:
        Path(args.json).write_text(json.dumps({"dtype": args.dtype, "fp32_precision": args.fp32_precision, "rows": rows}, indent=1))


if __name__ == "__main__":
    main()
