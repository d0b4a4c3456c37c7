"""Loader and timing helpers for upstream's own Triton kernels, run unmodified on the same GPU.

The upstream source file (jvp_flash_attention/jvp_attention.py of amorehead/jvp_flash_attention)
is expected under ``baseline/_ref/jvp_flash_attention/`` -- a folder that is kept out of version
control.  It is imported by path under an alias, so it never shadows this repository's own
``jvp_flash_attention`` drop-in package.  Nothing in the product imports this module: only the
GPU parity tests and the benchmark's comparison leg do.

Upstream's public keyword arguments ``warp_specialize`` and ``USE_TMA`` (jvp_attention.py:2322-2324)
select its code path; ``pick_kwargs`` tries the defaults first and records which combination the
installed Triton could compile for this GPU.
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import torch
import torch.autograd.forward_ad as fwAD

REF_FILE = Path(__file__).resolve().parent / "_ref" / "jvp_flash_attention" / "jvp_attention.py"
_ALIAS = "_upstream_jvp_attention"

KWARG_CANDIDATES = (
    {},  # upstream defaults: warp_specialize=True, USE_TMA=True
    {"warp_specialize": False},
    {"warp_specialize": False, "USE_TMA": False},
)


def available() -> bool:
    return REF_FILE.exists()


def load():
    """Imports upstream's module from baseline/_ref under an alias; raises FileNotFoundError when absent."""
    if _ALIAS in sys.modules:
        return sys.modules[_ALIAS]
    if not REF_FILE.exists():
        raise FileNotFoundError(f"{REF_FILE} is missing: upstream's kernels cannot be run")
    spec = importlib.util.spec_from_file_location(_ALIAS, REF_FILE)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[_ALIAS] = mod
    spec.loader.exec_module(mod)
    return mod


def fwd_dual(mod, q, k, v, tq, tk, tv, attn_mask=None, causal=False, **kw):
    """(O, tO) from upstream's JVPAttn.fwd_dual on dual tensors, as its harness calls it
    (tests/test_jvp_attention.py:572-574)."""
    with fwAD.dual_level():
        dq, dk, dv = (fwAD.make_dual(x, t) for x, t in ((q, tq), (k, tk), (v, tv)))
        out = mod.JVPAttn.fwd_dual(dq, dk, dv, attn_mask=attn_mask, causal=causal, **kw)
        o, to = fwAD.unpack_dual(out)
        return o.detach().clone(), to.detach().clone()


def grads_through_o(mod, q, k, v, w, attn_mask=None, causal=False, **kw):
    """(O, dq, dk, dv) for the loss sum(O * w): upstream differentiates through O only (jvp_attention.py:2831)."""
    a = [x.detach().clone().requires_grad_() for x in (q, k, v)]
    o = mod.JVPAttn.fwd(a[0], a[1], a[2], attn_mask=attn_mask, causal=causal, **kw)
    g = torch.autograd.grad((o.float() * w.float()).sum(), a)
    return o.detach(), g[0], g[1], g[2]


def pick_kwargs(mod, dtype=torch.bfloat16, device="cuda"):
    """First of KWARG_CANDIDATES with which a small fwd_dual + backward compiles and runs; None if none does.
    Returns (kwargs, errors) where errors lists why earlier candidates were rejected."""
    g = torch.Generator().manual_seed(0)
    x = [torch.randn(1, 2, 128, 64, generator=g).to(dtype).to(device) for _ in range(7)]
    errors = []
    for kw in KWARG_CANDIDATES:
        try:
            fwd_dual(mod, *x[:6], causal=True, **kw)
            grads_through_o(mod, x[0], x[1], x[2], x[6], causal=True, **kw)
            torch.cuda.synchronize()
            return dict(kw), errors
        except Exception as e:  # compile or launch failure of this variant: try the next one
            errors.append(f"{kw or 'defaults'}: {type(e).__name__}: {str(e).splitlines()[0][:200] if str(e) else ''}")
    return None, errors


def _time(fn, warmup: int, iters: int) -> float:
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


def time_fwd_dual(mod, q, k, v, tq, tk, tv, attn_mask=None, causal=False, warmup=10, iters=50, **kw) -> float:
    """ms per upstream fwd_dual call on prebuilt tensors (CUDA events; upstream's own closure,
    tests/test_jvp_attention.py:770-780, additionally clones six tensors per call)."""
    def run():
        with fwAD.dual_level():
            dq, dk, dv = (fwAD.make_dual(x, t) for x, t in ((q, tq), (k, tk), (v, tv)))
            mod.JVPAttn.fwd_dual(dq, dk, dv, attn_mask=attn_mask, causal=causal, **kw)

    return _time(run, warmup, iters)


def time_bwd_o(mod, q, k, v, w, attn_mask=None, causal=False, warmup=5, iters=20, **kw) -> float:
    """ms per upstream backward through O (the forward that builds the graph is outside the timed part)."""
    a = [x.detach().clone().requires_grad_() for x in (q, k, v)]
    o = mod.JVPAttn.fwd(a[0], a[1], a[2], attn_mask=attn_mask, causal=causal, **kw)
    go = w.to(o.dtype)

    def run():
        torch.autograd.grad(o, a, go, retain_graph=True)

    return _time(run, warmup, iters)
