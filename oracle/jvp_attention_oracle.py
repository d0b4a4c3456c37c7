"""CPU oracle for the JVP flash-attention path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package may import this file: it is the checker used by ``tests/``, by
``__graft_entry__.smoke()`` and by ``bench.py``'s CPU-baseline / reference legs.

Two independent statements of the same mathematics live here:

1. ``sdpa_jvp`` -- the ground truth the upstream harness itself uses
   (tests/test_jvp_attention.py:548-561): ``torch.func.jvp`` through
   ``F.scaled_dot_product_attention`` under ``SDPBackend.MATH``.  Run in float64 it also provides
   gradients through both outputs and double backward, by plain autograd.
2. ``tiled_forward`` / ``closed_form_backward`` -- a NumPy float64 restatement of upstream's
   *algorithm*: the tile loop with base-2 online softmax, running (m, l, mu) and the tangent
   epilogue of ``_attn_fwd_inner`` (jvp_flash_attention/jvp_attention.py:125-336, 1011-1033), and
   the recompute-from-logsumexp backward of ``_attn_bwd_dkdv`` / ``_attn_bwd_dq``
   (jvp_attention.py:1415-1707) extended with the cotangent of the tangent output.

Pinning: ``tests/golden/*.npz`` hold outputs of upstream's own kernels executed in this build's
container with ``TRITON_INTERPRET=1`` (generator: ``tests/golden/make_golden.py``);
``tests/test_oracle.py`` checks both statements against those files and against each other.
Gradients through the tangent output, Hessian-vector products and general (non {0,-100})
additive bias cannot be produced by upstream at all, so for those the parity is unpinned
against upstream and rests on statement 1.
"""
from __future__ import annotations

import math
from functools import partial

import numpy as np
import torch
import torch.nn.functional as F
from torch.nn.attention import SDPBackend, sdpa_kernel

LOG2E = 1.4426950408889634


# ---------------------------------------------------------------------------------------------
# Statement 1: torch.func.jvp over SDPA-MATH
# ---------------------------------------------------------------------------------------------
def _sdpa(q, k, v, attn_mask=None, causal=False, scale=None):
    with sdpa_kernel(SDPBackend.MATH):
        return F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask, is_causal=causal, scale=scale)


def sdpa_jvp(q, k, v, tq, tk, tv, attn_mask=None, causal=False, scale=None, dtype=torch.float64):
    """(O, tO) by ``torch.func.jvp`` over SDPA-MATH, computed in ``dtype`` on CPU.

    Inputs that require grad keep their graph, so the caller can differentiate O and tO.
    Rows without any attendable key are returned as zeros, the convention of upstream's kernel
    (jvp_attention.py:1011-1022); SDPA itself would give NaN there.
    """
    cast = lambda x: x if x is None else x.to("cpu", dtype)  # noqa: E731
    q, k, v, tq, tk, tv = (cast(x) for x in (q, k, v, tq, tk, tv))
    m = attn_mask
    if m is not None:
        m = m.cpu()
        if m.dtype != torch.bool:
            m = m.to(dtype)
    dead = None
    if m is not None and m.dtype == torch.bool:
        dead = ~m.any(dim=-1, keepdim=True)
        if bool(dead.any()):
            m = m | dead  # let SDPA see finite rows there; the rows are zeroed below (keeps gradients finite)
        else:
            dead = None
    o, to = torch.func.jvp(partial(_sdpa, attn_mask=m, causal=causal, scale=scale), (q, k, v), (tq, tk, tv))
    if dead is not None:
        dead = dead.expand(*o.shape[:-1], 1)
        o = torch.where(dead, torch.zeros_like(o), o)
        to = torch.where(dead, torch.zeros_like(to), to)
    return o, to


def sdpa_primal(q, k, v, attn_mask=None, causal=False, scale=None, dtype=torch.float64):
    q, k, v = (x.to("cpu", dtype) for x in (q, k, v))
    m = attn_mask
    if m is not None:
        m = m.cpu()
        if m.dtype != torch.bool:
            m = m.to(dtype)
    return _sdpa(q, k, v, m, causal, scale)


def grads_through_both(q, k, v, tq, tk, tv, go, gto, attn_mask=None, causal=False, scale=None):
    """fp64 (O, tO, dq, dk, dv) of <go, O> + <gto, tO>; go or gto may be None."""
    a = [x.detach().to("cpu", torch.float64).requires_grad_() for x in (q, k, v)]
    o, to = sdpa_jvp(*a, tq, tk, tv, attn_mask, causal, scale)
    loss = 0.0
    if go is not None:
        loss = loss + (o * go.to("cpu", torch.float64)).sum()
    if gto is not None:
        loss = loss + (to * gto.to("cpu", torch.float64)).sum()
    g = torch.autograd.grad(loss, a)
    return o.detach(), to.detach(), g[0], g[1], g[2]


def hvp_q(q, k, v, w, v_dir, attn_mask=None, causal=False, scale=None):
    """fp64 Hessian-vector product  d/dq < d/dq sum(O*w), v_dir >  by double backward."""
    q1 = q.detach().to("cpu", torch.float64).requires_grad_()
    o = sdpa_primal(q1, k, v, attn_mask, causal, scale)
    (g1,) = torch.autograd.grad((o * w.to("cpu", torch.float64)).sum(), q1, create_graph=True)
    (h,) = torch.autograd.grad((g1 * v_dir.to("cpu", torch.float64)).sum(), q1)
    return o.detach(), g1.detach(), h


# ---------------------------------------------------------------------------------------------
# Statement 2: NumPy restatement of the tiled algorithm
# ---------------------------------------------------------------------------------------------
def _dense_mask_bias(B, H, L, attn_mask, causal):
    """Boolean 'attend' array and additive bias array, both (B, H, L, L) float64/bool."""
    allow = np.ones((B, H, L, L), dtype=bool)
    bias = np.zeros((B, H, L, L), dtype=np.float64)
    if causal:
        allow &= np.tril(np.ones((L, L), dtype=bool))[None, None]
    if attn_mask is not None:
        m = attn_mask.detach().cpu()
        if m.dtype == torch.bool:
            allow &= np.broadcast_to(m.numpy(), (B, H, L, L))
        else:
            bias = bias + np.broadcast_to(m.to(torch.float64).numpy(), (B, H, L, L))
    return allow, bias


def tiled_forward(q, k, v, tq=None, tk=None, tv=None, attn_mask=None, causal=False, scale=None, block=32):
    """Tile-loop forward in float64, following upstream's kernel step by step.

    Per query tile it walks the key tiles and keeps the running maximum ``m`` (base-2 domain),
    denominator ``l``, ``mu = sum P*tS`` and two accumulators that are rescaled by
    ``alpha = 2^(m_old - m_new)`` each step (jvp_attention.py:262-322); the epilogue forms
    ``tO = acc_t/l - (mu/l) O`` and the base-2 logsumexp ``M = m + log2 l``
    (jvp_attention.py:1011-1033).  Bias is added after scaling (SDPA semantics).
    Returns dict(o, to, lse, mu) of NumPy arrays (to / mu are None without tangents).
    """
    f = lambda x: None if x is None else x.detach().cpu().to(torch.float64).numpy()  # noqa: E731
    q, k, v, tq, tk, tv = (f(x) for x in (q, k, v, tq, tk, tv))
    B, H, L, D = q.shape
    scale = D**-0.5 if scale is None else scale
    allow, bias = _dense_mask_bias(B, H, L, attn_mask, causal)
    dual = tq is not None
    o = np.zeros_like(q)
    to = np.zeros_like(q) if dual else None
    lse = np.zeros((B, H, L))
    mu_out = np.zeros((B, H, L)) if dual else None
    for m0 in range(0, L, block):
        m1 = min(L, m0 + block)
        qi = q[:, :, m0:m1]
        m_run = np.full((B, H, m1 - m0), -np.inf)
        l_run = np.zeros((B, H, m1 - m0))
        mu_run = np.zeros((B, H, m1 - m0))
        acc_o = np.zeros((B, H, m1 - m0, D))
        acc_t = np.zeros((B, H, m1 - m0, D))
        for n0 in range(0, L, block):
            n1 = min(L, n0 + block)
            kj, vj = k[:, :, n0:n1], v[:, :, n0:n1]
            a = allow[:, :, m0:m1, n0:n1]
            x = (qi @ kj.transpose(0, 1, 3, 2)) * (scale * LOG2E) + bias[:, :, m0:m1, n0:n1] * LOG2E
            x = np.where(a, x, -np.inf)
            m_new = np.maximum(m_run, x.max(-1))
            m_use = np.where(np.isinf(m_new), 0.0, m_new)
            alpha = np.exp2(m_run - m_use)
            p = np.exp2(x - m_use[..., None])
            l_run = l_run * alpha + p.sum(-1)
            acc_o = acc_o * alpha[..., None] + p @ vj
            if dual:
                ts = (tq[:, :, m0:m1] @ kj.transpose(0, 1, 3, 2) + qi @ tk[:, :, n0:n1].transpose(0, 1, 3, 2)) * scale
                ts = np.where(a, ts, 0.0)
                w = p * ts
                mu_run = mu_run * alpha + w.sum(-1)
                acc_t = acc_t * alpha[..., None] + w @ vj + p @ tv[:, :, n0:n1]
            m_run = m_new
        empty = l_run <= 0
        inv_l = np.where(empty, 0.0, 1.0 / np.where(empty, 1.0, l_run))
        oi = acc_o * inv_l[..., None]
        o[:, :, m0:m1] = oi
        with np.errstate(divide="ignore"):
            lse[:, :, m0:m1] = np.where(empty, np.inf, m_run + np.log2(np.where(empty, 1.0, l_run)))
        if dual:
            mun = mu_run * inv_l
            to[:, :, m0:m1] = acc_t * inv_l[..., None] - mun[..., None] * oi
            mu_out[:, :, m0:m1] = mun
    return dict(o=o, to=to, lse=lse, mu=mu_out)


def closed_form_backward(q, k, v, tq, tk, tv, go, gto, lse, mu, attn_mask=None, causal=False, scale=None):
    """Recompute-from-logsumexp backward in float64 (dense per head, no L x L state kept between heads).

    ``P = 2^(x - lse)`` as in upstream's backward (jvp_attention.py:1509-1512, 1659-1662); with
    ``gto`` present the tangent-path terms are added:
        gtS = P*(E - eps);  gS = P*(E*(tS-mu) - eps*tS + F + dP - delta - cterm)
        dV = P^T go + (P*(tS-mu))^T gto;  dQ = s(gS K + gtS tK);  dK = s(gS^T Q + gtS^T tQ).
    Returns (dq, dk, dv) NumPy arrays.
    """
    f = lambda x: None if x is None else (x if isinstance(x, np.ndarray) else x.detach().cpu().to(torch.float64).numpy())  # noqa: E731
    q, k, v, tq, tk, tv, go, gto, lse, mu = (f(x) for x in (q, k, v, tq, tk, tv, go, gto, lse, mu))
    B, H, L, D = q.shape
    scale = D**-0.5 if scale is None else scale
    allow, bias = _dense_mask_bias(B, H, L, attn_mask, causal)
    T = lambda a: a.transpose(0, 1, 3, 2)  # noqa: E731
    x = (q @ T(k)) * (scale * LOG2E) + bias * LOG2E
    p = np.where(allow, np.exp2(np.where(allow, x, 0.0) - lse[..., None]), 0.0)
    o = p @ v
    acc = np.zeros_like(p)
    dv = np.zeros_like(v)
    gts = None
    sub = np.zeros((B, H, L))
    if go is not None:
        sub = sub + (go * o).sum(-1)
        acc = acc + go @ T(v)
        dv = dv + T(p) @ go
    if gto is not None:
        ts = np.where(allow, (tq @ T(k) + q @ T(tk)) * scale, 0.0)
        to = (p * (ts - mu[..., None])) @ v + p @ tv
        eps = (gto * o).sum(-1)
        cterm = (gto * to).sum(-1) - eps * mu
        E = gto @ T(v)
        Fm = gto @ T(tv)
        gts = p * (E - eps[..., None])
        acc = acc + E * (ts - mu[..., None]) - eps[..., None] * ts + Fm
        sub = sub + cterm
        dv = dv + T(p * (ts - mu[..., None])) @ gto
    gs = p * (acc - sub[..., None])
    dq = gs @ k
    dk = T(gs) @ q
    if gts is not None:
        dq = dq + gts @ tk
        dk = dk + T(gts) @ tq
    return dq * scale, dk * scale, dv


# ---------------------------------------------------------------------------------------------
# Error metrics used by the tests (tolerances are stated in the tests themselves)
# ---------------------------------------------------------------------------------------------
def max_abs_err(x, ref) -> float:
    x = torch.as_tensor(np.asarray(x) if not isinstance(x, torch.Tensor) else x).detach().cpu().double()
    ref = torch.as_tensor(np.asarray(ref) if not isinstance(ref, torch.Tensor) else ref).detach().cpu().double()
    return (x - ref).abs().max().item()


def rel_err(x, ref) -> float:
    """max|x - ref| / max|ref| -- the relative error the fp32 tolerance is stated in."""
    ref_t = torch.as_tensor(np.asarray(ref) if not isinstance(ref, torch.Tensor) else ref).detach().cpu().double()
    den = ref_t.abs().max().item()
    return max_abs_err(x, ref) / (den if den > 0 else 1.0)


def cpu_reference_step(q, k, v, tq, tk, tv, loss_fn, attn_mask=None, causal=False, scale=None, dtype=torch.float32):
    """One fwd_dual + backward step of upstream's CPU path (torch.func.jvp over SDPA-MATH then
    autograd), used as the timed CPU baseline.  ``loss_fn(o, to)`` returns a scalar."""
    a = [x.detach().to("cpu", dtype).requires_grad_() for x in (q, k, v)]
    o, to = sdpa_jvp(*a, tq, tk, tv, attn_mask, causal, scale, dtype=dtype)
    loss = loss_fn(o, to)
    g = torch.autograd.grad(loss, a)
    return loss.detach(), g
