"""Test helper: float64 stand-ins for the two kernel launch helpers of the package, built on the
oracle.  They let the CPU suite exercise the autograd wiring (JVPAttn / _TangentBridge / _AttnBwd)
without a GPU.  Only tests may use this; the package itself never falls back to it."""
import torch

from jvp_flash_attention_b200 import _lib
from oracle import jvp_attention_oracle as orc


def _mask_from_spec(spec, like):
    B, H, L, _ = like.shape
    if spec.kind == _lib.MASK_NONE:
        return None, False
    if spec.kind == _lib.MASK_CAUSAL:
        return None, True
    if spec.kind == _lib.MASK_KVLEN:
        m = torch.arange(L)[None, :] < spec.tensor.cpu()[:, None]
        return m[:, None, None, :], False
    t = spec.tensor
    shape = [1 if s == 0 else n for s, n in zip(spec.strides, (B, H, L, L))]
    view = t.reshape(shape) if t.numel() == int(torch.tensor(shape).prod()) else t
    if spec.kind == _lib.MASK_BOOL:
        return view.bool(), False
    return view, False


def launch_fwd(q, k, v, tq, tk, tv, spec, sm_scale):
    mask, causal = _mask_from_spec(spec, q)
    r = orc.tiled_forward(q, k, v, tq, tk, tv, attn_mask=mask, causal=causal, scale=sm_scale)
    cv = lambda x, dt: None if x is None else torch.from_numpy(x).to(dt)  # noqa: E731
    return cv(r["o"], q.dtype), cv(r["to"], q.dtype), cv(r["lse"], torch.float64), cv(r["mu"], torch.float64)


def launch_bwd(q, k, v, tq, tk, tv, o, to, lse, mu, go, gto, spec, sm_scale):
    mask, causal = _mask_from_spec(spec, q)
    if gto is None:
        tq = tk = tv = mu = None
    d = orc.closed_form_backward(q, k, v, tq, tk, tv, go, gto, lse.double(), None if mu is None else mu.double(),
                                 attn_mask=mask, causal=causal, scale=sm_scale)
    return tuple(torch.from_numpy(x).to(q.dtype) for x in d)


def mask_check(spec, shape):
    """Stand-in for the device pass jvpfa_mask_check: the same three answers from eager reductions
    (what upstream computes, jvp_attention.py:2438-2457)."""
    t = spec.tensor.reshape(tuple(shape)) if spec.tensor.numel() == int(torch.tensor(tuple(shape)).prod()) else spec.tensor
    if spec.kind == _lib.MASK_BOOL:
        return bool(t.bool().any(dim=(-1, -2)).all()), False, False
    return bool((t != -100.0).any(dim=(-1, -2)).all()), bool(torch.isinf(t).any()), bool(torch.isnan(t).any())


def mask_tiles(spec, L):
    """Stand-in for jvpfa_mask_tiles: no tile bitmap on the host, so the caller takes its element-wise route."""
    raise _lib.Unsupported("no tile bitmap without the device pass")
