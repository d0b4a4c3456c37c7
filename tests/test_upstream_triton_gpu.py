"""GPU parity with upstream's own Triton kernels, run unmodified on the same B200 and the same tensors.

The upstream source file is expected under ``baseline/_ref/jvp_flash_attention/`` (kept out of version control); it
is loaded by path under an alias by ``baseline/upstream.py``.  When the file is absent the tests skip with that reason.

Compared: O and tO of ``fwd_dual`` and dq, dk, dv of a loss on O -- the quantities upstream can compute (its tangent
output carries no gradient and its backward ignores float masks that are not {0, -100},
jvp_attention.py:2828-2831, 1519-1522) -- for no mask, causal, a boolean (B,H,L,L) mask and a {0, -100} additive
mask, in upstream's own tolerances (tests/test_jvp_attention.py:688-693: float16 4e-3, bfloat16 3.2e-2, float32
2.35e-2, absolute).  Both sides are also held against the float64 oracle, so a shared mistake cannot hide.
"""
import pytest
import torch

import jvp_flash_attention_b200.jvp_attention as ja
from baseline import upstream
from oracle import jvp_attention_oracle as orc

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not upstream.available(), reason="upstream's source file is not under baseline/_ref")]

UPSTREAM_TOL = {torch.float16: 4e-3, torch.bfloat16: 3.2e-2, torch.float32: 2.35e-2}
DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}
_state = {}


def _upstream():
    """Module and the keyword arguments with which it compiles here (defaults first), found once per process."""
    if "mod" not in _state:
        mod = upstream.load()
        kw, errors = upstream.pick_kwargs(mod)
        _state.update(mod=mod, kw=kw, errors=errors)
    if _state["kw"] is None:
        pytest.skip(f"no upstream variant compiled and ran on this GPU: {_state['errors']}")
    return _state["mod"], _state["kw"]


def _case(dtype, L, kind, seed, dev):
    g = torch.Generator().manual_seed(seed)
    B, H, D = 1, 2, 64
    q, k, v, tq, tk, tv, w = [torch.randn(B, H, L, D, generator=g) for _ in range(7)]
    if dtype == torch.bfloat16:
        tq, tk, tv = tq * 0.1, tk * 0.1, tv * 0.1
    mask = None
    if kind == "boolean":
        mask = torch.rand(B, H, L, L, generator=g) > 0.5
    elif kind == "additive":
        mask = torch.where(torch.rand(B, H, L, L, generator=g) > 0.5, 0.0, ja.MASK_CONST).to(dtype)
    t = [x.to(dtype) for x in (q, k, v, tq, tk, tv, w)]
    return t, mask


CASES = [("bf16", 2048, "none"), ("bf16", 2048, "causal"), ("bf16", 2048, "boolean"), ("bf16", 2048, "additive"),
         ("bf16", 128, "causal"), ("bf16", 1024, "none"), ("fp16", 1024, "causal"), ("fp16", 1024, "boolean"),
         ("fp32", 1024, "none"), ("fp32", 1024, "additive")]


@pytest.mark.parametrize("dt,L,kind", CASES)
def test_forward_dual_and_backward_through_o_match_upstream_triton(dt, L, kind):
    mod, kw = _upstream()
    dtype, dev = DT[dt], torch.device("cuda:0")
    (q, k, v, tq, tk, tv, w), mask = _case(dtype, L, kind, seed=L + len(kind), dev=dev)
    causal = kind == "causal"
    cu = lambda x: None if x is None else x.to(dev)  # noqa: E731
    dq_, dk_, dv_, dtq, dtk, dtv, dw, dmask = (cu(x) for x in (q, k, v, tq, tk, tv, w, mask))

    # upstream (the reference's own fp32 arithmetic is single-pass TF32: compare in that mode as well as in the default)
    o_u, to_u = upstream.fwd_dual(mod, dq_, dk_, dv_, dtq, dtk, dtv, attn_mask=dmask, causal=causal, **kw)
    _, gq_u, gk_u, gv_u = upstream.grads_through_o(mod, dq_, dk_, dv_, dw, attn_mask=dmask, causal=causal, **kw)

    # this library, through its public API
    a = [x.detach().clone().requires_grad_() for x in (dq_, dk_, dv_)]
    o_m, to_m = torch.func.jvp(lambda q_, k_, v_: ja.JVPAttn.fwd_dual(q_, k_, v_, attn_mask=dmask, causal=causal), tuple(a),
                               (dtq, dtk, dtv))
    gq_m, gk_m, gv_m = torch.autograd.grad((o_m.float() * dw.float()).sum(), a)
    torch.cuda.synchronize()

    tol = UPSTREAM_TOL[dtype]
    pairs = {"O": (o_m, o_u), "tO": (to_m, to_u), "dq": (gq_m, gq_u), "dk": (gk_m, gk_u), "dv": (gv_m, gv_u)}
    for name, (mine, theirs) in pairs.items():
        assert torch.isfinite(mine.float()).all(), name
        err = (mine.float() - theirs.float()).abs().max().item()
        scale = max(1.0, theirs.float().abs().max().item()) if name[0] == "d" else 1.0
        assert err <= tol * scale, f"{name}: |ours - upstream| = {err:.3e} > {tol * scale:.3e}"

    # both against float64 (a boolean mask as is; the additive {0, -100} mask as the boolean mask it encodes)
    omask = mask if kind != "additive" else (mask.float() == 0)
    ro, rto = orc.sdpa_jvp(q, k, v, tq, tk, tv, attn_mask=omask, causal=causal)
    _, _, rdq, rdk, rdv = orc.grads_through_both(q, k, v, tq, tk, tv, w, None, attn_mask=omask, causal=causal)
    refs = {"O": ro, "tO": rto, "dq": rdq, "dk": rdk, "dv": rdv}
    for name, (mine, theirs) in pairs.items():
        scale = max(1.0, refs[name].abs().max().item()) if name[0] == "d" else 1.0
        e_m, e_u = orc.max_abs_err(mine, refs[name]), orc.max_abs_err(theirs, refs[name])
        assert e_m <= tol * scale, f"{name}: ours vs float64 {e_m:.3e}"
        assert e_u <= tol * scale, f"{name}: upstream vs float64 {e_u:.3e}"
        # this library should not be the less accurate of the two by more than rounding noise
        assert e_m <= 2.0 * e_u + 1e-6 * scale + (2e-3 if dtype != torch.float32 else 0.0), (
            f"{name}: ours {e_m:.3e} vs upstream {e_u:.3e} against float64")
