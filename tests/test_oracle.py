"""CPU tests that pin the oracle: against upstream's own kernel outputs (tests/golden, produced by
running upstream's Triton kernels in the Triton interpreter) and the two statements against
each other."""
import numpy as np
import pytest
import torch

from oracle import jvp_attention_oracle as orc

GOLDEN = [
    "none_L64_D32",
    "causal_L64_D32",
    "bool_L64_D32",
    "additive_L64_D32",
    "none_L128_D64",
    "causal_L128_D64",
]

# Upstream's interpreter run computes fp32 tile dots; agreement with the float64 oracle is limited
# by fp32 rounding only.
GOLDEN_TOL = 1e-5


def _load(golden_dir, name):
    z = np.load(golden_dir / f"upstream_{name}.npz")
    t = {k: torch.from_numpy(z[k]) for k in z.files if k not in ("causal", "mask_kind")}
    return t, bool(z["causal"]), str(z["mask_kind"])


@pytest.mark.parametrize("name", GOLDEN)
def test_sdpa_oracle_matches_upstream_kernel(golden_dir, name):
    t, causal, mkind = _load(golden_dir, name)
    mask = t.get("mask")
    o, to, dq, dk, dv = orc.grads_through_both(t["q"], t["k"], t["v"], t["tq"], t["tk"], t["tv"], t["w"], None,
                                               attn_mask=mask, causal=causal)
    for got, key in ((o, "o"), (to, "to"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert orc.rel_err(t[key], got) < GOLDEN_TOL, key


@pytest.mark.parametrize("name", GOLDEN)
def test_tiled_restatement_matches_upstream_kernel(golden_dir, name):
    t, causal, mkind = _load(golden_dir, name)
    mask = t.get("mask")
    r = orc.tiled_forward(t["q"], t["k"], t["v"], t["tq"], t["tk"], t["tv"], attn_mask=mask, causal=causal)
    assert orc.rel_err(t["o"], r["o"]) < GOLDEN_TOL
    assert orc.rel_err(t["to"], r["to"]) < GOLDEN_TOL
    dq, dk, dv = orc.closed_form_backward(t["q"], t["k"], t["v"], None, None, None, t["w"], None, r["lse"], None,
                                          attn_mask=mask, causal=causal)
    for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert orc.rel_err(t[key], got) < GOLDEN_TOL, key


def test_float_mask_semantics_are_those_of_torch_sdpa(golden_dir):
    """A float mask is added to the scaled scores, in forward and backward: the fixture holds PyTorch's own
    scaled_dot_product_attention (float64, math path) with a general additive mask, its tangent and the gradients through
    both outputs (tests/golden/make_sdpa_bias_golden.py).  Both statements of the oracle must reproduce it."""
    z = np.load(golden_dir / "sdpa_bias_L64_D32.npz")
    t = {k_: torch.from_numpy(z[k_]) for k_ in z.files}
    o, to, dq, dk, dv = orc.grads_through_both(t["q"], t["k"], t["v"], t["tq"], t["tk"], t["tv"], t["w1"], t["w2"],
                                               attn_mask=t["bias"])
    for got, key in ((o, "o"), (to, "to"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert orc.rel_err(t[key], got) < 1e-10, key
    r = orc.tiled_forward(t["q"], t["k"], t["v"], t["tq"], t["tk"], t["tv"], attn_mask=t["bias"])
    assert orc.rel_err(t["o"], r["o"]) < 1e-10 and orc.rel_err(t["to"], r["to"]) < 1e-10
    d = orc.closed_form_backward(t["q"], t["k"], t["v"], t["tq"], t["tk"], t["tv"], t["w1"], t["w2"], r["lse"], r["mu"],
                                 attn_mask=t["bias"])
    for got, key in zip(d, ("dq", "dk", "dv")):
        assert orc.rel_err(t[key], got) < 1e-10, key


@pytest.mark.parametrize("kind", ["none", "causal", "kvlen", "bool", "bias"])
def test_two_statements_agree_through_both_outputs(kind):
    """Closed-form backward (incl. the tangent-output cotangent) against autograd in float64."""
    g = torch.Generator().manual_seed(11)
    B, H, L, D = 2, 2, 48, 16
    q, k, v, tq, tk, tv, go, gto = [torch.randn(B, H, L, D, generator=g, dtype=torch.float64) for _ in range(8)]
    mask, causal = None, False
    if kind == "causal":
        causal = True
    elif kind == "kvlen":
        lens = torch.tensor([29, 48])
        mask = (torch.arange(L)[None, :] < lens[:, None])[:, None, None, :]
    elif kind == "bool":
        mask = torch.rand(B, H, L, L, generator=g) > 0.4
        mask[..., 0] = True
    elif kind == "bias":
        mask = torch.randn(B, 1, L, L, generator=g, dtype=torch.float64).clamp(-5, 5)
    o, to, dq, dk, dv = orc.grads_through_both(q, k, v, tq, tk, tv, go, gto, attn_mask=mask, causal=causal)
    r = orc.tiled_forward(q, k, v, tq, tk, tv, attn_mask=mask, causal=causal, block=16)
    assert orc.max_abs_err(r["o"], o) < 1e-12
    assert orc.max_abs_err(r["to"], to) < 1e-12
    d2 = orc.closed_form_backward(q, k, v, tq, tk, tv, go, gto, r["lse"], r["mu"], attn_mask=mask, causal=causal)
    for a, b in zip(d2, (dq, dk, dv)):
        assert orc.max_abs_err(a, b) < 1e-11


def test_fully_masked_rows_are_zero():
    g = torch.Generator().manual_seed(5)
    q, k, v, tq, tk, tv = [torch.randn(1, 1, 32, 16, generator=g, dtype=torch.float64) for _ in range(6)]
    mask = torch.ones(1, 1, 32, 32, dtype=torch.bool)
    mask[0, 0, 3] = False
    o, to = orc.sdpa_jvp(q, k, v, tq, tk, tv, attn_mask=mask)
    r = orc.tiled_forward(q, k, v, tq, tk, tv, attn_mask=mask)
    assert o[0, 0, 3].abs().max() == 0 and to[0, 0, 3].abs().max() == 0
    assert np.abs(r["o"][0, 0, 3]).max() == 0 and np.isinf(r["lse"][0, 0, 3])
    assert orc.max_abs_err(r["o"], o) < 1e-12 and orc.max_abs_err(r["to"], to) < 1e-12


def test_hvp_equals_grad_through_tangent():
    """The identity the double-backward path of the package relies on."""
    g = torch.Generator().manual_seed(3)
    q, k, v, w, vd = [torch.randn(1, 2, 32, 16, generator=g, dtype=torch.float64) for _ in range(5)]
    bias = torch.randn(1, 2, 32, 32, generator=g, dtype=torch.float64).clamp(-5, 5)
    _, _, h = orc.hvp_q(q, k, v, w, vd, attn_mask=bias)
    z = torch.zeros_like(q)
    _, _, dq, _, _ = orc.grads_through_both(q, k, v, vd, z, z, None, w, attn_mask=bias)
    assert orc.max_abs_err(dq, h) < 1e-12
