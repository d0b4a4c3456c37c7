"""GPU tests of the public surface around the kernels: upstream's import path, the SDPA-shaped wrapper, the fp32
precision recorded with a call, what a consumer sees right after a backward on the same stream, and how a failed
bounded wait shows in later results."""
import pytest
import torch
import torch.autograd.forward_ad as fwAD
import torch.nn.functional as F

import jvp_flash_attention_b200.jvp_attention as ja
from jvp_flash_attention_b200 import _lib
from oracle import jvp_attention_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rand(shape, dtype, seed, n):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(shape, generator=g).to(dtype).to(DEV) for _ in range(n)]


def test_upstream_import_path_and_readme_usage():
    """The lines of upstream's README (README.md:36-67) work unchanged: same import path, same call."""
    from jvp_flash_attention.jvp_attention import JVPAttn, attention as jvp_attention

    assert JVPAttn is ja.JVPAttn
    q, k, v = _rand((2, 4, 128, 64), torch.bfloat16, 0, 3)
    attn_mask = torch.rand(2, 4, 128, 128, device=DEV) > 0.3
    attn_mask[..., 0] = True
    x = jvp_attention(q, k, v, attn_mask=attn_mask)
    ref = orc.sdpa_primal(q.cpu(), k.cpu(), v.cpu(), attn_mask=attn_mask.cpu())
    assert orc.max_abs_err(x, ref) <= 2e-2
    # "make sure to use JVP Flash Attention in your model as JVPAttn.fwd_dual(q, k, v)" under torch.func.jvp
    (tq,) = _rand((2, 4, 128, 64), torch.bfloat16, 1, 1)
    pred, df = torch.func.jvp(lambda x_jvp: JVPAttn.fwd_dual(x_jvp, k, v), (q,), (tq * 0.1,))
    ro, rto = orc.sdpa_jvp(q.cpu(), k.cpu(), v.cpu(), (tq * 0.1).cpu(), torch.zeros_like(k).cpu(), torch.zeros_like(v).cpu())
    assert orc.max_abs_err(pred, ro) <= 2e-2 and orc.max_abs_err(df, rto) <= 2e-2


@pytest.mark.parametrize("is_causal,scale", [(False, None), (True, None), (False, 0.2)])
def test_sdpa_shaped_wrapper(is_causal, scale):
    """scaled_dot_product_attention(query, key, value, attn_mask, dropout_p, is_causal, scale): plain tensors give
    what torch's own function gives; dual tensors give primal and tangent; dropout is refused as upstream refuses it."""
    q, k, v, tq, tk, tv = _rand((2, 3, 192, 64), torch.float16, 3, 6)
    mask = None
    if not is_causal:
        mask = torch.rand(2, 1, 192, 192, device=DEV) > 0.4
        mask[..., 0] = True
    out = ja.scaled_dot_product_attention(q, k, v, attn_mask=mask, is_causal=is_causal, scale=scale)
    ref = F.scaled_dot_product_attention(q.float(), k.float(), v.float(), attn_mask=mask, is_causal=is_causal, scale=scale)
    assert (out.float() - ref).abs().max().item() <= 4e-3
    with fwAD.dual_level():
        d = [fwAD.make_dual(x, t) for x, t in ((q, tq), (k, tk), (v, tv))]
        o, to = fwAD.unpack_dual(ja.scaled_dot_product_attention(*d, attn_mask=mask, is_causal=is_causal, scale=scale))
    c = lambda x: None if x is None else x.cpu()  # noqa: E731
    ro, rto = orc.sdpa_jvp(c(q), c(k), c(v), c(tq), c(tk), c(tv), attn_mask=c(mask), causal=is_causal, scale=scale)
    assert orc.max_abs_err(o, ro) <= 2e-2 and orc.max_abs_err(to, rto) <= 2e-2
    with pytest.raises(NotImplementedError):
        ja.scaled_dot_product_attention(q, k, v, dropout_p=0.1)


def test_fp32_precision_is_recorded_with_the_call():
    """Flipping set_fp32_precision between a forward and its backward changes nothing: the backward recomputes the
    scores at the precision the forward used."""
    q, k, v, w = _rand((1, 2, 160, 64), torch.float32, 5, 4)

    def grads(flip):
        prev = ja.set_fp32_precision("3xtf32")
        try:
            a = [x.clone().requires_grad_() for x in (q, k, v)]
            o = ja.attention(*a, causal=True)
            if flip:
                ja.set_fp32_precision("tf32")
            return torch.autograd.grad((o * w).sum(), a)
        finally:
            ja.set_fp32_precision(prev)

    for x, y in zip(grads(False), grads(True)):
        assert torch.equal(x, y)
    # and the other way round: a forward in the single-pass mode keeps that mode in its backward
    prev = ja.set_fp32_precision("tf32")
    try:
        a = [x.clone().requires_grad_() for x in (q, k, v)]
        o = ja.attention(*a, causal=True)
        g1 = torch.autograd.grad((o * w).sum(), a, retain_graph=True)
        ja.set_fp32_precision("3xtf32")
        g2 = torch.autograd.grad((o * w).sum(), a)
    finally:
        ja.set_fp32_precision(prev)
    for x, y in zip(g1, g2):
        assert torch.equal(x, y)


@pytest.mark.parametrize("D", [64, 128])
def test_results_of_the_two_launch_backward_are_complete_for_the_next_kernel(D):
    """The own-queries launch of the two-launch backward starts while the own-keys launch is still running.  A kernel
    that follows on the same stream and reads dk / dv must see them complete.  Shape: key padding that leaves the
    own-queries launch almost nothing to do (so it would finish long before the own-keys launch), consumer = a copy
    of dk / dv issued straight after the call, no host synchronisation in between."""
    B, H, L = 6, 8, 2048
    q, k, v, tq, tk, tv, go, gto = _rand((B, H, L, D), torch.bfloat16, 7, 8)
    kv_len = torch.full((B,), 96, dtype=torch.int32, device=DEV)
    kv_len[0] = L  # one batch entry with full-length work for the own-keys launch
    spec = _lib.MaskSpec(_lib.MASK_KVLEN, kv_len)
    o, to = torch.empty_like(q), torch.empty_like(q)
    lse = torch.empty(B, H, L, device=DEV)
    mu = torch.empty_like(lse)
    _lib.fwd(q, k, v, tq, tk, tv, o, to, lse, mu, spec, D**-0.5)
    stats = torch.empty(3, B, H, L, device=DEV)
    _lib.bwd_preprocess(o, to, go, gto, mu, stats[0], stats[1], stats[2])
    dq, dk, dv = (torch.empty_like(q) for _ in range(3))
    call = lambda: _lib.bwd(q, k, v, tq, tk, tv, go, gto, lse, mu, stats[0], stats[1], stats[2], dq, dk, dv, spec, D**-0.5,  # noqa: E731
                            _lib.IMPL_TCGEN05)
    call()
    torch.cuda.synchronize()
    want_k, want_v = dk.clone(), dv.clone()
    for _ in range(5):
        dk.fill_(float("nan"))
        dv.fill_(float("nan"))
        call()
        got_k, got_v = dk.clone(), dv.clone()  # the very next kernels on the stream
        torch.cuda.synchronize()
        assert torch.equal(got_k, want_k) and torch.equal(got_v, want_v)
    assert _lib.device_status() == 0
