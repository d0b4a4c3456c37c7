"""CPU tests of the Python layer: autograd wiring, mask classification, argument errors, sharding.
The kernel launch helpers are replaced by float64 oracle stand-ins (tests/_oracle_launchers.py);
everything else is the shipped code."""
import pytest
import torch
import torch.autograd.forward_ad as fwAD

import jvp_flash_attention_b200.jvp_attention as ja
from jvp_flash_attention_b200 import _lib, workloads
from oracle import jvp_attention_oracle as orc
from tests import _oracle_launchers as stand_in


@pytest.fixture()
def cpu_kernels(monkeypatch):
    monkeypatch.setattr(ja, "_launch_fwd", stand_in.launch_fwd)
    monkeypatch.setattr(ja, "_launch_bwd", stand_in.launch_bwd)
    monkeypatch.setattr(ja, "_require_cuda", lambda *a: None)
    monkeypatch.setattr(_lib, "mask_check", stand_in.mask_check)
    monkeypatch.setattr(_lib, "mask_tiles", stand_in.mask_tiles)
    monkeypatch.setitem(_lib.DTYPE_ENUM, torch.float64, _lib.FP32)  # stand-ins compute in float64


def _inputs(seed=0, B=1, H=2, L=32, D=32, n=8):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(B, H, L, D, generator=g, dtype=torch.float64) for _ in range(n)]


@pytest.mark.parametrize("route", ["func_jvp", "fwad"])
@pytest.mark.parametrize("kind", ["none", "causal", "bias", "keypad"])
def test_grad_through_primal_and_tangent(cpu_kernels, route, kind):
    q, k, v, tq, tk, tv, w1, w2 = _inputs()
    mask, causal = None, False
    if kind == "causal":
        causal = True
    elif kind == "bias":
        mask = torch.randn(1, 2, 32, 32, dtype=torch.float64).clamp(-5, 5)
    elif kind == "keypad":
        mask = (torch.arange(32) < 20)[None, None, None, :]
    ro, rto, rdq, rdk, rdv = orc.grads_through_both(q, k, v, tq, tk, tv, w1, w2, attn_mask=mask, causal=causal)
    a = [x.clone().requires_grad_() for x in (q, k, v)]
    fn = lambda q_, k_, v_: ja.JVPAttn.fwd_dual(q_, k_, v_, attn_mask=mask, causal=causal)  # noqa: E731
    if route == "func_jvp":
        o, to = torch.func.jvp(fn, tuple(a), (tq, tk, tv))
        assert to.requires_grad
        g = torch.autograd.grad((o * w1).sum() + (to * w2).sum(), a)
    else:
        with fwAD.dual_level(), torch.enable_grad():
            d = [fwAD.make_dual(x, t) for x, t in zip(a, (tq, tk, tv))]
            out = fn(*d)
            o, to = fwAD.unpack_dual(out)
            assert to.requires_grad
            g = torch.autograd.grad((o * w1).sum() + (to * w2).sum(), a)
    assert orc.max_abs_err(o, ro) < 1e-10 and orc.max_abs_err(to, rto) < 1e-10
    for x, y in zip(g, (rdq, rdk, rdv)):
        assert orc.max_abs_err(x, y) < 1e-9


def test_mask_verification_is_remembered_per_tensor_object_and_version(cpu_kernels, monkeypatch):
    """The verification pass over a mask runs once while the same tensor object comes back unmodified; an in-place
    change (torch bumps the version counter) or another tensor object runs it again; a failed verification is not
    remembered."""
    q, k, v, *_ = _inputs(7)
    calls = []
    inner = stand_in.mask_tiles

    def counting(*args):
        calls.append(1)
        return inner(*args)

    monkeypatch.setattr(_lib, "mask_tiles", counting)
    ja._MASK_MEMO.clear()
    g = torch.Generator().manual_seed(1)
    mask = torch.rand(1, 2, 32, 32, generator=g) > 0.4
    mask[..., 0] = True
    o1 = ja.attention(q, k, v, attn_mask=mask)
    o2 = ja.attention(q, k, v, attn_mask=mask)
    assert len(calls) == 1 and torch.equal(o1, o2)
    mask[0, 0, 3, 5] = not bool(mask[0, 0, 3, 5])  # in place: the version counter moves
    o3 = ja.attention(q, k, v, attn_mask=mask)
    assert len(calls) == 2 and not torch.equal(o1, o3)
    ja.attention(q, k, v, attn_mask=mask.clone())  # another object
    assert len(calls) == 3
    bad = torch.zeros(1, 2, 32, 32, dtype=torch.bool)
    bad[:, :, ::2, 1] = True  # not a key-padding prefix; head rows exist, but make one head all False
    bad[0, 1] = False
    for _ in range(2):
        with pytest.raises(AssertionError, match="all False"):
            ja.attention(q, k, v, attn_mask=bad)
    # the memo does not outlive the caller's tensor object
    tmp = mask.clone()
    ja.attention(q, k, v, attn_mask=tmp)
    assert id(tmp) in ja._MASK_MEMO
    key_id = id(tmp)
    del tmp
    import gc
    gc.collect()
    assert key_id not in ja._MASK_MEMO
    monkeypatch.setattr(ja, "MASK_MEMO_ENABLED", False)
    n = len(calls)
    ja.attention(q, k, v, attn_mask=mask)
    ja.attention(q, k, v, attn_mask=mask)
    assert len(calls) == n + 2


def test_func_jvp_keeps_the_callers_grad_mode(cpu_kernels):
    """Inside torch.func.jvp the call runs one level down on the unwrapped tensors; the caller's no_grad must hold
    there as well, and with grad enabled both outputs take part in the graph."""
    q, k, v, tq, tk, tv, _, _ = _inputs(5)
    a = [x.clone().requires_grad_() for x in (q, k, v)]
    fn = lambda q_, k_, v_: ja.JVPAttn.fwd_dual(q_, k_, v_, causal=True)  # noqa: E731
    with torch.no_grad():
        o, to = torch.func.jvp(fn, tuple(a), (tq, tk, tv))
    assert not o.requires_grad and not to.requires_grad
    o2, to2 = torch.func.jvp(fn, tuple(a), (tq, tk, tv))
    assert o2.requires_grad and to2.requires_grad
    assert torch.equal(o, o2.detach()) and torch.equal(to, to2.detach())


@pytest.mark.parametrize("route", ["func_jvp", "fwad"])
@pytest.mark.parametrize("which", ["both", "o", "to"])
def test_one_backward_launch_per_step_whatever_the_loss_uses(cpu_kernels, monkeypatch, route, which):
    """A loss on O and tO reaches the kernels as one launch with both cotangents (the node of the tangent output hands
    its cotangent to the node of the primal output, which autograd runs after it), also when the backward is run twice
    over a retained graph; a loss on one of the two as one launch with that cotangent."""
    q, k, v, tq, tk, tv, w1, w2 = _inputs(3)
    calls = []
    inner = stand_in.launch_bwd

    def counting(*args):
        calls.append((args[10] is not None, args[11] is not None))  # (go given, gto given)
        return inner(*args)

    monkeypatch.setattr(ja, "_launch_bwd", counting)
    a = [x.clone().requires_grad_() for x in (q, k, v)]

    def loss_of(o, to):
        return {"both": (o * w1).sum() + (to * w2).sum(), "o": (o * w1).sum(), "to": (to * w2).sum()}[which]

    go = w1 if which != "to" else None
    gto = w2 if which != "o" else None
    _, _, rdq, rdk, rdv = orc.grads_through_both(q, k, v, tq, tk, tv, go, gto)
    if route == "func_jvp":
        o, to = torch.func.jvp(ja.JVPAttn.fwd_dual, tuple(a), (tq, tk, tv))
        loss = loss_of(o, to)
        g1 = torch.autograd.grad(loss, a, retain_graph=True)
        g2 = torch.autograd.grad(loss, a)
    else:
        with fwAD.dual_level(), torch.enable_grad():
            out = ja.JVPAttn.fwd_dual(*[fwAD.make_dual(x, t) for x, t in zip(a, (tq, tk, tv))])
            o, to = fwAD.unpack_dual(out)
            loss = loss_of(o, to)
            g1 = torch.autograd.grad(loss, a, retain_graph=True)
            g2 = torch.autograd.grad(loss, a)
    assert calls == [(which != "to", which != "o")] * 2, calls
    for g in (g1, g2):
        for x, y in zip(g, (rdq, rdk, rdv)):
            assert orc.max_abs_err(x, y) < 1e-9


def test_second_derivative_with_a_loss_on_both_outputs(cpu_kernels):
    """create_graph=True with a loss on O and tO: the part through O can be differentiated again (Hessian-vector
    product), the part through tO refuses loudly instead of being treated as a constant."""
    q, k, v, tq, tk, tv, w1, w2 = _inputs(4)
    a = [x.clone().requires_grad_() for x in (q, k, v)]
    o, to = torch.func.jvp(ja.JVPAttn.fwd_dual, tuple(a), (tq, tk, tv))
    (gq,) = torch.autograd.grad((o * w1).sum() + (to * w2).sum(), a[:1], create_graph=True)
    _, _, rdq, _, _ = orc.grads_through_both(q, k, v, tq, tk, tv, w1, w2)
    assert orc.max_abs_err(gq, rdq) < 1e-9
    with pytest.raises(RuntimeError, match="second time"):
        torch.autograd.grad((gq * tq).sum(), a[:1])


def test_loss_on_tangent_only_and_tangent_grads(cpu_kernels):
    q, k, v, tq, tk, tv, w1, w2 = _inputs(1)
    a = [x.clone().requires_grad_() for x in (q, k, v)]
    t = [x.clone().requires_grad_() for x in (tq, tk, tv)]
    o, to = torch.func.jvp(ja.JVPAttn.fwd_dual, tuple(a), tuple(t))
    g = torch.autograd.grad((to * w2).sum(), a + t)
    ref_in = [x.clone().requires_grad_() for x in (q, k, v, tq, tk, tv)]
    _, rto = orc.sdpa_jvp(*ref_in)
    rg = torch.autograd.grad((rto * w2).sum(), ref_in)
    for x, y in zip(g, rg):
        assert orc.max_abs_err(x, y) < 1e-9


def test_primal_only_backward_and_hvp(cpu_kernels):
    q, k, v, w, vd, *_ = _inputs(2)
    bias = torch.randn(1, 2, 32, 32, dtype=torch.float64).clamp(-5, 5)
    ro, rg1, rh = orc.hvp_q(q, k, v, w, vd, attn_mask=bias)
    q1 = q.clone().requires_grad_()
    o = ja.attention(q1, k, v, attn_mask=bias)
    (g1,) = torch.autograd.grad((o * w).sum(), q1, create_graph=True)
    (h,) = torch.autograd.grad((g1 * vd).sum(), q1)
    assert orc.max_abs_err(o, ro) < 1e-10
    assert orc.max_abs_err(g1, rg1) < 1e-9
    assert orc.max_abs_err(h, rh) < 1e-9


def test_fwd_dual_without_tangents_degrades_to_primal(cpu_kernels):
    q, k, v, *_ = _inputs(3)
    o = ja.JVPAttn.fwd_dual(q, k, v)
    assert orc.max_abs_err(o, orc.sdpa_primal(q, k, v)) < 1e-10
    out, ctx = ja.JVPAttn.apply(q, k, v, None, None, None, None, 0.0, False, None, True, True)
    assert ctx.o_t is None and ctx.M.shape == (1, 2, 32) and ctx.MASK_TYPE == 0


def test_argument_errors_match_upstream(cpu_kernels):
    q, k, v, *_ = _inputs(4)
    with pytest.raises(NotImplementedError):
        ja.attention(q, k, v, dropout_p=0.1)
    with pytest.raises(ValueError):
        ja.attention(q, k, v, attn_mask=torch.ones(1, 2, 32, 32, dtype=torch.bool), causal=True)
    with pytest.raises(AssertionError):
        ja.attention(q[:, :, :30], k[:, :, :30], v[:, :, :30])  # N_CTX < 32
    with pytest.raises(AssertionError):
        ja.attention(q[..., :24], k[..., :24], v[..., :24])  # head dim not in the allowed set
    with pytest.raises(AssertionError):
        ja.attention(q, k[..., :16], v)  # head-dim mismatch
    dead = torch.ones(1, 2, 32, 32, dtype=torch.bool)
    dead[0, 1] = False
    with pytest.raises(AssertionError):
        ja.attention(q, k, v, attn_mask=dead)
    with pytest.raises(AssertionError):
        ja.attention(q, k, v, attn_mask=torch.full((1, 2, 32, 32), float("nan"), dtype=torch.float64))
    with pytest.raises(AssertionError):
        ja.attention(q, k, v, attn_mask=torch.ones(1, 2, 32, 16, dtype=torch.bool))  # wrong key extent


def test_cpu_tensors_are_refused_without_the_stand_in():
    q, k, v, *_ = _inputs(5)
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        ja.attention(q.float(), k.float(), v.float())


def test_mask_classification(cpu_kernels):
    # (verification of mask contents is a device pass, jvpfa_mask_check: covered by the GPU tests)
    Z, H, N = 2, 3, 32
    spec, mt, _ = ja.classify_mask(None, True, Z, H, N, torch.float32, False)
    assert spec.kind == _lib.MASK_CAUSAL and mt == 0
    spec, mt, _ = ja.classify_mask(None, False, Z, H, N, torch.float32, False)
    assert spec.kind == _lib.MASK_NONE
    lens = torch.tensor([20, 32])
    pad = (torch.arange(N)[None, :] < lens[:, None])[:, None, None, :]
    spec, mt, _ = ja.classify_mask(pad, False, Z, H, N, torch.float32, False)
    assert spec.kind == _lib.MASK_KVLEN and mt == 1 and spec.tensor.tolist() == [20, 32]
    spec, _, _ = ja.classify_mask(pad[:1], False, Z, H, N, torch.float32, False)
    assert spec.kind == _lib.MASK_KVLEN and spec.tensor.tolist() == [20, 20]
    holes = pad.clone()
    holes[0, 0, 0, 3] = False  # not a prefix -> generic boolean mask with broadcast strides
    spec, _, _ = ja.classify_mask(holes, False, Z, H, N, torch.float32, False)
    assert spec.kind == _lib.MASK_BOOL and spec.strides == (N, 0, 0, 1)
    full = torch.rand(Z, H, N, N) > 0.3
    full[..., 0] = True
    spec, _, _ = ja.classify_mask(full, False, Z, H, N, torch.float32, False)
    assert spec.kind == _lib.MASK_BOOL and spec.strides == (H * N * N, N * N, N, 1)
    bias = torch.randn(1, H, N, N)
    spec, mt, _ = ja.classify_mask(bias, False, Z, H, N, torch.float32, False)
    assert spec.kind == _lib.MASK_BIAS and mt == 2 and spec.strides == (0, N * N, N, 1) and spec.bias_dtype == _lib.FP32
    spec, _, _ = ja.classify_mask(bias.double(), False, Z, H, N, torch.float32, False)
    assert spec.bias_dtype == _lib.FP32  # float64 bias is converted


def test_shard_range_partitions_exactly():
    for total in (1, 7, 64, 512):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                lo, hi = workloads.shard_range(total, r, world)
                seen += list(range(lo, hi))
            assert seen == list(range(total))
    with pytest.raises(ValueError):
        workloads.shard_range(8, 2, 2)


def test_flop_model_headline():
    w = workloads.Workload("x", torch.bfloat16, 4, 16, 2048, 64, causal=True)
    f = workloads.flops(w, ("fwd_dual", "bwd_to"))
    assert abs(f / 1e9 - 275.0) < 0.6  # 16 MMAs x 17.19 GFLOP


def test_fp32_precision_switch():
    assert _lib.FP32_PRECISION == "3xtf32"
    x32, x16 = torch.zeros(1), torch.zeros(1, dtype=torch.bfloat16)
    assert _lib.compute_enum(x32) == _lib.FP32
    prev = ja.set_fp32_precision("tf32")
    try:
        assert prev == "3xtf32" and _lib.compute_enum(x32) == _lib.FP32_TF32 and _lib.compute_enum(x16) == _lib.BF16
        with pytest.raises(ValueError):
            ja.set_fp32_precision("fp16")
    finally:
        ja.set_fp32_precision(prev)
    assert _lib.compute_enum(x32) == _lib.FP32
