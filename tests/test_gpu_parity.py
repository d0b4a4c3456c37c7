"""GPU parity tests: the CUDA kernels, called through the C ABI of libjvpfa.so, against the float64
oracle on the same seeded inputs, against upstream's golden outputs, and through the public
Python API (both forward-AD routes, gradients through O and tO, Hessian-vector product).

Tolerances are the ones the project states for itself:
  float32           max|x - ref| / max|ref| <= 1e-5   (3xTF32 tensor-core path)
  bfloat16/float16  max|x - ref|            <= 2e-2
"""
import numpy as np
import pytest
import torch
import torch.autograd.forward_ad as fwAD

import jvp_flash_attention_b200.jvp_attention as ja
from jvp_flash_attention_b200 import _lib, workloads
from oracle import jvp_attention_oracle as orc

pytestmark = pytest.mark.gpu

FP32_REL = 1e-5
HALF_ABS = 2e-2
DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def _close(x, ref, dtype, what):
    """O and tO are held to the stated tolerances as they are.  Gradients (names starting with
    'd', 'grad', 'hvp') of 16-bit runs can exceed 1 in magnitude, where 2e-2 is below the storage
    precision of bfloat16, so their absolute tolerance scales with max(1, max|ref|)."""
    if dtype == torch.float32:
        e = orc.rel_err(x, ref)
        assert e <= FP32_REL, f"{what}: rel err {e:.3e} > {FP32_REL}"
    else:
        e = orc.max_abs_err(x, ref)
        tol = HALF_ABS
        if what[0] in "dgh":
            tol *= max(1.0, torch.as_tensor(ref).abs().max().item())
        assert e <= tol, f"{what}: abs err {e:.3e} > {tol:.3e}"


def _make(B, H, L, D, dtype, seed, n=8, tangent_std=None):
    """Seeded N(0,1) tensors q,k,v,tq,tk,tv,+2.  bfloat16 cases draw tangents from N(0, 0.1^2), the
    distribution of the bf16 benchmark configurations: with unit tangents |tO| reaches 8, where the
    spacing of bfloat16 itself (2^-5) exceeds the 2e-2 absolute tolerance."""
    if tangent_std is None:
        tangent_std = 0.1 if dtype == torch.bfloat16 else 1.0
    g = torch.Generator().manual_seed(seed)
    ts = [torch.randn(B, H, L, D, generator=g) for _ in range(n)]
    for i in (3, 4, 5):
        ts[i] = ts[i] * tangent_std
    return [t.to(dtype) for t in ts]


def _mask(kind, B, H, L, dtype, seed):
    """Returns (user-facing mask tensor or None, causal flag)."""
    g = torch.Generator().manual_seed(1000 + seed)
    if kind == "none":
        return None, False
    if kind == "causal":
        return None, True
    if kind == "kvlen":
        lens = torch.randint(L // 2, L + 1, (B,), generator=g)
        lens[0] = L // 2 + 3  # ragged inside a tile
        return (torch.arange(L)[None, :] < lens[:, None])[:, None, None, :], False
    if kind == "bool":
        m = torch.rand(B, H, L, L, generator=g) > 0.5
        m[..., 0] = True
        return m, False
    if kind == "bool_bcast":
        m = torch.rand(1, H, L, L, generator=g) > 0.3
        m[..., 0] = True
        return m, False
    if kind == "bool_keys":  # one row of keys per batch entry, not a prefix: stays a boolean mask with row stride 0
        m = torch.rand(B, 1, 1, L, generator=g) > 0.4
        m[..., 0] = False
        m[..., 1] = True
        return m, False
    if kind == "bias":
        return torch.randn(B, H, L, L, generator=g).clamp_(-5, 5).to(dtype), False
    if kind == "bias_f32_bcast":
        return torch.randn(B, 1, L, L, generator=g).clamp_(-5, 5), False
    raise ValueError(kind)


def _run_kernels(q, k, v, tq, tk, tv, go, gto, mask, causal, impl=_lib.IMPL_GENERIC, single_pass=False, scale=None):
    """fwd + preprocess + bwd through the C ABI on cuda:0.  Returns o, to, lse, mu, dq, dk, dv.
    single_pass: hand jvpfa_bwd the fp32 dQ accumulation buffer, which selects the one-pass backward."""
    dev = torch.device("cuda:0")
    B, H, L, D = q.shape
    scale = D**-0.5 if scale is None else scale
    cu = lambda x: None if x is None else x.to(dev).contiguous()  # noqa: E731
    q, k, v, tq, tk, tv, go, gto = (cu(x) for x in (q, k, v, tq, tk, tv, go, gto))
    spec, _, _ = ja.classify_mask(cu(mask), causal, B, H, L, q.dtype, False)
    o = torch.empty_like(q)
    lse = torch.empty(B, H, L, device=dev, dtype=torch.float32)
    dual = tq is not None
    to = torch.empty_like(q) if dual else None
    mu = torch.empty_like(lse) if dual else None
    _lib.fwd(q, k, v, tq, tk, tv, o, to, lse, mu, spec, scale, impl)
    dq = dk = dv = None
    if go is not None or gto is not None:
        stats = torch.empty(3, B, H, L, device=dev, dtype=torch.float32)
        use_t = gto is not None
        _lib.bwd_preprocess(o, to if use_t else None, go, gto, mu if use_t else None, stats[0], stats[1], stats[2])
        dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
        acc = torch.full(q.shape, float("nan"), device=dev, dtype=torch.float32) if single_pass else None
        _lib.bwd(q, k, v, tq if use_t else None, tk if use_t else None, tv if use_t else None, go, gto, lse,
                 mu if use_t else None, stats[0], stats[1], stats[2], dq, dk, dv, spec, scale, impl, dq_accum=acc)
    torch.cuda.synchronize()
    return o, to, lse, mu, dq, dk, dv


FWD_CASES = [
    # dtype, D, L, mask kind
    ("fp32", 64, 64, "none"), ("fp32", 64, 96, "causal"), ("fp32", 128, 64, "bias"), ("fp32", 32, 160, "kvlen"),
    ("fp32", 64, 64, "bool"), ("fp32", 128, 96, "bool_bcast"),
    ("bf16", 64, 128, "none"), ("bf16", 64, 160, "causal"), ("bf16", 128, 96, "kvlen"), ("bf16", 32, 64, "bias"),
    ("bf16", 64, 64, "bias_f32_bcast"), ("bf16", 128, 128, "causal"),
    ("fp16", 64, 128, "kvlen"), ("fp16", 128, 64, "none"), ("fp16", 64, 96, "bool"), ("fp16", 32, 96, "causal"),
]


@pytest.mark.parametrize("dt,D,L,kind", FWD_CASES)
def test_forward_and_backward_through_both_outputs(dt, D, L, kind):
    dtype = DT[dt]
    B, H = 2, 2
    q, k, v, tq, tk, tv, go, gto = _make(B, H, L, D, dtype, seed=D + L)
    mask, causal = _mask(kind, B, H, L, dtype, seed=L)
    ro, rto, rdq, rdk, rdv = orc.grads_through_both(q, k, v, tq, tk, tv, go, gto, attn_mask=mask, causal=causal)
    o, to, lse, mu, dq, dk, dv = _run_kernels(q, k, v, tq, tk, tv, go, gto, mask, causal)
    _close(o, ro, dtype, "O")
    _close(to, rto, dtype, "tO")
    _close(dq, rdq, dtype, "dq")
    _close(dk, rdk, dtype, "dk")
    _close(dv, rdv, dtype, "dv")
    r = orc.tiled_forward(q, k, v, tq, tk, tv, attn_mask=mask, causal=causal)
    assert orc.max_abs_err(lse, r["lse"]) < (1e-4 if dtype == torch.float32 else 2e-2)
    assert orc.max_abs_err(mu, r["mu"]) < (1e-4 if dtype == torch.float32 else 5e-2)


TC5_CASES = [
    # dtype, B, H, L, D, mask kind, dual
    ("bf16", 1, 1, 128, 64, "none", False), ("bf16", 1, 1, 128, 64, "none", True),
    ("bf16", 2, 2, 256, 64, "causal", True), ("fp16", 2, 2, 192, 64, "kvlen", True),
    ("bf16", 1, 2, 160, 64, "causal", True), ("bf16", 1, 2, 256, 128, "none", True),
    ("fp16", 2, 1, 320, 128, "causal", True), ("fp16", 1, 3, 96, 128, "kvlen", False),
    ("bf16", 2, 2, 1024, 64, "causal", True), ("fp16", 1, 2, 34, 64, "none", True),
    # boolean masks and bias of the element type, read row by row by the softmax threads (D = 64)
    ("bf16", 2, 2, 256, 64, "bool", True), ("fp16", 2, 3, 192, 64, "bias", True), ("bf16", 1, 2, 160, 64, "bool_bcast", True),
    ("bf16", 2, 2, 128, 64, "bias", False), ("fp16", 1, 2, 96, 64, "bool", False), ("fp16", 3, 2, 224, 64, "bool_keys", True),
    ("bf16", 2, 2, 48, 64, "bias", True),
]


@pytest.mark.parametrize("dt,B,H,L,D,kind,dual", TC5_CASES)
def test_tcgen05_forward_against_oracle_and_generic_family(dt, B, H, L, D, kind, dual):
    """The TMA + tcgen05/TMEM forward, forced through the C ABI, against the float64 oracle, and
    the register-tiled family on the same inputs (the two must agree to 16-bit rounding)."""
    dtype = DT[dt]
    q, k, v, tq, tk, tv, *_ = _make(B, H, L, D, dtype, seed=L + D)
    if not dual:
        tq = tk = tv = None
    mask, causal = _mask(kind, B, H, L, dtype, seed=L)
    o, to, lse, mu, *_ = _run_kernels(q, k, v, tq, tk, tv, None, None, mask, causal, impl=_lib.IMPL_TCGEN05)
    assert _lib.device_status() == 0, "a bounded wait inside the tcgen05 kernel gave up"
    o2, to2, lse2, mu2, *_ = _run_kernels(q, k, v, tq, tk, tv, None, None, mask, causal, impl=_lib.IMPL_GENERIC)
    if dual:
        ro, rto = orc.sdpa_jvp(q, k, v, tq, tk, tv, attn_mask=mask, causal=causal)
        _close(to, rto, dtype, "tO")
        assert orc.max_abs_err(to, to2) <= HALF_ABS
        assert orc.max_abs_err(mu, mu2) < 1e-3
    else:
        ro = orc.sdpa_primal(q, k, v, attn_mask=mask, causal=causal)
        assert to is None
    _close(o, ro, dtype, "O")
    assert orc.max_abs_err(o, o2) <= HALF_ABS
    assert orc.max_abs_err(lse, lse2) < 1e-4


PERSISTENT_FWD_CASES = [
    # dtype, B, H, L, mask kind: more query tiles than two CTAs per SM can hold at once, so that the forward's CTAs
    # walk a list of items (causal, unmasked) or, with key padding, run one item each through the same code
    ("bf16", 40, 12, 256, "causal"), ("bf16", 40, 12, 160, "none"), ("fp16", 64, 12, 192, "kvlen"), ("bf16", 6, 16, 1100, "causal"),
]


@pytest.mark.parametrize("dt,B,H,L,kind", PERSISTENT_FWD_CASES)
def test_tcgen05_forward_many_items_per_cta(dt, B, H, L, kind):
    """The persistent tcgen05 forward (D = 64, with tangents) against the register-tiled family on the same inputs
    and, for the last (batch, head) slice, against the float64 oracle."""
    dtype = DT[dt]
    q, k, v, tq, tk, tv, *_ = _make(B, H, L, 64, dtype, seed=B + L)
    mask, causal = _mask(kind, B, H, L, dtype, seed=L)
    o, to, lse, mu, *_ = _run_kernels(q, k, v, tq, tk, tv, None, None, mask, causal, impl=_lib.IMPL_TCGEN05)
    assert _lib.device_status() == 0, "a bounded wait inside the tcgen05 kernel gave up"
    o2, to2, lse2, mu2, *_ = _run_kernels(q, k, v, tq, tk, tv, None, None, mask, causal, impl=_lib.IMPL_GENERIC)
    assert orc.max_abs_err(o, o2) <= HALF_ABS and orc.max_abs_err(to, to2) <= HALF_ABS
    assert orc.max_abs_err(lse, lse2) < 1e-4 and orc.max_abs_err(mu, mu2) < 1e-3
    sl = lambda x: x[B - 1:, H - 1:]  # noqa: E731
    msl = None if mask is None else mask[min(B, mask.shape[0]) - 1:, min(H, mask.shape[1]) - 1:]
    ro, rto = orc.sdpa_jvp(sl(q), sl(k), sl(v), sl(tq), sl(tk), sl(tv), attn_mask=msl, causal=causal)
    _close(sl(o), ro, dtype, "O")
    _close(sl(to), rto, dtype, "tO")


PERSISTENT_CASES = [
    # cotangents, mask kind, dtype, B, H, L: more work items than a B200 has SMs, so that every CTA of
    # the persistent backward walks several items; short items (1 to 5 sub-tiles of 32 rows), odd
    # sub-tile counts, items without any live key, all three cotangent modes
    ("gt", "kvlen", "bf16", 40, 12, 96), ("both", "kvlen", "fp16", 40, 12, 128), ("go", "causal", "bf16", 40, 12, 160),
    ("gt", "none", "bf16", 64, 12, 32), ("both", "none", "bf16", 8, 12, 1024), ("gt", "causal", "fp16", 24, 8, 224),
    # boolean masks and bias, fetched by the elementwise threads
    ("both", "bool", "bf16", 2, 3, 256), ("gt", "bias", "fp16", 2, 2, 192), ("go", "bool_bcast", "bf16", 2, 2, 160),
    ("gt", "bool_keys", "bf16", 3, 2, 224), ("both", "bias", "bf16", 40, 12, 96), ("gt", "bool", "fp16", 20, 12, 128),
    ("go", "bias", "bf16", 1, 2, 48),
]


@pytest.mark.parametrize("cot,kind,dt,B,H,L", PERSISTENT_CASES)
def test_tcgen05_backward_many_items_per_cta(cot, kind, dt, B, H, L):
    """The persistent tcgen05 backward (D = 64) against the register-tiled family on the same inputs,
    in shapes where each CTA processes a list of work items and the barrier phases carry over from
    one item to the next.  The bounded waits inside the kernel must not have given up."""
    dtype = DT[dt]
    q, k, v, tq, tk, tv, go, gto = _make(B, H, L, 64, dtype, seed=B + L)
    go = go if cot in ("go", "both") else None
    gto = gto if cot in ("gt", "both") else None
    mask, causal = _mask(kind, B, H, L, dtype, seed=L)
    *_, dq, dk, dv = _run_kernels(q, k, v, tq, tk, tv, go, gto, mask, causal, impl=_lib.IMPL_TCGEN05)
    assert _lib.device_status() == 0, "a bounded wait inside the tcgen05 kernel gave up"
    *_, dq2, dk2, dv2 = _run_kernels(q, k, v, tq, tk, tv, go, gto, mask, causal, impl=_lib.IMPL_GENERIC)
    for name, a, b in (("dq", dq, dq2), ("dk", dk, dk2), ("dv", dv, dv2)):
        assert torch.isfinite(a.float()).all(), name
        _close(a, b.float(), dtype, name)
    # one (batch, head) slice against the float64 oracle
    sl = lambda x: None if x is None else x[B - 1:, H - 1:]  # noqa: E731
    msl = None if mask is None else mask[min(B, mask.shape[0]) - 1:, min(H, mask.shape[1]) - 1:]
    _, _, rdq, rdk, rdv = orc.grads_through_both(sl(q), sl(k), sl(v), sl(tq), sl(tk), sl(tv), sl(go), sl(gto),
                                                 attn_mask=msl, causal=causal)
    _close(dq[B - 1:, H - 1:], rdq, dtype, "dq")
    _close(dk[B - 1:, H - 1:], rdk, dtype, "dk")
    _close(dv[B - 1:, H - 1:], rdv, dtype, "dv")


SINGLE_PASS_CASES = [c for c in PERSISTENT_CASES if c[1] in ("none", "causal", "kvlen")] + [
    # ragged lengths (last key tile and last query sub-tile partly out of range), one sub-tile, odd sub-tile counts
    ("gt", "causal", "bf16", 2, 3, 34), ("both", "none", "fp16", 3, 2, 200), ("go", "kvlen", "bf16", 2, 2, 328),
    ("gt", "none", "bf16", 1, 1, 64), ("both", "causal", "bf16", 5, 31, 448), ("gt", "kvlen", "fp16", 9, 17, 576),
    # boolean masks without tile bitmaps (full, broadcast over the batch, one row of keys per batch entry)
    ("gt", "bool", "bf16", 2, 3, 256), ("both", "bool_bcast", "fp16", 2, 4, 320), ("go", "bool_keys", "bf16", 3, 2, 192),
    ("both", "bool", "bf16", 3, 20, 1024),
    # additive bias of the tensors' type, backward through O alone
    ("go", "bias", "bf16", 2, 3, 256), ("go", "bias", "fp16", 3, 5, 448),
]


@pytest.mark.parametrize("cot,kind,dt,B,H,L", SINGLE_PASS_CASES)
def test_single_pass_backward_against_two_launch_and_oracle(cot, kind, dt, B, H, L):
    """The one-pass backward (every score tile formed once, dQ summed into the caller's fp32 buffer) against the
    two-launch tcgen05 kernels on the same inputs, and one (batch, head) slice against the float64 oracle.  The
    accumulation buffer is handed over full of NaN: the library must not rely on its contents."""
    dtype = DT[dt]
    q, k, v, tq, tk, tv, go, gto = _make(B, H, L, 64, dtype, seed=B + L)
    go = go if cot in ("go", "both") else None
    gto = gto if cot in ("gt", "both") else None
    mask, causal = _mask(kind, B, H, L, dtype, seed=L)
    *_, dq, dk, dv = _run_kernels(q, k, v, tq, tk, tv, go, gto, mask, causal, impl=_lib.IMPL_TCGEN05, single_pass=True)
    assert _lib.device_status() == 0, "a bounded wait inside the tcgen05 kernel gave up"
    *_, dq2, dk2, dv2 = _run_kernels(q, k, v, tq, tk, tv, go, gto, mask, causal, impl=_lib.IMPL_TCGEN05)
    for name, a, b in (("dq", dq, dq2), ("dk", dk, dk2), ("dv", dv, dv2)):
        assert torch.isfinite(a.float()).all(), name
        _close(a, b.float(), dtype, name)
    sl = lambda x: None if x is None else x[B - 1:, H - 1:]  # noqa: E731
    msl = None if mask is None else mask[min(B, mask.shape[0]) - 1:, min(H, mask.shape[1]) - 1:]
    _, _, rdq, rdk, rdv = orc.grads_through_both(sl(q), sl(k), sl(v), sl(tq), sl(tk), sl(tv), sl(go), sl(gto),
                                                 attn_mask=msl, causal=causal)
    _close(dq[B - 1:, H - 1:], rdq, dtype, "dq")
    _close(dk[B - 1:, H - 1:], rdk, dtype, "dk")
    _close(dv[B - 1:, H - 1:], rdv, dtype, "dv")


def test_tcgen05_dispatch_rules():
    """AUTO takes the tcgen05 kernels for 16-bit, D in {64,128} (D = 64: positive softmax scale), none / causal / key
    padding, and boolean masks or bias of the element type whose rows can be read as 16-byte pieces."""
    import ctypes as C

    lib = _lib.load()
    x = torch.zeros(1, 1, 64, 64, device="cuda:0", dtype=torch.bfloat16)
    lse = torch.zeros(1, 1, 64, device="cuda:0")
    a = _lib.FwdArgs()
    a.struct_size = C.sizeof(_lib.FwdArgs)
    a.dtype, a.B, a.H, a.L, a.D = _lib.BF16, 1, 1, 64, 64
    a.q = a.k = a.v = a.o = x.data_ptr()
    a.lse = lse.data_ptr()
    a.sm_scale = 0.125
    assert lib.jvpfa_fwd_uses_tcgen05(C.byref(a)) == 1
    a.sm_scale = -0.125  # the D = 64 kernel takes row maxima before scaling: positive scales only
    assert lib.jvpfa_fwd_uses_tcgen05(C.byref(a)) == 0
    a.D = 128
    assert lib.jvpfa_fwd_uses_tcgen05(C.byref(a)) == 1
    a.D, a.sm_scale = 64, 0.125
    a.impl = _lib.IMPL_GENERIC
    assert lib.jvpfa_fwd_uses_tcgen05(C.byref(a)) == 0
    a.impl = _lib.IMPL_AUTO
    a.D = 32
    assert lib.jvpfa_fwd_uses_tcgen05(C.byref(a)) == 0
    a.impl = _lib.IMPL_TCGEN05
    assert lib.jvpfa_fwd(C.byref(a), None) == -9  # forcing an ineligible shape is an error, not a fallback
    a.impl, a.D, a.dtype = _lib.IMPL_AUTO, 64, _lib.FP32
    assert lib.jvpfa_fwd_uses_tcgen05(C.byref(a)) == 0
    # boolean masks / bias: D = 64, unit key stride, 16-byte aligned rows, L % 16 == 0, bias of the element type
    a.dtype, a.sm_scale = _lib.FP16, 0.125
    a.mask.kind = _lib.MASK_BOOL
    a.mask.ptr = x.data_ptr()
    a.mask.stride[:] = [0, 0, 64, 1]
    assert lib.jvpfa_fwd_uses_tcgen05(C.byref(a)) == 1
    a.mask.stride[:] = [0, 0, 128, 2]
    assert lib.jvpfa_fwd_uses_tcgen05(C.byref(a)) == 0
    a.mask.stride[:] = [0, 0, 72, 1]
    assert lib.jvpfa_fwd_uses_tcgen05(C.byref(a)) == 0
    a.mask.stride[:] = [0, 0, 64, 1]
    a.mask.ptr = x.data_ptr() + 8
    assert lib.jvpfa_fwd_uses_tcgen05(C.byref(a)) == 0
    a.mask.ptr = x.data_ptr()
    a.mask.kind, a.mask.bias_dtype = _lib.MASK_BIAS, _lib.FP16
    assert lib.jvpfa_fwd_uses_tcgen05(C.byref(a)) == 1
    a.mask.bias_dtype = _lib.FP32
    assert lib.jvpfa_fwd_uses_tcgen05(C.byref(a)) == 0
    a.mask.bias_dtype, a.D = _lib.FP16, 128
    assert lib.jvpfa_fwd_uses_tcgen05(C.byref(a)) == 1
    a.L = 72  # not a multiple of 16: rows cannot be read as 16-byte pieces
    assert lib.jvpfa_fwd_uses_tcgen05(C.byref(a)) == 0


@pytest.mark.parametrize("dt", ["fp32", "bf16"])
@pytest.mark.parametrize("which", ["o_only", "to_only"])
def test_single_cotangent_modes(dt, which):
    dtype = DT[dt]
    B, H, L, D = 1, 3, 128, 64
    q, k, v, tq, tk, tv, go, gto = _make(B, H, L, D, dtype, seed=7)
    go_, gto_ = (go, None) if which == "o_only" else (None, gto)
    ro, rto, rdq, rdk, rdv = orc.grads_through_both(q, k, v, tq, tk, tv, go_, gto_, causal=True)
    o, to, _, _, dq, dk, dv = _run_kernels(q, k, v, tq, tk, tv, go_, gto_, None, True)
    for x, r_, n in ((o, ro, "O"), (to, rto, "tO"), (dq, rdq, "dq"), (dk, rdk, "dk"), (dv, rdv, "dv")):
        _close(x, r_, dtype, n)


def test_primal_only_forward_matches_dual_primal():
    q, k, v, tq, tk, tv, *_ = _make(2, 2, 96, 64, torch.float32, seed=9)
    o1, to1, lse1, mu1, *_ = _run_kernels(q, k, v, None, None, None, None, None, None, False)
    o2, *_ = _run_kernels(q, k, v, tq, tk, tv, None, None, None, False)
    assert to1 is None and mu1 is None
    assert torch.equal(o1, o2)
    _close(o1, orc.sdpa_primal(q, k, v), torch.float32, "O")


def test_fully_masked_rows_give_zero_and_no_nan():
    B, H, L, D = 1, 2, 64, 64
    q, k, v, tq, tk, tv, go, gto = _make(B, H, L, D, torch.float32, seed=3)
    mask = torch.rand(B, H, L, L, generator=torch.Generator().manual_seed(1)) > 0.5
    mask[0, 0, 5] = False
    mask[0, 1, 40:48] = False
    ro, rto, rdq, rdk, rdv = orc.grads_through_both(q, k, v, tq, tk, tv, go, gto, attn_mask=mask)
    o, to, lse, mu, dq, dk, dv = _run_kernels(q, k, v, tq, tk, tv, go, gto, mask, False)
    assert o[0, 0, 5].abs().max() == 0 and to[0, 1, 40:48].abs().max() == 0
    assert torch.isinf(lse[0, 0, 5])
    for x, r_, n in ((o, ro, "O"), (to, rto, "tO"), (dq, rdq, "dq"), (dk, rdk, "dk"), (dv, rdv, "dv")):
        assert torch.isfinite(x).all(), n
        _close(x, r_, torch.float32, n)
    # the same rows through the tcgen05 forward (16-bit inputs)
    h = lambda x: x.to(torch.bfloat16)  # noqa: E731
    o, to, lse, mu, *_ = _run_kernels(h(q), h(k), h(v), h(tq), h(tk), h(tv), None, None, mask, False, impl=_lib.IMPL_TCGEN05)
    assert _lib.device_status() == 0
    assert o[0, 0, 5].abs().max() == 0 and to[0, 1, 40:48].abs().max() == 0 and torch.isinf(lse[0, 0, 5])
    assert torch.isfinite(o).all() and torch.isfinite(to).all() and torch.isfinite(mu).all()
    ro, rto = orc.sdpa_jvp(h(q), h(k), h(v), h(tq), h(tk), h(tv), attn_mask=mask)
    _close(o, ro, torch.bfloat16, "O (tcgen05)")
    _close(to, rto, torch.bfloat16, "tO (tcgen05)")


def test_kvlen_zero_and_full():
    B, H, L, D = 3, 1, 64, 64
    q, k, v, tq, tk, tv, go, gto = _make(B, H, L, D, torch.float32, seed=4)
    lens = torch.tensor([0, 64, 1], dtype=torch.int32)
    dev = torch.device("cuda:0")
    spec = _lib.MaskSpec(_lib.MASK_KVLEN, lens.to(dev))
    cu = lambda x: x.to(dev)  # noqa: E731
    o, to = torch.empty_like(cu(q)), torch.empty_like(cu(q))
    lse = torch.empty(B, H, L, device=dev)
    mu = torch.empty_like(lse)
    _lib.fwd(cu(q), cu(k), cu(v), cu(tq), cu(tk), cu(tv), o, to, lse, mu, spec, D**-0.5, _lib.IMPL_GENERIC)
    torch.cuda.synchronize()
    assert o[0].abs().max() == 0 and to[0].abs().max() == 0
    ro, rto = orc.sdpa_jvp(q[1:2], k[1:2], v[1:2], tq[1:2], tk[1:2], tv[1:2])
    _close(o[1:2], ro, torch.float32, "O full")
    _close(to[1:2], rto, torch.float32, "tO full")
    # one valid key: O is that value row, tO is its tangent row
    _close(o[2], v[2, :, :1].expand(-1, L, -1), torch.float32, "O one key")
    _close(to[2], tv[2, :, :1].expand(-1, L, -1), torch.float32, "tO one key")


GOLDEN = ["none_L64_D32", "causal_L64_D32", "bool_L64_D32", "additive_L64_D32", "none_L128_D64", "causal_L128_D64"]


@pytest.mark.parametrize("name", GOLDEN)
def test_against_upstream_golden_outputs(golden_dir, name):
    """Same inputs as upstream's own kernels saw (interpreter run, fp32): forward-dual and the
    backward of sum(O*w).  2e-5 = this library's 1e-5 plus upstream's own fp32 rounding."""
    z = np.load(golden_dir / f"upstream_{name}.npz")
    t = {k_: torch.from_numpy(z[k_]) for k_ in z.files if k_ not in ("causal", "mask_kind")}
    o, to, _, _, dq, dk, dv = _run_kernels(t["q"], t["k"], t["v"], t["tq"], t["tk"], t["tv"], t["w"], None,
                                           t.get("mask"), bool(z["causal"]))
    for got, key in ((o, "o"), (to, "to"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        e = orc.rel_err(got, t[key])
        assert e <= 2e-5, f"{key}: {e:.3e}"


@pytest.mark.parametrize("dt", ["fp32", "bf16", "fp16"])
def test_float_mask_against_torch_sdpa_golden(golden_dir, dt):
    """A general float mask (not {0, -100}) means softmax(scale * Q K^T + mask) in forward and backward: the fixture is
    PyTorch's own scaled_dot_product_attention in float64 (tests/golden/make_sdpa_bias_golden.py).  fp32 on the
    register-tiled family, 16-bit on the tcgen05 kernels (bias of the element type)."""
    dtype = DT[dt]
    z = np.load(golden_dir / "sdpa_bias_L64_D32.npz")
    t = {k_: torch.from_numpy(z[k_]) for k_ in z.files}
    if dtype != torch.float32:  # the tcgen05 kernels need D = 64: pad the head dimension with zeros (changes nothing
        # but the scale, which is passed explicitly)
        pad = lambda x: torch.nn.functional.pad(x, (0, 32))  # noqa: E731
        ins = [pad(t[n]).to(dtype) for n in ("q", "k", "v", "tq", "tk", "tv", "w1", "w2")]
    else:
        ins = [t[n].to(dtype) for n in ("q", "k", "v", "tq", "tk", "tv", "w1", "w2")]
    q, k, v, tq, tk, tv, w1, w2 = ins
    bias = t["bias"].to(dtype)
    o, to, _, _, dq, dk, dv = _run_kernels(q, k, v, tq, tk, tv, w1, w2, bias, False, scale=32 ** -0.5,
                                           impl=_lib.IMPL_AUTO)
    assert _lib.device_status() == 0
    for got, key in ((o, "o"), (to, "to"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        ref = t[key]
        got = got[..., :32]
        if dtype == torch.float32:
            assert orc.rel_err(got, ref) <= FP32_REL, key
        else:
            # the inputs themselves were rounded to 16 bit: compare with the oracle on the rounded inputs instead of the
            # float64 fixture for the tight bound, and with the fixture for the meaning of the mask
            assert orc.max_abs_err(got, ref) <= 6e-2 * max(1.0, ref.abs().max().item()), key


# ------------------------------------------------------------------------------------------------
# Public API
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("route", ["func_jvp", "fwad"])
@pytest.mark.parametrize("dt,kind", [("fp32", "none"), ("bf16", "causal"), ("fp16", "kvlen"), ("fp32", "bias")])
def test_api_routes_and_grads_through_both(route, dt, kind):
    dtype = DT[dt]
    B, H, L, D = 2, 2, 128, 64
    q, k, v, tq, tk, tv, w1, w2 = _make(B, H, L, D, dtype, seed=21)
    mask, causal = _mask(kind, B, H, L, dtype, seed=2)
    ro, rto, rdq, rdk, rdv = orc.grads_through_both(q, k, v, tq, tk, tv, w1, w2, attn_mask=mask, causal=causal)
    dev = "cuda:0"
    a = [x.to(dev).requires_grad_() for x in (q, k, v)]
    t = [x.to(dev) for x in (tq, tk, tv)]
    m = None if mask is None else mask.to(dev)
    fn = lambda q_, k_, v_: ja.JVPAttn.fwd_dual(q_, k_, v_, attn_mask=m, causal=causal)  # noqa: E731
    if route == "func_jvp":
        o, to = torch.func.jvp(fn, tuple(a), tuple(t))
    else:
        with fwAD.dual_level(), torch.enable_grad():
            out = fn(*[fwAD.make_dual(x, y) for x, y in zip(a, t)])
            o, to = fwAD.unpack_dual(out)
    assert to.requires_grad
    g = torch.autograd.grad((o.float() * w1.to(dev).float()).sum() + (to.float() * w2.to(dev).float()).sum(), a)
    _close(o, ro, dtype, "O")
    _close(to, rto, dtype, "tO")
    for x, r_, n in zip(g, (rdq, rdk, rdv), ("dq", "dk", "dv")):
        _close(x, r_, dtype, n)


def test_api_hvp_with_bias_fp32():
    B, H, L, D = 1, 2, 128, 128
    q, k, v, w, vd, *_ = _make(B, H, L, D, torch.float32, seed=31)
    bias = torch.randn(B, H, L, L, generator=torch.Generator().manual_seed(3)).clamp_(-5, 5)
    ro, rg1, rh = orc.hvp_q(q, k, v, w, vd, attn_mask=bias)
    dev = "cuda:0"
    q1 = q.to(dev).requires_grad_()
    o = ja.attention(q1, k.to(dev), v.to(dev), attn_mask=bias.to(dev))
    (g1,) = torch.autograd.grad((o * w.to(dev)).sum(), q1, create_graph=True)
    (h,) = torch.autograd.grad((g1 * vd.to(dev)).sum(), q1)
    _close(o, ro, torch.float32, "O")
    _close(g1, rg1, torch.float32, "grad")
    _close(h, rh, torch.float32, "hvp")


def test_api_tangent_input_grads():
    B, H, L, D = 1, 2, 64, 64
    q, k, v, tq, tk, tv, w1, w2 = _make(B, H, L, D, torch.float32, seed=41)
    ref_in = [x.double().requires_grad_() for x in (q, k, v, tq, tk, tv)]
    _, rto = orc.sdpa_jvp(*ref_in)
    rg = torch.autograd.grad((rto * w2.double()).sum(), ref_in)
    dev = "cuda:0"
    a = [x.to(dev).requires_grad_() for x in (q, k, v, tq, tk, tv)]
    o, to = torch.func.jvp(ja.JVPAttn.fwd_dual, tuple(a[:3]), tuple(a[3:]))
    g = torch.autograd.grad((to * w2.to(dev)).sum(), a)
    for x, r_ in zip(g, rg):
        _close(x, r_, torch.float32, "grad")


def test_api_is_deterministic_and_does_not_touch_inputs():
    q, k, v, tq, tk, tv, *_ = _make(2, 2, 128, 64, torch.bfloat16, seed=51)
    dev = "cuda:0"
    a = [x.to(dev) for x in (q, k, v)]
    keep = [x.clone() for x in a]
    o1, to1 = torch.func.jvp(ja.JVPAttn.fwd_dual, tuple(a), tuple(x.to(dev) for x in (tq, tk, tv)))
    o2, to2 = torch.func.jvp(ja.JVPAttn.fwd_dual, tuple(a), tuple(x.to(dev) for x in (tq, tk, tv)))
    assert torch.equal(o1, o2) and torch.equal(to1, to2)
    assert all(torch.equal(x, y) for x, y in zip(a, keep))


# ------------------------------------------------------------------------------------------------
# Full-size configurations: sampled heads against the oracle + size-independent properties
# ------------------------------------------------------------------------------------------------
def _loss_grads_api(w, dev="cuda:0"):
    t = {k_: v_.to(dev) for k_, v_ in w.tensors.items() if isinstance(v_, torch.Tensor)}
    a = [t[n].requires_grad_() for n in ("q", "k", "v")]
    m = t.get("mask")
    o, to = torch.func.jvp(lambda q_, k_, v_: ja.JVPAttn.fwd_dual(q_, k_, v_, attn_mask=m, causal=w.causal),
                           tuple(a), (t["tq"], t["tk"], t["tv"]))
    return t, a, o, to


def test_config2_full_size_sampled_heads_and_linearity():
    """bf16 causal B4 H16 L2048 D64, loss = mean((tO - target)^2)."""
    w = workloads.make_workload("c2_bf16_causal")
    t, a, o, to = _loss_grads_api(w)
    loss = ((to.float() - t["target"].float()) ** 2).mean()
    g = torch.autograd.grad(loss, a)
    n = to.numel()
    for (b, h) in ((0, 0), (0, 9), (1, 3), (1, 14), (2, 0), (2, 7), (3, 5), (3, 15)):
        sl = lambda x: x[b:b + 1, h:h + 1]  # noqa: E731
        cpu = {k_: sl(v_) for k_, v_ in w.tensors.items()}
        ro, rto = orc.sdpa_jvp(cpu["q"], cpu["k"], cpu["v"], cpu["tq"], cpu["tk"], cpu["tv"], causal=True)
        gto = 2.0 * (sl(to).detach().cpu().double() - cpu["target"].double()) / n
        _, _, rdq, rdk, rdv = orc.grads_through_both(cpu["q"], cpu["k"], cpu["v"], cpu["tq"], cpu["tk"], cpu["tv"],
                                                     None, gto, causal=True)
        _close(sl(o), ro, torch.bfloat16, "O")
        _close(sl(to), rto, torch.bfloat16, "tO")
        # gradients of a mean over 8.4M elements are ~1e-7: compare relative to their scale
        for x, r_, nme in zip(g, (rdq, rdk, rdv), ("dq", "dk", "dv")):
            e = orc.rel_err(sl(x), r_)
            assert e < 3e-2, f"{nme} rel {e:.3e}"
    # linearity of tO in the tangents: tO(2t) == 2 tO(t) (exact in binary floating point)
    o2, to2 = torch.func.jvp(lambda q_, k_, v_: ja.JVPAttn.fwd_dual(q_, k_, v_, causal=True),
                             tuple(x.detach() for x in a), (2 * t["tq"], 2 * t["tk"], 2 * t["tv"]))
    assert torch.equal(o2, o.detach())
    assert (to2.float() - 2 * to.detach().float()).abs().max().item() <= 2e-2
    # Every one of the 64 heads, all five results: the tcgen05 kernels of the benchmark shape (whose persistent work
    # lists depend on the shape) against the register-tiled family, through the C ABI, with the cotangent of the loss.
    gto = (2.0 * (to.detach().float() - t["target"].float()) / n).to(torch.bfloat16)
    c = w.tensors
    res = {}
    for impl, single in ((_lib.IMPL_TCGEN05, True), (_lib.IMPL_TCGEN05, False), (_lib.IMPL_GENERIC, False)):
        res[(impl, single)] = _run_kernels(c["q"], c["k"], c["v"], c["tq"], c["tk"], c["tv"], None, gto.cpu(), None, True,
                                           impl=impl, single_pass=single)
        assert _lib.device_status() == 0
    ref = res[(_lib.IMPL_GENERIC, False)]
    for key in ((_lib.IMPL_TCGEN05, True), (_lib.IMPL_TCGEN05, False)):
        got = res[key]
        for idx, nme in ((0, "O"), (1, "tO")):
            _close(got[idx], ref[idx].float(), torch.bfloat16, nme)
        for idx, nme in ((4, "dq"), (5, "dk"), (6, "dv")):
            e = orc.rel_err(got[idx], ref[idx].float())
            assert e < 3e-2, f"{nme} all heads, tcgen05 {key} vs register-tiled: rel {e:.3e}"


def test_config3_full_size_keypad_sampled_heads():
    """fp16 B8 H12 L1024 D64 key padding (B,1,1,L), loss through both outputs."""
    w = workloads.make_workload("c3_fp16_keypad")
    t, a, o, to = _loss_grads_api(w)
    loss = (o.float() * t["w1"].float()).sum() + (to.float() * t["w2"].float()).sum()
    g = torch.autograd.grad(loss, a)
    lens = w.tensors["kv_len"]
    for (b, h) in ((0, 0), (7, 11)):
        sl = lambda x: x[b:b + 1, h:h + 1]  # noqa: E731
        c = {k_: sl(v_) for k_, v_ in w.tensors.items() if k_ not in ("kv_len", "mask")}
        mask = w.tensors["mask"][b:b + 1]
        ro, rto, rdq, rdk, rdv = orc.grads_through_both(c["q"], c["k"], c["v"], c["tq"], c["tk"], c["tv"], c["w1"],
                                                        c["w2"], attn_mask=mask)
        _close(sl(o), ro, torch.float16, "O")
        _close(sl(to), rto, torch.float16, "tO")
        # cotangents are N(0,1), tangent grads reach O(10): compare relative to scale (fp16 eps ~1e-3)
        for x, r_, nme in zip(g, (rdq, rdk, rdv), ("dq", "dk", "dv")):
            e = orc.rel_err(sl(x), r_)
            assert e < 1e-2, f"{nme} rel {e:.3e}"
        # padded keys get exactly zero gradient
        assert sl(g[1])[0, 0, int(lens[b]):].abs().max().item() == 0 if lens[b] < w.L else True


def test_config1_and_config4_reduced_checks():
    """C1 (fp32 B2 H4 L256 D64, loss sum(O)+sum(tO)) in full; C4 (fp32 D128 bias, HVP) at L=256."""
    w = workloads.make_workload("c1_fp32_plumbing")
    t, a, o, to = _loss_grads_api(w)
    g = torch.autograd.grad(o.sum() + to.sum(), a)
    c = w.tensors
    ones = torch.ones_like(c["q"])
    ro, rto, rdq, rdk, rdv = orc.grads_through_both(c["q"], c["k"], c["v"], c["tq"], c["tk"], c["tv"], ones, ones)
    for x, r_, nme in zip((o, to, *g), (ro, rto, rdq, rdk, rdv), ("O", "tO", "dq", "dk", "dv")):
        _close(x, r_, torch.float32, nme)

    w4 = workloads.make_workload("c4_fp32_bias_hvp", L=256)
    c = w4.tensors
    ro, rto = orc.sdpa_jvp(c["q"], c["k"], c["v"], c["tq"], c["tk"], c["tv"], attn_mask=c["mask"])
    _, _, rh = orc.hvp_q(c["q"], c["k"], c["v"], c["w"], c["v_dir"], attn_mask=c["mask"])
    dev = "cuda:0"
    d = {k_: v_.to(dev) for k_, v_ in c.items()}
    o, to = torch.func.jvp(lambda q_, k_, v_: ja.JVPAttn.fwd_dual(q_, k_, v_, attn_mask=d["mask"]),
                           (d["q"], d["k"], d["v"]), (d["tq"], d["tk"], d["tv"]))
    q1 = d["q"].clone().requires_grad_()
    o1 = ja.attention(q1, d["k"], d["v"], attn_mask=d["mask"])
    (g1,) = torch.autograd.grad((o1 * d["w"]).sum(), q1, create_graph=True)
    (h,) = torch.autograd.grad((g1 * d["v_dir"]).sum(), q1)
    _close(o, ro, torch.float32, "O")
    _close(to, rto, torch.float32, "tO")
    _close(h, rh, torch.float32, "hvp")


def test_library_rejects_bad_arguments_without_launching():
    import ctypes as C

    lib = _lib.load()
    a = _lib.FwdArgs()
    a.struct_size = 3
    assert lib.jvpfa_fwd(C.byref(a), None) == -7  # JVPFA_ERR_STRUCT
    a.struct_size = C.sizeof(_lib.FwdArgs)
    a.dtype, a.B, a.H, a.L, a.D = _lib.FP32, 1, 1, 64, 48
    assert lib.jvpfa_fwd(C.byref(a), None) == -2  # unsupported head dim
    a.D = 64
    assert lib.jvpfa_fwd(C.byref(a), None) == -1  # null pointers
    assert lib.jvpfa_fwd(None, None) == -1
    x = torch.zeros(1, 1, 64, 64, device="cuda:0")
    lse = torch.zeros(1, 1, 64, device="cuda:0")
    a.q, a.k, a.v, a.o, a.lse = x.data_ptr(), x.data_ptr(), x.data_ptr() + 4, x.data_ptr(), lse.data_ptr()
    assert lib.jvpfa_fwd(C.byref(a), None) == -8  # misaligned
    a.v = x.data_ptr()
    a.tq = x.data_ptr()
    assert lib.jvpfa_fwd(C.byref(a), None) == -1  # partial tangent set
    a.tq = None
    a.mask.kind = _lib.MASK_BOOL
    assert lib.jvpfa_fwd(C.byref(a), None) == -4  # mask without pointer
    assert b"mask" in lib.jvpfa_strerror(-4)


def test_calls_fail_loudly_after_a_wait_gave_up_until_the_status_is_cleared():
    """A kernel thread that gives up a bounded wait leaves its code in the status word and in the host-visible mirror.
    The failure is made on the host here (jvpfa_device_status_inject writes exactly those two words; no wait runs out
    on the GPU): from then on every call that would launch a tcgen05 kernel is refused with JVPFA_ERR_DEVICE_STATUS,
    through the C ABI and through the Python API, the register-tiled family still runs, and after
    jvpfa_device_status(clear=1) everything works again."""
    dev = "cuda:0"
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(1, 2, 128, 64, generator=g).to(torch.bfloat16).to(dev) for _ in range(3))
    assert _lib.device_status() == 0
    ref = ja.attention(q, k, v, causal=True)
    _lib.device_status_inject(7)
    try:
        with pytest.raises(RuntimeError, match="gave up a bounded wait"):
            ja.attention(q, k, v, causal=True)
        o, lse = torch.empty_like(q), torch.empty(1, 2, 128, device=dev)
        with pytest.raises(RuntimeError, match=r"\[-11\]"):
            _lib.fwd(q, k, v, None, None, None, o, None, lse, None, _lib.MaskSpec(_lib.MASK_CAUSAL), 0.125, _lib.IMPL_TCGEN05)
        # the other kernel family neither reads nor sets the word
        _lib.fwd(q, k, v, None, None, None, o, None, lse, None, _lib.MaskSpec(_lib.MASK_CAUSAL), 0.125, _lib.IMPL_GENERIC)
        torch.cuda.synchronize()
        assert (o.float() - ref.float()).abs().max().item() < 2e-2
        assert _lib.device_status(clear=False) == 7
    finally:
        assert _lib.device_status(clear=True) in (0, 7)
    assert _lib.device_status() == 0
    again = ja.attention(q, k, v, causal=True)
    torch.cuda.synchronize()
    assert torch.equal(again, ref)


def test_config4_full_size_bias_hvp_sampled_heads():
    """fp32 B2 H8 L1024 D128 with a (B,H,L,L) bias: primal + tangent forward and the Hessian-vector
    product d/dq <d/dq sum(O*w), v_dir>; two (batch, head) slices against the float64 oracle."""
    w = workloads.make_workload("c4_fp32_bias_hvp")
    c = w.tensors
    dev = "cuda:0"
    d = {k_: v_.to(dev) for k_, v_ in c.items()}
    o, to = torch.func.jvp(lambda q_, k_, v_: ja.JVPAttn.fwd_dual(q_, k_, v_, attn_mask=d["mask"]),
                           (d["q"], d["k"], d["v"]), (d["tq"], d["tk"], d["tv"]))
    q1 = d["q"].clone().requires_grad_()
    o1 = ja.attention(q1, d["k"], d["v"], attn_mask=d["mask"])
    (g1,) = torch.autograd.grad((o1 * d["w"]).sum(), q1, create_graph=True)
    (h,) = torch.autograd.grad((g1 * d["v_dir"]).sum(), q1)
    for (b, hh) in ((0, 0), (1, 7)):
        sl = lambda x: x[b:b + 1, hh:hh + 1]  # noqa: E731
        cc = {k_: sl(v_) for k_, v_ in c.items()}
        ro, rto = orc.sdpa_jvp(cc["q"], cc["k"], cc["v"], cc["tq"], cc["tk"], cc["tv"], attn_mask=cc["mask"])
        _, rg1, rh = orc.hvp_q(cc["q"], cc["k"], cc["v"], cc["w"], cc["v_dir"], attn_mask=cc["mask"])
        _close(sl(o), ro, torch.float32, "O")
        _close(sl(to), rto, torch.float32, "tO")
        _close(sl(g1), rg1, torch.float32, "grad")
        _close(sl(h), rh, torch.float32, "hvp")


def test_config5_shard_long_sequence_sampled_head():
    """bf16 L8192 D128 non-causal: the shard a rank would own (here 4 of the 512 (batch, head) units,
    generated per head as on any rank), fwd_dual + backward through both outputs; head 0 against the
    float64 oracle, and linearity of tO in the tangents on the whole shard."""
    w = workloads.make_workload("c5_bf16_long", heads=(0, 4))
    t = {k_: v_.to("cuda:0") for k_, v_ in w.tensors.items()}
    a = [t[n].requires_grad_() for n in ("q", "k", "v")]
    o, to = torch.func.jvp(ja.JVPAttn.fwd_dual, tuple(a), (t["tq"], t["tk"], t["tv"]))
    g = torch.autograd.grad((o.float() * t["w1"].float()).sum() + (to.float() * t["w2"].float()).sum(), a)
    assert _lib.device_status() == 0
    for hd in (0, 3):
        c = {k_: v_[:, hd:hd + 1] for k_, v_ in w.tensors.items()}
        ro, rto, rdq, rdk, rdv = orc.grads_through_both(c["q"], c["k"], c["v"], c["tq"], c["tk"], c["tv"], c["w1"], c["w2"])
        _close(o[:, hd:hd + 1], ro, torch.bfloat16, "O")
        _close(to[:, hd:hd + 1], rto, torch.bfloat16, "tO")
        for x, r_, nme in zip(g, (rdq, rdk, rdv), ("dq", "dk", "dv")):
            _close(x[:, hd:hd + 1], r_, torch.bfloat16, nme)
    o2, to2 = torch.func.jvp(ja.JVPAttn.fwd_dual, tuple(x.detach() for x in a), (2 * t["tq"], 2 * t["tk"], 2 * t["tv"]))
    assert torch.equal(o2, o.detach())
    assert (to2.float() - 2 * to.detach().float()).abs().max().item() <= 2e-2


@pytest.mark.parametrize("dt", ["bf16", "fp16", "fp32"])
def test_reference_harness_grid_short_lengths(dt):
    """The reference script's own check (tests/harness.py: same grid, seeds, comparator SDPA-MATH in the working dtype,
    tolerances 3.2e-2 / 4e-3 / 2.35e-2) for L <= 128, without its timing part."""
    from tests import harness

    rows = harness.run(DT[dt], 128, bench=False)
    assert len(rows) == 12
    bad = [(r["seq_len"], r["mask"], r["causal"], r["max_error"]) for r in rows if not r["pass"]]
    assert not bad, bad


@pytest.mark.parametrize("dt,kind,D", [("bf16", "causal", 64), ("fp16", "kvlen", 64), ("bf16", "none", 64),
                                        ("bf16", "causal", 128), ("fp16", "none", 128)])
def test_strided_views_are_read_in_place(dt, kind, D):
    """q, k, v (and tangents) given as the (B,H,L,D) view of (B,L,H,D) tensors -- what a model's projection layer
    produces before `.transpose(1, 2)` -- go to the tcgen05 kernels with their strides (no copy; the
    reference always calls `.contiguous()`, jvp_attention.py:2733-2734).  Results must equal those from
    contiguous copies bit for bit, through the C ABI and through the public API with gradients."""
    dtype, dev = DT[dt], torch.device("cuda:0")
    B, H, L = 3, 5, 200
    g = torch.Generator().manual_seed(11)
    base = [torch.randn(B, L, H, D, generator=g) for _ in range(8)]
    for i in (3, 4, 5):
        base[i] = base[i] * 0.1
    views = [x.to(dtype).to(dev).transpose(1, 2) for x in base]  # (B,H,L,D), strides (L*H*D, D, H*D, 1)
    q, k, v, tq, tk, tv, w1, w2 = views
    assert not q.is_contiguous()
    mask, causal = _mask(kind, B, H, L, dtype, seed=3)
    spec, _, _ = ja.classify_mask(None if mask is None else mask.to(dev), causal, B, H, L, dtype, False)

    def run_abi(ins, st):
        o, to = torch.empty(B, H, L, D, device=dev, dtype=dtype), torch.empty(B, H, L, D, device=dev, dtype=dtype)
        lse, mu = torch.empty(B, H, L, device=dev), torch.empty(B, H, L, device=dev)
        _lib.fwd(*ins, o, to, lse, mu, spec, D**-0.5, _lib.IMPL_TCGEN05, in_stride=st)
        go, gto = w1.contiguous(), w2.contiguous()
        stats = torch.empty(3, B, H, L, device=dev)
        _lib.bwd_preprocess(o, to, go, gto, mu, stats[0], stats[1], stats[2])
        dq, dk, dv = (torch.empty(B, H, L, D, device=dev, dtype=dtype) for _ in range(3))
        _lib.bwd(*ins, go, gto, lse, mu, stats[0], stats[1], stats[2], dq, dk, dv, spec, D**-0.5, _lib.IMPL_TCGEN05,
                 in_stride=st)
        torch.cuda.synchronize()
        return o, to, lse, mu, dq, dk, dv

    st = _lib.common_strides(q, k, v, tq, tk, tv)
    assert st == (L * H * D, D, H * D)
    strided = run_abi([q, k, v, tq, tk, tv], st)
    dense = run_abi([x.contiguous() for x in (q, k, v, tq, tk, tv)], None)
    assert _lib.device_status() == 0
    for name, a, b in zip(("o", "to", "lse", "mu", "dq", "dk", "dv"), strided, dense):
        assert torch.equal(a, b), name

    # public API: views in, gradients w.r.t. the views out
    def api(qq, kk, vv):
        a = [x.detach().clone().requires_grad_() if x.is_contiguous() else x.detach().requires_grad_() for x in (qq, kk, vv)]
        o, to = torch.func.jvp(lambda x, y, z: ja.JVPAttn.fwd_dual(x, y, z, attn_mask=None if mask is None else mask.to(dev),
                                                                  causal=causal), tuple(a), (tq, tk, tv))
        loss = (o.float() * w1.float()).sum() + (to.float() * w2.float()).sum()
        return (o.detach(), to.detach()) + torch.autograd.grad(loss, a)

    for a, b in zip(api(q, k, v), api(q.contiguous(), k.contiguous(), v.contiguous())):
        assert torch.equal(a.contiguous(), b.contiguous())
    # primal only (D = 64: the 32-key sub-tile kernel), views against copies
    assert torch.equal(ja.JVPAttn.fwd(q, k, v, causal=causal, attn_mask=None if mask is None else mask.to(dev)),
                       ja.JVPAttn.fwd(q.contiguous(), k.contiguous(), v.contiguous(), causal=causal,
                                      attn_mask=None if mask is None else mask.to(dev)))
    # a layout the kernels cannot read in place (fp32 goes to the register-tiled family) is still served
    o32 = ja.JVPAttn.fwd(q.float(), k.float(), v.float(), causal=causal)
    ro = orc.sdpa_primal(q.float().cpu(), k.float().cpu(), v.float().cpu(), causal=causal)
    assert orc.rel_err(o32, ro) < 1e-5


@pytest.mark.parametrize("dt,kind,D", [("fp32", "causal", 64), ("fp32", "bias", 128), ("bf16", "kvlen", 32), ("fp32", "none", 32)])
def test_register_tiled_family_reads_strided_views_in_place(dt, kind, D):
    """The same (B,H,L,D) views of (B,L,H,D) tensors through the register-tiled kernels (fp32, D = 32, anything forced
    there): their tile loads take the row stride, so nothing is copied; results equal those from contiguous copies bit
    for bit, forward and backward."""
    dtype, dev = DT[dt], torch.device("cuda:0")
    B, H, L = 2, 3, 200
    g = torch.Generator().manual_seed(12)
    base = [torch.randn(B, L, H, D, generator=g) for _ in range(8)]
    for i in (3, 4, 5):
        base[i] = base[i] * 0.1
    q, k, v, tq, tk, tv, w1, w2 = [x.to(dtype).to(dev).transpose(1, 2) for x in base]
    mask, causal = _mask(kind, B, H, L, dtype, seed=4)
    spec, _, _ = ja.classify_mask(None if mask is None else mask.to(dev), causal, B, H, L, dtype, False)

    def run_abi(ins, st):
        o, to = torch.empty(B, H, L, D, device=dev, dtype=dtype), torch.empty(B, H, L, D, device=dev, dtype=dtype)
        lse, mu = torch.empty(B, H, L, device=dev), torch.empty(B, H, L, device=dev)
        _lib.fwd(*ins, o, to, lse, mu, spec, D**-0.5, _lib.IMPL_GENERIC, in_stride=st)
        go, gto = w1.contiguous(), w2.contiguous()
        stats = torch.empty(3, B, H, L, device=dev)
        _lib.bwd_preprocess(o, to, go, gto, mu, stats[0], stats[1], stats[2])
        dq, dk, dv = (torch.empty(B, H, L, D, device=dev, dtype=dtype) for _ in range(3))
        _lib.bwd(*ins, go, gto, lse, mu, stats[0], stats[1], stats[2], dq, dk, dv, spec, D**-0.5, _lib.IMPL_GENERIC,
                 in_stride=st)
        torch.cuda.synchronize()
        return o, to, lse, mu, dq, dk, dv

    st = _lib.common_strides(q, k, v, tq, tk, tv)
    assert st == (L * H * D, D, H * D)
    strided = run_abi([q, k, v, tq, tk, tv], st)
    dense = run_abi([x.contiguous() for x in (q, k, v, tq, tk, tv)], None)
    for name, a_, b_ in zip(("o", "to", "lse", "mu", "dq", "dk", "dv"), strided, dense):
        assert torch.equal(a_, b_), name
    ro, rto = orc.sdpa_jvp(*(x.float().cpu() for x in (q, k, v, tq, tk, tv)), attn_mask=mask, causal=causal)
    _close(strided[0], ro, dtype, "O")
    _close(strided[1], rto, dtype, "tO")


@pytest.mark.parametrize("dt,D,L", [("bf16", 64, 33), ("fp16", 128, 7), ("fp32", 64, 31), ("bf16", 64, 1)])
def test_any_sequence_length_through_the_api_when_the_upstream_check_is_lifted(dt, D, L, monkeypatch):
    """Upstream's "multiple of 2 and >= 32" is a property of its block sizes, not of the kernels here: with
    STRICT_SEQUENCE_LENGTH = False odd and short lengths go through the public API, forward with tangents and backward."""
    dtype, dev = DT[dt], "cuda:0"
    q, k, v, tq, tk, tv, w1, w2 = _make(2, 2, L, D, dtype, seed=L)
    with pytest.raises(AssertionError, match="multiple of 2"):
        ja.attention(q.to(dev), k.to(dev), v.to(dev), causal=True)
    monkeypatch.setattr(ja, "STRICT_SEQUENCE_LENGTH", False)
    a = [x.to(dev).requires_grad_() for x in (q, k, v)]
    o, to = torch.func.jvp(lambda x, y, z: ja.JVPAttn.fwd_dual(x, y, z, causal=True), tuple(a),
                           (tq.to(dev), tk.to(dev), tv.to(dev)))
    g = torch.autograd.grad((o.float() * w1.to(dev).float()).sum() + (to.float() * w2.to(dev).float()).sum(), a)
    ro, rto, rdq, rdk, rdv = orc.grads_through_both(q, k, v, tq, tk, tv, w1, w2, causal=True)
    _close(o, ro, dtype, "O")
    _close(to, rto, dtype, "tO")
    for name, x, r in zip(("dq", "dk", "dv"), g, (rdq, rdk, rdv)):
        _close(x, r, dtype, name)


def test_mask_verification_is_one_device_pass():
    """`verify_attn_mask=True` (the default, as upstream: jvp_attention.py:2438-2457) raises what upstream raises,
    from the flags of one jvpfa_mask_check pass: a boolean head without a True, an inf, a NaN, a float head that
    is all MASK_CONST.  Vector and element-wise reading paths, broadcast extents, all mask dtypes."""
    dev = torch.device("cuda:0")
    B, H, L, D = 2, 3, 64, 64
    q, k, v, *_ = (x.to(dev) for x in _make(B, H, L, D, torch.bfloat16, seed=21))
    g = torch.Generator().manual_seed(5)
    ok = (torch.rand(B, H, L, L, generator=g) > 0.9)
    ok[..., 7] = True
    ja.attention(q, k, v, attn_mask=ok.to(dev))
    bad = ok.clone()
    bad[1, 2] = False
    with pytest.raises(AssertionError, match="all False"):
        ja.attention(q, k, v, attn_mask=bad.to(dev))
    # not looked at when switched off (the trailing optional argument of apply, as upstream: jvp_attention.py:2324)
    ja.JVPAttn.apply(q, k, v, None, None, None, bad.to(dev), 0.0, False, None, True, True, False)
    for own in ((1, H, L, L), (B, 1, 1, L), (B, H, L, L)):
        m = torch.rand(*own, generator=g) > 0.5
        m[..., 3] = True
        m[..., 5] = False  # never a key-padding prefix
        ja.attention(q, k, v, attn_mask=m.to(dev))
        m[own[0] - 1, own[1] - 1] = False
        with pytest.raises(AssertionError, match="all False"):
            ja.attention(q, k, v, attn_mask=m.to(dev))
    odd = ok.to(dev)[..., ::2].repeat_interleave(2, dim=-1)  # fresh tensor
    view = torch.zeros(B, H, L, 2 * L, dtype=torch.bool, device=dev)[..., ::2]  # key stride 2: element-wise path
    view.copy_(odd)
    spec, _, _ = ja.classify_mask(view, False, B, H, L, torch.bfloat16, True)
    for mdt in (torch.bfloat16, torch.float16, torch.float32):
        bias = torch.where(ok, 0.0, ja.MASK_CONST).to(mdt).to(dev)
        ja.attention(q, k, v, attn_mask=bias)
        x = bias.clone()
        x[0, 1] = ja.MASK_CONST
        with pytest.raises(AssertionError, match="masking constant"):
            ja.attention(q, k, v, attn_mask=x)
        x = bias.clone()
        x[1, 0, 5, 9] = float("inf")
        with pytest.raises(AssertionError, match="-inf or inf"):
            ja.attention(q, k, v, attn_mask=x)
        x[1, 0, 5, 9] = float("-inf")
        with pytest.raises(AssertionError, match="-inf or inf"):
            ja.attention(q, k, v, attn_mask=x)
        x[1, 0, 5, 9] = float("nan")
        with pytest.raises(AssertionError, match="NaNs"):
            ja.attention(q, k, v, attn_mask=x)
        sl = torch.zeros(B, H, L, L + 8, dtype=mdt, device=dev)[..., 4:L + 4]  # rows not 16-byte aligned
        sl.copy_(bias)
        ja.attention(q, k, v, attn_mask=sl)
        sl[0, 0] = ja.MASK_CONST
        with pytest.raises(AssertionError, match="masking constant"):
            ja.attention(q, k, v, attn_mask=sl)


def _tile_bitmap_reference(mask, L):
    """bit t of word t // 64 of entry [b][h][qt]: tile (128 queries x 64 keys) has a True."""
    B, H, R, _ = mask.shape
    n_kt, n_qt = (L + 63) // 64, 1 if R == 1 else (L + 127) // 128
    n_words = (n_kt + 63) // 64
    out = torch.zeros(B, H, n_qt, n_words, dtype=torch.int64)
    for qt in range(n_qt):
        rows = mask[:, :, qt * 128:(qt + 1) * 128] if R > 1 else mask
        for t in range(n_kt):
            live = rows[..., t * 64:(t + 1) * 64].any(dim=(-1, -2))
            bit = 1 << (t % 64)
            bit = bit - (1 << 64) if bit >= 1 << 63 else bit
            out[:, :, qt, t // 64] |= torch.where(live, bit, 0)
    return out.reshape(-1)


@pytest.mark.parametrize("dt,B,H,L,kind,dual", [
    ("bf16", 2, 3, 512, "documents", True), ("fp16", 1, 2, 1024, "window", True), ("bf16", 2, 2, 384, "documents", False),
    ("bf16", 3, 2, 448, "keys", True), ("fp16", 1, 2, 4224, "window", True),
])
def test_tcgen05_forward_steps_over_dead_mask_tiles(dt, B, H, L, kind, dual):
    """Boolean masks with whole 128 x 64 tiles of False (documents packed into one sequence, a sliding window,
    dropped key ranges): jvpfa_mask_tiles must report exactly the tiles with a True, and the forward given that
    bitmap must equal the forward without it (which visits every tile) and the oracle.  One query tile of one head
    is dead altogether: zeros and lse = +inf."""
    dtype, dev = DT[dt], torch.device("cuda:0")
    g = torch.Generator().manual_seed(L)
    i, j = torch.arange(L)[:, None], torch.arange(L)[None, :]
    if kind == "documents":
        cuts = torch.sort(torch.randint(1, L, (B, 3), generator=g), dim=1).values
        doc = (torch.arange(L)[None, :, None] >= cuts[:, None, :]).sum(-1)  # (B, L) document index
        mask = (doc[:, :, None] == doc[:, None, :])[:, None].expand(B, H, L, L).clone()
        mask &= torch.rand(B, H, L, L, generator=g) > 0.2
        mask[..., 0, 0] = True
    elif kind == "window":
        mask = ((i - j).abs() < 100)[None, None].expand(B, H, L, L).clone()
    else:  # keys dropped for all queries: one mask row per batch entry
        mask = torch.rand(B, 1, 1, L, generator=g) > 0.3
        mask[..., 64:192] = False
        mask[..., 5] = True
    if mask.shape[2] > 1:
        mask[0, H - 1, 128:256] = False  # a query tile without any key
    q, k, v, tq, tk, tv, *_ = _make(B, H, L, 64, dtype, seed=L + 1)
    if not dual:
        tq = tk = tv = None
    md = mask.to(dev)
    spec = _lib.MaskSpec(_lib.MASK_BOOL, md.view(torch.uint8), tuple(0 if md.shape[d] == 1 else md.stride(d) for d in range(4)))
    tile_live, head_live, tile_live_t = _lib.mask_tiles(spec, L)
    assert torch.equal(tile_live.cpu(), _tile_bitmap_reference(mask, L))
    assert torch.equal(head_live[:-1].cpu().bool(), mask.any(dim=(-1, -2)).reshape(-1))
    n_kt = (L + 63) // 64
    n_live = sum(bin(x & (2**64 - 1)).count("1") for x in tile_live.tolist())
    assert head_live[-1].item() == n_live
    assert 0 < n_live < n_kt * (tile_live.numel() // ((n_kt + 63) // 64))  # the case does have dead tiles

    cu = lambda x: None if x is None else x.to(dev)  # noqa: E731
    outs = []
    for bitmap in (None, tile_live):
        spec.tile_live = bitmap
        o = torch.empty(B, H, L, 64, device=dev, dtype=dtype)
        to = torch.empty_like(o) if dual else None
        lse = torch.empty(B, H, L, device=dev)
        mu = torch.empty_like(lse) if dual else None
        _lib.fwd(cu(q), cu(k), cu(v), cu(tq), cu(tk), cu(tv), o, to, lse, mu, spec, 0.125, _lib.IMPL_TCGEN05)
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        outs.append((o, to, lse, mu))
    for a_, b_ in zip(outs[0], outs[1]):
        if a_ is not None:
            assert torch.equal(a_, b_)  # dead tiles contribute exact zeros either way
    o, to, lse, mu = outs[1]
    if mask.shape[2] > 1:
        assert o[0, H - 1, 128:256].abs().max() == 0 and torch.isinf(lse[0, H - 1, 128:256]).all()
    if dual:
        ro, rto = orc.sdpa_jvp(q, k, v, tq, tk, tv, attn_mask=mask)
        _close(to, rto, dtype, "tO")
    else:
        ro = orc.sdpa_primal(q, k, v, attn_mask=mask)
    _close(o, ro, dtype, "O")
    # the same summary per 128-key tile: bit qt of entry [head][kt]
    n_qt, n_kt128 = (1 if mask.shape[2] == 1 else (L + 127) // 128), (L + 127) // 128
    ref_t = torch.zeros(mask.shape[0], mask.shape[1], n_kt128, (n_qt + 63) // 64, dtype=torch.int64)
    for kt in range(n_kt128):
        for qt in range(n_qt):
            rows = mask[:, :, qt * 128:(qt + 1) * 128] if mask.shape[2] > 1 else mask
            ref_t[:, :, kt, qt // 64] |= torch.where(rows[..., kt * 128:(kt + 1) * 128].any(dim=(-1, -2)), 1 << (qt % 64), 0)
    assert torch.equal(tile_live_t.cpu(), ref_t.reshape(-1))
    # backward: visiting only the sub-tiles of live tiles gives the gradients of visiting all of them
    if dual:
        gg = torch.Generator().manual_seed(L + 2)
        go, gto = (torch.randn(B, H, L, 64, generator=gg).to(dtype).to(dev) for _ in range(2))
        grads = []
        for bitmaps in ((None, None), (tile_live, tile_live_t)):
            spec.tile_live, spec.tile_live_t = bitmaps
            stats = torch.empty(3, B, H, L, device=dev)
            _lib.bwd_preprocess(o, to, go, gto, mu, stats[0], stats[1], stats[2])
            dq, dk, dv = (torch.empty(B, H, L, 64, device=dev, dtype=dtype) for _ in range(3))
            _lib.bwd(cu(q), cu(k), cu(v), cu(tq), cu(tk), cu(tv), go, gto, lse, mu, stats[0], stats[1], stats[2], dq, dk, dv,
                     spec, 0.125, _lib.IMPL_TCGEN05)
            torch.cuda.synchronize()
            assert _lib.device_status() == 0
            grads.append((dq, dk, dv))
        for name, x, y in zip(("dq", "dk", "dv"), grads[1], grads[0]):
            assert torch.isfinite(x.float()).all(), name
            _close(x, y.float(), dtype, name)  # summation order over sub-tiles is the same; dead ones add zeros
        _, _, rdq, rdk, rdv = orc.grads_through_both(q[:1, :1], k[:1, :1], v[:1, :1], tq[:1, :1], tk[:1, :1], tv[:1, :1],
                                                     go[:1, :1].cpu(), gto[:1, :1].cpu(), attn_mask=mask[:1, :1])
        for name, x, r in zip(("dq", "dk", "dv"), grads[1], (rdq, rdk, rdv)):
            _close(x[:1, :1], r, dtype, name)
    # and through the public API (classification builds the bitmaps), with gradients
    a = [cu(x).requires_grad_() for x in (q, k, v)]
    out = ja.attention(*a, attn_mask=md)
    assert torch.equal(out.detach(), o)
    torch.autograd.grad(out.float().sum(), a)


@pytest.mark.parametrize("dual", [True, False], ids=["dual", "primal"])
@pytest.mark.parametrize("kind", ["window", "blocks", "keys"])
def test_head_dim_128_forward_steps_over_dead_mask_tiles(kind, dual):
    """D = 128: with the tile bitmap the forward lists the live key tiles of its query tile and visits only those; the
    results are bit for bit those of the plain masked loop (dead tiles contribute exact zeros) and agree with the
    oracle; a query tile without any key gives zeros and lse = +inf; the public API takes the same route."""
    dev, dtype = "cuda:0", torch.bfloat16
    B, H, L = 2, 3, 640
    g = torch.Generator().manual_seed(11)
    i, j = torch.arange(L)[:, None], torch.arange(L)[None, :]
    if kind == "window":
        mask = ((i - j).abs() <= 96).expand(B, H, L, L).clone()
    elif kind == "blocks":
        mask = ((i // 128) % 3 == (j // 64) % 3).expand(1, H, L, L).clone() & (torch.rand(1, H, L, L, generator=g) > 0.2)
        mask[0, :, torch.arange(L), (torch.arange(L) // 128 % 3) * 64] = True  # every row keeps a key
        mask[0, H - 1, 128:256] = False  # a query tile without any key
    else:
        mask = torch.rand(B, 1, 1, L, generator=g) > 0.3
        mask[..., 64:256] = False
        mask[..., 5] = True
    q, k, v, tq, tk, tv, *_ = _make(B, H, L, 128, dtype, seed=77)
    if not dual:
        tq = tk = tv = None
    md = mask.to(dev)
    spec = _lib.MaskSpec(_lib.MASK_BOOL, md.view(torch.uint8), tuple(0 if md.shape[d] == 1 else md.stride(d) for d in range(4)))
    tile_live, head_live, _ = _lib.mask_tiles(spec, L)
    n_kt = (L + 63) // 64
    n_live = head_live[-1].item()
    assert 0 < n_live < n_kt * (tile_live.numel() // ((n_kt + 63) // 64))  # the case does have dead tiles
    cu = lambda x: None if x is None else x.to(dev)  # noqa: E731
    outs = []
    for bitmap in (None, tile_live):
        spec.tile_live = bitmap
        o = torch.empty(B, H, L, 128, device=dev, dtype=dtype)
        to = torch.empty_like(o) if dual else None
        lse = torch.empty(B, H, L, device=dev)
        mu = torch.empty_like(lse) if dual else None
        _lib.fwd(cu(q), cu(k), cu(v), cu(tq), cu(tk), cu(tv), o, to, lse, mu, spec, 128 ** -0.5, _lib.IMPL_TCGEN05)
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        outs.append((o, to, lse, mu))
    for a_, b_ in zip(outs[0], outs[1]):
        if a_ is not None:
            assert torch.equal(a_, b_)
    o, to, lse, mu = outs[1]
    if kind == "blocks":
        assert o[0, H - 1, 128:256].abs().max() == 0 and torch.isinf(lse[0, H - 1, 128:256]).all()
    if dual:
        ro, rto = orc.sdpa_jvp(q, k, v, tq, tk, tv, attn_mask=mask)
        _close(to, rto, dtype, "tO")
    else:
        ro = orc.sdpa_primal(q, k, v, attn_mask=mask)
    _close(o, ro, dtype, "O")
    out = ja.attention(cu(q), cu(k), cu(v), attn_mask=md)
    assert torch.equal(out, outs[1][0])
    # backward: both launches visit only loop tiles that overlap a live bitmap tile (own keys: 32-query tiles inside
    # live 128-query tiles; own queries: 48-key tiles overlapping a live 64-key tile); dead ones would add exact zeros
    gg = torch.Generator().manual_seed(78)
    go = torch.randn(B, H, L, 128, generator=gg).to(dtype).to(dev)
    gto = torch.randn(B, H, L, 128, generator=gg).to(dtype).to(dev) if dual else None
    _, _, tile_live_t = _lib.mask_tiles(spec, L)
    grads = []
    for bitmaps in ((None, None), (tile_live, tile_live_t)):
        spec.tile_live, spec.tile_live_t = bitmaps
        stats = torch.empty(3, B, H, L, device=dev)
        _lib.bwd_preprocess(o, to, go, gto, mu, stats[0], stats[1], stats[2])
        dq, dk, dv = (torch.empty(B, H, L, 128, device=dev, dtype=dtype) for _ in range(3))
        _lib.bwd(cu(q), cu(k), cu(v), cu(tq), cu(tk), cu(tv), go, gto, lse, mu, stats[0], stats[1], stats[2], dq, dk, dv,
                 spec, 128 ** -0.5, _lib.IMPL_TCGEN05)
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        grads.append((dq, dk, dv))
    for name, x, y in zip(("dq", "dk", "dv"), grads[1], grads[0]):
        assert torch.isfinite(x.float()).all(), name
        assert torch.equal(x, y), name  # same tiles in the same order; the skipped ones held zeros
    if dual:
        refs = orc.grads_through_both(q[:1, :1], k[:1, :1], v[:1, :1], tq[:1, :1], tk[:1, :1], tv[:1, :1],
                                      go[:1, :1].cpu(), gto[:1, :1].cpu(), attn_mask=mask[:1, :1])
        for name, x, r in zip(("dq", "dk", "dv"), grads[1], refs[2:]):
            _close(x[:1, :1], r, dtype, name)


@pytest.mark.parametrize("D,L,kind", [(64, 160, "causal"), (128, 96, "bias"), (32, 128, "bool"), (64, 256, "none")])
def test_fp32_single_pass_tf32_mode(D, L, kind):
    """`set_fp32_precision("tf32")`: fp32 tensors multiplied with one TF32 MMA per product, the precision of upstream's
    fp32 path (jvp_attention.py:233-236; its tolerance is 2.35e-2 absolute, tests/test_jvp_attention.py:688-693).
    Stated error of this mode: 5e-3 of max|ref| on every output here; the default three-pass mode on the same inputs
    stays at 1e-5."""
    B, H = 2, 2
    q, k, v, tq, tk, tv, go, gto = _make(B, H, L, D, torch.float32, seed=D + L)
    mask, causal = _mask(kind, B, H, L, torch.float32, seed=L)
    refs = orc.grads_through_both(q, k, v, tq, tk, tv, go, gto, attn_mask=mask, causal=causal)
    exact = _run_kernels(q, k, v, tq, tk, tv, go, gto, mask, causal)
    prev = ja.set_fp32_precision("tf32")
    try:
        fast = _run_kernels(q, k, v, tq, tk, tv, go, gto, mask, causal)
    finally:
        assert ja.set_fp32_precision(prev) == "tf32"
    worst_fast = 0.0
    for name, r, x3, x1 in zip(("O", "tO", "dq", "dk", "dv"), refs, (exact[0], exact[1], *exact[4:]), (fast[0], fast[1], *fast[4:])):
        assert orc.rel_err(x3, r) < 1e-5, name
        e = orc.rel_err(x1, r)
        assert e < 5e-3, (name, e)
        worst_fast = max(worst_fast, e)
    assert worst_fast > 2e-5  # the mode really multiplies in one pass


@pytest.mark.parametrize("mask_type", ["boolean", "additive"])
def test_reference_grid_largest_masked_case_on_tcgen05(mask_type):
    """The largest masked cases of the reference's grid (B=2, 12 heads, L=2048, D=64, 90 % masked; boolean and {0, -100}
    additive): forward and backward through both outputs on the tcgen05 kernels against the register-tiled family on
    all heads, and against the float64 oracle on one head."""
    from tests import harness as hz

    dev = torch.device("cuda:0")
    B, H, L, D = 2, 12, 2048, 64
    q, k, v, tq, tk, tv, target, mask = hz.make_case(L, mask_type, torch.bfloat16, dev)
    tq, tk, tv = tq * 0.1, tk * 0.1, tv * 0.1
    g = torch.Generator(device=dev).manual_seed(7)
    go, gto = (torch.randn(B, H, L, D, device=dev, dtype=torch.bfloat16, generator=g) for _ in range(2))
    c = lambda x: x.cpu()  # noqa: E731
    fast = _run_kernels(c(q), c(k), c(v), c(tq), c(tk), c(tv), c(go), c(gto), c(mask), False, impl=_lib.IMPL_TCGEN05)
    assert _lib.device_status() == 0
    slow = _run_kernels(c(q), c(k), c(v), c(tq), c(tk), c(tv), c(go), c(gto), c(mask), False, impl=_lib.IMPL_GENERIC)
    for name, x, y in zip(("O", "tO", "lse", "mu", "dq", "dk", "dv"), fast, slow):
        assert torch.isfinite(x.float()).all(), name
        if name in ("lse", "mu"):
            assert orc.max_abs_err(x, y) < 2e-3, name
        else:
            _close(x, y.float(), torch.bfloat16, name)
    b, h = 1, 7
    sl = lambda x: c(x)[b:b + 1, h:h + 1]  # noqa: E731
    ro, rto, rdq, rdk, rdv = orc.grads_through_both(sl(q), sl(k), sl(v), sl(tq), sl(tk), sl(tv), sl(go), sl(gto),
                                                    attn_mask=sl(mask))
    for name, x, r in zip(("O", "tO", "dq", "dk", "dv"), (fast[0], fast[1], fast[4], fast[5], fast[6]), (ro, rto, rdq, rdk, rdv)):
        _close(x[b:b + 1, h:h + 1], r, torch.bfloat16, name)


@pytest.mark.parametrize("cot,kind,dt,B,H,L", [
    ("both", "none", "bf16", 2, 2, 192), ("gt", "causal", "fp16", 1, 3, 320), ("both", "bool", "bf16", 2, 2, 256),
    ("gt", "bias", "fp16", 2, 2, 192), ("go", "bool_bcast", "bf16", 2, 2, 160), ("both", "bool_keys", "fp16", 3, 2, 224),
    ("gt", "bias", "bf16", 1, 2, 48),
    # the pipelined kernels (no user mask): ragged lengths, every cotangent combination, more than one ring lap
    ("go", "none", "fp16", 1, 2, 200), ("both", "kvlen", "bf16", 2, 2, 512), ("gt", "none", "bf16", 1, 2, 96),
    ("go", "causal", "bf16", 1, 2, 333), ("both", "causal", "bf16", 1, 2, 1024), ("gt", "kvlen", "fp16", 2, 1, 160),
    ("both", "none", "fp16", 1, 1, 31),
])
def test_tcgen05_head_dim_128_forward_and_backward(cot, kind, dt, B, H, L):
    """The D = 128 tcgen05 kernels (forward with tangents, both backward launches) on every mask kind they take,
    boolean masks and bias of the element type included, against the register-tiled family on all heads and the
    float64 oracle on one."""
    dtype = DT[dt]
    q, k, v, tq, tk, tv, go, gto = _make(B, H, L, 128, dtype, seed=B + L)
    go = go if cot in ("go", "both") else None
    gto = gto if cot in ("gt", "both") else None
    mask, causal = _mask(kind, B, H, L, dtype, seed=L)
    fast = _run_kernels(q, k, v, tq, tk, tv, go, gto, mask, causal, impl=_lib.IMPL_TCGEN05)
    assert _lib.device_status() == 0, "a bounded wait inside a tcgen05 kernel gave up"
    slow = _run_kernels(q, k, v, tq, tk, tv, go, gto, mask, causal, impl=_lib.IMPL_GENERIC)
    for name, x, y in zip(("O", "tO", "lse", "mu", "dq", "dk", "dv"), fast, slow):
        assert torch.isfinite(x.float()).all(), name
        if name in ("lse", "mu"):
            assert orc.max_abs_err(x, y) < 2e-3, name
        else:
            _close(x, y.float(), dtype, name)
    sl = lambda x: None if x is None else x[B - 1:, H - 1:]  # noqa: E731
    msl = None if mask is None else mask[min(B, mask.shape[0]) - 1:, min(H, mask.shape[1]) - 1:]
    ro, rto, rdq, rdk, rdv = orc.grads_through_both(sl(q), sl(k), sl(v), sl(tq), sl(tk), sl(tv), sl(go), sl(gto),
                                                    attn_mask=msl, causal=causal)
    for name, x, r in zip(("O", "tO", "dq", "dk", "dv"), (fast[0], fast[1], fast[4], fast[5], fast[6]), (ro, rto, rdq, rdk, rdv)):
        _close(x[B - 1:, H - 1:], r, dtype, name)
