"""Repeated launches of every tcgen05 kernel on one input: the device status word must stay 0 and the outputs must not
change from launch to launch.

A protocol flaw in a persistent, warp-specialised kernel shows as a rare stall (one launch in a hundred for the flaw
this test was written after: a waiter two phases behind a parity barrier), not as a wrong number in a single call, and a
race between roles shows as outputs that differ between launches.  A few hundred back-to-back launches per kernel,
some of them after an L2 flush (which changes the timing between the roles), catch both cheaply.  dQ of the single-pass
backward is the one output that may differ in the last bits (fp32 reductions in varying order); it is compared with a
tolerance.
"""
import pytest
import torch

from jvp_flash_attention_b200 import _lib

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
LAUNCHES = 300


def _tensors(B, H, L, D, dtype, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)

    def mk(s=1.0):
        return (torch.randn(B, H, L, D, device=DEV, generator=g) * s).to(dtype)

    return dict(q=mk(), k=mk(), v=mk(), tq=mk(0.1), tk=mk(0.1), tv=mk(0.1), go=mk(), gto=mk())


def _soak(fn, exact, close=()):
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=DEV)
    fn()
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    ref_exact = [o.clone() for o in exact]
    ref_close = [o.clone() for o in close]
    for batch in range(LAUNCHES // 50):
        for _ in range(50):
            if batch % 3 == 1:
                flush.zero_()
            fn()
        torch.cuda.synchronize()
        assert _lib.device_status() == 0, f"a bounded wait gave up within {50 * (batch + 1)} launches"
    for r, o in zip(ref_exact, exact):
        assert torch.equal(r, o), "an output changed between launches"
    for r, o in zip(ref_close, close):
        assert (r.float() - o.float()).abs().max().item() <= 2e-2 * max(1.0, r.float().abs().max().item())


CASES = [
    ("d64_causal", 2, 16, 2048, 64, _lib.MASK_CAUSAL),
    ("d64_ragged", 2, 8, 1000, 64, _lib.MASK_NONE),
    ("d128_causal", 1, 8, 2048, 128, _lib.MASK_CAUSAL),
    ("d128_ragged", 1, 4, 1111, 128, _lib.MASK_NONE),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("name,B,H,L,D,kind", CASES, ids=[c[0] for c in CASES])
def test_repeated_launches_stay_clean_and_reproducible(name, B, H, L, D, kind, dtype):
    d = _tensors(B, H, L, D, dtype)
    spec = _lib.MaskSpec(kind)
    scale = D ** -0.5
    o, to = torch.empty_like(d["q"]), torch.empty_like(d["q"])
    lse, mu = torch.empty(B, H, L, device=DEV), torch.empty(B, H, L, device=DEV)
    _soak(lambda: _lib.fwd(d["q"], d["k"], d["v"], d["tq"], d["tk"], d["tv"], o, to, lse, mu, spec, scale,
                           _lib.IMPL_TCGEN05), [o, to, lse, mu])
    o1, lse1 = torch.empty_like(o), torch.empty_like(lse)
    _soak(lambda: _lib.fwd(d["q"], d["k"], d["v"], None, None, None, o1, None, lse1, None, spec, scale,
                           _lib.IMPL_TCGEN05), [o1, lse1])
    stats = torch.empty(3, B, H, L, device=DEV)
    _lib.bwd_preprocess(o, to, d["go"], d["gto"], mu, stats[0], stats[1], stats[2])
    dq, dk, dv = (torch.empty_like(o) for _ in range(3))
    _soak(lambda: _lib.bwd(d["q"], d["k"], d["v"], d["tq"], d["tk"], d["tv"], d["go"], d["gto"], lse, mu, stats[0],
                           stats[1], stats[2], dq, dk, dv, spec, scale, _lib.IMPL_TCGEN05), [dq, dk, dv])
    if D == 64:  # the single-pass backward: through both outputs, through the tangent output alone
        acc = torch.empty(B, H, L, D, device=DEV, dtype=torch.float32)
        _soak(lambda: _lib.bwd(d["q"], d["k"], d["v"], d["tq"], d["tk"], d["tv"], d["go"], d["gto"], lse, mu, stats[0],
                               stats[1], stats[2], dq, dk, dv, spec, scale, _lib.IMPL_TCGEN05, dq_accum=acc),
              [dk, dv], close=[dq])
        _lib.bwd_preprocess(o, to, None, d["gto"], mu, stats[0], stats[1], stats[2])
        _soak(lambda: _lib.bwd(d["q"], d["k"], d["v"], d["tq"], d["tk"], d["tv"], None, d["gto"], lse, mu, stats[0],
                               stats[1], stats[2], dq, dk, dv, spec, scale, _lib.IMPL_TCGEN05, dq_accum=acc),
              [dk, dv], close=[dq])
        # ... and through O alone (the variant with two sets of own tiles)
        _lib.bwd_preprocess(o, None, d["go"], None, None, stats[0], stats[1], stats[2])
        _soak(lambda: _lib.bwd(d["q"], d["k"], d["v"], None, None, None, d["go"], None, lse, None, stats[0],
                               stats[1], stats[2], dq, dk, dv, spec, scale, _lib.IMPL_TCGEN05, dq_accum=acc),
              [dk, dv], close=[dq])


def test_repeated_launches_with_a_boolean_mask():
    B, H, L, D = 2, 4, 1024, 64
    d = _tensors(B, H, L, D, torch.bfloat16, seed=1)
    g = torch.Generator(device=DEV).manual_seed(5)
    m = torch.rand(B, H, L, L, device=DEV, generator=g) > 0.3
    m[..., 0] = True
    m8 = m.to(torch.uint8).contiguous()
    spec = _lib.MaskSpec(_lib.MASK_BOOL, m8, tuple(m8.stride()))
    o, to = torch.empty_like(d["q"]), torch.empty_like(d["q"])
    lse, mu = torch.empty(B, H, L, device=DEV), torch.empty(B, H, L, device=DEV)
    _soak(lambda: _lib.fwd(d["q"], d["k"], d["v"], d["tq"], d["tk"], d["tv"], o, to, lse, mu, spec, D ** -0.5,
                           _lib.IMPL_TCGEN05), [o, to, lse, mu])
    stats = torch.empty(3, B, H, L, device=DEV)
    _lib.bwd_preprocess(o, to, d["go"], d["gto"], mu, stats[0], stats[1], stats[2])
    dq, dk, dv = (torch.empty_like(o) for _ in range(3))
    _soak(lambda: _lib.bwd(d["q"], d["k"], d["v"], d["tq"], d["tk"], d["tv"], d["go"], d["gto"], lse, mu, stats[0],
                           stats[1], stats[2], dq, dk, dv, spec, D ** -0.5, _lib.IMPL_TCGEN05), [dq, dk, dv])
    acc = torch.empty(B, H, L, D, device=DEV, dtype=torch.float32)  # ... and the single pass with the mask
    _soak(lambda: _lib.bwd(d["q"], d["k"], d["v"], d["tq"], d["tk"], d["tv"], d["go"], d["gto"], lse, mu, stats[0],
                           stats[1], stats[2], dq, dk, dv, spec, D ** -0.5, _lib.IMPL_TCGEN05, dq_accum=acc),
          [dk, dv], close=[dq])
