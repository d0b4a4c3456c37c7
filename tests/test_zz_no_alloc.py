"""GPU test of jvpfa_bwd_noalloc, the backward entry point for callers that cannot allocate device
memory (a process whose own pool owns the whole GPU, a loop that must avoid cudaMalloc's
device-wide synchronisation, a C caller without a tensor library).  Its scratch rows live in a
fixed array inside libjvpfa.so instead of in caller-provided buffers.

The file name sorts last on purpose: if this test fails under ``pytest -x`` every other test
has already run.  It is self-contained, so it also passes alone in a fresh process.

Checked here, through the C ABI: two calls in a row (different shapes and values, so the second
call finds the first call's rows in the shared array) each reproduce the gradients of the ordinary
``jvpfa_bwd_preprocess`` + ``jvpfa_bwd`` pair, and a problem beyond the fixed capacity is refused.
"""
import ctypes as C

import pytest
import torch

from jvp_flash_attention_b200 import _lib
from oracle import jvp_attention_oracle as orc

pytestmark = pytest.mark.gpu

# Both routes run the same kernels on the same inputs; the tolerances are the suite's own
# (float32: 1e-5 of the largest reference magnitude, 16-bit: 2e-2 absolute, scaled for gradients).
FP32_REL = 1e-5
HALF_ABS = 2e-2


def _case(dtype, B, H, L, D, causal, seed, both, bool_mask=False, oracle=False):
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(seed)
    q, k, v, tq, tk, tv, go, gto = [torch.randn(B, H, L, D, generator=g).to(dtype).to(dev) for _ in range(8)]
    if dtype != torch.float32:
        tq, tk, tv = [(x.float() * 0.1).to(dtype) for x in (tq, tk, tv)]
    spec = _lib.MaskSpec(_lib.MASK_CAUSAL if causal else _lib.MASK_NONE)
    mask = None
    if bool_mask:
        mask = torch.rand(B, H, L, L, generator=g) > 0.4
        mask[..., 0] = True
        m8 = mask.to(dev).view(torch.uint8)
        spec = _lib.MaskSpec(_lib.MASK_BOOL, m8, m8.stride())
    scale = D**-0.5
    o, to = torch.empty_like(q), torch.empty_like(q)
    lse = torch.empty(B, H, L, device=dev, dtype=torch.float32)
    mu = torch.empty_like(lse)
    _lib.fwd(q, k, v, tq, tk, tv, o, to, lse, mu, spec, scale)
    if not both:
        go = None

    # existing entry points, scratch provided by the caller
    stats = torch.empty(3, B, H, L, device=dev, dtype=torch.float32)
    _lib.bwd_preprocess(o, to, go, gto, mu, stats[0], stats[1], stats[2])
    ref = [torch.empty_like(q) for _ in range(3)]
    _lib.bwd(q, k, v, tq, tk, tv, go, gto, lse, mu, stats[0], stats[1], stats[2], *ref, spec, scale)

    # new entry point: inputs and outputs only
    out = [torch.full_like(q, float("nan")) for _ in range(3)]
    _lib.bwd_noalloc(q, k, v, tq, tk, tv, o, to, go, gto, lse, mu, *out, spec, scale)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0, "a bounded wait inside a kernel gave up"
    for name, x, r in zip(("dq", "dk", "dv"), out, ref):
        assert torch.isfinite(x).all(), name
        err = (x.double() - r.double()).abs().max().item()
        mag = max(1.0, r.double().abs().max().item())
        tol = FP32_REL * mag if dtype == torch.float32 else HALF_ABS * mag
        assert err <= tol, f"{name}: {err:.3e} > {tol:.3e}"
    if oracle:  # the new entry point against the float64 oracle itself, not only against the ordinary pair
        c = lambda x: None if x is None else x.cpu()  # noqa: E731
        refs = orc.grads_through_both(c(q), c(k), c(v), c(tq), c(tk), c(tv), c(go), c(gto), attn_mask=mask, causal=causal)[2:]
        for name, x, r in zip(("dq", "dk", "dv"), out, refs):
            err = orc.max_abs_err(x, r)
            mag = max(1.0, r.abs().max().item())
            tol = FP32_REL * mag if dtype == torch.float32 else HALF_ABS * mag
            assert err <= tol, f"{name} vs oracle: {err:.3e} > {tol:.3e}"


def test_no_alloc_backward_matches_regular_backward_twice_in_a_row():
    # first call: larger problem, both cotangents, fp32
    _case(torch.float32, 2, 3, 192, 64, causal=False, seed=1, both=True)
    # second call: smaller, other dtype and mask; stale rows of call one sit behind its range
    _case(torch.bfloat16, 1, 2, 96, 128, causal=True, seed=2, both=False)
    # third: same shape as the first again, different values
    _case(torch.float32, 2, 3, 192, 64, causal=True, seed=3, both=True, oracle=True)


def test_no_alloc_backward_on_the_persistent_16bit_kernels_back_to_back():
    """bf16, head dimension 64: the two overlapping persistent launches read the shared rows while they run.  Two
    calls straight after one another (causal, then a boolean mask), so that the second call's row reductions follow
    the first call's last kernel on the stream without any host synchronisation in between."""
    _case(torch.bfloat16, 3, 5, 416, 64, causal=True, seed=4, both=False, oracle=True)
    _case(torch.bfloat16, 2, 3, 256, 64, causal=False, seed=5, both=True, bool_mask=True, oracle=True)


def test_no_alloc_backward_refuses_sizes_beyond_its_capacity():
    lib = _lib.load()
    a = _lib.BwdNoAllocArgs()
    a.struct_size = C.sizeof(_lib.BwdNoAllocArgs)
    a.dtype, a.D = _lib.BF16, 64
    a.B, a.H, a.L = 1, 1, _lib.NOALLOC_MAX_ROWS + 1
    assert lib.jvpfa_bwd_noalloc(C.byref(a), None) == -10  # JVPFA_ERR_TOO_LARGE, before any launch
    a.B, a.H, a.L = 64, 64, 256  # 2^20 rows
    assert lib.jvpfa_bwd_noalloc(C.byref(a), None) == -10
    a.struct_size = 8
    assert lib.jvpfa_bwd_noalloc(C.byref(a), None) == -7  # JVPFA_ERR_STRUCT
    assert lib.jvpfa_bwd_noalloc(None, None) == -1
    # every check of the two launches comes before the first of them: a call without output pointers is refused
    # with nothing launched (and the shared rows untouched)
    a.struct_size = C.sizeof(_lib.BwdNoAllocArgs)
    a.B, a.H, a.L = 1, 1, 64
    x = torch.zeros(64 * 64, device="cuda:0", dtype=torch.bfloat16)
    a.q = a.k = a.v = a.o = a.go = x.data_ptr()
    a.lse = torch.zeros(64, device="cuda:0").data_ptr()
    assert lib.jvpfa_bwd_noalloc(C.byref(a), None) == -1  # dq, dk, dv are NULL
    assert b"capacity" in lib.jvpfa_strerror(-10)
