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

pytestmark = pytest.mark.gpu

# Both routes run the same kernels on the same inputs; the tolerances are the suite's own
# (float32: 1e-5 of the largest reference magnitude, 16-bit: 2e-2 absolute, scaled for gradients).
FP32_REL = 1e-5
HALF_ABS = 2e-2


def _case(dtype, B, H, L, D, causal, seed, both):
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(seed)
    q, k, v, tq, tk, tv, go, gto = [torch.randn(B, H, L, D, generator=g).to(dtype).to(dev) for _ in range(8)]
    if dtype != torch.float32:
        tq, tk, tv = [(x.float() * 0.1).to(dtype) for x in (tq, tk, tv)]
    spec = _lib.MaskSpec(_lib.MASK_CAUSAL if causal else _lib.MASK_NONE)
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
    for name, x, r in zip(("dq", "dk", "dv"), out, ref):
        assert torch.isfinite(x).all(), name
        err = (x.double() - r.double()).abs().max().item()
        mag = max(1.0, r.double().abs().max().item())
        tol = FP32_REL * mag if dtype == torch.float32 else HALF_ABS * mag
        assert err <= tol, f"{name}: {err:.3e} > {tol:.3e}"


def test_no_alloc_backward_matches_regular_backward_twice_in_a_row():
    # first call: larger problem, both cotangents, fp32
    _case(torch.float32, 2, 3, 192, 64, causal=False, seed=1, both=True)
    # second call: smaller, other dtype and mask; stale rows of call one sit behind its range
    _case(torch.bfloat16, 1, 2, 96, 128, causal=True, seed=2, both=False)
    # third: same shape as the first again, different values
    _case(torch.float32, 2, 3, 192, 64, causal=True, seed=3, both=True)


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
    assert b"capacity" in lib.jvpfa_strerror(-10)
