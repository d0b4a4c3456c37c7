"""Seeded synthetic workloads: the five benchmark configurations and (batch x head) sharding.

Inputs are always drawn on the CPU in float32 from ``torch.Generator().manual_seed(seed)`` in the
fixed order q, k, v, tq, tk, tv, extras, then cast, so the CPU oracle and every GPU rank see the
same bits.  The values follow upstream's harness, which measures only on ``torch.randn`` tensors
(tests/test_jvp_attention.py:290-304); no dataset is involved.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class Workload:
    name: str
    dtype: torch.dtype
    B: int
    H: int
    L: int
    D: int
    causal: bool = False
    mask_kind: str = "none"  # none | kvlen | bias
    seed: int = 0
    tangent_std: float = 1.0
    loss: str = "sum_both"  # sum_both | mse_tangent | weighted_both | hvp
    tensors: dict = field(default_factory=dict)

    @property
    def scale(self) -> float:
        return self.D**-0.5

    def attended_pairs(self) -> int:
        """Number of (query, key) pairs that attend: the N_pairs of the FLOP model."""
        if self.causal:
            return self.B * self.H * self.L * (self.L + 1) // 2
        if self.mask_kind == "kvlen":
            return int(self.H * self.L * int(self.tensors["kv_len"].sum()))
        return self.B * self.H * self.L * self.L


SPECS = {
    # name: (dtype, B, H, L, D, causal, mask_kind, seed, tangent_std, loss)
    "c1_fp32_plumbing": (torch.float32, 2, 4, 256, 64, False, "none", 0, 1.0, "sum_both"),
    "c2_bf16_causal": (torch.bfloat16, 4, 16, 2048, 64, True, "none", 1, 0.1, "mse_tangent"),
    "c3_fp16_keypad": (torch.float16, 8, 12, 1024, 64, False, "kvlen", 2, 1.0, "weighted_both"),
    "c4_fp32_bias_hvp": (torch.float32, 2, 8, 1024, 128, False, "bias", 3, 0.5, "hvp"),
    "c5_bf16_long": (torch.bfloat16, 32, 16, 8192, 128, False, "none", 4, 0.1, "weighted_both"),
}


def make_workload(name: str, B: int | None = None, H: int | None = None, L: int | None = None,
                  heads: tuple[int, int] | None = None) -> Workload:
    """Builds a workload on the CPU.  ``B/H/L`` override the size (reduced-size parity cases);
    ``heads=(start, stop)`` builds only that slice of the flattened (batch*head) axis, generated
    per head from ``seed*100003 + bh`` so that any rank can produce its shard independently
    (used by the long-sequence configuration)."""
    dtype, b, h, l, d, causal, mask_kind, seed, tstd, loss = SPECS[name]
    B, H, L = B or b, H or h, L or l
    w = Workload(name, dtype, B, H, L, d, causal, mask_kind, seed, tstd, loss)
    if heads is not None:
        lo, hi = heads
        per = []
        for bh in range(lo, hi):
            g = torch.Generator().manual_seed(seed * 100003 + bh)
            per.append([torch.randn(L, d, generator=g) for _ in range(8)])
        stack = [torch.stack([p[i] for p in per]).unsqueeze(0) for i in range(8)]  # (1, n, L, D)
        names = ["q", "k", "v", "tq", "tk", "tv", "w1", "w2"]
        t = dict(zip(names, stack))
        for n in ("tq", "tk", "tv"):
            t[n] = t[n] * tstd
        w.B, w.H = 1, hi - lo
        w.tensors = {k_: v_.to(dtype) for k_, v_ in t.items()}
        return w
    g = torch.Generator().manual_seed(seed)
    shape = (B, H, L, d)
    t = {n: torch.randn(shape, generator=g) for n in ("q", "k", "v")}
    for n in ("tq", "tk", "tv"):
        t[n] = torch.randn(shape, generator=g) * tstd
    if loss == "mse_tangent":
        t["target"] = torch.randn(shape, generator=g)
    elif loss in ("weighted_both",):
        t["w1"] = torch.randn(shape, generator=g)
        t["w2"] = torch.randn(shape, generator=g)
    elif loss == "hvp":
        t["w"] = torch.randn(shape, generator=g)
        t["v_dir"] = torch.randn(shape, generator=g)
    cast = {k_: v_.to(dtype) for k_, v_ in t.items()}
    if mask_kind == "kvlen":
        lens = torch.randint(L // 2, L + 1, (B,), generator=g)
        cast["kv_len"] = lens
        cast["mask"] = (torch.arange(L)[None, :] < lens[:, None])[:, None, None, :]
    elif mask_kind == "bias":
        cast["mask"] = torch.randn((B, H, L, L), generator=g).clamp_(-5, 5).to(dtype)
    w.tensors = cast
    return w


def make_workload_on_device(name: str, heads: tuple[int, int], device) -> Workload:
    """The (batch*head) units ``heads=(start, stop)`` of a configuration drawn on the GPU itself, one generator per
    unit seeded ``seed*100003 + bh``: a rank produces its shard of the long-sequence configuration without a host
    copy, and any other rank can reproduce one of those units bit for bit on a GPU of the same kind.  (The values
    differ from ``make_workload(..., heads=...)``, which draws on the CPU.)  Tensors: q, k, v, tq, tk, tv, w1, w2 of
    shape (1, stop-start, L, D)."""
    dtype, b, h, l, d, causal, mask_kind, seed, tstd, loss = SPECS[name]
    lo, hi = heads
    w = Workload(name, dtype, 1, hi - lo, l, d, causal, mask_kind, seed, tstd, loss)
    names = ["q", "k", "v", "tq", "tk", "tv", "w1", "w2"]
    out = {n: torch.empty((1, hi - lo, l, d), device=device, dtype=dtype) for n in names}
    g = torch.Generator(device=device)
    for j, bh in enumerate(range(lo, hi)):
        g.manual_seed(seed * 100003 + bh)
        for n in names:
            x = torch.randn((l, d), generator=g, device=device, dtype=torch.float32)
            if n in ("tq", "tk", "tv"):
                x = x * tstd
            out[n][0, j] = x.to(dtype)
    w.tensors = out
    return w


def shard_range(total: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous slice [start, stop) of ``total`` (batch*head) units owned by ``rank``.

    The first ``total % world`` ranks take one extra unit; every unit belongs to exactly one rank
    and a world larger than ``total`` leaves the surplus ranks empty."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, rem = divmod(total, world)
    start = rank * base + min(rank, rem)
    stop = start + base + (1 if rank < rem else 0)
    return start, stop


# MMA-count model: FLOPs = 2 * D * N_pairs * n_mma (softmax and elementwise work excluded).
N_MMA = {"fwd": 2, "fwd_dual": 6, "bwd_o": 5, "bwd_to": 10, "bwd_both": 12}


def flops(w: Workload, stages: tuple[str, ...]) -> float:
    return 2.0 * w.D * w.attended_pairs() * sum(N_MMA[s] for s in stages)
