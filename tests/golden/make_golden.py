"""Generates tests/golden/upstream_*.npz by running upstream's own Triton kernels on CPU tensors.

Run once, in a container that has the upstream checkout and Triton:
    TRITON_INTERPRET=1 python tests/golden/make_golden.py --upstream /path/to/jvp_flash_attention_checkout
With TRITON_INTERPRET=1 Triton executes ``_attn_fwd*`` / ``_attn_bwd*`` in its NumPy interpreter,
so the files hold what upstream's kernels compute (fp32 tile dots), not an approximation of it.
Each file stores the seeded inputs next to the outputs, so the tests never need upstream.
"""
import argparse
import os
import sys
from functools import partial
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"
import numpy as np  # noqa: E402
import torch  # noqa: E402

HERE = Path(__file__).resolve().parent

CASES = {
    # name: (B, H, L, D, mask kind, causal, seed)
    "none_L64_D32": (1, 2, 64, 32, "none", False, 0),
    "causal_L64_D32": (1, 2, 64, 32, "none", True, 1),
    "bool_L64_D32": (1, 2, 64, 32, "bool", False, 2),
    "additive_L64_D32": (1, 2, 64, 32, "additive", False, 3),
    "none_L128_D64": (2, 2, 128, 64, "none", False, 4),
    "causal_L128_D64": (1, 2, 128, 64, "none", True, 5),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--upstream", required=True)
    args = ap.parse_args()
    sys.path.insert(0, args.upstream)
    from jvp_flash_attention.jvp_attention import MASK_CONST, JVPAttn  # noqa: E402

    for name, (B, H, L, D, mkind, causal, seed) in CASES.items():
        g = torch.Generator().manual_seed(seed)
        q, k, v, tq, tk, tv, w = [torch.randn(B, H, L, D, generator=g) for _ in range(7)]
        mask = None
        if mkind == "bool":
            mask = torch.rand(B, H, L, L, generator=g) > 0.5
        elif mkind == "additive":
            mask = torch.where(torch.rand(B, H, L, L, generator=g) > 0.5, 0.0, MASK_CONST)
        qp, kp, vp = [x.clone().requires_grad_() for x in (q, k, v)]
        op, ot = torch.func.jvp(partial(JVPAttn.fwd_dual, attn_mask=mask, causal=causal), (qp, kp, vp), (tq, tk, tv))
        (op * w).sum().backward()
        out = dict(q=q, k=k, v=v, tq=tq, tk=tk, tv=tv, w=w, o=op.detach(), to=ot.detach(), dq=qp.grad, dk=kp.grad,
                   dv=vp.grad)
        if mask is not None:
            out["mask"] = mask
        np.savez_compressed(HERE / f"upstream_{name}.npz", causal=np.array(causal), mask_kind=np.array(mkind),
                            **{kk: vv.numpy() for kk, vv in out.items()})
        print("wrote", name)


if __name__ == "__main__":
    main()
