"""Generates tests/golden/sdpa_bias_L64_D32.npz: PyTorch's own scaled_dot_product_attention (math path, float64) with a
general additive float mask, its forward-mode tangent and the gradients of <w1, O> + <w2, tO>.

This pins the meaning this library gives to a float ``attn_mask`` -- softmax(scale * Q K^T + mask), in forward and
backward -- which differs from upstream's for masks that are not {0, -100} (upstream scales the mask with the scores and
drops it in its backward, jvp_attention.py:247-251, 1519-1522).  Run once:  python tests/golden/make_sdpa_bias_golden.py
"""
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent


def main():
    g = torch.Generator().manual_seed(17)
    B, H, L, D = 1, 2, 64, 32
    q, k, v, tq, tk, tv, w1, w2 = [torch.randn(B, H, L, D, generator=g, dtype=torch.float64) for _ in range(8)]
    bias = (1.5 * torch.randn(B, H, L, L, generator=g, dtype=torch.float64)).clamp(-6, 6)
    a = [x.clone().requires_grad_() for x in (q, k, v)]
    with torch.nn.attention.sdpa_kernel(torch.nn.attention.SDPBackend.MATH):
        o, to = torch.func.jvp(lambda q_, k_, v_: F.scaled_dot_product_attention(q_, k_, v_, attn_mask=bias), tuple(a),
                               (tq, tk, tv))
        dq, dk, dv = torch.autograd.grad((o * w1).sum() + (to * w2).sum(), a)
    out = dict(q=q, k=k, v=v, tq=tq, tk=tk, tv=tv, w1=w1, w2=w2, bias=bias, o=o.detach(), to=to.detach(), dq=dq, dk=dk, dv=dv)
    np.savez_compressed(HERE / "sdpa_bias_L64_D32.npz", **{kk: vv.numpy() for kk, vv in out.items()})
    print("wrote sdpa_bias_L64_D32.npz")


if __name__ == "__main__":
    main()
