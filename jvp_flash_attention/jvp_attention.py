"""``jvp_flash_attention.jvp_attention`` -- the import path of upstream's module (README: ``from
jvp_flash_attention.jvp_attention import JVPAttn, attention``), served by the sm_100a implementation.

Code written against upstream keeps its imports: every public name of upstream's module
(jvp_flash_attention/jvp_attention.py:48-91, 2236-2981) is re-exported from
``jvp_flash_attention_b200.jvp_attention``, where the implementation and its documentation live.
"""
from jvp_flash_attention_b200.jvp_attention import (  # noqa: F401
    MASK_CONST,
    MIN_SEQUENCE_LENGTH,
    JVPAttn,
    attention,
    is_blackwell,
    is_cuda,
    is_hip,
    scaled_dot_product_attention,
    set_fp32_precision,
    supports_host_descriptor,
    supports_tma,
)

__all__ = [
    "MASK_CONST", "MIN_SEQUENCE_LENGTH", "JVPAttn", "attention", "is_hip", "is_cuda", "supports_host_descriptor",
    "supports_tma", "is_blackwell", "scaled_dot_product_attention", "set_fp32_precision",
]
