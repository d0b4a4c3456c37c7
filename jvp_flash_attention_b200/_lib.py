"""ctypes binding of ``libjvpfa.so`` (declared in ``include/jvpfa.h``).

The library is the only compute path of this package: there is no PyTorch, Triton or CPU
fallback.  ``load()`` raises if the shared object is missing, and every launch helper raises
``RuntimeError`` on a non-zero status, so a broken build cannot pass silently.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libjvpfa.so"

# enums of include/jvpfa.h
BF16, FP16, FP32 = 0, 1, 2
MASK_NONE, MASK_CAUSAL, MASK_KVLEN, MASK_BOOL, MASK_BIAS = 0, 1, 2, 3, 4
IMPL_AUTO, IMPL_GENERIC, IMPL_TCGEN05 = 0, 1, 2
INDEX_MASKS = (MASK_NONE, MASK_CAUSAL, MASK_KVLEN)  # masks applied by index comparison inside the kernels

DTYPE_ENUM = {torch.bfloat16: BF16, torch.float16: FP16, torch.float32: FP32}
FP32_TF32 = 3  # JVPFA_FP32_TF32: fp32 tensors, products as one TF32 MMA

# How fp32 inputs are multiplied: "3xtf32" (default; error ~1e-6 relative) or "tf32" (one TF32 MMA per product, the
# precision of upstream's fp32 path; error ~5e-4, about 2.5x faster).  Set through jvp_attention.set_fp32_precision.
FP32_PRECISION = "3xtf32"


def compute_enum(t: torch.Tensor, fp32_mode: str | None = None) -> int:
    """jvpfa_dtype for the arithmetic on tensors like ``t``.  ``fp32_mode``: the precision recorded when the call's
    forward ran (so that a backward recomputes the scores exactly as the forward formed them); None = the current
    process-wide setting."""
    if t.dtype == torch.float32 and (fp32_mode or FP32_PRECISION) == "tf32":
        return FP32_TF32
    return DTYPE_ENUM[t.dtype]

EXPORTS = (
    "jvpfa_fwd",
    "jvpfa_bwd_preprocess",
    "jvpfa_bwd",
    "jvpfa_strerror",
    "jvpfa_version",
    "jvpfa_last_cuda_error",
    "jvpfa_fwd_uses_tcgen05",
    "jvpfa_bwd_uses_tcgen05",
    "jvpfa_device_status",
    "jvpfa_device_status_inject",
    "jvpfa_bwd_noalloc",
    "jvpfa_mask_check",
    "jvpfa_mask_tiles",
)

NOALLOC_MAX_ROWS = 524288  # JVPFA_NOALLOC_MAX_ROWS


class Mask(C.Structure):
    _fields_ = [
        ("kind", C.c_int32),
        ("bias_dtype", C.c_int32),
        ("ptr", C.c_void_p),
        ("stride", C.c_int64 * 4),
        ("kv_len", C.c_void_p),
    ]


class FwdArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_int32),
        ("dtype", C.c_int32),
        ("B", C.c_int32),
        ("H", C.c_int32),
        ("L", C.c_int32),
        ("D", C.c_int32),
        ("impl", C.c_int32),
        ("sm_scale", C.c_float),
        ("q", C.c_void_p),
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("tq", C.c_void_p),
        ("tk", C.c_void_p),
        ("tv", C.c_void_p),
        ("o", C.c_void_p),
        ("to", C.c_void_p),
        ("lse", C.c_void_p),
        ("mu", C.c_void_p),
        ("mask", Mask),
        ("in_stride", C.c_int64 * 3),
        ("mask_tile_live", C.c_void_p),
    ]


class PreArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_int32),
        ("dtype", C.c_int32),
        ("B", C.c_int32),
        ("H", C.c_int32),
        ("L", C.c_int32),
        ("D", C.c_int32),
        ("o", C.c_void_p),
        ("to", C.c_void_p),
        ("go", C.c_void_p),
        ("gto", C.c_void_p),
        ("mu", C.c_void_p),
        ("delta", C.c_void_p),
        ("eps", C.c_void_p),
        ("cterm", C.c_void_p),
    ]


class BwdArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_int32),
        ("dtype", C.c_int32),
        ("B", C.c_int32),
        ("H", C.c_int32),
        ("L", C.c_int32),
        ("D", C.c_int32),
        ("impl", C.c_int32),
        ("sm_scale", C.c_float),
        ("q", C.c_void_p),
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("tq", C.c_void_p),
        ("tk", C.c_void_p),
        ("tv", C.c_void_p),
        ("go", C.c_void_p),
        ("gto", C.c_void_p),
        ("lse", C.c_void_p),
        ("mu", C.c_void_p),
        ("delta", C.c_void_p),
        ("eps", C.c_void_p),
        ("cterm", C.c_void_p),
        ("dq", C.c_void_p),
        ("dk", C.c_void_p),
        ("dv", C.c_void_p),
        ("mask", Mask),
        ("in_stride", C.c_int64 * 3),
        ("mask_tile_live", C.c_void_p),
        ("mask_tile_live_t", C.c_void_p),
        ("dq_accum", C.c_void_p),
    ]


class BwdNoAllocArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_int32),
        ("dtype", C.c_int32),
        ("B", C.c_int32),
        ("H", C.c_int32),
        ("L", C.c_int32),
        ("D", C.c_int32),
        ("impl", C.c_int32),
        ("sm_scale", C.c_float),
        ("q", C.c_void_p),
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("tq", C.c_void_p),
        ("tk", C.c_void_p),
        ("tv", C.c_void_p),
        ("o", C.c_void_p),
        ("to", C.c_void_p),
        ("go", C.c_void_p),
        ("gto", C.c_void_p),
        ("lse", C.c_void_p),
        ("mu", C.c_void_p),
        ("dq", C.c_void_p),
        ("dk", C.c_void_p),
        ("dv", C.c_void_p),
        ("mask", Mask),
    ]


class MaskCheckArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_int32),
        ("n_b", C.c_int32),
        ("n_h", C.c_int32),
        ("n_rows", C.c_int32),
        ("L", C.c_int32),
        ("mask", Mask),
        ("out", C.c_void_p),
    ]


class MaskTilesArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_int32),
        ("n_b", C.c_int32),
        ("n_h", C.c_int32),
        ("n_rows", C.c_int32),
        ("L", C.c_int32),
        ("mask", Mask),
        ("tile_live", C.c_void_p),
        ("head_live", C.c_void_p),
        ("tile_live_t", C.c_void_p),
    ]


_lib = None


def load() -> C.CDLL:
    """Loads libjvpfa.so once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m jvp_flash_attention_b200.build` "
            "(this package has no fallback path)"
        )
    lib = C.CDLL(str(LIB_PATH))
    lib.jvpfa_fwd.argtypes = [C.POINTER(FwdArgs), C.c_void_p]
    lib.jvpfa_fwd.restype = C.c_int
    lib.jvpfa_bwd_preprocess.argtypes = [C.POINTER(PreArgs), C.c_void_p]
    lib.jvpfa_bwd_preprocess.restype = C.c_int
    lib.jvpfa_bwd.argtypes = [C.POINTER(BwdArgs), C.c_void_p]
    lib.jvpfa_bwd.restype = C.c_int
    lib.jvpfa_strerror.argtypes = [C.c_int]
    lib.jvpfa_strerror.restype = C.c_char_p
    lib.jvpfa_version.argtypes = []
    lib.jvpfa_version.restype = C.c_int
    lib.jvpfa_last_cuda_error.argtypes = []
    lib.jvpfa_last_cuda_error.restype = C.c_char_p
    lib.jvpfa_fwd_uses_tcgen05.argtypes = [C.POINTER(FwdArgs)]
    lib.jvpfa_fwd_uses_tcgen05.restype = C.c_int
    lib.jvpfa_bwd_uses_tcgen05.argtypes = [C.POINTER(BwdArgs)]
    lib.jvpfa_bwd_uses_tcgen05.restype = C.c_int
    lib.jvpfa_device_status.argtypes = [C.POINTER(C.c_int), C.c_int]
    lib.jvpfa_device_status.restype = C.c_int
    lib.jvpfa_device_status_inject.argtypes = [C.c_int]
    lib.jvpfa_device_status_inject.restype = C.c_int
    lib.jvpfa_bwd_noalloc.argtypes = [C.POINTER(BwdNoAllocArgs), C.c_void_p]
    lib.jvpfa_bwd_noalloc.restype = C.c_int
    lib.jvpfa_mask_check.argtypes = [C.POINTER(MaskCheckArgs), C.c_void_p]
    lib.jvpfa_mask_check.restype = C.c_int
    lib.jvpfa_mask_tiles.argtypes = [C.POINTER(MaskTilesArgs), C.c_void_p]
    lib.jvpfa_mask_tiles.restype = C.c_int
    _lib = lib
    return lib


def device_status(clear: bool = True) -> int:
    """Synchronises and returns the status word of the tcgen05 kernels (0 = no wait gave up)."""
    lib = load()
    out = C.c_int(0)
    check(lib.jvpfa_device_status(C.byref(out), 1 if clear else 0), "jvpfa_device_status")
    return out.value


def device_status_inject(code: int) -> None:
    """Sets the status word from the host as a kernel that gave up a wait would (``jvpfa_device_status_inject``):
    every tcgen05 call then fails with JVPFA_ERR_DEVICE_STATUS until ``device_status(clear=True)``."""
    check(load().jvpfa_device_status_inject(int(code)), "jvpfa_device_status_inject")


def check(status: int, what: str) -> None:
    """Raises RuntimeError with the library's message when ``status`` is not JVPFA_OK."""
    if status != 0:
        lib = load()
        msg = lib.jvpfa_strerror(status).decode()
        cuda = lib.jvpfa_last_cuda_error().decode()
        raise RuntimeError(f"{what} failed: [{status}] {msg}" + (f" | {cuda}" if cuda else ""))


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


class MaskSpec:
    """Host description of the mask handed to the kernels.

    ``kind`` is one of the MASK_* enums; ``tensor`` keeps the device buffer alive (uint8 mask,
    bias, or int32 kv_len) and ``strides`` are the broadcast element strides of a (B,H,L,L) view.
    """

    __slots__ = ("kind", "tensor", "strides", "bias_dtype", "tile_live", "tile_live_t", "fp32_mode")

    def __init__(self, kind=MASK_NONE, tensor=None, strides=(0, 0, 0, 0), bias_dtype=FP32):
        self.kind = kind
        self.tensor = tensor
        self.strides = tuple(int(s) for s in strides)
        self.bias_dtype = bias_dtype
        self.tile_live = None  # MASK_BOOL: bitmap from mask_tiles(), lets the forward step over dead tiles
        self.tile_live_t = None  # ... and its transpose (per 128-key tile), for the backward launch that owns keys
        self.fp32_mode = None  # fp32 precision the forward of this call ran under ("3xtf32" / "tf32"); None = current

    def to_c(self) -> Mask:
        m = Mask()
        m.kind = self.kind
        m.bias_dtype = self.bias_dtype
        m.ptr = None
        m.kv_len = None
        for i in range(4):
            m.stride[i] = self.strides[i]
        if self.kind == MASK_KVLEN:
            m.kv_len = self.tensor.data_ptr()
        elif self.kind in (MASK_BOOL, MASK_BIAS):
            m.ptr = self.tensor.data_ptr()
        return m


def _launch(t: torch.Tensor, entry, args) -> int:
    """Calls a library entry point with ``t``'s device current and its current stream.  Switching the device
    through the context manager costs a few microseconds, so it is done only when another device is current."""
    if t.device.index == torch.cuda.current_device():
        return entry(C.byref(args), _stream(t))
    with torch.cuda.device(t.device):
        return entry(C.byref(args), _stream(t))


def _stream(t: torch.Tensor) -> int:
    # the raw handle of the device's current stream, without building a torch.cuda.Stream object (~3 us per call)
    return torch._C._cuda_getCurrentRawStream(t.device.index)


ERR_UNSUPPORTED = -9


class Unsupported(RuntimeError):
    """The library understood the request but this build cannot serve it (JVPFA_ERR_UNSUPPORTED)."""


def common_strides(*ts) -> tuple[int, int, int] | None:
    """(batch, head, row) element strides shared by the given (B,H,L,D) tensors, or None when they are all
    row-major.  Raises ValueError when the tensors disagree or the layout cannot be described that way
    (last dimension not contiguous, strides not multiples of 8 elements, base not 16-byte aligned)."""
    ts = [t for t in ts if t is not None]
    if all(t.is_contiguous() for t in ts):
        return None
    st = ts[0].stride()
    for t in ts:
        if t.stride() != st or t.stride(-1) != 1 or any(x <= 0 or x % 8 for x in t.stride()[:3]) or t.data_ptr() % 16:
            raise ValueError("layouts differ or are not expressible as (batch, head, row) strides")
    return st[0], st[1], st[2]


def fwd(q, k, v, tq, tk, tv, o, to, lse, mu, mask: MaskSpec, sm_scale: float, impl: int = IMPL_AUTO,
        in_stride: tuple[int, int, int] | None = None) -> None:
    """Launches jvpfa_fwd on the current stream of ``q``'s device.  Outputs are contiguous BHLD; the inputs too,
    unless ``in_stride`` gives their common (batch, head, row) element strides."""
    lib = load()
    B, H, L, D = q.shape
    a = FwdArgs()
    a.struct_size = C.sizeof(FwdArgs)
    a.dtype = compute_enum(q, mask.fp32_mode)
    a.B, a.H, a.L, a.D = B, H, L, D
    a.impl = impl
    a.sm_scale = sm_scale
    a.q, a.k, a.v = ptr(q), ptr(k), ptr(v)
    a.tq, a.tk, a.tv = ptr(tq), ptr(tk), ptr(tv)
    a.o, a.to, a.lse, a.mu = ptr(o), ptr(to), ptr(lse), ptr(mu)
    a.mask = mask.to_c()
    a.mask_tile_live = ptr(mask.tile_live)
    if in_stride is not None:
        a.in_stride[0], a.in_stride[1], a.in_stride[2] = in_stride
    rc = _launch(q, lib.jvpfa_fwd, a)
    if rc == ERR_UNSUPPORTED and in_stride is not None:
        raise Unsupported("jvpfa_fwd cannot read this layout in place")
    check(rc, "jvpfa_fwd")


def mask_check(mask: "MaskSpec", shape) -> tuple[bool, bool]:
    """Launches jvpfa_mask_check over a boolean or floating-point mask of the given own shape
    (n_b, n_h, n_rows, L) and reads the answer back (one synchronisation).  Returns
    ``(every head has a live entry, an inf is present, a NaN is present)``."""
    lib = load()
    t = mask.tensor
    n_b, n_h, n_rows, L = (int(x) for x in shape)
    out = torch.zeros(1 + n_b * n_h, device=t.device, dtype=torch.int32)
    a = MaskCheckArgs()
    a.struct_size = C.sizeof(MaskCheckArgs)
    a.n_b, a.n_h, a.n_rows, a.L = n_b, n_h, n_rows, L
    a.mask = mask.to_c()
    a.out = out.data_ptr()
    check(_launch(t, lib.jvpfa_mask_check, a), "jvpfa_mask_check")
    flags = out.tolist()
    return all(flags[1:]), bool(flags[0] & 1), bool(flags[0] & 2)


def mask_tiles(mask: "MaskSpec", L: int):
    """Launches jvpfa_mask_tiles over a boolean mask (no synchronisation).  Returns ``(tile_live, head_live,
    tile_live_t)``: the int64 bitmap of 128 x 64 tiles with a true entry, which jvpfa_fwd / jvpfa_bwd take for block
    skipping, the int32 per-head flags followed by the count of live tiles, and the bitmap per 128-key tile.  The mask's own extents follow its strides (0 = broadcast).  Raises Unsupported when the
    layout cannot be read as 16-byte pieces (key stride, alignment, L % 16)."""
    lib = load()
    t = mask.tensor
    n_b, n_h = (t.shape[d] if mask.strides[d] else 1 for d in (0, 1))
    n_rows = L if mask.strides[2] else 1
    n_qt = 1 if n_rows == 1 else (L + 127) // 128
    n_words = ((L + 63) // 64 + 63) // 64
    n_bitmap = n_b * n_h * n_qt * n_words * 2
    n_bitmap_t = n_b * n_h * ((L + 127) // 128) * ((n_qt + 63) // 64) * 2
    buf = torch.zeros(n_bitmap + n_bitmap_t + n_b * n_h + 1, device=t.device, dtype=torch.int32)  # one memset for all
    tile_live = buf[:n_bitmap].view(torch.int64)
    tile_live_t = buf[n_bitmap:n_bitmap + n_bitmap_t].view(torch.int64)
    head_live = buf[n_bitmap + n_bitmap_t:]
    a = MaskTilesArgs()
    a.struct_size = C.sizeof(MaskTilesArgs)
    a.n_b, a.n_h, a.n_rows, a.L = n_b, n_h, n_rows, L
    a.mask = mask.to_c()
    a.tile_live = tile_live.data_ptr()
    a.head_live = head_live.data_ptr()
    a.tile_live_t = tile_live_t.data_ptr()
    rc = _launch(t, lib.jvpfa_mask_tiles, a)
    if rc == ERR_UNSUPPORTED:
        raise Unsupported("jvpfa_mask_tiles cannot read this mask layout")
    check(rc, "jvpfa_mask_tiles")
    return tile_live, head_live, tile_live_t


def bwd_preprocess(o, to, go, gto, mu, delta, eps, cterm, fp32_mode: str | None = None) -> None:
    """Launches jvpfa_bwd_preprocess (row reductions delta / eps / cterm)."""
    lib = load()
    B, H, L, D = o.shape
    a = PreArgs()
    a.struct_size = C.sizeof(PreArgs)
    a.dtype = compute_enum(o, fp32_mode)
    a.B, a.H, a.L, a.D = B, H, L, D
    a.o, a.to, a.go, a.gto = ptr(o), ptr(to), ptr(go), ptr(gto)
    a.mu, a.delta, a.eps, a.cterm = ptr(mu), ptr(delta), ptr(eps), ptr(cterm)
    check(_launch(o, lib.jvpfa_bwd_preprocess, a), "jvpfa_bwd_preprocess")


def bwd(q, k, v, tq, tk, tv, go, gto, lse, mu, delta, eps, cterm, dq, dk, dv, mask: MaskSpec,
        sm_scale: float, impl: int = IMPL_AUTO, in_stride: tuple[int, int, int] | None = None,
        dq_accum: torch.Tensor | None = None) -> None:
    """Launches jvpfa_bwd (gradients of <go,O> + <gto,tO> w.r.t. q, k, v).  ``dq_accum``: optional fp32 scratch of
    q's shape; with it the library may run its single-pass backward (see jvpfa_bwd_args.dq_accum)."""
    lib = load()
    B, H, L, D = q.shape
    a = BwdArgs()
    a.struct_size = C.sizeof(BwdArgs)
    a.dtype = compute_enum(q, mask.fp32_mode)
    a.B, a.H, a.L, a.D = B, H, L, D
    a.impl = impl
    a.sm_scale = sm_scale
    a.q, a.k, a.v = ptr(q), ptr(k), ptr(v)
    a.tq, a.tk, a.tv = ptr(tq), ptr(tk), ptr(tv)
    a.go, a.gto = ptr(go), ptr(gto)
    a.lse, a.mu = ptr(lse), ptr(mu)
    a.delta, a.eps, a.cterm = ptr(delta), ptr(eps), ptr(cterm)
    a.dq, a.dk, a.dv = ptr(dq), ptr(dk), ptr(dv)
    a.mask = mask.to_c()
    if mask.tile_live is not None and mask.tile_live_t is not None and L <= 8192:
        a.mask_tile_live, a.mask_tile_live_t = ptr(mask.tile_live), ptr(mask.tile_live_t)
    if in_stride is not None:
        a.in_stride[0], a.in_stride[1], a.in_stride[2] = in_stride
    a.dq_accum = ptr(dq_accum)
    rc = _launch(q, lib.jvpfa_bwd, a)
    if rc == ERR_UNSUPPORTED and in_stride is not None:
        raise Unsupported("jvpfa_bwd cannot read this layout in place")
    check(rc, "jvpfa_bwd")


def bwd_noalloc(q, k, v, tq, tk, tv, o, to, go, gto, lse, mu, dq, dk, dv, mask: MaskSpec, sm_scale: float,
                impl: int = IMPL_AUTO) -> None:
    """Launches jvpfa_bwd_noalloc: the backward for callers that cannot allocate device memory.

    Same gradients as ``bwd_preprocess`` + ``bwd``, but the three (B,H,L) scratch rows live in a
    fixed 6 MiB array inside libjvpfa.so, so the caller passes only inputs and outputs.
    B*H*L must not exceed ``NOALLOC_MAX_ROWS``; calls on one device share the array and must
    not overlap on the GPU; the first call per device should precede any stream capture."""
    lib = load()
    B, H, L, D = q.shape
    a = BwdNoAllocArgs()
    a.struct_size = C.sizeof(BwdNoAllocArgs)
    a.dtype = compute_enum(q, mask.fp32_mode)
    a.B, a.H, a.L, a.D = B, H, L, D
    a.impl = impl
    a.sm_scale = sm_scale
    a.q, a.k, a.v = ptr(q), ptr(k), ptr(v)
    a.tq, a.tk, a.tv = ptr(tq), ptr(tk), ptr(tv)
    a.o, a.to, a.go, a.gto = ptr(o), ptr(to), ptr(go), ptr(gto)
    a.lse, a.mu = ptr(lse), ptr(mu)
    a.dq, a.dk, a.dv = ptr(dq), ptr(dk), ptr(dv)
    a.mask = mask.to_c()
    check(_launch(q, lib.jvpfa_bwd_noalloc, a), "jvpfa_bwd_noalloc")
