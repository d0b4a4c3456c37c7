/*
 * jvpfa.h -- C ABI of libjvpfa.so: JVP flash attention for NVIDIA B200 (sm_100a).
 *
 * The upstream project (amorehead/jvp_flash_attention) has no native boundary: its
 * kernels are launched through Triton's Python launcher, `kernel[grid](...)`
 * (jvp_flash_attention/jvp_attention.py:2558, 2592, 2921, 2939).  Each entry point
 * below replaces one of those launch sites and is what a ctypes/cffi binding of the
 * Python layer calls instead.
 *
 * Conventions shared by every entry point
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer on the
 *     current CUDA device unless stated otherwise;
 *   - q, k, v, tangents, outputs and gradients are (B, H, L, D) row-major
 *     contiguous (the layout the upstream TMA path requires,
 *     jvp_attention.py:2483-2488, 2858-2877);
 *   - returns JVPFA_OK (0) or a negative jvpfa_status; never throws, never aborts;
 *   - allocates nothing and never synchronises the device: the caller owns every
 *     buffer (scratch included) and the launch is asynchronous on `stream`;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 */
#ifndef JVPFA_H_
#define JVPFA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define JVPFA_VERSION 100 /* major*100 + minor */

typedef enum {
  JVPFA_OK = 0,
  JVPFA_ERR_NULL = -1,        /* a required pointer is NULL                         */
  JVPFA_ERR_SHAPE = -2,       /* B/H/L/D out of range or unsupported head dim       */
  JVPFA_ERR_DTYPE = -3,       /* unknown dtype enum                                 */
  JVPFA_ERR_MASK = -4,        /* inconsistent mask description                      */
  JVPFA_ERR_ARCH = -5,        /* current device is not compute capability 10.x      */
  JVPFA_ERR_CUDA = -6,        /* a CUDA runtime/driver call failed                  */
  JVPFA_ERR_STRUCT = -7,      /* struct_size does not match this library            */
  JVPFA_ERR_ALIGN = -8,       /* a tensor base pointer is not 16-byte aligned       */
  JVPFA_ERR_UNSUPPORTED = -9, /* valid request that this build cannot serve         */
  JVPFA_ERR_TOO_LARGE = -10,  /* problem exceeds a fixed internal capacity          */
  JVPFA_ERR_DEVICE_STATUS = -11 /* an earlier tcgen05 launch gave up a bounded wait; see jvpfa_device_status */
} jvpfa_status;

typedef enum {
  JVPFA_BF16 = 0,
  JVPFA_FP16 = 1,
  JVPFA_FP32 = 2,      /* fp32 tensors; every product as three TF32 MMAs on a hi/lo split (error ~1e-6 relative) */
  JVPFA_FP32_TF32 = 3  /* fp32 tensors; every product as one TF32 MMA, the precision of upstream's fp32 path
                          (tl.dot on TF32 tensor cores, jvp_attention.py:233-236); error ~5e-4 relative, about
                          2.5x faster.  Not a bias dtype: an fp32 bias is JVPFA_FP32. */
} jvpfa_dtype;

/* How scores are masked / biased inside the tile loop. */
typedef enum {
  JVPFA_MASK_NONE = 0,
  JVPFA_MASK_CAUSAL = 1, /* key j attends iff j <= query i; upper tiles are skipped       */
  JVPFA_MASK_KVLEN = 2,  /* key padding: key j attends iff j < kv_len[b]; tiles skipped    */
  JVPFA_MASK_BOOL = 3,   /* uint8 mask, nonzero = attend, broadcast through strides        */
  JVPFA_MASK_BIAS = 4    /* additive bias, SDPA semantics: softmax(scale*QK^T + bias)      */
} jvpfa_mask_kind;

/* Kernel family selection (flags field).  AUTO picks the tcgen05 kernels when the
 * shape qualifies and the portable tensor-core kernels otherwise. */
typedef enum {
  JVPFA_IMPL_AUTO = 0,
  JVPFA_IMPL_GENERIC = 1, /* force the register-tiled mma.sync kernels                    */
  JVPFA_IMPL_TCGEN05 = 2  /* force the TMA + tcgen05/TMEM kernels; error if not eligible  */
} jvpfa_impl;

/* Mask / bias description shared by forward and backward.
 * Element (b, h, i, j) lives at ptr[b*stride[0] + h*stride[1] + i*stride[2] + j*stride[3]]
 * (strides in ELEMENTS; 0 = broadcast along that dimension). */
typedef struct {
  int32_t kind;         /* jvpfa_mask_kind                                            */
  int32_t bias_dtype;   /* JVPFA_MASK_BIAS only: jvpfa_dtype of the bias elements     */
  const void* ptr;      /* BOOL: const uint8_t*; BIAS: bias elements; else NULL       */
  int64_t stride[4];
  const int32_t* kv_len; /* JVPFA_MASK_KVLEN only: (B) valid key counts, 0..L         */
} jvpfa_mask;

/*
 * jvpfa_fwd -- fused primal (+ tangent) attention forward.
 * Replaces the `_attn_fwd_tma[grid](...)` / `_attn_fwd[grid](...)` launches in
 * JVPAttn.forward (jvp_attention.py:2558-2631).
 *
 *   S = sm_scale*Q K^T (+bias), P = softmax(S), O = P V
 *   tS = sm_scale*(tQ K^T + Q tK^T), mu = rowsum(P*tS)
 *   tO = (P*tS) V - mu*O + P tV
 *
 * tq/tk/tv/to/mu are all NULL (primal only) or all non-NULL.
 * lse receives the base-2 logsumexp of the scaled (and biased) scores, the same
 * quantity upstream stores in `M` (jvp_attention.py:1017-1026); rows with no
 * attendable key produce O = tO = 0 (jvp_attention.py:1011-1022) and lse = +inf.
 * mu receives rowsum(P*tS) (already normalised by the softmax denominator).
 */
typedef struct {
  int32_t struct_size; /* sizeof(jvpfa_fwd_args) */
  int32_t dtype;       /* jvpfa_dtype of q,k,v,tq,tk,tv,o,to */
  int32_t B, H, L, D;  /* D in {32, 64, 128}; L >= 1 */
  int32_t impl;        /* jvpfa_impl */
  float sm_scale;
  const void *q, *k, *v;
  const void *tq, *tk, *tv;
  void *o, *to;
  float* lse; /* (B,H,L) */
  float* mu;  /* (B,H,L) or NULL */
  jvpfa_mask mask;
  /* Element strides of the batch, head and row dimensions of q, k, v, tq, tk, tv (all six alike; the
   * head dimension D is always contiguous).  {0,0,0} means (B,H,L,D) row-major.  Anything else, e.g. the
   * (B,H,L,D) view of a (B,L,H,D) tensor, {L*H*D, D, H*D}, is read in place by both kernel families (tensor
   * maps with those strides, or tile loads with the row stride); strides must be positive multiples of 8
   * elements.  Upstream always copies: jvp_attention.py:2733-2734, 2787-2788.  Outputs are always (B,H,L,D)
   * row-major. */
  int64_t in_stride[3];
  /* Optional, JVPFA_MASK_BOOL only: the bitmap written by jvpfa_mask_tiles for this mask.  The tcgen05
   * kernel then steps over 128 x 64 tiles without a true entry; other kernels ignore it.  NULL = none. */
  const void* mask_tile_live;
} jvpfa_fwd_args;

int jvpfa_fwd(const jvpfa_fwd_args* args, void* stream);

/*
 * jvpfa_bwd_preprocess -- per-row reductions needed by jvpfa_bwd.
 * Replaces `_attn_bwd_preprocess[pre_grid](...)` (jvp_attention.py:2921-2928), which
 * computes only delta; the two extra rows exist because this library also
 * differentiates through the tangent output.
 *
 *   delta = rowsum(go*o)                 (0 when go == NULL)
 *   eps   = rowsum(gto*o)                (0 when gto == NULL)
 *   cterm = rowsum(gto*to) - eps*mu      (0 when gto == NULL)
 *
 * go and gto may each be NULL (not both).  to and mu are required iff gto != NULL.
 */
typedef struct {
  int32_t struct_size;
  int32_t dtype;
  int32_t B, H, L, D;
  const void *o, *to;
  const void *go, *gto;
  const float* mu;
  float *delta, *eps, *cterm; /* (B,H,L) each; caller-owned scratch */
} jvpfa_pre_args;

int jvpfa_bwd_preprocess(const jvpfa_pre_args* args, void* stream);

/*
 * jvpfa_bwd -- gradients w.r.t. q, k, v of  <go, O> + <gto, tO>.
 * Replaces `_attn_bwd[grid](...)` / `_attn_bwd_causal[grid](...)`
 * (jvp_attention.py:2932-2974) together with the eager `k * (sm_scale/ln2)`
 * pre-scale (jvp_attention.py:2901-2903), which is folded into the kernels.
 * Upstream differentiates through O only (jvp_attention.py:2831); gto != NULL adds
 * the path through the tangent output and then tq, tk, tv and mu are required.
 * Score tiles are recomputed from lse; nothing of size L x L is stored.
 *
 * delta/eps/cterm must have been produced by jvpfa_bwd_preprocess for the same
 * (o, to, go, gto, mu).  dq, dk, dv are fully overwritten.
 */
typedef struct {
  int32_t struct_size;
  int32_t dtype;
  int32_t B, H, L, D;
  int32_t impl;
  float sm_scale;
  const void *q, *k, *v;
  const void *tq, *tk, *tv; /* required iff gto != NULL */
  const void *go, *gto;     /* either may be NULL, not both */
  const float* lse;
  const float* mu; /* required iff gto != NULL */
  const float *delta, *eps, *cterm;
  void *dq, *dk, *dv;
  jvpfa_mask mask;
  int64_t in_stride[3]; /* of q, k, v, tq, tk, tv, as in jvpfa_fwd_args; go, gto, dq, dk, dv are row-major */
  /* Optional, JVPFA_MASK_BOOL only, both or neither: tile_live and tile_live_t of jvpfa_mask_tiles.  The two-launch
   * tcgen05 kernels (D = 64: L <= 8192) then visit only the loop tiles that overlap a live tile; other kernels ignore
   * them. */
  const void* mask_tile_live;
  const void* mask_tile_live_t;
  /* Optional caller-owned scratch: B*H*L*D floats, 16-byte aligned, contents irrelevant on entry.  With it (D = 64,
   * 16-bit types, mask kinds NONE / CAUSAL / KVLEN, BOOL without the two bitmaps above, or - through O alone - BIAS of
   * the tensors' type) the backward runs as ONE pass that forms every score tile once:
   * dK and dV accumulate on chip, dQ is summed into this buffer with floating-point reductions and converted at the
   * end, so dQ is reproducible to rounding but not bitwise from run to run.  NULL: the two-launch kernels, which
   * recompute the score tiles for dQ (as upstream does, jvp_attention.py:1415-1707) and are bitwise reproducible. */
  float* dq_accum;
} jvpfa_bwd_args;

int jvpfa_bwd(const jvpfa_bwd_args* args, void* stream);

/*
 * jvpfa_bwd_noalloc -- jvpfa_bwd_preprocess + jvpfa_bwd in one call, with the three scratch rows
 * kept inside the library.  It has no counterpart in the reference (whose backward allocates
 * `delta` with torch, jvp_attention.py:2883); it exists for callers that cannot allocate device
 * memory at all: programs whose own pool already owns the whole GPU, loops that must avoid
 * cudaMalloc's device-wide synchronisation, and C-level users of this ABI with no tensor library
 * to provide scratch.
 *
 * Inputs and outputs are the caller's, exactly as for jvpfa_bwd, plus o (and to when gto is
 * given), which the row reductions read.  The scratch is a fixed device array of
 * 3 * JVPFA_NOALLOC_MAX_ROWS floats (6 MiB) that every GPU loading the library holds until
 * process exit.  Limits and rules:
 *   - B*H*L <= JVPFA_NOALLOC_MAX_ROWS, otherwise JVPFA_ERR_TOO_LARGE; this and every argument check of
 *     jvpfa_bwd_preprocess and jvpfa_bwd come before the first launch, so a refused call launches nothing and
 *     leaves the array as it was;
 *   - all calls on one device share the array, so calls that can overlap on the GPU race:
 *     issue them on one stream (or otherwise serialise them);
 *   - the array keeps the last call's contents; no part of it needs to be zero beforehand;
 *   - the first call on each device performs a one-time address look-up for that device and
 *     should therefore be made before any stream capture is begun there;
 *   - no cudaMalloc / cudaFree / allocating library routine is called, on any call.
 */
#define JVPFA_NOALLOC_MAX_ROWS 524288 /* 2^19 (batch*head*query) rows */

typedef struct {
  int32_t struct_size;
  int32_t dtype;
  int32_t B, H, L, D;
  int32_t impl;
  float sm_scale;
  const void *q, *k, *v;
  const void *tq, *tk, *tv; /* required iff gto != NULL */
  const void *o, *to;       /* forward outputs; to required iff gto != NULL */
  const void *go, *gto;     /* either may be NULL, not both */
  const float* lse;
  const float* mu; /* required iff gto != NULL */
  void *dq, *dk, *dv;
  jvpfa_mask mask;
} jvpfa_bwd_noalloc_args;

int jvpfa_bwd_noalloc(const jvpfa_bwd_noalloc_args* args, void* stream);

/*
 * jvpfa_mask_check -- the checks upstream makes on a user mask before a forward, in one pass.
 * Replaces the eager reductions `attn_mask.any(dim=(-1, -2)).all()`, `torch.isinf(attn_mask).any()`,
 * `torch.isnan(attn_mask).any()` and `(attn_mask != MASK_CONST).any(dim=(-1, -2)).all()`
 * (jvp_attention.py:2438-2457), each of which sweeps the whole mask and synchronises with the host.
 *
 * mask describes the tensor as for jvpfa_fwd (kind BOOL or BIAS; strides in elements); n_b, n_h,
 * n_rows are the mask's OWN extents along batch, head and query (1 where it broadcasts), L its key
 * extent.  out points to 1 + n_b*n_h int32 that the caller has zeroed:
 *   out[0]            bit 0: a floating-point mask holds an inf; bit 1: it holds a NaN
 *   out[1 + b*n_h+h]  1 if head (b, h) has an entry that is true (BOOL) / not -100.0 (BIAS)
 * The caller copies out back to the host (the one synchronisation) and raises what upstream raises.
 */
typedef struct {
  int32_t struct_size; /* sizeof(jvpfa_mask_check_args) */
  int32_t n_b, n_h, n_rows, L;
  jvpfa_mask mask;
  int32_t* out;
} jvpfa_mask_check_args;

int jvpfa_mask_check(const jvpfa_mask_check_args* args, void* stream);

/*
 * jvpfa_mask_tiles -- per-tile summary of a boolean mask for block skipping, and the per-head check of
 * jvpfa_mask_check from the same pass.  No upstream counterpart: upstream reads every L x L mask tile
 * in every kernel (jvp_attention.py:453) and has no block skipping.
 *
 * The mask (kind BOOL) must have key stride 1, 16-byte aligned rows and L % 16 == 0 (else
 * JVPFA_ERR_UNSUPPORTED).  n_b, n_h, n_rows are its own extents (1 where it broadcasts, i.e. where its
 * stride is 0; n_rows is 1 or L).  Tiles are 128 queries x 64 keys (one tile row when n_rows == 1).
 *   tile_live  n_b*n_h * n_qt * n_words uint64, n_qt = n_rows == 1 ? 1 : ceil(L/128),
 *              n_words = ceil(ceil(L/64) / 64); bit (t % 64) of word t / 64 of entry [b*n_h + h][qt] is
 *              set iff tile (qt, t) of head (b, h) has a true entry.  Caller zeroes it first.
 *   head_live  n_b*n_h + 1 int32 (caller-zeroed): 1 iff the head has a true entry, and in the last
 *              element the number of live tiles of the whole mask (a caller that reads it back can leave
 *              the bitmap away when nearly every tile is live); may be NULL.
 *   tile_live_t  the same summary the other way round, for the backward launch that owns key tiles:
 *              n_b*n_h * ceil(L/128) * ceil(n_qt/64) uint64 (caller-zeroed); bit (qt % 64) of word qt / 64 of
 *              entry [b*n_h + h][kt] is set iff the 128-query x 128-key tile (qt, kt) has a true entry.  May be NULL.
 */
typedef struct {
  int32_t struct_size; /* sizeof(jvpfa_mask_tiles_args) */
  int32_t n_b, n_h, n_rows, L;
  jvpfa_mask mask;
  void* tile_live;
  int32_t* head_live;
  void* tile_live_t;
} jvpfa_mask_tiles_args;

int jvpfa_mask_tiles(const jvpfa_mask_tiles_args* args, void* stream);

/* Human-readable text for a jvpfa_status (static storage, never NULL). */
const char* jvpfa_strerror(int status);

/* JVPFA_VERSION of the loaded library. */
int jvpfa_version(void);

/* Text of the last CUDA error recorded by this thread inside the library
 * (empty string if none).  Static thread-local storage. */
const char* jvpfa_last_cuda_error(void);

/* Reads the device-side status word of the tcgen05 kernels on the current device into *status:
 * 0 = every bounded wait completed; otherwise the code of the first wait that gave up.  The
 * kernels then drained and exited early, the output rows of the affected CTAs (lse in the
 * forward; dq / dk / dv rows in the backward) hold NaN, and while the word stays non-zero every
 * later tcgen05 launch on the device writes NaN and returns at once.  clear != 0 resets the
 * word.  This call synchronises with the device (it copies the word): poll it where the caller
 * synchronises anyway, not per launch.  A caller that never polls is still told: the thread that
 * gives up also writes the code to a host-visible mirror (pinned, mapped memory), and jvpfa_fwd,
 * jvpfa_bwd and jvpfa_bwd_noalloc look at that mirror (a host read, no synchronisation) before they
 * launch a tcgen05 kernel and return JVPFA_ERR_DEVICE_STATUS while it is non-zero, i.e. from the
 * first call after the failing kernel has run until jvpfa_device_status(.., 1) clears the word.
 * No upstream counterpart: Triton kernels have no such waits. */
int jvpfa_device_status(int* status, int clear);

/* Sets the status word and its mirror to `code` from the host, exactly what a kernel thread that gives
 * up a wait leaves behind (without the NaN rows).  For exercising a caller's handling of
 * JVPFA_ERR_DEVICE_STATUS without a device fault; code 0 is the same as clearing.  Synchronises. */
int jvpfa_device_status_inject(int code);

/* 1 if jvpfa_fwd / jvpfa_bwd with impl == JVPFA_IMPL_AUTO would take the
 * tcgen05 kernels for this shape, else 0 (pure host logic; no CUDA call). */
int jvpfa_fwd_uses_tcgen05(const jvpfa_fwd_args* args);
int jvpfa_bwd_uses_tcgen05(const jvpfa_bwd_args* args);

#ifdef __cplusplus
}
#endif
#endif /* JVPFA_H_ */
