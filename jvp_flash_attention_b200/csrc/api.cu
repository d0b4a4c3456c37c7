// C ABI of libjvpfa.so: argument validation and dispatch.  No allocation, no device
// synchronisation, no exceptions across the boundary.
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace jvpfa {

static thread_local char g_last_cuda_error[256] = {0};

void set_last_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s: %s (%s)", where, cudaGetErrorName(e),
           cudaGetErrorString(e));
}

static int check_arch() {
  static thread_local int cached_dev = -1;
  static thread_local int cached_ok = 0;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaGetDevice");
    return JVPFA_ERR_CUDA;
  }
  if (dev != cached_dev) {
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) {
      set_last_cuda_error(e, "cudaDeviceGetAttribute");
      return JVPFA_ERR_CUDA;
    }
    cached_dev = dev;
    cached_ok = (major == 10);
  }
  return cached_ok ? JVPFA_OK : JVPFA_ERR_ARCH;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int check_shape(int dtype, int B, int H, int L, int D) {
  if (dtype != JVPFA_BF16 && dtype != JVPFA_FP16 && dtype != JVPFA_FP32 && dtype != JVPFA_FP32_TF32) return JVPFA_ERR_DTYPE;
  if (B < 1 || H < 1 || L < 1) return JVPFA_ERR_SHAPE;
  if (D != 32 && D != 64 && D != 128) return JVPFA_ERR_SHAPE;
  if ((long long)B * H > 65535LL) return JVPFA_ERR_TOO_LARGE;  // grid.y limit
  if ((long long)B * H > 2147483647LL / L) return JVPFA_ERR_TOO_LARGE;  // row index fits int32
  return JVPFA_OK;
}

static int check_mask(const jvpfa_mask& m) {
  switch (m.kind) {
    case JVPFA_MASK_NONE:
    case JVPFA_MASK_CAUSAL:
      return JVPFA_OK;
    case JVPFA_MASK_KVLEN:
      return m.kv_len ? JVPFA_OK : JVPFA_ERR_MASK;
    case JVPFA_MASK_BOOL:
      return m.ptr ? JVPFA_OK : JVPFA_ERR_MASK;
    case JVPFA_MASK_BIAS:
      if (!m.ptr) return JVPFA_ERR_MASK;
      if (m.bias_dtype != JVPFA_BF16 && m.bias_dtype != JVPFA_FP16 && m.bias_dtype != JVPFA_FP32)
        return JVPFA_ERR_MASK;
      return JVPFA_OK;
    default:
      return JVPFA_ERR_MASK;
  }
}

// in_stride: all zero (row-major) or three positive multiples of 8 elements (16 bytes, a TMA requirement)
static bool has_strides(const int64_t* st) { return (st[0] | st[1] | st[2]) != 0; }
static int check_strides(const int64_t* st) {
  if (!has_strides(st)) return JVPFA_OK;
  for (int i = 0; i < 3; ++i)
    if (st[i] <= 0 || (st[i] & 7) != 0) return JVPFA_ERR_SHAPE;
  return JVPFA_OK;
}

static int validate_fwd(const jvpfa_fwd_args* a) {
  if (!a) return JVPFA_ERR_NULL;
  if (a->struct_size != (int32_t)sizeof(jvpfa_fwd_args)) return JVPFA_ERR_STRUCT;
  int rc = check_shape(a->dtype, a->B, a->H, a->L, a->D);
  if (rc) return rc;
  if (!a->q || !a->k || !a->v || !a->o || !a->lse) return JVPFA_ERR_NULL;
  const int nt = (a->tq != nullptr) + (a->tk != nullptr) + (a->tv != nullptr) + (a->to != nullptr) +
                 (a->mu != nullptr);
  if (nt != 0 && nt != 5) return JVPFA_ERR_NULL;
  const void* ptrs[] = {a->q, a->k, a->v, a->tq, a->tk, a->tv, a->o, a->to};
  for (const void* p : ptrs)
    if (p && !aligned16(p)) return JVPFA_ERR_ALIGN;
  if (a->impl < JVPFA_IMPL_AUTO || a->impl > JVPFA_IMPL_TCGEN05) return JVPFA_ERR_UNSUPPORTED;
  rc = check_strides(a->in_stride);
  if (rc) return rc;
  return check_mask(a->mask);
}

static int impl_family(int impl) { return impl; }

static int validate_bwd(const jvpfa_bwd_args* a) {
  if (!a) return JVPFA_ERR_NULL;
  if (a->struct_size != (int32_t)sizeof(jvpfa_bwd_args)) return JVPFA_ERR_STRUCT;
  int rc = check_shape(a->dtype, a->B, a->H, a->L, a->D);
  if (rc) return rc;
  if (!a->q || !a->k || !a->v || !a->lse || !a->delta || !a->dq || !a->dk || !a->dv) return JVPFA_ERR_NULL;
  if (!a->go && !a->gto) return JVPFA_ERR_NULL;
  if (a->gto && (!a->tq || !a->tk || !a->tv || !a->mu || !a->eps || !a->cterm)) return JVPFA_ERR_NULL;
  const void* ptrs[] = {a->q, a->k, a->v, a->tq, a->tk, a->tv, a->go, a->gto, a->dq, a->dk, a->dv};
  for (const void* p : ptrs)
    if (p && !aligned16(p)) return JVPFA_ERR_ALIGN;
  if (a->dq_accum && !aligned16(a->dq_accum)) return JVPFA_ERR_ALIGN;
  if (a->impl < JVPFA_IMPL_AUTO || a->impl > JVPFA_IMPL_TCGEN05) return JVPFA_ERR_UNSUPPORTED;
  rc = check_strides(a->in_stride);
  if (rc) return rc;
  return check_mask(a->mask);
}

static int validate_pre(const jvpfa_pre_args* a) {
  if (!a) return JVPFA_ERR_NULL;
  if (a->struct_size != (int32_t)sizeof(jvpfa_pre_args)) return JVPFA_ERR_STRUCT;
  int rc = check_shape(a->dtype, a->B, a->H, a->L, a->D);
  if (rc) return rc;
  if (!a->o || !a->delta || !a->eps || !a->cterm) return JVPFA_ERR_NULL;
  if (!a->go && !a->gto) return JVPFA_ERR_NULL;
  if (a->gto && (!a->to || !a->mu)) return JVPFA_ERR_NULL;
  const void* ptrs[] = {a->o, a->to, a->go, a->gto};
  for (const void* p : ptrs)
    if (p && !aligned16(p)) return JVPFA_ERR_ALIGN;
  return JVPFA_OK;
}

// Everything jvpfa_bwd_preprocess / jvpfa_bwd check before they launch, without launching: used by callers inside
// the library that issue several launches and must not have run any of them when a later one is refused.
int check_pre_request(const jvpfa_pre_args* a) {
  const int rc = validate_pre(a);
  return rc ? rc : check_arch();
}

int check_bwd_request(const jvpfa_bwd_args* a) {
  int rc = validate_bwd(a);
  if (rc) return rc;
  rc = check_arch();
  if (rc) return rc;
  const bool tc5 = bwd_tc5_eligible(*a);
  const int fam = impl_family(a->impl);
  if (fam == JVPFA_IMPL_TCGEN05 && !tc5) return JVPFA_ERR_UNSUPPORTED;
  return JVPFA_OK;
}

}  // namespace jvpfa

using namespace jvpfa;

extern "C" {

int jvpfa_fwd_uses_tcgen05(const jvpfa_fwd_args* a) {
  if (validate_fwd(a) != JVPFA_OK) return 0;
  if (a->impl == JVPFA_IMPL_GENERIC) return 0;
  return fwd_tc5_eligible(*a) ? 1 : 0;
}

int jvpfa_bwd_uses_tcgen05(const jvpfa_bwd_args* a) {
  if (validate_bwd(a) != JVPFA_OK) return 0;
  if (impl_family(a->impl) == JVPFA_IMPL_GENERIC) return 0;
  return bwd_tc5_eligible(*a) ? 1 : 0;
}

int jvpfa_fwd(const jvpfa_fwd_args* a, void* stream) {
  int rc = validate_fwd(a);
  if (rc) return rc;
  rc = check_arch();
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool tc5 = fwd_tc5_eligible(*a);
  if (a->impl == JVPFA_IMPL_TCGEN05 && !tc5) return JVPFA_ERR_UNSUPPORTED;
  // strided inputs are read in place by both kernel families (tensor maps or plain row strides)
  if (tc5 && a->impl != JVPFA_IMPL_GENERIC) {
    if (tc5_status_peek() != 0) return JVPFA_ERR_DEVICE_STATUS;
    return launch_fwd_tc5(*a, s);
  }
  return launch_fwd_generic(*a, s);
}

int jvpfa_bwd_preprocess(const jvpfa_pre_args* a, void* stream) {
  const int rc = check_pre_request(a);
  if (rc) return rc;
  return launch_pre(*a, static_cast<cudaStream_t>(stream));
}

int jvpfa_bwd(const jvpfa_bwd_args* a, void* stream) {
  const int rc = check_bwd_request(a);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool tc5 = bwd_tc5_eligible(*a);
  const int fam = impl_family(a->impl);
  if (tc5 && fam != JVPFA_IMPL_GENERIC) {
    if (tc5_status_peek() != 0) return JVPFA_ERR_DEVICE_STATUS;
    return launch_bwd_tc5(*a, s);
  }
  return launch_bwd_generic(*a, s);
}

int jvpfa_mask_check(const jvpfa_mask_check_args* a, void* stream) {
  if (!a) return JVPFA_ERR_NULL;
  if (a->struct_size != (int32_t)sizeof(jvpfa_mask_check_args)) return JVPFA_ERR_STRUCT;
  if (a->n_b < 1 || a->n_h < 1 || a->n_rows < 1 || a->L < 1) return JVPFA_ERR_SHAPE;
  if ((long long)a->n_b * a->n_h > 65535LL) return JVPFA_ERR_TOO_LARGE;  // grid.y limit
  if (!a->out) return JVPFA_ERR_NULL;
  if (a->mask.kind != JVPFA_MASK_BOOL && a->mask.kind != JVPFA_MASK_BIAS) return JVPFA_ERR_MASK;
  int rc = check_mask(a->mask);
  if (rc) return rc;
  for (int d = 0; d < 4; ++d)
    if (a->mask.stride[d] < 0) return JVPFA_ERR_MASK;
  rc = check_arch();
  if (rc) return rc;
  return launch_mask_check(*a, static_cast<cudaStream_t>(stream));
}

int jvpfa_mask_tiles(const jvpfa_mask_tiles_args* a, void* stream) {
  if (!a) return JVPFA_ERR_NULL;
  if (a->struct_size != (int32_t)sizeof(jvpfa_mask_tiles_args)) return JVPFA_ERR_STRUCT;
  if (a->n_b < 1 || a->n_h < 1 || a->L < 1 || (a->n_rows != 1 && a->n_rows != a->L)) return JVPFA_ERR_SHAPE;
  if ((long long)a->n_b * a->n_h > 65535LL || (a->L + 127) / 128 > 65535) return JVPFA_ERR_TOO_LARGE;  // grid limits
  if (!a->tile_live) return JVPFA_ERR_NULL;
  if (a->mask.kind != JVPFA_MASK_BOOL || !a->mask.ptr) return JVPFA_ERR_MASK;
  for (int d = 0; d < 4; ++d)
    if (a->mask.stride[d] < 0) return JVPFA_ERR_MASK;
  if (a->mask.stride[3] != 1 || (a->L & 15) != 0 || !aligned16(a->mask.ptr) || (a->mask.stride[0] & 15) != 0 ||
      (a->mask.stride[1] & 15) != 0 || (a->mask.stride[2] & 15) != 0)
    return JVPFA_ERR_UNSUPPORTED;
  const int rc = check_arch();
  if (rc) return rc;
  return launch_mask_tiles(*a, static_cast<cudaStream_t>(stream));
}

int jvpfa_device_status(int* status, int clear) {
  if (!status) return JVPFA_ERR_NULL;
  return tc5_read_status(status, clear);
}

int jvpfa_device_status_inject(int code) {
  const int rc = check_arch();
  if (rc) return rc;
  return tc5_inject_status(code);
}

const char* jvpfa_strerror(int status) {
  switch (status) {
    case JVPFA_OK:
      return "ok";
    case JVPFA_ERR_NULL:
      return "a required pointer is NULL (or tangent pointers are only partly given)";
    case JVPFA_ERR_SHAPE:
      return "unsupported shape: need B,H,L >= 1 and D in {32, 64, 128}";
    case JVPFA_ERR_DTYPE:
      return "unknown dtype";
    case JVPFA_ERR_MASK:
      return "inconsistent mask description";
    case JVPFA_ERR_ARCH:
      return "current CUDA device is not compute capability 10.x (B200)";
    case JVPFA_ERR_CUDA:
      return "CUDA call failed (see jvpfa_last_cuda_error)";
    case JVPFA_ERR_STRUCT:
      return "struct_size mismatch between caller and library";
    case JVPFA_ERR_ALIGN:
      return "tensor base pointer is not 16-byte aligned";
    case JVPFA_ERR_UNSUPPORTED:
      return "request not supported by the selected kernel family";
    case JVPFA_ERR_TOO_LARGE:
      return "problem exceeds a fixed internal capacity";
    case JVPFA_ERR_DEVICE_STATUS:
      return "an earlier tcgen05 launch on this device gave up a bounded wait: its outputs hold NaN; read and clear the "
             "status word with jvpfa_device_status";
    default:
      return "unknown status";
  }
}

int jvpfa_version(void) { return JVPFA_VERSION; }

const char* jvpfa_last_cuda_error(void) { return g_last_cuda_error; }

}  // extern "C"
