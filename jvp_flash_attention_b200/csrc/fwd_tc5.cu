// What the tcgen05 kernels share on the host side: the device status word of the bounded waits (with its host-visible
// mirror), the TMA tensor-map encoders, and the forward dispatch
//   D = 64  -> fwd_tc5_pair64.cu  (two query tiles per CTA share every key stage)
//   D = 128 -> fwd_tc5_pipe128.cu (score products of the next key tile under the softmax of this one)
// Both follow the register-tiled kernel in fwd_generic.cu in what they compute (jvp_attention.py:125-336, 1011-1033).
#include "tc5_common.cuh"

namespace jvpfa {

// [0]: the status word.  [2], [3]: device address of its host-visible mirror (pinned, mapped host memory), written by
// a thread that gives up a wait, so that the host can see a failure without synchronising.
__device__ __align__(16) int g_tc5_status[4] = {0, 0, 0, 0};

namespace {
struct StatusSlot {
  int* dev = nullptr;            // device address of g_tc5_status on that device
  volatile int* mirror = nullptr;  // host address of the mirror (null if it could not be set up)
};
StatusSlot* status_slot() {
  static StatusSlot cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  StatusSlot& sl = cache[dev];
  if (!sl.dev) {
    int* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_tc5_status) != cudaSuccess) return nullptr;
    int* host = nullptr;
    int* host_dev = nullptr;
    if (cudaHostAlloc(reinterpret_cast<void**>(&host), sizeof(int), cudaHostAllocMapped) == cudaSuccess) {
      *host = 0;
      if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&host_dev), host, 0) == cudaSuccess &&
          cudaMemcpy(p + 2, &host_dev, sizeof(host_dev), cudaMemcpyHostToDevice) == cudaSuccess) {
        sl.mirror = host;
      } else {
        cudaFreeHost(host);
      }
    }
    (void)cudaGetLastError();  // a missing mirror only costs the early warning
    sl.dev = p;
  }
  return &sl;
}
}  // namespace

// Device address of the status word on the current device (other translation units receive it
// as a kernel argument).  Looked up once per device.
int* tc5_status_device_ptr() {
  StatusSlot* sl = status_slot();
  return sl ? sl->dev : nullptr;
}

// The mirror's value: non-zero once a kernel on the current device has given up a wait (no CUDA call, no
// synchronisation; it can lag behind the device by the kernels still in flight).
int tc5_status_peek() {
  StatusSlot* sl = status_slot();
  return (sl && sl->mirror) ? *sl->mirror : 0;
}

namespace tc5 {

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

bool encode_map4d(CUtensorMap* m, CUtensorMapDataType dt, const void* ptr, int D, int L, int H, int B, const int64_t* st,
                  int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  const bool dense = st == nullptr || (st[0] == 0 && st[1] == 0 && st[2] == 0);
  const cuuint64_t sb = dense ? (cuuint64_t)H * L * D : (cuuint64_t)st[0];
  const cuuint64_t sh = dense ? (cuuint64_t)L * D : (cuuint64_t)st[1];
  const cuuint64_t sl = dense ? (cuuint64_t)D : (cuuint64_t)st[2];
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)L, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {sl * 2, sh * 2, sb * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(m, dt, 4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Row-major fp32 (B, H, L, D) tensor as a 4-D map with 32-column (128-byte) swizzled boxes: target of TMA reductions.
bool encode_map4d_f32(CUtensorMap* m, const void* ptr, int D, int L, int H, int B, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)L, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)D * 4, (cuuint64_t)L * D * 4, (cuuint64_t)H * L * D * 4};
  cuuint32_t box[4] = {32, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool encode_map4(CUtensorMap* m, CUtensorMapDataType dt, const void* ptr, int L, int H, int B, const int64_t* st,
                 int box_rows) {
  return encode_map4d(m, dt, ptr, 64, L, H, B, st, box_rows);
}

}  // namespace tc5

bool fwd_tc5_eligible(const jvpfa_fwd_args& a) {
  if (a.dtype != JVPFA_BF16 && a.dtype != JVPFA_FP16) return false;
  if (a.D != 64 && a.D != 128) return false;
  // The D = 64 kernel takes the row maximum before scaling and therefore needs a positive softmax scale (any other
  // goes to the register-tiled kernels).
  if (a.D == 64 && !(a.sm_scale > 0.f)) return false;
  const int k = a.mask.kind;
  if (k == JVPFA_MASK_NONE || k == JVPFA_MASK_CAUSAL || k == JVPFA_MASK_KVLEN) return true;
  // Boolean masks and bias: the softmax threads read 16-byte pieces of mask rows
  if ((a.L & 15) != 0) return false;
  if (k == JVPFA_MASK_BIAS && a.mask.bias_dtype != a.dtype) return false;
  const long long esz = k == JVPFA_MASK_BOOL ? 1 : 2;
  if (a.mask.stride[3] != 1 || (reinterpret_cast<uintptr_t>(a.mask.ptr) & 15u) != 0) return false;
  for (int d = 0; d < 3; ++d)
    if (a.mask.stride[d] < 0 || ((a.mask.stride[d] * esz) & 15) != 0) return false;
  return true;
}

int launch_fwd_tc5(const jvpfa_fwd_args& a, cudaStream_t s) {
  if (a.D == 64) return launch_fwd_tc5_pair64(a, s);
  return launch_fwd_tc5_pipe128(a, s);
}

int tc5_read_status(int* out, int clear) {
  StatusSlot* sl = status_slot();
  if (!sl) {
    set_last_cuda_error(cudaErrorUnknown, "status word address");
    return JVPFA_ERR_CUDA;
  }
  int v = 0;
  cudaError_t e = cudaMemcpy(&v, sl->dev, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaMemcpy(status)");
    return JVPFA_ERR_CUDA;
  }
  if (clear && v != 0) {
    const int zero = 0;
    e = cudaMemcpy(sl->dev, &zero, sizeof(int), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
      set_last_cuda_error(e, "cudaMemcpy(status)");
      return JVPFA_ERR_CUDA;
    }
    if (sl->mirror) *sl->mirror = 0;
  }
  *out = v;
  return JVPFA_OK;
}

// Puts `code` into the status word and its mirror from the host, as a kernel that gave up a wait would.
int tc5_inject_status(int code) {
  StatusSlot* sl = status_slot();
  if (!sl) {
    set_last_cuda_error(cudaErrorUnknown, "status word address");
    return JVPFA_ERR_CUDA;
  }
  cudaError_t e = cudaMemcpy(sl->dev, &code, sizeof(int), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaMemcpy(status)");
    return JVPFA_ERR_CUDA;
  }
  if (sl->mirror) *sl->mirror = code;
  return JVPFA_OK;
}

}  // namespace jvpfa
