// jvpfa_bwd_noalloc: backward (row reductions + gradient kernels) for callers that cannot
// allocate device memory.
//
// Who that is: a host program that handed the whole GPU to its own memory pool at start-up (a
// serving runtime, a simulator with a fixed arena) and therefore gets cudaErrorMemoryAllocation
// from any later cudaMalloc; a latency-critical loop that must not hit cudaMalloc's implicit
// device-wide synchronisation; or a plain C / Fortran / Go caller of this ABI that has no tensor
// library to hand it a scratch buffer.  The ordinary pair jvpfa_bwd_preprocess + jvpfa_bwd asks
// such callers for three (B,H,L) fp32 rows of scratch; this entry point keeps that scratch inside
// the library instead, in a fixed array that lives in the module's device data segment.
//
// Consequences the caller has to know:
//  * the array costs 6 MiB of every GPU that loads libjvpfa.so, from load until process exit;
//  * B*H*L may not exceed JVPFA_NOALLOC_MAX_ROWS (larger problems are refused with
//    JVPFA_ERR_TOO_LARGE, nothing is launched);
//  * every call on a device shares the one array: two calls whose kernels may overlap on the GPU
//    (different streams, different host threads) race on it.  Serialise them on one stream;
//  * the array keeps the previous call's rows.  Nothing in it has to start at zero: the reduction
//    kernel overwrites rows [0, B*H*L) of each of the three sections before the gradient kernels
//    read them, and nothing beyond that range is read;
//  * the first call on each device looks up the array's device address (set-up, see below).  Make
//    that first call before starting any stream capture on that device.
#include <mutex>

#include "common.cuh"

namespace jvpfa {

constexpr long long kNoAllocMaxRows = JVPFA_NOALLOC_MAX_ROWS;
constexpr int kNoAllocMaxDevices = 64;

// delta | eps | cterm, kNoAllocMaxRows floats each.
static __device__ __align__(256) float g_noalloc_scratch[3 * kNoAllocMaxRows];

static std::mutex g_noalloc_mutex;
static float* g_noalloc_addr[kNoAllocMaxDevices] = {};

// In host code `g_noalloc_scratch` is only a handle for the runtime, not an address a kernel can
// use.  The usable device address differs per GPU and is fetched once per device, with that
// device current, through cudaGetSymbolAddress.
static int noalloc_scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    set_last_cuda_error(e, "cudaGetDevice(noalloc)");
    return JVPFA_ERR_CUDA;
  }
  if (dev < 0 || dev >= kNoAllocMaxDevices) return JVPFA_ERR_TOO_LARGE;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_last_cuda_error(e, "cudaGetSymbolAddress(noalloc scratch)");
      return JVPFA_ERR_CUDA;
    }
    g_noalloc_addr[dev] = static_cast<float*>(p);
  }
  *out = g_noalloc_addr[dev];
  return JVPFA_OK;
}

}  // namespace jvpfa

using namespace jvpfa;

extern "C" int jvpfa_bwd_noalloc(const jvpfa_bwd_noalloc_args* a, void* stream) {
  if (!a) return JVPFA_ERR_NULL;
  if (a->struct_size != (int32_t)sizeof(jvpfa_bwd_noalloc_args)) return JVPFA_ERR_STRUCT;
  if (a->B < 1 || a->H < 1 || a->L < 1) return JVPFA_ERR_SHAPE;
  const long long rows = (long long)a->B * a->H * a->L;
  if (rows > kNoAllocMaxRows) return JVPFA_ERR_TOO_LARGE;

  float* scratch = nullptr;
  int rc = noalloc_scratch_for_current_device(&scratch);
  if (rc) return rc;
  float* delta = scratch;
  float* eps = scratch + kNoAllocMaxRows;
  float* cterm = scratch + 2 * kNoAllocMaxRows;

  jvpfa_pre_args p{};
  p.struct_size = (int32_t)sizeof(p);
  p.dtype = a->dtype;
  p.B = a->B, p.H = a->H, p.L = a->L, p.D = a->D;
  p.o = a->o, p.to = a->gto ? a->to : nullptr;
  p.go = a->go, p.gto = a->gto;
  p.mu = a->gto ? a->mu : nullptr;
  p.delta = delta, p.eps = eps, p.cterm = cterm;

  jvpfa_bwd_args g{};
  g.struct_size = (int32_t)sizeof(g);
  g.dtype = a->dtype;
  g.B = a->B, g.H = a->H, g.L = a->L, g.D = a->D;
  g.impl = a->impl;
  g.sm_scale = a->sm_scale;
  g.q = a->q, g.k = a->k, g.v = a->v;
  g.tq = a->gto ? a->tq : nullptr, g.tk = a->gto ? a->tk : nullptr, g.tv = a->gto ? a->tv : nullptr;
  g.go = a->go, g.gto = a->gto;
  g.lse = a->lse, g.mu = a->gto ? a->mu : nullptr;
  g.delta = delta, g.eps = eps, g.cterm = cterm;
  g.dq = a->dq, g.dk = a->dk, g.dv = a->dv;
  g.mask = a->mask;
  // Both requests are checked in full before the first launch: a refused call leaves the shared array untouched.
  rc = check_pre_request(&p);
  if (rc) return rc;
  rc = check_bwd_request(&g);
  if (rc) return rc;
  if (jvpfa_bwd_uses_tcgen05(&g) && tc5_status_peek() != 0) return JVPFA_ERR_DEVICE_STATUS;
  rc = jvpfa_bwd_preprocess(&p, stream);
  if (rc) return rc;
  return jvpfa_bwd(&g, stream);
}
