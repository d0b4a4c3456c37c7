// Backward of <gO, O> + <gtO, tO> for bf16 / fp16 on tcgen05 tensor cores: which requests the tcgen05 kernels take,
// and which of them.
//   head dimension 64 : bwd_tc5_fused64.cu (one pass; needs the dQ accumulation buffer; index masks, boolean masks
//                       without tile bitmaps, bias through O alone) or bwd_tc5_d64.cu (two launches; every mask kind, steps over dead tiles)
//   head dimension 128: bwd_tc5_pipe128.cu (two launches; every mask kind)
#include "tc5_common.cuh"

namespace jvpfa {

bool bwd_tc5_eligible(const jvpfa_bwd_args& a) {
  if (a.dtype != JVPFA_BF16 && a.dtype != JVPFA_FP16) return false;
  if (a.D != 64 && a.D != 128) return false;
  const int k = a.mask.kind;
  if (k == JVPFA_MASK_NONE || k == JVPFA_MASK_CAUSAL || k == JVPFA_MASK_KVLEN) return true;
  // Boolean masks and bias: the elementwise threads read 16-byte pieces of mask rows
  if ((a.L & 15) != 0) return false;
  if (k == JVPFA_MASK_BIAS && a.mask.bias_dtype != a.dtype) return false;
  const long long esz = k == JVPFA_MASK_BOOL ? 1 : 2;
  if (a.mask.stride[3] != 1 || (reinterpret_cast<uintptr_t>(a.mask.ptr) & 15u) != 0) return false;
  for (int d = 0; d < 3; ++d)
    if (a.mask.stride[d] < 0 || ((a.mask.stride[d] * esz) & 15) != 0) return false;
  return true;
}

int launch_bwd_tc5(const jvpfa_bwd_args& a, cudaStream_t s) {
  if (a.D == 64) {
    // one pass over the score tiles when the caller gave the dQ accumulation buffer (bwd_tc5_fused64.cu)
    if (bwd_tc5_fused64_eligible(a)) return launch_bwd_tc5_fused64(a, s);
    return launch_bwd_tc5_d64(a, s);  // two pipelined launches (bwd_tc5_d64.cu)
  }
  if (bwd_tc5_pipe128_eligible(a)) return launch_bwd_tc5_pipe128(a, s);  // head dimension 128 (bwd_tc5_pipe128.cu)
  return JVPFA_ERR_UNSUPPORTED;
}

}  // namespace jvpfa
