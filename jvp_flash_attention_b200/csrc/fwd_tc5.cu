// Placeholder translation unit for the TMA + tcgen05 forward (filled in separately).
#include "common.cuh"
namespace jvpfa {
bool fwd_tc5_eligible(const jvpfa_fwd_args&) { return false; }
int launch_fwd_tc5(const jvpfa_fwd_args&, cudaStream_t) { return JVPFA_ERR_UNSUPPORTED; }
}  // namespace jvpfa
