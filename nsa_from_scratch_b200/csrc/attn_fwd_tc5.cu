// tcgen05 / TMEM / TMA attention forward (performance path).  Placeholder until the kernel lands:
// reports that no shape is supported so that every call takes the generic kernel.
#include "common.cuh"

namespace nsa {

bool attention_fwd_tc5_supports(const nsa_fwd_args&) { return false; }

int attention_fwd_tc5(const nsa_fwd_args&, cudaStream_t) {
  return fail(NSA_ERR_UNSUPPORTED, "attention forward: tcgen05 kernel not built");
}

}  // namespace nsa
