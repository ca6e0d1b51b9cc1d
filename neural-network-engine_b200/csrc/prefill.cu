// Tensor-core forward for m > 16 (placeholder until the tcgen05 kernel lands): reports that no
// shape is supported so dispatch uses the streaming kernel.
#include "common.cuh"

namespace nne {
bool prefill_supports(const nne_qlinear *, size_t) { return false; }
int prefill_prepare_layer(nne_qlinear *) { return NNE_OK; }
void prefill_release_layer(nne_qlinear *) {}
int launch_prefill(nne_qlinear *, const float *, float *, size_t, size_t, cudaStream_t) {
    return fail(NNE_ERR_UNSUPPORTED, "tensor-core path not built");
}
}  // namespace nne
