// Prefill path placeholder: the tensor-core contraction is built in a later step of this file's history.
#include "common.cuh"
#include "kernels.h"

namespace weft {

bool prefill_supported(int, long long, long long, long long, const void *, const void *) { return false; }

cudaError_t launch_prefill(const PrefillArgs &, int, cudaStream_t) { return cudaErrorNotSupported; }

}  // namespace weft
