// Tensor-core (tcgen05) kernel of the quantized Blocked-ELL projection for 32x32 blocks.
// Until its shape constraints hold the launcher reports "not taken" and the general kernel
// in qbell_forward.cu runs.
#include "kernels.cuh"

namespace cb200 {

cb200_status launch_qbell_tcgen05(const qbell_view &, const dense_args &, std::int64_t, std::int64_t, int,
                                  cudaStream_t, bool *taken) {
    *taken = false;
    return CB200_STATUS_SUCCESS;
}

} // namespace cb200
