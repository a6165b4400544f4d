// decode_kernel for V codes stored in 3 bit(s): one translation unit per stored width so that the
// instantiations compile in parallel.
#include "bgtq_decode_kernel.cuh"

namespace bgtq {
cudaError_t launch_decode_vb3(const DecParams& P, int nu, dim3 grid, size_t smem, cudaStream_t stream,
                              bool programmatic) {
    return launch_decode<3>(P, nu, grid, smem, stream, programmatic);
}
}  // namespace bgtq
