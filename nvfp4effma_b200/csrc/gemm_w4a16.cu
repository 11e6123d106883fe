#include "operands.cuh"
namespace nvb {
bool gemm_w4a16_supports(const GemmArgs &) { return false; }
cudaError_t launch_gemm_w4a16(const GemmArgs &, cudaStream_t) { return cudaErrorNotSupported; }
}
