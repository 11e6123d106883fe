#include "operands.cuh"
namespace nvb {
bool gemv_supports(const GemmArgs &) { return false; }
cudaError_t launch_gemv(const GemmArgs &, cudaStream_t) { return cudaErrorNotSupported; }
}
