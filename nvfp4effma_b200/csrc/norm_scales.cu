// RMSNorm column scales of the extended epilogue for all tokens of a GEMM at once: s_j = RN(1 / sqrt(sum_j * inv_n + eps)),
// sum_j over the token's partial sums of squares in the defining order (reference include/nvfp4effma.h:224-226 there): lane
// l of a warp adds parts l, l + 32, ... ascending, then an xor butterfly 16..1.  One warp per token.  The tcgen05 GEMM then
// reads one float per token instead of summing the parts again for every tile of weight rows.
#include "operands.cuh"

namespace nvb {

__global__ void __launch_bounds__(256) norm_scales_kernel(const EpilogueEx x, int n, float *out) {
  const int j = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (j >= n) return;
  const float s = warp_norm_scale(x, j, lane);
  if (lane == 0) out[j] = s;
}

cudaError_t launch_norm_scales(const EpilogueEx &x, int n, float *out, cudaStream_t s) {
  norm_scales_kernel<<<(n + 7) / 8, 256, 0, s>>>(x, n, out);
  return cudaGetLastError();
}

}  // namespace nvb
