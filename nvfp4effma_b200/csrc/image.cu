// Operand images (nvfp4a_tc_image and friends): an NVFP4 matrix re-laid into 128-row x 256-k tiles of 16384 nibble bytes
// followed by 2048 scale bytes in the swizzled 128 x 4 form (operands.cuh).  A tile is exactly what one pipeline stage of
// the tcgen05 GEMM consumes: the nibble part is one TMA box, the scale part one contiguous bulk copy that tcgen05.cp
// moves to tensor memory unchanged.  The reference's images (src/tensors/image.cuh:14-46 there) serve its mma.sync
// kernels and have another byte order; the size formula is the same: ceil(rows/128) * ceil(k/256) * 18432 bytes.
#include "operands.cuh"

namespace nvb {

// one thread per (padded row, padded k-block)
__global__ void image_build_kernel(Fp4Operand src, int rows, int k, uint8_t *__restrict__ image) {
  const int ktiles = (k + kImgK - 1) / kImgK, pk16 = ktiles * (kImgK / 16);
  const long long total = (long long)((rows + kImgRows - 1) / kImgRows * kImgRows) * pk16;
  for (long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x; u < total; u += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(u / pk16), kb = (int)(u - (long long)r * pk16);
    const bool in = r < rows && 16 * kb < k;
    uint2 w = make_uint2(0, 0);
    uint32_t code = 0;
    if (in) { w = src.block(r, kb); code = src.scale_code(r, kb); }
    uint8_t *tile = image + ((size_t)(r >> 7) * ktiles + (kb >> 4)) * kImgTileBytes;
    const int rr = r & 127, kq = kb & 15;
    *(uint2 *)(tile + rr * 128 + kq * 8) = w;
    tile[kImgDataBytes + (kq >> 2) * 512 + (rr & 31) * 16 + (rr >> 5) * 4 + (kq & 3)] = (uint8_t)code;
  }
}

// one thread per (row, k-block) of the matrix: image -> plain data and linear scales
__global__ void image_to_raw_kernel(const uint8_t *__restrict__ image, int rows, int k, uint8_t *__restrict__ data, int ld,
                                    uint8_t *__restrict__ sc, int lds) {
  Fp4Operand img;
  img.data = image; img.sc = nullptr; img.ld = 0; img.sld = 0; img.image = 1; img.ktiles = (k + kImgK - 1) / kImgK; img.ue = 0;
  const int bpr = k / 16;
  const long long total = (long long)rows * bpr;
  for (long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x; u < total; u += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(u / bpr), kb = (int)(u - (long long)r * bpr);
    *(uint2 *)(data + (size_t)r * (ld / 2) + 8 * kb) = img.block(r, kb);
    sc[(size_t)r * lds + kb] = (uint8_t)img.scale_code(r, kb);
  }
}

static int grid_of(long long threads) {
  const long long want = (threads + 255) / 256, cap = (long long)device_sms() * 8;
  return (int)(want < 1 ? 1 : want < cap ? want : cap);
}

cudaError_t launch_image_build(const Fp4Operand &src, int rows, int k, uint8_t *image, cudaStream_t s) {
  const long long total = (long long)((rows + kImgRows - 1) / kImgRows * kImgRows) * ((k + kImgK - 1) / kImgK * (kImgK / 16));
  image_build_kernel<<<grid_of(total), 256, 0, s>>>(src, rows, k, image);
  return cudaGetLastError();
}
cudaError_t launch_image_to_raw(const uint8_t *image, int rows, int k, uint8_t *data, int ld, uint8_t *sc, int lds, cudaStream_t s) {
  image_to_raw_kernel<<<grid_of((long long)rows * (k / 16)), 256, 0, s>>>(image, rows, k, data, ld, sc, lds);
  return cudaGetLastError();
}

}  // namespace nvb
