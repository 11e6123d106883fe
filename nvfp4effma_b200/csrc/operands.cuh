// Device views of GEMM operands and the internal launch interface between the host API (gemm_api.cu) and the kernels.
#pragma once
#include "common.cuh"
#include "tp_barrier.cuh"

namespace nvb {

// Image geometry: rows in tiles of 128, k in tiles of 256.  One tile = 16384 bytes of nibbles (128 rows x 128 bytes, row
// major) + 2048 bytes of block scales (four swizzled 128 x 4 tiles, one per 64 values of k).  Rows and k positions outside
// the matrix hold zero nibbles and zero scales.
constexpr int kImgRows = 128, kImgK = 256;
constexpr int kImgDataBytes = kImgRows * kImgK / 2, kImgScaleBytes = kImgRows * kImgK / 16;
constexpr int kImgTileBytes = kImgDataBytes + kImgScaleBytes;  // 18432
__host__ __device__ inline size_t image_bytes(int rows, int k) {
  return (size_t)((rows + kImgRows - 1) / kImgRows) * (size_t)((k + kImgK - 1) / kImgK) * kImgTileBytes;
}

// An NVFP4 operand [rows][k]: plain (data + scales, linear or swizzled) or an image.
struct Fp4Operand {
  const uint8_t *data;   // plain: nibbles; image: the image
  const uint8_t *sc;     // plain: block scales
  int ld;                // plain: values between rows
  int sld;               // plain: ScalePos ld (> 0 linear, < 0 swizzled)
  int image;             // 1: data is an image
  int ktiles;            // image: tiles along k
  int ue;                // UE5M3 scales

  // the 8 bytes (16 nibbles) of block kb of row r, and its scale code
  __device__ __forceinline__ uint2 block(int r, int kb) const {
    if (image) {
      const size_t t = (size_t)(r >> 7) * ktiles + (kb >> 4);
      return *(const uint2 *)(data + t * kImgTileBytes + (size_t)(r & 127) * 128 + (kb & 15) * 8);
    }
    return *(const uint2 *)(data + (size_t)r * (ld >> 1) + (size_t)kb * 8);
  }
  __device__ __forceinline__ uint32_t scale_code(int r, int kb) const {
    if (image) {
      const size_t t = (size_t)(r >> 7) * ktiles + (kb >> 4);
      const int rr = r & 127, kq = kb & 15;
      return data[t * kImgTileBytes + kImgDataBytes + (kq >> 2) * 512 + (rr & 31) * 16 + (rr >> 5) * 4 + (kq & 3)];
    }
    return sc[ScalePos{sld}.at(r, kb)];
  }
  __device__ __forceinline__ float scale(int r, int kb) const { return scale_to_f32(scale_code(r, kb), ue != 0); }
};

// B of any type: NVFP4 (fp4 view), INT8 (+ FP32 scales per 16), or dense BF16 / FP16 / FP32.
struct BOperand {
  int dtype;
  Fp4Operand q;            // NVFP4
  const void *data; int ld;  // INT8 / dense: [n][ld]
  const float *s8; int lds8; // INT8: FP32 block scales [n][lds8]
};

struct GemmArgs {
  int m, n, k;
  Fp4Operand A;
  BOperand B;
  Epilogue e;
  EpilogueEx x;
  TpPush tp;   // tensor-parallel GEMV: D also goes to the peers, then the ranks' barrier (world <= 1: off)
  int no_alloc;   // the call must not allocate (nvfp4a_b200_gemm_ex_static): routes that take scratch from the stream's memory pool step aside
};

// kernels (each returns the launch error)
cudaError_t launch_gemm_generic(const GemmArgs &g, cudaStream_t s);  // any operand combination, exact tiled order (CUDA cores)
cudaError_t launch_gemm_grouped(const GemmArgs &g, const int *seg, int groups, cudaStream_t s);  // the same kernel over groups of columns
cudaError_t launch_gemv(const GemmArgs &g, cudaStream_t s);          // n <= 8: HBM-streaming split-k GEMV
bool gemv_supports(const GemmArgs &g);
cudaError_t launch_gemv_fp4(const GemmArgs &g, cudaStream_t s);      // n <= 2: weights straight into tcgen05 kind::mxf4nvf4, activations as FP4 digit planes
bool gemv_fp4_supports(const GemmArgs &g);
void set_gemv_fp4_splits(int s);
cudaError_t launch_gemv_blocked(const GemmArgs &g, cudaStream_t s);  // n <= 8, INT8 or NVFP4 activations: exact DP4A block sums
bool gemv_blocked_supports(const GemmArgs &g);
cudaError_t launch_gemm_w4a4(const GemmArgs &g, cudaStream_t s);     // tcgen05 kind::mxf4nvf4 (E4M3 scales)
bool gemm_w4a4_supports(const GemmArgs &g);
cudaError_t launch_gemm_dp4a(const GemmArgs &g, cudaStream_t s);     // W4A8, n > 8: DP4A block sums in the reference's tiled order
bool gemm_dp4a_supports(const GemmArgs &g);
cudaError_t launch_gemm_w4a16(const GemmArgs &g, cudaStream_t s);    // tcgen05 kind::f16 with weights expanded to BF16 in smem
bool gemm_w4a16_supports(const GemmArgs &g);
bool gemm_w4a16_pushes(const GemmArgs &g);
cudaError_t launch_gemm_w4a8_tc(const GemmArgs &g, cudaStream_t s);  // INT8 activations as three BF16 planes on the same tcgen05 kernel
bool gemm_w4a8_tc_supports(const GemmArgs &g);
cudaError_t trim_planes_pool();   // gives the W4A8 planes' pool memory of the current device back to the system
// s_j of every token (the RMSNorm column scale of the extended epilogue) -> out[0 .. n)
cudaError_t launch_norm_scales(const EpilogueEx &x, int n, float *out, cudaStream_t s);
cudaError_t launch_image_build(const Fp4Operand &src, int rows, int k, uint8_t *image, cudaStream_t s);
cudaError_t launch_image_to_raw(const uint8_t *image, int rows, int k, uint8_t *data, int ld, uint8_t *sc, int lds, cudaStream_t s);

}  // namespace nvb
