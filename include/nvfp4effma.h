/* nvfp4effma.h -- C ABI of the B200 (sm_100a) NVFP4 compute library.
 *
 * The declarations here are binary- and source-compatible with the public C header of srose69/nvfp4effma v0.7.0
 * (its include/nvfp4effma.h): same type names, enum values, struct field order, symbol names and argument lists, so a
 * program built against that header links against this library unchanged.  Each entry point cites the declaration of the
 * reference header it replaces as "ref include/nvfp4effma.h:LINE".  Everything behind the ABI is new code: tcgen05
 * block-scaled MMA GEMMs, an HBM-streaming GEMV and a bandwidth-bound quantizer, all for compute capability 10.0 only.
 *
 * Conventions shared by every entry point
 *   - all pointers inside nvfp4a_tensor / nvfp4a_epilogue are DEVICE pointers of the current device; the structs
 *     themselves live on the host;
 *   - work is enqueued on `stream`; nothing is synchronised and no device memory is read on the host;
 *   - the library allocates no device memory in any entry point;
 *   - every argument is validated before anything is launched; a failed call launches nothing;
 *   - a status other than NVFP4A_OK leaves a message for nvfp4a_last_error() on the calling thread.
 */
#ifndef NVFP4EFFMA_H
#define NVFP4EFFMA_H

#define NVFP4EFFMA_VERSION "0.7.0"
#define NVFP4EFFMA_B200 1 /* this implementation: sm_100a only */

#include <stddef.h>
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ref include/nvfp4effma.h:22-23 */
typedef enum { NVFP4A_NVFP4 = 0, NVFP4A_BF16 = 1, NVFP4A_FP16 = 2, NVFP4A_FP32 = 3, NVFP4A_INT8 = 4 } nvfp4a_dtype;
typedef enum { NVFP4A_OK = 0, NVFP4A_INVALID_VALUE = 1, NVFP4A_NOT_SUPPORTED = 2, NVFP4A_CUDA_ERROR = 3 } nvfp4a_status;

/* NVFP4 matrices: [rows][cols] row-major E2M1 codes, two per byte, the even column in the low nibble; `ld` values
 * between rows.  One 8-bit block scale per 16 consecutive values of a row (E4M3 by default, UE5M3 on request) and one
 * FP32 global factor: value = e2m1 * block_scale * g.
 * Linear scale layout: scale of block (r, c/16) at byte r * ld_scale + c/16.
 * Swizzled scale layout (cuBLASLt / Transformer Engine GEMM layout): the scale matrix padded to multiples of 128 rows
 * and 4 columns, stored as 128 x 4 tiles of 512 bytes along a row of tiles; with sc = roundup(cols/16, 4) the scale of
 * block (r, c) is byte ((r/128) * (sc/4) + c/4) * 512 + (r%32) * 16 + ((r/32)%4) * 4 + c%4.
 * (ref include/nvfp4effma.h:25-31) */

/* nvfp4a_tensor.flags, NVFP4 tensors only (ref include/nvfp4effma.h:34-37) */
#define NVFP4A_SCALES_SWIZZLED 0x1u /* block scales in the swizzled GEMM layout */
#define NVFP4A_SCALES_UE5M3    0x2u /* block scales are UE5M3 (unsigned, exponent bias 15, 3 mantissa bits) */
#define NVFP4A_GLOBAL_AMAX     0x4u /* global_scale holds amax: g = amax / (6 * scale_max) */
#define NVFP4A_GLOBAL_PER_ROW  0x8u /* global_scale holds one value per row */

/* Operand descriptor (ref include/nvfp4effma.h:46-57).  INT8 tensors (W4A8 activations) carry one FP32 scale per 16
 * values in block_scale (ld_scale counts floats): value = q * block_scale * g. */
typedef struct {
  void *data;                /* device */
  nvfp4a_dtype dtype;
  void *block_scale;         /* device: NVFP4 -> bytes (E4M3 / UE5M3), INT8 -> floats; one per 16 values */
  int ld_scale;              /* linear layout: scales between consecutive rows; 0 = cols / 16 */
  const float *global_scale; /* device: decode factor g, or amax with NVFP4A_GLOBAL_AMAX; NULL = 1 */
  float *amax;               /* device, optional output: max |v| is max-reduced into the value already there */
  unsigned flags;            /* NVFP4A_SCALES_* | NVFP4A_GLOBAL_* */
  int scale_max;             /* bound M of the global encoding: 0 = 448 (E4M3) / 114688 (UE5M3); 256 = 4over6 headroom */
} nvfp4a_tensor;

/* A tensor with a rowwise and a columnwise quantization (ref include/nvfp4effma.h:62-65). */
typedef struct {
  nvfp4a_tensor row, col;
  int ld_row, ld_col;
} nvfp4a_dual_tensor;

/* GEMM, column-major D:  D[i + j*ldd] = alpha * sum_k A(i,k) B(j,k) + bias[i] + beta * C[i + j*ldc].
 * For a linear layer y = x W^T: A = W (m = out features), B = x (n = tokens), k = in features.
 * A: NVFP4 [m][k] (lda).  B: NVFP4, INT8, BF16, FP16 or FP32 [n][k] (ldb).  C, D, bias: BF16, FP16 or FP32, each
 * on its own.  C may alias D; C == NULL with beta != 0 means C = D.
 * Requirements: k, lda, ldb multiples of 64; A, B data 16-byte aligned; NVFP4 scales 4-byte, INT8 scales 16-byte
 * aligned; ld_scale a multiple of 4; m, n, ldc, ldd free (ldc, ldd >= m).  m == 0 or n == 0 is a successful no-op;
 * k == 0 yields D = bias + beta * C.
 * Epilogue, FP32, one rounding per step: v = acc * s, s = ((alpha * vA(i)) * vB(j)) * f with vX the global of operand
 * X for that row / column (1 if none) and f the product of 1 / (6 * scale_max) over operands whose global is an amax;
 * v += bias[i]; v = fma(beta, C, v); amax = max(amax, |v|); D = RNE(v).
 * Accumulation: FP32.  Columns n <= 8 run the streaming GEMV kernel (fixed split-k order, deterministic); larger n
 * run the tcgen05 kernels, whose sums follow the tensor cores' order.  Either way results agree with the exact
 * block-sum definition of the reference (ref include/nvfp4effma.h:78-92) within an FP32 accumulation bound.
 * Block scales on the tensor-core routes: the FP4 tensor cores read E4M3 block scales as UNSIGNED (UE4M3).  Codes with the sign bit
 * set -- which the reference decodes as negative factors (ref src/nvfp4effma.cuh:56-60) but which neither quantizer ever emits -- give
 * other results on the tcgen05 routes (NVFP4 B with n > 8, and the FP4 tensor-core GEMV) than the reference.  Tensors that carry such
 * codes must be run with nvfp4a_b200_set_route(1), whose CUDA-core kernels decode them exactly as the reference does.
 * ref include/nvfp4effma.h:93 */
nvfp4a_status nvfp4a_gemm(int m, int n, int k, float alpha, const nvfp4a_tensor *A, int lda,
                          const nvfp4a_tensor *B, int ldb, float beta, const nvfp4a_tensor *C, int ldc,
                          const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias, cudaStream_t stream);

/* nvfp4a_gemm on dual tensors: trans_x = 0 takes the row half of X, 1 the column half (the operand stored
 * transposed), so that blocks always run along k.  ref include/nvfp4effma.h:100 */
nvfp4a_status nvfp4a_gemm_dual(int m, int n, int k, float alpha, const nvfp4a_dual_tensor *A, int trans_a,
                               const nvfp4a_dual_tensor *B, int trans_b, float beta, const nvfp4a_tensor *C,
                               int ldc, const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias,
                               cudaStream_t stream);

/* Grouped (mixture-of-experts) GEMM.  Declared for link compatibility; this build returns NVFP4A_NOT_SUPPORTED.
 * ref include/nvfp4effma.h:114 */
nvfp4a_status nvfp4a_gemm_grouped(int groups, int m, int k, int rows, float alpha, const nvfp4a_tensor *A, int lda,
                                  const nvfp4a_tensor *B, int ldb, float beta, const nvfp4a_tensor *C, int ldc,
                                  const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias, const int *seg,
                                  cudaStream_t stream);

/* Quantization in Transformer Engine's arithmetic, bit for bit.  With M = scale_max:
 *   amax global:     S_enc = min(6 M / amax, FLT_MAX) (1 when amax or S_enc is 0), S_dec = 1 / S_enc
 *   decode factor g: S_dec = g, S_enc = min(1 / g, FLT_MAX)
 *   per block:       sb = scale_RNE_satfinite(min(bmax * (S_enc * (1/6)), FLT_MAX))
 *                    q  = E2M1_RNE_satfinite(x * min(1 / (sb * S_dec), FLT_MAX))
 * nvfp4a_quantize: dense src [rows][cols] (lds) -> NVFP4 dst (1 x 16 blocks, the destination's global as given), or
 * INT8 dst (sb = bmax / 127, q = RNE(x / sb), 0 where sb == 0).  dst->amax receives max |x|.
 * cols, lds, ldd multiples of 16; src 16-byte, NVFP4 data 8-byte, INT8 data 16-byte aligned.
 * ref include/nvfp4effma.h:127 */
nvfp4a_status nvfp4a_quantize(const nvfp4a_tensor *src, int lds, const nvfp4a_tensor *dst, int ldd, int rows,
                              int cols, cudaStream_t stream);

/* Recipe of nvfp4a_quantize_ex (ref include/nvfp4effma.h:135-142).  4over6: two scale candidates per block
 * (map-to-6: base = (bmax / 6) * S_enc; map-to-4: 1.5 * base), the one with the smaller summed |d| (MAE) or d^2 (MSE)
 * wins, ties to map-to-6; d = ((e2m1 * sb) * amax) / (6 M) - x. */
typedef enum { NVFP4A_4OVER6_OFF = 0, NVFP4A_4OVER6_MAE = 1, NVFP4A_4OVER6_MSE = 2 } nvfp4a_4over6;
typedef struct {
  int tile_rows;             /* 1: 1 x 16 blocks; 16: 16 x 16 tiles sharing one scale */
  nvfp4a_4over6 four_over_six;
  int compute_amax;          /* 1: first store the amax of src (per row with NVFP4A_GLOBAL_PER_ROW) in the
                                global_scale of the NVFP4A_GLOBAL_AMAX destinations, then quantize with it */
} nvfp4a_quant_config;

/* src [rows][cols] -> rowwise NVFP4 [rows][cols] (ld_row) and / or columnwise NVFP4 [cols][roundup(rows,16)] (the
 * quantization of src^T, ld_col); either may be NULL.  cfg NULL = {1, OFF, 0}.  Scale buffers hold the padded matrix;
 * padding is never written.  ref include/nvfp4effma.h:151 */
nvfp4a_status nvfp4a_quantize_ex(const nvfp4a_tensor *src, int lds, int rows, int cols, const nvfp4a_tensor *rowwise,
                                 int ld_row, const nvfp4a_tensor *columnwise, int ld_col,
                                 const nvfp4a_quant_config *cfg, cudaStream_t stream);

/* NVFP4 src -> BF16 / FP16 / FP32 dst: (e2m1 * sb) * g, or with an amax global e2m1 * ((sb * amax) * (1 / (6 M))),
 * rounded once; dst->amax receives max |v|.  ref include/nvfp4effma.h:158 */
nvfp4a_status nvfp4a_dequantize(const nvfp4a_tensor *src, int lds, const nvfp4a_tensor *dst, int ldd, int rows,
                                int cols, cudaStream_t stream);

/* Block scales of a [rows][cols] NVFP4 matrix: linear (ld_linear bytes per row) -> swizzled (to_swizzled = 1, padding
 * written as 0) or back (0).  ref include/nvfp4effma.h:164 */
nvfp4a_status nvfp4a_swizzle_scales(const void *src, void *dst, int ld_linear, int rows, int cols, int to_swizzled,
                                    cudaStream_t stream);

/* Transpose of an NVFP4 matrix quantized with 16 x 16 tiles: src [rows][cols] -> dst [cols][rows], data and scales.
 * ref include/nvfp4effma.h:170 */
nvfp4a_status nvfp4a_transpose(const nvfp4a_tensor *src, int lds, const nvfp4a_tensor *dst, int ldd, int rows,
                               int cols, cudaStream_t stream);

/* ---- Image API (ref include/nvfp4effma.h:173-218) ------------------------------------------------------------------
 * An image is the operand re-laid for streaming: rows in tiles of 128, k in tiles of 256; per tile 16384 bytes of
 * nibbles (128 rows x 128 bytes) followed by 2048 bytes of block scales as four 128 x 4 swizzled tiles.  The format is
 * opaque to callers.  Weights are imaged once, activations per call.  Here one layout serves both weight kinds, so
 * NVFP4A_TC_A16 and NVFP4A_TC_A8 images hold the same bytes. */
#define NVFP4A_TC_A16 0
#define NVFP4A_TC_B 1
#define NVFP4A_TC_A8 2

/* Bytes of an image; 0 for an invalid combination.  A kinds: NVFP4.  B kind: NVFP4, INT8, BF16.
 * ref include/nvfp4effma.h:188 */
size_t nvfp4a_tc_image_bytes(int operand, nvfp4a_dtype dtype, int rows, int k);

/* src [rows][k] (ld) -> image (16-byte aligned).  ref include/nvfp4effma.h:193 */
nvfp4a_status nvfp4a_tc_image(int operand, const nvfp4a_tensor *src, int ld, int rows, int k, void *image,
                              cudaStream_t stream);

/* Weight image -> the other weight kind, or back to the plain tensor (linear scales), byte-exact.
 * ref include/nvfp4effma.h:199-200 */
nvfp4a_status nvfp4a_tc_image_convert(int from, int to, const void *image, int rows, int k, void *dst, cudaStream_t stream);
nvfp4a_status nvfp4a_tc_image_to_raw(int from, const void *image, int rows, int k, const nvfp4a_tensor *dst, int ld, cudaStream_t stream);

/* Bytes of the workspace nvfp4a_gemm_tc takes on the current device.  The caller zeroes it once; every call leaves
 * it zeroed; one call at a time per workspace.  ref include/nvfp4effma.h:204 */
size_t nvfp4a_tc_workspace_bytes(void);

/* GEMM from images (A->data, B->data are images; flags, globals, scale_max as in nvfp4a_gemm).
 * ref include/nvfp4effma.h:209 */
nvfp4a_status nvfp4a_gemm_tc(int m, int n, int k, float alpha, const nvfp4a_tensor *A, const nvfp4a_tensor *B, float beta,
                             const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias,
                             void *workspace, cudaStream_t stream);

/* GEMV, 1 <= n <= 8, A its image, B as for nvfp4a_gemm.  ref include/nvfp4effma.h:216 */
nvfp4a_status nvfp4a_gemv_tc(int m, int n, int k, float alpha, const nvfp4a_tensor *A, const nvfp4a_tensor *B, int ldb, float beta,
                             const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias,
                             cudaStream_t stream);

/* ---- Extended epilogue (ref include/nvfp4effma.h:223-246) ------------------------------------------------------------
 * norm_parts: deferred RMSNorm column scale s_j = RN(1 / sqrt(sum_j * norm_inv_n + norm_eps)), sum_j over the
 *   norm_nparts floats at norm_parts + j * norm_ld (lane l of 32 adds parts l, l+32, ... then an xor butterfly
 *   16,8,4,2,1); s_j multiplies B's global in the output scale.
 * swiglu: A's rows come in slices of 16 (8 gate rows, then their 8 up rows); D has m/2 rows,
 *   D[8q + r] = silu(g) * u with g, u the plain epilogue values of rows 16q + r and 16q + 8 + r.
 * d2 / w2 / sq: second output d2[i + j*ldd2] = RN(v * w2[i]) and per 16-row slice s the sum of RN(v*v) over its rows
 *   ascending in sq[j * ld_sq + s].
 * With any addition: A's scales linear E4M3 (E4M3 for the image entries), B BF16 or INT8, m a multiple of 16. */
typedef struct {
  const float *norm_parts;
  int norm_nparts, norm_ld;
  float norm_inv_n, norm_eps;
  int swiglu;
  void *d2;
  nvfp4a_dtype d2_dtype;
  int ldd2;
  const void *w2;
  nvfp4a_dtype w2_dtype;
  float *sq;
  int ld_sq;
} nvfp4a_epilogue;

/* ref include/nvfp4effma.h:248, :251, :254 */
nvfp4a_status nvfp4a_gemm_ex(int m, int n, int k, float alpha, const nvfp4a_tensor *A, int lda, const nvfp4a_tensor *B, int ldb,
                             float beta, const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias,
                             const nvfp4a_epilogue *ex, cudaStream_t stream);
nvfp4a_status nvfp4a_gemv_tc_ex(int m, int n, int k, float alpha, const nvfp4a_tensor *A, const nvfp4a_tensor *B, int ldb, float beta,
                                const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias,
                                const nvfp4a_epilogue *ex, cudaStream_t stream);
nvfp4a_status nvfp4a_gemm_tc_ex(int m, int n, int k, float alpha, const nvfp4a_tensor *A, const nvfp4a_tensor *B, float beta,
                                const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias,
                                const nvfp4a_epilogue *ex, void *workspace, cudaStream_t stream);

/* ref include/nvfp4effma.h:258, :262 */
const char *nvfp4a_status_string(nvfp4a_status status);
const char *nvfp4a_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* NVFP4EFFMA_H */
