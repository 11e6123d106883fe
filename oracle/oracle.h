/* CPU oracle for the NVFP4 hot path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain C++ restatement (no CUDA) of the arithmetic that srose69/nvfp4effma documents in include/nvfp4effma.h and
 * emulates on the host in its tests.  Only tests, the smoke check and the bench's cpu_baseline / reference arm may load
 * this library; the product (nvfp4effma_b200) never does.  Build with -ffp-contract=off: every operation below is one
 * IEEE FP32 operation with its own rounding, as in the reference's host code (its Makefile:20).
 *
 * Parity pins: the encoders and the scale addressing are checked exhaustively against the reference's own
 * __host__ codecs compiled from its sources (oracle/ref_codecs.cu -> oracle/_ref/), the quantizer against the
 * reference's independent torch statement (tests/golden/), and -- on a B200 -- quantizer, GEMM and GEMV against the
 * reference's own CUDA-core kernels (oracle/ref.mk -> oracle/_ref/libnvfp4effma_ref.so).
 */
#ifndef NVFP4_ORACLE_H
#define NVFP4_ORACLE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORC_NVFP4 = 0, ORC_BF16 = 1, ORC_FP16 = 2, ORC_FP32 = 3, ORC_INT8 = 4 };
enum { ORC_SWIZZLED = 1, ORC_UE5M3 = 2, ORC_GLOBAL_AMAX = 4, ORC_PER_ROW = 8 };

/* Host-memory mirror of nvfp4a_tensor (every pointer is a HOST pointer). */
typedef struct {
  void *data;
  int dtype;
  void *block_scale;
  int ld_scale;
  const float *global_scale;
  unsigned flags;
  int scale_max;
} orc_tensor;

/* ---- element codecs --------------------------------------------------------------------------------- */
float orc_e4m3_value(uint32_t code);     /* any finite E4M3 code, sign included */
float orc_ue5m3_value(uint32_t code);
float orc_e2m1_value(uint32_t nibble);
uint32_t orc_f32_to_e4m3(float x);       /* RNE, saturating at +-448, NaN -> 0x7F */
uint32_t orc_f32_to_e2m1(float x);       /* RNE to the even code, saturating at +-6, sign of zero kept, NaN -> +-6 */
uint32_t orc_f32_to_ue5m3(float x);      /* RNE, saturating at 114688; negative, -0, NaN -> 0 */
uint32_t orc_f32_to_bf16(float x);       /* RNE, NaN -> 0x7FC0 */
uint32_t orc_f32_to_f16(float x);
float orc_bf16_to_f32(uint32_t h);
float orc_f16_to_f32(uint32_t h);
size_t orc_scale_pos(int swizzled, int ld, int cols, int r, int c); /* byte of block scale (r, c) */
size_t orc_scale_bytes(int swizzled, int ld, int rows, int cols);

/* Exhaustive folds for the pins: a 64-bit multiplicative hash over code(x) for the FP32 bit patterns
 * [first, first + count), which = 0 e4m3, 1 e2m1, 2 ue5m3, 3 bf16. */
uint64_t orc_encoder_fold(int which, uint64_t first, uint64_t count, int nthreads);
/* codes for an array of inputs (which as above) */
void orc_encode_array(int which, const float *x, uint32_t *codes, size_t n);

/* ---- quantization -------------------------------------------------------------------------------------
 * x: FP32 copy of the source [rows][cols] (ldx); BF16 / FP16 sources convert exactly.  dst: NVFP4 tensor
 * [orows][ocols]; transposed = 1 quantizes x^T (the columnwise destination: orows = cols, ocols = roundup(rows,16)).
 * tile 1 / 16; fos 0 / 1 (MAE) / 2 (MSE).  compute_amax: 1 = first write the global(s) as max |x| (per row with
 * ORC_PER_ROW) through dst->global_scale (cast away const).  amax_out (optional): max-reduced with max |x|.
 * Follows ref tests/test_nvfp4effma.cu:205-276 and include/nvfp4effma.h:118-132. */
int orc_quantize(const float *x, int ldx, int rows, int cols, const orc_tensor *dst, int ldd, int transposed,
                 int tile, int fos, int compute_amax, float *amax_out, int nthreads);
/* INT8 destination: sb = bmax / 127, q = clamp(rint(x / sb), +-127), 0 where sb == 0.
 * ref tests/test_nvfp4effma.cu:415-423 */
int orc_quantize_int8(const float *x, int ldx, int rows, int cols, int8_t *q, int ldq, float *scales, int ld_scale,
                      float *amax_out, int nthreads);
/* NVFP4 -> FP32 values rounded to out_dtype and widened again: (e * sb) * g, or e * ((sb * amax) * (1 / (6 M))).
 * ref tests/test_nvfp4effma.cu:351-360 */
int orc_dequantize(const orc_tensor *src, int lds, int rows, int cols, int out_dtype, float *y, int ldy, float *amax_out);
/* linear <-> swizzled block scales, padding of the swizzled buffer written as 0.  ref tests/test_nvfp4effma.cu:434-451 */
int orc_swizzle_scales(const uint8_t *src, uint8_t *dst, int ld_linear, int rows, int cols, int to_swizzled);

/* ---- GEMM / GEMV -----------------------------------------------------------------------------------------
 * D[i + j*ldd] = alpha * sum_k A(i,k) B(j,k) + bias[i] + beta * C[i + j*ldc], the exact definition of
 * ref include/nvfp4effma.h:78-92 as emulated in ref tests/test_util.h:241-291.
 * order 0: tiled (16-blocks ascending in k; dense B one FMA per MAC ascending);
 * order 1: the reference GEMV kernel's lane order (lane l takes blocks 32c + l, xor butterfly 16..1).
 * D, C, bias: dtype codes ORC_BF16 / FP16 / FP32, raw host buffers of that type.  C NULL with beta != 0 = D.
 * acc_out (optional, [n][m] FP32): the accumulator before the epilogue (after the 1/4 or 1/2 factor).
 * ref64 / bound (optional, [n][m] double): the float64 value and the FP32-accumulation tolerance of
 * ref tests/test_util.h:292-302 for kernels that sum in another order.
 * amax_out (optional): max |v| over the outputs is max-reduced into it. */
int orc_gemm(int m, int n, int k, float alpha, const orc_tensor *A, int lda, const orc_tensor *B, int ldb, float beta,
             const void *C, int c_dtype, int ldc, void *D, int d_dtype, int ldd, const void *bias, int bias_dtype,
             int order, float *amax_out, float *acc_out, double *ref64, double *bound, int nthreads);

/* Extended epilogue applied to accumulators acc [n][m] (ref tests/test_epilogue.cu:11-23, :130-168;
 * include/nvfp4effma.h:223-246).  ga: A's globals (NULL = 1; per_row_a), gb: B's global value, gf: amax factor.
 * mask bit 0 NORM, 1 SWIGLU, 2 OUT2.  Outputs: v_out [n][m] FP32 (value before rounding, optional), D, d2, sq.
 * SwiGLU here is evaluated in double (silu(g) * u); compare with the tolerance of ref tests/test_epilogue.cu:146. */
int orc_epilogue_ex(int m, int n, const float *acc, float alpha, const float *ga, int per_row_a, float gb, float gf,
                    float beta, const void *C, int c_dtype, int ldc, const void *bias, int bias_dtype, int mask,
                    const float *norm_parts, int norm_nparts, int norm_ld, float norm_inv_n, float norm_eps,
                    void *D, int d_dtype, int ldd, double *swiglu64, void *d2, int d2_dtype, int ldd2, const void *w2,
                    int w2_dtype, float *sq, int ld_sq, float *v_out);
float orc_norm_scale(const float *parts, int nparts, float inv_n, float eps);

#ifdef __cplusplus
}
#endif
#endif
