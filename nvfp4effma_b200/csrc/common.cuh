// Device / host core shared by every kernel of the library: element codecs, block-scale addressing, typed loads and
// stores, the GEMM / GEMV epilogue, and the host-side error state.  Compute capability 10.0 (sm_100a) only.
//
// Numerical contract (restated from the reference's public header, include/nvfp4effma.h:78-92 and :118-122 there):
// every epilogue and quantizer step is one IEEE FP32 operation with its own rounding, denormals honoured, so all such
// steps use the explicit __f*_rn intrinsics and nothing is compiled with fast-math.
#pragma once
#include <stdint.h>
#include <string.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include "../../include/nvfp4effma.h"

namespace nvb {

constexpr float kFltMax = 3.40282347e38f;

// ---- block scale bytes -> FP32 (exact) --------------------------------------------------------------------------
// E4M3 (bias 7): a finite code c decodes as c's magnitude bits placed at FP32 bits [20, 27) times 2^120: the FP32
// exponent field then reads e (biased 127) and the three mantissa bits sit on top; e = 0 lands on FP32 subnormals, so one
// multiply by 2^(127-7) restores normals and subnormals alike.  UE5M3 (bias 15): the same with 2^(127-15).
__device__ __forceinline__ float e4m3_to_f32(uint32_t c) {
  return __fmul_rn(__uint_as_float(((c & 0x80u) << 24) | ((c & 0x7Fu) << 20)), 0x1p120f);
}
__device__ __forceinline__ float ue5m3_to_f32(uint32_t c) { return __fmul_rn(__uint_as_float((c & 0xFFu) << 20), 0x1p112f); }
__device__ __forceinline__ float scale_to_f32(uint32_t c, bool ue) { return ue ? ue5m3_to_f32(c) : e4m3_to_f32(c); }

// E2M1 nibble -> FP32 (exact): magnitude bits at FP32 bits [22, 25) give value * 2^-126 (0.5 is the FP32 subnormal
// 2^-127), one multiply restores it.
__device__ __forceinline__ float e2m1_to_f32(uint32_t nib) {
  return __fmul_rn(__uint_as_float(((nib & 8u) << 28) | ((nib & 7u) << 22)), 0x1p126f);
}
// 2 * e2m1 as a small integer (0, +-1, 2, 3, 4, 6, 8, 12)
__device__ __forceinline__ int e2m1_x2(uint32_t nib) {
  const int mag = (0x0C08060403020100ull >> (8 * (nib & 7u))) & 0xFF;
  return (nib & 8u) ? -mag : mag;
}

// ---- FP32 -> narrow formats, round to nearest even, saturating -----------------------------------------------------
// Software versions (exhaustively equal to the reference's encoders: checked on the CPU oracle, which is pinned against
// the reference, and on the GPU by tests/test_codecs_gpu.py).  x + 2^23 trick: adding 1.5 * 2^23-free 2^23 to a
// non-negative value below 2^23 rounds it to an integer in one FP32 addition.
__host__ __device__ __forceinline__ uint32_t f32_bits(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
__host__ __device__ __forceinline__ float bits_f32(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }

__host__ __device__ __forceinline__ uint32_t f32_to_e2m1_sw(float x) {
  const uint32_t u = f32_bits(x), sign = (u >> 28) & 8u, a = u & 0x7FFFFFFFu;
  if (a >= 0x40C00000u) return sign | 7u;  // |x| >= 6, Inf, NaN
  // step of the target grid: 0.5 below 2, 1 in [2, 4), 2 in [4, 6); rounding |x| / step to an integer gives the code offset
  const float mag = bits_f32(a);
  float scaled; uint32_t base;
  if (a < 0x40000000u) { scaled = mag * 2.0f; base = 0u; }        // codes 0..4
  else if (a < 0x40800000u) { scaled = mag; base = 2u; }          // integer 2..4 -> codes 4..6
  else { scaled = mag * 0.5f; base = 4u; }                        // integer 2..3 -> codes 6..7
  const uint32_t q = f32_bits(scaled + 8388608.0f) - 0x4B000000u;
  return sign | (q + base);
}
__host__ __device__ __forceinline__ uint32_t f32_to_e4m3_sw(float x) {
  const uint32_t u = f32_bits(x), sign = (u >> 24) & 0x80u, a = u & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return 0x7Fu;
  if (a >= 0x43E00000u) return sign | 0x7Eu;                      // >= 448
  if (a < 0x3C800000u) {                                          // < 2^-6: subnormal grid of 2^-9
    const uint32_t q = f32_bits(bits_f32(a) * 512.0f + 8388608.0f) - 0x4B000000u;
    return sign | q;                                              // q = 8 is the smallest normal, code 0x08
  }
  const uint32_t r = a + 0x7FFFFu + ((a >> 20) & 1u);             // RNE at mantissa bit 20
  return sign | (((r >> 23) - 120u) << 3) | ((r >> 20) & 7u);
}
__host__ __device__ __forceinline__ uint32_t f32_to_ue5m3_sw(float x) {
  const uint32_t a = f32_bits(x);
  if (a >= 0x80000000u || a > 0x7F800000u) return 0u;             // negative, -0, NaN
  if (a >= 0x47E00000u) return 0xFEu;                             // >= 114688
  if (a < 0x38800000u) return f32_bits(bits_f32(a) * 131072.0f + 8388608.0f) - 0x4B000000u;
  const uint32_t r = a + 0x7FFFFu + ((a >> 20) & 1u);
  const uint32_t c = (((r >> 23) - 112u) << 3) | ((r >> 20) & 7u);
  return c > 0xFEu ? 0xFEu : c;
}
__host__ __device__ __forceinline__ uint32_t f32_to_bf16_bits(float x) {
  const uint32_t u = f32_bits(x);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FC0u;
  return (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;
}

// 32 FP32 values (bit patterns in r[]) -> BF16 bit patterns in the low halves of r[], round to nearest even, NaN -> 0x7FC0:
// the same results as f32_to_bf16_bits, by the hardware's packed conversion (16 instructions with short dependency chains
// instead of 32 chains of integer arithmetic; the epilogues of the tensor-core GEMMs run on one warp per scheduler, where
// chain latency is what costs).  The conversion turns every NaN into 0x7FFF, which no other input produces.
__device__ __forceinline__ void round32_to_bf16(uint32_t (&r)[32]) {
  uint32_t nan = 0;
#pragma unroll
  for (int q = 0; q < 16; ++q) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(__uint_as_float(r[2 * q + 1])), "f"(__uint_as_float(r[2 * q])));
    nan |= (d & 0x7FFF7FFFu) + 0x00010001u;   // a half that was 0x7FFF carries into its top bit
    r[2 * q] = d & 0xFFFFu;
    r[2 * q + 1] = d >> 16;
  }
  if (nan & 0x80008000u) {
#pragma unroll
    for (int jj = 0; jj < 32; ++jj)
      if ((r[jj] & 0x7FFFu) == 0x7FFFu) r[jj] = 0x7FC0u;
  }
}

// ---- block scale addressing ----------------------------------------------------------------------------------------
// ld > 0: linear, ld scales per row.  ld < 0: swizzled 128 x 4 tiles, -ld = padded scale columns.
struct ScalePos {
  int ld;
  __host__ __device__ __forceinline__ size_t row(int r) const {
    if (ld > 0) return (size_t)r * ld;
    return ((size_t)(r >> 7) * (size_t)((-ld) >> 2)) * 512 + (size_t)(r & 31) * 16 + (size_t)((r >> 5) & 3) * 4;
  }
  __host__ __device__ __forceinline__ size_t col(int c) const { return ld > 0 ? (size_t)c : (size_t)(c >> 2) * 512 + (c & 3); }
  __host__ __device__ __forceinline__ size_t at(int r, int c) const { return row(r) + col(c); }
};

// ---- dense element access ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float load_dense(int dtype, const void *p, size_t i) {
  if (dtype == NVFP4A_BF16) return __uint_as_float((uint32_t)((const uint16_t *)p)[i] << 16);
  if (dtype == NVFP4A_FP16) return __half2float(((const __half *)p)[i]);
  return ((const float *)p)[i];
}
__device__ __forceinline__ void store_dense(int dtype, void *p, size_t i, float v) {
  if (dtype == NVFP4A_BF16) ((uint16_t *)p)[i] = (uint16_t)f32_to_bf16_bits(v);
  else if (dtype == NVFP4A_FP16) ((__half *)p)[i] = __float2half_rn(v);
  else ((float *)p)[i] = v;
}
__host__ __device__ __forceinline__ int dense_bytes(int dtype) { return dtype == NVFP4A_FP32 ? 4 : 2; }

// max-reduce a non-negative float into *dst (non-negative floats order like their bit patterns)
__device__ __forceinline__ void warp_amax_commit(float *dst, float m) {
#pragma unroll
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
  if ((threadIdx.x & 31) == 0 && m > 0.f) atomicMax((int *)dst, __float_as_int(m));
}

// ---- epilogue ----------------------------------------------------------------------------------------------------------
// v = acc * s(i, j); v += bias[i]; v = fma(beta, C, v); amax; D = RNE(v), with
// s = ((alpha * gA(i)) * (gB(j) [* s_j])) * gf      (reference include/nvfp4effma.h:90-92, :227)
struct Epilogue {
  const float *ga, *gb;   // globals of A / B (NULL = 1)
  int ga_stride, gb_stride;  // 0: one value, 1: one per row (A: output row i, B: column j)
  float gf, alpha, beta;
  const void *c; int ldc, c_dtype;
  void *d; int ldd, d_dtype;
  float *amax;
  const void *bias; int bias_dtype;
};
// extended epilogue descriptor (mask bits: 1 NORM, 2 SWIGLU, 4 OUT2)
struct EpilogueEx {
  int mask;
  const float *norm_parts; int norm_nparts, norm_ld; float norm_inv_n, norm_eps;
  void *d2; int d2_dtype, ldd2; const void *w2; int w2_dtype;
  float *sq; int ld_sq;
  const float *colscales;  // kExNorm: the column scales s_j, already computed (one float per token), or NULL
};
constexpr int kExNorm = 1, kExSwiglu = 2, kExOut2 = 4;

__device__ __forceinline__ float epi_row_part(const Epilogue &e, int i) {
  return __fmul_rn(e.alpha, e.ga ? e.ga[(size_t)i * e.ga_stride] : 1.f);
}
__device__ __forceinline__ float epi_col_part(const Epilogue &e, int j) { return e.gb ? e.gb[(size_t)j * e.gb_stride] : 1.f; }
__device__ __forceinline__ float epi_scale(const Epilogue &e, float row_part, float col_part) {
  return __fmul_rn(__fmul_rn(row_part, col_part), e.gf);
}
// the value before the output rounding
__device__ __forceinline__ float epi_value(const Epilogue &e, int i, int j, float acc, float s) {
  float v = __fmul_rn(acc, s);
  if (e.bias) v = __fadd_rn(v, load_dense(e.bias_dtype, e.bias, i));
  if (e.beta != 0.f) v = __fmaf_rn(e.beta, load_dense(e.c_dtype, e.c, (size_t)j * e.ldc + i), v);
  return v;
}
// RMSNorm column scale of column j, computed by a full warp: lane l adds parts l, l + 32, ... ascending, xor butterfly
// 16..1, then the correctly rounded reciprocal square root (reference include/nvfp4effma.h:224-226).
__device__ __forceinline__ float warp_norm_scale(const EpilogueEx &x, int j, int lane) {
  const float *p = x.norm_parts + (size_t)j * x.norm_ld;
  float s = 0.f;
  for (int i = lane; i < x.norm_nparts; i += 32) s = __fadd_rn(s, __ldcg(p + i));
#pragma unroll
  for (int o = 16; o; o >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xFFFFFFFFu, s, o));
  return __frsqrt_rn(__fadd_rn(__fmul_rn(s, x.norm_inv_n), x.norm_eps));
}
// silu(g) * u with the GPU's fast exponential and division, as the reference computes it (src/nvfp4effma.cuh:358 there)
__device__ __forceinline__ float silu_mul(float g, float u) { return __fmul_rn(__fdividef(g, __fadd_rn(1.f, __expf(-g))), u); }

// ---- host side: error state and shared checks ---------------------------------------------------------------------------
void clear_error();
nvfp4a_status fail(nvfp4a_status s, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
nvfp4a_status cuda_fail(cudaError_t e, const char *what);
nvfp4a_status check_device();                 // OK only on compute capability 10.x
int device_sms();
float scale_max_of(const nvfp4a_tensor *t);   // 0 = invalid combination
nvfp4a_status check_scales(const char *fn, const char *name, const nvfp4a_tensor *t, int rows, int cols, int *ld);
float amax_factor(const nvfp4a_tensor *A, const nvfp4a_tensor *B);

}  // namespace nvb
