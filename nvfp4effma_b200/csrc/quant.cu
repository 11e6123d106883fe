// Quantization side of the C ABI: nvfp4a_quantize_ex, nvfp4a_quantize (NVFP4 and INT8 destinations), nvfp4a_dequantize,
// nvfp4a_swizzle_scales, nvfp4a_transpose.
//
// All of these are HBM-bandwidth-bound byte shuffles with a little FP32 arithmetic.  The arithmetic is Transformer
// Engine's, bit for bit, as the reference states it (include/nvfp4effma.h:118-132, src/quant_nvfp4effma.cuh:39-48 and
// :147-169 there); the kernels are organised for B200: 16-byte loads with every thread owning one 16-value block, grid
// sized in multiples of the SM count, and -- when the global amax has to be computed first -- the second pass walking
// the matrix backwards so that it starts on the bytes the first pass left in the 126 MB L2.
#include <stdio.h>
#include <stdlib.h>
#include <atomic>
#include <type_traits>
#include "common.cuh"

namespace nvb {

#ifndef NVB_HW_CVT
#define NVB_HW_CVT 1  // FP32 -> E2M1 / E4M3 through cvt.rn.satfinite (equal to the software encoders on all finite inputs)
#endif

// ---- element packing ---------------------------------------------------------------------------------------------------
// 8 FP32 -> 8 E2M1 nibbles, value 0 in bits 0..3.  cvt packs its first source into the high nibble.
__device__ __forceinline__ uint32_t e2m1_pack8(const float *v) {
#if NVB_HW_CVT
  uint32_t out;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(out)
      : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
  return out;
#else
  uint32_t out = 0;
#pragma unroll
  for (int e = 0; e < 8; ++e) out |= f32_to_e2m1_sw(v[e]) << (4 * e);
  return out;
#endif
}
__device__ __forceinline__ uint32_t e4m3_encode(float d) {
#if NVB_HW_CVT
  uint32_t out;
  asm("{\n\t.reg .b16 h;\n\tcvt.rn.satfinite.e4m3x2.f32 h, %1, %2;\n\tcvt.u32.u16 %0, h;\n\t}" : "=r"(out) : "f"(0.f), "f"(d));
  return out & 0xFFu;
#else
  return f32_to_e4m3_sw(d);
#endif
}
__device__ __forceinline__ uint32_t scale_encode(float d, bool ue) { return ue ? f32_to_ue5m3_sw(d) : e4m3_encode(d); }

// 16-byte read-only loads with an L2 eviction priority: the amax pass asks L2 to keep what it reads (evict_last), the
// encode pass that follows releases it as it goes (evict_first).
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint4 ldg16_hint(const uint4 *ptr, uint64_t policy) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr), "l"(policy));
  return v;
}
// 16 consecutive dense values (16-byte aligned start) -> FP32
template <int T>
__device__ __forceinline__ void load16(const uint8_t *p, float v[16]) {
  if (T == NVFP4A_FP32) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4 f = __ldg((const float4 *)p + q);
      v[4 * q] = f.x; v[4 * q + 1] = f.y; v[4 * q + 2] = f.z; v[4 * q + 3] = f.w;
    }
  } else {
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const uint4 w = __ldg((const uint4 *)p + q);
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (T == NVFP4A_BF16) {
          v[8 * q + 2 * i] = __uint_as_float(ws[i] << 16);
          v[8 * q + 2 * i + 1] = __uint_as_float(ws[i] & 0xFFFF0000u);
        } else {
          const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&ws[i]));
          v[8 * q + 2 * i] = f.x; v[8 * q + 2 * i + 1] = f.y;
        }
      }
    }
  }
}
template <int T> struct ElemBytes { static constexpr int value = T == NVFP4A_FP32 ? 4 : 2; };

// Encode / decode factors of one global value (reference src/quant_nvfp4effma.cuh:39-48).
struct QGlobal { float gv, s_enc, s_dec; };
__device__ __forceinline__ QGlobal make_global(float gv, float smax, bool amax) {
  if (amax) {
    float s_enc = fminf(__fdiv_rn(__fmul_rn(smax, 6.f), gv), kFltMax);
    if (gv == 0.f || s_enc == 0.f) s_enc = 1.f;
    return {gv, s_enc, __fdiv_rn(1.f, s_enc)};
  }
  return {gv, fminf(__fdiv_rn(1.f, gv), kFltMax), gv};
}

// Destination as the kernels see it.
struct QOut {
  uint8_t *data; int ld;      // nibbles, ld values per row
  uint8_t *sc; int sld;       // scales: > 0 linear, < 0 swizzled (ScalePos)
  const float *g;             // global(s), NULL = 1
  float smax;
  int amax_mode, per_row, ue;
};

// ---- pass 1: global amax ----------------------------------------------------------------------------------------------
// Pure streaming read.  A warp takes units of 256 consecutive 16-byte words of one row (4 KiB), ascending; a lane has
// eight 16-byte loads in flight.  BF16 / FP16 stay packed: |x| is a mask and the maximum a two-lane max (one instruction
// per two values; the bit patterns of non-negative floats order like the floats).  One atomicMax per warp at the end.
template <int T>
__device__ __forceinline__ uint32_t packed_absmax(uint32_t m, uint32_t w) {
  const uint32_t a = w & 0x7FFF7FFFu;
  uint32_t d;
  if (T == NVFP4A_BF16) asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(m), "r"(a));
  else asm("max.f16x2 %0, %1, %2;" : "=r"(d) : "r"(m), "r"(a));
  return d;
}
template <int T>
__global__ void __launch_bounds__(256, 4) amax_kernel(const uint8_t *__restrict__ src, int lds, int rows, int bpr, float *a0, float *a1) {
  const int lane = threadIdx.x & 31;
  const int wpr = bpr * (T == NVFP4A_FP32 ? 4 : 2);        // 16-byte words per row
  const int upr = (wpr + 255) / 256;                        // units per row
  const long long units = (long long)rows * upr, wstride = (long long)gridDim.x * (blockDim.x >> 5);
  float m = 0.f;
  uint32_t pm = 0;
  const uint64_t keep = l2_policy_evict_last();
  for (long long u = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); u < units; u += wstride) {
    const int r = (int)(u / upr), seg = (int)(u - (long long)r * upr);
    const uint4 *rowp = (const uint4 *)(src + (size_t)r * lds * ElemBytes<T>::value) + seg * 256;
    uint4 w[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int c = k * 32 + lane;
      w[k] = seg * 256 + c < wpr ? ldg16_hint(rowp + c, keep) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (T == NVFP4A_FP32) {
        m = fmaxf(m, fmaxf(fmaxf(fabsf(__uint_as_float(w[k].x)), fabsf(__uint_as_float(w[k].y))),
                           fmaxf(fabsf(__uint_as_float(w[k].z)), fabsf(__uint_as_float(w[k].w)))));
      } else {
        pm = packed_absmax<T>(packed_absmax<T>(packed_absmax<T>(packed_absmax<T>(pm, w[k].x), w[k].y), w[k].z), w[k].w);
      }
    }
  }
  if (T == NVFP4A_BF16) m = fmaxf(__uint_as_float(pm << 16), __uint_as_float(pm & 0xFFFF0000u));
  else if (T == NVFP4A_FP16) { const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&pm)); m = fmaxf(f.x, f.y); }
  warp_amax_commit(a0, m);
  if (a1 && a1 != a0) warp_amax_commit(a1, m);
}
// per-row amax: one warp per row
template <int T>
__global__ void __launch_bounds__(256) amax_rows_kernel(const uint8_t *__restrict__ src, int lds, int rows, int bpr, float *a0) {
  const int lane = threadIdx.x & 31, wpb = blockDim.x / 32;
  for (int r = blockIdx.x * wpb + threadIdx.x / 32; r < rows; r += gridDim.x * wpb) {
    float m = 0.f;
    for (int c = lane; c < bpr; c += 32) {
      float v[16];
      load16<T>(src + ((size_t)r * lds + 16 * c) * ElemBytes<T>::value, v);
#pragma unroll
      for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[i]));
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if (lane == 0) a0[r] = m;
  }
}

// ---- pass 2, fast path: rowwise 1 x 16 blocks, one global per tensor, no 4over6 --------------------------------------------
// A warp takes units of 32 consecutive blocks of one row, a lane one block (two 16-byte loads for 16-bit sources).  The
// loads of the next two units are already in flight while a unit is processed (register double buffering), so a warp
// keeps 3 x 1 KiB outstanding.  A lane writes 8 bytes of nibbles (256 contiguous bytes per warp) and contributes its scale
// byte to a 4-byte word that every fourth lane stores -- the same code for the linear and the swizzled layout, where the
// four scales of a 64-value group are contiguous too.  Units are visited from the END of the matrix: after an amax pass
// the tail of the matrix is what L2 still holds.
template <int T> struct PackedBlock { uint4 w[T == NVFP4A_FP32 ? 4 : 2]; };
template <int T>
__device__ __forceinline__ PackedBlock<T> load_block(const uint8_t *p, bool live, uint64_t policy) {
  PackedBlock<T> b;
#pragma unroll
  for (int q = 0; q < (T == NVFP4A_FP32 ? 4 : 2); ++q) b.w[q] = live ? ldg16_hint((const uint4 *)p + q, policy) : make_uint4(0, 0, 0, 0);
  return b;
}
template <int T>
__device__ __forceinline__ void unpack_block(const PackedBlock<T> &b, float v[16]) {
  if (T == NVFP4A_FP32) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      v[4 * q] = __uint_as_float(b.w[q].x); v[4 * q + 1] = __uint_as_float(b.w[q].y);
      v[4 * q + 2] = __uint_as_float(b.w[q].z); v[4 * q + 3] = __uint_as_float(b.w[q].w);
    }
  } else {
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const uint32_t ws[4] = {b.w[q].x, b.w[q].y, b.w[q].z, b.w[q].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (T == NVFP4A_BF16) {
          v[8 * q + 2 * i] = __uint_as_float(ws[i] << 16);
          v[8 * q + 2 * i + 1] = __uint_as_float(ws[i] & 0xFFFF0000u);
        } else {
          const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&ws[i]));
          v[8 * q + 2 * i] = f.x; v[8 * q + 2 * i + 1] = f.y;
        }
      }
    }
  }
}
// One block: 16 values -> scale code and 16 nibbles.  1 / y is the correctly rounded reciprocal (rcp.rn), the same value
// as the IEEE division 1 / y of the reference.
template <bool UE>
__device__ __forceinline__ uint2 quant_block16(float v[16], float enc6, float s_dec, uint32_t &code, float &bmax) {
  bmax = 0.f;
#pragma unroll
  for (int k = 0; k < 16; ++k) bmax = fmaxf(bmax, fabsf(v[k]));
  code = UE ? f32_to_ue5m3_sw(fminf(__fmul_rn(bmax, enc6), kFltMax)) : e4m3_encode(fminf(__fmul_rn(bmax, enc6), kFltMax));
  const float inv = fminf(__frcp_rn(__fmul_rn(UE ? ue5m3_to_f32(code) : e4m3_to_f32(code), s_dec)), kFltMax);
#pragma unroll
  for (int k = 0; k < 16; ++k) v[k] = __fmul_rn(v[k], inv);
  return make_uint2(e2m1_pack8(v), e2m1_pack8(v + 8));
}
// Warps sit side by side along a row (64 blocks = 2 KiB of BF16 each: a lane owns blocks lane and lane + 32 of its
// segment) and walk UP the matrix from its last rows, `rstep` rows per iteration, with the next iteration's loads in flight.
template <int T, bool UE>
__global__ void __launch_bounds__(256, 3) quant_rows_kernel(const uint8_t *__restrict__ src, int lds, int rows, int bpr, QOut o, float *stat) {
  const int lane = threadIdx.x & 31;
  const int upr = (bpr + 63) >> 6;                 // 64-block segments per row
  const int nwarps = gridDim.x * (blockDim.x >> 5), wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int wps = upr < nwarps ? upr : nwarps, rstep = nwarps / wps;
  const QGlobal G = make_global(o.g ? o.g[0] : 1.f, o.smax, o.amax_mode != 0);
  const float enc6 = __fmul_rn(G.s_enc, 1.f / 6.f), s_dec = G.s_dec;
  const ScalePos sp{o.sld};
  // 4-byte scale stores need 4-byte aligned words: always true in the swizzled layout, in the linear one only for an aligned base and row pitch
  const bool words = (bpr & 3) == 0 && (o.sld < 0 || ((o.sld & 3) == 0 && ((uintptr_t)o.sc & 3) == 0));
  uint8_t *const data = o.data, *const sc = o.sc;
  const int ldq = o.ld >> 1;
  const size_t row_bytes = (size_t)lds * ElemBytes<T>::value;
  constexpr int kBlockBytes = 16 * ElemBytes<T>::value;
  const uint64_t drop = l2_policy_evict_first();
  float mx = 0.f;
  if (wid < wps * rstep) {
    for (int seg = wid % wps; seg < upr; seg += wps) {
      const int c0 = seg * 64 + lane, c1 = c0 + 32;
      const bool live0 = c0 < bpr, live1 = c1 < bpr;
      const uint8_t *p = src + (size_t)c0 * kBlockBytes;
      int r = rows - 1 - wid / wps;
      PackedBlock<T> a0 = load_block<T>(p + (size_t)(r < 0 ? 0 : r) * row_bytes, live0 && r >= 0, drop);
      PackedBlock<T> a1 = load_block<T>(p + (size_t)(r < 0 ? 0 : r) * row_bytes + 32 * kBlockBytes, live1 && r >= 0, drop);
      for (; r >= 0; r -= rstep) {
        const int rn = r - rstep;
        const PackedBlock<T> n0 = load_block<T>(p + (size_t)(rn < 0 ? 0 : rn) * row_bytes, live0 && rn >= 0, drop);
        const PackedBlock<T> n1 = load_block<T>(p + (size_t)(rn < 0 ? 0 : rn) * row_bytes + 32 * kBlockBytes, live1 && rn >= 0, drop);
        float v[16], bmax;
        uint32_t code0, code1;
        unpack_block<T>(a0, v);
        const uint2 q0 = quant_block16<UE>(v, enc6, s_dec, code0, bmax);
        mx = fmaxf(mx, bmax);
        unpack_block<T>(a1, v);
        const uint2 q1 = quant_block16<UE>(v, enc6, s_dec, code1, bmax);
        mx = fmaxf(mx, bmax);
        uint8_t *drow = data + (size_t)r * ldq;
        if (live0) __stcs((uint2 *)(drow + 8 * c0), q0);   // streaming stores: the output is not read again here
        if (live1) __stcs((uint2 *)(drow + 8 * c1), q1);
        if (words) {  // lanes 4 t .. 4 t + 3 hold the four scales of one 64-value group (bpr % 4 == 0: all live or none)
          uint32_t w0 = live0 ? code0 << (8 * (lane & 3)) : 0u, w1 = live1 ? code1 << (8 * (lane & 3)) : 0u;
          w0 |= __shfl_xor_sync(0xFFFFFFFFu, w0, 1); w1 |= __shfl_xor_sync(0xFFFFFFFFu, w1, 1);
          w0 |= __shfl_xor_sync(0xFFFFFFFFu, w0, 2); w1 |= __shfl_xor_sync(0xFFFFFFFFu, w1, 2);
          if ((lane & 3) == 0) {
            const size_t rowpos = sp.row(r);
            if (live0) *(uint32_t *)(sc + rowpos + sp.col(c0)) = w0;
            if (live1) *(uint32_t *)(sc + rowpos + sp.col(c1)) = w1;
          }
        } else {
          if (live0) sc[sp.at(r, c0)] = (uint8_t)code0;
          if (live1) sc[sp.at(r, c1)] = (uint8_t)code1;
        }
        a0 = n0; a1 = n1;
      }
    }
  }
  if (stat) warp_amax_commit(stat, mx);
}

// ---- one read: amax and encode in ONE cooperative kernel ------------------------------------------------------------------------
// The global amax must be known before the first block scale, so the matrix is visited twice; this kernel keeps part of it on the
// chip between the visits instead of paying a second full trip to HBM.  One CTA per SM (cooperative launch: all CTAs are resident,
// so the grid barrier between the visits cannot starve), each with a contiguous share of the matrix in units of 64 blocks of one
// row (2 KiB of 16-bit values), dealt to its 16 warps in turn.  Visit 1 takes the amax, four units per warp in flight.  A warp
// keeps its last four units in registers and the six before them in shared memory (10 x 2 KiB x 16 warps = 320 KiB per SM, 47 MB
// over the chip: a third of an 8192 x 8192 BF16 matrix).  After the barrier every step of a warp encodes one on-chip unit and one
// unit read again from memory (in descending order), whose load was issued a step earlier.
// Measured on 8192 x 8192: HBM traffic 159 MB against 287 MB for the two launches, the same 55 us -- the encode arithmetic (about
// 170 instructions per block of 16) at 16 warps per SM, not memory, is what bounds the second visit.
// Per-CTA maxima meet in a device array (no atomics on floats, no memset launch): every CTA reads all of them after the barrier.
// The barrier's wait is bounded like every wait of this library; on expiry the status word gets 0x601 and the kernel goes on
// (with whatever maxima have arrived) so that it always terminates.
constexpr int kQfSmemBytes = 96 * 2048;            // 96 units of 2 KiB stay in shared memory per CTA
constexpr int kQfMaxGrid = 1024;
static __device__ unsigned long long g_qf_arrivals;   // arrivals of every launch so far on this device (each launch adds its grid size, which never changes)
static __device__ float g_qf_max[kQfMaxGrid];      // per-CTA maxima of the current launch

// max |x| of a block of 16-bit values taken on the packed words (bit patterns of non-negative BF16 / FP16 values order like the values)
template <int T>
__device__ __forceinline__ float packed_block_max(const PackedBlock<T> &a) {
  uint32_t pm = 0;
#pragma unroll
  for (int q = 0; q < 2; ++q) pm = packed_absmax<T>(packed_absmax<T>(packed_absmax<T>(packed_absmax<T>(pm, a.w[q].x), a.w[q].y), a.w[q].z), a.w[q].w);
  if (T == NVFP4A_BF16) return fmaxf(__uint_as_float(pm << 16), __uint_as_float(pm & 0xFFFF0000u));
  const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&pm));
  return fmaxf(f.x, f.y);
}
// quant_block16 with the block's maximum already known
// (the factor 1 / (scale * S_dec) depends on the scale code only: it comes from a 256-entry table the CTA fills once)
template <bool UE>
__device__ __forceinline__ uint2 quant_block16_given_max(float v[16], float bmax, float enc6, const float *inv_of_code, uint32_t &code) {
  code = UE ? f32_to_ue5m3_sw(fminf(__fmul_rn(bmax, enc6), kFltMax)) : e4m3_encode(fminf(__fmul_rn(bmax, enc6), kFltMax));
  const float inv = inv_of_code[code];
#pragma unroll
  for (int k = 0; k < 16; ++k) v[k] = __fmul_rn(v[k], inv);
  return make_uint2(e2m1_pack8(v), e2m1_pack8(v + 8));
}
// the two blocks (lane and lane + 32 of a 64-block unit) a lane owns, encoded and stored: nibbles, and the scale bytes as words
// shared by four lanes (the same code for the linear and the swizzled layout)
template <int T, bool UE>
__device__ __forceinline__ void emit_two_blocks(const PackedBlock<T> a0, const PackedBlock<T> a1, int r, int c0, int c1, bool live0, bool live1,
                                             float enc6, const float *inv_of_code, uint8_t *data, int ldq, uint8_t *sc, const ScalePos sp, bool words, int lane) {
  float v[16];
  uint32_t code0, code1;
  unpack_block<T>(a0, v);
  const uint2 q0 = quant_block16_given_max<UE>(v, packed_block_max<T>(a0), enc6, inv_of_code, code0);
  unpack_block<T>(a1, v);
  const uint2 q1 = quant_block16_given_max<UE>(v, packed_block_max<T>(a1), enc6, inv_of_code, code1);
  uint8_t *drow = data + (size_t)r * ldq;
  if (live0) __stcs((uint2 *)(drow + 8 * c0), q0);
  if (live1) __stcs((uint2 *)(drow + 8 * c1), q1);
  if (words) {
    uint32_t w0 = live0 ? code0 << (8 * (lane & 3)) : 0u, w1 = live1 ? code1 << (8 * (lane & 3)) : 0u;
    w0 |= __shfl_xor_sync(0xFFFFFFFFu, w0, 1); w1 |= __shfl_xor_sync(0xFFFFFFFFu, w1, 1);
    w0 |= __shfl_xor_sync(0xFFFFFFFFu, w0, 2); w1 |= __shfl_xor_sync(0xFFFFFFFFu, w1, 2);
    if ((lane & 3) == 0) {
      const size_t rowpos = sp.row(r);
      if (live0) *(uint32_t *)(sc + rowpos + sp.col(c0)) = w0;
      if (live1) *(uint32_t *)(sc + rowpos + sp.col(c1)) = w1;
    }
  } else {
    if (live0) sc[sp.at(r, c0)] = (uint8_t)code0;
    if (live1) sc[sp.at(r, c1)] = (uint8_t)code1;
  }
}

template <int T, bool UE, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1)
quant_fused_kernel(const uint8_t *__restrict__ src, int lds, int rows, int bpr, QOut o, float *gout, float *stat, unsigned *status, unsigned tag) {
  static_assert(T != NVFP4A_FP32, "16-bit sources");
  extern __shared__ uint4 qf_keep[];   // [warp][unit][4 words][32 lanes]
  constexpr int kQfWarps = WARPS, kQfRegUnits = WARPS == 16 ? 4 : 0, kQfSmemUnits = 96 / WARPS, kFlight = WARPS == 16 ? 4 : 2;
  __shared__ float warp_max[kQfWarps];
  __shared__ float gmax_s;
  __shared__ float inv_of_code[256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int upr = (bpr + 63) >> 6;
  const long long U = (long long)rows * upr;   // (below 2^31: the host checks)
  const unsigned u_begin = (unsigned)(U * blockIdx.x / gridDim.x), u_end = (unsigned)(U * (blockIdx.x + 1) / gridDim.x);
  const int n_cta = (int)(u_end - u_begin);
  const int n_w = n_cta > warp ? (n_cta - warp + kQfWarps - 1) / kQfWarps : 0;   // this warp's units: u_begin + warp + 16 j
  // of a warp's units the last n_rg stay in registers, the n_sm before them in shared memory; the first n_glob are read again
  const int n_ret = n_w < kQfRegUnits + kQfSmemUnits ? n_w : kQfRegUnits + kQfSmemUnits;
  const int n_rg = n_ret < kQfRegUnits ? n_ret : kQfRegUnits, n_sm = n_ret - n_rg, n_glob = n_w - n_ret;
  const size_t row_bytes = (size_t)lds * 2;
  // every load tells L2 to drop the line early: asking it to keep lines (evict_last) slowed the first visit from 22 to 28 us and
  // bought no hits for the second
  const uint64_t drop_pol = l2_policy_evict_first();
  uint4 *const my_smem = qf_keep + (size_t)warp * kQfSmemUnits * 128;
  struct Unit { int r, c0; };
  auto unit_of = [&](int j) {
    const unsigned u = u_begin + warp + (unsigned)(kQfWarps * j), r = u / (unsigned)upr;
    return Unit{(int)r, (int)(u - r * (unsigned)upr) * 64 + lane};
  };
  auto load_unit = [&](int j, uint64_t pol, PackedBlock<T> &a0, PackedBlock<T> &a1) {
    const Unit t = unit_of(j);
    const uint8_t *p = src + (size_t)t.r * row_bytes + (size_t)t.c0 * 32;
    a0 = load_block<T>(p, t.c0 < bpr, pol);
    a1 = load_block<T>(p + 32 * 32, t.c0 + 32 < bpr, pol);
  };
  auto absmax_of = [&](uint32_t pm, const PackedBlock<T> &a) {
#pragma unroll
    for (int q = 0; q < 2; ++q) pm = packed_absmax<T>(packed_absmax<T>(packed_absmax<T>(packed_absmax<T>(pm, a.w[q].x), a.w[q].y), a.w[q].z), a.w[q].w);
    return pm;
  };

  // ---- visit 1: amax; the last units stay on chip ----
  uint32_t pm = 0;
  int j = 0;
  for (; j + kFlight <= n_glob; j += kFlight) {   // several units per warp in flight; nothing of them is kept
    PackedBlock<T> x[2 * kFlight];
#pragma unroll
    for (int q = 0; q < kFlight; ++q) load_unit(j + q, drop_pol, x[2 * q], x[2 * q + 1]);
#pragma unroll
    for (int q = 0; q < 2 * kFlight; ++q) pm = absmax_of(pm, x[q]);
  }
  for (; j < n_glob + n_sm; ++j) {    // the rest of those, then the units that stay in shared memory
    PackedBlock<T> a0, a1;
    load_unit(j, drop_pol, a0, a1);
    pm = absmax_of(absmax_of(pm, a0), a1);
    if (j >= n_glob) {
      uint4 *d = my_smem + (j - n_glob) * 128 + lane;
      d[0] = a0.w[0]; d[32] = a0.w[1]; d[64] = a1.w[0]; d[96] = a1.w[1];
    }
  }
  // the last units stay in registers (named, not an array: they must not end up in local memory); all four loads fly together
  PackedBlock<T> rk0_0, rk1_0, rk0_1, rk1_1, rk0_2, rk1_2, rk0_3, rk1_3;
  rk0_0.w[0] = rk0_0.w[1] = make_uint4(0, 0, 0, 0);
  rk1_0 = rk0_1 = rk1_1 = rk0_2 = rk1_2 = rk0_3 = rk1_3 = rk0_0;
  if (kQfRegUnits) {
    if (n_rg > 0) load_unit(j, drop_pol, rk0_0, rk1_0);
    if (n_rg > 1) load_unit(j + 1, drop_pol, rk0_1, rk1_1);
    if (n_rg > 2) load_unit(j + 2, drop_pol, rk0_2, rk1_2);
    if (n_rg > 3) load_unit(j + 3, drop_pol, rk0_3, rk1_3);
    pm = absmax_of(absmax_of(absmax_of(absmax_of(pm, rk0_0), rk1_0), rk0_1), rk1_1);
    pm = absmax_of(absmax_of(absmax_of(absmax_of(pm, rk0_2), rk1_2), rk0_3), rk1_3);
  }
  float m = T == NVFP4A_BF16 ? fmaxf(__uint_as_float(pm << 16), __uint_as_float(pm & 0xFFFF0000u))
                             : fmaxf(__half2float(__ushort_as_half((unsigned short)(pm & 0xFFFFu))), __half2float(__ushort_as_half((unsigned short)(pm >> 16))));
#pragma unroll
  for (int of = 16; of; of >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, of));
  if (lane == 0) warp_max[warp] = m;
  __syncthreads();

  // ---- grid barrier (bounded) ----
  // One 64-bit arrival counter that only grows: every launch of this kernel on a device has the same grid (one CTA per SM), so the
  // arrival that returns `old` belongs to the round that is complete at (old / grid + 1) * grid.  Three dependent trips to L2 in all:
  // the arrival (which publishes this CTA's maximum), the poll that sees the last arrival, the read of all CTAs' maxima by ONE warp
  // per CTA (a line that thousands of warps read at once is served one request at a time).
  if (warp == 0) {
    float cm = lane < kQfWarps ? warp_max[lane] : 0.f;
#pragma unroll
    for (int of = 16; of; of >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xFFFFFFFFu, cm, of));
    if (lane == 0) {
      g_qf_max[blockIdx.x] = cm;
      unsigned long long old, now;
      asm volatile("atom.add.acq_rel.gpu.global.u64 %0, [%1], 1;" : "=l"(old) : "l"(&g_qf_arrivals) : "memory");
      const unsigned long long target = (old / gridDim.x + 1) * gridDim.x;
      const long long start = clock64();
      for (;;) {
        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(now) : "l"(&g_qf_arrivals) : "memory");
        if (now >= target) break;
        if (clock64() - start > 2000000000ll) { atomicCAS(status, 0u, 0x601u | tag); break; }
      }
    }
    __syncwarp();
    float all = 0.f;
    for (unsigned i = lane; i < gridDim.x; i += 32) all = fmaxf(all, __ldcg(&g_qf_max[i]));
#pragma unroll
    for (int of = 16; of; of >>= 1) all = fmaxf(all, __shfl_xor_sync(0xFFFFFFFFu, all, of));
    if (lane == 0) gmax_s = all;
  }
  __syncthreads();
  const float gmax = gmax_s;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    *gout = gmax;
    if (stat && gmax > 0.f) atomicMax((int *)stat, __float_as_int(gmax));
  }

  // ---- visit 2: encode, on-chip units first, then back through L2 ----
  const QGlobal G = make_global(gmax, o.smax, true);
  const float enc6 = __fmul_rn(G.s_enc, 1.f / 6.f), s_dec = G.s_dec;
  if (threadIdx.x < 256) inv_of_code[threadIdx.x] = fminf(__frcp_rn(__fmul_rn(scale_to_f32(threadIdx.x, UE), s_dec)), kFltMax);
  __syncthreads();
  const ScalePos sp{o.sld};
  const bool words = (bpr & 3) == 0 && (o.sld < 0 || ((o.sld & 3) == 0 && ((uintptr_t)o.sc & 3) == 0));
  uint8_t *const data = o.data, *const sc = o.sc;
  const int ldq = o.ld >> 1;
  auto emit = [&](int j, const PackedBlock<T> &x0, const PackedBlock<T> &x1) {
    const Unit t = unit_of(j);
    emit_two_blocks<T, UE>(x0, x1, t.r, t.c0, t.c0 + 32, t.c0 < bpr, t.c0 + 32 < bpr, enc6, inv_of_code, data, ldq, sc, sp, words, lane);
  };
  // Interleaved: every step encodes one on-chip unit (registers first, then shared memory) and one re-read unit whose load was
  // issued a step earlier, so the arithmetic of the on-chip units hides the latency of the re-reads.  The encoder is a long
  // stretch of code: it appears at two places only (one loop), so that it stays in the instruction cache.
  PackedBlock<T> n0, n1;
  int jg = n_glob - 1;
  if (jg >= 0) load_unit(jg, drop_pol, n0, n1);
  for (int i = 0; i < n_ret || jg >= 0; ++i) {
    if (i < n_ret) {
      PackedBlock<T> x0, x1;
      int j;
      if (kQfRegUnits && i < n_rg) {   // (i is the same for the whole warp)
        x0 = i == 0 ? rk0_0 : i == 1 ? rk0_1 : i == 2 ? rk0_2 : rk0_3;
        x1 = i == 0 ? rk1_0 : i == 1 ? rk1_1 : i == 2 ? rk1_2 : rk1_3;
        j = n_glob + n_sm + i;
      } else {
        const uint4 *d = my_smem + (i - n_rg) * 128 + lane;
        x0.w[0] = d[0]; x0.w[1] = d[32]; x1.w[0] = d[64]; x1.w[1] = d[96];
        j = n_glob + i - n_rg;
      }
      emit(j, x0, x1);
    }
    if (jg >= 0) {
      const PackedBlock<T> c0 = n0, c1 = n1;
      if (jg >= 1) load_unit(jg - 1, drop_pol, n0, n1);
      emit(jg, c0, c1);
      --jg;
    }
  }
  __syncthreads();
}

// ---- pass 2, general path ----------------------------------------------------------------------------------------------
// 16 consecutive lanes own one 16 x 16 tile of the OUTPUT matrix (lane i its row 16 t + i): rowwise or columnwise
// (COL: output row = source column), 1 x 16 blocks or 16 x 16 tiles, 4over6, per-row globals, either scale type.
__device__ __forceinline__ float group16_max(float v, unsigned mask) {
#pragma unroll
  for (int o = 8; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(mask, v, o, 16));
  return v;
}
// Transformer Engine's 16-lane tree: shfl_down by 8, 4, 2, 1, the result of lane 0
__device__ __forceinline__ float group16_tree(float v, unsigned mask) {
#pragma unroll
  for (int o = 8; o; o >>= 1) v = __fadd_rn(v, __shfl_down_sync(mask, v, o, 16));
  return __shfl_sync(mask, v, 0, 16);
}
__device__ __forceinline__ uint2 pack16_scaled(const float *x, float inv) {
  float v[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __fmul_rn(x[i], inv);
  return make_uint2(e2m1_pack8(v), e2m1_pack8(v + 8));
}
// error of one 4over6 candidate, element order; d = ((e2m1 * sf) * amax) / (6 M) - x with an IEEE division
__device__ __forceinline__ float fos_error(const float *x, uint2 q, float sf, float amax, float denom, int fos) {
  float err = 0.f;
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    const uint32_t nib = ((e < 8 ? q.x : q.y) >> (4 * (e & 7))) & 15u;
    const float val = __fdiv_rn(__fmul_rn(__fmul_rn(e2m1_to_f32(nib), sf), amax), denom);
    const float d = __fsub_rn(val, x[e]);
    err = __fadd_rn(err, fos == NVFP4A_4OVER6_MSE ? __fmul_rn(d, d) : fabsf(d));
  }
  return err;
}
template <int T, bool COL>
__global__ void __launch_bounds__(256) quant_general_kernel(const uint8_t *__restrict__ src, int lds, int rows, int cols, QOut o, int tile,
                                                            int fos, float *stat) {
  const int orows = COL ? cols : rows, ocols = COL ? rows : cols;
  const int ocb = (ocols + 15) / 16, tiles = (orows + 15) / 16;
  const long long units = (long long)tiles * ocb;
  const int lane = threadIdx.x & 15;
  const unsigned gmask = 0xFFFFu << (threadIdx.x & 16);
  const ScalePos sp{o.sld};
  const bool ue = o.ue != 0;
  QGlobal G0 = {};
  if (!o.per_row) G0 = make_global(o.g ? o.g[0] : 1.f, o.smax, o.amax_mode != 0);
  const float denom = __fmul_rn(6.f, o.smax);
  float mx = 0.f;
  for (long long u = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / 16; u < units; u += (long long)gridDim.x * blockDim.x / 16) {
    const int t = (int)(u / ocb), c = (int)(u - (long long)t * ocb), orow = 16 * t + lane;
    const bool live = orow < orows;
    float x[16];
    if (!COL) {
      if (live) load16<T>(src + ((size_t)orow * lds + 16 * c) * ElemBytes<T>::value, x);
      else {
#pragma unroll
        for (int e = 0; e < 16; ++e) x[e] = 0.f;
      }
    } else {
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const int sr = 16 * c + e;
        x[e] = live && sr < rows ? load_dense(T, src, (size_t)sr * lds + orow) : 0.f;
      }
    }
    float bmax = 0.f;
#pragma unroll
    for (int e = 0; e < 16; ++e) bmax = fmaxf(bmax, fabsf(x[e]));
    mx = fmaxf(mx, bmax);
    if (tile == 16) bmax = group16_max(bmax, gmask);
    const QGlobal G = o.per_row ? make_global(o.g[live ? orow : 0], o.smax, o.amax_mode != 0) : G0;
    uint32_t code; uint2 q;
    if (fos == NVFP4A_4OVER6_OFF) {
      code = scale_encode(fminf(__fmul_rn(bmax, __fmul_rn(G.s_enc, 1.f / 6.f)), kFltMax), ue);
      q = pack16_scaled(x, fminf(__fdiv_rn(1.f, __fmul_rn(scale_to_f32(code, ue), G.s_dec)), kFltMax));
    } else {
      const float base = __fmul_rn(__fdiv_rn(bmax, 6.f), G.s_enc);
      const uint32_t c4 = e4m3_encode(fminf(__fmul_rn(base, 1.5f), 448.f)), c6 = e4m3_encode(fminf(base, 448.f));
      const float sf4 = e4m3_to_f32(c4), sf6 = e4m3_to_f32(c6);
      const uint2 q4 = pack16_scaled(x, fminf(__fdiv_rn(1.f, __fmul_rn(sf4, G.s_dec)), kFltMax));
      const uint2 q6 = pack16_scaled(x, fminf(__fdiv_rn(1.f, __fmul_rn(sf6, G.s_dec)), kFltMax));
      float e4 = fos_error(x, q4, sf4, G.gv, denom, fos), e6 = fos_error(x, q6, sf6, G.gv, denom, fos);
      if (tile == 16) { e4 = group16_tree(e4, gmask); e6 = group16_tree(e6, gmask); }
      const bool pick4 = e4 < e6;  // ties keep map-to-6
      code = pick4 ? c4 : c6;
      q = pick4 ? q4 : q6;
    }
    if (live) {
      *(uint2 *)(o.data + (size_t)orow * (o.ld / 2) + 8 * c) = q;
      o.sc[sp.at(orow, c)] = (uint8_t)code;
    }
  }
  if (stat) warp_amax_commit(stat, mx);
}

// ---- INT8 destination (W4A8 activations): sb = bmax / 127, q = clamp(rint(x / sb), +-127), 0 where sb == 0 -------------------
template <int T>
__global__ void __launch_bounds__(256) quant_int8_kernel(const uint8_t *__restrict__ src, int lds, int8_t *__restrict__ dst, int ldd,
                                                         float *__restrict__ scales, int ld_scale, int rows, int bpr, float *stat) {
  const long long total = (long long)rows * bpr, stride = (long long)gridDim.x * blockDim.x;
  float mx = 0.f;
  for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < total; b += stride) {
    const int r = (int)(b / bpr), c = (int)(b - (long long)r * bpr);
    float v[16];
    load16<T>(src + ((size_t)r * lds + 16 * c) * ElemBytes<T>::value, v);
    float bmax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) bmax = fmaxf(bmax, fabsf(v[i]));
    mx = fmaxf(mx, bmax);
    const float sb = __fdiv_rn(bmax, 127.f);
    uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int q = sb > 0.f ? (int)fminf(fmaxf(rintf(__fdiv_rn(v[i], sb)), -127.f), 127.f) : 0;
      w[i >> 2] |= (uint32_t)(uint8_t)(int8_t)q << (8 * (i & 3));
    }
    *(uint4 *)(dst + (size_t)r * ldd + 16 * c) = make_uint4(w[0], w[1], w[2], w[3]);
    scales[(size_t)r * ld_scale + c] = sb;
  }
  if (stat) warp_amax_commit(stat, mx);
}

// ---- dequantize: (e * sb) * g, or e * ((sb * amax) * (1 / (6 M))) -------------------------------------------------------------
template <int T>
__global__ void __launch_bounds__(256) dequant_kernel(QOut q, uint8_t *__restrict__ dst, int ldd, int rows, int bpr, float *stat) {
  const long long total = (long long)rows * bpr, stride = (long long)gridDim.x * blockDim.x;
  const ScalePos sp{q.sld};
  const float finv = 1.0f / (6.f * q.smax);
  const float g0 = q.g ? q.g[0] : (q.amax_mode ? 6.f * q.smax : 1.f);
  float mx = 0.f;
  for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < total; b += stride) {
    const int r = (int)(b / bpr), c = (int)(b - (long long)r * bpr);
    const uint2 w = *(const uint2 *)(q.data + (size_t)r * (q.ld / 2) + 8 * c);
    const float sb = scale_to_f32(q.sc[sp.at(r, c)], q.ue != 0);
    const float gv = q.per_row ? q.g[r] : g0;
    const float fin = q.amax_mode ? __fmul_rn(__fmul_rn(sb, gv), finv) : 0.f;
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float e = e2m1_to_f32(((i < 8 ? w.x : w.y) >> (4 * (i & 7))) & 15u);
      v[i] = q.amax_mode ? __fmul_rn(e, fin) : __fmul_rn(__fmul_rn(e, sb), gv);
      mx = fmaxf(mx, fabsf(v[i]));
    }
    uint8_t *p = dst + ((size_t)r * ldd + 16 * c) * ElemBytes<T>::value;
    if (T == NVFP4A_FP32) {
#pragma unroll
      for (int k = 0; k < 4; ++k) ((float4 *)p)[k] = make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
    } else {
      uint32_t h[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (T == NVFP4A_BF16) h[k] = f32_to_bf16_bits(v[2 * k]) | (f32_to_bf16_bits(v[2 * k + 1]) << 16);
        else { const __half2 t = __floats2half2_rn(v[2 * k], v[2 * k + 1]); h[k] = *reinterpret_cast<const uint32_t *>(&t); }
      }
      ((uint4 *)p)[0] = make_uint4(h[0], h[1], h[2], h[3]);
      ((uint4 *)p)[1] = make_uint4(h[4], h[5], h[6], h[7]);
    }
  }
  if (stat) warp_amax_commit(stat, mx);
}

// ---- scale layout conversion: one thread per scale of the padded swizzled matrix ----------------------------------------------
__global__ void swizzle_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, int ld, int rows, int cols16, int sc, int to_swz) {
  const ScalePos sp{-sc};
  const long long n = (long long)((rows + 127) / 128 * 128) * sc;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / sc), c = (int)(i - (long long)r * sc);
    const bool inside = r < rows && c < cols16;
    if (to_swz) dst[sp.at(r, c)] = inside ? src[(size_t)r * ld + c] : (uint8_t)0;
    else if (inside) dst[(size_t)r * ld + c] = src[sp.at(r, c)];
  }
}

// ---- transpose of a 16 x 16-tiled matrix: one thread per tile ------------------------------------------------------------------
__global__ void transpose_kernel(QOut s, QOut d, int rows, int cols) {
  const int tr = rows / 16, tc = cols / 16;
  const ScalePos ss{s.sld}, ds{d.sld};
  for (long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x; u < (long long)tr * tc; u += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(u / tc), c = (int)(u - (long long)t * tc);
    uint2 in[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) in[i] = *(const uint2 *)(s.data + (size_t)(16 * t + i) * (s.ld / 2) + 8 * c);
    const uint8_t code = s.sc[ss.at(16 * t, c)];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      uint32_t w[2] = {0, 0};
#pragma unroll
      for (int i = 0; i < 16; ++i) w[i >> 3] |= (((j < 8 ? in[i].x : in[i].y) >> (4 * (j & 7))) & 15u) << (4 * (i & 7));
      *(uint2 *)(d.data + (size_t)(16 * c + j) * (d.ld / 2) + 8 * t) = make_uint2(w[0], w[1]);
      d.sc[ds.at(16 * c + j, t)] = code;
    }
  }
}

// ---- host helpers ---------------------------------------------------------------------------------------------------------------
static int grid_for(long long threads, int per_sm = 8) {
  const long long want = (threads + 255) / 256;
  const long long cap = (long long)device_sms() * per_sm;  // a whole number of CTAs per SM
  return (int)(want < 1 ? 1 : want < cap ? want : cap);
}
template <class F> static void by_dense(int t, F f) {
  if (t == NVFP4A_BF16) f(std::integral_constant<int, NVFP4A_BF16>());
  else if (t == NVFP4A_FP16) f(std::integral_constant<int, NVFP4A_FP16>());
  else f(std::integral_constant<int, NVFP4A_FP32>());
}
static bool is_dense(nvfp4a_dtype t) { return t == NVFP4A_BF16 || t == NVFP4A_FP16 || t == NVFP4A_FP32; }

// Checks shared by quantize / dequantize: q is the NVFP4 side ([rows][qcols]), x the dense one ([rows][cols]).
static nvfp4a_status check_convert(const char *fn, const nvfp4a_tensor *q, int ldq, const nvfp4a_tensor *x, int ldx, int rows,
                                   int cols, int qcols = -1) {
  if (qcols < 0) qcols = cols;
  if (!q || !x || !q->data || !x->data) return fail(NVFP4A_INVALID_VALUE, "%s: a tensor or its data pointer is NULL", fn);
  if (q->dtype != NVFP4A_NVFP4) return fail(NVFP4A_INVALID_VALUE, "%s: the quantized side must be NVFP4 (dtype %d)", fn, (int)q->dtype);
  if (!is_dense(x->dtype)) return fail(NVFP4A_INVALID_VALUE, "%s: the dense side must be BF16, FP16 or FP32 (dtype %d)", fn, (int)x->dtype);
  if (!q->block_scale) return fail(NVFP4A_INVALID_VALUE, "%s: block_scale is NULL", fn);
  if (rows < 0 || cols < 0) return fail(NVFP4A_INVALID_VALUE, "%s: negative size (rows = %d, cols = %d)", fn, rows, cols);
  if (cols % 16 || ldq % 16 || ldx % 16)
    return fail(NVFP4A_INVALID_VALUE, "%s: cols (%d) and both leading dimensions (%d, %d) must be multiples of 16", fn, cols, ldq, ldx);
  if (ldq < qcols || ldx < cols) return fail(NVFP4A_INVALID_VALUE, "%s: a leading dimension is below its row length (%d, %d)", fn, qcols, cols);
  if (((uintptr_t)q->data & 7) || ((uintptr_t)x->data & 15))
    return fail(NVFP4A_INVALID_VALUE, "%s: NVFP4 data must be 8-byte and dense data 16-byte aligned", fn);
  return NVFP4A_OK;
}
static QOut make_qout(const nvfp4a_tensor *t, int ld, int sld) {
  QOut o;
  o.data = (uint8_t *)t->data; o.ld = ld; o.sc = (uint8_t *)t->block_scale; o.sld = sld; o.g = t->global_scale;
  o.smax = scale_max_of(t);
  o.amax_mode = (t->flags & NVFP4A_GLOBAL_AMAX) ? 1 : 0;
  o.per_row = (t->flags & NVFP4A_GLOBAL_PER_ROW) ? 1 : 0;
  o.ue = (t->flags & NVFP4A_SCALES_UE5M3) ? 1 : 0;
  return o;
}

unsigned int *kernel_status_device_ptr();
unsigned next_launch_tag();
static std::atomic<int> g_quant_fused{1};
static bool quant_fused_enabled() { return g_quant_fused.load() != 0; }

template <int T, bool UE, int WARPS>
static cudaError_t launch_quant_fused_w(const uint8_t *src, int lds, int rows, int bpr, QOut o, const nvfp4a_tensor *dst, cudaStream_t stream) {
  static std::atomic<int> ready[64];   // per device: 0 unknown, 1 usable, -1 no cooperative launch
  int dev = 0;
  cudaGetDevice(&dev);
  int st = ready[dev & 63].load();
  if (st == 0) {
    int coop = 0;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    int per_sm = 0;
    if (coop && cudaFuncSetAttribute(quant_fused_kernel<T, UE, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, kQfSmemBytes) == cudaSuccess)
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quant_fused_kernel<T, UE, WARPS>, WARPS * 32, kQfSmemBytes);
    st = (coop && per_sm >= 1) ? 1 : -1;
    ready[dev & 63] = st;
    (void)cudaGetLastError();
  }
  if (st < 0 || device_sms() > kQfMaxGrid) return cudaErrorNotSupported;
  if (cudaError_t e = cudaFuncSetAttribute(quant_fused_kernel<T, UE, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, kQfSmemBytes)) return e;
  float *gout = (float *)dst->global_scale, *stat = dst->amax;
  unsigned *status = kernel_status_device_ptr();
  unsigned tag = next_launch_tag();
  void *args[] = {(void *)&src, (void *)&lds, (void *)&rows, (void *)&bpr, (void *)&o, (void *)&gout, (void *)&stat, (void *)&status, (void *)&tag};
  return cudaLaunchCooperativeKernel((const void *)quant_fused_kernel<T, UE, WARPS>, dim3(device_sms()), dim3(WARPS * 32), args, kQfSmemBytes, stream);
}
template <int T, bool UE>
static cudaError_t launch_quant_fused(const uint8_t *src, int lds, int rows, int bpr, QOut o, const nvfp4a_tensor *dst, cudaStream_t stream) {
  if ((long long)rows * ((bpr + 63) / 64) >= (1ll << 31)) return cudaErrorNotSupported;
  return launch_quant_fused_w<T, UE, 16>(src, lds, rows, bpr, o, dst, stream);
}

}  // namespace nvb

using namespace nvb;


extern "C" int nvfp4a_b200_set_quant_fused(int on) {
  nvb::g_quant_fused = on ? 1 : 0;
  return 0;
}

extern "C" nvfp4a_status nvfp4a_quantize_ex(const nvfp4a_tensor *src, int lds, int rows, int cols, const nvfp4a_tensor *rowwise,
                                            int ld_row, const nvfp4a_tensor *columnwise, int ld_col, const nvfp4a_quant_config *cfg,
                                            cudaStream_t stream) {
  clear_error();
  const char *fn = "nvfp4a_quantize_ex";
  nvfp4a_quant_config c = {1, NVFP4A_4OVER6_OFF, 0};
  if (cfg) c = *cfg;
  if (!src || !src->data) return fail(NVFP4A_INVALID_VALUE, "%s: src or src->data is NULL", fn);
  if (!rowwise && !columnwise) return fail(NVFP4A_INVALID_VALUE, "%s: neither a rowwise nor a columnwise destination", fn);
  if (c.tile_rows != 1 && c.tile_rows != 16) return fail(NVFP4A_INVALID_VALUE, "%s: tile_rows = %d (must be 1 or 16)", fn, c.tile_rows);
  if (c.four_over_six < NVFP4A_4OVER6_OFF || c.four_over_six > NVFP4A_4OVER6_MSE)
    return fail(NVFP4A_INVALID_VALUE, "%s: four_over_six = %d is not a valid mode", fn, (int)c.four_over_six);
  const int rows16 = (rows + 15) / 16 * 16;
  int sld[2] = {0, 0};
  for (int col = 0; col < 2; ++col) {
    const nvfp4a_tensor *d = col ? columnwise : rowwise;
    if (!d) continue;
    const char *name = col ? "columnwise" : "rowwise";
    const int ld = col ? ld_col : ld_row, orows = col ? cols : rows, ocols = col ? rows16 : cols;
    if (nvfp4a_status st = check_convert(fn, d, ld, src, lds, rows, cols, ocols)) return st;
    if (nvfp4a_status st = check_scales(fn, name, d, orows, ocols, &sld[col])) return st;
    if (col && (d->flags & NVFP4A_GLOBAL_PER_ROW))
      return fail(NVFP4A_INVALID_VALUE, "%s: per-row globals exist for the rowwise destination only", fn);
    if ((d->flags & NVFP4A_GLOBAL_PER_ROW) && c.tile_rows != 1)
      return fail(NVFP4A_INVALID_VALUE, "%s: per-row globals need 1 x 16 blocks", fn);
    if (c.four_over_six && (!(d->flags & NVFP4A_GLOBAL_AMAX) || (d->flags & NVFP4A_SCALES_UE5M3)))
      return fail(NVFP4A_INVALID_VALUE, "%s: 4over6 needs an amax global and E4M3 scales (%s)", fn, name);
    if (c.compute_amax && (!(d->flags & NVFP4A_GLOBAL_AMAX) || !d->global_scale))
      return fail(NVFP4A_INVALID_VALUE, "%s: compute_amax needs NVFP4A_GLOBAL_AMAX and global_scale storage (%s)", fn, name);
  }
  if (cols % 16) return fail(NVFP4A_INVALID_VALUE, "%s: cols = %d is not a multiple of 16", fn, cols);
  if ((long long)rows * cols == 0) return NVFP4A_OK;
  if (nvfp4a_status st = check_device()) return st;

  const uint8_t *s = (const uint8_t *)src->data;
  const int bpr = cols / 16;
  const long long blocks = (long long)rows * bpr;
  // One-read path: the common recipe (rowwise 1 x 16 blocks, one amax for the tensor, no 4over6, 16-bit source) on a matrix large
  // enough to occupy every SM runs as ONE cooperative kernel that reads most of the source once (quant_fused_kernel).
  if (c.compute_amax && rowwise && !columnwise && c.tile_rows == 1 && c.four_over_six == NVFP4A_4OVER6_OFF &&
      !(rowwise->flags & NVFP4A_GLOBAL_PER_ROW) && src->dtype != NVFP4A_FP32 && (bpr & 3) == 0 && (long long)rows * cols >= (8ll << 20) &&
      quant_fused_enabled()) {
    const QOut o = make_qout(rowwise, ld_row, sld[0]);
    cudaError_t e = cudaSuccess;
    by_dense(src->dtype, [&](auto tc) {
      constexpr int T = decltype(tc)::value;
      if constexpr (T != NVFP4A_FP32) e = o.ue ? launch_quant_fused<T, true>(s, lds, rows, bpr, o, rowwise, stream) : launch_quant_fused<T, false>(s, lds, rows, bpr, o, rowwise, stream);
    });
    if (e != cudaErrorNotSupported) return cuda_fail(e, "nvfp4a_quantize_ex: kernel launch");
    // (a device without cooperative launch takes the two-pass path below)
  }
  if (c.compute_amax) {
    float *ar = rowwise ? (float *)rowwise->global_scale : nullptr, *ac = columnwise ? (float *)columnwise->global_scale : nullptr;
    const bool row_per_row = rowwise && (rowwise->flags & NVFP4A_GLOBAL_PER_ROW);
    by_dense(src->dtype, [&](auto tc) {
      constexpr int T = decltype(tc)::value;
      if (row_per_row) {
        amax_rows_kernel<T><<<grid_for((long long)rows * 32), 256, 0, stream>>>(s, lds, rows, bpr, ar);
        ar = nullptr;
      }
      if (ar || ac) {
        float *p0 = ar ? ar : ac, *p1 = ar ? ac : nullptr;
        cudaMemsetAsync(p0, 0, 4, stream);
        if (p1 && p1 != p0) cudaMemsetAsync(p1, 0, 4, stream);
        amax_kernel<T><<<device_sms() * 4, 256, 0, stream>>>(s, lds, rows, bpr, p0, p1);
      }
    });
  }
  for (int col = 0; col < 2; ++col) {
    const nvfp4a_tensor *d = col ? columnwise : rowwise;
    if (!d) continue;
    const QOut o = make_qout(d, col ? ld_col : ld_row, sld[col]);
    const bool fast = !col && c.tile_rows == 1 && c.four_over_six == NVFP4A_4OVER6_OFF && !o.per_row;
    by_dense(src->dtype, [&](auto tc) {
      constexpr int T = decltype(tc)::value;
      if (fast) {
        // one wave: 3 CTAs of 256 threads per SM
        if (o.ue) quant_rows_kernel<T, true><<<device_sms() * 3, 256, 0, stream>>>(s, lds, rows, bpr, o, d->amax);
        else quant_rows_kernel<T, false><<<device_sms() * 3, 256, 0, stream>>>(s, lds, rows, bpr, o, d->amax);
      } else {
        const int orows = col ? cols : rows, ocols = col ? rows : cols;
        const long long units = (long long)((orows + 15) / 16) * ((ocols + 15) / 16);
        if (col) quant_general_kernel<T, true><<<grid_for(units * 16), 256, 0, stream>>>(s, lds, rows, cols, o, c.tile_rows, (int)c.four_over_six, d->amax);
        else quant_general_kernel<T, false><<<grid_for(units * 16), 256, 0, stream>>>(s, lds, rows, cols, o, c.tile_rows, (int)c.four_over_six, d->amax);
      }
    });
  }
  return cuda_fail(cudaGetLastError(), "nvfp4a_quantize_ex: kernel launch");
}

extern "C" nvfp4a_status nvfp4a_quantize(const nvfp4a_tensor *src, int lds, const nvfp4a_tensor *dst, int ldd, int rows, int cols,
                                         cudaStream_t stream) {
  clear_error();
  const char *fn = "nvfp4a_quantize";
  if (dst && dst->dtype == NVFP4A_INT8) {
    nvfp4a_tensor q = *dst;
    q.dtype = NVFP4A_NVFP4;  // the shared checks, then the INT8 specifics
    if (nvfp4a_status st = check_convert(fn, &q, ldd, src, lds, rows, cols)) return st;
    if (dst->flags) return fail(NVFP4A_INVALID_VALUE, "%s: flags apply to NVFP4 destinations only", fn);
    if (dst->ld_scale && dst->ld_scale < cols / 16)
      return fail(NVFP4A_INVALID_VALUE, "%s: ld_scale = %d is below cols / 16 = %d", fn, dst->ld_scale, cols / 16);
    if (((uintptr_t)dst->data & 15) || ((uintptr_t)dst->block_scale & 3))
      return fail(NVFP4A_INVALID_VALUE, "%s: INT8 data must be 16-byte and its FP32 scales 4-byte aligned", fn);
    if ((long long)rows * cols == 0) return NVFP4A_OK;
    if (nvfp4a_status st = check_device()) return st;
    const int bpr = cols / 16, lsc = dst->ld_scale ? dst->ld_scale : bpr;
    by_dense(src->dtype, [&](auto tc) {
      quant_int8_kernel<decltype(tc)::value><<<grid_for((long long)rows * bpr), 256, 0, stream>>>(
          (const uint8_t *)src->data, lds, (int8_t *)dst->data, ldd, (float *)dst->block_scale, lsc, rows, bpr, dst->amax);
    });
    return cuda_fail(cudaGetLastError(), "nvfp4a_quantize: kernel launch");
  }
  const nvfp4a_status st = nvfp4a_quantize_ex(src, lds, rows, cols, dst, ldd, nullptr, 0, nullptr, stream);
  if (st != NVFP4A_OK) {  // report under this entry's name
    char msg[512];
    snprintf(msg, sizeof msg, "%s", nvfp4a_last_error());
    const char *tag = "nvfp4a_quantize_ex";
    if (strncmp(msg, tag, strlen(tag)) == 0) fail(st, "nvfp4a_quantize%s", msg + strlen(tag));
  }
  return st;
}

extern "C" nvfp4a_status nvfp4a_dequantize(const nvfp4a_tensor *src, int lds, const nvfp4a_tensor *dst, int ldd, int rows, int cols,
                                           cudaStream_t stream) {
  clear_error();
  const char *fn = "nvfp4a_dequantize";
  if (nvfp4a_status st = check_convert(fn, src, lds, dst, ldd, rows, cols)) return st;
  int sld = 0;
  if (nvfp4a_status st = check_scales(fn, "src", src, rows, cols, &sld)) return st;
  if (dst->flags) return fail(NVFP4A_INVALID_VALUE, "%s: flags apply to NVFP4 tensors only (dst)", fn);
  if ((long long)rows * cols == 0) return NVFP4A_OK;
  if (nvfp4a_status st = check_device()) return st;
  const QOut q = make_qout(src, lds, sld);
  const int bpr = cols / 16;
  by_dense(dst->dtype, [&](auto tc) {
    dequant_kernel<decltype(tc)::value><<<grid_for((long long)rows * bpr), 256, 0, stream>>>(q, (uint8_t *)dst->data, ldd, rows, bpr, dst->amax);
  });
  return cuda_fail(cudaGetLastError(), "nvfp4a_dequantize: kernel launch");
}

extern "C" nvfp4a_status nvfp4a_swizzle_scales(const void *src, void *dst, int ld_linear, int rows, int cols, int to_swizzled,
                                               cudaStream_t stream) {
  clear_error();
  const char *fn = "nvfp4a_swizzle_scales";
  if (!src || !dst) return fail(NVFP4A_INVALID_VALUE, "%s: src or dst is NULL", fn);
  if (rows < 0 || cols < 0 || cols % 16) return fail(NVFP4A_INVALID_VALUE, "%s: rows = %d, cols = %d (cols must be a multiple of 16)", fn, rows, cols);
  if (ld_linear < cols / 16) return fail(NVFP4A_INVALID_VALUE, "%s: ld_linear = %d is below cols / 16 = %d", fn, ld_linear, cols / 16);
  if ((long long)rows * cols == 0) return NVFP4A_OK;
  if (nvfp4a_status st = check_device()) return st;
  const int sc = (cols / 16 + 3) / 4 * 4;
  swizzle_kernel<<<grid_for((long long)((rows + 127) / 128 * 128) * sc), 256, 0, stream>>>((const uint8_t *)src, (uint8_t *)dst, ld_linear,
                                                                                          rows, cols / 16, sc, to_swizzled != 0);
  return cuda_fail(cudaGetLastError(), "nvfp4a_swizzle_scales: kernel launch");
}

extern "C" nvfp4a_status nvfp4a_transpose(const nvfp4a_tensor *src, int lds, const nvfp4a_tensor *dst, int ldd, int rows, int cols,
                                          cudaStream_t stream) {
  clear_error();
  const char *fn = "nvfp4a_transpose";
  if (!src || !dst || !src->data || !dst->data || !src->block_scale || !dst->block_scale)
    return fail(NVFP4A_INVALID_VALUE, "%s: a tensor, its data or its block scales are NULL", fn);
  if (src->dtype != NVFP4A_NVFP4 || dst->dtype != NVFP4A_NVFP4) return fail(NVFP4A_INVALID_VALUE, "%s: both tensors must be NVFP4", fn);
  if (rows < 0 || cols < 0 || rows % 16 || cols % 16)
    return fail(NVFP4A_INVALID_VALUE, "%s: rows = %d and cols = %d must be multiples of 16", fn, rows, cols);
  if (lds % 16 || ldd % 16 || lds < cols || ldd < rows)
    return fail(NVFP4A_INVALID_VALUE, "%s: lds = %d (>= cols) and ldd = %d (>= rows) must be multiples of 16", fn, lds, ldd);
  if (((uintptr_t)src->data & 7) || ((uintptr_t)dst->data & 7)) return fail(NVFP4A_INVALID_VALUE, "%s: data must be 8-byte aligned", fn);
  if ((src->flags ^ dst->flags) & NVFP4A_SCALES_UE5M3) return fail(NVFP4A_INVALID_VALUE, "%s: src and dst use different scale types", fn);
  int sls = 0, sld = 0;
  if (nvfp4a_status st = check_scales(fn, "src", src, rows, cols, &sls)) return st;
  if (nvfp4a_status st = check_scales(fn, "dst", dst, cols, rows, &sld)) return st;
  if ((src->flags | dst->flags) & NVFP4A_GLOBAL_PER_ROW) return fail(NVFP4A_INVALID_VALUE, "%s: per-row globals cannot be transposed", fn);
  if ((long long)rows * cols == 0) return NVFP4A_OK;
  if (nvfp4a_status st = check_device()) return st;
  transpose_kernel<<<grid_for((long long)(rows / 16) * (cols / 16)), 256, 0, stream>>>(make_qout(src, lds, sls), make_qout(dst, ldd, sld), rows, cols);
  return cuda_fail(cudaGetLastError(), "nvfp4a_transpose: kernel launch");
}

// ---- self-test of the hardware conversions -------------------------------------------------------------------------------------
// Counts, over FP32 bit patterns [first, first + count), the inputs on which cvt.rn.satfinite.{e2m1x2,e4m3x2}.f32 and the
// software encoders disagree (NaN inputs excluded: outside the quantizer's contract).  out[0]: E2M1 as the low nibble,
// out[1]: E2M1 as the high nibble, out[2]: E4M3, out[3]: the packed BF16 rounding of the GEMM epilogues (NaN included).
__global__ void codec_selftest_kernel(unsigned long long first, unsigned long long count, unsigned long long *out) {
  unsigned long long bad0 = 0, bad1 = 0, bad2 = 0, bad3 = 0;
  for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < count;
       i += (unsigned long long)gridDim.x * blockDim.x) {
    const uint32_t u = (uint32_t)(first + i);
    {
      uint32_t r[32];
#pragma unroll
      for (int q = 0; q < 32; ++q) r[q] = (q & 1) ? u : (u ^ (uint32_t)q * 0x01010101u);
      uint32_t want[32];
#pragma unroll
      for (int q = 0; q < 32; ++q) want[q] = nvb::f32_to_bf16_bits(__uint_as_float(r[q]));
      nvb::round32_to_bf16(r);
      bool bad = false;
#pragma unroll
      for (int q = 0; q < 32; ++q) bad |= r[q] != want[q];
      bad3 += bad;
    }
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) continue;
    const float x = __uint_as_float(u);
    float v[8] = {x, 1.0f, -3.0f, x, 0.f, 0.f, 0.f, 0.f};
    const uint32_t p = nvb::e2m1_pack8(v), want = nvb::f32_to_e2m1_sw(x);
    bad0 += (p & 15u) != want || ((p >> 4) & 15u) != 2u;
    bad1 += ((p >> 12) & 15u) != want || ((p >> 8) & 15u) != 13u;
    bad2 += nvb::e4m3_encode(x) != nvb::f32_to_e4m3_sw(x);
  }
  if (bad0) atomicAdd(out, bad0);
  if (bad1) atomicAdd(out + 1, bad1);
  if (bad2) atomicAdd(out + 2, bad2);
  if (bad3) atomicAdd(out + 3, bad3);
}
extern "C" nvfp4a_status nvfp4a_b200_codec_selftest(unsigned long long first, unsigned long long count, unsigned long long *mismatches,
                                                    cudaStream_t stream) {
  clear_error();
  if (!mismatches) return fail(NVFP4A_INVALID_VALUE, "nvfp4a_b200_codec_selftest: mismatches is NULL");
  if (nvfp4a_status st = check_device()) return st;
  codec_selftest_kernel<<<device_sms() * 8, 256, 0, stream>>>(first, count, mismatches);
  return cuda_fail(cudaGetLastError(), "nvfp4a_b200_codec_selftest: kernel launch");
}
