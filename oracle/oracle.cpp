// CPU oracle for the NVFP4 hot path -- TEST INFRASTRUCTURE ONLY (see oracle.h).  Compile with -ffp-contract=off.
#include "oracle.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

namespace {

const float kFltMax = 3.40282347e38f;

inline uint32_t bits_of(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
inline float float_of(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }

// Runs f(t, nthreads) on nthreads host threads.
void parallel(int nthreads, const std::function<void(int, int)> &f) {
  if (nthreads <= 1) { f(0, 1); return; }
  std::vector<std::thread> pool;
  for (int t = 0; t < nthreads; ++t) pool.emplace_back(f, t, nthreads);
  for (auto &th : pool) th.join();
}

// Generic "round |x| to a small float format": e_min = exponent of the smallest normal, mbits mantissa bits.
// Returns (exponent field, mantissa) of the nearest value, ties to even, computed exactly in double.
struct SmallFloat { int e; int m; };
inline SmallFloat round_small(double a, int e_min, int mbits, int bias) {
  // a > 0 and finite.  Exponent of a, clamped to the subnormal range.
  int ex;
  std::frexp(a, &ex);            // a = f * 2^ex, f in [0.5, 1)
  int e = ex - 1;                // a in [2^e, 2^(e+1))
  if (e < e_min) e = e_min;
  const double ulp = std::ldexp(1.0, e - mbits);
  double q = std::nearbyint(a / ulp);  // default rounding mode: to nearest even; a / ulp is exact (power of two)
  int top = 1 << mbits;
  if (q >= 2.0 * top) { q = top; ++e; }
  if (q < top) return {0, (int)q};          // subnormal (or zero)
  return {e + bias, (int)q - top};
}

}  // namespace

extern "C" {

// ---- decoders (ref tests/test_util.h:27-35, :46-49) -------------------------------------------------------
float orc_e4m3_value(uint32_t code) {
  const int e = (code >> 3) & 15, f = code & 7;
  const float mag = e ? std::ldexp(1.f + f / 8.f, e - 7) : std::ldexp(f / 8.f, -6);
  return (code & 0x80) ? -mag : mag;
}
float orc_ue5m3_value(uint32_t code) {
  const int e = (code >> 3) & 31, f = code & 7;
  return e ? std::ldexp(1.f + f / 8.f, e - 15) : std::ldexp(f / 8.f, -14);
}
float orc_e2m1_value(uint32_t nib) {
  static const float mag[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  return (nib & 8) ? -mag[nib & 7] : mag[nib & 7];
}

// ---- encoders: written from the formats' definitions (nearest value, ties to the even code, saturation), not from
// the reference's bit tricks; equality with ref src/nvfp4effma.cuh:137-210 is checked exhaustively (oracle/ref_codecs.cu).
uint32_t orc_f32_to_e4m3(float x) {
  const uint32_t u = bits_of(x), sign = (u >> 24) & 0x80u;
  if (x != x) return 0x7Fu;
  const double a = std::fabs((double)x);
  if (a >= 448.0) return sign | 0x7Eu;  // satfinite: everything at or beyond the largest finite value
  if (a == 0.0) return sign;
  const SmallFloat r = round_small(a, -6, 3, 7);
  return sign | (uint32_t)(r.e << 3) | (uint32_t)r.m;
}
uint32_t orc_f32_to_ue5m3(float x) {
  const uint32_t u = bits_of(x);
  if (x != x || (u >> 31)) return 0u;   // NaN, negative values and -0
  const double a = (double)x;
  if (a >= 114688.0) return 0xFEu;
  if (a == 0.0) return 0u;
  const SmallFloat r = round_small(a, -14, 3, 15);
  const uint32_t c = (uint32_t)(r.e << 3) | (uint32_t)r.m;
  return c > 0xFEu ? 0xFEu : c;
}
uint32_t orc_f32_to_e2m1(float x) {
  const uint32_t sign = (bits_of(x) >> 28) & 8u;
  if (x != x) return sign | 7u;
  const double a = std::fabs((double)x);
  // midpoints between consecutive code values; a tie goes to the even code
  static const double mid[7] = {0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0};
  uint32_t c = 0;
  while (c < 7 && (a > mid[c] || (a == mid[c] && (c & 1)))) ++c;
  return sign | c;
}
uint32_t orc_f32_to_bf16(float x) {
  const uint32_t u = bits_of(x);
  if (x != x) return 0x7FC0u;
  const uint32_t keep = u >> 16, rest = u & 0xFFFFu;
  const uint32_t up = rest > 0x8000u || (rest == 0x8000u && (keep & 1u));
  return (keep + up) & 0xFFFFu;  // a carry out of the mantissa correctly bumps the exponent (up to Inf)
}
uint32_t orc_f32_to_f16(float x) {
  const _Float16 h = (_Float16)x;  // IEEE round-to-nearest-even conversion
  uint16_t b; memcpy(&b, &h, 2); return b;
}
float orc_bf16_to_f32(uint32_t h) { return float_of((h & 0xFFFFu) << 16); }
float orc_f16_to_f32(uint32_t h) { uint16_t b = (uint16_t)h; _Float16 v; memcpy(&v, &b, 2); return (float)v; }

// ref include/nvfp4effma.h:29-31, tests/test_util.h:38-45
size_t orc_scale_pos(int swizzled, int ld, int cols, int r, int c) {
  if (!swizzled) return (size_t)r * ld + c;
  const int sc = (cols / 16 + 3) / 4 * 4;
  const size_t tile = (size_t)(r / 128) * (sc / 4) + c / 4;
  return tile * 512 + (size_t)(r % 32) * 16 + (size_t)((r / 32) % 4) * 4 + c % 4;
}
size_t orc_scale_bytes(int swizzled, int ld, int rows, int cols) {
  if (!swizzled) return (size_t)rows * ld;
  return (size_t)((rows + 127) / 128 * 128) * (size_t)((cols / 16 + 3) / 4 * 4);
}

static inline uint32_t encode_one(int which, float x) {
  switch (which) {
    case 0: return orc_f32_to_e4m3(x);
    case 1: return orc_f32_to_e2m1(x);
    case 2: return orc_f32_to_ue5m3(x);
    default: return orc_f32_to_bf16(x);
  }
}
// Order-independent fold: sum over u of mix(u) * (code + 1) mod 2^64, so chunks can be summed in any order.
uint64_t orc_encoder_fold(int which, uint64_t first, uint64_t count, int nthreads) {
  std::vector<uint64_t> part(std::max(nthreads, 1), 0);
  parallel(std::max(nthreads, 1), [&](int t, int nt) {
    uint64_t s = 0;
    const uint64_t lo = first + count * t / nt, hi = first + count * (t + 1) / nt;
    for (uint64_t v = lo; v < hi; ++v) {
      const uint32_t u = (uint32_t)v;
      const uint64_t mix = ((uint64_t)u * 0x9E3779B97F4A7C15ull) ^ 0xD1B54A32D192ED03ull;
      s += mix * (uint64_t)(encode_one(which, float_of(u)) + 1u);
    }
    part[t] = s;
  });
  uint64_t s = 0;
  for (uint64_t p : part) s += p;
  return s;
}
void orc_encode_array(int which, const float *x, uint32_t *codes, size_t n) {
  for (size_t i = 0; i < n; ++i) codes[i] = encode_one(which, x[i]);
}

}  // extern "C"

// ---- helpers over orc_tensor -----------------------------------------------------------------------------------
namespace {

struct Fp4View {
  const uint8_t *data; const uint8_t *sc; int ld, ldsc, cols; bool swz, ue; const float *g; bool per_row, amax; float M;
  Fp4View(const orc_tensor *t, int ld_, int cols_) {
    data = (const uint8_t *)t->data; sc = (const uint8_t *)t->block_scale; ld = ld_; cols = cols_;
    swz = t->flags & ORC_SWIZZLED; ue = t->flags & ORC_UE5M3; per_row = t->flags & ORC_PER_ROW; amax = t->flags & ORC_GLOBAL_AMAX;
    ldsc = t->ld_scale ? t->ld_scale : cols_ / 16;
    g = t->global_scale;
    M = t->scale_max ? (float)t->scale_max : ue ? 114688.f : 448.f;
  }
  uint32_t nib(int r, int c) const { return (data[(size_t)r * (ld / 2) + c / 2] >> (4 * (c & 1))) & 15u; }
  uint8_t code(int r, int c) const { return sc[orc_scale_pos(swz, ldsc, cols, r, c / 16)]; }
  float scale(int r, int c) const { return ue ? orc_ue5m3_value(code(r, c)) : orc_e4m3_value(code(r, c)); }
  float val(int r, int c) const { return orc_e2m1_value(nib(r, c)) * scale(r, c); }  // exact product
  float global(int r) const { return g ? g[per_row ? r : 0] : 1.f; }
};

inline float load_dense(int dtype, const void *p, size_t i) {
  switch (dtype) {
    case ORC_BF16: return orc_bf16_to_f32(((const uint16_t *)p)[i]);
    case ORC_FP16: return orc_f16_to_f32(((const uint16_t *)p)[i]);
    default: return ((const float *)p)[i];
  }
}
inline void store_dense(int dtype, void *p, size_t i, float v) {
  switch (dtype) {
    case ORC_BF16: ((uint16_t *)p)[i] = (uint16_t)orc_f32_to_bf16(v); break;
    case ORC_FP16: ((uint16_t *)p)[i] = (uint16_t)orc_f32_to_f16(v); break;
    default: ((float *)p)[i] = v;
  }
}
inline double out_rel(int t) { return t == ORC_BF16 ? 0x1p-8 : t == ORC_FP16 ? 0x1p-11 : 0x1p-24; }
inline double out_abs(int t) { return t == ORC_FP16 ? 0x1p-24 : t == ORC_BF16 ? 0x1p-133 : 0x1p-149; }

inline float scale_value(uint32_t code, bool ue) { return ue ? orc_ue5m3_value(code) : orc_e4m3_value(code); }
inline uint32_t scale_code(float d, bool ue) { return ue ? orc_f32_to_ue5m3(d) : orc_f32_to_e4m3(d); }

// 16 values * inv -> 16 E2M1 nibbles in 8 bytes (even element in the low nibble)
inline void pack16(const float *x, float inv, uint8_t out[8]) {
  for (int e = 0; e < 8; ++e)
    out[e] = (uint8_t)(orc_f32_to_e2m1(x[2 * e] * inv) | (orc_f32_to_e2m1(x[2 * e + 1] * inv) << 4));
}
inline float nib_of(const uint8_t q[8], int e) { return orc_e2m1_value((q[e / 2] >> (4 * (e & 1))) & 15u); }
// 4over6 candidate error, element order (ref tests/test_nvfp4effma.cu:212-219)
inline float fos_error(const float *x, const uint8_t q[8], float sf, float am, float denom, int fos) {
  float err = 0.f;
  for (int e = 0; e < 16; ++e) {
    const float v = ((nib_of(q, e) * sf) * am) / denom, d = v - x[e];
    err = err + (fos == 2 ? d * d : std::fabs(d));
  }
  return err;
}
// shfl_down tree over 16 lanes, lane 0's value (ref tests/test_nvfp4effma.cu:220-227)
inline float tree16(float v[16]) {
  for (int o = 8; o; o >>= 1) {
    float nx[16];
    for (int i = 0; i < 16; ++i) nx[i] = i + o < 16 ? v[i] + v[i + o] : v[i];
    memcpy(v, nx, sizeof nx);
  }
  return v[0];
}

}  // namespace

extern "C" {

int orc_quantize(const float *x, int ldx, int rows, int cols, const orc_tensor *dst, int ldd, int transposed, int tile,
                 int fos, int compute_amax, float *amax_out, int nthreads) {
  if (!x || !dst || !dst->data || !dst->block_scale) return 1;
  if (tile != 1 && tile != 16) return 1;
  const bool swz = dst->flags & ORC_SWIZZLED, ue = dst->flags & ORC_UE5M3, amax_mode = dst->flags & ORC_GLOBAL_AMAX;
  const bool per_row = dst->flags & ORC_PER_ROW;
  const float M = dst->scale_max ? (float)dst->scale_max : ue ? 114688.f : 448.f;
  const int orows = transposed ? cols : rows, ocols = transposed ? (rows + 15) / 16 * 16 : cols;
  const int sld = dst->ld_scale ? dst->ld_scale : ocols / 16;
  uint8_t *qd = (uint8_t *)dst->data, *qs = (uint8_t *)dst->block_scale;
  auto X = [&](int r, int c) -> float {  // element (r, c) of the matrix being quantized, 0 outside the source
    const int sr = transposed ? c : r, sc = transposed ? r : c;
    return sr < rows && sc < cols ? x[(size_t)sr * ldx + sc] : 0.f;
  };
  // statistic and (optionally) the computed globals
  float tam = 0.f;
  std::vector<float> ram(per_row ? rows : 0, 0.f);
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < cols; ++c) {
      const float a = std::fabs(x[(size_t)r * ldx + c]);
      tam = std::max(tam, a);
      if (per_row) ram[r] = std::max(ram[r], a);
    }
  if (amax_out) *amax_out = std::max(*amax_out, tam);
  if (compute_amax) {
    if (!amax_mode || !dst->global_scale) return 1;
    float *g = const_cast<float *>(dst->global_scale);
    if (per_row) for (int r = 0; r < rows; ++r) g[r] = ram[r]; else g[0] = tam;
  }
  auto G = [&](int r) -> float { return dst->global_scale ? dst->global_scale[per_row ? r : 0] : 1.f; };

  const int ocb = (ocols + 15) / 16, tiles = (orows + 15) / 16;
  parallel(std::max(nthreads, 1), [&](int th, int nt) {
    for (int t = th; t < tiles; t += nt)
      for (int c = 0; c < ocb; ++c) {
        float xs[16][16], bmax[16], tmax = 0.f;
        for (int i = 0; i < 16; ++i) {
          bmax[i] = 0.f;
          for (int e = 0; e < 16; ++e) { xs[i][e] = X(16 * t + i, 16 * c + e); bmax[i] = std::max(bmax[i], std::fabs(xs[i][e])); }
          tmax = std::max(tmax, bmax[i]);
        }
        uint32_t code[16], c4[16], c6[16];
        uint8_t q[16][8], q4[16][8], q6[16][8];
        float e4v[16], e6v[16];
        for (int i = 0; i < 16; ++i) {
          const int orow = 16 * t + i;
          const float bm = tile == 16 ? tmax : bmax[i], gv = G(orow < orows ? orow : 0);
          float se, sd;
          if (amax_mode) { se = std::min((M * 6.f) / gv, kFltMax); if (gv == 0.f || se == 0.f) se = 1.f; sd = 1.f / se; }
          else { sd = gv; se = std::min(1.f / gv, kFltMax); }
          if (!fos) {
            code[i] = scale_code(std::min(bm * (se * (1.f / 6.f)), kFltMax), ue);
            pack16(xs[i], std::min(1.f / (scale_value(code[i], ue) * sd), kFltMax), q[i]);
          } else {
            const float base = (bm / 6.f) * se;
            c4[i] = orc_f32_to_e4m3(std::min(base * 1.5f, 448.f));
            c6[i] = orc_f32_to_e4m3(std::min(base, 448.f));
            const float sf4 = orc_e4m3_value(c4[i]), sf6 = orc_e4m3_value(c6[i]);
            pack16(xs[i], std::min(1.f / (sf4 * sd), kFltMax), q4[i]);
            pack16(xs[i], std::min(1.f / (sf6 * sd), kFltMax), q6[i]);
            e4v[i] = fos_error(xs[i], q4[i], sf4, gv, 6.f * M, fos);
            e6v[i] = fos_error(xs[i], q6[i], sf6, gv, 6.f * M, fos);
          }
        }
        if (fos) {
          float t4 = 0.f, t6 = 0.f;
          if (tile == 16) { float a[16], b[16]; memcpy(a, e4v, sizeof a); memcpy(b, e6v, sizeof b); t4 = tree16(a); t6 = tree16(b); }
          for (int i = 0; i < 16; ++i) {
            const bool pick4 = tile == 16 ? t4 < t6 : e4v[i] < e6v[i];  // ties: map-to-6
            code[i] = pick4 ? c4[i] : c6[i];
            memcpy(q[i], pick4 ? q4[i] : q6[i], 8);
          }
        }
        for (int i = 0; i < 16; ++i) {
          const int orow = 16 * t + i;
          if (orow >= orows) continue;
          memcpy(qd + (size_t)orow * (ldd / 2) + 8 * c, q[i], 8);
          qs[orc_scale_pos(swz, sld, ocols, orow, c)] = (uint8_t)code[i];
        }
      }
  });
  return 0;
}

int orc_quantize_int8(const float *x, int ldx, int rows, int cols, int8_t *q, int ldq, float *scales, int ld_scale,
                      float *amax_out, int nthreads) {
  if (!x || !q || !scales || cols % 16) return 1;
  const int lsc = ld_scale ? ld_scale : cols / 16;
  std::vector<float> tmax(std::max(nthreads, 1), 0.f);
  parallel(std::max(nthreads, 1), [&](int th, int nt) {
    float mx = 0.f;
    for (int r = th; r < rows; r += nt)
      for (int b = 0; b < cols / 16; ++b) {
        const float *p = x + (size_t)r * ldx + 16 * b;
        float bmax = 0.f;
        for (int i = 0; i < 16; ++i) bmax = std::max(bmax, std::fabs(p[i]));
        mx = std::max(mx, bmax);
        const float sb = bmax / 127.f;
        for (int i = 0; i < 16; ++i)
          q[(size_t)r * ldq + 16 * b + i] = (int8_t)(sb > 0.f ? std::min(std::max(std::rint(p[i] / sb), -127.f), 127.f) : 0.f);
        scales[(size_t)r * lsc + b] = sb;
      }
    tmax[th] = mx;
  });
  if (amax_out) for (float v : tmax) *amax_out = std::max(*amax_out, v);
  return 0;
}

int orc_dequantize(const orc_tensor *src, int lds, int rows, int cols, int out_dtype, float *y, int ldy, float *amax_out) {
  if (!src || !y) return 1;
  const Fp4View q(src, lds, cols);
  const float finv = 1.0f / (6.f * q.M);
  float am = 0.f;
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < cols; ++c) {
      const float en = orc_e2m1_value(q.nib(r, c)), sb = q.scale(r, c);
      // with an amax global and no storage the factor is 1: amax = 6 M (ref src/quant_nvfp4effma.cuh:250)
      const float gv = q.g ? q.global(r) : (q.amax ? 6.f * q.M : 1.f);
      const float v = q.amax ? en * ((sb * gv) * finv) : (en * sb) * gv;
      am = std::max(am, std::fabs(v));
      uint32_t tmp[1];
      store_dense(out_dtype, tmp, 0, v);
      y[(size_t)r * ldy + c] = load_dense(out_dtype, tmp, 0);
    }
  if (amax_out) *amax_out = std::max(*amax_out, am);
  return 0;
}

int orc_swizzle_scales(const uint8_t *src, uint8_t *dst, int ld_linear, int rows, int cols, int to_swizzled) {
  if (!src || !dst || cols % 16 || ld_linear < cols / 16) return 1;
  if (to_swizzled) memset(dst, 0, orc_scale_bytes(1, 0, rows, cols));
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < cols / 16; ++c) {
      const size_t s = orc_scale_pos(1, 0, cols, r, c), l = (size_t)r * ld_linear + c;
      if (to_swizzled) dst[s] = src[l]; else dst[l] = src[s];
    }
  return 0;
}

int orc_gemm(int m, int n, int k, float alpha, const orc_tensor *A, int lda, const orc_tensor *B, int ldb, float beta,
             const void *C, int c_dtype, int ldc, void *D, int d_dtype, int ldd, const void *bias, int bias_dtype,
             int order, float *amax_out, float *acc_out, double *ref64, double *bound, int nthreads) {
  if (!A || !B || !D || A->dtype != ORC_NVFP4 || k % 16) return 1;
  const bool fp4b = B->dtype == ORC_NVFP4, q8b = B->dtype == ORC_INT8, blk = fp4b || q8b;
  const Fp4View a(A, lda, k);
  const Fp4View bq(B, ldb, k);  // meaningful for NVFP4 B only
  const int8_t *b8 = (const int8_t *)B->data;
  const float *s8 = (const float *)B->block_scale;
  const int lds8 = B->ld_scale ? B->ld_scale : k / 16;
  if (beta != 0.f && !C) { C = D; c_dtype = d_dtype; ldc = ldd; }
  const bool aa = A->flags & ORC_GLOBAL_AMAX, ab = fp4b && (B->flags & ORC_GLOBAL_AMAX);
  const float gf = aa && ab ? 1.0f / (6.f * 6.f * a.M * bq.M) : aa ? 1.0f / (6.f * a.M) : ab ? 1.0f / (6.f * bq.M) : 1.f;
  const float kout = fp4b ? 0.25f : 0.5f;
  const int nt = std::max(nthreads, 1);
  std::vector<float> tmax(nt, 0.f);

  // pre-decode A once: 2 * e2m1 as int8, scale per block, exact value a * sa
  std::vector<int8_t> a2((size_t)m * k);
  std::vector<float> asc((size_t)m * (k / 16)), aval(blk ? 0 : (size_t)m * k);
  for (int i = 0; i < m; ++i) {
    for (int kk = 0; kk < k; ++kk) a2[(size_t)i * k + kk] = (int8_t)(2.f * orc_e2m1_value(a.nib(i, kk)));
    for (int kb = 0; kb < k / 16; ++kb) asc[(size_t)i * (k / 16) + kb] = a.scale(i, 16 * kb);
    if (!blk) for (int kk = 0; kk < k; ++kk) aval[(size_t)i * k + kk] = a.val(i, kk);
  }

  parallel(nt, [&](int th, int nth) {
    std::vector<int8_t> bj(blk ? k : 0);
    std::vector<float> bs(blk ? k / 16 : 0), bv(blk ? 0 : k);
    float mx = 0.f;
    for (int j = th; j < n; j += nth) {
      if (fp4b) {
        for (int kk = 0; kk < k; ++kk) bj[kk] = (int8_t)(2.f * orc_e2m1_value(bq.nib(j, kk)));
        for (int kb = 0; kb < k / 16; ++kb) bs[kb] = bq.scale(j, 16 * kb);
      } else if (q8b) {
        for (int kk = 0; kk < k; ++kk) bj[kk] = b8[(size_t)j * ldb + kk];
        for (int kb = 0; kb < k / 16; ++kb) bs[kb] = s8[(size_t)j * lds8 + kb];
      } else {
        for (int kk = 0; kk < k; ++kk) bv[kk] = load_dense(B->dtype, B->data, (size_t)j * ldb + kk);
      }
      const float gb = fp4b ? bq.global(j) : q8b ? (B->global_scale ? B->global_scale[0] : 1.f) : 1.f;
      for (int i = 0; i < m; ++i) {
        const int8_t *ai = &a2[(size_t)i * k];
        const float *sai = &asc[(size_t)i * (k / 16)];
        auto block = [&](int kb, float acc) {  // exact integer block sum, then acc = fma(p * sa, sb, acc)
          int p = 0;
          for (int e = 0; e < 16; ++e) p += (int)ai[16 * kb + e] * (int)bj[16 * kb + e];
          return std::fmaf((float)p * sai[kb], bs[kb], acc);
        };
        float acc = 0.f;
        if (order == 1) {  // the reference GEMV kernel's lane order (ref tests/test_util.h:262-280)
          float lanes[32];
          for (int l = 0; l < 32; ++l) {
            float p = 0.f;
            for (int kb = l; kb < k / 16; kb += 32) {
              if (blk) p = block(kb, p);
              else for (int e = 0; e < 16; ++e) p = std::fmaf(aval[(size_t)i * k + 16 * kb + e], bv[16 * kb + e], p);
            }
            lanes[l] = p;
          }
          for (int o = 16; o; o >>= 1) {
            float nx[32];
            for (int l = 0; l < 32; ++l) nx[l] = lanes[l] + lanes[l ^ o];
            memcpy(lanes, nx, sizeof nx);
          }
          acc = blk ? lanes[0] * kout : lanes[0];
        } else if (blk) {
          for (int kb = 0; kb < k / 16; ++kb) acc = block(kb, acc);
          acc *= kout;
        } else {
          for (int kk = 0; kk < k; ++kk) acc = std::fmaf(aval[(size_t)i * k + kk], bv[kk], acc);
        }
        if (acc_out) acc_out[(size_t)j * m + i] = acc;
        const float s = ((alpha * a.global(i)) * gb) * gf;
        float v = acc * s;
        const float bi = bias ? load_dense(bias_dtype, bias, i) : 0.f;
        if (bias) v = v + bi;
        const float cv = beta != 0.f ? load_dense(c_dtype, C, (size_t)j * ldc + i) : 0.f;
        if (beta != 0.f) v = std::fmaf(beta, cv, v);
        mx = std::max(mx, std::fabs(v));
        if (ref64 || bound) {  // ref tests/test_util.h:292-302
          double r = 0., ab_ = 0.;
          for (int kk = 0; kk < k; ++kk) {
            const double av = (double)orc_e2m1_value(a.nib(i, kk)) * (double)sai[kk / 16];
            const double bvv = fp4b ? 0.5 * (double)bj[kk] * (double)bs[kk / 16]
                              : q8b ? (double)bj[kk] * (double)bs[kk / 16] : (double)bv[kk];
            const double t = av * bvv;
            r += t; ab_ += std::fabs(t);
          }
          const double sd = s, cb = beta != 0.f ? (double)beta * (double)cv : 0.;
          const double v64 = r * sd + (double)bi + cb;
          if (ref64) ref64[(size_t)j * m + i] = v64;
          if (bound)
            bound[(size_t)j * m + i] = (k + 2) * 0x1p-24 * ab_ * std::fabs(sd) +
                                       4 * 0x1p-24 * (std::fabs(r * sd) + std::fabs((double)bi) + std::fabs(cb)) +
                                       out_rel(d_dtype) * std::fabs(v64) + out_abs(d_dtype);
        }
        store_dense(d_dtype, D, (size_t)j * ldd + i, v);
      }
    }
    tmax[th] = mx;
  });
  if (amax_out) for (float v : tmax) *amax_out = std::max(*amax_out, v);
  return 0;
}

// ref tests/test_epilogue.cu:11-23: lane l adds parts l, l + 32, ... in order, xor butterfly, 1 / sqrt to nearest
float orc_norm_scale(const float *p, int np, float inv_n, float eps) {
  float s[32];
  for (int l = 0; l < 32; ++l) {
    s[l] = 0.f;
    for (int i = l; i < np; i += 32) s[l] = s[l] + p[i];
  }
  for (int o = 16; o; o >>= 1) {
    float t[32];
    for (int l = 0; l < 32; ++l) t[l] = s[l] + s[l ^ o];
    memcpy(s, t, sizeof s);
  }
  return (float)(1.0L / sqrtl((long double)(s[0] * inv_n + eps)));
}

int orc_epilogue_ex(int m, int n, const float *acc, float alpha, const float *ga, int per_row_a, float gb, float gf,
                    float beta, const void *C, int c_dtype, int ldc, const void *bias, int bias_dtype, int mask,
                    const float *norm_parts, int norm_nparts, int norm_ld, float norm_inv_n, float norm_eps, void *D,
                    int d_dtype, int ldd, double *swiglu64, void *d2, int d2_dtype, int ldd2, const void *w2, int w2_dtype,
                    float *sq, int ld_sq, float *v_out) {
  const bool norm = mask & 1, glu = mask & 2, out2 = mask & 4;
  if ((glu || out2) && m % 16) return 1;
  std::vector<float> v(m);
  for (int j = 0; j < n; ++j) {
    const float cs = norm ? orc_norm_scale(norm_parts + (size_t)j * norm_ld, norm_nparts, norm_inv_n, norm_eps) : 1.f;
    for (int i = 0; i < m; ++i) {
      const float av = ga ? ga[per_row_a ? i : 0] : 1.f;
      // ((alpha * vA(i)) * (vB(j) * s_j)) * f  (ref src/nvfp4effma.cuh:352-357)
      const float s = ((alpha * av) * (norm ? gb * cs : gb)) * gf;
      float x = acc[(size_t)j * m + i] * s;
      if (bias) x = x + load_dense(bias_dtype, bias, i);
      if (beta != 0.f) x = std::fmaf(beta, load_dense(c_dtype, C, (size_t)j * ldc + i), x);
      v[i] = x;
      if (v_out) v_out[(size_t)j * m + i] = x;
    }
    if (glu) {
      for (int i = 0; i < m / 2; ++i) {
        const int g = (i / 8) * 16 + i % 8;
        const double h = (double)v[g] / (1. + std::exp(-(double)v[g])) * (double)v[g + 8];
        if (swiglu64) swiglu64[(size_t)j * (m / 2) + i] = h;
        if (D) store_dense(d_dtype, D, (size_t)j * ldd + i, (float)h);
      }
    } else if (D) {
      for (int i = 0; i < m; ++i) store_dense(d_dtype, D, (size_t)j * ldd + i, v[i]);
    }
    if (out2) {
      for (int i = 0; i < m; ++i) store_dense(d2_dtype, d2, (size_t)j * ldd2 + i, v[i] * load_dense(w2_dtype, w2, i));
      for (int s = 0; s < m / 16; ++s) {
        float q = 0.f;
        for (int r = 0; r < 16; ++r) q = q + v[16 * s + r] * v[16 * s + r];
        sq[(size_t)j * ld_sq + s] = q;
      }
    }
  }
  return 0;
}

}  // extern "C"
