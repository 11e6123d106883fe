// Decode GEMV for block-scaled activations: D[m x n] = A[m x k] (NVFP4) * B[n x k]^T with 1 <= n <= 8 and B either INT8 with one
// FP32 scale per 16 values (W4A8) or NVFP4 (W4A4).  Per output and 16-block the kernel forms the EXACT integer sum of
// (2 a) * b (DP4A on weights expanded to 2 * e2m1, activations as int8 / 2 * e2m1), then acc = fma(p * sa, sb, acc) in FP32
// and a final * 1/2 (INT8) or * 1/4 (NVFP4) -- the arithmetic of the reference's blocked GEMV
// (src/gemv_nvfp4effma.cuh:26-234 there); the order of the FP32 additions over k is this kernel's own, so results agree
// with the exact definition within the FP32 accumulation bound.
//
// One CTA owns 32 (or, for matrices of few rows, 16) consecutive rows; the activations (int8, n x k bytes) and their block scales (FP32) are staged once per
// CTA in shared memory.  A warp takes a row at a time: lane l reads the 16-byte weight chunks l, l + 32, ... of the row
// (two blocks each), so a warp load covers 512 contiguous bytes; the n <= 8 dot products of a chunk reuse its decoded
// weights.  The lanes' sums are added by an xor butterfly; the CTA's 32 x n results then run the plain or extended epilogue.
#include <atomic>
#include "operands.cuh"

namespace nvb {

namespace {

constexpr int kWarps = 8, kMaxN = 8;   // a CTA owns kWarps * R rows: R = 4 rows per warp, or 2 when the matrix has few rows
constexpr int kSmemLimit = 200 * 1024;

struct GemvQArgs {
  int m, n, k;
  Fp4Operand A;
  BOperand B;
  Epilogue e;
  EpilogueEx ex;
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
// four E2M1 nibbles (the low 16 bits of h) -> four int8 values 2 * e2m1 (bytes in nibble order)
__device__ __forceinline__ uint32_t dec4(uint32_t h) {
  const uint32_t sel = h & 0x7777u;
  const uint32_t pos = prmt(0x03020100u, 0x0C080604u, sel);           // 0 1 2 3 | 4 6 8 12
  const uint32_t neg = prmt(0xFDFEFF00u, 0xF4F8FAFCu, sel);           // 0 -1 -2 -3 | -4 -6 -8 -12
  // sign bits (3, 7, 11, 15) -> byte masks: nibbles 1, 3 have theirs at the top of bytes 0, 1; nibbles 0, 2 after << 4
  const uint32_t x = ((h << 4) & 0x8080u) | ((h & 0x8080u) << 16);
  const uint32_t mask = prmt(x, 0u, 0xB9A8u);                         // replicate the top bit of bytes 0, 2, 1, 3
  return (pos & ~mask) | (neg & mask);
}
__device__ __forceinline__ int dp4a(uint32_t a, uint32_t b, int c) { return __dp4a((int)a, (int)b, c); }

template <int R>
__global__ void __launch_bounds__(kWarps * 32) gemv_blocked_kernel(const GemvQArgs g) {
  constexpr int kRows = kWarps * R;
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ float vtile[kMaxN][32];
  __shared__ float colscale[kMaxN];
  const int gm = g.m, gn = g.n, gk = g.k, nb = gk >> 4;
  int8_t *xq = (int8_t *)smem;                       // [n][k]
  float *xs = (float *)(smem + (size_t)gn * gk);     // [n][k / 16]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool fp4b = g.B.dtype == NVFP4A_NVFP4;
  const bool ue_a = g.A.ue != 0;

  // ---- stage the activations: int8 values and FP32 block scales ----
  if (fp4b) {
    for (int idx = tid; idx < gn * nb; idx += blockDim.x) {
      const int j = idx / nb, kb = idx - j * nb;
      const uint2 w = g.B.q.block(j, kb);
      *(uint4 *)(xq + (size_t)j * gk + 16 * kb) = make_uint4(dec4(w.x), dec4(w.x >> 16), dec4(w.y), dec4(w.y >> 16));
      xs[idx] = g.B.q.scale(j, kb);
    }
  } else {
    for (int idx = tid; idx < gn * nb; idx += blockDim.x) {
      const int j = idx / nb, kb = idx - j * nb;
      *(uint4 *)(xq + (size_t)j * gk + 16 * kb) = __ldg((const uint4 *)((const int8_t *)g.B.data + (size_t)j * g.B.ld + 16 * kb));
      xs[idx] = g.B.s8[(size_t)j * g.B.lds8 + kb];
    }
  }
  if ((g.ex.mask & kExNorm) && warp < gn) {
    const float s = warp_norm_scale(g.ex, warp, lane);
    if (lane == 0) colscale[warp] = s;
  }
  __syncthreads();

  // ---- rows: warp w takes rows w, w + 8, w + 16, w + 24 of the CTA's 32, all four at once so that their loads fly together ----
  const int i0 = blockIdx.x * kRows;
  const int nchunks = gk >> 5;   // 32 values = 16 bytes = two blocks
  const ScalePos sp{g.A.sld};
  const bool img = g.A.image;
  const uint8_t *const adata = g.A.data, *const asc = g.A.sc;
  const int ald2 = g.A.ld >> 1, aktiles = g.A.ktiles;
  auto load_chunk = [&](int row, int c, uint4 &w, uint32_t &sc) {   // 32 nibbles and the two scale codes of chunk c of a row
    if (img) {
      const uint8_t *tile = adata + ((size_t)(row >> 7) * aktiles + (c >> 3)) * kImgTileBytes;
      const int rr = row & 127, cc = c & 7;
      w = __ldg((const uint4 *)(tile + rr * 128 + cc * 16));
      sc = __ldg((const uint16_t *)(tile + kImgDataBytes + (cc >> 1) * 512 + (rr & 31) * 16 + (rr >> 5) * 4 + (cc & 1) * 2));
    } else {
      w = __ldg((const uint4 *)(adata + (size_t)row * ald2 + (size_t)c * 16));
      sc = __ldg((const uint16_t *)(asc + sp.at(row, 2 * c)));
    }
  };
  float acc[R][kMaxN];
#pragma unroll
  for (int q = 0; q < R; ++q)
#pragma unroll
    for (int j = 0; j < kMaxN; ++j) acc[q][j] = 0.f;
  int rows4[R];
#pragma unroll
  for (int q = 0; q < R; ++q) rows4[q] = min(i0 + warp + kWarps * q, gm - 1);
  for (int c = lane; c < nchunks; c += 32) {
    uint4 w[R];
    uint32_t sc[R];
#pragma unroll
    for (int q = 0; q < R; ++q) load_chunk(rows4[q], c, w[q], sc[q]);
    // decode the four rows' chunks once, then walk the activation vectors: a vector's 32 values and two scales are read from
    // shared memory once per chunk and serve all four rows (read per row, shared memory set the pace: 16 bytes of it per weight byte)
    float sa[R][2];
    uint32_t a0[R][4], a1[R][4];
#pragma unroll
    for (int q = 0; q < R; ++q) {
      sa[q][0] = scale_to_f32(sc[q] & 0xFFu, ue_a); sa[q][1] = scale_to_f32(sc[q] >> 8, ue_a);
      a0[q][0] = dec4(w[q].x); a0[q][1] = dec4(w[q].x >> 16); a0[q][2] = dec4(w[q].y); a0[q][3] = dec4(w[q].y >> 16);
      a1[q][0] = dec4(w[q].z); a1[q][1] = dec4(w[q].z >> 16); a1[q][2] = dec4(w[q].w); a1[q][3] = dec4(w[q].w >> 16);
    }
#pragma unroll
    for (int j = 0; j < kMaxN; ++j) {
      if (j >= gn) break;
      const uint4 x0 = *(const uint4 *)(xq + (size_t)j * gk + 32 * c), x1 = *(const uint4 *)(xq + (size_t)j * gk + 32 * c + 16);
      const float xs0 = xs[j * nb + 2 * c], xs1 = xs[j * nb + 2 * c + 1];
#pragma unroll
      for (int q = 0; q < R; ++q) {
        const int p0 = dp4a(a0[q][3], x0.w, dp4a(a0[q][2], x0.z, dp4a(a0[q][1], x0.y, dp4a(a0[q][0], x0.x, 0))));
        const int p1 = dp4a(a1[q][3], x1.w, dp4a(a1[q][2], x1.z, dp4a(a1[q][1], x1.y, dp4a(a1[q][0], x1.x, 0))));
        acc[q][j] = __fmaf_rn(__fmul_rn((float)p0, sa[q][0]), xs0, acc[q][j]);
        acc[q][j] = __fmaf_rn(__fmul_rn((float)p1, sa[q][1]), xs1, acc[q][j]);
      }
    }
  }
#pragma unroll
  for (int q = 0; q < R; ++q)
#pragma unroll
    for (int j = 0; j < kMaxN; ++j) {
      float a = acc[q][j];
#pragma unroll
      for (int o = 16; o; o >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
      if (lane == 0 && j < gn) vtile[j][warp + kWarps * q] = __fmul_rn(a, fp4b ? 0.25f : 0.5f);
    }
  __syncthreads();

  // ---- epilogue: thread t owns (row t % 32, column t / 32) ----
  const Epilogue &e = g.e;
  const int ri = tid & 31, cj = tid >> 5, i = i0 + ri;
  const bool live = ri < kRows && i < gm && cj < gn;
  float v = 0.f, amax = 0.f;
  if (live) {
    float colp = epi_col_part(e, cj);
    if (g.ex.mask & kExNorm) colp = __fmul_rn(colp, colscale[cj]);
    v = epi_value(e, i, cj, vtile[cj][ri], epi_scale(e, epi_row_part(e, i), colp));
  }
  if (!(g.ex.mask & (kExSwiglu | kExOut2))) {
    if (live) { store_dense(e.d_dtype, e.d, (size_t)cj * e.ldd + i, v); amax = fabsf(v); }
  } else {
    __syncthreads();
    if (cj < kMaxN) vtile[cj][ri] = v;
    __syncthreads();
    if (g.ex.mask & kExSwiglu) {
      if (live && !(ri & 8)) {
        const float h = silu_mul(v, vtile[cj][ri + 8]);
        store_dense(e.d_dtype, e.d, (size_t)cj * e.ldd + (i >> 4) * 8 + (i & 7), h);
        amax = fabsf(h);
      }
    } else if (live) {
      store_dense(e.d_dtype, e.d, (size_t)cj * e.ldd + i, v);
      amax = fabsf(v);
    }
    if (g.ex.mask & kExOut2) {
      if (live) store_dense(g.ex.d2_dtype, g.ex.d2, (size_t)cj * g.ex.ldd2 + i, __fmul_rn(v, load_dense(g.ex.w2_dtype, g.ex.w2, i)));
      if (live && !(ri & 15)) {
        float sq = 0.f;
#pragma unroll
        for (int r = 0; r < 16; ++r) sq = __fadd_rn(sq, __fmul_rn(vtile[cj][ri + r], vtile[cj][ri + r]));
        g.ex.sq[(size_t)cj * g.ex.ld_sq + (i >> 4)] = sq;
      }
    }
  }
  if (e.amax) warp_amax_commit(e.amax, amax);
}

size_t smem_bytes(const GemmArgs &g) { return (size_t)g.n * g.k + (size_t)g.n * (g.k / 16) * sizeof(float); }

}  // namespace

bool gemv_blocked_supports(const GemmArgs &g) {
  if (!(g.n >= 1 && g.n <= kMaxN && g.k >= 64 && (g.B.dtype == NVFP4A_INT8 || g.B.dtype == NVFP4A_NVFP4))) return false;
  if (g.B.dtype == NVFP4A_NVFP4 && g.B.q.image) return false;
  if (g.B.dtype == NVFP4A_INT8 && (((uintptr_t)g.B.data & 15) || g.B.ld % 16)) return false;
  return smem_bytes(g) <= (size_t)kSmemLimit;
}

cudaError_t launch_gemv_blocked(const GemmArgs &g, cudaStream_t s) {
  GemvQArgs a;
  a.m = g.m; a.n = g.n; a.k = g.k;
  a.A = g.A; a.B = g.B; a.e = g.e; a.ex = g.x;
  static std::atomic<bool> attr_set[64];   // zero-initialised; set once per device (a repeated cudaFuncSetAttribute is harmless)
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_blocked_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_blocked_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e != cudaSuccess) return e;
    attr_set[dev & 63] = true;
  }
  // 32 rows per CTA give every SM a CTA from about 4700 rows up; below that, 16 rows per CTA put twice as many warps on the
  // SMs (4096 x 4096, 8 vectors: 17.2 -> 14.1 us; at 8192 rows the doubled staging of the activations costs more than it brings).
  // A row's sum does not depend on the choice: a warp walks its rows' chunks in the same order either way.
  if ((g.m + 31) / 32 >= device_sms()) gemv_blocked_kernel<4><<<(g.m + 31) / 32, kWarps * 32, smem_bytes(g), s>>>(a);
  else gemv_blocked_kernel<2><<<(g.m + 15) / 16, kWarps * 32, smem_bytes(g), s>>>(a);
  return cudaGetLastError();
}

}  // namespace nvb
