// W4A8 GEMM for n > 8: NVFP4 weights x INT8 activations with one FP32 scale per 16 values, on the CUDA cores' DP4A.
//
// Per output and 16-block the kernel forms the exact integer sum p of (2 a) * b, then acc = fma(p * sa, sb, acc) in FP32
// with blocks ascending in k, and a final * 1/2: the arithmetic AND the order of the reference's tiled DP4A kernel
// (src/gemm_nvfp4effma.cuh:345-573 there), so results are bit-identical to the exact definition (include/nvfp4effma.h:78-84).
// Block scales on both operands at a granularity of 16 values do not map onto the K = 32 integer tcgen05.mma, so this path
// stays on DP4A; the integer-to-float conversion rides on the DP4A accumulator (it starts at the bit pattern of 1.5 * 2^23,
// so that the sum, read as a float, is 1.5 * 2^23 + p) and one FMA forms p * sa.
//
// Tile 128 rows x 128 tokens, 64 values of k per step; 256 threads, each 8 x 8 outputs.  Weights are expanded to int8
// (2 * e2m1) while they are staged in shared memory; the next step's global loads are in flight during the current step's
// arithmetic.  The finished tile goes through shared memory to the plain / extended epilogue, one thread per weight row.
#include <atomic>
#include "operands.cuh"

namespace nvb {

namespace {

constexpr int TM = 128, TN = 128, TK = 64;
constexpr int kSmemBytes = TN * (TM + 1) * 4;   // the tile's FP32 values for the epilogue: [token][row], padded

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
// four E2M1 nibbles (the low 16 bits of h) -> four int8 values 2 * e2m1 (bytes in nibble order)
__device__ __forceinline__ uint32_t dec4(uint32_t h) {
  const uint32_t sel = h & 0x7777u;
  const uint32_t pos = prmt(0x03020100u, 0x0C080604u, sel);
  const uint32_t neg = prmt(0xFDFEFF00u, 0xF4F8FAFCu, sel);
  const uint32_t x = ((h << 4) & 0x8080u) | ((h & 0x8080u) << 16);
  const uint32_t mask = prmt(x, 0u, 0xB9A8u);
  return (pos & ~mask) | (neg & mask);
}

// GROUPED (nvfp4a_gemm_grouped with INT8 activations): A stacks `groups` weights of g.m rows, group q owns the tokens
// [seg[q], seg[q + 1]); blockIdx.y counts token tiles over the groups in order, each group's last tile partial.
template <bool GROUPED>
__global__ void __launch_bounds__(256) gemm_dp4a_kernel(GemmArgs g, const int *__restrict__ seg, int groups) {
  extern __shared__ __align__(16) uint8_t dyn[];
  __shared__ __align__(16) uint32_t a_s[TM][TK / 4 + 1];   // int8 x 4 per word, one padding word per row
  __shared__ __align__(16) uint32_t b_s[TN][TK / 4 + 1];
  __shared__ float sa_s[TK / 16][TM], sb_s[TK / 16][TN];
  __shared__ float colscale[TN];
  float *vt = (float *)dyn;                                   // [TN][TM + 1]

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;  // outputs: rows 8 ty .., tokens 8 tx ..
  int j0 = blockIdx.y * TN, ro = 0;   // ro: first row of this group's weight in the stacked A (and in its per-row globals, bias)
  if (GROUPED) {
    int t = blockIdx.y, q = 0, lo = 0, hi = 0;
    for (; q < groups; ++q) {
      lo = seg[q]; hi = seg[q + 1];
      const int tiles = (hi - lo + TN - 1) / TN;
      if (t < tiles) break;
      t -= tiles;
    }
    if (q == groups || hi > g.n) return;   // past the last group's tiles (the grid is sized for the worst case), or seg beyond `rows`
    j0 = lo + t * TN;
    g.n = hi;
    ro = q * g.m;
  }
  const int gm = g.m, gn = g.n, gk = g.k;
  const int i0 = blockIdx.x * TM;
  const bool ue_a = g.A.ue != 0;
  const int8_t *const bdata = (const int8_t *)g.B.data;
  const int ldb = g.B.ld, lds8 = g.B.lds8;
  const float *const bs8 = g.B.s8;

  if (g.x.mask & kExNorm) {
    const int w = tid >> 5, lane = tid & 31;
    for (int c = w; c < TN; c += 8) {
      const float s = warp_norm_scale(g.x, min(j0 + c, gn - 1), lane);
      if (lane == 0) colscale[c] = s;
    }
  }

  // staging assignment: thread t stages 32 values (two blocks) of A row t / 2 and of B token t / 2, half t % 2 of the k step
  const int sr = tid >> 1, sh = tid & 1;
  const int arow = ro + min(i0 + sr, gm - 1), bcol = min(j0 + sr, gn - 1);
  uint4 aw, bw0, bw1;
  float asc0, asc1, bsc0, bsc1;
  auto fetch = [&](int k0) {
    const int kb = (k0 >> 4) + 2 * sh;
    const uint2 w0 = g.A.block(arow, kb), w1 = g.A.block(arow, kb + 1);
    aw = make_uint4(w0.x, w0.y, w1.x, w1.y);
    asc0 = scale_to_f32(g.A.scale_code(arow, kb), ue_a);
    asc1 = scale_to_f32(g.A.scale_code(arow, kb + 1), ue_a);
    const uint4 *bp = (const uint4 *)(bdata + (size_t)bcol * ldb + k0 + 32 * sh);
    bw0 = __ldg(bp); bw1 = __ldg(bp + 1);
    bsc0 = bs8[(size_t)bcol * lds8 + kb]; bsc1 = bs8[(size_t)bcol * lds8 + kb + 1];
  };

  float acc[8][8];
#pragma unroll
  for (int r = 0; r < 8; ++r)
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[r][c] = 0.f;

  fetch(0);
  for (int k0 = 0; k0 < gk; k0 += TK) {
    __syncthreads();   // the previous step's arithmetic is done with the staging buffers
    {
      uint32_t *ad = &a_s[sr][8 * sh];
      const uint32_t wv[4] = {aw.x, aw.y, aw.z, aw.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) { ad[2 * q] = dec4(wv[q]); ad[2 * q + 1] = dec4(wv[q] >> 16); }
      uint32_t *bd = &b_s[sr][8 * sh];
      bd[0] = bw0.x; bd[1] = bw0.y; bd[2] = bw0.z; bd[3] = bw0.w; bd[4] = bw1.x; bd[5] = bw1.y; bd[6] = bw1.z; bd[7] = bw1.w;
      sa_s[2 * sh][sr] = asc0; sa_s[2 * sh + 1][sr] = asc1;
      sb_s[2 * sh][sr] = bsc0; sb_s[2 * sh + 1][sr] = bsc1;
    }
    __syncthreads();
    if (k0 + TK < gk) fetch(k0 + TK);   // in flight during the arithmetic below
#pragma unroll
    for (int blk = 0; blk < TK / 16; ++blk) {
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {   // four tokens at a time keeps the register count at two CTAs per SM
        uint32_t bq[4][4];
        float sb[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int q = 0; q < 4; ++q) bq[c][q] = b_s[8 * tx + 4 * ch + c][4 * blk + q];
          sb[c] = sb_s[blk][8 * tx + 4 * ch + c];
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          uint32_t aq[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) aq[q] = a_s[8 * ty + r][4 * blk + q];
          const float sa = sa_s[blk][8 * ty + r];
          const float bias_term = __fmul_rn(-12582912.f, sa);   // exact: a power-of-two multiple of sa's 4 significant bits
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            int p = 0x4B400000;   // 1.5 * 2^23 as a float: the integer sum rides in its mantissa
#pragma unroll
            for (int q = 0; q < 4; ++q) p = __dp4a((int)aq[q], (int)bq[c][q], p);
            const float psa = __fmaf_rn(__int_as_float(p), sa, bias_term);   // = p * sa, rounded once
            acc[r][4 * ch + c] = __fmaf_rn(psa, sb[c], acc[r][4 * ch + c]);
          }
        }
      }
    }
  }

  // ---- the tile's values to shared memory, then the epilogue: thread t owns row t % 128 and the tokens of parity t / 128 ----
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 8; ++r)
#pragma unroll
    for (int c = 0; c < 8; ++c) vt[(8 * tx + c) * (TM + 1) + 8 * ty + r] = __fmul_rn(acc[r][c], 0.5f);
  __syncthreads();
  const Epilogue &e = g.e;
  const int ri = tid & 127, i = i0 + ri;
  const bool row_ok = i < gm;
  const int mask = g.x.mask;
  const float rowp = row_ok ? epi_row_part(e, ro + i) : 0.f;
  float amax = 0.f;
  // pass 1: v = epilogue value (before the output rounding), written back for the neighbours' use
  for (int c = tid >> 7; c < TN; c += 2) {
    const int j = j0 + c;
    float v = 0.f;
    if (row_ok && j < gn) {
      float colp = epi_col_part(e, j);
      if (mask & kExNorm) colp = __fmul_rn(colp, colscale[c]);
      if (GROUPED) {   // bias is stacked like A, C like D
        v = __fmul_rn(vt[c * (TM + 1) + ri], epi_scale(e, rowp, colp));
        if (e.bias) v = __fadd_rn(v, load_dense(e.bias_dtype, e.bias, ro + i));
        if (e.beta != 0.f) v = __fmaf_rn(e.beta, load_dense(e.c_dtype, e.c, (size_t)j * e.ldc + i), v);
      } else {
        v = epi_value(e, i, j, vt[c * (TM + 1) + ri], epi_scale(e, rowp, colp));
      }
    }
    vt[c * (TM + 1) + ri] = v;
  }
  __syncthreads();
  for (int c = tid >> 7; c < TN; c += 2) {
    const int j = j0 + c;
    if (!(row_ok && j < gn)) continue;
    const float v = vt[c * (TM + 1) + ri];
    if (mask & kExSwiglu) {
      if (!(ri & 8)) {
        const float h = silu_mul(v, vt[c * (TM + 1) + ri + 8]);
        store_dense(e.d_dtype, e.d, (size_t)j * e.ldd + (i >> 4) * 8 + (i & 7), h);
        amax = fmaxf(amax, fabsf(h));
      }
    } else {
      store_dense(e.d_dtype, e.d, (size_t)j * e.ldd + i, v);
      amax = fmaxf(amax, fabsf(v));
    }
    if (mask & kExOut2) {
      store_dense(g.x.d2_dtype, g.x.d2, (size_t)j * g.x.ldd2 + i, __fmul_rn(v, load_dense(g.x.w2_dtype, g.x.w2, i)));
      if (!(ri & 15)) {
        float sq = 0.f;
#pragma unroll
        for (int r = 0; r < 16; ++r) { const float u = vt[c * (TM + 1) + ri + r]; sq = __fadd_rn(sq, __fmul_rn(u, u)); }
        g.x.sq[(size_t)j * g.x.ld_sq + (i >> 4)] = sq;
      }
    }
  }
  if (e.amax) warp_amax_commit(e.amax, amax);
}

}  // namespace

bool gemm_dp4a_supports(const GemmArgs &g) {
  return g.B.dtype == NVFP4A_INT8 && g.k >= 64 && ((uintptr_t)g.B.data & 15) == 0 && g.B.ld % 16 == 0;
}

static cudaError_t dp4a_prepare() {
  static std::atomic<bool> attr_set[64];   // zero-initialised; set once per device (a repeated cudaFuncSetAttribute is harmless)
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_dp4a_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_dp4a_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set[dev & 63] = true;
  }
  return cudaSuccess;
}

cudaError_t launch_gemm_dp4a(const GemmArgs &g, cudaStream_t s) {
  const cudaError_t e = dp4a_prepare();
  if (e != cudaSuccess) return e;
  const dim3 grid((g.m + TM - 1) / TM, (g.n + TN - 1) / TN);
  gemm_dp4a_kernel<false><<<grid, 256, kSmemBytes, s>>>(g, nullptr, 0);
  return cudaGetLastError();
}

// g.m = rows of ONE group's weight, g.n = the bound `rows` on seg[groups]; every group may end in a partial tile
cudaError_t launch_gemm_dp4a_grouped(const GemmArgs &g, const int *seg, int groups, cudaStream_t s) {
  const cudaError_t e = dp4a_prepare();
  if (e != cudaSuccess) return e;
  const dim3 grid((g.m + TM - 1) / TM, (g.n + TN - 1) / TN + groups);
  if (grid.y > 65535) return cudaErrorInvalidConfiguration;
  gemm_dp4a_kernel<true><<<grid, 256, kSmemBytes, s>>>(g, seg, groups);
  return cudaGetLastError();
}

}  // namespace nvb
