// NVFP4 weights x BF16 activations (W4A16) GEMM on the 5th-generation tensor cores: tcgen05.mma kind::f16 (BF16 in, FP32
// accumulators in tensor memory) on weights expanded to exact BF16 in shared memory.
//
// An NVFP4 value times its block scale has at most 2 + 4 significant bits, so e2m1 * scale is exact in BF16; the tensor
// cores then form exact products with the BF16 activations and accumulate in FP32 -- the reference's "exact" W4A16
// definition (include/nvfp4effma.h:82-92 there) up to the order of the FP32 additions, like its own tensor-core path.
//
// Tile: 128 weight rows (MMA M) x BN tokens (MMA N) x 64 values of k per stage; a stage in shared memory is
// [A 128 rows x 128 B | B BN rows x 128 B], both K-major with the 128-byte swizzle.
//   warp 0      TMA producer of the activation tiles (2-D tensor map over B, no multicast)
//   warp 1      MMA issuer (4 x K16 per stage), owner of the tensor memory: 2 accumulators of BN columns
//   warps 2-5   epilogue, one 32-lane quadrant each: plain or extended (RMSNorm column scale, SwiGLU, second output + sums
//               of squares), D through a shared-memory staging tile and TMA stores when its layout allows
//   warps 6-13  weight expansion, two groups of four warps on alternate stages: each thread owns a row of its stage (64
//               nibbles + 4 scale bytes, fetched from global memory ahead of use), decodes them with shifts and masks to BF16 pairs (value * 2^-126, the
//               subnormal trick), multiplies by the block scale in BF16 (exact) and stores 64 bytes into the swizzled
//               A tile.  To keep scale * 2^126 inside BF16, weights are carried as a * sa * 2^-Z (Z = 8 for E4M3, 16 for
//               UE5M3 scales) and the accumulator is multiplied by 2^Z in the epilogue.
// Every wait is bounded; a wait that gives up raises the CTA's abort flag and the kernel status word.
//
// INT8 activations (W4A8, FP32 scale per 16 values) run on the same kernel with PLANES = 3: an activation is the FP32 value
// x = q * s_b (one rounding: within the accumulation bound of the exact definition, not bit-identical to the integer block sums
// of the DP4A kernels), split exactly into three BF16 terms x = t1 + t2 + t3 (8 + 8 + 8 significant bits) by a small kernel
// that runs first.  The terms lie side by side as [token][3][k]; a stage then holds one expanded weight tile and the three
// activation tiles of its 64 values of k, and the MMA issuer accumulates weight x t1, weight x t2, weight x t3 into the same
// accumulator -- three times the tensor-core work per expanded weight tile, which is what this kernel otherwise lacks.
#include <atomic>
#include <cuda_bf16.h>
#include "operands.cuh"
#include "sm100.cuh"

namespace nvb {

using namespace sm100;

namespace {

struct W4A16Args {
  int m, n, k;
  Fp4Operand A;
  Epilogue e;
  EpilogueEx x;
  unsigned *status;
  unsigned tag;  // this launch's tag in the status word
  int d_tma;     // the output goes through the staging tile and TMA stores (SwiGLU: 64 output rows per tile)
};

// tensor maps of D in the peers' buffers (tensor-parallel all-gather fused into the epilogue's TMA stores); n = 0: none
struct alignas(64) PeerMaps {
  CUtensorMap map[kMaxRanks - 1];
  int n;
};

template <int BN, int PLANES = 1>
struct Cfg {
  static constexpr int kStages = PLANES == 3 ? 3 : BN == 256 ? 4 : 6;
  static constexpr int kABytes = 128 * 128, kPlaneBytes = BN * 128, kBBytes = PLANES * kPlaneBytes, kStageBytes = kABytes + kBBytes;
  static constexpr int kStagingBytes = 8192;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kStagingBytes + 1024 /* scale table */ + BN * 4 /* column scales */ + 256;
};

constexpr int kThreads = 448, kConvWarps = 8;
constexpr unsigned kStWaitFullA = 0x301, kStWaitFullB = 0x302, kStWaitEmpty = 0x303, kStWaitTmemFull = 0x304, kStWaitTmemEmpty = 0x305,
                   kStWaitConv = 0x306;

__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
// nibbles p and p + 4 of w -> BF16 pair (low half: nibble p), each value * 2^-126: magnitude bits to [6, 9), sign to 15
template <int P>
__device__ __forceinline__ uint32_t decode_pair(uint32_t w) {
  const uint32_t mag = (P < 2 ? w << (6 - 4 * P) : w >> (4 * P - 6)) & 0x01C001C0u;
  const uint32_t sgn = (w << (12 - 4 * P)) & 0x80008000u;
  return mag | sgn;
}

// four MMAs of K = 16 over one 128-byte-row stage without a commit (elected lane of a converged warp): the first and second
// activation plane of a stage; the third goes through mma4_f16_commit_elect
__device__ __forceinline__ void mma4_f16_elect(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p, q, t;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.eq.u32 t, %3, %3;\n\telect.sync _|q, 0xFFFFFFFF;\n\t"
               "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
               "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %5, %6, %3, t;\n\t"
               "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %7, %8, %3, t;\n\t"
               "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %9, %10, %3, t;\n\t}"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "l"(a_desc + 2), "l"(b_desc + 2), "l"(a_desc + 4), "l"(b_desc + 4),
                 "l"(a_desc + 6), "l"(b_desc + 6) : "memory");
}

// what a conversion thread fetches for one stage: the 64 nibbles and 4 scale bytes of its row
struct RawRow {
  uint4 w0, w1;
  uint32_t sc;
};

template <int BN, int PLANES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_w4a16_kernel(const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_d, const __grid_constant__ PeerMaps peers,
                  const W4A16Args g) {
  using C = Cfg<BN, PLANES>;
  constexpr int kStages = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *staging = smem + kStages * C::kStageBytes;
  uint32_t *lut = (uint32_t *)(staging + C::kStagingBytes);      // scale code -> BF16 pair (sa * 2^(126 - Z), twice)
  float *colscale = (float *)(lut + 256);                           // RMSNorm column scales of the current token tile
  uint64_t *bars = (uint64_t *)(colscale + BN);
  uint64_t *full = bars, *empty = bars + kStages, *tmem_full = bars + 2 * kStages, *tmem_empty = tmem_full + 2;
  uint32_t *tmem_slot = (uint32_t *)(tmem_empty + 2);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gm = g.m, gn = g.n, gk = g.k;
  const int tiles_m = (gm + 127) / 128, tiles_n = (gn + BN - 1) / BN, ntiles = tiles_m * tiles_n;
  const int nk = gk / 64;
  const bool ue = g.A.ue != 0;
  unsigned *const status_word = g.status;

  if (threadIdx.x == 0) {
    // one `full` barrier per stage: the four conversion warps of the stage's group and the producer's expect-tx arrival
    for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], kConvWarps / 2 + 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 4); }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_b);
  }
  if (threadIdx.x < 256) {
    const float s = scale_to_f32((uint32_t)threadIdx.x, ue) * (ue ? 0x1p110f : 0x1p118f);  // exact: 4 significant bits
    const uint32_t h = __float_as_uint(s) >> 16;
    lut[threadIdx.x] = h | (h << 16);
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const unsigned tag = g.tag;
  auto wait = [abort_flag, status_word, tag](uint64_t *bar, uint32_t parity, unsigned code) -> bool {
    if (mbar_try(bar, parity)) return true;   // the common case: no flag read, no clock read
    if (*abort_flag) return false;
    if (mbar_wait(bar, parity)) return true;
    *abort_flag = 1;
    atomicCAS(status_word, 0u, code | tag);
    return false;
  };

  if (warp == 0) {
    // ---------------- producer: activation tiles ----------------
    // (the whole warp runs the loop, one elected lane issues: see tma_load_2d_elect)
    uint32_t it = 0;
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
      const int tn = t / tiles_m;
      for (int ks = 0; ks < nk; ++ks, ++it) {
        const int s = it % kStages;
        if (!__all_sync(0xFFFFFFFFu, wait(&empty[s], ((it / kStages) & 1) ^ 1, kStWaitEmpty))) goto done;
        mbar_arrive_expect_tx_elect(&full[s], C::kBBytes);
#pragma unroll
        for (int p = 0; p < PLANES; ++p)   // plane p of a token's row starts 2 k bytes after plane p - 1
          tma_load_2d_elect(smem_u32(smem + (size_t)s * C::kStageBytes + C::kABytes + p * C::kPlaneBytes), &tmap_b, p * 2 * gk + ks * 128, tn * BN,
                            smem_u32(&full[s]));
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // The whole warp runs the loop and one elected lane issues a stage's four MMAs (K = 16 each: 32 bytes along the row) and the
    // commit in one statement; from inside a one-lane branch every tcgen05.mma costs ~150 cycles, more than the 128 the tensor
    // pipe needs for 128 x 256 x 16.
    constexpr uint32_t idesc = idesc_f16(128, BN, 1);
    const uint64_t da0 = smem_desc_sw128(smem_u32(smem));
    uint32_t it = 0, tile_i = 0;
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++tile_i) {
      const int acc = tile_i & 1;
      if (!__all_sync(0xFFFFFFFFu, wait(&tmem_empty[acc], ((tile_i >> 1) & 1) ^ 1, kStWaitTmemEmpty))) goto done;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int ks = 0; ks < nk; ++ks, ++it) {
        const int s = it % kStages;
        if (!__all_sync(0xFFFFFFFFu, wait(&full[s], (it / kStages) & 1, kStWaitFullA))) goto done;
        tc_fence_after();
        const uint64_t da = da0 + (uint32_t)s * (uint32_t)(C::kStageBytes >> 4), db = da + (C::kABytes >> 4);
        if (PLANES == 3) {
          mma4_f16_elect(d_tmem, da, db, idesc, (uint32_t)(ks != 0));
          mma4_f16_elect(d_tmem, da, db + (C::kPlaneBytes >> 4), idesc, 1u);
          mma4_f16_commit_elect(d_tmem, da, db + 2 * (C::kPlaneBytes >> 4), idesc, 1u, &empty[s]);
        } else {
          mma4_f16_commit_elect(d_tmem, da, db, idesc, (uint32_t)(ks != 0), &empty[s]);
        }
      }
      tc_commit_elect(&tmem_full[acc]);
    }
  } else if (warp < 6) {
    // ---------------- epilogue ----------------
    const int quad = warp & 3;
    const float *const ga = g.e.ga;
    const int ga_stride = g.e.ga_stride;
    const float gf = g.e.gf, alpha = g.e.alpha, beta = g.e.beta;
    const float gb0 = g.e.gb ? __ldg(g.e.gb) : 1.f;   // B's global: dense B has none, INT8 B one for the tensor (a multiply by 1 is exact)
    const void *const cptr = g.e.c, *const biasptr = g.e.bias;
    const int ldc = g.e.ldc, c_dtype = g.e.c_dtype, bias_dtype = g.e.bias_dtype;
    uint8_t *const dptr = (uint8_t *)g.e.d;
    const int ldd = g.e.ldd, d_dtype = g.e.d_dtype;
    float *const amax_out = g.e.amax;
    const int mask = g.x.mask;
    const float *const norm_parts = g.x.norm_parts;
    const int norm_nparts = g.x.norm_nparts, norm_ld = g.x.norm_ld;
    const float norm_inv_n = g.x.norm_inv_n, norm_eps = g.x.norm_eps;
    const float *const colscales = g.x.colscales;
    uint8_t *const d2ptr = (uint8_t *)g.x.d2;
    const int d2_dtype = g.x.d2_dtype, ldd2 = g.x.ldd2, w2_dtype = g.x.w2_dtype, ld_sq = g.x.ld_sq;
    const void *const w2ptr = g.x.w2;
    float *const sqptr = g.x.sq;
    const bool d_tma = g.d_tma;
    const int esz = dense_bytes(d_dtype);
    const int cw = esz == 2 ? 32 : 16;
    const bool leader = warp == 2 && lane == 0;
    const float zf = ue ? 65536.f : 256.f;
    float amax = 0.f;
    uint32_t tile_i = 0;
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++tile_i) {
      const int tm = t % tiles_m, tn = t / tiles_m, acc = tile_i & 1;
      const int i = tm * 128 + quad * 32 + lane;
      const bool row_ok = i < gm;
      const float rowp = row_ok ? __fmul_rn(alpha, ga ? ga[(size_t)i * ga_stride] : 1.f) : 0.f;
      const float bias = (row_ok && biasptr) ? load_dense(bias_dtype, biasptr, i) : 0.f;
      const float w2 = (row_ok && (mask & kExOut2)) ? load_dense(w2_dtype, w2ptr, i) : 0.f;
      const float s_plain = __fmul_rn(__fmul_rn(rowp, gb0), gf);   // ((alpha gA) * gB) * gf
      if (mask & kExNorm) {  // column scales of this token tile (the previous tile's are no longer in use: see the barrier below)
        named_barrier(1, 128);
        if (colscales) {  // computed before the launch, one float per token
          for (int jj = quad * 32 + lane; jj < BN; jj += 128) colscale[jj] = __ldcg(colscales + min(tn * BN + jj, gn - 1));
        }
        // The defining order (reference include/nvfp4effma.h:224-226 there): lane l adds parts l, l + 32, ... in ascending
        // order, then an xor butterfly 16..1.  A warp takes 8 tokens at a time so that their loads fly together.
        for (int j8 = quad * 8; j8 < BN && !colscales; j8 += 32) {
          float sum[8];
          if (norm_nparts <= 256) {
            float v[8][8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int j = min(tn * BN + j8 + u, gn - 1);
              const float *p = norm_parts + (size_t)j * norm_ld + lane;
#pragma unroll
              for (int q = 0; q < 8; ++q) v[u][q] = (32 * q + lane < norm_nparts) ? __ldcg(p + 32 * q) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              float a = 0.f;
#pragma unroll
              for (int q = 0; q < 8; ++q)
                if (32 * q + lane < norm_nparts) a = __fadd_rn(a, v[u][q]);
              sum[u] = a;
            }
          } else {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int j = min(tn * BN + j8 + u, gn - 1);
              const float *p = norm_parts + (size_t)j * norm_ld;
              float a = 0.f;
              for (int q = lane; q < norm_nparts; q += 32) a = __fadd_rn(a, __ldcg(p + q));
              sum[u] = a;
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            float a = sum[u];
#pragma unroll
            for (int o = 16; o; o >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
            if (lane == 0) colscale[j8 + u] = __frsqrt_rn(__fadd_rn(__fmul_rn(a, norm_inv_n), norm_eps));
          }
        }
      }
      if (!wait(&tmem_full[acc], (tile_i >> 1) & 1, kStWaitTmemFull)) *abort_flag = 1;
      named_barrier(1, 128);   // the four epilogue warps go on together or not at all
      if (*abort_flag) goto done;
      tc_fence_after();
      const int nchunks = min(BN / 32, (gn - tn * BN + 31) / 32);
      for (int c = 0; c < nchunks; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN + c * 32, r);
        tmem_ld_wait();
        if (c == nchunks - 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[acc]);
        }
        const int j0 = tn * BN + c * 32;
        const int nvalid = min(32, gn - j0);
        // values before the output rounding, kept in r[] as FP32 bits
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) {
          const float a = __fmul_rn(__uint_as_float(r[jj]), zf);
          const float s = (mask & kExNorm) ? __fmul_rn(__fmul_rn(rowp, __fmul_rn(gb0, colscale[c * 32 + jj])), gf) : s_plain;
          float v = __fmul_rn(a, s);
          if (biasptr) v = __fadd_rn(v, bias);
          if (beta != 0.f && row_ok && jj < nvalid) v = __fmaf_rn(beta, load_dense(c_dtype, cptr, (size_t)(j0 + jj) * ldc + i), v);
          r[jj] = __float_as_uint(v);
        }
        if (mask & kExOut2) {  // second output v * w2[i] and the slice's sum of squares (rows 16 q .. 16 q + 15 in ascending order)
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) {
            const float v = __uint_as_float(r[jj]);
            if (row_ok && jj < nvalid) store_dense(d2_dtype, d2ptr, (size_t)(j0 + jj) * ldd2 + i, __fmul_rn(v, w2));
            const float vv = __fmul_rn(v, v);
            float sq = 0.f;
#pragma unroll
            for (int q = 0; q < 16; ++q) sq = __fadd_rn(sq, __shfl_sync(0xFFFFFFFFu, vv, (lane & 16) + q));
            if (row_ok && !(lane & 15) && jj < nvalid) sqptr[(size_t)(j0 + jj) * ld_sq + (i >> 4)] = sq;
          }
        }
        if (mask & kExSwiglu) {  // rows 16 q + r (gate) and 16 q + 8 + r (up) -> output row 8 q + r: 64 output rows per tile
          // The gate lane and its up lane (lane ^ 8) share the work: the gate lane forms the even columns of their output
          // row, the up lane the odd ones; one shuffle per column pair carries what each needs from the other.
          const int io = (i >> 4) * 8 + (i & 7);
          const bool gate = !(lane & 8);
          const int odd = gate ? 0 : 1;
#pragma unroll
          for (int q = 0; q < 16; ++q) {
            const float v0 = __uint_as_float(r[2 * q]), v1 = __uint_as_float(r[2 * q + 1]);
            const float got = __shfl_xor_sync(0xFFFFFFFFu, gate ? v1 : v0, 8);
            const float h = gate ? silu_mul(v0, got) : silu_mul(got, v1);
            if (row_ok && 2 * q + odd < nvalid) amax = fmaxf(amax, fabsf(h));
            if (d_dtype == NVFP4A_BF16) r[q] = f32_to_bf16_bits(h);
            else if (d_dtype == NVFP4A_FP16) r[q] = (uint32_t)__half_as_ushort(__float2half_rn(h));
            else r[q] = __float_as_uint(h);
          }
          if (!d_tma) {
            if (row_ok) {
#pragma unroll
              for (int q = 0; q < 16; ++q)
                if (2 * q + odd < nvalid) {
                  if (esz == 2) ((uint16_t *)dptr)[(size_t)(j0 + 2 * q + odd) * ldd + io] = (uint16_t)r[q];
                  else ((uint32_t *)dptr)[(size_t)(j0 + 2 * q + odd) * ldd + io] = r[q];
                }
            }
            continue;
          }
          const int lr = quad * 16 + (lane >> 4) * 8 + (lane & 7);  // output row inside the tile's 64
          for (int half = 0; half < 32 / cw; ++half) {
            if (leader) bulk_wait_read_all();
            named_barrier(1, 128);
            if (esz == 2) {
#pragma unroll
              for (int q = 0; q < 16; ++q) ((uint16_t *)staging)[(2 * q + odd) * 64 + lr] = (uint16_t)r[q];
            } else {
#pragma unroll
              for (int q = 0; q < 8; ++q) ((uint32_t *)staging)[(2 * q + odd) * 64 + lr] = half ? r[8 + q] : r[q];
            }
            fence_proxy_async_smem();
            named_barrier(1, 128);
            if (leader) {
              tma_store_2d(&tmap_d, staging, tm * 64, j0 + half * cw);
              for (int p = 0; p < peers.n; ++p) tma_store_2d(&peers.map[p], staging, tm * 64, j0 + half * cw);   // the same tile into every peer's buffer
              bulk_commit();
            }
          }
          continue;
        }
        if (amax_out && row_ok) {
#pragma unroll
          for (int jj = 0; jj < 32; ++jj)
            if (jj < nvalid) amax = fmaxf(amax, fabsf(__uint_as_float(r[jj])));
        }
        if (d_dtype == NVFP4A_BF16) {
          round32_to_bf16(r);
        } else if (d_dtype == NVFP4A_FP16) {
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) r[jj] = (uint32_t)__half_as_ushort(__float2half_rn(__uint_as_float(r[jj])));
        }
        if (!d_tma) {
          if (row_ok) {
            if (esz == 2) {
              uint16_t *d16 = (uint16_t *)dptr + (size_t)j0 * ldd + i;
#pragma unroll
              for (int jj = 0; jj < 32; ++jj)
                if (jj < nvalid) d16[(size_t)jj * ldd] = (uint16_t)r[jj];
            } else {
              uint32_t *d32 = (uint32_t *)dptr + (size_t)j0 * ldd + i;
#pragma unroll
              for (int jj = 0; jj < 32; ++jj)
                if (jj < nvalid) d32[(size_t)jj * ldd] = r[jj];
            }
          }
          continue;
        }
        for (int half = 0; half < 32 / cw; ++half) {
          if (leader) bulk_wait_read_all();
          named_barrier(1, 128);
          const int rr = quad * 32 + lane;
          if (esz == 2) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) ((uint16_t *)staging)[jj * 128 + rr] = (uint16_t)r[jj];
          } else {
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) ((uint32_t *)staging)[jj * 128 + rr] = half ? r[16 + jj] : r[jj];
          }
          fence_proxy_async_smem();
          named_barrier(1, 128);
          if (leader) {
            tma_store_2d(&tmap_d, staging, tm * 128, j0 + half * cw);
            for (int p = 0; p < peers.n; ++p) tma_store_2d(&peers.map[p], staging, tm * 128, j0 + half * cw);   // the same tile into every peer's buffer
            bulk_commit();
          }
        }
      }
    }
    if (leader) bulk_wait_all();
    if (amax_out) warp_amax_commit(amax_out, amax);
  } else {
    // ---------------- weight expansion: NVFP4 -> BF16 into the swizzled A tile ----------------
    // Two groups of four warps take alternate stages; inside a group thread r owns row r of the stage: 64 nibbles (32
    // contiguous bytes) and their 4 scale bytes, fetched one of its own stages (two pipeline stages) ahead.
    const int cwarp = warp - 6, group = cwarp >> 2;
    const int row = (cwarp & 3) * 32 + lane;
    const Fp4Operand A = g.A;
    const ScalePos sp{A.sld};
    // source pointers of (tile t, k step 0) for this thread's row; a k step advances nibbles by 32 bytes and scales by 4
    auto tile_ptrs = [&](int t, const uint8_t *&wp, const uint8_t *&scp) {
      const int r = min((t % tiles_m) * 128 + row, gm - 1);
      if (A.image) {
        const uint8_t *tile = A.data + (size_t)(r >> 7) * A.ktiles * kImgTileBytes;
        const int rr = r & 127;
        wp = tile + rr * 128;
        scp = tile + kImgDataBytes + (rr & 31) * 16 + (rr >> 5) * 4;
      } else {
        wp = A.data + (size_t)r * (A.ld >> 1);
        scp = A.sc + sp.row(r);
      }
    };
    const bool img = A.image, swz = A.sld < 0;
    auto fetch = [&](const uint8_t *wp, const uint8_t *scp, int ks, RawRow &v) {
      size_t woff, soff;
      if (img) { woff = (size_t)(ks >> 2) * kImgTileBytes + (ks & 3) * 32; soff = (size_t)(ks >> 2) * kImgTileBytes + (ks & 3) * 512; }
      else { woff = (size_t)ks * 32; soff = swz ? (size_t)ks * 512 : (size_t)ks * 4; }
      v.w0 = __ldg((const uint4 *)(wp + woff));
      v.w1 = __ldg((const uint4 *)(wp + woff + 16));
      v.sc = __ldg((const uint32_t *)(scp + soff));
    };
    // prefetch cursor: this group's next stage (tile pf_t, k step pf_ks)
    int pf_t = blockIdx.x, pf_ks = group;
    const uint8_t *pf_w = nullptr, *pf_s = nullptr;
    auto advance = [&]() {  // to the group's following stage
      pf_ks += 2;
      while (pf_ks >= nk && pf_t < ntiles) { pf_ks -= nk; pf_t += gridDim.x; if (pf_t < ntiles) tile_ptrs(pf_t, pf_w, pf_s); }
    };
    RawRow cur, nxt;
    cur.w0 = cur.w1 = nxt.w0 = nxt.w1 = make_uint4(0, 0, 0, 0); cur.sc = nxt.sc = 0;
    if (pf_t < ntiles) tile_ptrs(pf_t, pf_w, pf_s);
    while (pf_ks >= nk && pf_t < ntiles) { pf_ks -= nk; pf_t += gridDim.x; if (pf_t < ntiles) tile_ptrs(pf_t, pf_w, pf_s); }
    if (pf_t < ntiles) { fetch(pf_w, pf_s, pf_ks, cur); advance(); }
    uint32_t it = 0;
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
      for (int ks = 0; ks < nk; ++ks, ++it) {
        if ((int)(it & 1) != group) continue;
        if (pf_t < ntiles) { fetch(pf_w, pf_s, pf_ks, nxt); advance(); }
        const int s = it % kStages;
        if (!wait(&empty[s], ((it / kStages) & 1) ^ 1, kStWaitConv)) goto done;
        uint8_t *sA = smem + (size_t)s * C::kStageBytes + row * 128;
        const uint32_t wv[8] = {cur.w0.x, cur.w0.y, cur.w0.z, cur.w0.w, cur.w1.x, cur.w1.y, cur.w1.z, cur.w1.w};
#pragma unroll
        for (int q = 0; q < 8; ++q) {  // word q: k = 8 q .. 8 q + 7 of the stage, block q / 2
          const uint32_t sc = lut[(cur.sc >> (8 * (q >> 1))) & 0xFF];
          const uint32_t d0 = bf16x2_mul(decode_pair<0>(wv[q]), sc), d1 = bf16x2_mul(decode_pair<1>(wv[q]), sc);
          const uint32_t d2 = bf16x2_mul(decode_pair<2>(wv[q]), sc), d3 = bf16x2_mul(decode_pair<3>(wv[q]), sc);
          // (n0 n4)(n1 n5)(n2 n6)(n3 n7) -> (n0 n1)(n2 n3)(n4 n5)(n6 n7)
          const uint4 o = make_uint4(prmt(d0, d1, 0x5410), prmt(d2, d3, 0x5410), prmt(d0, d1, 0x7632), prmt(d2, d3, 0x7632));
          *(uint4 *)(sA + ((q ^ (row & 7)) << 4)) = o;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full[s]);
        cur = nxt;
      }
    }
  }
done:
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int BN, int PLANES = 1>
cudaError_t launch_cfg(const CUtensorMap &tb, const CUtensorMap &td, const PeerMaps &pm, const W4A16Args &a, cudaStream_t s) {
  using C = Cfg<BN, PLANES>;
  static std::atomic<bool> attr_set[64];   // zero-initialised; set once per device (a repeated cudaFuncSetAttribute is harmless)
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    const cudaError_t e = cudaFuncSetAttribute(gemm_w4a16_kernel<BN, PLANES>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set[dev & 63] = true;
  }
  const int tiles = ((a.m + 127) / 128) * ((a.n + BN - 1) / BN);
  const int grid = tiles < device_sms() ? tiles : device_sms();
  gemm_w4a16_kernel<BN, PLANES><<<grid, kThreads, C::kSmemBytes, s>>>(tb, td, pm, a);
  return cudaGetLastError();
}

// INT8 activations q [n][ld] with one FP32 scale per 16 values -> three BF16 planes [n][3][k] with t1 + t2 + t3 = fl(q * s) exactly.
// One thread per 8 values: 8 bytes in, three 16-byte stores out.
__global__ void __launch_bounds__(256) w4a8_planes_kernel(const int8_t *__restrict__ q, int ld, const float *__restrict__ sc, int lds, int n, int k,
                                                          uint16_t *__restrict__ planes) {
  const long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x, per_row = k >> 3;
  if (v >= per_row * n) return;
  const int j = (int)(v / per_row), c = (int)(v - (long long)j * per_row);   // token, group of 8 values
  const uint2 raw = *(const uint2 *)(q + (size_t)j * ld + 8 * c);
  const float s = sc[(size_t)j * lds + (c >> 1)];
  uint32_t t[3][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int qi = (int)(int8_t)(((i < 4 ? raw.x : raw.y) >> (8 * (i & 3))) & 0xFFu);
    float r = __fmul_rn((float)qi, s);
#pragma unroll
    for (int p = 0; p < 3; ++p) {
      const float tp = __bfloat162float(__float2bfloat16_rn(r));   // 8 significant bits, round to nearest even
      const uint32_t h = __float_as_uint(tp) >> 16;
      if (i & 1) t[p][i >> 1] |= h << 16;
      else t[p][i >> 1] = h;
      r = __fsub_rn(r, tp);   // exact: the remainder has at most 16, then 8 significant bits
    }
  }
  uint16_t *row = planes + (size_t)j * 3 * k + 8 * c;
#pragma unroll
  for (int p = 0; p < 3; ++p) *(uint4 *)(row + (size_t)p * k) = make_uint4(t[p][0], t[p][1], t[p][2], t[p][3]);
}

}  // namespace

// tensor parallel: true when this kernel stores D into the peers' buffers itself (its output path is the TMA store)
bool gemm_w4a16_pushes(const GemmArgs &g) {
  if (g.tp.world <= 1) return false;
  const int esz = dense_bytes(g.e.d_dtype);
  const int drows = (g.x.mask & kExSwiglu) ? g.m / 2 : g.m;
  return ((uintptr_t)g.e.d & 15) == 0 && ((size_t)g.e.ldd * esz) % 16 == 0 && ((size_t)drows * esz) % 16 == 0;
}

bool gemm_w4a16_supports(const GemmArgs &g) {
  if (g.B.dtype != NVFP4A_BF16 || g.k < 64 || ((uintptr_t)g.B.data & 15) || g.B.ld % 8) return false;
  if (!g.A.image && (((uintptr_t)g.A.data & 15) || g.A.ld % 32 || ((uintptr_t)g.A.sc & 1))) return false;
  return true;
}

// The planes' memory comes from a pool of this library's own, one per device, that keeps what it has been given (release threshold
// at the maximum): a stream-ordered allocation from it costs microseconds and synchronises nothing, whereas the device's default
// pool hands its memory back at every synchronisation, so that a caller who synchronises once per step would pay a fresh
// allocation per call.  The pool holds the largest planes buffer in use so far until nvfp4a_b200_trim_scratch or process exit.
static std::atomic<cudaMemPool_t> g_planes_pool[64];
static cudaError_t planes_pool(cudaMemPool_t *pool) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  cudaMemPool_t p = g_planes_pool[dev & 63].load();
  if (!p) {
    cudaMemPoolProps props;
    memset(&props, 0, sizeof props);
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = dev;
    e = cudaMemPoolCreate(&p, &props);
    if (e != cudaSuccess) return e;
    unsigned long long keep = ~0ull;
    cudaMemPoolSetAttribute(p, cudaMemPoolAttrReleaseThreshold, &keep);
    cudaMemPool_t expected = nullptr;
    if (!g_planes_pool[dev & 63].compare_exchange_strong(expected, p)) {   // another thread was first: use its pool
      cudaMemPoolDestroy(p);
      p = expected;
    }
  }
  *pool = p;
  return cudaSuccess;
}
cudaError_t trim_planes_pool() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  cudaMemPool_t p = g_planes_pool[dev & 63].load();
  return p ? cudaMemPoolTrimTo(p, 0) : cudaSuccess;
}

// W4A8 on the tensor cores (see the header): from 64 tokens and 128 weight rows up, where the planes' set-up pays.  The call
// takes the planes from the pool above (stream-ordered: capturable, no synchronisation) and gives them back after the GEMM.
bool gemm_w4a8_tc_supports(const GemmArgs &g) {
  if (g.B.dtype != NVFP4A_INT8 || g.k < 64 || g.n < 64 || g.m < 128 || g.no_alloc || g.tp.world > 1 || g.e.gb_stride) return false;
  if (((uintptr_t)g.B.data & 7) || g.B.ld % 8 || !g.B.s8 || ((uintptr_t)g.B.s8 & 3)) return false;
  if (!g.A.image && (((uintptr_t)g.A.data & 15) || g.A.ld % 32 || ((uintptr_t)g.A.sc & 1))) return false;
  return true;
}

cudaError_t launch_gemm_w4a8_tc(const GemmArgs &g, cudaStream_t s) {
  W4A16Args a;
  memset(&a, 0, sizeof a);
  a.m = g.m; a.n = g.n; a.k = g.k;
  a.A = g.A;
  a.e = g.e; a.x = g.x;
  a.status = kernel_status_device_ptr();
  a.tag = next_launch_tag();
  uint16_t *planes = nullptr;
  cudaMemPool_t pool;
  cudaError_t e = planes_pool(&pool);
  if (e != cudaSuccess) return e;
  e = cudaMallocFromPoolAsync((void **)&planes, (size_t)g.n * 3 * g.k * sizeof(uint16_t), pool, s);
  if (e != cudaSuccess) return e;
  const long long groups = (long long)g.n * (g.k >> 3);
  w4a8_planes_kernel<<<(unsigned)((groups + 255) / 256), 256, 0, s>>>((const int8_t *)g.B.data, g.B.ld, g.B.s8, g.B.lds8, g.n, g.k, planes);
  e = cudaGetLastError();
  CUtensorMap tb, td;
  memset(&td, 0, sizeof td);
  if (e == cudaSuccess && !make_tmap_bytes(&tb, planes, (uint64_t)g.k * 6, (uint64_t)g.n, (uint64_t)g.k * 6, 128)) e = cudaErrorInvalidValue;
  if (e == cudaSuccess) {
    const int esz = dense_bytes(g.e.d_dtype);
    const bool glu = (g.x.mask & kExSwiglu) != 0;
    const int drows = glu ? g.m / 2 : g.m;
    a.d_tma = ((uintptr_t)g.e.d & 15) == 0 && ((size_t)g.e.ldd * esz) % 16 == 0 && ((size_t)drows * esz) % 16 == 0 &&
              make_tmap_dense(&td, g.e.d, esz, (uint64_t)drows, (uint64_t)g.n, (uint64_t)g.e.ldd * esz, glu ? 64 : 128, esz == 2 ? 32 : 16);
    PeerMaps pm;
    memset(&pm, 0, sizeof pm);
    e = launch_cfg<128, 3>(tb, td, pm, a, s);
  }
  const cudaError_t ef = cudaFreeAsync(planes, s);
  return e != cudaSuccess ? e : ef;
}

cudaError_t launch_gemm_w4a16(const GemmArgs &g, cudaStream_t s) {
  W4A16Args a;
  memset(&a, 0, sizeof a);
  a.m = g.m; a.n = g.n; a.k = g.k;
  a.A = g.A;
  a.e = g.e; a.x = g.x;
  a.status = kernel_status_device_ptr();
  a.tag = next_launch_tag();
  const int bn = g.n > 128 ? 256 : 128;
  CUtensorMap tb, td;
  if (!make_tmap_bytes(&tb, g.B.data, (uint64_t)g.k * 2, (uint64_t)g.n, (uint64_t)g.B.ld * 2, bn)) return cudaErrorInvalidValue;
  memset(&td, 0, sizeof td);
  const int esz = dense_bytes(g.e.d_dtype);
  const bool glu = (g.x.mask & kExSwiglu) != 0;
  const int drows = glu ? g.m / 2 : g.m;   // SwiGLU: the output has m / 2 rows, 64 per tile
  a.d_tma = ((uintptr_t)g.e.d & 15) == 0 && ((size_t)g.e.ldd * esz) % 16 == 0 && ((size_t)drows * esz) % 16 == 0 &&
            make_tmap_dense(&td, g.e.d, esz, (uint64_t)drows, (uint64_t)g.n, (uint64_t)g.e.ldd * esz, glu ? 64 : 128, esz == 2 ? 32 : 16);
  PeerMaps pm;
  memset(&pm, 0, sizeof pm);
  if (gemm_w4a16_pushes(g)) {   // tensor parallel: the epilogue's TMA stores also go to every peer's copy of D
    for (int p = 0; p < g.tp.world; ++p) {
      if (p == g.tp.rank) continue;
      if (!make_tmap_dense(&pm.map[pm.n], (uint8_t *)g.e.d + g.tp.delta[p], esz, (uint64_t)drows, (uint64_t)g.n, (uint64_t)g.e.ldd * esz, glu ? 64 : 128,
                           esz == 2 ? 32 : 16))
        return cudaErrorInvalidValue;
      ++pm.n;
    }
  }
  return bn == 256 ? launch_cfg<256>(tb, td, pm, a, s) : launch_cfg<128>(tb, td, pm, a, s);
}

}  // namespace nvb
