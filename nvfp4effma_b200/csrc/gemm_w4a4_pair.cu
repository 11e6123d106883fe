// NVFP4 x NVFP4 (W4A4) GEMM on CTA pairs: tcgen05.mma.cta_group::2 kind::mxf4nvf4 on 256 x 256 tiles, the fast form of the
// W4A4 route for large problems whose D is a 16-bit matrix that TMA can store and whose block scales lie in aligned
// 512-byte tiles (the GEMM-swizzled layout, or images).  Everything else runs on the single-CTA kernel (gemm_w4a4.cu).
//
// Why pairs: one MMA of 128 x 256 x 64 keeps an SM's tensor pipe busy for 128 cycles (measured: nvfp4a_b200_mma_ceiling), so
// a stage of 256 values of k is consumed in 512 cycles.  A single CTA has to pull 54 KB through L2 for that (128 + 256 operand
// rows and their scales); with a memory round trip of about 2000 cycles that needs more bytes in flight than shared memory
// holds.  In a pair each CTA loads its 128 rows of the M side and only HALF of the 256 rows of the N side -- 38 KB per
// stage -- and five stages fit beside the epilogue's staging tiles.
//
// Orientation: the call's B (tokens) is the MMA's M side (tensor memory lanes), the call's A (weight rows) its N side
// (columns), so that a lane's accumulator columns are consecutive elements of column-major D.
//
// Per CTA, 16 warps:
//   warp 0      operand producer: the stage's two nibble tiles (its 128 M rows, its 128 of the 256 N rows) by ONE TMA
//               instruction of two lanes; both CTAs' bytes are counted on the even CTA's `full` barrier
//   warp 1      lane 0 of the EVEN CTA issues the MMAs for the pair; the warp owns the tensor memory allocation
//   warp 2      scale producer: the stage's three 2 KiB scale tiles into a ring of their own, several stages ahead
//   warps 4-7   scale warps: shared memory -> registers -> tensor memory (tcgen05.st; one 32-lane quadrant each), so the
//               MMA thread never waits for scales and issues nothing but MMAs (tcgen05.cp on its queue costs the tensor
//               pipe about 27 cycles per 512-byte tile: measured)
//   warps 8-15  epilogue: quadrant = warp % 4, column half = (warp - 8) / 4.  A warp pulls its 32 x 128 accumulator block
//               out of tensor memory in four loads, hands the accumulator back as soon as the last has landed, and
//               stores two 32 x 64 boxes from its own 4 KiB staging tile (128-byte TMA swizzle: conflict-free 16-byte
//               shared-memory stores), the second after the next tile's MMAs are already running.
// Every wait is bounded; a wait that gives up raises the CTA's abort flag and the kernel status word.
//
// Edges need no special code: TMA loads outside an operand read zeros (zero nibbles under zero scales contribute nothing),
// TMA stores clip at the edge of D.  Block scales are consumed as UNSIGNED E4M3, as in gemm_w4a4.cu.
#include <atomic>
#include "operands.cuh"
#include "sm100.cuh"

namespace nvb {

using namespace sm100;

struct PairArgs {
  int xm, yn, k;             // rows of the M-side operand (tokens), rows of the N-side operand (weight rows), k
  int x_image, y_image;      // operand is an image (3-D maps: one tile per z)
  int ktiles;                // image: 256-k tiles per row tile
  const float *g_tok;        // global of the M-side operand (the call's B): NULL = 1
  int g_tok_stride;          // 0: one value, 1: one per token
  const float *g_w;          // global of the N-side operand (the call's A), one value: NULL = 1
  float alpha, gf;           // an output is acc * (((alpha * g_w) * g_tok(token)) * gf), the order of the definition
  int d_dtype;
  float *amax;
  unsigned *status;
};

constexpr int kPairThreads = 512, kPairStages = 5, kPairSlots = 4;
constexpr int kXBytes = 16384, kYBytes = 16384, kPStage = kXBytes + kYBytes, kSlotBytes = 6144, kPSfCols = 48, kPAccCols = 256;
constexpr int kPStagingBytes = 8 * 4096, kPBarrierBytes = 512;
constexpr int kPairSmem = kPairStages * kPStage + kPStagingBytes + kPairSlots * kSlotBytes + kPBarrierBytes + 1024;
static_assert(kPairSmem <= 232448, "shared memory budget");
static_assert(kPAccCols + kPairStages * kPSfCols <= 512, "tensor memory budget");
constexpr unsigned kPStatFull = 0x111, kPStatEmpty = 0x112, kPStatTmemFull = 0x113, kPStatTmemEmpty = 0x114, kPStatScale = 0x115, kPStatSf = 0x116;

__global__ void __launch_bounds__(kPairThreads, 1)
gemm_w4a4_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_y,
                      const __grid_constant__ CUtensorMap tmap_sx, const __grid_constant__ CUtensorMap tmap_sy,
                      const __grid_constant__ CUtensorMap tmap_d, const PairArgs g) {
  constexpr int S = kPairStages, SD = kPairSlots;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *staging = smem + S * kPStage;
  uint8_t *scale_ring = staging + kPStagingBytes;
  uint64_t *bars = (uint64_t *)(scale_ring + SD * kSlotBytes);
  uint64_t *full = bars, *empty = full + S, *sf_ready = empty + S, *sfs_full = sf_ready + S, *sfs_empty = sfs_full + SD,
           *tmem_full = sfs_empty + SD, *tmem_empty = tmem_full + 1;
  uint32_t *tmem_slot = (uint32_t *)(tmem_empty + 1);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)cluster_ctarank();
  const int xm = g.xm, yn = g.yn, ktiles = g.ktiles;
  const int tiles_x = (xm + 255) / 256, ntiles = tiles_x * ((yn + 255) / 256);
  const int tile_first = blockIdx.x >> 1, tile_step = gridDim.x >> 1;
  const int nk = (g.k + 255) / 256;
  const int my_tiles = tile_first < ntiles ? (ntiles - tile_first + tile_step - 1) / tile_step : 0;
  const int total = my_tiles * nk;
  unsigned *const status_word = g.status;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); mbar_init(&sf_ready[s], 8); }
    for (int q = 0; q < SD; ++q) { mbar_init(&sfs_full[q], 1); mbar_init(&sfs_empty[q], 4); }
    mbar_init(tmem_full, 1);
    mbar_init(tmem_empty, 16);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_x);
    prefetch_tensormap(&tmap_y);
    prefetch_tensormap(&tmap_sx);
    prefetch_tensormap(&tmap_sy);
    prefetch_tensormap(&tmap_d);
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, 512);
  tc_fence_before();
  cluster_sync_all();   // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto wait = [abort_flag, status_word](uint64_t *bar, uint32_t parity, unsigned code) -> bool {
    if (mbar_try(bar, parity)) return true;   // the common case: no flag read, no clock read
    if (*abort_flag) return false;
    if (mbar_wait(bar, parity)) return true;
    *abort_flag = 1;
    atomicCAS(status_word, 0u, code);
    return false;
  };

  if (warp == 0) {
    // ---------------- operand producer ----------------
    // lane 0: this CTA's 128 rows of the M side; lane 1: its 128 of the tile's 256 N-side rows.  Bytes of both CTAs count on
    // the even CTA's barrier, whose MMA thread reads both CTAs' shared memory.
    const bool image = lane == 0 ? g.x_image : g.y_image;
    const CUtensorMap *const map = lane == 0 ? &tmap_x : &tmap_y;
    const uint32_t dst_off = lane == 0 ? 0 : kXBytes;
    int t = tile_first, ks = 0;
    int row_tile = 0;   // this lane's 128-row tile of its operand
    auto tile_setup = [&]() {
      const int tx = t % tiles_x, ty = t / tiles_x;
      row_tile = lane == 0 ? 2 * tx + rank : 2 * ty + rank;
    };
    if (total > 0) tile_setup();
    for (int it = 0; it < total; ++it) {
      const int s = it % S;
      if (!wait(&empty[s], ((it / S) & 1) ^ 1, kPStatEmpty)) break;
      if (lane == 0 && rank == 0) mbar_arrive_expect_tx(&full[s], 2 * kPStage);
      __syncwarp();
      if (lane < 2) {
        const uint32_t dst = smem_u32(smem + (size_t)s * kPStage + dst_off);
        const uint32_t bar = mbar_addr_rank(&full[s], 0);
        if (image) tma_load_3d_pair(dst, map, 0, 0, row_tile * ktiles + ks, bar);
        else tma_load_3d_pair(dst, map, ks * 128, row_tile * 128, 0, bar);
      }
      if (++ks == nk) { ks = 0; t += tile_step; tile_setup(); }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA) ----------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = idesc_mxf4nvf4(256, 256);
      const uint64_t da0 = smem_desc_sw128(smem_u32(smem));
      int it = 0;
      for (int tile_i = 0; tile_i < my_tiles; ++tile_i) {
        if (!wait(tmem_empty, (tile_i & 1) ^ 1, kPStatTmemEmpty)) goto done;
        tc_fence_after();
        for (int ks = 0; ks < nk; ++ks, ++it) {
          const int s = it % S;
          const uint32_t par = (it / S) & 1;
          if (!wait(&sf_ready[s], par, kPStatSf) || !wait(&full[s], par, kPStatFull)) goto done;
          tc_fence_after();
          const uint64_t da = da0 + (uint32_t)s * (uint32_t)(kPStage >> 4), db = da + (kXBytes >> 4);
          const uint32_t sfa = tmem_base + kPAccCols + s * kPSfCols, sfb = sfa + 16;
#pragma unroll
          for (int j = 0; j < 4; ++j)   // 64 values of k each: 32 bytes further along every 128-byte row
            mma_mxf4nvf4_pair(tmem_base, da + 2 * j, db + 2 * j, idesc, sfa + 4 * j, sfb + 8 * j, j ? 1u : (uint32_t)(ks != 0));
          tc_commit_pair(&empty[s]);   // both CTAs: stage s and scale buffer s are free once these MMAs have read them
        }
        tc_commit_pair(tmem_full);
      }
    }
  } else if (warp == 2) {
    // ---------------- scale producer ----------------
    // lane 0: the scale tiles of this CTA's 128 M-side rows; lanes 1, 2: those of the tile's two 128-row halves of the N side
    // (every CTA needs all of them in its tensor memory).  A box is the four 512-byte tiles of 256 values of k.
    const bool image = lane == 0 ? g.x_image : g.y_image;
    const CUtensorMap *const map = lane == 0 ? &tmap_sx : &tmap_sy;
    const uint32_t dst_off = lane == 0 ? 0 : 2048 * lane;
    int t = tile_first, ks = 0, row_tile = 0;
    auto tile_setup = [&]() {
      const int tx = t % tiles_x, ty = t / tiles_x;
      row_tile = lane == 0 ? 2 * tx + rank : 2 * ty + (lane - 1);
    };
    if (total > 0) tile_setup();
    for (int it = 0; it < total; ++it) {
      const int q = it % SD;
      if (!wait(&sfs_empty[q], ((it / SD) & 1) ^ 1, kPStatScale)) break;
      if (lane == 0) mbar_arrive_expect_tx(&sfs_full[q], kSlotBytes);
      __syncwarp();
      if (lane < 3) {
        const uint32_t dst = smem_u32(scale_ring + q * kSlotBytes + dst_off);
        const uint32_t bar = mbar_addr_rank(&sfs_full[q], rank);
        if (image) tma_load_3d_pair(dst, map, 0, row_tile * ktiles + ks, 0, bar);
        else tma_load_3d_pair(dst, map, ks * 256, row_tile, 0, bar);
      }
      if (++ks == nk) { ks = 0; t += tile_step; tile_setup(); }
    }
  } else if (warp >= 4 && warp < 8) {
    // ---------------- scale warps ----------------
    // A 512-byte tile's 16 bytes at offset 16 l are what lane l of every quadrant holds in four scale columns; each of the four
    // warps writes its own quadrant.  Buffer s of tensor memory is free when the MMAs of the stage's previous round are done.
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    for (int it = 0; it < total; ++it) {
      const int q = it % SD, s = it % S;
      if (!wait(&sfs_full[q], (it / SD) & 1, kPStatScale)) break;
      const uint8_t *src = scale_ring + q * kSlotBytes + lane * 16;
      uint4 va[4], vb[2][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) va[j] = *(const uint4 *)(src + j * 512);
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int j = 0; j < 4; ++j) vb[h][j] = *(const uint4 *)(src + 2048 + h * 2048 + j * 512);
      __syncwarp();
      if (lane == 0) mbar_arrive(&sfs_empty[q]);
      if (!wait(&empty[s], ((it / S) & 1) ^ 1, kPStatScale)) break;
      tc_fence_after();
      const uint32_t sf = tmem_base + kPAccCols + s * kPSfCols + lane_base;
      uint32_t r[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) { r[4 * j] = va[j].x; r[4 * j + 1] = va[j].y; r[4 * j + 2] = va[j].z; r[4 * j + 3] = va[j].w; }
      tmem_st16(sf, r);
#pragma unroll
      for (int part = 0; part < 2; ++part) {   // N-side columns: per 64 values of k [rows 0-127: 4 columns | rows 128-255: 4 columns]
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int j = 2 * part + (c >> 1), h = c & 1;
          r[4 * c] = vb[h][j].x; r[4 * c + 1] = vb[h][j].y; r[4 * c + 2] = vb[h][j].z; r[4 * c + 3] = vb[h][j].w;
        }
        tmem_st16(sf + 16 + part * 16, r);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_rank(&sf_ready[s], 0);
    }
  } else if (warp >= 8) {
    // ---------------- epilogue ----------------
    const int ew = warp - 8, quad = ew & 3, half = ew >> 2;
    uint8_t *const box = staging + ew * 4096, *const row = box + lane * 128;
    const int sw = lane & 7;
    const float *const g_tok = g.g_tok;
    const int g_tok_stride = g.g_tok_stride, d_dtype = g.d_dtype;
    const float gf = g.gf, s_uniform = __fmul_rn(g.alpha, g.g_w ? g.g_w[0] : 1.f);
    float *const amax_out = g.amax;
    const uint32_t acc_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + half * 128;
    float amax = 0.f;
    int tile_i = 0;
    for (int t = tile_first; t < ntiles; t += tile_step, ++tile_i) {
      const int tx = t % tiles_x, ty = t / tiles_x;
      const int tok0 = tx * 256 + rank * 128 + quad * 32, tok = tok0 + lane, col0 = ty * 256 + half * 128;
      const float tokp = (g_tok && tok < xm) ? g_tok[(size_t)tok * g_tok_stride] : 1.f;
      const float s_tok = __fmul_rn(__fmul_rn(s_uniform, tokp), gf);
      // scale, amax, round, pack: 32 accumulator columns -> 64 bytes of the lane's row of the box, as four swizzled 16-byte stores
      auto stage32 = [&](uint32_t (&r)[32], int chunk0) {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) r[jj] = __float_as_uint(__fmul_rn(__uint_as_float(r[jj]), s_tok));
        if (amax_out) {
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) amax = fmaxf(amax, fabsf(__uint_as_float(r[jj])));
        }
        if (d_dtype == NVFP4A_BF16) {
          round32_to_bf16(r);
        } else {
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) r[jj] = (uint32_t)__half_as_ushort(__float2half_rn(__uint_as_float(r[jj])));
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int b = 8 * q;
          *(uint4 *)(row + (((chunk0 + q) ^ sw) << 4)) = make_uint4(r[b] | (r[b + 1] << 16), r[b + 2] | (r[b + 3] << 16), r[b + 4] | (r[b + 5] << 16),
                                                                  r[b + 6] | (r[b + 7] << 16));
        }
      };
      auto store_box = [&](int col) {   // (a box that lies outside D altogether is not stored; one that straddles the edge is clipped)
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && tok0 < xm && col < yn) {
          tma_store_2d(&tmap_d, box, col, tok0);
          bulk_commit();
        }
      };
      auto box_free = [&]() {   // this warp's previous store has finished reading the staging tile
        if (lane == 0) bulk_wait_read_all();
        __syncwarp();
      };
      bool okw = wait(tmem_full, tile_i & 1, kPStatTmemFull);
      if (!__all_sync(0xFFFFFFFFu, okw)) break;
      tc_fence_after();
      uint32_t ra[32], rb[32];
      tmem_ld32(acc_addr, ra);
      tmem_ld32(acc_addr + 32, rb);
      box_free();
      tmem_ld_wait();
      stage32(ra, 0);
      tmem_ld32(acc_addr + 64, ra);
      stage32(rb, 4);
      tmem_ld32(acc_addr + 96, rb);
      store_box(col0);
      tmem_ld_wait();
      // every column of this warp's block is in registers: the accumulator goes back to the MMA thread
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_rank(tmem_empty, 0);
      box_free();
      stage32(ra, 0);
      stage32(rb, 4);
      store_box(col0 + 64);
    }
    if (lane == 0) bulk_wait_all();
    if (amax_out) warp_amax_commit(amax_out, amax);
  }
done:
  __syncwarp();
  tc_fence_before();
  cluster_sync_all();   // neither CTA leaves (or frees tensor memory) while the other may still arrive on its barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// ---- host ------------------------------------------------------------------------------------------------------------------
static bool pair_tiled_ok(const Fp4Operand &o) { return o.image || (o.sld < 0 && ((uintptr_t)o.sc & 15) == 0); }

// Does the problem qualify, and is the pair kernel the faster choice?  (`force`: take it wherever it applies.)
bool gemm_w4a4_pair_applies(const GemmArgs &g, bool force) {
  const int esz = dense_bytes(g.e.d_dtype);
  if (esz != 2 || ((uintptr_t)g.e.d & 15) || ((size_t)g.e.ldd * esz) % 16 || ((size_t)g.m * esz) % 16) return false;
  if (g.e.beta != 0.f || g.e.bias || g.e.ga_stride) return false;
  if (!pair_tiled_ok(g.A) || !pair_tiled_ok(g.B.q)) return false;
  if (force) return true;
  if (g.n < 256 || g.m < 256) return false;
  // rounds of tiles over the SMs, weighted by what a tile costs: a 256 x 256 tile on a pair ~ 2 units, a 128 x 256 tile on one CTA ~ 3
  const long long sms = device_sms(), pairs = sms / 2;
  const long long ptiles = (long long)((g.n + 255) / 256) * ((g.m + 255) / 256), stiles = (long long)((g.n + 127) / 128) * ((g.m + 255) / 256);
  return ((ptiles + pairs - 1) / pairs) * 2 <= ((stiles + sms - 1) / sms) * 3;
}

cudaError_t launch_gemm_w4a4_pair(const GemmArgs &g, cudaStream_t s) {
  PairArgs a;
  memset(&a, 0, sizeof a);
  const Fp4Operand &X = g.B.q, &Y = g.A;   // X: tokens (lanes), Y: weight rows (columns)
  a.xm = g.n; a.yn = g.m; a.k = g.k;
  a.ktiles = (g.k + kImgK - 1) / kImgK;
  a.x_image = X.image; a.y_image = Y.image;
  a.g_tok = g.e.gb; a.g_tok_stride = g.e.gb_stride;
  a.g_w = g.e.ga; a.alpha = g.e.alpha; a.gf = g.e.gf;
  a.d_dtype = g.e.d_dtype;
  a.amax = g.e.amax;
  a.status = kernel_status_device_ptr();
  CUtensorMap tx, ty, tsx, tsy, td;
  auto maps = [&](const Fp4Operand &o, int rows, CUtensorMap *tn, CUtensorMap *ts) {
    if (o.image) {
      const uint64_t tiles = (uint64_t)((rows + 127) / 128) * a.ktiles;
      return make_tmap_bytes(tn, o.data, 128, 128, 128, 128, tiles, kImgTileBytes) &&
             make_tmap_scales(ts, (const uint8_t *)o.data + kImgDataBytes, 2048, tiles, kImgTileBytes);
    }
    const uint64_t tile_row_bytes = (uint64_t)((-o.sld) >> 2) * 512;
    return make_tmap_bytes(tn, o.data, (uint64_t)g.k / 2, (uint64_t)rows, (uint64_t)o.ld / 2, 128, 1, (uint64_t)o.ld / 2 * rows) &&
           make_tmap_scales(ts, o.sc, tile_row_bytes, (uint64_t)(rows + 127) / 128, tile_row_bytes);
  };
  if (!maps(X, a.xm, &tx, &tsx) || !maps(Y, a.yn, &ty, &tsy)) return cudaErrorInvalidValue;
  if (!make_tmap_dense(&td, g.e.d, 2, (uint64_t)g.m, (uint64_t)g.n, (uint64_t)g.e.ldd * 2, 64, 32, 128)) return cudaErrorInvalidValue;
  static std::atomic<unsigned long long> attr_set{0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(attr_set.load() >> (dev & 63) & 1)) {
    const cudaError_t e = cudaFuncSetAttribute(gemm_w4a4_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem);
    if (e != cudaSuccess) return e;
    attr_set.fetch_or(1ull << (dev & 63));
  }
  const int tiles = ((a.xm + 255) / 256) * ((a.yn + 255) / 256), pairs = device_sms() / 2;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = dim3(2 * (tiles < pairs ? tiles : pairs), 1, 1);
  cfg.blockDim = dim3(kPairThreads, 1, 1);
  cfg.dynamicSmemBytes = kPairSmem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, gemm_w4a4_pair_kernel, tx, ty, tsx, tsy, td, a);
}

}  // namespace nvb
