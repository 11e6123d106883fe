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
//   warp 0      operand producer: the stage's two nibble tiles (its 128 M rows, its half of the N rows).  Both CTAs' bytes are
//               counted on the even CTA's `full` barrier, on which the scale warps of both CTAs arrive too, so the MMA warp
//               waits once per stage.
//   warp 1      MMA warp of the EVEN CTA: the whole warp runs the loop and one elected lane issues a stage's four MMAs and
//               its commit in one statement.  Issued from inside a one-lane branch, every tcgen05.mma costs about 150 cycles
//               whatever its shape -- more than the 128 the tensor pipe needs for it (measured; see sm100.cuh).  The warp owns
//               the tensor memory allocation.
//   warps 2, 3  scale producers (alternate stages): the stage's three 2 KiB scale tiles into a ring of their own, several
//               stages ahead of the operands
//   warps 4-7   scale warps: shared memory -> registers -> tensor memory (tcgen05.st; one 32-lane quadrant each), so the
//               MMA warp never waits for scales and issues nothing but MMAs (tcgen05.cp on its queue costs the tensor pipe
//               about 27 cycles per 512-byte tile: measured)
//   warps 8-15  epilogue (168 registers each, taken from the other eight warps by setmaxnreg): quadrant = warp % 4, column
//               half = (warp - 8) / 4.  A warp pulls its whole 32 x 128 accumulator block into registers with four loads and
//               hands the accumulator back at once; scaling, rounding and the two 32 x 64 box stores from its 4 KiB staging
//               tile (128-byte TMA swizzle: conflict-free 16-byte shared-memory stores) run under the next tile's MMAs.
// Tiles that would fill at most half of the SM pairs in the last round are cut into two 128-wide halves.
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
  int nfull, nhalf;          // tiles 0 .. nfull - 1 are 256 columns wide, the nhalf tiles after them 128 (two per 256-wide tile)
  const float *g_tok;        // global of the M-side operand (the call's B): NULL = 1
  int g_tok_stride;          // 0: one value, 1: one per token
  const float *g_w;          // global of the N-side operand (the call's A), one value: NULL = 1
  float alpha, gf;           // an output is acc * (((alpha * g_w) * g_tok(token)) * gf), the order of the definition
  int d_dtype;
  float *amax;
  unsigned *status;
  unsigned tag;              // this launch's tag in the status word
};

constexpr int kPairThreads = 512, kPairStages = 5, kPairSlots = 4;
constexpr int kXBytes = 16384, kYBytes = 16384, kPStage = kXBytes + kYBytes, kSlotBytes = 6144, kPSfCols = 48, kPAccCols = 256;
constexpr int kPStagingBytes = 8 * 4096, kPBarrierBytes = 512;
constexpr int kPairSmem = kPairStages * kPStage + kPStagingBytes + kPairSlots * kSlotBytes + kPBarrierBytes + 1024;
static_assert(kPairSmem <= 232448, "shared memory budget");
static_assert(kPAccCols + kPairStages * kPSfCols <= 512, "tensor memory budget");
constexpr unsigned kPStatFull = 0x111, kPStatEmpty = 0x112, kPStatTmemFull = 0x113, kPStatTmemEmpty = 0x114, kPStatScale = 0x115;


// Tile t of the schedule: the 256 tokens [256 tx, +256) against `width` N-side rows starting at the 128-row tile y128.  The tiles
// that would fill only part of the last round over the SM pairs are cut in two 128-wide halves, so that round costs half.
struct PairTile { int tx, y128, width; };
__device__ __forceinline__ PairTile pair_tile(int t, int tiles_x, int nfull) {
  if (t < nfull) return PairTile{t % tiles_x, 2 * (t / tiles_x), 256};
  const int h = t - nfull, f = nfull + (h >> 1);
  return PairTile{f % tiles_x, 2 * (f / tiles_x) + (h & 1), 128};
}




__global__ void __launch_bounds__(kPairThreads, 1)
gemm_w4a4_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_y,
                      const __grid_constant__ CUtensorMap tmap_y64, const __grid_constant__ CUtensorMap tmap_sx, const __grid_constant__ CUtensorMap tmap_sy,
                      const __grid_constant__ CUtensorMap tmap_d, const PairArgs g) {
  constexpr int S = kPairStages, SD = kPairSlots;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *staging = smem + S * kPStage;
  uint8_t *scale_ring = staging + kPStagingBytes;
  uint64_t *bars = (uint64_t *)(scale_ring + SD * kSlotBytes);
  uint64_t *full = bars, *empty = full + S, *sfs_full = empty + S, *sfs_empty = sfs_full + SD, *tmem_full = sfs_empty + SD,
           *tmem_empty = tmem_full + 1;
  uint32_t *tmem_slot = (uint32_t *)(tmem_empty + 1);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)cluster_ctarank();
  const int xm = g.xm, yn = g.yn, ktiles = g.ktiles;
  const int tiles_x = (xm + 255) / 256, nfull = g.nfull, ntiles = nfull + g.nhalf;
  const int tile_first = blockIdx.x >> 1, tile_step = gridDim.x >> 1;
  const int nk = (g.k + 255) / 256;
  const int my_tiles = tile_first < ntiles ? (ntiles - tile_first + tile_step - 1) / tile_step : 0;
  const int total = my_tiles * nk;
  unsigned *const status_word = g.status;

  // The set-up touches no global memory: under programmatic dependent launch it runs while the stream's previous kernel drains.
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&full[s], 9); mbar_init(&empty[s], 1); }
    for (int q = 0; q < SD; ++q) { mbar_init(&sfs_full[q], 1); mbar_init(&sfs_empty[q], 4); }
    mbar_init(tmem_full, 1);
    mbar_init(tmem_empty, 16);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_x);
    prefetch_tensormap(&tmap_y);
    prefetch_tensormap(&tmap_y64);
    prefetch_tensormap(&tmap_sx);
    prefetch_tensormap(&tmap_sy);
    prefetch_tensormap(&tmap_d);
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, 512);
  tc_fence_before();
  cluster_sync_all();   // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();   // from here on the previous kernel has completed and its writes are visible

  const unsigned tag = g.tag;
  auto wait = [abort_flag, status_word, tag](uint64_t *bar, uint32_t parity, unsigned code) -> bool {
    if (mbar_try(bar, parity)) return true;   // the common case: no flag read, no clock read
    if (*abort_flag) return false;
    if (mbar_wait(bar, parity)) return true;
    *abort_flag = 1;
    atomicCAS(status_word, 0u, code | tag);
    return false;
  };

  // The epilogue warps hold a 32 x 128 accumulator block in registers at once (so that the accumulator goes back to the MMA thread
  // after four loads, before any arithmetic); the registers come from the eight warps that need few.
  if (warp < 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
  if (warp == 0) {
    // ---------------- operand producer ----------------
    // The stage's two nibble tiles: this CTA's 128 rows of the M side, and its half of the tile's N-side rows (128 of 256, or 64
    // of 128).  Bytes of both CTAs count on the even CTA's barrier, whose MMA warp reads both CTAs' shared memory.  The whole warp
    // runs the loop and one elected lane issues (see tma_load_3d_pair_elect).
    const bool x_image = g.x_image, y_image = g.y_image;
    int t = tile_first, ks = 0;
    const CUtensorMap *map_y = &tmap_y;
    int x_tile = 0, y_tile = 0, y_row = 0;   // 128-row tile of each operand and, for the N side, the first row inside it
    uint32_t stage_bytes = 0;
    auto tile_setup = [&]() {
      const PairTile p = pair_tile(t, tiles_x, nfull);
      stage_bytes = 2u * (kXBytes + p.width * 64);
      x_tile = 2 * p.tx + rank;
      if (p.width == 256) { map_y = &tmap_y; y_tile = p.y128 + rank; y_row = 0; }
      else { map_y = &tmap_y64; y_tile = p.y128; y_row = rank * 64; }
    };
    if (total > 0) tile_setup();
    for (int it = 0; it < total; ++it) {
      const int s = it % S;
      if (!__all_sync(0xFFFFFFFFu, wait(&empty[s], ((it / S) & 1) ^ 1, kPStatEmpty))) break;
      if (rank == 0) mbar_arrive_expect_tx_elect(&full[s], stage_bytes);
      const uint32_t dst = smem_u32(smem + (size_t)s * kPStage), bar = mbar_addr_rank(&full[s], 0);
      if (x_image) tma_load_3d_pair_elect(dst, &tmap_x, 0, 0, x_tile * ktiles + ks, bar);
      else tma_load_3d_pair_elect(dst, &tmap_x, ks * 128, x_tile * 128, 0, bar);
      if (y_image) tma_load_3d_pair_elect(dst + kXBytes, map_y, 0, y_row, y_tile * ktiles + ks, bar);
      else tma_load_3d_pair_elect(dst + kXBytes, map_y, ks * 128, y_tile * 128 + y_row, 0, bar);
      if (++ks == nk) { ks = 0; t += tile_step; tile_setup(); }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA) ----------------
    // The WHOLE warp runs this loop and one elected lane issues each instruction: descriptors, tensor memory addresses and loop
    // state then stay on the uniform datapath, from which tcgen05 instructions take their operands.  Issued from inside a
    // one-lane branch, every MMA costs about 150 cycles whatever its shape (measured with nvfp4a_b200_mma_ceiling) -- more than
    // the 128 cycles the tensor pipe needs for 128 x 256 x 64.
    if (rank == 0) {
      const uint64_t da0 = smem_desc_sw128(smem_u32(smem));
      int it = 0;
      for (int tile_i = 0; tile_i < my_tiles; ++tile_i) {
        const int width = pair_tile(tile_first + tile_i * tile_step, tiles_x, nfull).width;
        const uint32_t idesc = idesc_mxf4nvf4(256, width), sfb_step = (uint32_t)width >> 5;
        if (!__all_sync(0xFFFFFFFFu, wait(tmem_empty, (tile_i & 1) ^ 1, kPStatTmemEmpty))) goto done;
        tc_fence_after();
        for (int ks = 0; ks < nk; ++ks, ++it) {
          const int s = it % S;
          const uint32_t par = (it / S) & 1;
          // one barrier per stage: the operand bytes of both CTAs and the eight scale warps' arrivals (scales in tensor memory)
          if (!__all_sync(0xFFFFFFFFu, wait(&full[s], par, kPStatFull))) goto done;
          tc_fence_after();
          const uint64_t da = da0 + (uint32_t)s * (uint32_t)(kPStage >> 4), db = da + (kXBytes >> 4);
          const uint32_t sfa = tmem_base + kPAccCols + s * kPSfCols;
          // the stage's four MMAs (64 values of k each: 32 bytes further along every 128-byte row) and the commit that frees stage s
          // and scale buffer s in both CTAs once they have been read
          mma4_commit_pair_elect(tmem_base, da, db, idesc, sfa, sfa + 16, sfb_step, (uint32_t)(ks != 0), &empty[s]);
        }
        tc_commit_pair_elect(tmem_full);
      }
    }
  } else if (warp == 2 || warp == 3) {
    // ---------------- scale producers ----------------
    // Per stage: the scale tiles of this CTA's 128 M-side rows (lane 0) and those of ALL of the tile's N-side rows (lanes 1, 2: every
    // CTA needs them in its tensor memory), one TMA instruction of up to three lanes; a box is the four 512-byte tiles of 256 values
    // of k.  The ring has its own slots and barriers, so the scales run several stages ahead of the operands and their trip
    // through registers into tensor memory costs the MMAs nothing.  Issuing a TMA instruction occupies a warp for a few hundred
    // cycles, so two warps take alternate stages.
    const bool image = lane == 0 ? g.x_image : g.y_image;
    const CUtensorMap *const map = lane == 0 ? &tmap_sx : &tmap_sy;
    for (int it = warp - 2; it < total; it += 2) {
      const int q = it % SD, ks = it % nk;
      const PairTile p = pair_tile(tile_first + (it / nk) * tile_step, tiles_x, nfull);
      const int boxes = 1 + p.width / 128, row_tile = lane == 0 ? 2 * p.tx + rank : p.y128 + lane - 1;
      if (!wait(&sfs_empty[q], ((it / SD) & 1) ^ 1, kPStatScale)) break;
      if (lane == 0) mbar_arrive_expect_tx(&sfs_full[q], 2048u * boxes);
      __syncwarp();
      if (lane < boxes) {
        const uint32_t dst = smem_u32(scale_ring + q * kSlotBytes) + 2048 * lane, bar = mbar_addr_rank(&sfs_full[q], rank);
        if (image) tma_load_3d_pair(dst, map, 0, row_tile * ktiles + ks, 0, bar);
        else tma_load_3d_pair(dst, map, ks * 256, row_tile, 0, bar);
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ---------------- scale warps ----------------
    // A 512-byte tile's 16 bytes at offset 16 l are what lane l of every quadrant holds in four scale columns; each of the four
    // warps writes its own quadrant.  Buffer s of tensor memory is free when the MMAs of the stage's previous round are done.
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    int ks = 0, tile_i = 0;
    bool wide = total > 0 && pair_tile(tile_first, tiles_x, nfull).width == 256;
    for (int it = 0; it < total; ++it) {
      const int q = it % SD, s = it % S;
      if (!wait(&sfs_full[q], (it / SD) & 1, kPStatScale)) break;
      const uint8_t *src = scale_ring + q * kSlotBytes + lane * 16;
      if (!wait(&empty[s], ((it / S) & 1) ^ 1, kPStatScale)) break;   // scale buffer s: the MMAs of the stage's previous round have read it
      tc_fence_after();
      const uint32_t sf = tmem_base + kPAccCols + s * kPSfCols + lane_base;
      // groups of four 512-byte tiles -> 16 scale columns each: the M side's; then the N side's -- 256 rows: k groups 0-1 and 2-3, per
      // 64 values of k [rows 0-127: 4 columns | rows 128-255: 4 columns]; 128 rows: the four k groups, 4 columns each
#pragma unroll
      for (int part = 0; part < 3; ++part) {
        if (part == 2 && !wide) break;
        uint32_t r[16];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int off = part == 0 ? c * 512 : wide ? 2048 + (c & 1) * 2048 + (2 * (part - 1) + (c >> 1)) * 512 : 2048 + c * 512;
          const uint4 v = *(const uint4 *)(src + off);
          r[4 * c] = v.x; r[4 * c + 1] = v.y; r[4 * c + 2] = v.z; r[4 * c + 3] = v.w;
        }
        tmem_st16(sf + 16 * part, r);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sfs_empty[q]);
      if (lane == 0) mbar_arrive_rank(&full[s], 0);
      if (++ks == nk) { ks = 0; ++tile_i; wide = pair_tile(tile_first + tile_i * tile_step, tiles_x, nfull).width == 256; }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 168;");
    // ---------------- epilogue ----------------
    const int ew = warp - 8, quad = ew & 3, half = ew >> 2;
    uint8_t *const box = staging + ew * 4096, *const row = box + lane * 128;
    const int sw = lane & 7;
    const float *const g_tok = g.g_tok;
    const int g_tok_stride = g.g_tok_stride, d_dtype = g.d_dtype;
    const float gf = g.gf, s_uniform = __fmul_rn(g.alpha, g.g_w ? g.g_w[0] : 1.f);
    float *const amax_out = g.amax;
    const uint32_t acc_lanes = tmem_base + ((uint32_t)(quad * 32) << 16);
    float amax = 0.f;
    int tile_i = 0;
    for (int t = tile_first; t < ntiles; t += tile_step, ++tile_i) {
      const PairTile p = pair_tile(t, tiles_x, nfull);
      const bool wide = p.width == 256;          // this warp's block: 128 columns of a 256-wide tile, 64 of a 128-wide one
      const int tok0 = p.tx * 256 + rank * 128 + quad * 32, tok = tok0 + lane, col0 = p.y128 * 128 + half * (p.width >> 1);
      const uint32_t acc_addr = acc_lanes + half * (p.width >> 1);
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
      uint32_t r0[32], r1[32], r2[32], r3[32];
      tmem_ld32(acc_addr, r0);
      tmem_ld32(acc_addr + 32, r1);
      if (wide) {
        tmem_ld32(acc_addr + 64, r2);
        tmem_ld32(acc_addr + 96, r3);
      }
      tmem_ld_wait();
      // every column of this warp's block is in registers: the accumulator goes back to the MMA thread
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_rank(tmem_empty, 0);
      box_free();
      stage32(r0, 0);
      stage32(r1, 4);
      store_box(col0);
      if (wide) {
        box_free();
        stage32(r2, 0);
        stage32(r3, 4);
        store_box(col0 + 64);
      }
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
  a.tag = next_launch_tag();
  CUtensorMap tx, ty, ty64, tsx, tsy, td;
  auto nibble_map = [&](const Fp4Operand &o, int rows, int box_rows, CUtensorMap *tn) {
    if (o.image) return make_tmap_bytes(tn, o.data, 128, 128, 128, box_rows, (uint64_t)((rows + 127) / 128) * a.ktiles, kImgTileBytes);
    return make_tmap_bytes(tn, o.data, (uint64_t)g.k / 2, (uint64_t)rows, (uint64_t)o.ld / 2, box_rows, 1, (uint64_t)o.ld / 2 * rows);
  };
  auto scale_map = [&](const Fp4Operand &o, int rows, CUtensorMap *ts) {
    if (o.image) return make_tmap_scales(ts, (const uint8_t *)o.data + kImgDataBytes, 2048, (uint64_t)((rows + 127) / 128) * a.ktiles, kImgTileBytes);
    const uint64_t tile_row_bytes = (uint64_t)((-o.sld) >> 2) * 512;
    return make_tmap_scales(ts, o.sc, tile_row_bytes, (uint64_t)(rows + 127) / 128, tile_row_bytes);
  };
  if (!nibble_map(X, a.xm, 128, &tx) || !nibble_map(Y, a.yn, 128, &ty) || !nibble_map(Y, a.yn, 64, &ty64) || !scale_map(X, a.xm, &tsx) ||
      !scale_map(Y, a.yn, &tsy))
    return cudaErrorInvalidValue;
  if (!make_tmap_dense(&td, g.e.d, 2, (uint64_t)g.m, (uint64_t)g.n, (uint64_t)g.e.ldd * 2, 64, 32, 128)) return cudaErrorInvalidValue;
  static std::atomic<unsigned long long> attr_set{0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(attr_set.load() >> (dev & 63) & 1)) {
    const cudaError_t e = cudaFuncSetAttribute(gemm_w4a4_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem);
    if (e != cudaSuccess) return e;
    attr_set.fetch_or(1ull << (dev & 63));
  }
  // The 256-wide tiles that would occupy at most half of the SM pairs in the last round are cut into two 128-wide halves each.
  const int tiles256 = ((a.xm + 255) / 256) * ((a.yn + 255) / 256), pairs = device_sms() / 2;
  const int rest = tiles256 % pairs, cut = (tiles256 > pairs && rest > 0 && 2 * rest <= pairs) ? rest : 0;
  a.nfull = tiles256 - cut; a.nhalf = 2 * cut;
  const int tiles = a.nfull + a.nhalf;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = dim3(2 * (tiles < pairs ? tiles : pairs), 1, 1);
  cfg.blockDim = dim3(kPairThreads, 1, 1);
  cfg.dynamicSmemBytes = kPairSmem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, gemm_w4a4_pair_kernel, tx, ty, ty64, tsx, tsy, td, a);
}

}  // namespace nvb




