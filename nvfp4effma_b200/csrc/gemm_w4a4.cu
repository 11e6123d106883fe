// The single-CTA W4A4 kernel: the route for what the CTA-pair kernel (gemm_w4a4_pair.cu, the default for large problems with a
// 16-bit D and tiled scales) does not take -- FP32 D, beta * C, bias, per-row globals, linear or unaligned block scales, small
// shapes.  (The PAIR template parameter of this file predates that kernel and is no longer instantiated.)
//
// NVFP4 x NVFP4 (W4A4) GEMM on the 5th-generation tensor cores: tcgen05.mma kind::mxf4nvf4 with 1 x 16 UE4M3 block scales
// (scale_vec::4X), FP32 accumulators in tensor memory, operands fed by TMA through a multi-stage mbarrier ring, persistent
// tile scheduling, epilogue (global scales, bias, beta * C, amax, output rounding) straight out of tensor memory.
//
// Tile: 128 rows of A (weight rows = MMA M) x BN rows of B (tokens = MMA N) x 256 values of k per stage.  A stage in shared
// memory is [A nibbles 16 KiB | B nibbles BN * 128 B | A scales 2 KiB | B scales BN * 16 B]: one 128-byte row per operand
// row (the TMA 128-byte swizzle), and the scales as 512-byte 128 x 4 tiles -- the cuBLASLt "swizzled" layout, which is what
// tcgen05.cp.32x128b.warpx4 copies into the scale columns of tensor memory unchanged.
//
// Warp roles (320 threads): warp 0 issues the copies of an iteration as ONE TMA instruction (lanes 0-5 name the nibble and
// scale tensors, see the producer); warp 1 lane 0 issues tcgen05.mma (and tcgen05.cp for gathered scales) and warp 1 owns
// the tensor memory allocation; warps 2-5 drain accumulators (one 32-lane quadrant each); warps 6-9 move the stage's
// scale tiles from shared memory through registers into the scale columns of tensor memory (tcgen05.st, off the MMA
// issuer's queue) -- or, for block scales that are not stored as aligned 512-byte tiles (linear layout, unaligned
// buffers), gather them into the tile form, one stage each in rotation.  Every wait is bounded; a wait that gives up
// raises the CTA's abort flag and the kernel status word.
//
// What the single-thread roles cost sets the pace of this kernel: a TMA instruction costs its issuing warp 150-200 cycles
// whatever it moves, and a tcgen05.mma about as much, so an iteration has one of the former and four of the latter
// (k = 64 is the largest MMA of this kind), and nothing else on those threads' paths that can be avoided.
//
// Semantics (reference include/nvfp4effma.h:78-92): the reference's tiled kernels round once per 16-block in FP32; the
// tensor cores accumulate the same exact block products in their own order, so results agree within the FP32
// accumulation bound the reference applies to its own tensor-core path (tests/test_util.h:292-302 there).
// Block scales are consumed as UNSIGNED E4M3: codes with the sign bit set are outside this kernel's contract (the
// reference's quantizer never emits them).
#include <atomic>
#include "operands.cuh"
#include "sm100.cuh"

namespace nvb {

using namespace sm100;

struct W4A4Args {
  int m, n, k;
  int a_image, b_image;        // operand is an image (3-D tensor map, scales inside the image)
  const uint8_t *sa, *sb;      // plain: block scale base; image: image base
  int sa_ld, sb_ld;            // plain: ScalePos ld
  int sa_gather, sb_gather;    // 1: scale warps gather (linear layout / unaligned); 0: 512-byte tiles by bulk copy
  int ktiles;                  // image: 256-k tiles per row tile
  Epilogue e;
  unsigned *status;
  unsigned tag;                // this launch's tag in the status word
  int transposed;              // the operands were swapped: TMEM lanes are tokens (B of the call), columns are A's rows
  int d_tma;                   // D is stored by TMA from a shared-memory staging tile (needs 16-byte aligned D and column stride)
};

template <int BN, int ACC, int STAGES, bool PAIR = false>
struct W4A4Cfg {
  // PAIR: a CTA holds 128 rows of A, HALF of the tile's B rows, and the scales of its A rows and of all BN rows of B
  // A pair keeps the scale tiles out of the stages, in a ring of kScaleSlots slots of their own that the producer fills
  // several iterations ahead of the operands (the scales' trip through registers into tensor memory then costs the MMA
  // nothing), and kSfBuffers scale buffers in tensor memory instead of one per stage.
  static constexpr int kABytes = 128 * 128, kBBytes = (PAIR ? BN / 2 : BN) * 128, kSfaBytes = 2048, kSfbBytes = BN * 16;
  static constexpr int kStageBytes = kABytes + kBBytes + (PAIR ? 0 : kSfaBytes + kSfbBytes);
  static constexpr int kScaleSlots = PAIR ? 8 : 0, kScaleLead = 4, kScaleSlotBytes = kSfaBytes + kSfbBytes;
  static constexpr int kSfCols = 16 + BN / 8;      // per scale buffer: A 4 groups x 4 columns, B 4 groups x BN / 32 columns
  static constexpr int kSfBuffers = PAIR ? 5 : STAGES;   // single CTA: one per pipeline stage
  static constexpr int kAccCols = ACC * BN;
  static constexpr int kTmemCols = 512;
  static constexpr int kStagingBytes = 8192;       // epilogue staging: 128 rows x 32 (16-bit) or 16 (32-bit) columns
  static constexpr int kBarrierBytes = 512;
  static constexpr int kRingBytes = STAGES * kStageBytes + kScaleSlots * kScaleSlotBytes;
  static constexpr int kSmemBytes = kRingBytes + 1024 /* alignment slack */ + kBarrierBytes + kStagingBytes;
  static_assert((2 * STAGES + 2 * kSfBuffers + 2 * kScaleSlots + 2 * ACC) * 8 + 8 <= kBarrierBytes, "barrier block");
  static_assert(kSmemBytes <= 232448, "shared memory budget");
  static_assert(kAccCols + kSfBuffers * kSfCols <= kTmemCols, "tensor memory budget");
};

constexpr int kThreads = 448;
constexpr unsigned kStatusWaitFull = 0x101, kStatusWaitEmpty = 0x102, kStatusWaitTmemFull = 0x103, kStatusWaitTmemEmpty = 0x104,
                   kStatusWaitGather = 0x105, kStatusWaitSf = 0x106;

// PAIR: the two CTAs of a cluster work on one 256 x BN tile with tcgen05.mma.cta_group::2 -- each CTA loads its 128 rows of A
// and half of the B rows, so a CTA pulls a third less through L2 per output than alone.  Each CTA runs its own TMA ring and
// scale warps against its own `full` barriers and drains its own half of the accumulator; what crosses the pair: the scale
// warps and the epilogue warps of both CTAs arrive on the even CTA's `sf_ready` / `tmem_empty` barriers (its MMA thread is
// the only issuer), and the MMA commits arrive on `empty` / `tmem_full` in both CTAs.  PAIR takes tiled scales only.
template <int BN, int ACC, int STAGES, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
gemm_w4a4_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_sa, const __grid_constant__ CUtensorMap tmap_sb,
                 const __grid_constant__ CUtensorMap tmap_d, const W4A4Args g) {
  using Cfg = W4A4Cfg<BN, ACC, STAGES, PAIR>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int NSF = Cfg::kSfBuffers, SD = Cfg::kScaleSlots;
  uint8_t *scale_ring = smem + STAGES * Cfg::kStageBytes;
  uint64_t *bars = (uint64_t *)(smem + Cfg::kRingBytes);
  uint64_t *full = bars, *empty = bars + STAGES, *sf_ready = bars + 2 * STAGES, *sf_free = sf_ready + NSF, *sfs_full = sf_free + NSF,
           *sfs_empty = sfs_full + SD, *tmem_full = sfs_empty + SD, *tmem_empty = tmem_full + ACC;
  uint32_t *tmem_slot = (uint32_t *)(tmem_empty + ACC);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
  uint8_t *staging = smem + Cfg::kRingBytes + Cfg::kBarrierBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gm = g.m, gn = g.n, gk = g.k, ktiles = g.ktiles;
  const bool a_image = g.a_image, b_image = g.b_image, sa_gather = g.sa_gather, sb_gather = g.sb_gather, d_tma = g.d_tma;
  const bool transposed = g.transposed;
  const uint8_t *const sa_base = g.sa, *const sb_base = g.sb;
  const int sa_ld = g.sa_ld, sb_ld = g.sb_ld;
  // tiles_m counts row tiles of 128 (256 for a pair, whose CTA `rank` takes the 128-row tile 2 * (t % tiles_m) + rank)
  const int rank = PAIR ? (int)cluster_ctarank() : 0;
  const int tiles_m = PAIR ? (gm + 255) / 256 : (gm + 127) / 128, tiles_n = (gn + BN - 1) / BN, ntiles = tiles_m * tiles_n;
  const int tile_first = PAIR ? blockIdx.x >> 1 : blockIdx.x, tile_step = PAIR ? gridDim.x >> 1 : gridDim.x;
  const int nk = (gk + 255) / 256;
  const bool any_gather = !PAIR && (sa_gather || sb_gather);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], any_gather ? 2 : 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < NSF; ++b) { mbar_init(&sf_ready[b], PAIR ? 8 : 4); mbar_init(&sf_free[b], 1); }
    for (int q = 0; q < SD; ++q) { mbar_init(&sfs_full[q], 1); mbar_init(&sfs_empty[q], 4); }
    for (int a = 0; a < ACC; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], PAIR ? 16 : 8); }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    if (PAIR) tmem_alloc_pair(tmem_slot, Cfg::kTmemCols);
    else tmem_alloc(tmem_slot, Cfg::kTmemCols);
  }
  tc_fence_before();
  if (PAIR) cluster_sync_all();   // the peer's barriers are initialised before anything arrives on them
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Kernel parameters are copied into registers here: a parameter struct whose members are reached through references
  // is re-read from parameter memory (hundreds of cycles) at every use inside the loops below.
  unsigned *const status_word = g.status;
  const unsigned tag = g.tag;
  // wait that also ends when another role has raised the abort flag
  auto wait = [abort_flag, status_word, tag](uint64_t *bar, uint32_t parity, unsigned code) -> bool {
    if (mbar_try(bar, parity)) return true;   // the common case: no flag read, no clock read
    if (*abort_flag) return false;
    if (mbar_wait(bar, parity)) return true;
    *abort_flag = 1;
    atomicCAS(status_word, 0u, code | tag);
    return false;
  };

  if (warp == 0) {
    // ---------------- producer: one TMA instruction per iteration ----------------
    // Issuing a copy instruction costs the issuing warp more than a hundred cycles whatever it moves, so every copy of an
    // iteration -- A and B nibbles, and the 2 KiB scale tiles, which are tensors of their own ([row tile][k] of 8-byte
    // words; a box is the four 512-byte tiles of 256 values of k, zero-filled past k) -- is issued by ONE instruction whose
    // lanes name different tensor maps, coordinates, destinations and barriers:
    //   lane 0: A nibbles; lanes 1, 2: B nibbles (lane 2: the second 128 rows when B is an image and a CTA holds 256 of
    //   them); lane 3: A scales; lanes 4, 5: B scales of the tile's two 128-row halves.
    // Single CTA: the scale tiles land in the stage, counted on `full` with the nibbles.  Pair: the nibbles of both CTAs
    // count on the even CTA's `full`; the scale tiles go to the scale ring, kScaleLead iterations ahead of the nibbles.
    {
      const int my_tiles = tile_first < ntiles ? (ntiles - tile_first + tile_step - 1) / tile_step : 0;
      const int total = my_tiles * nk;
      const bool scale_lane = lane >= 3 && lane < 6, copy_lane = lane < 6;
      const bool for_a = lane == 0 || lane == 3;
      const int part = lane < 3 ? lane - 1 : lane - 4;               // B: which 128-row part this lane serves
      const bool image = for_a ? a_image : b_image;
      const CUtensorMap *const map = lane == 0 ? &tmap_a : lane < 3 ? &tmap_b : lane == 3 ? &tmap_sa : &tmap_sb;
      const int lead = (PAIR && scale_lane) ? Cfg::kScaleLead : 0;   // this lane's copies run `lead` iterations ahead
      const uint32_t nibble_bytes = Cfg::kABytes + Cfg::kBBytes;
      // this lane's cursor: iteration l_it = (tile l_t, k step l_ks), and what the tile fixes: is there a copy, its row / tile coordinates
      int l_it = 0, l_t = tile_first, l_ks = 0;
      bool live = false;
      int y0 = 0, z0 = 0;
      uint32_t dst_off = 0;
      int n_sf = 0;   // lane 0: scale tiles per iteration of the tile (for the byte count)
      auto tile_setup = [&]() {
        const int tm = PAIR ? 2 * (l_t % tiles_m) + rank : l_t % tiles_m, tn = l_t / tiles_m;
        const bool a_live = tm * 128 < gm;   // a pair's second row tile may lie past m: zero nibbles, no scales to fetch
        live = false; y0 = 0; z0 = 0;
        if (lane == 0) { live = true; dst_off = 0; if (image) z0 = tm * ktiles; else y0 = tm * 128; }
        else if (lane < 3) {
          if (PAIR) { live = part == 0; dst_off = Cfg::kABytes; if (image) z0 = (tn * (BN / 128) + rank) * ktiles; else y0 = tn * BN + rank * (BN / 2); }
          else if (image) { live = part < BN / 128; dst_off = Cfg::kABytes + part * 16384; z0 = (tn * (BN / 128) + part) * ktiles; }
          else { live = part == 0; dst_off = Cfg::kABytes; y0 = tn * BN; }
        } else if (scale_lane) {
          const int rt = for_a ? tm : tn * (BN / 128) + part;
          live = for_a ? (!sa_gather && a_live) : (!sb_gather && part < BN / 128 && rt * 128 < gn);
          dst_off = (PAIR ? 0 : Cfg::kABytes + Cfg::kBBytes) + (for_a ? 0 : Cfg::kSfaBytes + part * 2048);
          y0 = image ? rt * ktiles : rt;   // image: one row of the scale tensor per (row tile, k tile); plain: per row tile
        }
        n_sf = 0;
        if (!sa_gather && a_live) ++n_sf;
        if (!sb_gather)
          for (int h = 0; h < BN / 128; ++h) n_sf += tn * BN + h * 128 < gn;
      };
      if (total > 0) tile_setup();
      // the scale lanes of a pair start `lead` iterations early: iterations it < 0 issue scale tiles only
      for (int it = PAIR ? -Cfg::kScaleLead : 0; it < total; ++it) {
        const int s = it % STAGES;
        bool okw = true;
        if (it >= 0) okw = wait(&empty[s], ((it / STAGES) & 1) ^ 1, kStatusWaitEmpty);
        const int sj = it + Cfg::kScaleLead, slot = PAIR ? sj % (SD ? SD : 1) : 0;   // pair: the scale iteration issued now
        const bool scales_now = PAIR && sj < total;
        if (scales_now) okw = okw && wait(&sfs_empty[slot], ((sj / (SD ? SD : 1)) & 1) ^ 1, kStatusWaitEmpty);
        if (!__all_sync(0xFFFFFFFFu, okw)) goto done;
        if (lane == 0) {
          if (PAIR) {
            if (it >= 0 && rank == 0) mbar_arrive_expect_tx(&full[s], 2 * nibble_bytes);
          } else {
            mbar_arrive_expect_tx(&full[s], nibble_bytes + n_sf * 2048);
          }
        }
        if (PAIR && lane == 3 && scales_now) {
          // lane 3's cursor stands at iteration sj: its tile's scale tile count (A's may be missing past m)
          mbar_arrive_expect_tx(&sfs_full[slot], n_sf * 2048);
        }
        __syncwarp();
        const bool mine = copy_lane && live && (lead ? scales_now : it >= 0);
        if (mine) {
          uint32_t dst, bar;   // pair: barrier addresses in the cluster's window (the nibbles' in the even CTA, the scales' here)
          if (PAIR && scale_lane) {
            dst = smem_u32(scale_ring + slot * Cfg::kScaleSlotBytes + dst_off);
            bar = mbar_addr_rank(&sfs_full[slot], rank);
          } else {
            dst = smem_u32(smem + (size_t)s * Cfg::kStageBytes + dst_off);
            bar = PAIR ? mbar_addr_rank(&full[s], 0) : smem_u32(&full[s]);
          }
          int x, y, z;
          if (scale_lane) { x = image ? 0 : l_ks * 256; y = image ? y0 + l_ks : y0; z = 0; }
          else { x = image ? 0 : l_ks * 128; y = y0; z = image ? z0 + l_ks : 0; }
          if (PAIR) tma_load_3d_pair(dst, map, x, y, z, bar);
          else tma_load_3d_at(dst, map, x, y, z, bar);
        }
        // advance this lane's cursor (scale lanes of a pair run from iteration 0 while it < 0 ... they start at l_it = 0 when it = -lead)
        if (lead ? scales_now : it >= 0) {
          ++l_it;
          if (++l_ks == nk) { l_ks = 0; l_t += tile_step; if (l_it < total) tile_setup(); }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = idesc_mxf4nvf4(PAIR ? 256 : 128, BN);
      const uint32_t smem0 = smem_u32(smem);
      const uint64_t da0 = smem_desc_sw128(smem0);
      const int nfull = gk / 256;   // iterations with all four 64-value groups
      uint32_t it = 0, tile_i = 0;
      for (int t = tile_first; t < ntiles; t += tile_step, ++tile_i) {
        const int acc = tile_i % ACC;
        bool okw;
        okw = wait(&tmem_empty[acc], ((tile_i / ACC) & 1) ^ 1, kStatusWaitTmemEmpty);
        if (!okw) goto done;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int ks = 0; ks < nk; ++ks, ++it) {
          const int s = it % STAGES;
          // tiled scales: four warps have put the stage's scale columns into tensor memory (which implies the operands landed);
          // gathered scales: this thread copies them from shared memory itself
          const int b = PAIR ? it % NSF : s;   // scale buffer in tensor memory
          if (PAIR) okw = wait(&full[s], (it / STAGES) & 1, kStatusWaitFull) && wait(&sf_ready[b], (it / NSF) & 1, kStatusWaitSf);
          else okw = any_gather ? wait(&full[s], (it / STAGES) & 1, kStatusWaitFull) : wait(&sf_ready[s], (it / STAGES) & 1, kStatusWaitSf);
          if (!okw) goto done;
          tc_fence_after();
          // descriptors of a stage = those of stage 0 plus the stage's offset in the address field's 16-byte units
          const uint64_t da = da0 + (uint32_t)s * (uint32_t)(Cfg::kStageBytes >> 4), db = da + (Cfg::kABytes >> 4);
          const uint32_t sf_tmem = tmem_base + Cfg::kAccCols + b * Cfg::kSfCols;
          const uint32_t sfa_tmem = sf_tmem, sfb_tmem = sf_tmem + 16;
          const uint32_t sSfa = smem0 + s * Cfg::kStageBytes + Cfg::kABytes + Cfg::kBBytes, sSfb = sSfa + Cfg::kSfaBytes;   // gathered scales only
          const int ng = ks < nfull ? 4 : (gk - ks * 256) / 64;
          // per 64 values of k: (the scale tiles of that group, then) its MMA, 32 bytes further along each 128-byte row
          if (!any_gather && ks < nfull) {   // the common iteration, straight-line: nothing but the four MMAs on this thread's path
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (PAIR) mma_mxf4nvf4_pair(d_tmem, da + 2 * j, db + 2 * j, idesc, sfa_tmem + 4 * j, sfb_tmem + (BN / 32) * j, j ? 1u : (uint32_t)(ks != 0));
              else mma_mxf4nvf4(d_tmem, da + 2 * j, db + 2 * j, idesc, sfa_tmem + 4 * j, sfb_tmem + (BN / 32) * j, j ? 1u : (uint32_t)(ks != 0));
            }
          } else
          for (int j = 0; j < ng; ++j) {
            if (any_gather) {
              tmem_cp_32x128b_warpx4(sfa_tmem + 4 * j, smem_desc_sf(sSfa + j * 512));
#pragma unroll
              for (int h = 0; h < BN / 128; ++h)
                tmem_cp_32x128b_warpx4(sfb_tmem + (BN / 32) * j + 4 * h, smem_desc_sf(sSfb + h * 2048 + j * 512));
            }
            if (PAIR) mma_mxf4nvf4_pair(d_tmem, da + 2 * j, db + 2 * j, idesc, sfa_tmem + 4 * j, sfb_tmem + (BN / 32) * j, (ks | j) != 0);
            else mma_mxf4nvf4(d_tmem, da + 2 * j, db + 2 * j, idesc, sfa_tmem + 4 * j, sfb_tmem + (BN / 32) * j, (ks | j) != 0);
          }
          if (PAIR) { tc_commit_pair(&empty[s]); tc_commit_pair(&sf_free[b]); }
          else tc_commit(&empty[s]);
        }
        if (PAIR) tc_commit_pair(&tmem_full[acc]);
        else tc_commit(&tmem_full[acc]);
      }
    }
  } else if (warp < 6 || warp >= 10) {
    // ---------------- epilogue: TMEM -> registers -> (staging tile -> TMA store | direct stores) ----------------
    // Two groups of four warps (2-5 and 10-13, one warp per 32-lane quadrant in each) take alternate 32-column chunks of the
    // accumulator, each with its own 4 KiB staging tile, named barrier and store-issuing lane: the groups' TMEM loads,
    // arithmetic, shared-memory stores and waits for the TMA unit overlap on the four schedulers.
    // Everything the loops need is held in plain locals (see the note on kernel parameters above).
    const int group = warp >= 10, bar_id = 1 + group;
    uint8_t *const stg = staging + group * 4096;
    const int quad = warp & 3;
    const float *const ga = g.e.ga, *const gb = g.e.gb;
    const int ga_stride = g.e.ga_stride, gb_stride = g.e.gb_stride;
    const float gf = g.e.gf, alpha = g.e.alpha, beta = g.e.beta;
    const void *const cptr = g.e.c, *const biasptr = g.e.bias;
    const int ldc = g.e.ldc, c_dtype = g.e.c_dtype, bias_dtype = g.e.bias_dtype;
    uint8_t *const dptr = (uint8_t *)g.e.d;
    const int ldd = g.e.ldd, d_dtype = g.e.d_dtype;
    float *const amax_out = g.e.amax;
    const int esz = dense_bytes(d_dtype);
    const int cw = esz == 2 ? 16 : 8;           // columns per staging round: 128 rows x cw columns = 4 KiB
    const bool leader = (warp == 2 || warp == 10) && lane == 0; // issues and tracks its group's TMA stores
    const bool fast = beta == 0.f && gb_stride == 0;  // one scale per lane, no C: the common case
    const float colp0 = (gb && !gb_stride) ? gb[0] : 1.f;
    float amax = 0.f;
    uint32_t tile_i = 0;
    for (int t = tile_first; t < ntiles; t += tile_step, ++tile_i) {
      const int tm = PAIR ? 2 * (t % tiles_m) + rank : t % tiles_m, tn = t / tiles_m, acc = tile_i % ACC;
      const int i = tm * 128 + quad * 32 + lane;
      const bool row_ok = i < gm;
      const float rowp = (row_ok && !transposed) ? __fmul_rn(alpha, ga ? ga[(size_t)i * ga_stride] : 1.f) : 0.f;
      const float bias = (row_ok && biasptr && !transposed) ? load_dense(bias_dtype, biasptr, i) : 0.f;
      const float s_lane = __fmul_rn(__fmul_rn(rowp, colp0), gf);
      // the four warps of a group decide together whether to go on: none may be left alone at a named barrier
      bool okw;
      okw = wait(&tmem_full[acc], (tile_i / ACC) & 1, kStatusWaitTmemFull);
      if (!okw) *abort_flag = 1;
      named_barrier(bar_id, 128);
      if (*abort_flag) goto done;
      tc_fence_after();
      const int nchunks = min(BN / 32, (gn - tn * BN + 31) / 32);
      // Swapped operands: this lane is token jt and the accumulator's columns are 32 consecutive rows of D, which lie side by
      // side in memory -- scaled, rounded, packed two to a word and staged with four 16-byte stores per lane (swizzled as the
      // TMA unit expects, so they meet no bank conflict), against 32 two-byte stores the other way round.  Every warp stages
      // and stores its own 32 tokens: no barrier between warps, eight independent store pipelines.
      const int jt = i;   // (the lane's index on the M side is a token here)
      const float tokp = (transposed && row_ok && gb) ? gb[(size_t)jt * gb_stride] : 1.f;
      const float ga0 = (ga && !ga_stride) ? ga[0] : 1.f;
      const bool fast_t = beta == 0.f && ga_stride == 0 && !biasptr;
      const float s_tok = __fmul_rn(__fmul_rn(__fmul_rn(alpha, ga0), tokp), gf);
      auto drain_t = [&](uint32_t (&r)[32], int c) {
        const int i0 = tn * BN + c * 32;
        const int nvalid = min(32, gn - i0);
        if (fast_t) {
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) r[jj] = __float_as_uint(__fmul_rn(__uint_as_float(r[jj]), s_tok));
        } else {
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) {
            const int ii = i0 + jj;
            const bool in = jj < nvalid;
            const float rp = __fmul_rn(alpha, (ga && in) ? ga[(size_t)ii * ga_stride] : 1.f);
            float v = __fmul_rn(__uint_as_float(r[jj]), __fmul_rn(__fmul_rn(rp, tokp), gf));
            if (biasptr && in) v = __fadd_rn(v, load_dense(bias_dtype, biasptr, ii));
            if (beta != 0.f && in && row_ok) v = __fmaf_rn(beta, load_dense(c_dtype, cptr, (size_t)jt * ldc + ii), v);
            r[jj] = __float_as_uint(v);
          }
        }
        if (amax_out && row_ok) {
#pragma unroll
          for (int jj = 0; jj < 32; ++jj)
            if (jj < nvalid) amax = fmaxf(amax, fabsf(__uint_as_float(r[jj])));
        }
        if (d_dtype == NVFP4A_BF16) {
          round32_to_bf16(r);
        } else {
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) r[jj] = (uint32_t)__half_as_ushort(__float2half_rn(__uint_as_float(r[jj])));
        }
        // every warp on its own: 32 tokens x 16 elements (1 KiB, 32-byte rows in the TMA unit's 32-byte swizzle) per store
        uint8_t *const mine = staging + (group * 4 + quad) * 1024, *const row = mine + lane * 32;
        const int sw = (lane >> 2) & 1;
#pragma unroll
        for (int rd = 0; rd < 2; ++rd) {
          if (lane == 0) bulk_wait_read_all();   // this warp's previous store has finished reading its staging tile
          __syncwarp();
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int b = rd * 16 + q * 8;
            *(uint4 *)(row + ((q ^ sw) << 4)) = make_uint4(r[b] | (r[b + 1] << 16), r[b + 2] | (r[b + 3] << 16), r[b + 4] | (r[b + 5] << 16),
                                                           r[b + 6] | (r[b + 7] << 16));
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmap_d, mine, i0 + rd * 16, tm * 128 + quad * 32);
            bulk_commit();
          }
        }
      };
      const int cstep = 2, cfirst = group;
      // The accumulator leaves tensor memory 32 columns at a time; the load of the next 32 is in flight while these are
      // scaled, rounded and staged (two register sets alternate).
      auto drain = [&](uint32_t (&r)[32], int c) {
        const int j0 = tn * BN + c * 32;
        const int nvalid = min(32, gn - j0);
        // values before rounding, kept in r[] as FP32 bits
        if (fast) {
          if (biasptr) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) r[jj] = __float_as_uint(__fadd_rn(__fmul_rn(__uint_as_float(r[jj]), s_lane), bias));
          } else {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) r[jj] = __float_as_uint(__fmul_rn(__uint_as_float(r[jj]), s_lane));
          }
        } else {
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) {
            const int j = j0 + jj;
            const bool ok = row_ok && jj < nvalid;
            const float colp = (gb_stride && jj < nvalid) ? gb[j] : colp0;
            float v = __fmul_rn(__uint_as_float(r[jj]), __fmul_rn(__fmul_rn(rowp, colp), gf));
            if (biasptr) v = __fadd_rn(v, bias);
            if (beta != 0.f && ok) v = __fmaf_rn(beta, load_dense(c_dtype, cptr, (size_t)j * ldc + i), v);
            r[jj] = __float_as_uint(v);
          }
        }
        if (amax_out && row_ok) {
#pragma unroll
          for (int jj = 0; jj < 32; ++jj)
            if (jj < nvalid) amax = fmaxf(amax, fabsf(__uint_as_float(r[jj])));
        }
        // rounding to the output type (in place, low bits of r[])
        if (d_dtype == NVFP4A_BF16) {
          round32_to_bf16(r);
        } else if (d_dtype == NVFP4A_FP16) {
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) r[jj] = (uint32_t)__half_as_ushort(__float2half_rn(__uint_as_float(r[jj])));
        }
        if (!d_tma) {  // plain stores: any alignment, any ldd
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
          return;
        }
        const int rr = quad * 32 + lane;
        auto round_begin = [&]() {
          if (leader) bulk_wait_read_all();   // the group's previous store has finished reading its staging tile
          named_barrier(bar_id, 128);
        };
        auto round_end = [&](int col) {
          fence_proxy_async_smem();
          named_barrier(bar_id, 128);
          if (leader) {
            tma_store_2d(&tmap_d, stg, tm * 128, col);
            bulk_commit();
          }
        };
        if (esz == 2) {
#pragma unroll
          for (int rd = 0; rd < 2; ++rd) {
            round_begin();
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) ((uint16_t *)stg)[jj * 128 + rr] = (uint16_t)r[rd * 16 + jj];
            round_end(j0 + rd * 16);
          }
        } else {
#pragma unroll
          for (int rd = 0; rd < 4; ++rd) {
            round_begin();
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) ((uint32_t *)stg)[jj * 128 + rr] = r[rd * 8 + jj];
            round_end(j0 + rd * 8);
          }
        }
      };
      const uint32_t acc_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
      auto release_acc = [&]() {  // every column is in registers: the MMA warp may start the next tile on this accumulator
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (PAIR) mbar_arrive_rank(&tmem_empty[acc], 0);
          else mbar_arrive(&tmem_empty[acc]);
        }
      };
      uint32_t ra[32], rb[32];
      // The accumulator goes back to the MMA thread as soon as the warp's last load has landed, before the chunks still in
      // registers are drained: a drain waits on the TMA unit between its stores.
      bool released = false;
      auto last_load = [&]() { tmem_ld_wait(); release_acc(); released = true; };
      if (cfirst < nchunks) {
        tmem_ld32(acc_addr + cfirst * 32, ra);
        if (cfirst + cstep >= nchunks) last_load();
      } else {
        release_acc();   // no chunk of this tile for the group
      }
      for (int c = cfirst; c < nchunks; c += 2 * cstep) {
        if (!released) tmem_ld_wait();
        if (c + cstep < nchunks) {
          tmem_ld32(acc_addr + (c + cstep) * 32, rb);
          if (c + 2 * cstep >= nchunks) last_load();
        }
        if (transposed) drain_t(ra, c);
        else drain(ra, c);
        if (c + cstep < nchunks) {
          if (!released) tmem_ld_wait();
          if (c + 2 * cstep < nchunks) {
            tmem_ld32(acc_addr + (c + 2 * cstep) * 32, ra);
            if (c + 3 * cstep >= nchunks) last_load();
          }
          if (transposed) drain_t(rb, c + cstep);
          else drain(rb, c + cstep);
        }
      }
    }
    if (lane == 0) bulk_wait_all();   // (a lane that issued no store has nothing to wait for)
    if (amax_out) warp_amax_commit(amax_out, amax);
  } else if (!any_gather) {
    // ---------------- scale warps: the stage's 512-byte scale tiles, shared memory -> registers -> tensor memory ----------------
    // A tile's 16 bytes at offset 16 l are what lane l of every quadrant holds in four scale columns (the layout
    // tcgen05.cp.32x128b.warpx4 would produce); each of the four warps writes its own quadrant, off the MMA issuer's queue.
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    uint32_t it = 0;
    for (int t = tile_first; t < ntiles; t += tile_step) {
      const bool a_live = !PAIR || (2 * (t % tiles_m) + rank) * 128 < gm;
      for (int ks = 0; ks < nk; ++ks, ++it) {
        // single CTA: the tiles came with stage s; pair: they lie in slot it % SD of the scale ring
        const int s = it % STAGES, slot = it % (SD ? SD : 1), b = PAIR ? it % NSF : s;
        if (PAIR ? !wait(&sfs_full[slot], (it / (SD ? SD : 1)) & 1, kStatusWaitGather) : !wait(&full[s], (it / STAGES) & 1, kStatusWaitGather)) goto done;
        const uint8_t *st = smem + (size_t)s * Cfg::kStageBytes;
        const uint8_t *sSfa = PAIR ? scale_ring + slot * Cfg::kScaleSlotBytes : st + Cfg::kABytes + Cfg::kBBytes, *sSfb = sSfa + Cfg::kSfaBytes;
        const uint32_t sf_tmem = tmem_base + Cfg::kAccCols + b * Cfg::kSfCols + lane_base;
        const int ng = min(4, (gk - ks * 256) / 64);
        uint4 va[4], vb[BN / 128][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) va[j] = (j < ng && a_live) ? *(const uint4 *)(sSfa + j * 512 + lane * 16) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int h = 0; h < BN / 128; ++h)
#pragma unroll
          for (int j = 0; j < 4; ++j) vb[h][j] = j < ng ? *(const uint4 *)(sSfb + h * 2048 + j * 512 + lane * 16) : make_uint4(0, 0, 0, 0);
        if (PAIR) {   // the slot is free again; the tensor memory buffer must have been read by the MMAs that last used it
          __syncwarp();
          if (lane == 0) mbar_arrive(&sfs_empty[slot]);
          if (!wait(&sf_free[b], ((it / NSF) & 1) ^ 1, kStatusWaitGather)) goto done;
          tc_fence_after();
        }
        uint32_t r[16];
#pragma unroll
        for (int j = 0; j < 4; ++j) { r[4 * j] = va[j].x; r[4 * j + 1] = va[j].y; r[4 * j + 2] = va[j].z; r[4 * j + 3] = va[j].w; }
        tmem_st16(sf_tmem, r);
#pragma unroll
        for (int part = 0; part < BN / 128; ++part) {   // B: group j occupies BN / 32 columns: [half 0: 4 | half 1: 4]
#pragma unroll
          for (int q = 0; q < 4; ++q) {                 // register quad q of this part = columns 4 q .. 4 q + 3 of the 16
            const int col = part * 16 + 4 * q, j = col / (BN / 32), h = (col % (BN / 32)) / 4;
            r[4 * q] = vb[h][j].x; r[4 * q + 1] = vb[h][j].y; r[4 * q + 2] = vb[h][j].z; r[4 * q + 3] = vb[h][j].w;
          }
          tmem_st16(sf_tmem + 16 + part * 16, r);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (PAIR) mbar_arrive_rank(&sf_ready[b], 0);
          else mbar_arrive(&sf_ready[s]);
        }
      }
    }
  } else {
    // ---------------- scale gather: linear / unaligned block scales -> 512-byte tiles in shared memory ----------------
    // Warp w of the four takes the pipeline iterations it % 4 == w, so four stages' loads are in flight together.
    const int w = warp - 6;
    const ScalePos pa{sa_ld}, pb{sb_ld};
    uint32_t it = 0;
    for (int t = tile_first; t < ntiles; t += tile_step) {
      const int tm = t % tiles_m, tn = t / tiles_m;
      for (int ks = 0; ks < nk; ++ks, ++it) {
        if ((int)(it & 3) != w) continue;
        const int s = it % STAGES;
        if (!wait(&empty[s], ((it / STAGES) & 1) ^ 1, kStatusWaitGather)) goto done;
        uint8_t *st = smem + (size_t)s * Cfg::kStageBytes;
        uint8_t *sSfa = st + Cfg::kABytes + Cfg::kBBytes, *sSfb = sSfa + Cfg::kSfaBytes;
        const int ng = min(4, (gk - ks * 256) / 64);
        // one 128-row tile: lane l owns rows l, l + 32, l + 64, l + 96; per 64-k group the four rows' words form 16 bytes
        auto gather_tile = [&](const uint8_t *sc, const ScalePos &p, int row0, int rows, uint8_t *dst) {
          uint32_t wd[4][4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int r = min(row0 + 32 * q + lane, rows - 1);
            const uint8_t *src = sc + p.row(r);
#pragma unroll
            for (int j = 0; j < 4; ++j) wd[q][j] = j < ng ? __ldg((const uint32_t *)(src + p.col(16 * ks + 4 * j))) : 0u;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) *(uint4 *)(dst + j * 512 + lane * 16) = make_uint4(wd[0][j], wd[1][j], wd[2][j], wd[3][j]);
        };
        if (sa_gather) gather_tile(sa_base, pa, tm * 128, gm, sSfa);
        if (sb_gather)
          for (int h = 0; h < BN / 128; ++h)
            if (tn * BN + h * 128 < gn) gather_tile(sb_base, pb, tn * BN + h * 128, gn, sSfb + h * 2048);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full[s]);
      }
    }
  }
done:
  __syncwarp();   // lanes that left a role's loop early rejoin their warp before the aligned barriers below
  tc_fence_before();
  if (PAIR) cluster_sync_all();   // neither CTA leaves (or frees tensor memory) while the other may still arrive on its barriers
  else __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    else tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ---- host ------------------------------------------------------------------------------------------------------------------
static __device__ unsigned int g_kernel_status;
static std::atomic<unsigned> g_launch_seq{0};
static thread_local unsigned g_last_launch = 0;
unsigned next_launch_tag() {
  g_last_launch = (g_launch_seq.fetch_add(1) + 1) & 0xFFFFFu;
  return g_last_launch << 12;
}
static std::atomic<long long> g_tp_wait_limit{2000000000ll};
long long tp_wait_limit() { return g_tp_wait_limit.load(); }
static std::atomic<int> g_pdl{1};
bool pdl_enabled() { return g_pdl.load() != 0; }
unsigned int *kernel_status_device_ptr() {
  unsigned int *p = nullptr;
  cudaGetSymbolAddress((void **)&p, g_kernel_status);
  return p;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}
bool make_tmap_bytes(CUtensorMap *map, const void *base, uint64_t row_bytes, uint64_t rows, uint64_t stride, uint32_t box_rows,
                     uint64_t tiles, uint64_t tile_stride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {row_bytes, rows, tiles ? tiles : 1};
  cuuint64_t strides[2] = {stride, tile_stride ? tile_stride : stride * rows};
  cuuint32_t box[3] = {128, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const cuuint32_t rank = tiles ? 3 : 2;
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, rank, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_tmap_dense(CUtensorMap *map, const void *base, int elem_bytes, uint64_t inner, uint64_t outer, uint64_t stride,
                     uint32_t box_inner, uint32_t box_outer, int swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {stride};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(base), dims, strides,
            box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : swizzle == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : swizzle == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Block scales in 512-byte tiles as a tensor of 8-byte words: `rows` rows (one per 128-row tile of the operand; one per
// image tile for an image) of row_bytes bytes, `stride` bytes apart; a box is 2 KiB of one row (the four tiles of 256
// values of k), zero-filled where it passes the end of the row.  Rank 3 like the nibble maps, so that one instruction
// can issue both.
bool make_tmap_scales(CUtensorMap *map, const void *base, uint64_t row_bytes, uint64_t rows, uint64_t stride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {row_bytes / 8, rows, 1};
  cuuint64_t strides[2] = {stride, stride * rows};
  cuuint32_t box[3] = {256, 1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_tmap_image_pair(CUtensorMap *map, const void *base, uint32_t rows, uint64_t ktiles, uint64_t tiles128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {128, rows, ktiles, tiles128};
  cuuint64_t strides[3] = {128, (cuuint64_t)kImgTileBytes, (cuuint64_t)kImgTileBytes * ktiles};
  cuuint32_t box[4] = {128, rows, 1, 2};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            rows == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool gemm_w4a4_supports(const GemmArgs &g) {
  return g.B.dtype == NVFP4A_NVFP4 && !g.A.ue && !g.B.q.ue && !g.x.mask && g.k >= 64 && encode_fn() != nullptr;
}

template <int BN, int ACC, int STAGES, bool PAIR>
static cudaError_t launch_cfg(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tsa, const CUtensorMap &tsb, const CUtensorMap &td,
                              const W4A4Args &a, cudaStream_t s) {
  using Cfg = W4A4Cfg<BN, ACC, STAGES, PAIR>;
  static std::atomic<bool> attr_set[64];   // zero-initialised; set once per device (a repeated cudaFuncSetAttribute is harmless)
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    const cudaError_t e = cudaFuncSetAttribute(gemm_w4a4_kernel<BN, ACC, STAGES, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set[dev & 63] = true;
  }
  if (PAIR) {   // clusters of two CTAs, one pair per 256 x BN tile in flight
    const int tiles = ((a.m + 255) / 256) * ((a.n + BN - 1) / BN), pairs = device_sms() / 2;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(2 * (tiles < pairs ? tiles : pairs), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemm_w4a4_kernel<BN, ACC, STAGES, PAIR>, ta, tb, tsa, tsb, td, a);
  }
  const int tiles = ((a.m + 127) / 128) * ((a.n + BN - 1) / BN);
  const int grid = tiles < device_sms() ? tiles : device_sms();
  gemm_w4a4_kernel<BN, ACC, STAGES, PAIR><<<grid, kThreads, Cfg::kSmemBytes, s>>>(ta, tb, tsa, tsb, td, a);
  return cudaGetLastError();
}

static std::atomic<int> g_w4a4_bn{0};  // 0 = choose by n; tests and tuning may pin 128 or 256 (nvfp4a_b200_set_tile_n)
void set_w4a4_tile_n(int bn) { g_w4a4_bn = bn; }
// -1 = automatic; 0 / 1 pin the CTA-pair kernel off / on where it applies (nvfp4a_b200_set_pair).  Automatic currently means
// off: at 4096^3 the pair form takes 64 us against 58 us (its producer warp, with two rings to feed, is the slower issuer).
static std::atomic<int> g_w4a4_pair{-1};
void set_w4a4_pair(int mode) { g_w4a4_pair = mode; }

static std::atomic<int> g_w4a4_swap{-1};  // 1: tokens on the MMA's M side whenever D can be stored that way; -1: unless that costs a round of tiles; 0: never
void set_w4a4_swap(int mode) { g_w4a4_swap = mode; }

bool gemm_w4a4_pair_applies(const GemmArgs &g, bool force);
cudaError_t launch_gemm_w4a4_pair(const GemmArgs &g, cudaStream_t s);

cudaError_t launch_gemm_w4a4(const GemmArgs &g, cudaStream_t s) {
  const int pin_bn = g_w4a4_bn.load(), pin_pair = g_w4a4_pair.load(), pin_swap = g_w4a4_swap.load();
  // large problems with a TMA-storable 16-bit D and tiled scales: the CTA-pair kernel (gemm_w4a4_pair.cu)
  if (pin_pair != 0 && pin_swap != 0 && !pin_bn && gemm_w4a4_pair_applies(g, pin_pair == 1)) return launch_gemm_w4a4_pair(g, s);
  W4A4Args a;
  memset(&a, 0, sizeof a);
  a.k = g.k;
  a.e = g.e;
  a.status = kernel_status_device_ptr();
  a.tag = next_launch_tag();
  a.ktiles = (g.k + kImgK - 1) / kImgK;
  // D through TMA when its base and column stride are 16-byte aligned; otherwise plain stores from registers
  const int esz = dense_bytes(g.e.d_dtype);
  const bool d_tma_ok = ((uintptr_t)g.e.d & 15) == 0 && ((size_t)g.e.ldd * esz) % 16 == 0 && ((size_t)g.m * esz) % 16 == 0;
  // Swapped roles: B of the call (tokens) feeds the MMA's M side (tensor memory lanes) and A (output rows) its N side, so that a
  // lane's accumulator columns are consecutive elements of D in memory.  Needs a 16-bit D that TMA can store.
  // Automatic: swapped unless the other orientation needs fewer rounds of tiles over the SMs.
  auto rounds = [&](int lanes_rows, int col_rows) {
    const int bn_ = pin_bn ? pin_bn : (col_rows > 128 ? 256 : 128);
    const long long tiles = (long long)((lanes_rows + 127) / 128) * ((col_rows + bn_ - 1) / bn_);
    return (tiles + device_sms() - 1) / device_sms() * bn_;   // rounds weighted by the tile's width
  };
  const bool swap = pin_swap != 0 && esz == 2 && d_tma_ok && (pin_swap == 1 || rounds(g.n, g.m) <= rounds(g.m, g.n));
  a.transposed = swap;
  const Fp4Operand &X = swap ? g.B.q : g.A, &Y = swap ? g.A : g.B.q;   // X: rows on lanes (128 per tile); Y: rows on columns (BN per tile)
  const int xm = swap ? g.n : g.m, yn = swap ? g.m : g.n;
  a.m = xm; a.n = yn;
  const int bn = pin_bn ? pin_bn : (yn > 128 ? 256 : 128);
  CUtensorMap ta, tb, tsa, tsb;
  memset(&tsa, 0, sizeof tsa);
  memset(&tsb, 0, sizeof tsb);
  a.a_image = X.image; a.b_image = Y.image;
  auto tiled_ok = [](const Fp4Operand &o) { return o.sld < 0 && ((uintptr_t)o.sc & 15) == 0; };
  // the CTA-pair kernel: 256 x 256 tiles, scales in aligned tiles (or images) on both sides, more than one row tile
  const bool pair = false;   // pairs run in gemm_w4a4_pair.cu; this kernel's own pair form is no longer instantiated
  if (X.image) {
    const uint64_t tiles = (uint64_t)((xm + 127) / 128) * a.ktiles;
    if (!make_tmap_bytes(&ta, X.data, 128, 128, 128, 128, tiles, kImgTileBytes)) return cudaErrorInvalidValue;
    if (!make_tmap_scales(&tsa, (const uint8_t *)X.data + kImgDataBytes, 2048, tiles, kImgTileBytes)) return cudaErrorInvalidValue;
    a.sa = X.data; a.sa_gather = 0;
  } else {
    if (!make_tmap_bytes(&ta, X.data, (uint64_t)g.k / 2, (uint64_t)xm, (uint64_t)X.ld / 2, 128, 1, (uint64_t)X.ld / 2 * xm)) return cudaErrorInvalidValue;
    a.sa = X.sc; a.sa_ld = X.sld; a.sa_gather = tiled_ok(X) ? 0 : 1;
    if (!a.sa_gather && !make_tmap_scales(&tsa, X.sc, (uint64_t)((-X.sld) >> 2) * 512, (uint64_t)(xm + 127) / 128, (uint64_t)((-X.sld) >> 2) * 512))
      return cudaErrorInvalidValue;
  }
  if (Y.image) {
    const uint64_t tiles = (uint64_t)((yn + 127) / 128) * a.ktiles;
    if (!make_tmap_bytes(&tb, Y.data, 128, 128, 128, 128, tiles, kImgTileBytes)) return cudaErrorInvalidValue;
    if (!make_tmap_scales(&tsb, (const uint8_t *)Y.data + kImgDataBytes, 2048, tiles, kImgTileBytes)) return cudaErrorInvalidValue;
    a.sb = Y.data; a.sb_gather = 0;
  } else {
    if (!make_tmap_bytes(&tb, Y.data, (uint64_t)g.k / 2, (uint64_t)yn, (uint64_t)Y.ld / 2, pair ? 128 : bn, 1, (uint64_t)Y.ld / 2 * yn)) return cudaErrorInvalidValue;
    a.sb = Y.sc; a.sb_ld = Y.sld; a.sb_gather = tiled_ok(Y) ? 0 : 1;
    if (!a.sb_gather && !make_tmap_scales(&tsb, Y.sc, (uint64_t)((-Y.sld) >> 2) * 512, (uint64_t)(yn + 127) / 128, (uint64_t)((-Y.sld) >> 2) * 512))
      return cudaErrorInvalidValue;
  }
  CUtensorMap td;
  memset(&td, 0, sizeof td);
  if (swap) {   // boxes of 16 consecutive elements of D (32 bytes) for 32 tokens, staged in the 32-byte swizzle
    if (!make_tmap_dense(&td, g.e.d, esz, (uint64_t)g.m, (uint64_t)g.n, (uint64_t)g.e.ldd * esz, 16, 32, 32)) return cudaErrorInvalidValue;
    a.d_tma = 1;
  } else {
    a.d_tma = d_tma_ok && make_tmap_dense(&td, g.e.d, esz, (uint64_t)g.m, (uint64_t)g.n, (uint64_t)g.e.ldd * esz, 128, esz == 2 ? 16 : 8);
  }
  if (bn == 256) return launch_cfg<256, 1, 4, false>(ta, tb, tsa, tsb, td, a, s);
  return launch_cfg<128, 2, 6, false>(ta, tb, tsa, tsb, td, a, s);
}

}  // namespace nvb

extern "C" nvfp4a_status nvfp4a_b200_kernel_status(unsigned int *status, int reset) {
  using namespace nvb;
  clear_error();
  if (!status) return fail(NVFP4A_INVALID_VALUE, "nvfp4a_b200_kernel_status: status is NULL");
  if (nvfp4a_status st = check_device()) return st;
  unsigned int *p = kernel_status_device_ptr();
  cudaError_t e = cudaMemcpy(status, p, sizeof(unsigned int), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && reset) e = cudaMemset(p, 0, sizeof(unsigned int));
  return cuda_fail(e, "nvfp4a_b200_kernel_status");
}

extern "C" unsigned int nvfp4a_b200_last_launch(void) { return nvb::g_last_launch; }

extern "C" int nvfp4a_b200_set_wait_limit(long long cycles) {
  if (cycles < 1000) return -1;
  nvb::g_tp_wait_limit = cycles;
  return 0;
}

extern "C" int nvfp4a_b200_set_pdl(int on) {
  nvb::g_pdl = on ? 1 : 0;
  return 0;
}

extern "C" int nvfp4a_b200_set_pair(int mode) {
  if (mode < -1 || mode > 1) return -1;
  nvb::set_w4a4_pair(mode);
  return 0;
}

extern "C" int nvfp4a_b200_set_swap(int mode) {
  if (mode < -1 || mode > 1) return -1;
  nvb::set_w4a4_swap(mode);
  return 0;
}

extern "C" int nvfp4a_b200_set_tile_n(int bn) {
  if (bn != 0 && bn != 128 && bn != 256) return -1;
  nvb::set_w4a4_tile_n(bn);
  return 0;
}
