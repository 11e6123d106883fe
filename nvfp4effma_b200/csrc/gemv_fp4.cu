// Decode GEMV on the FP4 tensor cores: D[m x n] = A[m x k] (NVFP4) * B[n x k]^T for n = 1 or 2 BF16 activation vectors (W4A16).
//
// The weights are consumed as they are stored: TMA streams 256-row x 256-k tiles of nibbles and their block scales from
// HBM into a shared-memory ring and tcgen05.mma kind::mxf4nvf4 reads them with the E4M3 block scales in tensor memory.  No
// CUDA-core instruction touches a weight, so the kernel runs at the speed the memory system delivers A (0.5625 bytes per
// weight).
//
// The BF16 activations become FP4 operands by an exact digit expansion.  For one token and the k range of one CTA let eb be
// the largest biased exponent; every |x_i| is written as X_i * 2^(eb - 158) with the 32-bit integer X_i (for BF16, whose
// significand has 8 bits, this is exact unless |x_i| < 2^-24 max|x|: such elements lose their bits below 2^-31 max|x|).
// X_i = sum over d of t_d(i) * 4^d with the base-4 digits t_d in {0, 1, 2, 3}; the E2M1 codes 0..3 are the values t / 2, so
// "piece" d of the token is the FP4 vector sign(x_i) * t_d(i) / 2 and
//     sum_i a_i x_i = 2^(eb - 157) * sum_d 4^d * (sum_i a_i * piece_d(i)).
// The 16 pieces of a token are 16 rows of the MMA's M dimension (block scales 1.0), 256 weight rows are its N dimension,
// and the inner sums are what the tensor cores compute: accumulator lane d, column r holds piece d against weight row r.
// Two warps read the 16 (or 32) lanes, join piece d with piece d + 8 and leave the sums in shared memory, where each of 256
// threads adds its weight row's eight values with their powers of four in FP32.  Pieces are built once per CTA
// in shared memory (8 warps, while the first weight tiles are in flight) in the 128-byte-swizzled K-major layout the MMA
// reads.  The MMA's M is 128: the rows past the pieces read whatever follows them in shared memory and produce
// accumulator lanes nobody looks at (every FP4 bit pattern is a finite number).
//
// Work split: grid = (splits, 256-row tiles); the CTAs of one row tile form a thread-block cluster and each takes a
// contiguous range of 256-k chunks.  Partial results meet through distributed shared memory: rank 0 adds the partials of
// ranks 1, 2, ... in rank order -- deterministic, no atomics, no global scratch -- and runs the plain or extended epilogue,
// one thread per weight row.
//
// Timeline of a launch (8192 x 8192, 128 CTAs, about 10 us between the previous kernel's end and this one's): the set-up
// (barriers, tensor memory) touches no global memory and runs under programmatic dependent launch while the previous kernel
// drains; the ring's first fill is requested by five warps at once right after the block-wide barrier, because a copy
// instruction costs its warp 150-300 ns to issue whatever it moves (an image stage is therefore two rank-4 tensor copies: 32
// KiB of nibbles, 4 KiB of scales); the epilogue's operands are fetched only after the pieces are built.
//
// Semantics: FP32 accumulation in the tensor cores' order, within the FP32 accumulation bound of the exact definition
// (reference include/nvfp4effma.h:82-92 there), as the reference's own tensor-core GEMV (src/tensors/gemv_tc.cuh there).
// Block scales are consumed as unsigned E4M3.
#include <atomic>
#include "operands.cuh"
#include "sm100.cuh"
#include "tp_barrier.cuh"

namespace nvb {

using namespace sm100;

namespace {

struct GemvFp4Args {
  int m, n, k;
  int a_image;
  const uint8_t *sa;   // plain: block scale base; image: image base
  int sa_ld, ktiles;
  int linear;          // plain operand with linear block scales: a TMA box brings [256 rows][16 bytes], four warps re-tile it
  const uint16_t *x; int ldx;
  Epilogue e;
  EpilogueEx ex;
  unsigned *status;
  unsigned tag;        // this launch's tag in the status word
  int tp_world, tp_rank;                       // > 1: wait for the peers' posts before the activations are read (TpPush::deferred bit 0)
  unsigned long long *tp_flags[kMaxRanks];
  long long tp_wait_cycles;
  int stages;          // ring depth (2..6), chosen by the host from the shared memory left beside the pieces
  int piece_bytes;     // shared memory of the activation pieces: chunks per CTA x piece rows x 128
};

constexpr int kThreads = 320, kDecompThreads = 256;
constexpr int kRows = 256;                                  // weight rows per tile (the MMA's N)
constexpr int kDataBytes = kRows * 128, kSfBytes = kRows * 16, kStageBytes = kDataBytes + kSfBytes;  // 36 KiB per 256-k chunk
constexpr int kMaxChunks = 16;                              // 256-k chunks per CTA: 4096 values of k
constexpr int kTmemCols = 512;                              // accumulator [0, 256), A scales (1.0) [256, 260), B scales [272, 272 + 32 * stages), stages <= 6
constexpr int kMaxStages = 6;
constexpr int kSmemLimit = 232448 - 1024;                   // dynamic shared memory of one CTA on sm_100, less the alignment slack
constexpr unsigned kStWaitFull = 0x201, kStWaitEmpty = 0x202, kStWaitAcc = 0x203, kStWaitPieces = 0x204, kStWaitRetile = 0x205;
constexpr int kRawSfBytes = kRows * 16;                      // linear scales of one chunk as they lie in memory: [256 rows][16 bytes]

// Shared memory of a CTA: [pieces | stages x 36 KiB | unit scales 512 | results splits x NTOK x 256 floats | barriers 256].
// The MMA reads 16 KiB from the start of a pieces chunk (its M is 128 rows), which stays inside the stages.
__host__ __device__ constexpr int fixed_bytes(int ntok, int splits) { return 512 + splits * ntok * 1024 + 320; }

__device__ __forceinline__ float pow2f(int e) { return __int_as_float((e + 127) << 23); }  // -126 <= e <= 127

template <int NTOK>
__global__ void __launch_bounds__(kThreads, 1)
gemv_fp4_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_s, const GemvFp4Args g) {
  constexpr int PR = 16 * NTOK;
  const int kStages = g.stages;
  const uint32_t rank = cluster_ctarank(), splits = gridDim.x;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *pieces = smem;
  uint8_t *stages = smem + g.piece_bytes;
  const bool linear = g.linear;
  const int stage_bytes = kStageBytes + (linear ? kRawSfBytes : 0);
  uint8_t *unit_sf = stages + kStages * stage_bytes;
  float *res = (float *)(unit_sf + 512);                   // [splits][NTOK][256]: slot p is written by the cluster's rank p (into rank 0's memory)
  uint64_t *bars = (uint64_t *)(unit_sf + 512 + splits * NTOK * 1024);
  uint64_t *full = bars, *empty = bars + kMaxStages, *sf_ready = bars + 2 * kMaxStages, *acc_full = bars + 3 * kMaxStages, *pieces_ready = acc_full + 1;
  uint32_t *tmem_slot = (uint32_t *)(pieces_ready + 1);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
  uint32_t *wmax = tmem_slot + 2;                          // [8 warps][NTOK] largest |x| bit pattern
  volatile int *inexact = (volatile int *)(wmax + 8 * NTOK);   // some activation of this CTA does not fit the digit planes
  int *consumed = (int *)(wmax + 8 * NTOK + 1);                // [stage] warps done with the stage (the CUDA-core consumer)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gm = g.m, gn = g.n;
  const int tiles128 = (gm + 127) >> 7;
  const int tm = blockIdx.y;                               // 256-row tile
  const bool a_image = g.a_image;
  const uint8_t *const sa_base = g.sa;
  const int sa_ld = g.sa_ld;
  const int nk = g.k >> 8;
  const int c0 = (int)((long long)rank * nk / splits), c1 = (int)((long long)(rank + 1) * nk / splits), nloc = c1 - c0;
  unsigned *const status_word = g.status;
  const bool second = tm * 2 + 1 < tiles128;               // the tile's second 128 rows exist

  // One stage of the weight ring.  A copy instruction costs the issuing warp 150-200 cycles per active lane whatever it moves,
  // so a stage is as few copies as its layout allows, issued by as many lanes of ONE instruction: an image's nibbles (32 KiB, both
  // 128-row halves) and block scales (4 KiB) are two rank-4 tensor copies in lanes 0 and 1.
  auto request_stage = [&](int it) {
    const int s = it % kStages, c = c0 + it;
    uint8_t *sW = stages + (size_t)s * stage_bytes, *sSf = sW + kDataBytes;
    if (lane == 0) mbar_arrive_expect_tx(&full[s], kDataBytes + (linear ? (uint32_t)kRawSfBytes : ((second || a_image) ? 4096u : 2048u)));
    __syncwarp();
    if (a_image) {
      if (lane < 2) tma_load_4d(lane ? sSf : sW, lane ? &tmap_s : &tmap_a, 0, 0, c, 2 * tm, &full[s]);
    } else if (lane < 2) {
      if (lane == 0) {
        tma_load_2d(sW, &tmap_a, c * 128, tm * 256, &full[s]);
      } else if (linear) {
        tma_load_2d(sW + kStageBytes, &tmap_s, c * 4, tm * 256, &full[s]);   // 16 bytes (4 words) of 256 rows; rows past m read zeros
      }
    } else if (lane < 4 && !linear) {
      const int h = lane - 2;
      if (h == 0 || second) bulk_load(sSf + h * 2048, sa_base + (size_t)(2 * tm + h) * ((size_t)((-sa_ld) >> 2) * 512) + (size_t)c * 2048, 2048, &full[s]);
    }
  };

  const int early = nloc < kStages ? nloc : kStages;   // the ring's first fill needs no wait

  // The set-up touches no global memory, so it may run while the stream's previous kernel finishes (programmatic dependent
  // launch); nothing before the block-wide barrier waits for memory either: the first weights are requested right after it.
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmap_a);
    if (a_image || linear) prefetch_tensormap(&tmap_s);
    for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); mbar_init(&sf_ready[s], 1); }
    mbar_init(acc_full, 1);
    mbar_init(pieces_ready, kDecompThreads / 32);
    *abort_flag = 0;
    *inexact = 0;
    for (int s = 0; s < kStages; ++s) consumed[s] = 0;
    fence_barrier_init();
  }
  if (threadIdx.x < 128) ((uint32_t *)unit_sf)[threadIdx.x] = 0x38383838u;  // E4M3 1.0
  fence_proxy_async_smem();
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
  pdl_wait();
  // tensor-parallel layers in the deferred form: the activations are complete once every peer has posted the previous gather
  if (g.tp_world > 1) tp_wait_posts(g.tp_flags, g.tp_world, g.tp_rank, g.status, g.tag, g.tp_wait_cycles);
  // the decomposition warps ask for their activations first: the loads fly while the barrier below gathers the CTA
  const int t2 = threadIdx.x - 64, nvec = nloc * 32;  // vectors of 8 consecutive k; at most 2 per thread and token
  uint4 xq[NTOK][2];
  if (warp >= 2) {
#pragma unroll
    for (int t = 0; t < NTOK; ++t)
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int v = t2 + u * kDecompThreads;
        xq[t][u] = (t < gn && v < nvec) ? __ldg((const uint4 *)(g.x + (size_t)t * g.ldx + (size_t)c0 * 256) + v) : make_uint4(0, 0, 0, 0);
      }
  }

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

  // rank 0 runs the epilogue, one thread per weight row; its operands are fetched once the pieces are built, far ahead of their use
  const int erow = t2, ei = tm * 256 + erow;
  const bool erow_ok = warp >= 2 && rank == 0 && ei < gm;
  float e_rowp = 0.f, e_bias = 0.f, e_c[NTOK];
#pragma unroll
  for (int t = 0; t < NTOK; ++t) e_c[t] = 0.f;

  // The ring's first fill, one stage per warp: a copy instruction is slow to issue (see request_stage), and the decomposition
  // warps among these have nothing to do until their activations arrive.
  if (warp < early) request_stage(warp);

  if (warp == 0) {
    // ---------------- producer: after the first fill, each stage as its slot comes free ----------------
    int requested = early;
    for (int it = early; it < nloc; ++it) {
      const int s = it % kStages;
      const bool okw = wait(&empty[s], ((it / kStages) & 1) ^ 1, kStWaitEmpty);
      if (!__all_sync(0xFFFFFFFFu, okw)) break;
      request_stage(it);
      requested = it + 1;
    }
    // No copy may be in flight when the CTA leaves.  On the normal path every fill has long been consumed and these waits return
    // at once; after a wait somewhere gave up they hold the CTA (bounded) until the last requested fill of every stage has landed.
    for (int it = requested - 1; it >= 0 && it >= requested - kStages; --it) mbar_wait(&full[it % kStages], (it / kStages) & 1);
  } else if (warp == 1) {
    // ---------------- MMA issuer: D[piece][weight row] += pieces (A, M = 128) x weights (B, N = 256) ----------------
    // The whole warp runs the loop and one elected lane issues: from inside a one-lane branch every tcgen05 instruction costs the
    // warp about 150 cycles, and a chunk needs twelve of them (eight scale-tile copies, four MMAs).
    if (nloc > 0) {
      constexpr uint32_t idesc = idesc_mxf4nvf4(128, kRows);
      const uint32_t sfa_tmem = tmem_base + 256;
      tmem_cp_32x128b_warpx4_elect(sfa_tmem, smem_desc_sf(smem_u32(unit_sf)));
      if (__all_sync(0xFFFFFFFFu, wait(pieces_ready, 0, kStWaitPieces)) && !*inexact) {   // (the CUDA cores consume the ring otherwise)
        tc_fence_after();
        bool ok = true;
        const uint64_t da0 = smem_desc_sw128(smem_u32(pieces));
        for (int it = 0; it < nloc; ++it) {
          const int s = it % kStages;
          ok = __all_sync(0xFFFFFFFFu, linear ? wait(&sf_ready[s], (it / kStages) & 1, kStWaitRetile) : wait(&full[s], (it / kStages) & 1, kStWaitFull));
          if (!ok) break;
          tc_fence_after();
          const uint32_t sW = smem_u32(stages + (size_t)s * stage_bytes), sSf = sW + kDataBytes;
          const uint32_t sfb_tmem = tmem_base + 272 + 32 * s;
          const uint64_t da = da0 + (uint32_t)(it * (PR * 128 >> 4)), db = smem_desc_sw128(sW);
          const uint64_t sf0 = smem_desc_sf(sSf), sf1 = smem_desc_sf(sSf + 2048);
#pragma unroll
          for (int j = 0; j < 4; ++j)   // descriptors advance in 16-byte units: 32 bytes along the operand rows, 512 bytes per scale tile
            cp2_mma_mxf4nvf4_elect(sfb_tmem + 8 * j, sf0 + 32 * j, sf1 + 32 * j, tmem_base, da + 2 * j, db + 2 * j, idesc, sfa_tmem, (uint32_t)((it | j) != 0));
          tc_commit_elect(&empty[s]);
        }
        if (ok) tc_commit_elect(acc_full);
      }
    }
  } else {
    // ---------------- 8 warps: activations -> FP4 pieces in shared memory ----------------
    const int w2 = warp - 2;
    int ebs[NTOK];  // biased exponent the token's pieces refer to
    uint32_t lost = 0;
#pragma unroll
    for (int t = 0; t < NTOK; ++t) {
      uint32_t a = 0;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const uint32_t w[4] = {xq[t][u].x, xq[t][u].y, xq[t][u].z, xq[t][u].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) a = max(a, max(w[i] & 0x7FFFu, (w[i] >> 16) & 0x7FFFu));
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) a = max(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
      if (lane == 0) wmax[w2 * NTOK + t] = a;
    }
    named_barrier(2, kDecompThreads);
#pragma unroll
    for (int t = 0; t < NTOK; ++t) {
      uint32_t a = 0;
#pragma unroll
      for (int w = 0; w < 8; ++w) a = max(a, wmax[w * NTOK + t]);
      const int eb = max((int)(a >> 7), 1);
      ebs[t] = eb;
      if (eb == 255) lost = 1;   // Inf or NaN: IEEE arithmetic on the CUDA cores gives each output its own Inf or NaN
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int v = t2 + u * kDecompThreads;
        if (v >= nvec) break;
        uint32_t X[8], sgn = 0;
        const uint32_t w[4] = {xq[t][u].x, xq[t][u].y, xq[t][u].z, xq[t][u].w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t h = (w[i >> 1] >> (16 * (i & 1))) & 0xFFFFu;
          const uint32_t e = (h >> 7) & 0xFFu;
          const uint32_t mant = (h & 0x7Fu) | (e ? 0x80u : 0u);
          const int sh = (int)max(e, 1u) - eb + 24;  // <= 24
          X[i] = sh >= 0 ? mant << sh : (sh > -8 ? mant >> (-sh) : 0u);
          if (sh < 0) lost |= mant & ((1u << min(-sh, 8)) - 1u);   // bits of this element below the last digit plane
          sgn |= (h >> 15) << (4 * i + 3);
        }
        const int chunk = v >> 5, b = (v & 31) * 4;
        uint8_t *base = pieces + (size_t)chunk * (PR * 128);
#pragma unroll
        for (int d = 0; d < 16; ++d) {
          uint32_t word = sgn;
#pragma unroll
          for (int i = 0; i < 8; ++i) word |= ((X[i] >> (2 * d)) & 3u) << (4 * i);
          const int row = t * 16 + d;
          *(uint32_t *)(base + (row >> 3) * 1024 + (row & 7) * 128 + ((((b >> 4) ^ (row & 7)) << 4) | (b & 15))) = word;
        }
      }
    }
    if (lost) *inexact = 1;
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(pieces_ready);
    named_barrier(3, kDecompThreads);   // every warp's verdict is in
    const bool exact = *inexact == 0;
    if (erow_ok) {
      e_rowp = epi_row_part(g.e, ei);
      if (g.e.bias) e_bias = load_dense(g.e.bias_dtype, g.e.bias, ei);
      if (g.e.beta != 0.f)
#pragma unroll
        for (int t = 0; t < NTOK; ++t)
          if (t < gn) e_c[t] = load_dense(g.e.c_dtype, g.e.c, (size_t)t * g.e.ldc + ei);
    }

    if (!exact) {
      // ---------------- the exact route for activations the digit planes cannot hold ----------------
      // Some element lies more than 2^24 below its token's largest, so its low bits (or all of it) would be dropped -- far below
      // the FP32 accumulation bound unless the large elements meet zero weights.  Then the tensor cores sit this CTA out: the
      // eight warps consume the ring themselves, one thread per weight row, decoding nibbles and block scales from the stages
      // and accumulating in FP32 against the activations (kept as FP32 in the pieces' memory).  Several times slower; rare.
      float *xs = (float *)pieces;   // [token][k of this CTA]
#pragma unroll
      for (int t = 0; t < NTOK; ++t)
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int v = t2 + u * kDecompThreads;
          if (v >= nvec) break;
          const uint32_t w[4] = {xq[t][u].x, xq[t][u].y, xq[t][u].z, xq[t][u].w};
          float *dst = xs + (size_t)t * nloc * 256 + (size_t)v * 8;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            dst[2 * i] = __uint_as_float(w[i] << 16);
            dst[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
          }
        }
      named_barrier(3, kDecompThreads);
      float acc[NTOK];
#pragma unroll
      for (int t = 0; t < NTOK; ++t) acc[t] = 0.f;
      const int r = t2;
      bool ok = true;
      for (int it = 0; it < nloc && ok; ++it) {
        const int s = it % kStages;
        ok = wait(&full[s], (it / kStages) & 1, kStWaitFull);
        if (!ok) break;
        const uint8_t *st = stages + (size_t)s * stage_bytes;
        const uint8_t *rowp = st + (r >> 3) * 1024 + (r & 7) * 128;
        const uint8_t *sfp = linear ? st + kStageBytes + r * 16 : st + kDataBytes + (r >> 7) * 2048 + (r & 31) * 16 + ((r & 127) >> 5) * 4;
#pragma unroll 2
        for (int u16 = 0; u16 < 8; ++u16) {
          const uint4 q = *(const uint4 *)(rowp + ((u16 ^ (r & 7)) << 4));
          const uint32_t wd[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            const int jj = 2 * u16 + b;   // block of 16 values within the chunk
            const float sc = __fmul_rn(e4m3_to_f32((linear ? sfp[jj] : sfp[(jj >> 2) * 512 + (jj & 3)]) & 0x7Fu), 0.5f);
#pragma unroll
            for (int t = 0; t < NTOK; ++t) {
              const float *xv = xs + (size_t)t * nloc * 256 + (size_t)it * 256 + jj * 16;
              float part = 0.f;
#pragma unroll
              for (int i = 0; i < 16; ++i)
                part = __fmaf_rn((float)e2m1_x2((wd[2 * b + (i >> 3)] >> (4 * (i & 7))) & 0xFu), xv[i], part);
              acc[t] = __fmaf_rn(sc, part, acc[t]);
            }
          }
        }
        __threadfence_block();
        __syncwarp();
        // the eighth warp hands the stage back; the count is per stage because a warp may run several stages ahead of another,
        // but never a whole fill ahead on the same stage
        if (lane == 0 && (atomicAdd(&consumed[s], 1) & 7) == 7) mbar_arrive(&empty[s]);
      }
      if (ok)
#pragma unroll
        for (int t = 0; t < NTOK; ++t) st_peer_f32(&res[(rank * NTOK + t) * 256 + r], 0, acc[t]);
    } else if ((warp & 3) == 0) {
      // ---------------- warps 4 and 8 (tensor-memory lanes 0..31): accumulator -> shared memory, 128 weight rows each ----------------
      // A thread of the 16 x 256-bit load holds pieces d and d + 8 (d = lane / 4) of sixteen weight rows; it joins the two and
      // leaves them in red[token][weight row][9] (the stage ring is free by now: every MMA has completed), from where all 256
      // threads sum their row's eight values.
      const int half = warp >> 3;  // 0: columns 0..127, 1: columns 128..255
      if (nloc > 0 && wait(acc_full, 0, kStWaitAcc)) {
        tc_fence_after();
        const int dlo = lane >> 2;
        const float flo = pow2f(2 * dlo), fhi = pow2f(2 * dlo + 16);
#pragma unroll
        for (int t = 0; t < NTOK; ++t)
#pragma unroll
          for (int q = 0; q < 2; ++q) {            // 64 columns per load
            uint32_t r[32];
            tmem_ld_16x256b_x8(tmem_base + ((uint32_t)(16 * t) << 16) + half * 128 + q * 64, r);
            tmem_ld_wait();
            float *red = (float *)stages + ((size_t)t * 256 + half * 128 + q * 64 + 2 * (lane & 3)) * 9 + dlo;
#pragma unroll
            for (int gq = 0; gq < 8; ++gq) {
              red[(gq * 8) * 9] = __fmaf_rn(__uint_as_float(r[4 * gq + 2]), fhi, __fmul_rn(__uint_as_float(r[4 * gq]), flo));
              red[(gq * 8 + 1) * 9] = __fmaf_rn(__uint_as_float(r[4 * gq + 3]), fhi, __fmul_rn(__uint_as_float(r[4 * gq + 1]), flo));
            }
          }
      }
    }
    if (exact && linear && (warp & 3) != 0 && warp >= 5) {
      // ---------------- warps 5, 6, 7, 9: linear block scales [256 rows][16 bytes] -> the eight 512-byte tiles of the stage ----------------
      // A stage belongs to one warp for the whole launch: a wait on the parity of fill f is only meaningful to a thread that
      // has seen fill f - 1 complete (on a barrier still in its first phase, a wait for the second fill's parity returns at once).
      const int w = warp == 9 ? 3 : warp - 5;
      for (int it = 0; it < nloc; ++it) {
        const int s = it % kStages;
        if ((s & 3) != w) continue;
        if (!wait(&full[s], (it / kStages) & 1, kStWaitRetile)) break;
        uint8_t *st = stages + (size_t)s * stage_bytes;
        const uint8_t *raw = st + kStageBytes;
        uint8_t *sf = st + kDataBytes;
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t wd[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) wd[q] = *(const uint32_t *)(raw + (h * 128 + 32 * q + lane) * 16 + 4 * j);
            *(uint4 *)(sf + h * 2048 + j * 512 + lane * 16) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
          }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sf_ready[s]);
      }
    }
    if (exact) {
      // ---------------- all eight warps: each thread sums the sixteen pieces of its weight row and hands the result to rank 0 ----------------
      // (the order of the additions is that of a butterfly over the piece pairs)
      named_barrier(3, kDecompThreads);
      if (nloc > 0 && !*abort_flag) {
#pragma unroll
        for (int t = 0; t < NTOK; ++t) {
          const float *v = (const float *)stages + ((size_t)t * 256 + t2) * 9;
          const float sum = __fadd_rn(__fadd_rn(__fadd_rn(v[0], v[1]), __fadd_rn(v[2], v[3])), __fadd_rn(__fadd_rn(v[4], v[5]), __fadd_rn(v[6], v[7])));
          const int ex = ebs[t] - 157, e1 = max(ex, -100);
          const float s1 = pow2f(e1), s2 = pow2f(ex - e1);
          const bool bad = ebs[t] == 255;  // Inf or NaN among the activations
          st_peer_f32(&res[(rank * NTOK + t) * 256 + t2], 0, bad ? __int_as_float(0x7FC00000) : __fmul_rn(__fmul_rn(sum, s1), s2));
        }
      }
    }
  }

  // ---------------- rank 0: add the ranks' results in rank order, then the epilogue, one thread per weight row ----------------
  // Every rank has stored its results into rank 0's shared memory; the peers arrive on the cluster barrier and leave.
  tc_fence_before();
  __syncthreads();
  if (splits > 1) {
    cluster_arrive_release();
    if (rank == 0) cluster_wait_acquire();
  }
  if (rank == 0 && warp >= 2 && !*abort_flag) {
    const Epilogue &e = g.e;
    const int mask = g.ex.mask, row = erow, i = ei;
    const bool row_ok = erow_ok;
    float amax = 0.f;
    float v[NTOK];
#pragma unroll
    for (int t = 0; t < NTOK; ++t) {
      v[t] = 0.f;
      if (t >= gn) continue;
      float acc = 0.f;
      if (nk >= (int)splits)  // every rank had at least one chunk
        for (uint32_t p = 0; p < splits; ++p) acc = p ? __fadd_rn(acc, res[(p * NTOK + t) * 256 + row]) : res[t * 256 + row];
      float colp = epi_col_part(e, t);
      if (mask & kExNorm) colp = __fmul_rn(colp, warp_norm_scale(g.ex, t, lane));
      float val = __fmul_rn(acc, epi_scale(e, e_rowp, colp));
      if (e.bias) val = __fadd_rn(val, e_bias);
      if (e.beta != 0.f) val = __fmaf_rn(e.beta, e_c[t], val);
      v[t] = row_ok ? val : 0.f;
    }
    if (mask & (kExSwiglu | kExOut2)) {  // neighbours' values through shared memory (the results are consumed by now)
      named_barrier(2, kDecompThreads);
#pragma unroll
      for (int t = 0; t < NTOK; ++t) res[t * 256 + row] = v[t];
      named_barrier(2, kDecompThreads);
    }
#pragma unroll
    for (int t = 0; t < NTOK; ++t) {
      if (t >= gn) continue;
      if (mask & kExSwiglu) {
        if (row_ok && !(row & 8)) {
          const float hh = silu_mul(v[t], res[t * 256 + row + 8]);
          store_dense(e.d_dtype, e.d, (size_t)t * e.ldd + (i >> 4) * 8 + (i & 7), hh);
          amax = fmaxf(amax, fabsf(hh));
        }
      } else if (row_ok) {
        store_dense(e.d_dtype, e.d, (size_t)t * e.ldd + i, v[t]);
        amax = fmaxf(amax, fabsf(v[t]));
      }
      if ((mask & kExOut2) && row_ok) {
        store_dense(g.ex.d2_dtype, g.ex.d2, (size_t)t * g.ex.ldd2 + i, __fmul_rn(v[t], load_dense(g.ex.w2_dtype, g.ex.w2, i)));
        if (!(row & 15)) {
          float sq = 0.f;
#pragma unroll
          for (int r = 0; r < 16; ++r) sq = __fadd_rn(sq, __fmul_rn(res[t * 256 + row + r], res[t * 256 + row + r]));
          g.ex.sq[(size_t)t * g.ex.ld_sq + (i >> 4)] = sq;
        }
      }
    }
    if (e.amax) warp_amax_commit(e.amax, amax);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

static std::atomic<int> g_gemv_splits{0};  // 0 = automatic
void set_gemv_fp4_splits(int s) { g_gemv_splits = s; }

// splits: power of two, at most 8 and nk; every CTA's k range is at most kMaxChunks chunks (its pieces' shared memory).
// Pinned (nvfp4a_b200_set_gemv_splits): that value if the problem can use it.  Automatic: this kernel pays about 5 us of
// set-up and tail per launch (pieces, cluster, two-step epilogue), so it takes only problems that stream at least 32 MB of
// weights over at least 96 CTAs; smaller ones go to the mma.sync GEMV.  Returns 0 when the kernel should not run.
static int choose_splits(int m, int k) {
  const int nk = k >> 8, tiles = (m + kRows - 1) / kRows;
  const int need = (nk + kMaxChunks - 1) / kMaxChunks;
  int s = 1;
  while (s < need) s *= 2;
  if (const int f = g_gemv_splits.load()) {
    return (f >= s && f <= 8 && f <= nk && !(f & (f - 1))) ? f : 0;
  }
  if (s > 4 || s > nk) return 0;
  while (s * 2 <= 4 && nk / (s * 2) >= 8 && tiles * s * 2 <= device_sms()) s *= 2;
  if (tiles * s < 96 || (double)m * k * 0.5625 < 32e6) return 0;
  return s;
}

bool gemv_fp4_supports(const GemmArgs &g) {
  if (!(g.n >= 1 && g.n <= 2 && g.B.dtype == NVFP4A_BF16 && !g.A.ue && g.k >= 256 && g.k % 256 == 0)) return false;
  if (((uintptr_t)g.B.data & 15) || g.B.ld % 8) return false;
  // plain operands: scales in aligned 512-byte tiles (the swizzled layout), or linear with a 16-byte aligned base and pitch (TMA)
  if (!g.A.image && (((uintptr_t)g.A.data & 15) || g.A.ld % 32 || ((uintptr_t)g.A.sc & 15) || (g.A.sld > 0 && g.A.sld % 16))) return false;
  return choose_splits(g.m, g.k) > 0;
}

cudaError_t launch_gemv_fp4(const GemmArgs &g, cudaStream_t s) {
  GemvFp4Args a;
  memset(&a, 0, sizeof a);
  a.m = g.m; a.n = g.n; a.k = g.k;
  a.x = (const uint16_t *)g.B.data; a.ldx = g.B.ld;
  a.e = g.e; a.ex = g.x;
  a.status = kernel_status_device_ptr();
  a.tag = next_launch_tag();
  if (g.tp.world > 1 && (g.tp.deferred & 1)) {
    a.tp_world = g.tp.world; a.tp_rank = g.tp.rank; a.tp_wait_cycles = tp_wait_limit();
    for (int p = 0; p < g.tp.world; ++p) a.tp_flags[p] = g.tp.flags[p];
  }
  a.ktiles = (g.k + kImgK - 1) / kImgK;
  a.a_image = g.A.image;
  CUtensorMap ta, ts;
  memset(&ts, 0, sizeof ts);
  if (g.A.image) {
    if (!make_tmap_image_pair(&ta, g.A.data, 128, (uint64_t)a.ktiles, (uint64_t)((g.m + 127) / 128))) return cudaErrorInvalidValue;
    if (!make_tmap_image_pair(&ts, (const uint8_t *)g.A.data + kImgDataBytes, 16, (uint64_t)a.ktiles, (uint64_t)((g.m + 127) / 128))) return cudaErrorInvalidValue;
    a.sa = g.A.data;
  } else {
    if (!make_tmap_bytes(&ta, g.A.data, (uint64_t)g.k / 2, (uint64_t)g.m, (uint64_t)g.A.ld / 2, kRows)) return cudaErrorInvalidValue;
    a.sa = g.A.sc; a.sa_ld = g.A.sld;
    a.linear = g.A.sld > 0;
    if (a.linear && !make_tmap_dense(&ts, g.A.sc, 4, (uint64_t)g.k / 64, (uint64_t)g.m, (uint64_t)g.A.sld, 4, kRows)) return cudaErrorInvalidValue;
  }
  const int splits = choose_splits(g.m, g.k);
  if (splits <= 0) return cudaErrorInvalidValue;
  void (*kern)(CUtensorMap, CUtensorMap, GemvFp4Args) = g.n == 1 ? gemv_fp4_kernel<1> : gemv_fp4_kernel<2>;
  static std::atomic<bool> attr_set[64][2];   // zero-initialised; set once per device and kernel
  int dev = 0;
  cudaGetDevice(&dev);
  const int nk = g.k >> 8, nloc_max = (nk + splits - 1) / splits;
  a.piece_bytes = nloc_max * 16 * g.n * 128;
  const int stage_bytes = kStageBytes + (a.linear ? kRawSfBytes : 0);
  a.stages = (kSmemLimit - a.piece_bytes - fixed_bytes(g.n, splits)) / stage_bytes;
  if (a.stages > kMaxStages) a.stages = kMaxStages;
  if (a.stages < 2) return cudaErrorInvalidValue;
  const int smem_bytes = 1024 + a.piece_bytes + a.stages * stage_bytes + fixed_bytes(g.n, splits);
  if (!attr_set[dev & 63][g.n - 1]) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit + 1024);
    if (e != cudaSuccess) return e;
    attr_set[dev & 63][g.n - 1] = true;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = dim3(splits, (g.m + kRows - 1) / kRows, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // the kernel's set-up overlaps the previous kernel's tail
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, ta, ts, a);
}

}  // namespace nvb

