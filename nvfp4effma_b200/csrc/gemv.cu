// Streaming GEMV for decoding: D[m x n] = A[m x k] (NVFP4) * B[n x k]^T with 1 <= n <= 8 and BF16 activations (W4A16).
//
// The kernel is bound by reading A once from HBM (0.5625 bytes per weight), so it is built around 16-byte loads and as
// few instructions per weight as an exact decode allows:
//   * one CTA owns 16 consecutive rows (one m16 slice), its warps split k in steps of 128 values; per step a lane loads
//     16 bytes of nibbles for two rows (a quad of lanes covers 64 contiguous bytes of a row) and the two scale bytes of its
//     32 values;
//   * nibbles are decoded to exact BF16 pairs with shifts and masks (value * 2^-126, the subnormal trick), multiplied by
//     the block scale in BF16 (exact: 2 x 4 significant bits) and fed to mma.sync.m16n8k16 (BF16 in, FP32 accumulate),
//     whose 8 columns are the n <= 8 activation vectors.  The order of k inside a step is permuted the same way for A
//     and B, which a dot product allows;
//   * the warps' partial sums are added in warp order through shared memory (deterministic, no atomics), then the plain
//     or extended epilogue runs on the slice;
//   * a long reduction (k >= 8192) is cut into 2 or 4 contiguous sections of steps, each with its own partial sums per warp,
//     added at the end in (section, warp) order.  The sections are the unit of a second level of parallelism: when the
//     matrix has few rows (a decode shard of a few hundred rows fills neither the SMs nor the memory pipeline with one CTA
//     walking all of k per 16-row slice) a cluster of as many CTAs takes one section each, the peers store their partial
//     sums into the first CTA's shared memory (DSMEM) and leave; otherwise one CTA walks the sections in turn.  The
//     arithmetic is the same either way, so a row's sum depends on k alone, not on how many rows the matrix (or a
//     tensor-parallel shard of it) has.
// Accumulation is FP32 in the tensor cores' order: results agree with the reference's exact definition
// (include/nvfp4effma.h:82-92 there) within the FP32 accumulation bound, as its own tensor-core GEMV does
// (src/tensors/gemv_tc.cuh there).  To keep scale * 2^126 inside BF16, weights are carried as a * sa * 2^-Z (Z = 8 for
// E4M3, 16 for UE5M3 scales) and the sum is multiplied by 2^Z at the end; this is exact unless a product is below
// 2^-118 in magnitude.
#include <cuda_bf16.h>
#include "operands.cuh"
#include "sm100.cuh"

namespace nvb {

constexpr int kGemvWarps = 8, kGemvMaxSplit = 4;

struct GemvArgs {
  int m, n, k;
  Fp4Operand A;
  const uint16_t *x; int ldx;   // BF16 activations [n][ldx]
  Epilogue e;
  EpilogueEx ex;
  TpPush tp;
  int sections;                 // sections of k (1, 2 or 4; chosen from k alone)
  int ksplit;                   // CTAs per 16-row slice (cluster size along x): 1, or `sections`
};

__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// nibbles p and p + 4 of w -> BF16 pair (low half: nibble p), each value * 2^-126: magnitude bits to [6, 9), sign to 15
template <int P>
__device__ __forceinline__ uint32_t decode_pair(uint32_t w) {
  const uint32_t mag = (P < 2 ? w << (6 - 4 * P) : w >> (4 * P - 6)) & 0x01C001C0u;
  const uint32_t sgn = (w << (12 - 4 * P)) & 0x80008000u;
  return mag | sgn;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

// One step of one lane: 32 values of k (one 16-byte word of nibbles) for rows gq and gq + 8, two scale codes per row,
// and -- for the lanes that carry an activation column -- the 32 matching activations.
struct GemvStep {
  uint4 w0, w1;
  uint32_t sc0, sc1;
  uint4 x[4];
};

// LAYOUT 0: plain operand, linear scales; 1: plain operand, swizzled scales; 2: image
template <int LAYOUT>
__global__ void __launch_bounds__(kGemvWarps * 32, 3) gemv_kernel(const GemvArgs g) {
  __shared__ uint32_t lut[256];                       // scale code -> BF16 pair (sa * 2^(126 - Z), twice)
  __shared__ float part[kGemvMaxSplit * kGemvWarps][16][8];   // [CTA of the cluster x warp]; the first CTA's copy collects all
  __shared__ float vtile[8][16];
  __shared__ float colscale[8];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, q = lane & 3;
  const int ksplit = g.ksplit, krank = ksplit > 1 ? (int)sm100::cluster_ctarank() : 0;
  const int i0 = (blockIdx.x / ksplit) * 16;
  const int gm = g.m, gn = g.n, gk = g.k;
  const bool ue = g.A.ue != 0;
  {
    const float s = scale_to_f32((uint32_t)tid, ue) * (ue ? 0x1p110f : 0x1p118f);  // exact: 4 significant bits
    const uint32_t h = __float_as_uint(s) >> 16;
    lut[tid] = h | (h << 16);
  }
  // Tensor-parallel layers in the deferred form: the activations (and the buffer this kernel writes) belong to this kernel only
  // once every peer has posted the previous gather; the weights do not, so a first step's weights could be requested before.
  if (g.tp.world > 1 && (g.tp.deferred & 1)) tp_wait_posts(g.tp.flags, g.tp.world, g.tp.rank, g.tp.status, g.tp.tag, g.tp.wait_cycles);
  if ((g.ex.mask & kExNorm) && warp < gn) {
    const float s = warp_norm_scale(g.ex, warp, lane);
    if (lane == 0) colscale[warp] = s;
  }
  __syncthreads();

  // rows of this lane (clamped for the loads; rows past m are never stored)
  const int r0 = min(i0 + gq, gm - 1), r1 = min(i0 + gq + 8, gm - 1);
  const bool has_col = gq < gn;
  const uint4 *xrow = (const uint4 *)(g.x + (size_t)(has_col ? gq : 0) * g.ldx);
  const uint8_t *a0p, *a1p, *s0p, *s1p;
  if (LAYOUT != 2) {
    const ScalePos sp{g.A.sld};
    a0p = g.A.data + (size_t)r0 * (g.A.ld >> 1); a1p = g.A.data + (size_t)r1 * (g.A.ld >> 1);
    s0p = g.A.sc + sp.row(r0); s1p = g.A.sc + sp.row(r1);
  } else {
    const size_t t0 = (size_t)(r0 >> 7) * g.A.ktiles * kImgTileBytes, t1 = (size_t)(r1 >> 7) * g.A.ktiles * kImgTileBytes;
    a0p = g.A.data + t0 + (r0 & 127) * 128;
    a1p = g.A.data + t1 + (r1 & 127) * 128;
    s0p = g.A.data + t0 + kImgDataBytes + (r0 & 31) * 16 + ((r0 & 127) >> 5) * 4;
    s1p = g.A.data + t1 + kImgDataBytes + (r1 & 31) * 16 + ((r1 & 127) >> 5) * 4;
  }
  const int chunks = gk >> 5;  // 32-value chunks; a step is 4 of them (one per lane of a quad)
  const int nsteps_all = (chunks + 3) >> 2;
  const int sections = g.sections, per_section = (nsteps_all + sections - 1) / sections;
  const int sec_per_cta = sections / ksplit;   // ksplit is 1 or `sections`

  auto load_step = [&](int st) {
    GemvStep v;
    const int c = 4 * st + q;          // this lane's chunk: k in [32 c, 32 c + 32)
    const bool in = c < chunks;
    v.w0 = v.w1 = make_uint4(0, 0, 0, 0);
    v.sc0 = v.sc1 = 0;
    if (in) {
      size_t doff, soff;
      if (LAYOUT == 0) { doff = 16 * (size_t)c; soff = 2 * (size_t)c; }
      else if (LAYOUT == 1) { doff = 16 * (size_t)c; soff = (size_t)(c >> 1) * 512 + (c & 1) * 2; }
      else {
        const size_t t = (size_t)(c >> 3) * kImgTileBytes;  // 256-k tile = 8 chunks
        const int cc = c & 7;
        doff = t + 16 * cc; soff = t + (cc >> 1) * 512 + (cc & 1) * 2;
      }
      v.w0 = __ldg((const uint4 *)(a0p + doff));
      v.w1 = __ldg((const uint4 *)(a1p + doff));
      v.sc0 = __ldg((const uint16_t *)(s0p + soff));
      v.sc1 = __ldg((const uint16_t *)(s1p + soff));
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) v.x[i] = (in && has_col) ? __ldg(xrow + 4 * c + i) : make_uint4(0, 0, 0, 0);
    return v;
  };

  float acc[4];
  auto consume = [&](const GemvStep &cur) {
    const uint32_t S0[2] = {lut[cur.sc0 & 0xFF], lut[(cur.sc0 >> 8) & 0xFF]}, S1[2] = {lut[cur.sc1 & 0xFF], lut[(cur.sc1 >> 8) & 0xFF]};
    const uint32_t ww0[4] = {cur.w0.x, cur.w0.y, cur.w0.z, cur.w0.w}, ww1[4] = {cur.w1.x, cur.w1.y, cur.w1.z, cur.w1.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // word i: 8 values, k = 32 c + 8 i ..; block i / 2 of the chunk
      const uint32_t a = ww0[i], b = ww1[i], sa = S0[i >> 1], sb = S1[i >> 1];
      // B pairs (x[p], x[p + 4]) to match the decode's pairing
      const uint32_t x04 = prmt(cur.x[i].x, cur.x[i].z, 0x5410), x15 = prmt(cur.x[i].x, cur.x[i].z, 0x7632);
      const uint32_t x26 = prmt(cur.x[i].y, cur.x[i].w, 0x5410), x37 = prmt(cur.x[i].y, cur.x[i].w, 0x7632);
      mma_bf16_16816(acc, bf16x2_mul(decode_pair<0>(a), sa), bf16x2_mul(decode_pair<0>(b), sb), bf16x2_mul(decode_pair<1>(a), sa),
                     bf16x2_mul(decode_pair<1>(b), sb), x04, x15);
      mma_bf16_16816(acc, bf16x2_mul(decode_pair<2>(a), sa), bf16x2_mul(decode_pair<2>(b), sb), bf16x2_mul(decode_pair<3>(a), sa),
                     bf16x2_mul(decode_pair<3>(b), sb), x26, x37);
    }
  };
  // Two of the warp's steps are requested before the first is consumed (80 registers, three CTAs per SM).  Measured on one
  // GPU against one step in flight (64 registers, four CTAs) and four (128 registers, two CTAs): two is best or within 4 % of
  // the best on every decode shape of a Llama-3-8B layer and of its 2- and 8-way shards; four wins only on long reductions
  // of few rows and loses 15-25 % on the large matrices, one the other way round.  The steps are consumed in their order, so
  // the sums are those of a plain loop.
  for (int sc = krank * sec_per_cta; sc < (krank + 1) * sec_per_cta; ++sc) {
    const int step0 = sc * per_section, nsteps = min(nsteps_all, step0 + per_section);   // this section's steps: [step0, nsteps)
    acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
    int st = step0 + warp;
    for (; st + kGemvWarps < nsteps; st += 2 * kGemvWarps) {
      const GemvStep s0 = load_step(st), s1 = load_step(st + kGemvWarps);
      consume(s0); consume(s1);
    }
    for (; st < nsteps; st += kGemvWarps) consume(load_step(st));
    // partial sums of this warp and section: c0, c1 -> (row gq, columns 2 q, 2 q + 1); c2, c3 -> row gq + 8
    float *p = &part[sc * kGemvWarps + warp][0][0];
    if (ksplit == 1) {
      p[gq * 8 + 2 * q] = acc[0]; p[gq * 8 + 2 * q + 1] = acc[1];
      p[(gq + 8) * 8 + 2 * q] = acc[2]; p[(gq + 8) * 8 + 2 * q + 1] = acc[3];
    } else {
      sm100::st_peer_f32(p + gq * 8 + 2 * q, 0, acc[0]); sm100::st_peer_f32(p + gq * 8 + 2 * q + 1, 0, acc[1]);
      sm100::st_peer_f32(p + (gq + 8) * 8 + 2 * q, 0, acc[2]); sm100::st_peer_f32(p + (gq + 8) * 8 + 2 * q + 1, 0, acc[3]);
    }
  }
  if (ksplit == 1) {
    __syncthreads();
  } else {
    sm100::cluster_arrive_release();
    if (krank != 0) return;          // the first CTA stays until every peer has arrived, so the stores above land in live memory
    sm100::cluster_wait_acquire();
  }

  // ---- epilogue on the slice: thread t < 128 owns (row t % 16, column t / 16) ----
  const Epilogue &e = g.e;
  const int ri = tid & 15, cj = tid >> 4, i = i0 + ri;
  const bool live = tid < 128 && i < gm && cj < gn;
  float v = 0.f, amax = 0.f;
  if (live) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < sections * kGemvWarps; ++w) s = __fadd_rn(s, part[w][ri][cj]);
    s = __fmul_rn(s, ue ? 65536.f : 256.f);
    float colp = epi_col_part(e, cj);
    if (g.ex.mask & kExNorm) colp = __fmul_rn(colp, colscale[cj]);
    v = epi_value(e, i, cj, s, epi_scale(e, epi_row_part(e, i), colp));
  }
  auto store_d = [&](size_t idx, float val) { store_dense(e.d_dtype, e.d, idx, val); };
  if (!(g.ex.mask & (kExSwiglu | kExOut2))) {
    if (live) { store_d((size_t)cj * e.ldd + i, v); amax = fabsf(v); }
  } else {
    if (tid < 128) vtile[cj][ri] = v;
    __syncthreads();
    if (g.ex.mask & kExSwiglu) {
      if (live && ri < 8) {
        const float h = silu_mul(vtile[cj][ri], vtile[cj][ri + 8]);
        store_d((size_t)cj * e.ldd + (i0 >> 1) + ri, h);
        amax = fabsf(h);
      }
    } else if (live) {
      store_d((size_t)cj * e.ldd + i, v);
      amax = fabsf(v);
    }
    if (g.ex.mask & kExOut2) {
      if (live) store_dense(g.ex.d2_dtype, g.ex.d2, (size_t)cj * g.ex.ldd2 + i, __fmul_rn(v, load_dense(g.ex.w2_dtype, g.ex.w2, i)));
      if (live && ri == 0) {
        float sq = 0.f;
#pragma unroll
        for (int r = 0; r < 16; ++r) sq = __fadd_rn(sq, __fmul_rn(vtile[cj][r], vtile[cj][r]));
        g.ex.sq[(size_t)cj * g.ex.ld_sq + (i0 >> 4)] = sq;
      }
    }
  }
  if (e.amax && tid < 128) warp_amax_commit(e.amax, amax);
  if (g.tp.world > 1 && (g.tp.deferred == 0 || (g.tp.deferred & 2))) {
    // All-gather fused into this kernel: the CTA that finishes last copies the rank's outputs (n rows of the activation
    // buffer, just written and still in L2) into every peer's buffer with 16-byte stores and joins the ranks' barrier.
    __shared__ int last_cta;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      unsigned *ctas = (unsigned *)(g.tp.flags[g.tp.rank] + kFlagCtas);
      const unsigned ticket = atomicAdd(ctas, 1u);
      last_cta = ticket == gridDim.x / ksplit - 1;   // one ticket per slice
      if (last_cta) *ctas = 0;
    }
    __syncthreads();
    if (last_cta) {
      __threadfence();
      const int esz = dense_bytes(e.d_dtype);
      const int drows = (g.ex.mask & kExSwiglu) ? gm / 2 : gm;
      const int vec_per_row = drows * esz / 16;
      for (int v = tid; v < vec_per_row * gn; v += blockDim.x) {
        const int j = v / vec_per_row, c = v - j * vec_per_row;
        uint8_t *src = (uint8_t *)e.d + ((size_t)j * e.ldd * esz + (size_t)c * 16);
        const uint4 x = __ldcg((const uint4 *)src);
        for (int p = 0; p < g.tp.world; ++p)
          if (p != g.tp.rank) *(uint4 *)(src + g.tp.delta[p]) = x;
      }
      __syncthreads();   // the flags' release stores order every thread's copies (see tp_barrier_cta)
      // deferred form: tell the peers and leave; the next kernel of every rank waits for the posts at its start
      if (g.tp.deferred & 2) tp_post_epoch(g.tp.flags, g.tp.world, g.tp.rank);
      else tp_barrier_cta(g.tp.flags, g.tp.world, g.tp.rank, g.tp.status, g.tp.tag, g.tp.wait_cycles);
    }
  }
}

bool gemv_supports(const GemmArgs &g) {
  return g.n >= 1 && g.n <= 8 && g.B.dtype == NVFP4A_BF16 && g.k > 0 && ((uintptr_t)g.B.data & 15) == 0 &&
         (g.A.image || ((uintptr_t)g.A.sc & 1) == 0);
}

cudaError_t launch_gemv(const GemmArgs &g, cudaStream_t s) {
  GemvArgs a;
  a.m = g.m; a.n = g.n; a.k = g.k;
  a.A = g.A;
  a.x = (const uint16_t *)g.B.data; a.ldx = g.B.ld;
  a.e = g.e; a.ex = g.x; a.tp = g.tp;
  a.tp.status = kernel_status_device_ptr();
  a.tp.tag = next_launch_tag();
  a.tp.wait_cycles = tp_wait_limit();
  a.sections = g.k >= 8192 ? (g.k >= 12288 ? 4 : 2) : 1;   // by k alone: see the header
  const int slices = (g.m + 15) / 16;
  a.ksplit = slices * a.sections <= 2 * device_sms() ? a.sections : 1;   // a cluster per slice only while the CTAs fit the GPU at once
  void (*kern)(GemvArgs) = a.A.image ? gemv_kernel<2> : a.A.sld < 0 ? gemv_kernel<1> : gemv_kernel<0>;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = dim3(slices * a.ksplit, 1, 1);
  cfg.blockDim = dim3(kGemvWarps * 32, 1, 1);
  cfg.stream = s;
  // (No programmatic dependent launch here: measured on the decode step of a 32-layer stack it costs 5-7 us per layer, this
  // kernel's CTAs taking their places on the SMs while the FP4 GEMV before or after them still needs whole SMs.)
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = a.ksplit; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = a.ksplit > 1 ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, a);
}

}  // namespace nvb
