// CUDA-core GEMM for every operand combination of the C ABI, in the reference's exact "tiled" order
// (include/nvfp4effma.h:78-84 there): NVFP4 x NVFP4 / INT8 -- per output and 16-block an exact integer sum p, then
// acc = fma(p * sa, sb, acc) with blocks ascending in k and a final * 1/4 or * 1/2; NVFP4 x dense -- acc = fma(a * sa, b, acc)
// per MAC, k ascending.  Outputs are therefore bit-identical to the reference's tiled CUDA-core kernels.
//
// This is the library's correctness anchor and the route for operand formats that have no tensor-core form on sm_100a
// (UE5M3 block scales, FP32 / FP16 activations, INT8 activations with FP32 block scales).  It carries the plain and the
// extended epilogue.  One CTA computes a 16-row slice x 16 columns; it is not a fast path.
#include "operands.cuh"

namespace nvb {

constexpr int GR = 16, GC = 16, GK = 64;  // rows, columns, k per staging step

// GROUPED (nvfp4a_gemm_grouped, reference include/nvfp4effma.h:104-116): A is the stack of `groups` weights of g.m rows each,
// group q owns the columns (rows of B, D, C) [seg[q], seg[q + 1]); blockIdx.x counts 16-column tiles over the groups in order, each
// group's last tile partial, and the CTA finds its group by walking seg (device memory: the row counts never visit the host).
template <bool GROUPED>
__global__ void __launch_bounds__(256) gemm_generic_kernel(GemmArgs g, const int *__restrict__ seg, int groups) {
  __shared__ __align__(16) int8_t a_i8[GR][GK];
  __shared__ float a_sc[GR][GK / 16];
  __shared__ __align__(16) int8_t b_i8[GC][GK];
  __shared__ float b_sc[GC][GK / 16];
  __shared__ float b_f32[GC][GK + 1];
  __shared__ float vtile[GC][GR];   // epilogue values of the slice (extended epilogue)
  __shared__ float colscale[GC];

  const int tid = threadIdx.x, ri = tid & 15, cj = tid >> 4;
  int j0 = blockIdx.x * GC, ro = 0;   // ro: first row of this group's weight in the stacked A (and in its per-row globals, bias)
  if (GROUPED) {
    int t = blockIdx.x, q = 0, lo = 0, hi = 0;
    for (; q < groups; ++q) {
      lo = seg[q]; hi = seg[q + 1];
      const int tiles = (hi - lo + GC - 1) / GC;
      if (t < tiles) break;
      t -= tiles;
    }
    if (q == groups || hi > g.n) return;   // past the last group's tiles (the grid is sized for the worst case), or seg beyond `rows`
    j0 = lo + t * GC;
    g.n = hi;
    ro = q * g.m;
  }
  const int i0 = blockIdx.y * GR;
  const int i = i0 + ri, j = j0 + cj;
  const int bt = g.B.dtype;
  const bool fp4b = bt == NVFP4A_NVFP4, q8b = bt == NVFP4A_INT8, blocked = fp4b || q8b;
  const bool ue_a = g.A.ue != 0;

  if (g.x.mask & kExNorm) {  // s_j of the CTA's columns: warp w computes columns w and w + 8
    const int w = tid >> 5, lane = tid & 31;
    for (int c = w; c < GC; c += 8) {
      const float s = warp_norm_scale(g.x, j0 + c < g.n ? j0 + c : 0, lane);
      if (lane == 0) colscale[c] = s;
    }
  }

  float acc = 0.f;
  for (int k0 = 0; k0 < g.k; k0 += GK) {
    __syncthreads();
    if (tid < 128) {  // 64 (row, block) items of A, 64 (column, block) items of B
      const bool is_a = tid < 64;
      const int item = tid & 63, rr = item >> 2, bb = item & 3, kb = (k0 >> 4) + bb;
      const bool kin = k0 + 16 * bb < g.k;
      if (is_a) {
        const int row = i0 + rr;
        uint2 w = make_uint2(0, 0);
        float sc = 0.f;
        if (row < g.m && kin) { w = g.A.block(ro + row, kb); sc = scale_to_f32(g.A.scale_code(ro + row, kb), ue_a); }
#pragma unroll
        for (int e = 0; e < 16; ++e) a_i8[rr][16 * bb + e] = (int8_t)e2m1_x2(((e < 8 ? w.x : w.y) >> (4 * (e & 7))) & 15u);
        a_sc[rr][bb] = sc;
      } else {
        const int col = j0 + rr;
        const bool in = col < g.n && kin;
        if (fp4b) {
          uint2 w = make_uint2(0, 0);
          float sc = 0.f;
          if (in) { w = g.B.q.block(col, kb); sc = g.B.q.scale(col, kb); }
#pragma unroll
          for (int e = 0; e < 16; ++e) b_i8[rr][16 * bb + e] = (int8_t)e2m1_x2(((e < 8 ? w.x : w.y) >> (4 * (e & 7))) & 15u);
          b_sc[rr][bb] = sc;
        } else if (q8b) {
          uint4 w = make_uint4(0, 0, 0, 0);
          float sc = 0.f;
          if (in) {
            w = *(const uint4 *)((const int8_t *)g.B.data + (size_t)col * g.B.ld + 16 * kb);
            sc = g.B.s8[(size_t)col * g.B.lds8 + kb];
          }
          *(uint4 *)&b_i8[rr][16 * bb] = w;
          b_sc[rr][bb] = sc;
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) b_f32[rr][16 * bb + e] = in ? load_dense(bt, g.B.data, (size_t)col * g.B.ld + 16 * kb + e) : 0.f;
        }
      }
    }
    __syncthreads();
    const int nb = min(GK, g.k - k0) >> 4;
    if (blocked) {
      for (int bb = 0; bb < nb; ++bb) {
        int p = 0;
#pragma unroll
        for (int q = 0; q < 4; ++q) p = __dp4a(*(const int *)&a_i8[ri][16 * bb + 4 * q], *(const int *)&b_i8[cj][16 * bb + 4 * q], p);
        acc = __fmaf_rn(__fmul_rn((float)p, a_sc[ri][bb]), b_sc[cj][bb], acc);
      }
    } else {
      for (int bb = 0; bb < nb; ++bb) {
        const float sa = a_sc[ri][bb];
#pragma unroll
        for (int e = 0; e < 16; ++e)
          acc = __fmaf_rn(__fmul_rn(0.5f * (float)a_i8[ri][16 * bb + e], sa), b_f32[cj][16 * bb + e], acc);
      }
    }
  }
  if (blocked) acc = __fmul_rn(acc, fp4b ? 0.25f : 0.5f);

  // ---- epilogue ----
  const bool live = i < g.m && j < g.n;
  const Epilogue &e = g.e;
  float amax = 0.f, v = 0.f;
  if (live) {
    float colp = epi_col_part(e, j);
    if (g.x.mask & kExNorm) colp = __fmul_rn(colp, colscale[cj]);
    if (GROUPED) {
      v = __fmul_rn(acc, epi_scale(e, epi_row_part(e, ro + i), colp));
      if (e.bias) v = __fadd_rn(v, load_dense(e.bias_dtype, e.bias, ro + i));
      if (e.beta != 0.f) v = __fmaf_rn(e.beta, load_dense(e.c_dtype, e.c, (size_t)j * e.ldc + i), v);
    } else {
      v = epi_value(e, i, j, acc, epi_scale(e, epi_row_part(e, i), colp));
    }
  }
  if (!(g.x.mask & (kExSwiglu | kExOut2))) {
    if (live) { store_dense(e.d_dtype, e.d, (size_t)j * e.ldd + i, v); amax = fabsf(v); }
  } else {
    __syncthreads();
    vtile[cj][ri] = v;
    __syncthreads();
    if (g.x.mask & kExSwiglu) {
      if (live && ri < 8) {  // gate rows 0..7 of the slice, their up rows 8..15
        const float h = silu_mul(vtile[cj][ri], vtile[cj][ri + 8]);
        store_dense(e.d_dtype, e.d, (size_t)j * e.ldd + (i0 >> 1) + ri, h);
        amax = fabsf(h);
      }
    } else if (live) {
      store_dense(e.d_dtype, e.d, (size_t)j * e.ldd + i, v);
      amax = fabsf(v);
    }
    if (g.x.mask & kExOut2) {
      if (live) store_dense(g.x.d2_dtype, g.x.d2, (size_t)j * g.x.ldd2 + i, __fmul_rn(v, load_dense(g.x.w2_dtype, g.x.w2, i)));
      if (ri == 0 && live) {  // one thread per (slice, column): 16 rows ascending
        float q = 0.f;
#pragma unroll
        for (int r = 0; r < 16; ++r) q = __fadd_rn(q, __fmul_rn(vtile[cj][r], vtile[cj][r]));
        g.x.sq[(size_t)j * g.x.ld_sq + (i0 >> 4)] = q;
      }
    }
  }
  if (e.amax) warp_amax_commit(e.amax, amax);
}

cudaError_t launch_gemm_generic(const GemmArgs &g, cudaStream_t s) {
  // grid.y is limited to 65535 slices of 16 rows (m up to ~1M), grid.x unbounded in practice
  const dim3 grid((g.n + GC - 1) / GC, (g.m + GR - 1) / GR);
  if (grid.y > 65535) return cudaErrorInvalidConfiguration;
  gemm_generic_kernel<false><<<grid, 256, 0, s>>>(g, nullptr, 0);
  return cudaGetLastError();
}

// g.m = rows of ONE group's weight, g.n = the bound `rows` on seg[groups]; every group may end in a partial tile
cudaError_t launch_gemm_grouped(const GemmArgs &g, const int *seg, int groups, cudaStream_t s) {
  const dim3 grid((g.n + GC - 1) / GC + groups, (g.m + GR - 1) / GR);
  if (grid.y > 65535) return cudaErrorInvalidConfiguration;
  gemm_generic_kernel<true><<<grid, 256, 0, s>>>(g, seg, groups);
  return cudaGetLastError();
}

}  // namespace nvb
