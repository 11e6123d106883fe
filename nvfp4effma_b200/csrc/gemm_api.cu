// GEMM / GEMV side of the C ABI: argument validation, epilogue set-up and routing for nvfp4a_gemm, _gemm_ex, _gemm_dual,
// _gemm_grouped, _gemm_tc(_ex), _gemv_tc(_ex) and the image entry points.  Conditions and status codes follow the
// reference's host layer (src/gemm_nvfp4effma.cu:465-557, :614-930 there); everything is checked before anything is launched.
//
// Routing on sm_100a:
//   n <= kGemvMaxN (or k == 0)                          -> streaming split-k GEMV (gemv.cu) when it takes the operand types
//   NVFP4 x NVFP4, E4M3 scales on both                  -> tcgen05 kind::mxf4nvf4 block-scaled GEMM (gemm_w4a4.cu)
//   NVFP4 (E4M3 scales) x BF16                          -> tcgen05 kind::f16 GEMM on weights expanded to exact BF16 (gemm_w4a16.cu)
//   anything else                                       -> exact CUDA-core GEMM (gemm_generic.cu)
#include <stdio.h>
#include <stdlib.h>
#include <atomic>
#include "operands.cuh"

namespace nvb {

constexpr int kGemvMaxN = 8;

static bool dense_t(const nvfp4a_tensor *t) { return t->dtype >= NVFP4A_BF16 && t->dtype <= NVFP4A_FP32; }
static bool blocked_t(const nvfp4a_tensor *t) { return t->dtype == NVFP4A_NVFP4 || t->dtype == NVFP4A_INT8; }
static bool aligned(const void *p, unsigned a) { return ((uintptr_t)p & (a - 1)) == 0; }
static bool dense_dt(nvfp4a_dtype t) { return t >= NVFP4A_BF16 && t <= NVFP4A_FP32; }

// Route override (nvfp4a_b200_set_route): 0 = automatic, 1 = always the exact CUDA-core kernel, 2 = automatic without the
// FP4 tensor-core GEMV, 3 = automatic without the tensor-core W4A8 GEMM (INT8 activations then keep the exact integer block sums
// of the DP4A kernel).  The environment variable NVFP4A_B200_ROUTE=generic sets the initial value to 1.
static std::atomic<int> g_route{-1};
static int forced_route() {
  int r = g_route.load();
  if (r < 0) {
    const char *v = getenv("NVFP4A_B200_ROUTE");
    r = v && !strcmp(v, "generic") ? 1 : 0;
    g_route = r;
  }
  return r;
}

static Epilogue make_epilogue(float alpha, const nvfp4a_tensor *A, const nvfp4a_tensor *B, float beta, const nvfp4a_tensor *C, int ldc,
                              const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias) {
  const bool blocked = blocked_t(B);
  const bool c_is_d = beta != 0.f && (!C || !C->data);  // accumulate into D
  Epilogue e;
  e.ga = A->global_scale;
  e.gb = blocked ? B->global_scale : nullptr;
  e.gf = amax_factor(A, blocked ? B : nullptr);
  e.ga_stride = (A->flags & NVFP4A_GLOBAL_PER_ROW) ? 1 : 0;
  e.gb_stride = (B->flags & NVFP4A_GLOBAL_PER_ROW) ? 1 : 0;
  e.alpha = alpha; e.beta = beta;
  const nvfp4a_tensor *Cx = c_is_d ? D : C;
  e.c = beta != 0.f ? Cx->data : nullptr;
  e.ldc = beta != 0.f ? (c_is_d ? ldd : ldc) : 0;
  e.c_dtype = beta != 0.f ? Cx->dtype : NVFP4A_FP32;
  e.d = D->data; e.ldd = ldd; e.d_dtype = D->dtype; e.amax = D->amax;
  e.bias = bias && bias->data ? bias->data : nullptr;
  e.bias_dtype = bias ? bias->dtype : NVFP4A_FP32;
  return e;
}

static nvfp4a_status make_epilogue_ex(const char *fn, const nvfp4a_epilogue *x, int m, float beta, int ldd, EpilogueEx *ex) {
  memset(ex, 0, sizeof *ex);
  if (!x) return NVFP4A_OK;
  if (x->norm_parts) {
    if (x->norm_nparts <= 0 || x->norm_ld < x->norm_nparts || !(x->norm_inv_n > 0.f) || !(x->norm_eps >= 0.f))
      return fail(NVFP4A_INVALID_VALUE, "%s: norm_parts needs norm_nparts > 0, norm_ld >= norm_nparts, norm_inv_n > 0 and norm_eps >= 0", fn);
    ex->norm_parts = x->norm_parts; ex->norm_nparts = x->norm_nparts; ex->norm_ld = x->norm_ld;
    ex->norm_inv_n = x->norm_inv_n; ex->norm_eps = x->norm_eps;
    ex->mask |= kExNorm;
  }
  if (x->swiglu) {
    if (m % 16 || beta != 0.f || x->d2) return fail(NVFP4A_INVALID_VALUE, "%s: swiglu needs m %% 16 == 0, beta == 0 and no second output", fn);
    if (ldd < m / 2) return fail(NVFP4A_INVALID_VALUE, "%s: swiglu: ldd = %d is below m / 2 = %d", fn, ldd, m / 2);
    ex->mask |= kExSwiglu;
  }
  if (x->d2) {
    if (m % 16 || !x->w2 || !x->sq || !dense_dt(x->d2_dtype) || !dense_dt(x->w2_dtype) || x->ldd2 < m || x->ld_sq < m / 16)
      return fail(NVFP4A_INVALID_VALUE, "%s: the second output needs m %% 16 == 0, w2 and sq, dense d2 / w2 dtypes, ldd2 >= m and ld_sq >= m / 16", fn);
    ex->d2 = x->d2; ex->d2_dtype = x->d2_dtype; ex->ldd2 = x->ldd2; ex->w2 = x->w2; ex->w2_dtype = x->w2_dtype;
    ex->sq = x->sq; ex->ld_sq = x->ld_sq;
    ex->mask |= kExOut2;
  }
  return NVFP4A_OK;
}

static nvfp4a_status check_epilogue_operands(const char *fn, int m, float beta, const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd,
                                             const nvfp4a_tensor *bias, int ex_mask) {
  const int drows = (ex_mask & kExSwiglu) ? m / 2 : m;
  if (ldd < drows) return fail(NVFP4A_INVALID_VALUE, "%s: ldd = %d is below the %d rows of D", fn, ldd, drows);
  if (bias && bias->data && !dense_t(bias)) return fail(NVFP4A_INVALID_VALUE, "%s: bias has dtype %d (BF16, FP16 or FP32)", fn, (int)bias->dtype);
  if (beta != 0.f && C && C->data && !dense_t(C)) return fail(NVFP4A_INVALID_VALUE, "%s: C has dtype %d (BF16, FP16 or FP32)", fn, (int)C->dtype);
  if (beta != 0.f && C && C->data && ldc < m) return fail(NVFP4A_INVALID_VALUE, "%s: ldc = %d is below m = %d", fn, ldc, m);
  return NVFP4A_OK;
}

// kernel the last GEMM call of this thread launched (nvfp4a_b200_last_route): 1 CUDA cores, 2 mma.sync GEMV, 3 FP4 tensor-core
// GEMV, 4 W4A4 tcgen05 GEMM, 5 W4A16 tcgen05 GEMM, 6 DP4A GEMV for INT8 / NVFP4 activations, 7 DP4A GEMM for INT8 activations,
// 8 W4A8 on the W4A16 tcgen05 kernel (INT8 activations as three BF16 planes)
static thread_local int g_last_route = 0;
// (defined in gemm_dp4a.cu) the DP4A GEMM over groups of tokens: nvfp4a_gemm_grouped with INT8 activations
cudaError_t launch_gemm_dp4a_grouped(const GemmArgs &g, const int *seg, int groups, cudaStream_t s);
// set around the call of an entry that must not allocate (nvfp4a_b200_gemm_ex_static)
static thread_local int g_no_alloc = 0;

// The workspace of nvfp4a_gemm_tc_ex holds the RMSNorm column scales of up to kWorkspaceTokens tokens while a call runs (a
// small kernel fills it before the GEMM, a memset restores the zeros after it); the other tensor-core calls leave it alone.
constexpr int kWorkspaceTokens = 16384;

extern "C" nvfp4a_status nvfp4a_b200_tp_gather(void *const *buffers, void *const *flags, int world, int rank, int rows, long long row_pitch_bytes,
                                               long long col_offset_bytes, long long shard_bytes, cudaStream_t stream);

static nvfp4a_status dispatch(const char *fn, const GemmArgs &g, cudaStream_t stream) {
  cudaError_t err;
  const bool gemv = g.k == 0 || g.n <= kGemvMaxN;
  if (g.tp.world > 1 && g.tp.deferred) {
    // The deferred tensor-parallel form: the mma.sync GEMV waits at its start and (bit 1) pushes at its end; the FP4 tensor-core
    // GEMV only waits, so with bit 1 unset either may run and the caller's nvfp4a_b200_tp_gather_post follows.
    if (!(gemv && gemv_supports(g))) return fail(NVFP4A_NOT_SUPPORTED, "%s: the deferred tensor-parallel form takes 1 to 8 BF16 activation vectors", fn);
    if (!(g.tp.deferred & 2) && g.k > 0 && forced_route() != 2 && gemv_fp4_supports(g)) { g_last_route = 3; return cuda_fail(launch_gemv_fp4(g, stream), fn); }
    g_last_route = 2;
    return cuda_fail(launch_gemv(g, stream), fn);
  }
  if (forced_route() == 1) { g_last_route = 1; err = launch_gemm_generic(g, stream); }
  else if (gemv && g.k > 0 && forced_route() != 2 && gemv_fp4_supports(g)) { g_last_route = 3; err = launch_gemv_fp4(g, stream); }
  else if (gemv && gemv_supports(g)) { g_last_route = 2; err = launch_gemv(g, stream); }
  else if (gemv && g.k > 0 && gemv_blocked_supports(g)) { g_last_route = 6; err = launch_gemv_blocked(g, stream); }
  else if (!gemv && gemm_w4a4_supports(g)) { g_last_route = 4; err = launch_gemm_w4a4(g, stream); }
  else if (!gemv && gemm_w4a16_supports(g)) { g_last_route = 5; err = launch_gemm_w4a16(g, stream); }
  else if (!gemv && forced_route() != 3 && gemm_w4a8_tc_supports(g)) { g_last_route = 8; err = launch_gemm_w4a8_tc(g, stream); }
  else if (!gemv && gemm_dp4a_supports(g)) { g_last_route = 7; err = launch_gemm_dp4a(g, stream); }
  else { g_last_route = 1; err = launch_gemm_generic(g, stream); }
  if (err == cudaSuccess && g.tp.world > 1 && g_last_route != 2) {
    // only the mma.sync GEMV pushes its results to the peers itself; after any other kernel a copy launch does it
    void *bufs[kMaxRanks], *flags[kMaxRanks];
    for (int p = 0; p < g.tp.world; ++p) { bufs[p] = g.tp.local_base + g.tp.delta[p]; flags[p] = g.tp.flags[p]; }
    const int esz = dense_bytes(g.e.d_dtype);
    const long long drows = (g.x.mask & kExSwiglu) ? g.m / 2 : g.m;
    const bool pushed = g_last_route == 5 && gemm_w4a16_pushes(g);   // the W4A16 GEMM stored to the peers itself: only the barrier is left
    return nvfp4a_b200_tp_gather(bufs, flags, g.tp.world, g.tp.rank, pushed ? 0 : g.n, (long long)g.e.ldd * esz,
                                 (long long)((uint8_t *)g.e.d - g.tp.local_base), drows * esz, stream);
  }
  return cuda_fail(err, fn);
}

static BOperand make_b(const nvfp4a_tensor *B, int ldb, int ldsb, int k, bool image) {
  BOperand b;
  memset(&b, 0, sizeof b);
  b.dtype = B->dtype;
  if (B->dtype == NVFP4A_NVFP4) {
    b.q.data = (const uint8_t *)B->data; b.q.sc = (const uint8_t *)B->block_scale; b.q.ld = ldb; b.q.sld = ldsb;
    b.q.image = image; b.q.ktiles = (k + kImgK - 1) / kImgK; b.q.ue = (B->flags & NVFP4A_SCALES_UE5M3) ? 1 : 0;
  } else {
    b.data = B->data; b.ld = ldb; b.s8 = (const float *)B->block_scale; b.lds8 = ldsb;
  }
  return b;
}

// nvfp4a_gemm / nvfp4a_gemm_ex
static nvfp4a_status gemm_run(const char *fn, int m, int n, int k, float alpha, const nvfp4a_tensor *A, int lda, const nvfp4a_tensor *B, int ldb,
                              float beta, const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias,
                              const EpilogueEx &ex, cudaStream_t stream, bool validate_only = false, int a_groups = 1, GemmArgs *args_out = nullptr) {
  // a_groups > 1 (nvfp4a_gemm_grouped): A holds a_groups stacked weights of m rows; nothing is launched, the arguments go to args_out
  if (!A || !B || !D || !A->data || !B->data || !D->data) return fail(NVFP4A_INVALID_VALUE, "%s: A, B or D (or its data pointer) is NULL", fn);
  if (m < 0 || n < 0 || k < 0) return fail(NVFP4A_INVALID_VALUE, "%s: negative size (m = %d, n = %d, k = %d)", fn, m, n, k);
  if (A->dtype != NVFP4A_NVFP4) return fail(NVFP4A_NOT_SUPPORTED, "%s: A must be NVFP4 (dtype %d)", fn, (int)A->dtype);
  if (!blocked_t(B) && !dense_t(B)) return fail(NVFP4A_INVALID_VALUE, "%s: B has an invalid dtype %d", fn, (int)B->dtype);
  if (!dense_t(D)) return fail(NVFP4A_INVALID_VALUE, "%s: D must be BF16, FP16 or FP32 (dtype %d)", fn, (int)D->dtype);
  if (m == 0 || n == 0) return NVFP4A_OK;
  if (k % 64) return fail(NVFP4A_INVALID_VALUE, "%s: k = %d is not a multiple of 64", fn, k);
  if (lda % 64 || ldb % 64) return fail(NVFP4A_INVALID_VALUE, "%s: lda = %d and ldb = %d must be multiples of 64", fn, lda, ldb);
  if (lda < k || ldb < k) return fail(NVFP4A_INVALID_VALUE, "%s: lda = %d or ldb = %d is below k = %d", fn, lda, ldb, k);
  if (!aligned(A->data, 16) || !aligned(B->data, 16)) return fail(NVFP4A_INVALID_VALUE, "%s: A and B data must be 16-byte aligned", fn);
  int ldsa = 0, ldsb = 0;
  for (int which = 0; which < 2; ++which) {
    const nvfp4a_tensor *t = which ? B : A;
    if (!blocked_t(t)) {
      if (t->flags) return fail(NVFP4A_INVALID_VALUE, "%s: flags apply to NVFP4 tensors only (dtype %d)", fn, (int)t->dtype);
      continue;
    }
    const unsigned al = t->dtype == NVFP4A_INT8 ? 16 : 4;
    if (!t->block_scale) return fail(NVFP4A_INVALID_VALUE, "%s: %s is NVFP4 / INT8 but has no block_scale", fn, which ? "B" : "A");
    if (!aligned(t->block_scale, al) || t->ld_scale % 4 || (t->ld_scale && t->ld_scale < k / 16))
      return fail(NVFP4A_INVALID_VALUE, "%s: block scales of %s must be %u-byte aligned, ld_scale a multiple of 4 and >= k / 16 (ld_scale = %d)",
                  fn, which ? "B" : "A", al, t->ld_scale);
    if (nvfp4a_status st = check_scales(fn, which ? "B" : "A", t, which ? n : m * a_groups, k, which ? &ldsb : &ldsa)) return st;
  }
  if (nvfp4a_status st = check_epilogue_operands(fn, m, beta, C, ldc, D, ldd, bias, ex.mask)) return st;
  if (nvfp4a_status st = check_device()) return st;
  if (ex.mask) {
    if (A->flags & (NVFP4A_SCALES_SWIZZLED | NVFP4A_SCALES_UE5M3))
      return fail(NVFP4A_NOT_SUPPORTED, "%s: the extended epilogue takes A with linear E4M3 block scales", fn);
    if (B->dtype != NVFP4A_BF16 && B->dtype != NVFP4A_INT8) return fail(NVFP4A_NOT_SUPPORTED, "%s: the extended epilogue takes B BF16 or INT8", fn);
  }
  GemmArgs g;
  memset(&g, 0, sizeof g);
  g.m = m; g.n = n; g.k = k;
  g.A.data = (const uint8_t *)A->data; g.A.sc = (const uint8_t *)A->block_scale; g.A.ld = lda; g.A.sld = ldsa;
  g.A.ue = (A->flags & NVFP4A_SCALES_UE5M3) ? 1 : 0;
  g.B = make_b(B, ldb, ldsb, k, false);
  g.e = make_epilogue(alpha, A, B, beta, C, ldc, D, ldd, bias);
  g.x = ex;
  g.no_alloc = g_no_alloc;
  if (args_out) *args_out = g;
  if (validate_only || args_out) return NVFP4A_OK;
  return dispatch(fn, g, stream);
}

// record kinds of the image API: 1 weight image, 2 NVFP4 activations, 3 INT8, 4 BF16; 0 invalid
static int image_kind(int operand, nvfp4a_dtype dtype) {
  if (operand == NVFP4A_TC_A16 || operand == NVFP4A_TC_A8) return dtype == NVFP4A_NVFP4 ? 1 : 0;
  if (operand != NVFP4A_TC_B) return 0;
  return dtype == NVFP4A_NVFP4 ? 2 : dtype == NVFP4A_INT8 ? 3 : dtype == NVFP4A_BF16 ? 4 : 0;
}
// INT8 activation image: [rows][k] int8, then (16-byte aligned) [rows][k / 16] FP32 scales.  BF16: [rows][k] values.
static size_t int8_image_scale_offset(int rows, int k) { return ((size_t)rows * k + 15) / 16 * 16; }

static nvfp4a_status check_flags_only(const char *fn, const nvfp4a_tensor *t) {
  const unsigned known = NVFP4A_SCALES_SWIZZLED | NVFP4A_SCALES_UE5M3 | NVFP4A_GLOBAL_AMAX | NVFP4A_GLOBAL_PER_ROW;
  if (t->dtype != NVFP4A_NVFP4 && t->flags) return fail(NVFP4A_INVALID_VALUE, "%s: flags apply to NVFP4 tensors only", fn);
  if (t->flags & ~known) return fail(NVFP4A_INVALID_VALUE, "%s: unknown flag bits 0x%x", fn, t->flags & ~known);
  if (t->dtype == NVFP4A_NVFP4 && scale_max_of(t) == 0.f) return fail(NVFP4A_INVALID_VALUE, "%s: scale_max = %d is not valid", fn, t->scale_max);
  if ((t->flags & NVFP4A_GLOBAL_PER_ROW) && !t->global_scale) return fail(NVFP4A_INVALID_VALUE, "%s: NVFP4A_GLOBAL_PER_ROW without global_scale", fn);
  return NVFP4A_OK;
}

static nvfp4a_status gemm_tc_run(const char *fn, int m, int n, int k, float alpha, const nvfp4a_tensor *A, const nvfp4a_tensor *B, float beta,
                                 const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias, void *workspace,
                                 const EpilogueEx &ex, cudaStream_t stream, const TpPush *tp = nullptr) {
  if (!A || !B || !D || !A->data || !B->data || !D->data || !workspace)
    return fail(NVFP4A_INVALID_VALUE, "%s: A, B, D (or a data pointer) or the workspace is NULL", fn);
  if (m < 0 || n < 0 || k < 0) return fail(NVFP4A_INVALID_VALUE, "%s: negative size (m = %d, n = %d, k = %d)", fn, m, n, k);
  if (A->dtype != NVFP4A_NVFP4) return fail(NVFP4A_NOT_SUPPORTED, "%s: A must be NVFP4 (dtype %d)", fn, (int)A->dtype);
  if (!image_kind(NVFP4A_TC_B, B->dtype)) return fail(NVFP4A_NOT_SUPPORTED, "%s: B must be NVFP4, INT8 or BF16 (dtype %d)", fn, (int)B->dtype);
  if (!dense_t(D)) return fail(NVFP4A_INVALID_VALUE, "%s: D must be BF16, FP16 or FP32 (dtype %d)", fn, (int)D->dtype);
  if (m == 0 || n == 0) return NVFP4A_OK;
  if (k % 64) return fail(NVFP4A_INVALID_VALUE, "%s: k = %d is not a multiple of 64", fn, k);
  if (!aligned(A->data, 16) || !aligned(B->data, 16) || !aligned(workspace, 16))
    return fail(NVFP4A_INVALID_VALUE, "%s: the images and the workspace must be 16-byte aligned", fn);
  if (nvfp4a_status st = check_flags_only(fn, A)) return st;
  if (nvfp4a_status st = check_flags_only(fn, B)) return st;
  if (nvfp4a_status st = check_epilogue_operands(fn, m, beta, C, ldc, D, ldd, bias, ex.mask)) return st;
  if (nvfp4a_status st = check_device()) return st;
  if (ex.mask) {
    if (A->flags & NVFP4A_SCALES_UE5M3) return fail(NVFP4A_NOT_SUPPORTED, "%s: the extended epilogue takes A with E4M3 block scales", fn);
    if (B->dtype != NVFP4A_BF16 && B->dtype != NVFP4A_INT8) return fail(NVFP4A_NOT_SUPPORTED, "%s: the extended epilogue takes B BF16 or INT8", fn);
  }
  GemmArgs g;
  memset(&g, 0, sizeof g);
  g.m = m; g.n = n; g.k = k;
  g.A.data = (const uint8_t *)A->data; g.A.image = 1; g.A.ktiles = (k + kImgK - 1) / kImgK;
  g.A.ue = (A->flags & NVFP4A_SCALES_UE5M3) ? 1 : 0;
  if (B->dtype == NVFP4A_NVFP4) g.B = make_b(B, 0, 0, k, true);
  else if (B->dtype == NVFP4A_INT8) {
    g.B = make_b(B, k, k / 16, k, false);
    g.B.s8 = (const float *)((const uint8_t *)B->data + int8_image_scale_offset(n, k));
  } else g.B = make_b(B, k, 0, k, false);
  g.e = make_epilogue(alpha, A, B, beta, C, ldc, D, ldd, bias);
  g.x = ex;
  if (tp) g.tp = *tp;
  // RMSNorm column scales once per call instead of once per tile of weight rows (the tcgen05 W4A16 GEMM reads them)
  const bool stage_scales = (ex.mask & kExNorm) && n > kGemvMaxN && n <= kWorkspaceTokens && forced_route() != 1 && gemm_w4a16_supports(g);
  if (stage_scales) {
    if (nvfp4a_status st = cuda_fail(launch_norm_scales(ex, n, (float *)workspace, stream), fn)) return st;
    g.x.colscales = (const float *)workspace;
  }
  const nvfp4a_status st = dispatch(fn, g, stream);
  if (stage_scales && st == NVFP4A_OK) return cuda_fail(cudaMemsetAsync(workspace, 0, (size_t)n * sizeof(float), stream), fn);
  return st;
}

static nvfp4a_status gemv_tc_run(const char *fn, int m, int n, int k, float alpha, const nvfp4a_tensor *A, const nvfp4a_tensor *B, int ldb,
                                 float beta, const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias,
                                 const EpilogueEx &ex, cudaStream_t stream, const TpPush *tp = nullptr) {
  if (!A || !B || !D || !A->data || !B->data || !D->data) return fail(NVFP4A_INVALID_VALUE, "%s: A, B or D (or its data pointer) is NULL", fn);
  if (m < 0 || k < 0 || n < 1 || n > 8) return fail(NVFP4A_INVALID_VALUE, "%s: m = %d, n = %d, k = %d (needs 1 <= n <= 8)", fn, m, n, k);
  if (A->dtype != NVFP4A_NVFP4) return fail(NVFP4A_NOT_SUPPORTED, "%s: A must be NVFP4 (dtype %d)", fn, (int)A->dtype);
  if (!image_kind(NVFP4A_TC_B, B->dtype)) return fail(NVFP4A_NOT_SUPPORTED, "%s: B must be NVFP4, INT8 or BF16 (dtype %d)", fn, (int)B->dtype);
  if (!dense_t(D)) return fail(NVFP4A_INVALID_VALUE, "%s: D must be BF16, FP16 or FP32 (dtype %d)", fn, (int)D->dtype);
  if (m == 0) return NVFP4A_OK;
  if (k % 64) return fail(NVFP4A_INVALID_VALUE, "%s: k = %d is not a multiple of 64", fn, k);
  if (ldb % 64 || ldb < k) return fail(NVFP4A_INVALID_VALUE, "%s: ldb = %d must be a multiple of 64 and >= k = %d", fn, ldb, k);
  if (!aligned(A->data, 16) || !aligned(B->data, 16)) return fail(NVFP4A_INVALID_VALUE, "%s: A's image and B must be 16-byte aligned", fn);
  if (nvfp4a_status st = check_flags_only(fn, A)) return st;
  int ldsb = 0;
  if (B->dtype == NVFP4A_BF16) {
    if (B->flags) return fail(NVFP4A_INVALID_VALUE, "%s: flags apply to NVFP4 tensors only", fn);
  } else {
    const unsigned al = B->dtype == NVFP4A_INT8 ? 16 : 4;
    if (!B->block_scale) return fail(NVFP4A_INVALID_VALUE, "%s: B is NVFP4 / INT8 but has no block_scale", fn);
    if (!aligned(B->block_scale, al) || B->ld_scale % 4 || (B->ld_scale && B->ld_scale < k / 16))
      return fail(NVFP4A_INVALID_VALUE, "%s: B's block scales must be %u-byte aligned, ld_scale a multiple of 4 and >= k / 16 (ld_scale = %d)", fn,
                  al, B->ld_scale);
    if (nvfp4a_status st = check_scales(fn, "B", B, n, k, &ldsb)) return st;
  }
  if (nvfp4a_status st = check_epilogue_operands(fn, m, beta, C, ldc, D, ldd, bias, ex.mask)) return st;
  if (nvfp4a_status st = check_device()) return st;
  if (ex.mask) {
    if (A->flags & NVFP4A_SCALES_UE5M3) return fail(NVFP4A_NOT_SUPPORTED, "%s: the extended epilogue takes A with E4M3 block scales", fn);
    if (B->dtype != NVFP4A_BF16 && B->dtype != NVFP4A_INT8) return fail(NVFP4A_NOT_SUPPORTED, "%s: the extended epilogue takes B BF16 or INT8", fn);
  }
  GemmArgs g;
  memset(&g, 0, sizeof g);
  g.m = m; g.n = n; g.k = k;
  g.A.data = (const uint8_t *)A->data; g.A.image = 1; g.A.ktiles = (k + kImgK - 1) / kImgK;
  g.A.ue = (A->flags & NVFP4A_SCALES_UE5M3) ? 1 : 0;
  g.B = make_b(B, ldb, ldsb, k, false);
  g.e = make_epilogue(alpha, A, B, beta, C, ldc, D, ldd, bias);
  g.x = ex;
  if (tp) g.tp = *tp;
  return dispatch(fn, g, stream);
}

static nvfp4a_status check_weight_image(const char *fn, int kind, const void *image, int rows, int k) {
  if (kind != NVFP4A_TC_A16 && kind != NVFP4A_TC_A8) return fail(NVFP4A_INVALID_VALUE, "%s: image kind %d is not NVFP4A_TC_A16 or NVFP4A_TC_A8", fn, kind);
  if (!image) return fail(NVFP4A_INVALID_VALUE, "%s: image is NULL", fn);
  if (rows < 0 || k < 0 || k % 64) return fail(NVFP4A_INVALID_VALUE, "%s: rows = %d, k = %d (k must be a multiple of 64)", fn, rows, k);
  if ((uintptr_t)image & 15) return fail(NVFP4A_INVALID_VALUE, "%s: the image must be 16-byte aligned", fn);
  return NVFP4A_OK;
}

// nvfp4a_gemm_ex with the RMSNorm column scales of all n tokens computed first into `colscales` (n floats the caller of this
// function owns for the duration of the call); used by nvfp4a_b200_gemm_ex_static.  Every argument is validated first (a failed
// call launches nothing); the scales kernel then runs before the GEMM and writes nothing but `colscales`.
nvfp4a_status gemm_ex_with_scales(const char *fn, int m, int n, int k, float alpha, const nvfp4a_tensor *A, int lda, const nvfp4a_tensor *B, int ldb,
                                  float beta, const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias,
                                  const nvfp4a_epilogue *ex, float *colscales, cudaStream_t stream) {
  EpilogueEx x;
  if (nvfp4a_status st = make_epilogue_ex(fn, ex, m, beta, ldd, &x)) return st;
  if ((x.mask & kExNorm) && colscales && n > kGemvMaxN && B && B->dtype == NVFP4A_BF16 && forced_route() != 1 && m > 0) {
    if (nvfp4a_status st = gemm_run(fn, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, D, ldd, bias, x, stream, true)) return st;
    if (nvfp4a_status st = cuda_fail(launch_norm_scales(x, n, colscales, stream), fn)) return st;
    x.colscales = colscales;
  }
  g_no_alloc = 1;   // this path serves the entry that allocates nothing: kernels that take scratch from the memory pool step aside
  const nvfp4a_status st = gemm_run(fn, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, D, ldd, bias, x, stream);
  g_no_alloc = 0;
  return st;
}

}  // namespace nvb

using namespace nvb;

extern "C" int nvfp4a_b200_set_route(int route) {
  const int old = forced_route();
  g_route = (route == 2 || route == 3) ? route : (route ? 1 : 0);
  return old;
}

extern "C" int nvfp4a_b200_last_route(void) { return g_last_route; }

extern "C" nvfp4a_status nvfp4a_b200_trim_scratch(void) {
  clear_error();
  return cuda_fail(trim_planes_pool(), "nvfp4a_b200_trim_scratch");
}

extern "C" int nvfp4a_b200_set_gemv_splits(int splits) {
  if (splits < 0 || splits > 8 || (splits & (splits - 1))) return -1;
  set_gemv_fp4_splits(splits);
  return 0;
}

extern "C" nvfp4a_status nvfp4a_gemm(int m, int n, int k, float alpha, const nvfp4a_tensor *A, int lda, const nvfp4a_tensor *B, int ldb, float beta,
                                     const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias, cudaStream_t stream) {
  clear_error();
  EpilogueEx x;
  memset(&x, 0, sizeof x);
  return gemm_run("nvfp4a_gemm", m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, D, ldd, bias, x, stream);
}

extern "C" nvfp4a_status nvfp4a_gemm_ex(int m, int n, int k, float alpha, const nvfp4a_tensor *A, int lda, const nvfp4a_tensor *B, int ldb, float beta,
                                        const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias,
                                        const nvfp4a_epilogue *ex, cudaStream_t stream) {
  clear_error();
  EpilogueEx x;
  if (nvfp4a_status st = make_epilogue_ex("nvfp4a_gemm_ex", ex, m, beta, ldd, &x)) return st;
  return gemm_run("nvfp4a_gemm_ex", m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, D, ldd, bias, x, stream);
}

extern "C" nvfp4a_status nvfp4a_gemm_dual(int m, int n, int k, float alpha, const nvfp4a_dual_tensor *A, int trans_a, const nvfp4a_dual_tensor *B,
                                          int trans_b, float beta, const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd,
                                          const nvfp4a_tensor *bias, cudaStream_t stream) {
  clear_error();
  if (!A || !B) return fail(NVFP4A_INVALID_VALUE, "nvfp4a_gemm_dual: A or B is NULL");
  // the half whose blocks run along k: the row half of an [m][k] operand, the column half of a [k][m] one
  const nvfp4a_tensor *a = trans_a ? &A->col : &A->row, *b = trans_b ? &B->col : &B->row;
  if (!a->data) return fail(NVFP4A_INVALID_VALUE, "nvfp4a_gemm_dual: A has no %s half (trans_a = %d)", trans_a ? "column" : "row", trans_a);
  if (!b->data) return fail(NVFP4A_INVALID_VALUE, "nvfp4a_gemm_dual: B has no %s half (trans_b = %d)", trans_b ? "column" : "row", trans_b);
  return nvfp4a_gemm(m, n, k, alpha, a, trans_a ? A->ld_col : A->ld_row, b, trans_b ? B->ld_col : B->ld_row, beta, C, ldc, D, ldd, bias, stream);
}

extern "C" nvfp4a_status nvfp4a_gemm_grouped(int groups, int m, int k, int rows, float alpha, const nvfp4a_tensor *A, int lda, const nvfp4a_tensor *B,
                                             int ldb, float beta, const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd,
                                             const nvfp4a_tensor *bias, const int *seg, cudaStream_t stream) {
  clear_error();
  const char *fn = "nvfp4a_gemm_grouped";
  if (groups < 0 || rows < 0) return fail(NVFP4A_INVALID_VALUE, "%s: negative groups = %d or rows = %d", fn, groups, rows);
  if (groups > 0 && m > 0 && (long long)groups * m > 0x7FFFFFFFll) return fail(NVFP4A_INVALID_VALUE, "%s: groups * m = %d * %d exceeds 2^31 - 1", fn, groups, m);
  if (groups == 0) return NVFP4A_OK;
  if (rows > 0 && m > 0 && !seg) return fail(NVFP4A_INVALID_VALUE, "%s: seg is NULL", fn);
  GemmArgs g;
  memset(&g, 0, sizeof g);
  const EpilogueEx none = {};
  // the checks of nvfp4a_gemm with A taken as [groups * m][k]; an empty problem returns before anything is filled in
  if (nvfp4a_status st = gemm_run(fn, m, rows, k, alpha, A, lda, B, ldb, beta, C, ldc, D, ldd, bias, none, stream, false, groups, &g)) return st;
  if (m == 0 || rows == 0) return NVFP4A_OK;
  // Every group runs a CUDA-core kernel in the reference's tiled order: the bytes of nvfp4a_gemm's tiled kernel for that group.
  // INT8 activations take the 128 x 128 DP4A kernel, everything else the generic one.
  if (forced_route() != 1 && gemm_dp4a_supports(g)) {
    g_last_route = 7;
    return cuda_fail(launch_gemm_dp4a_grouped(g, seg, groups, stream), "nvfp4a_gemm_grouped: kernel launch");
  }
  g_last_route = 1;
  return cuda_fail(launch_gemm_grouped(g, seg, groups, stream), "nvfp4a_gemm_grouped: kernel launch");
}

extern "C" size_t nvfp4a_tc_image_bytes(int operand, nvfp4a_dtype dtype, int rows, int k) {
  const int kind = image_kind(operand, dtype);
  if (!kind || rows < 0 || k < 0 || k % 64) return 0;
  if (kind <= 2) return image_bytes(rows, k);
  if (kind == 3) return int8_image_scale_offset(rows, k) + (size_t)rows * (k / 16) * 4;
  return (size_t)rows * k * 2;
}

extern "C" size_t nvfp4a_tc_workspace_bytes(void) { return (size_t)kWorkspaceTokens * sizeof(float); }

extern "C" nvfp4a_status nvfp4a_tc_image(int operand, const nvfp4a_tensor *src, int ld, int rows, int k, void *image, cudaStream_t stream) {
  clear_error();
  const char *fn = "nvfp4a_tc_image";
  if (!src || !src->data || !image) return fail(NVFP4A_INVALID_VALUE, "%s: src, src->data or image is NULL", fn);
  const int kind = image_kind(operand, src->dtype);
  if (!kind) return fail(NVFP4A_NOT_SUPPORTED, "%s: no image of kind %d for dtype %d (A16 / A8: NVFP4; B: NVFP4, INT8, BF16)", fn, operand, (int)src->dtype);
  if (rows < 0 || k < 0 || k % 64) return fail(NVFP4A_INVALID_VALUE, "%s: rows = %d, k = %d (k must be a multiple of 64)", fn, rows, k);
  if (rows == 0 || k == 0) return NVFP4A_OK;
  if (ld % 64 || ld < k) return fail(NVFP4A_INVALID_VALUE, "%s: ld = %d must be a multiple of 64 and >= k = %d", fn, ld, k);
  if (!aligned(src->data, 16) || !aligned(image, 16)) return fail(NVFP4A_INVALID_VALUE, "%s: src data and image must be 16-byte aligned", fn);
  int ldsc = 0;
  if (src->dtype == NVFP4A_BF16) {
    if (src->flags) return fail(NVFP4A_INVALID_VALUE, "%s: flags apply to NVFP4 tensors only", fn);
  } else {
    const unsigned al = src->dtype == NVFP4A_INT8 ? 16 : 4;
    if (!src->block_scale) return fail(NVFP4A_INVALID_VALUE, "%s: src is NVFP4 / INT8 but has no block_scale", fn);
    if (!aligned(src->block_scale, al) || src->ld_scale % 4 || (src->ld_scale && src->ld_scale < k / 16))
      return fail(NVFP4A_INVALID_VALUE, "%s: block scales must be %u-byte aligned, ld_scale a multiple of 4 and >= k / 16 (ld_scale = %d)", fn, al,
                  src->ld_scale);
    if (nvfp4a_status st = check_scales(fn, "src", src, rows, k, &ldsc)) return st;
  }
  if (nvfp4a_status st = check_device()) return st;
  if (kind <= 2) {
    Fp4Operand s;
    memset(&s, 0, sizeof s);
    s.data = (const uint8_t *)src->data; s.sc = (const uint8_t *)src->block_scale; s.ld = ld; s.sld = ldsc;
    return cuda_fail(launch_image_build(s, rows, k, (uint8_t *)image, stream), "nvfp4a_tc_image: kernel launch");
  }
  // INT8 / BF16 activations: compact row-major copies
  if (kind == 3) {
    cudaError_t e = cudaMemcpy2DAsync(image, k, src->data, ld, k, rows, cudaMemcpyDeviceToDevice, stream);
    if (e == cudaSuccess)
      e = cudaMemcpy2DAsync((uint8_t *)image + int8_image_scale_offset(rows, k), (size_t)(k / 16) * 4, src->block_scale, (size_t)ldsc * 4,
                            (size_t)(k / 16) * 4, rows, cudaMemcpyDeviceToDevice, stream);
    return cuda_fail(e, "nvfp4a_tc_image: copy");
  }
  return cuda_fail(cudaMemcpy2DAsync(image, (size_t)k * 2, src->data, (size_t)ld * 2, (size_t)k * 2, rows, cudaMemcpyDeviceToDevice, stream),
                   "nvfp4a_tc_image: copy");
}

extern "C" nvfp4a_status nvfp4a_tc_image_convert(int from, int to, const void *image, int rows, int k, void *dst, cudaStream_t stream) {
  clear_error();
  const char *fn = "nvfp4a_tc_image_convert";
  if (nvfp4a_status st = check_weight_image(fn, from, image, rows, k)) return st;
  if (nvfp4a_status st = check_weight_image(fn, to, dst, rows, k)) return st;
  if (from == to) return fail(NVFP4A_INVALID_VALUE, "%s: from and to are the same kind", fn);
  if (rows == 0 || k == 0) return NVFP4A_OK;
  if (nvfp4a_status st = check_device()) return st;
  // both weight kinds share one layout here
  return cuda_fail(cudaMemcpyAsync(dst, image, image_bytes(rows, k), cudaMemcpyDeviceToDevice, stream), "nvfp4a_tc_image_convert: copy");
}

extern "C" nvfp4a_status nvfp4a_tc_image_to_raw(int from, const void *image, int rows, int k, const nvfp4a_tensor *dst, int ld, cudaStream_t stream) {
  clear_error();
  const char *fn = "nvfp4a_tc_image_to_raw";
  if (nvfp4a_status st = check_weight_image(fn, from, image, rows, k)) return st;
  if (!dst || !dst->data || !dst->block_scale || dst->dtype != NVFP4A_NVFP4)
    return fail(NVFP4A_INVALID_VALUE, "%s: dst must be an NVFP4 tensor with data and block_scale", fn);
  const int lds = dst->ld_scale ? dst->ld_scale : k / 16;
  if (ld % 64 || ld < k || lds % 4 || lds < k / 16 || ((uintptr_t)dst->data & 15) || ((uintptr_t)dst->block_scale & 3))
    return fail(NVFP4A_INVALID_VALUE, "%s: ld = %d (multiple of 64, >= k), ld_scale = %d (multiple of 4, >= k / 16), data 16-byte and scales 4-byte aligned",
                fn, ld, dst->ld_scale);
  if (dst->flags & NVFP4A_SCALES_SWIZZLED) return fail(NVFP4A_INVALID_VALUE, "%s: dst takes linear block scales", fn);
  if (rows == 0 || k == 0) return NVFP4A_OK;
  if (nvfp4a_status st = check_device()) return st;
  return cuda_fail(launch_image_to_raw((const uint8_t *)image, rows, k, (uint8_t *)dst->data, ld, (uint8_t *)dst->block_scale, lds, stream),
                   "nvfp4a_tc_image_to_raw: kernel launch");
}

extern "C" nvfp4a_status nvfp4a_gemm_tc(int m, int n, int k, float alpha, const nvfp4a_tensor *A, const nvfp4a_tensor *B, float beta,
                                        const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias, void *workspace,
                                        cudaStream_t stream) {
  clear_error();
  EpilogueEx x;
  memset(&x, 0, sizeof x);
  return gemm_tc_run("nvfp4a_gemm_tc", m, n, k, alpha, A, B, beta, C, ldc, D, ldd, bias, workspace, x, stream);
}

extern "C" nvfp4a_status nvfp4a_gemm_tc_ex(int m, int n, int k, float alpha, const nvfp4a_tensor *A, const nvfp4a_tensor *B, float beta,
                                           const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias,
                                           const nvfp4a_epilogue *ex, void *workspace, cudaStream_t stream) {
  clear_error();
  EpilogueEx x;
  if (nvfp4a_status st = make_epilogue_ex("nvfp4a_gemm_tc_ex", ex, m, beta, ldd, &x)) return st;
  return gemm_tc_run("nvfp4a_gemm_tc_ex", m, n, k, alpha, A, B, beta, C, ldc, D, ldd, bias, workspace, x, stream);
}

extern "C" nvfp4a_status nvfp4a_gemv_tc(int m, int n, int k, float alpha, const nvfp4a_tensor *A, const nvfp4a_tensor *B, int ldb, float beta,
                                        const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias, cudaStream_t stream) {
  clear_error();
  EpilogueEx x;
  memset(&x, 0, sizeof x);
  return gemv_tc_run("nvfp4a_gemv_tc", m, n, k, alpha, A, B, ldb, beta, C, ldc, D, ldd, bias, x, stream);
}

extern "C" nvfp4a_status nvfp4a_gemv_tc_ex(int m, int n, int k, float alpha, const nvfp4a_tensor *A, const nvfp4a_tensor *B, int ldb, float beta,
                                           const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias,
                                           const nvfp4a_epilogue *ex, cudaStream_t stream) {
  clear_error();
  EpilogueEx x;
  if (nvfp4a_status st = make_epilogue_ex("nvfp4a_gemv_tc_ex", ex, m, beta, ldd, &x)) return st;
  return gemv_tc_run("nvfp4a_gemv_tc_ex", m, n, k, alpha, A, B, ldb, beta, C, ldc, D, ldd, bias, x, stream);
}

// What the fused all-gather needs of D inside the rank's buffer: the push moves 16-byte vectors (GEMV) or TMA boxes (GEMM), so D's
// base, its column pitch and a shard row must all be multiples of 16 bytes; checked before anything is launched.
static nvfp4a_status check_tp_layout(const char *fn, const nvfp4a_tensor *D, int ldd, int m, bool swiglu, const unsigned char *local_base, int world) {
  if (world <= 1 || !D || !D->data) return NVFP4A_OK;
  if (!dense_t(D)) return NVFP4A_OK;   // (rejected with its own message later)
  const long long esz = dense_bytes(D->dtype), drows = swiglu ? m / 2 : m;
  if ((const unsigned char *)D->data < local_base) return fail(NVFP4A_INVALID_VALUE, "%s: D must lie inside buffers[rank]", fn);
  if (((uintptr_t)D->data & 15) || ((long long)ldd * esz) % 16 || (drows * esz) % 16)
    return fail(NVFP4A_INVALID_VALUE, "%s: with world > 1, D's base (%p), its column pitch (%lld bytes) and a shard row (%lld bytes) must be multiples of 16 bytes",
                fn, D->data, (long long)ldd * esz, drows * esz);
  return NVFP4A_OK;
}

// nvfp4a_gemv_tc(_ex) of one rank of a tensor-parallel group with the all-gather fused in: D (inside buffers[rank]) is also
// stored at the same place of every peer's buffer and the ranks meet in a barrier before the stream goes on.
extern "C" nvfp4a_status nvfp4a_b200_gemv_tc_tp(int m, int n, int k, float alpha, const nvfp4a_tensor *A, const nvfp4a_tensor *B, int ldb,
                                                const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias, const nvfp4a_epilogue *ex,
                                                void *const *buffers, void *const *flags, int world, int rank, cudaStream_t stream) {
  const char *fn = "nvfp4a_b200_gemv_tc_tp";
  clear_error();
  if (!buffers || !flags || world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
    return fail(NVFP4A_INVALID_VALUE, "%s: needs buffers, flags and 0 <= rank < world <= %d", fn, kMaxRanks);
  TpPush tp;
  memset(&tp, 0, sizeof tp);
  tp.world = world; tp.rank = rank;
  tp.local_base = (unsigned char *)buffers[rank];
  for (int p = 0; p < world; ++p) {
    if (!buffers[p] || !flags[p] || ((uintptr_t)buffers[p] & 15) || ((uintptr_t)flags[p] & 7))
      return fail(NVFP4A_INVALID_VALUE, "%s: buffer / flag pointer of rank %d is NULL or misaligned", fn, p);
    tp.delta[p] = (long long)((unsigned char *)buffers[p] - tp.local_base);
    tp.flags[p] = (unsigned long long *)flags[p];
  }
  EpilogueEx x;
  if (nvfp4a_status st = make_epilogue_ex(fn, ex, m, 0.f, ldd, &x)) return st;
  if (x.mask & kExOut2) return fail(NVFP4A_NOT_SUPPORTED, "%s: the second output is not gathered; use nvfp4a_gemv_tc_ex and nvfp4a_b200_tp_gather", fn);
  if (nvfp4a_status st = check_tp_layout(fn, D, ldd, m, (x.mask & kExSwiglu) != 0, tp.local_base, world)) return st;
  return gemv_tc_run(fn, m, n, k, alpha, A, B, ldb, 0.f, nullptr, 0, D, ldd, bias, x, stream, world > 1 ? &tp : nullptr);
}

// The same with the wait moved from the end of this kernel to the start of the next one (see TpPush::deferred).
extern "C" nvfp4a_status nvfp4a_b200_gemv_tc_tp_deferred(int m, int n, int k, float alpha, const nvfp4a_tensor *A, const nvfp4a_tensor *B, int ldb,
                                                         const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias, const nvfp4a_epilogue *ex,
                                                         void *const *buffers, void *const *flags, int world, int rank, int push, cudaStream_t stream) {
  const char *fn = "nvfp4a_b200_gemv_tc_tp_deferred";
  clear_error();
  if (!buffers || !flags || world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
    return fail(NVFP4A_INVALID_VALUE, "%s: needs buffers, flags and 0 <= rank < world <= %d", fn, kMaxRanks);
  TpPush tp;
  memset(&tp, 0, sizeof tp);
  tp.world = world; tp.rank = rank; tp.deferred = push ? 3 : 1;
  tp.local_base = (unsigned char *)buffers[rank];
  for (int p = 0; p < world; ++p) {
    if (!buffers[p] || !flags[p] || ((uintptr_t)buffers[p] & 15) || ((uintptr_t)flags[p] & 7))
      return fail(NVFP4A_INVALID_VALUE, "%s: buffer / flag pointer of rank %d is NULL or misaligned", fn, p);
    tp.delta[p] = (long long)((unsigned char *)buffers[p] - tp.local_base);
    tp.flags[p] = (unsigned long long *)flags[p];
  }
  EpilogueEx x;
  if (nvfp4a_status st = make_epilogue_ex(fn, ex, m, 0.f, ldd, &x)) return st;
  if (x.mask & kExOut2) return fail(NVFP4A_NOT_SUPPORTED, "%s: the second output is not gathered", fn);
  if (nvfp4a_status st = check_tp_layout(fn, D, ldd, m, (x.mask & kExSwiglu) != 0, tp.local_base, world)) return st;
  return gemv_tc_run(fn, m, n, k, alpha, A, B, ldb, 0.f, nullptr, 0, D, ldd, bias, x, stream, world > 1 ? &tp : nullptr);
}

// nvfp4a_gemm_tc(_ex) (beta = 0) of one rank of a tensor-parallel group with the all-gather fused in: the W4A16 tcgen05 GEMM's
// epilogue stores every tile of D into all ranks' buffers by TMA, then the ranks meet in a barrier.
extern "C" nvfp4a_status nvfp4a_b200_gemm_tc_tp(int m, int n, int k, float alpha, const nvfp4a_tensor *A, const nvfp4a_tensor *B,
                                                const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias, const nvfp4a_epilogue *ex, void *workspace,
                                                void *const *buffers, void *const *flags, int world, int rank, cudaStream_t stream) {
  const char *fn = "nvfp4a_b200_gemm_tc_tp";
  clear_error();
  if (!buffers || !flags || world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
    return fail(NVFP4A_INVALID_VALUE, "%s: needs buffers, flags and 0 <= rank < world <= %d", fn, kMaxRanks);
  TpPush tp;
  memset(&tp, 0, sizeof tp);
  tp.world = world; tp.rank = rank;
  tp.local_base = (unsigned char *)buffers[rank];
  for (int p = 0; p < world; ++p) {
    if (!buffers[p] || !flags[p] || ((uintptr_t)buffers[p] & 15) || ((uintptr_t)flags[p] & 7))
      return fail(NVFP4A_INVALID_VALUE, "%s: buffer / flag pointer of rank %d is NULL or misaligned", fn, p);
    tp.delta[p] = (long long)((unsigned char *)buffers[p] - tp.local_base);
    tp.flags[p] = (unsigned long long *)flags[p];
  }
  EpilogueEx x;
  if (nvfp4a_status st = make_epilogue_ex(fn, ex, m, 0.f, ldd, &x)) return st;
  if (x.mask & kExOut2) return fail(NVFP4A_NOT_SUPPORTED, "%s: the second output is not gathered; use nvfp4a_gemm_tc_ex and nvfp4a_b200_tp_gather", fn);
  if (nvfp4a_status st = check_tp_layout(fn, D, ldd, m, (x.mask & kExSwiglu) != 0, tp.local_base, world)) return st;
  return gemm_tc_run(fn, m, n, k, alpha, A, B, 0.f, nullptr, 0, D, ldd, bias, workspace, x, stream, world > 1 ? &tp : nullptr);
}
