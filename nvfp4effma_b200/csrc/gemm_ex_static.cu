// nvfp4a_b200_gemm_ex_static: nvfp4a_gemm_ex with the RMSNorm column scales staged in a device array that is part of the
// library image, so that the call allocates nothing.
//
// nvfp4a_gemm_tc_ex computes the column scales s_j once per call into the caller's workspace and the tcgen05 W4A16 GEMM
// reads one float per token.  nvfp4a_gemm_ex has no workspace argument, so its GEMM sums the parts again for every tile
// of weight rows.  A caller of nvfp4a_gemm_ex that wants the faster form but cannot provide memory at that point -- it is
// inside a CUDA-graph capture, or its framework's allocator owns all device memory and a cudaMalloc from a library would
// fail or synchronise the device -- calls this entry instead: same arguments, same results bit for bit.
//
// The scratch is a file-scope array of kStaticTokens floats (64 KiB), so n is limited to kStaticTokens tokens; a larger n
// is refused.  Its address is looked up once per device with cudaGetSymbolAddress (no allocation; the array is loaded
// with the module).  That first call on a device should be made outside stream capture: looking a symbol up can load
// the module, which a capturing stream does not allow.  Nothing in the scratch needs to start at zero -- the first
// kernel of a call writes every entry the GEMM then reads.  There is ONE array per device: two calls in flight at the same
// time on one device (two streams, or two host threads) race on it and must be serialised by the caller.
#include <mutex>
#include "operands.cuh"

namespace nvb {

constexpr int kStaticTokens = 16384;
static __device__ __align__(256) float g_static_colscales[kStaticTokens];

// nvfp4a_gemm_ex's validation and dispatch (gemm_api.cu)
nvfp4a_status gemm_ex_with_scales(const char *fn, int m, int n, int k, float alpha, const nvfp4a_tensor *A, int lda, const nvfp4a_tensor *B, int ldb,
                                  float beta, const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias,
                                  const nvfp4a_epilogue *ex, float *colscales, cudaStream_t stream);

// the array's address on the current device, looked up on the first call per device
static nvfp4a_status static_scratch(const char *fn, float **out) {
  static std::mutex mu;
  static float *ptr[64] = {};
  int dev = 0;
  if (cudaError_t e = cudaGetDevice(&dev)) return cuda_fail(e, fn);
  if (dev < 0 || dev >= 64) return fail(NVFP4A_NOT_SUPPORTED, "%s: device ordinal %d is outside the table of 64 devices", fn, dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!ptr[dev]) {
    float *p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress((void **)&p, g_static_colscales);  // the current device is `dev`
    if (e != cudaSuccess || !p) return cuda_fail(e != cudaSuccess ? e : cudaErrorInvalidSymbol, fn);
    ptr[dev] = p;
  }
  *out = ptr[dev];
  return NVFP4A_OK;
}

}  // namespace nvb

using namespace nvb;

extern "C" nvfp4a_status nvfp4a_b200_gemm_ex_static(int m, int n, int k, float alpha, const nvfp4a_tensor *A, int lda, const nvfp4a_tensor *B, int ldb,
                                                    float beta, const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd,
                                                    const nvfp4a_tensor *bias, const nvfp4a_epilogue *ex, cudaStream_t stream) {
  const char *fn = "nvfp4a_b200_gemm_ex_static";
  clear_error();
  if (n > kStaticTokens)
    return fail(NVFP4A_INVALID_VALUE, "%s: n = %d exceeds the %d tokens the static scratch holds; use nvfp4a_gemm_ex or nvfp4a_gemm_tc_ex", fn, n,
                kStaticTokens);
  if (nvfp4a_status st = check_device()) return st;
  float *scratch = nullptr;
  if (nvfp4a_status st = static_scratch(fn, &scratch)) return st;
  return gemm_ex_with_scales(fn, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, D, ldd, bias, ex, scratch, stream);
}

extern "C" int nvfp4a_b200_static_scratch_tokens(void) { return kStaticTokens; }
