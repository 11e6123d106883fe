// Host-side core of the C ABI: the thread-local error text, device probing, status strings and the checks of the
// NVFP4-specific fields of nvfp4a_tensor that every entry point shares.  Behaviour follows the reference's host layer
// (src/nvfp4effma.cu:12-25, :134-143 and src/gemm_nvfp4effma.cu:208-252 there): same conditions, same status codes;
// messages name the offending argument but are worded independently.
#include <stdarg.h>
#include <stdio.h>
#include "common.cuh"

namespace nvb {

static thread_local char g_error[512];

void clear_error() { g_error[0] = 0; }

nvfp4a_status fail(nvfp4a_status s, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
  return s;
}

nvfp4a_status cuda_fail(cudaError_t e, const char *what) {
  if (e == cudaSuccess) return NVFP4A_OK;
  return fail(NVFP4A_CUDA_ERROR, "%s: CUDA error %d (%s): %s", what, (int)e, cudaGetErrorName(e), cudaGetErrorString(e));
}

struct DevInfo { int probed, cc, sms; };
static DevInfo g_dev[64];

static const DevInfo &dev_info(int dev) {
  DevInfo &d = g_dev[dev & 63];
  if (!d.probed) {
    int ma = 0, mi = 0, sms = 0;
    cudaDeviceGetAttribute(&ma, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&mi, cudaDevAttrComputeCapabilityMinor, dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    d.cc = ma * 10 + mi;
    d.sms = sms;
    d.probed = 1;
  }
  return d;
}

nvfp4a_status check_device() {
  int dev = -1;
  const cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  const DevInfo &d = dev_info(dev);
  if (d.cc / 10 != 10)
    return fail(NVFP4A_NOT_SUPPORTED, "device %d has compute capability %d.%d; this library is built for sm_100a (B200) only",
                dev, d.cc / 10, d.cc % 10);
  return NVFP4A_OK;
}

int device_sms() {
  int dev = 0;
  cudaGetDevice(&dev);
  return dev_info(dev).sms;
}

// Bound M of the global encoding: 0 selects the scale type's maximum; only the combinations Transformer Engine defines
// are valid (E4M3: 448 or 256; UE5M3: 114688).
float scale_max_of(const nvfp4a_tensor *t) {
  const bool ue = t->flags & NVFP4A_SCALES_UE5M3;
  if (t->scale_max == 0) return ue ? 114688.f : 448.f;
  if (ue) return t->scale_max == 114688 ? 114688.f : 0.f;
  return (t->scale_max == 448 || t->scale_max == 256) ? (float)t->scale_max : 0.f;
}

nvfp4a_status check_scales(const char *fn, const char *name, const nvfp4a_tensor *t, int rows, int cols, int *ld) {
  (void)rows;
  const unsigned known = NVFP4A_SCALES_SWIZZLED | NVFP4A_SCALES_UE5M3 | NVFP4A_GLOBAL_AMAX | NVFP4A_GLOBAL_PER_ROW;
  if (t->flags & ~known) return fail(NVFP4A_INVALID_VALUE, "%s: %s: unknown flag bits 0x%x", fn, name, t->flags & ~known);
  if (t->dtype != NVFP4A_NVFP4 && t->flags)
    return fail(NVFP4A_INVALID_VALUE, "%s: %s: flags apply to NVFP4 tensors only (dtype %d)", fn, name, (int)t->dtype);
  if (t->dtype == NVFP4A_NVFP4 && scale_max_of(t) == 0.f)
    return fail(NVFP4A_INVALID_VALUE, "%s: %s: scale_max = %d is not valid (E4M3 scales: 0, 448, 256; UE5M3: 0, 114688)", fn,
                name, t->scale_max);
  if ((t->flags & NVFP4A_GLOBAL_PER_ROW) && !t->global_scale)
    return fail(NVFP4A_INVALID_VALUE, "%s: %s: NVFP4A_GLOBAL_PER_ROW without global_scale", fn, name);
  const int padded = (cols / 16 + 3) / 4 * 4;
  if (t->flags & NVFP4A_SCALES_SWIZZLED) {
    if (t->ld_scale != 0 && t->ld_scale != padded)
      return fail(NVFP4A_INVALID_VALUE, "%s: %s: swizzled scales have %d scales per padded row, ld_scale must be 0 or %d", fn,
                  name, padded, padded);
    *ld = -padded;
  } else {
    if (t->ld_scale && t->ld_scale < cols / 16)
      return fail(NVFP4A_INVALID_VALUE, "%s: %s: ld_scale = %d is below cols / 16 = %d", fn, name, t->ld_scale, cols / 16);
    *ld = t->ld_scale ? t->ld_scale : cols / 16;
  }
  return NVFP4A_OK;
}

// 1 / (6 M) per operand whose global is an amax, multiplied in FP32 in Transformer Engine's order.
float amax_factor(const nvfp4a_tensor *A, const nvfp4a_tensor *B) {
  const bool aa = A && (A->flags & NVFP4A_GLOBAL_AMAX), ab = B && (B->flags & NVFP4A_GLOBAL_AMAX);
  if (aa && ab) return 1.0f / (6.f * 6.f * scale_max_of(A) * scale_max_of(B));
  if (aa) return 1.0f / (6.f * scale_max_of(A));
  if (ab) return 1.0f / (6.f * scale_max_of(B));
  return 1.0f;
}

}  // namespace nvb

extern "C" const char *nvfp4a_last_error(void) { return nvb::g_error; }

extern "C" const char *nvfp4a_status_string(nvfp4a_status s) {
  switch (s) {
    case NVFP4A_OK: return "NVFP4A_OK";
    case NVFP4A_INVALID_VALUE: return "NVFP4A_INVALID_VALUE";
    case NVFP4A_NOT_SUPPORTED: return "NVFP4A_NOT_SUPPORTED";
    case NVFP4A_CUDA_ERROR: return "NVFP4A_CUDA_ERROR";
  }
  return "unknown nvfp4a_status";
}
