// Thin C wrappers around the REFERENCE's own host-callable codecs, compiled from the reference sources where they lie
// (-I$(REF); nothing of the reference is copied here).  Built by oracle/Makefile into oracle/_ref/libref_codecs.so
// and used only by the pin tests: the CPU oracle's encoders, decoders and scale addressing must agree with these on
// every input.  TEST INFRASTRUCTURE ONLY.
#include <thread>
#include <vector>
#include "tests/test_util.h"  // the reference's host helpers: e4, ue5, e2, sc_pos, to_bf; pulls in src/nvfp4effma.cuh

static uint32_t ref_encode(int which, float x) {
  switch (which) {
    case 0: return nvfp4a::f32_to_e4m3(x);   // ref src/nvfp4effma.cuh:137
    case 1: return nvfp4a::f32_to_e2m1(x);   // ref src/nvfp4effma.cuh:156
    case 2: return nvfp4a::f32_to_ue5m3(x);  // ref src/nvfp4effma.cuh:196
    default: return to_bf(x);                // ref tests/test_util.h:51
  }
}

extern "C" {
uint64_t ref_encoder_fold(int which, uint64_t first, uint64_t count, int nthreads) {
  if (nthreads < 1) nthreads = 1;
  std::vector<uint64_t> part(nthreads, 0);
  std::vector<std::thread> pool;
  for (int t = 0; t < nthreads; ++t)
    pool.emplace_back([&, t] {
      uint64_t s = 0;
      const uint64_t lo = first + count * t / nthreads, hi = first + count * (t + 1) / nthreads;
      for (uint64_t v = lo; v < hi; ++v) {
        const uint32_t u = (uint32_t)v;
        float x; memcpy(&x, &u, 4);
        const uint64_t mix = ((uint64_t)u * 0x9E3779B97F4A7C15ull) ^ 0xD1B54A32D192ED03ull;
        s += mix * (uint64_t)(ref_encode(which, x) + 1u);
      }
      part[t] = s;
    });
  for (auto &th : pool) th.join();
  uint64_t s = 0;
  for (uint64_t p : part) s += p;
  return s;
}
void ref_encode_array(int which, const float *x, uint32_t *codes, size_t n) {
  for (size_t i = 0; i < n; ++i) codes[i] = ref_encode(which, x[i]);
}
float ref_e4m3_value(uint32_t b) { return e4((uint8_t)b); }
float ref_ue5m3_value(uint32_t b) { return ue5((uint8_t)b); }
float ref_e2m1_value(uint32_t n) { return e2(n); }
size_t ref_scale_pos(int swz, int ld, int cols, int r, int c) { return sc_pos(swz != 0, ld, cols, r, c); }
size_t ref_scale_idx(int ld, int r, int c) { return nvfp4a::ScaleIdx{ld}.at(r, c); }  // ref src/nvfp4effma.cuh:71-79
}
