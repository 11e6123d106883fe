// Barrier among the ranks of a tensor-parallel group on flags in peer-mapped memory (one rank per GPU).
#pragma once
#include <stdint.h>

namespace nvb {

constexpr int kMaxRanks = 8;
// flag array of a rank: slots 0..7 = the epochs its peers have reached, slot 8 = its own epoch counter, slot 9 = a CTA
// counter for kernels whose last CTA joins the barrier
constexpr int kFlagEpoch = 8, kFlagCtas = 9;

// The all-gather fused into a kernel's stores: results also go to every peer's buffer (peer address = local address +
// delta[p] bytes), and the kernel's last CTA joins the ranks' barrier.  world <= 1: nothing happens.
struct TpPush {
  int world, rank;
  long long delta[kMaxRanks];
  unsigned long long *flags[kMaxRanks];
  unsigned *status;
  unsigned tag;                // this launch's tag in the status word
  long long wait_cycles;       // SM clock cycles the barrier waits for its peers
  unsigned char *local_base;   // host side: this rank's buffer (peer p's is local_base + delta[p])
};

__device__ __forceinline__ void st_release_sys(unsigned long long *p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Called by all threads of ONE CTA per rank after the rank's stores to its peers are complete (and fenced): bumps the
// rank's epoch, writes it into slot `rank` of every rank's flag array and waits until every slot of its own array has reached the
// epoch -- bounded: after wait_cycles of SM clock (by default about a second) it records code 0x401 in *status and returns.  A peer
// that is more than that behind (first-call module loads, a stalled host) therefore shows up as 0x401, and the buffers are then
// incomplete: callers poll the status word at a convenient point (nvfp4a_b200_kernel_status).
__device__ __forceinline__ void tp_barrier_cta(unsigned long long *const *flags, int world, int rank, unsigned *status, unsigned tag, long long wait_cycles) {
  __shared__ unsigned long long epoch_s;
  unsigned long long *mine = flags[rank];
  if (threadIdx.x == 0) {
    epoch_s = mine[kFlagEpoch] + 1;
    mine[kFlagEpoch] = epoch_s;
  }
  __syncthreads();
  const unsigned long long epoch = epoch_s;
  if ((int)threadIdx.x < world) {
    const int p = threadIdx.x;
    __threadfence_system();
    st_release_sys(flags[p] + rank, epoch);
    const long long start = clock64();
    while (ld_acquire_sys(mine + p) < epoch) {
      if (clock64() - start > wait_cycles) {
        atomicCAS(status, 0u, 0x401u | tag);
        break;
      }
    }
  }
}

}  // namespace nvb
