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
  int deferred;                // the deferred form: nobody waits at the END of a gather; the next kernel waits at its START for the
                               // peers' posts (tp_wait_posts), where the wait hides behind the launch and the set-up.
                               // bit 0: this kernel waits at its start; bit 1: its last CTA copies the outputs to the peers and
                               // posts the rank's epoch (otherwise a nvfp4a_b200_tp_gather_post launch follows)
};

__device__ __forceinline__ void st_release_sys(unsigned long long *p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Called by all threads of ONE CTA per rank after a CTA barrier that follows the rank's stores to its peers (the release store of
// the flag below orders, at system scope, everything that happened before that barrier: one fence per poster instead of one per
// storing thread -- a system-scope fence waits out an NVLink round trip): bumps the
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

// Deferred form, producer side: called by all threads of ONE CTA after a CTA barrier that follows the rank's stores to the peers:
// bumps the rank's epoch and writes it (release, system scope) into slot `rank` of every peer's flag array.  Nobody waits.
__device__ __forceinline__ void tp_post_epoch(unsigned long long *const *flags, int world, int rank) {
  __shared__ unsigned long long post_epoch_s;
  unsigned long long *mine = flags[rank];
  if (threadIdx.x == 0) {
    post_epoch_s = mine[kFlagEpoch] + 1;
    mine[kFlagEpoch] = post_epoch_s;
  }
  __syncthreads();
  if ((int)threadIdx.x < world && (int)threadIdx.x != rank) st_release_sys(flags[threadIdx.x] + rank, post_epoch_s);
}

// Deferred form, consumer side: threads 0 .. world - 1 of a CTA wait until every peer has posted the epoch this rank itself has
// reached (the rank's previous kernel in the stream posted it; every rank makes the same sequence of calls, so the numbers agree).
// After it the previous gather's data is complete in this rank's buffer, and every peer has finished the kernel that read the
// buffer this kernel is about to overwrite.  Bounded like the barrier (0x401).  The caller follows with a CTA barrier.
__device__ __forceinline__ void tp_wait_posts(unsigned long long *const *flags, int world, int rank, unsigned *status, unsigned tag, long long wait_cycles) {
  if ((int)threadIdx.x < world && (int)threadIdx.x != rank) {
    const unsigned long long *mine = flags[rank];
    const unsigned long long epoch = ld_acquire_sys(mine + kFlagEpoch);
    const long long start = clock64();
    while (ld_acquire_sys(mine + threadIdx.x) < epoch) {
      if (clock64() - start > wait_cycles) {
        atomicCAS(status, 0u, 0x401u | tag);
        break;
      }
    }
  }
}

}  // namespace nvb
