// Thin inline-PTX layer over the Blackwell (sm_100a) features the GEMM kernels use: mbarriers with BOUNDED waits, TMA
// (cp.async.bulk[.tensor]) loads without multicast, tensor memory (tcgen05.alloc / ld / cp / commit) and the UMMA shared
// memory and instruction descriptors.  Every wait gives up after a fixed number of polls and reports failure to its
// caller, which raises the kernel's abort flag: no kernel of this library can spin forever.
#pragma once
#include <stdint.h>
#include <cuda.h>
#include <cuda_runtime.h>

namespace nvb {
namespace sm100 {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Polls the barrier's phase `parity`; gives up (false) after kMaxWaitCycles SM clock cycles -- about two seconds, far
// longer than any healthy wait of these kernels.
constexpr long long kMaxWaitCycles = 4000000000ll;
constexpr uint32_t kWaitHintNs = 1000000u;   // one millisecond per parked poll
// one poll of the barrier's phase `parity`
__device__ __forceinline__ bool mbar_try(uint64_t *bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
  if (mbar_try(bar, parity)) return true;   // the common case costs no clock read
  const uint32_t addr = smem_u32(bar);
  const long long start = clock64();
  for (;;) {
    // The time hint lets the hardware park the thread until the phase completes (or the hint runs out) instead of having
    // it spin: a spinning warp takes issue slots from the warps of its scheduler that have work (the epilogue warps).
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(addr), "r"(parity), "r"(kWaitHintNs) : "memory");
    if (done) return true;
    if (clock64() - start > kMaxWaitCycles) return false;
  }
}
// arrive on the barrier that sits at `own_bar`'s address in CTA `rank` of the cluster
__device__ __forceinline__ void mbar_arrive_rank(uint64_t *own_bar, uint32_t rank) {
  uint32_t addr;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(smem_u32(own_bar)), "r"(rank));
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(addr) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// generic-proxy writes to shared memory -> visible to the async proxy (TMA, tcgen05.cp / mma operand reads)
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- programmatic dependent launch ---------------------------------------------------------------------------------------------
// A kernel launched with the programmatic-stream-serialization attribute may start while its predecessor in the stream still
// runs, once every CTA of the predecessor has executed pdl_launch_dependents() (or exited).  It must execute pdl_wait()
// before it touches any memory the predecessor reads or writes: the wait returns when the predecessor has completed and its
// writes are visible.  Both are no-ops in a launch without the attribute or without a predecessor.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- thread-block clusters: rank, barrier, loads from a peer CTA's shared memory ---------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// every thread of every CTA of the cluster arrives and waits (release / acquire)
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// store into the shared memory of CTA `peer_rank` of the cluster, at the address `own_smem` has in this CTA
__device__ __forceinline__ void st_peer_f32(void *own_smem, uint32_t peer_rank, float v) {
  uint32_t addr;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(smem_u32(own_smem)), "r"(peer_rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ float ld_peer_f32(const void *own_smem, uint32_t peer_rank) {
  uint32_t addr;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(smem_u32(own_smem)), "r"(peer_rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

// ---- TMA (no multicast anywhere) -----------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, int x, int y, int z, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *map, int x, int y, int z, int w, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_u32(bar)) : "memory");
}
// CTA pair: the copy lands in this CTA's shared memory, its bytes are counted on the barrier at `own_bar`'s address in the
// pair's even CTA (rank 0 of a cluster of two), whose MMA thread waits for both CTAs' operands on that one barrier.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar_addr) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar_addr) : "memory");
}
// Issued by one elected lane of a CONVERGED warp (the whole warp runs the surrounding loop): coordinates, addresses and the
// descriptor pointer then stay on the uniform datapath from which the TMA instruction takes its operands.  Inside a one-lane
// branch the same instruction costs its warp several times as many cycles.
__device__ __forceinline__ void tma_load_3d_pair_elect(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar_addr) {
  asm volatile("{\n\t.reg .pred q;\n\telect.sync _|q, 0xFFFFFFFF;\n\t"
               "@q cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n\t}"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar_addr) : "memory");
}
__device__ __forceinline__ void tma_load_3d_elect(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar_addr) {
  asm volatile("{\n\t.reg .pred q;\n\telect.sync _|q, 0xFFFFFFFF;\n\t"
               "@q cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n\t}"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_elect(uint64_t *bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .pred q;\n\telect.sync _|q, 0xFFFFFFFF;\n\t"
               "@q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t}" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// the same with the barrier given as a shared-memory address (lanes of one instruction may name different barriers)
__device__ __forceinline__ void tma_load_3d_at(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar_addr) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar_addr) : "memory");
}
__device__ __forceinline__ uint32_t mbar_addr_rank(uint64_t *own_bar, uint32_t rank) {
  uint32_t addr;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(smem_u32(own_bar)), "r"(rank));
  return addr;
}
// contiguous copy: both addresses 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// shared -> global tile store (elements outside the tensor are clipped), tracked by bulk async-groups
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, const void *src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// barrier among `threads` threads of the CTA (id 1..15; 0 is __syncthreads)
__device__ __forceinline__ void named_barrier(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- tensor memory ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t *slot, uint32_t cols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// CTA pair (cta_group::2): one warp of EACH of the two CTAs issues these, with the same shared memory slot offset
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *slot, uint32_t cols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// arrives on the barrier once every tcgen05 operation this thread issued before has completed
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// pair MMAs: arrives on the barrier at this address in both CTAs of the pair (cluster of two: ranks 0 and 1)
__device__ __forceinline__ void tc_commit_pair(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
// 32 lanes x 32 consecutive columns of 32 bits -> 32 registers per thread (warp w reads lanes 32 (w % 4) ..)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t *r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
      "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
// 32 lanes x 16 consecutive columns -> 16 registers per thread
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t *r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
// 16 lanes x 64 consecutive columns -> 32 registers per thread.  For every group of 8 columns (registers 4 g .. 4 g + 3):
// thread t holds (lane t / 4, columns 2 (t % 4) and 2 (t % 4) + 1) in the first two and (lane t / 4 + 8, same columns) in the
// last two -- the fragment layout of an MMA accumulator.
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t taddr, uint32_t *r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
      "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
// 16 registers per thread -> 32 lanes x 16 consecutive columns (warp w writes lanes 32 (w % 4) ..)
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t *r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// shared memory (32 rows x 16 bytes, described by sdesc) -> 4 columns of all 128 lanes (the 32 rows replicated per quadrant)
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

__device__ __forceinline__ void tmem_cp_32x128b_warpx4_pair(uint32_t taddr, uint64_t sdesc) {   // both CTAs of a pair, each from its own shared memory
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// ---- UMMA descriptors --------------------------------------------------------------------------------------------------------
// Shared memory matrix descriptor (64 bit): start address >> 4 in bits [0, 14), leading byte offset >> 4 in [16, 30),
// stride byte offset >> 4 in [32, 46), descriptor version 1 in [46, 48), layout type in [61, 64)
// (0 none, 2 128-byte swizzle, 4 64-byte, 6 32-byte).
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) |
         (1ull << 46) | ((uint64_t)layout << 61);
}
// K-major operand tile of rows x 128 bytes written by TMA with the 128-byte swizzle: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) { return smem_desc(saddr, 16, 1024, 2); }
// 32 rows x 16 bytes, contiguous (one quarter... the source of tcgen05.cp.32x128b): 8-row groups 128 bytes apart, no swizzle
__device__ __forceinline__ uint64_t smem_desc_sf(uint32_t saddr) { return smem_desc(saddr, 0, 128, 0); }

// Instruction descriptor of kind::mxf4nvf4 (block scaled): a / b format E2M1 (1) at bits [7, 10) / [10, 13), K-major both,
// N >> 3 at [17, 23), scale format UE4M3 (0) at bit 23, M >> 4 at [24, 29), scale-factor ids 0, K = 64 (bit 31 = 0).
__host__ __device__ constexpr uint32_t idesc_mxf4nvf4(int m, int n) {
  return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// Instruction descriptor of kind::f16: D format F32 (1) at [4, 6), a / b format BF16 (1) or F16 (0) at [7, 10) / [10, 13),
// K-major both, N >> 3 at [17, 23), M >> 4 at [24, 29).
__host__ __device__ constexpr uint32_t idesc_f16(int m, int n, int bf16) {
  return (1u << 4) | ((uint32_t)bf16 << 7) | ((uint32_t)bf16 << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem] with block scales from tensor memory; one thread issues.
__device__ __forceinline__ void mma_mxf4nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                                             uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
// The same over a CTA pair, issued by one thread of the even CTA: M = 256 (128 rows of A from each CTA's shared memory), B's
// N rows half from each CTA, D and the block scales at the same tensor memory addresses in both CTAs (each CTA holds the
// scales of its own 128 rows of A and of ALL N rows of B).
__device__ __forceinline__ void mma_mxf4nvf4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                                                  uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
// The same instructions issued by ONE elected lane of a converged warp: the whole warp runs the surrounding loop, so that the
// compiler keeps descriptors, addresses and loop state on the uniform datapath, where tcgen05 instructions take their operands.
__device__ __forceinline__ void mma_mxf4nvf4_elect(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                                                   uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\telect.sync _|q, 0xFFFFFFFF;\n\t"
               "@q tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
__device__ __forceinline__ void mma_mxf4nvf4_pair_elect(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                                                        uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\telect.sync _|q, 0xFFFFFFFF;\n\t"
               "@q tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
// One pipeline stage of a block-scaled FP4 GEMM in one statement, issued by one elected lane of a converged warp: four MMAs over the
// stage's four 64-value k groups (descriptors 32 bytes apart, A-side scale columns 4 apart, B-side `sfb_step` apart), the first
// accumulating or not as `accumulate` says, then the commit that hands the stage back.  One election serves all five instructions.
#define NVB_MMA4_BODY(GROUP, COMMIT)                                                                                               \
  asm volatile("{\n\t.reg .pred p, q, t;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.eq.u32 t, %3, %3;\n\telect.sync _|q, 0xFFFFFFFF;\n\t"      \
               "@q tcgen05.mma.cta_group::" GROUP ".kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t"     \
               "@q tcgen05.mma.cta_group::" GROUP ".kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %7, %8, %3, [%9], [%10], t;\n\t"    \
               "@q tcgen05.mma.cta_group::" GROUP ".kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %11, %12, %3, [%13], [%14], t;\n\t" \
               "@q tcgen05.mma.cta_group::" GROUP ".kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %15, %16, %3, [%17], [%18], t;\n\t" \
               COMMIT "\n\t}"                                                                                                     \
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb),                              \
                 "l"(a_desc + 2), "l"(b_desc + 2), "r"(sfa + 4), "r"(sfb + sfb_step),                                                 \
                 "l"(a_desc + 4), "l"(b_desc + 4), "r"(sfa + 8), "r"(sfb + 2 * sfb_step),                                             \
                 "l"(a_desc + 6), "l"(b_desc + 6), "r"(sfa + 12), "r"(sfb + 3 * sfb_step), "r"(smem_u32(bar)), "h"((uint16_t)3) : "memory")
__device__ __forceinline__ void mma4_commit_pair_elect(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                                       uint32_t sfb_step, uint32_t accumulate, uint64_t *bar) {
  NVB_MMA4_BODY("2", "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%19], %20;");
}
__device__ __forceinline__ void mma4_commit_elect(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                                  uint32_t sfb_step, uint32_t accumulate, uint64_t *bar) {
  NVB_MMA4_BODY("1", "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%19];");
}
// One 64-value k group of the FP4 GEMV in one statement (elected lane of a converged warp): the two 512-byte scale tiles of the
// group's 256 weight rows copied into tensor memory (tcgen05.cp), then the MMA that reads them.
__device__ __forceinline__ void cp2_mma_mxf4nvf4_elect(uint32_t sfb_tmem, uint64_t sf_desc0, uint64_t sf_desc1, uint32_t d_tmem, uint64_t a_desc,
                                                       uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %8, 0;\n\telect.sync _|q, 0xFFFFFFFF;\n\t"
               "@q tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n\t"
               "@q tcgen05.cp.cta_group::1.32x128b.warpx4 [%2], %3;\n\t"
               "@q tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%4], %5, %6, %7, [%9], [%0], p;\n\t}"
               ::"r"(sfb_tmem), "l"(sf_desc0), "r"(sfb_tmem + 4), "l"(sf_desc1), "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc),
                 "r"(accumulate), "r"(sfa_tmem) : "memory");
}
__device__ __forceinline__ void tmem_cp_32x128b_warpx4_elect(uint32_t taddr, uint64_t sdesc) {
  asm volatile("{\n\t.reg .pred q;\n\telect.sync _|q, 0xFFFFFFFF;\n\t@q tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n\t}"
               ::"r"(taddr), "l"(sdesc) : "memory");
}
// The same for kind::f16 (K = 16 per instruction: four MMAs cover the 64 values of k of a 128-byte-row stage).
__device__ __forceinline__ void mma4_f16_commit_elect(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate, uint64_t *bar) {
  asm volatile("{\n\t.reg .pred p, q, t;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.eq.u32 t, %3, %3;\n\telect.sync _|q, 0xFFFFFFFF;\n\t"
               "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
               "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %5, %6, %3, t;\n\t"
               "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %7, %8, %3, t;\n\t"
               "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %9, %10, %3, t;\n\t"
               "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%11];\n\t}"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "l"(a_desc + 2), "l"(b_desc + 2), "l"(a_desc + 4), "l"(b_desc + 4),
                 "l"(a_desc + 6), "l"(b_desc + 6), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_2d_elect(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar_addr) {
  asm volatile("{\n\t.reg .pred q;\n\telect.sync _|q, 0xFFFFFFFF;\n\t"
               "@q cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n\t}"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar_addr) : "memory");
}
__device__ __forceinline__ void tc_commit_elect(uint64_t *bar) {
  asm volatile("{\n\t.reg .pred q;\n\telect.sync _|q, 0xFFFFFFFF;\n\t"
               "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_commit_pair_elect(uint64_t *bar) {
  asm volatile("{\n\t.reg .pred q;\n\telect.sync _|q, 0xFFFFFFFF;\n\t"
               "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n\t}"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

}  // namespace sm100

// ---- host: tensor maps ---------------------------------------------------------------------------------------------------------
// bytes matrix [rows][row_bytes] with `stride` bytes between rows (and optionally `tiles` such matrices tile_stride apart),
// box = box_rows x 128 bytes, 128-byte swizzle, zero fill outside.  Returns false if the driver refuses.
bool make_tmap_bytes(CUtensorMap *map, const void *base, uint64_t row_bytes, uint64_t rows, uint64_t stride, uint32_t box_rows,
                     uint64_t tiles = 0, uint64_t tile_stride = 0);
// dense matrix [outer][inner] of 2- or 4-byte elements, `stride` bytes between outer indices, box = box_inner x box_outer,
// no swizzle (the epilogue's store of D)
bool make_tmap_dense(CUtensorMap *map, const void *base, int elem_bytes, uint64_t inner, uint64_t outer, uint64_t stride,
                     uint32_t box_inner, uint32_t box_outer, int swizzle = 0);
// Block scales stored as 512-byte tiles (the swizzled layout), as a tensor of 8-byte words: `rows` rows of row_bytes bytes `stride`
// bytes apart; a box is 2 KiB of one row (the four tiles of 256 values of k), zero-filled past the end of the row.
bool make_tmap_scales(CUtensorMap *map, const void *base, uint64_t row_bytes, uint64_t rows, uint64_t stride);
// A tensor-core image as a rank-4 tensor of bytes [128-row tile][k tile][row of 128 bytes]: `rows` = 128 with the 128-byte swizzle
// for the nibbles (base = the image), 16 without swizzle for a tile's 2 KiB of block scales (base = the image + 16 KiB).  One
// box is that part of two vertically adjacent tiles (the two halves of 256 weight rows); a tile past the image reads zeros.
bool make_tmap_image_pair(CUtensorMap *map, const void *base, uint32_t rows, uint64_t ktiles, uint64_t tiles128);
// Tag of a launch for the status word: (library-wide launch sequence number mod 2^20) << 12.  A kernel that gives up a wait records
// code | tag, so the word names the kind of wait (low 12 bits: 0x1xx W4A4 GEMM, 0x2xx FP4 GEMV, 0x3xx W4A16 GEMM, 0x4xx tensor-parallel
// barrier, 0x5xx ceiling measurement) and the launch (nvfp4a_b200_last_launch gives the calling thread's latest sequence number).
unsigned next_launch_tag();
// SM clock cycles a tensor-parallel barrier waits for its peers before it gives up (nvfp4a_b200_set_wait_limit; default 2e9, about a second)
long long tp_wait_limit();
// whether launches ask for programmatic stream serialization (nvfp4a_b200_set_pdl; on by default)
bool pdl_enabled();
// kernel status word: 0 = healthy; kernels that gave up a wait write a non-zero code (see nvfp4a_b200_kernel_status)
unsigned int *kernel_status_device_ptr();

}  // namespace nvb
