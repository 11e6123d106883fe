// nvfp4a_b200_mma_ceiling: what the tensor cores of this GPU sustain on tcgen05.mma kind::mxf4nvf4 (block-scaled FP4) when
// nothing else is in the way -- the measured denominator beside the nominal FP4 peak for the W4A4 GEMM's roofline.
//
// Every CTA (one per SM; one cluster of two per SM pair in the cta_group::2 form) fills one operand stage in shared memory
// with a byte pattern, writes unit block scales (E4M3 0x38) into tensor memory, and its MMA thread then issues
// 4 * iters MMAs of 128 (or 256) x bn x 64 back to back into one accumulator: no loads, no epilogue, no waits between
// instructions (optionally one tcgen05.commit per four, as the GEMM's main loop issues).  The thread stamps the SM clock
// before the first issue and after the final commit has arrived; the host times the launch with events.  Test and
// measurement aid; the results are not read.
#include "operands.cuh"
#include "sm100.cuh"

namespace nvb {

using namespace sm100;

constexpr int kCeilThreads = 128, kCeilABytes = 16384, kCeilBBytes = 32768, kCeilSfBytes = 6144, kCeilSmem = kCeilABytes + kCeilBBytes + kCeilSfBytes + 1024 + 64;

template <bool PAIR>
__global__ void __launch_bounds__(kCeilThreads, 1) mma_ceiling_kernel(int bn, int iters, int commit_each, unsigned long long *cycles, unsigned *status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t *sf_smem = smem + kCeilABytes + kCeilBBytes;   // twelve 512-byte scale tiles (A: 4, B: 8), all 0x38
  uint64_t *bar_done = (uint64_t *)(sf_smem + kCeilSfBytes), *bar_step = bar_done + 1;
  uint64_t *bar_ring = bar_step + 1;
  uint32_t *tmem_slot = (uint32_t *)(bar_ring + 4);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = PAIR ? (int)cluster_ctarank() : 0;

  for (int i = threadIdx.x; i < (kCeilABytes + kCeilBBytes) / 4; i += kCeilThreads)   // every nibble pattern, cheaply
    ((uint32_t *)smem)[i] = (uint32_t)(i + blockIdx.x * 977) * 2654435761u;
  for (int i = threadIdx.x; i < kCeilSfBytes / 4; i += kCeilThreads) ((uint32_t *)sf_smem)[i] = 0x38383838u;
  fence_proxy_async_smem();
  if (threadIdx.x == 0) {
    mbar_init(bar_done, 1);
    mbar_init(bar_step, 1);
    for (int i = 0; i < 4; ++i) mbar_init(&bar_ring[i], 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    if (PAIR) tmem_alloc_pair(tmem_slot, 512);
    else tmem_alloc(tmem_slot, 512);
  }
  tc_fence_before();
  if (PAIR) cluster_sync_all();
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // unit block scales in columns 256 .. 303 of every lane (A: 16 columns, B: 32), each warp its own quadrant
  {
    uint32_t ones[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) ones[i] = 0x38383838u;
    const uint32_t base = tmem_base + ((uint32_t)(warp * 32) << 16) + 256;
    tmem_st16(base, ones);
    tmem_st16(base + 16, ones);
    tmem_st16(base + 32, ones);
    tmem_st_wait();
  }
  tc_fence_before();
  if (PAIR) cluster_sync_all();
  else __syncthreads();
  tc_fence_after();

  if (warp == 1 && rank == 0 && (commit_each & 16)) {
    // the whole warp runs the loop; one elected lane issues (see mma_mxf4nvf4_elect)
    const uint32_t idesc = idesc_mxf4nvf4(PAIR ? 256 : 128, bn);
    const uint64_t da = smem_desc_sw128(smem_u32(smem)), db = smem_desc_sw128(smem_u32(smem + kCeilABytes));
    const uint32_t sfa = tmem_base + 256, sfb = sfa + 16, sfb_step = (uint32_t)((bn + 127) / 128) * 4;
    const long long t0 = clock64();
    bool ok = true;
    for (int it = 0; it < iters; ++it) {
      if (commit_each & 4) tc_fence_after();
      if (commit_each & 8) { if (it >= 3 && !mbar_wait(&bar_ring[(it - 3) & 3], ((it - 3) >> 2) & 1)) { ok = false; break; } tc_fence_after(); }
      const uint32_t rot = (commit_each & 32) ? (uint32_t)(it & 1) * 4u : 0u;   // alternate between two descriptor pairs, as stages do
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (PAIR) mma_mxf4nvf4_pair_elect(tmem_base, da + 2 * j + rot, db + 2 * j + rot, idesc, sfa + 4 * j, sfb + sfb_step * j, (uint32_t)((it | j) != 0));
        else mma_mxf4nvf4_elect(tmem_base, da + 2 * j + rot, db + 2 * j + rot, idesc, sfa + 4 * j, sfb + sfb_step * j, (uint32_t)((it | j) != 0));
      }
      if (commit_each & 8) {
        if (PAIR) tc_commit_pair_elect(&bar_ring[it & 3]);
        else tc_commit_elect(&bar_ring[it & 3]);
      } else if (commit_each & 1) {
        if (PAIR) tc_commit_pair_elect(bar_step);
        else tc_commit_elect(bar_step);
      }
    }
    const long long t1 = clock64();
    if (PAIR) tc_commit_pair_elect(bar_done);
    else tc_commit_elect(bar_done);
    if (!mbar_wait(bar_done, 0) || !ok) atomicCAS(status, 0u, 0x501u);
    const long long t2 = clock64();
    if (lane == 0) {
      cycles[2 * blockIdx.x] = (unsigned long long)(t1 - t0);
      cycles[2 * blockIdx.x + 1] = (unsigned long long)(t2 - t0);
    }
  } else if (warp == 1 && lane == 0 && rank == 0) {
    const uint32_t idesc = idesc_mxf4nvf4(PAIR ? 256 : 128, bn);
    const uint64_t da = smem_desc_sw128(smem_u32(smem)), db = smem_desc_sw128(smem_u32(smem + kCeilABytes));
    const uint32_t sfa = tmem_base + 256, sfb = sfa + 16, sfb_step = (uint32_t)((bn + 127) / 128) * 4;
    const long long t0 = clock64();
    const uint32_t sf_addr = smem_u32(sf_smem);
    for (int it = 0; it < iters; ++it) {
      if (commit_each & 4) tc_fence_after();   // as after a barrier wait in the GEMM's main loop
      if (commit_each & 8) { if (it >= 3 && !mbar_wait(&bar_ring[(it - 3) & 3], ((it - 3) >> 2) & 1)) break; tc_fence_after(); }   // wait for the MMAs of three iterations ago
      if (commit_each & 2) {   // the stage's scale tiles copied from shared memory by this thread (tcgen05.cp), as a GEMM without scale warps would
#pragma unroll
        for (int q = 0; q < 12; ++q) {
          const uint32_t col = q < 4 ? sfa + 4 * q : sfb + 4 * (q - 4);
          if (PAIR) tmem_cp_32x128b_warpx4_pair(col, smem_desc_sf(sf_addr + q * 512));
          else tmem_cp_32x128b_warpx4(col, smem_desc_sf(sf_addr + q * 512));
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (PAIR) mma_mxf4nvf4_pair(tmem_base, da + 2 * j, db + 2 * j, idesc, sfa + 4 * j, sfb + sfb_step * j, (uint32_t)((it | j) != 0));
        else mma_mxf4nvf4(tmem_base, da + 2 * j, db + 2 * j, idesc, sfa + 4 * j, sfb + sfb_step * j, (uint32_t)((it | j) != 0));
      }
      if (commit_each & 8) {
        if (PAIR) tc_commit_pair(&bar_ring[it & 3]);
        else tc_commit(&bar_ring[it & 3]);
      } else if (commit_each & 1) {   // as the GEMM's main loop does to hand a stage back; nobody waits on this barrier
        if (PAIR) tc_commit_pair(bar_step);
        else tc_commit(bar_step);
      }
    }
    const long long t1 = clock64();   // all issued
    if (PAIR) tc_commit_pair(bar_done);
    else tc_commit(bar_done);
    if (!mbar_wait(bar_done, 0)) atomicCAS(status, 0u, 0x501u);
    const long long t2 = clock64();   // all complete
    cycles[2 * blockIdx.x] = (unsigned long long)(t1 - t0);
    cycles[2 * blockIdx.x + 1] = (unsigned long long)(t2 - t0);
  }
  __syncwarp();
  tc_fence_before();
  if (PAIR) cluster_sync_all();   // the odd CTA keeps its tensor memory and shared memory until the pair's MMAs are done
  else __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, 512);
    else tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace nvb

using namespace nvb;

extern "C" nvfp4a_status nvfp4a_b200_mma_ceiling(int bn, int pair, int iters, int commit_each, unsigned long long *cycles, cudaStream_t stream) {
  const char *fn = "nvfp4a_b200_mma_ceiling";
  clear_error();
  if (bn < 64 || bn > 256 || bn % 64 || iters < 1 || iters > (1 << 20) || !cycles)
    return fail(NVFP4A_INVALID_VALUE, "%s: bn = %d (64, 128, 192, 256), iters = %d (1 .. 2^20), cycles must not be NULL", fn, bn, iters);
  if (nvfp4a_status st = check_device()) return st;
  const int sms = device_sms(), grid = pair ? sms / 2 * 2 : sms;
  cudaError_t e;
  if (pair) {
    e = cudaFuncSetAttribute(mma_ceiling_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCeilSmem);
    if (e != cudaSuccess) return cuda_fail(e, fn);
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(kCeilThreads, 1, 1);
    cfg.dynamicSmemBytes = kCeilSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, mma_ceiling_kernel<true>, bn, iters, commit_each, cycles, kernel_status_device_ptr());
  } else {
    e = cudaFuncSetAttribute(mma_ceiling_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCeilSmem);
    if (e != cudaSuccess) return cuda_fail(e, fn);
    mma_ceiling_kernel<false><<<grid, kCeilThreads, kCeilSmem, stream>>>(bn, iters, commit_each, cycles, kernel_status_device_ptr());
    e = cudaGetLastError();
  }
  return cuda_fail(e, fn);
}
