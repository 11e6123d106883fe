// All-gather of a tensor-parallel layer's output over peer memory: every rank has written its own columns of the activation
// matrix [T][M] (row pitch M elements) into its local copy of a buffer that exists at the same place on every GPU of the
// node (peer-mapped); this kernel copies those columns into every peer's copy with plain 16-byte stores over NVLink and
// then runs a barrier among the ranks on flags in the same kind of memory, so that after it the whole matrix is present
// everywhere -- one launch instead of an NCCL all-gather plus a reassembly copy.  There are no multicast loads or stores.
//
// Barrier: rank r bumps its epoch (a counter in its own memory, so that a replayed CUDA graph keeps counting), fences,
// writes the epoch into slot r of every peer's flag array and waits until all slots of its own array have reached the
// epoch.  The wait is bounded (about a second of SM clock); on expiry the kernel records code 0x401 in the kernel status
// word and returns.  Copies larger than one CTA handles well are split into a copy launch and a one-CTA barrier launch.
// Ranks live on different GPUs: kernels that wait on one another must never share a GPU.
#include "operands.cuh"
#include "sm100.cuh"
#include "tp_barrier.cuh"

namespace nvb {

struct TpGatherArgs {
  uint8_t *buf[kMaxRanks];                 // the activation buffer on every rank (buf[rank] is local)
  unsigned long long *flags[kMaxRanks];    // flag array on every rank
  int world, rank;
  int rows;                                // T
  long long row_pitch_bytes, col_offset_bytes, shard_bytes;  // this rank's columns: [col_offset, col_offset + shard_bytes) of every row
  unsigned *status;
  unsigned tag;
  long long wait_cycles;
  int copy, barrier;                       // barrier: 1 post and wait, 2 post only (deferred form)
};

__global__ void __launch_bounds__(1024) tp_gather_kernel(const TpGatherArgs a) {
  if (a.copy) {
    const long long vec_per_row = a.shard_bytes >> 4;   // 16-byte vectors (the shard is a multiple of 128 elements)
    const long long total = vec_per_row * a.rows;
    const uint8_t *src = a.buf[a.rank];
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (long long)gridDim.x * blockDim.x) {
      const long long r = v / vec_per_row, c = v - r * vec_per_row;
      const long long off = r * a.row_pitch_bytes + a.col_offset_bytes + (c << 4);
      const uint4 x = *(const uint4 *)(src + off);
      for (int p = 0; p < a.world; ++p)
        if (p != a.rank) *(uint4 *)(a.buf[p] + off) = x;
    }
    if (!a.barrier) __threadfence_system();   // a copy-only launch: the barrier launch that follows cannot order these stores
  }
  if (!a.barrier) return;
  __syncthreads();   // the flags' release stores below order every thread's copies (see tp_barrier_cta)
  if (a.barrier == 2) tp_post_epoch(a.flags, a.world, a.rank);
  else tp_barrier_cta(a.flags, a.world, a.rank, a.status, a.tag, a.wait_cycles);
}

// the consumer side of the deferred form on its own: one small CTA waits for the peers' posts (closes a sequence of deferred calls)
__global__ void __launch_bounds__(32) tp_wait_kernel(const TpGatherArgs a) {
  tp_wait_posts(a.flags, a.world, a.rank, a.status, a.tag, a.wait_cycles);
}

}  // namespace nvb

using namespace nvb;

// buffers / flags: `world` device pointers each (peer mappings of one symmetric allocation; entry `rank` is local).
// The shard is columns [col_offset_bytes, col_offset_bytes + shard_bytes) of each of `rows` rows of row_pitch_bytes; all
// three are multiples of 16.  The flag array holds 16 unsigned 64-bit words, zero before the first use and owned by this
// function afterwards.
static void launch_gather(const TpGatherArgs &a, int grid, int block, cudaStream_t stream) {
  tp_gather_kernel<<<grid, block, 0, stream>>>(a);
}

static nvfp4a_status tp_gather_run(const char *fn, void *const *buffers, void *const *flags, int world, int rank, int rows, long long row_pitch_bytes,
                                   long long col_offset_bytes, long long shard_bytes, int post_only, cudaStream_t stream) {
  clear_error();
  if (!buffers || !flags || world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
    return fail(NVFP4A_INVALID_VALUE, "%s: needs buffers, flags and 0 <= rank < world <= %d", fn, kMaxRanks);
  if (rows < 0 || row_pitch_bytes < 0 || ((row_pitch_bytes | col_offset_bytes | shard_bytes) & 15) || col_offset_bytes < 0 || shard_bytes < 0 ||
      col_offset_bytes + shard_bytes > row_pitch_bytes)
    return fail(NVFP4A_INVALID_VALUE, "%s: pitch, offset and shard bytes must be non-negative multiples of 16 with the shard inside a row", fn);
  if (nvfp4a_status st = check_device()) return st;
  TpGatherArgs a;
  memset(&a, 0, sizeof a);
  for (int p = 0; p < world; ++p) {
    if (!buffers[p] || !flags[p] || ((uintptr_t)buffers[p] & 15) || ((uintptr_t)flags[p] & 7))
      return fail(NVFP4A_INVALID_VALUE, "%s: buffer / flag pointer of rank %d is NULL or misaligned", fn, p);
    a.buf[p] = (uint8_t *)buffers[p];
    a.flags[p] = (unsigned long long *)flags[p];
  }
  a.world = world; a.rank = rank; a.rows = rows;
  a.row_pitch_bytes = row_pitch_bytes; a.col_offset_bytes = col_offset_bytes; a.shard_bytes = shard_bytes;
  a.status = kernel_status_device_ptr();
  a.tag = next_launch_tag();
  a.wait_cycles = tp_wait_limit();
  const long long bytes = (long long)rows * shard_bytes * (world - 1);
  if (world == 1) return NVFP4A_OK;
  const int bar = post_only ? 2 : 1;
  if (bytes <= (1 << 20)) {   // one CTA copies and joins the barrier
    a.copy = 1; a.barrier = bar;
    launch_gather(a, 1, 1024, stream);
  } else {
    a.copy = 1; a.barrier = 0;
    const long long vecs = (long long)rows * (shard_bytes >> 4);
    long long grid = (vecs + 1023) / 1024;
    const int cap = device_sms() * 2;
    launch_gather(a, (int)(grid < cap ? grid : cap), 1024, stream);
    a.copy = 0; a.barrier = bar;
    launch_gather(a, 1, 32, stream);
  }
  return cuda_fail(cudaGetLastError(), fn);
}

extern "C" nvfp4a_status nvfp4a_b200_tp_gather(void *const *buffers, void *const *flags, int world, int rank, int rows, long long row_pitch_bytes,
                                               long long col_offset_bytes, long long shard_bytes, cudaStream_t stream) {
  return tp_gather_run("nvfp4a_b200_tp_gather", buffers, flags, world, rank, rows, row_pitch_bytes, col_offset_bytes, shard_bytes, 0, stream);
}

// The deferred form of the gather: copy and post, no wait (the next kernel of every rank waits at its start).
extern "C" nvfp4a_status nvfp4a_b200_tp_gather_post(void *const *buffers, void *const *flags, int world, int rank, int rows, long long row_pitch_bytes,
                                                    long long col_offset_bytes, long long shard_bytes, cudaStream_t stream) {
  return tp_gather_run("nvfp4a_b200_tp_gather_post", buffers, flags, world, rank, rows, row_pitch_bytes, col_offset_bytes, shard_bytes, 1, stream);
}

extern "C" nvfp4a_status nvfp4a_b200_tp_wait(void *const *flags, int world, int rank, cudaStream_t stream) {
  const char *fn = "nvfp4a_b200_tp_wait";
  clear_error();
  if (!flags || world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
    return fail(NVFP4A_INVALID_VALUE, "%s: needs flags and 0 <= rank < world <= %d", fn, kMaxRanks);
  if (nvfp4a_status st = check_device()) return st;
  if (world == 1) return NVFP4A_OK;
  TpGatherArgs a;
  memset(&a, 0, sizeof a);
  for (int p = 0; p < world; ++p) {
    if (!flags[p] || ((uintptr_t)flags[p] & 7)) return fail(NVFP4A_INVALID_VALUE, "%s: flag pointer of rank %d is NULL or misaligned", fn, p);
    a.flags[p] = (unsigned long long *)flags[p];
  }
  a.world = world; a.rank = rank;
  a.status = kernel_status_device_ptr();
  a.tag = next_launch_tag();
  a.wait_cycles = tp_wait_limit();
  tp_wait_kernel<<<1, 32, 0, stream>>>(a);
  return cuda_fail(cudaGetLastError(), fn);
}
