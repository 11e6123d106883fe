/* nvfp4effma_b200.h -- entry points of this implementation that have no counterpart in the reference's C header.
 * They never change what the reference-compatible entry points of nvfp4effma.h compute. */
#ifndef NVFP4EFFMA_B200_H
#define NVFP4EFFMA_B200_H
#include "nvfp4effma.h"
#ifdef __cplusplus
extern "C" {
#endif

/* Self-test of the hardware FP32 -> E2M1 / E4M3 conversions the quantizer uses (no counterpart in the reference, whose
 * encoders are software; the reference proves its own exhaustively in tests/test_nvfp4effma.cu:487-495).  Adds to
 * mismatches[0..3] (device, 4 x unsigned long long, zeroed by the caller) the number of FP32 bit patterns in
 * [first, first + count) on which the hardware conversion differs from the software encoder: [0] E2M1 in the low
 * nibble, [1] E2M1 in the high nibble, [2] E4M3 (NaN inputs are skipped for these three), [3] the packed FP32 -> BF16 rounding
 * of the GEMM epilogues against the software rounding (NaN -> 0x7FC0 included). */
nvfp4a_status nvfp4a_b200_codec_selftest(unsigned long long first, unsigned long long count, unsigned long long *mismatches,
                                         cudaStream_t stream);

/* Kernel route of the GEMM entry points (no counterpart in the reference, which picks kernels from per-architecture
 * tables): 0 = automatic (GEMV for n <= 8, tcgen05 GEMMs where the operand formats have a tensor-core form, CUDA cores
 * otherwise), 1 = always the CUDA-core kernel, whose results are bit-identical to the reference's tiled kernels, 2 = automatic
 * but with the mma.sync GEMV in place of the FP4 tensor-core GEMV (n <= 2), 3 = automatic but INT8 activations keep the exact
 * integer block sums of the DP4A kernel instead of the tensor-core W4A8 GEMM (which takes a call's scratch from the stream's
 * memory pool and agrees with the exact definition within the FP32 accumulation bound).
 * Process-wide, not thread-safe; meant for tests and debugging.  Returns the previous value. */
int nvfp4a_b200_set_route(int route);

/* Health word of the tensor-core kernels (no counterpart in the reference, whose device-side waits are unbounded:
 * src/tensors/mma.cuh:108-114, src/tensors/gemm_tc.cuh:555 there).  Every wait inside this library's kernels gives up
 * after about a second; the kernel then records what it was waiting for and returns.  The first such record of a device stays in
 * the word: bits 0-11 the wait (0x101 operands not delivered, 0x102 stage never released, 0x103 accumulator never completed, 0x104
 * accumulator never drained, 0x105 scale gather, 0x11x the same of the CTA-pair W4A4 kernel; 0x2xx the FP4 GEMV; 0x3xx the W4A16
 * GEMM; 0x401 a peer missing at the tensor-parallel barrier; 0x501 the ceiling measurement), bits 12-31 the sequence number
 * (mod 2^20) of the launch that gave up -- nvfp4a_b200_last_launch() returns the number of the calling thread's latest launch of
 * such a kernel, so a caller can tell its own call from another stream's.  Kernels are asynchronous: the entry point that
 * launched a kernel which later gives up has long returned NVFP4A_OK, and the kernel's outputs are then incomplete.  Callers that
 * need to know poll this word at a point where synchronising is acceptable (the end of a forward pass, outside stream capture).
 * This call SYNCHRONISES the device, copies the word to *status (0 = healthy) and clears it when reset != 0. */
nvfp4a_status nvfp4a_b200_kernel_status(unsigned int *status, int reset);
unsigned int nvfp4a_b200_last_launch(void);

/* Test aid (no counterpart in the reference): the number of SM clock cycles a tensor-parallel barrier (nvfp4a_b200_tp_gather and the
 * fused entries) waits for its peers before it records 0x401 and returns; at least 1000, by default 2e9 (about a second -- ranks
 * that drift further apart than that, e.g. during first-call module loads, trip it).  Process-wide.  Returns 0, or -1 for a
 * value below 1000. */
int nvfp4a_b200_set_wait_limit(long long cycles);

/* Tuning aid (no counterpart in the reference): kernels that support it are launched with programmatic stream serialization, so
 * that their set-up (barriers, tensor-memory allocation, descriptor prefetch -- nothing that touches global memory) runs while the
 * stream's previous kernel drains; they wait for that kernel's completion before their first global access, so stream order is
 * kept as without it.  on = 0 turns the attribute off for launches made after the call.  Process-wide; on by default.  Returns 0. */
int nvfp4a_b200_set_pdl(int on);

/* Measured ceiling of the block-scaled FP4 tensor-core instruction (no counterpart in the reference, which has no sm_100 kernel):
 * every SM's MMA thread issues 4 * iters tcgen05.mma kind::mxf4nvf4 of 128 x bn x 64 (pair != 0: cta_group::2, 256 x bn x 64 per SM
 * pair) back to back on one resident operand stage -- no loads, no epilogue; commit_each bit 0: one tcgen05.commit per four, bit 1: the twelve
 * 512-byte scale tiles of a stage copied into tensor memory by tcgen05.cp before each four.
 * cycles (device, 2 x unsigned long long per CTA of the launch: one CTA per SM) receives, for CTAs that issue, the SM clocks from the
 * first issue to the last issue and to the completion of all MMAs.  The launch is timed by the caller (CUDA events); its flop count
 * is SMs * 4 * iters * 2 * 128 * bn * 64.  Measurement aid: the numbers under profiles/ that the W4A4 GEMM's fraction is quoted
 * against come from this call. */
nvfp4a_status nvfp4a_b200_mma_ceiling(int bn, int pair, int iters, int commit_each, unsigned long long *cycles, cudaStream_t stream);

/* Test aid (no counterpart in the reference): 0 keeps nvfp4a_quantize_ex on its two-launch path (an amax kernel, then the encode kernel)
 * where it would otherwise run the one-read cooperative kernel; 1 (default) restores the choice.  Results are identical bit for bit. */
int nvfp4a_b200_set_quant_fused(int on);

/* Pins the token-tile width of the W4A4 tcgen05 GEMM: 0 = by problem size, 128 (two accumulators in tensor memory, the
 * epilogue overlaps the next tile) or 256 (one accumulator, less shared-memory traffic per flop).  Tuning / test aid, no
 * counterpart in the reference.  Returns 0, or -1 for another value. */
int nvfp4a_b200_set_tile_n(int bn);

/* The W4A4 GEMM's CTA-pair kernel (tcgen05.mma.cta_group::2 on 256 x 256 tiles, csrc/gemm_w4a4_pair.cu; it takes a 16-bit D that
 * TMA can store, beta = 0, no bias, one global per operand, and block scales in aligned 512-byte tiles or images on both
 * operands): -1 = automatic (m, n >= 256 and its rounds of 256 x 256 tiles over the SM pairs estimated no dearer than the
 * single-CTA kernel's rounds; 4096^3: 31 us against 49 us on single CTAs), 0 = never, 1 = wherever it applies.  Results are bit-identical either way.
 * Tuning / test aid, no counterpart in the reference.  Returns 0, or -1 for another value. */
int nvfp4a_b200_set_pair(int mode);

/* Orientation of the W4A4 GEMM on the tensor cores: 1 = B of the call (tokens) on the MMA's M side whenever D is a 16-bit
 * matrix that TMA can store (16-byte aligned base and column pitch, m a multiple of 8), so that a thread holds consecutive
 * elements of D; -1 (default) = the same unless the other orientation needs fewer rounds of tiles; 0 = always A on the M side.  Results lie within the same bound either way.  Tuning / test aid, no
 * counterpart in the reference.  Returns 0, or -1 for another value. */
int nvfp4a_b200_set_swap(int mode);

/* The kernel the calling thread's last GEMM / GEMV call launched: 1 CUDA cores, 2 mma.sync GEMV, 3 FP4 tensor-core GEMV, 4 W4A4
 * tcgen05 GEMM, 5 W4A16 tcgen05 GEMM, 6 DP4A GEMV for INT8 / NVFP4 activations, 7 DP4A GEMM for INT8
 * activations, 8 W4A8 on the W4A16 tcgen05 kernel (INT8 activations as three BF16 planes); 0 before any call.  Test aid, no
 * counterpart in the reference. */
int nvfp4a_b200_last_route(void);

/* The tensor-core W4A8 GEMM keeps the memory of its activation planes (6 bytes per INT8 activation of the largest call so far) in
 * a memory pool of its own per device, so that later calls allocate in microseconds and without synchronising.  This call gives
 * the current device's pool memory that is not in use back to the system (no counterpart in the reference). */
nvfp4a_status nvfp4a_b200_trim_scratch(void);

/* Pins the number of k ranges (CTAs per cluster) of the FP4 tensor-core GEMV: 0 = by problem size, else 1, 2, 4 or 8; a
 * value the problem cannot use (shared memory for the activation digit planes, k / 256) makes that GEMV step aside for the
 * mma.sync one.  A pinned value also lifts the size threshold below which the automatic choice prefers the mma.sync GEMV.  Tuning / test aid, no counterpart in the reference.  Returns 0, or -1 for another value. */
int nvfp4a_b200_set_gemv_splits(int splits);

/* All-gather of a tensor-parallel layer's output over peer memory (no counterpart in the reference, which is single-GPU).
 * buffers[p] / flags[p], p < world <= 8: the activation buffer [rows][row_pitch_bytes] and a flag array of 16 64-bit words
 * (zero before the first use) as mapped on this GPU for every rank of the node (peer mappings of symmetric allocations;
 * entry `rank` is local).  The rank's own columns [col_offset_bytes, + shard_bytes) of every row, already written locally,
 * are stored into every peer's buffer (plain 16-byte stores over NVLink, no multicast), then the ranks meet in a barrier:
 * after the call's kernels the complete matrix is in `buffers[rank]` on every rank.  Every rank must make the same
 * sequence of calls.  The barrier's wait is bounded; nvfp4a_b200_kernel_status reports 0x401 if a peer never arrived. */
nvfp4a_status nvfp4a_b200_tp_gather(void *const *buffers, void *const *flags, int world, int rank, int rows, long long row_pitch_bytes,
                                    long long col_offset_bytes, long long shard_bytes, cudaStream_t stream);

/* nvfp4a_gemv_tc / nvfp4a_gemv_tc_ex (beta = 0) of one rank of a tensor-parallel group with the all-gather fused into the
 * kernel (no counterpart in the reference): D->data points into buffers[rank]; every output is also stored at the same place
 * of each peer's buffer (plain peer stores), and the kernel's last CTA joins the ranks' barrier of nvfp4a_b200_tp_gather
 * (same buffers / flags, same rules).  When the problem runs on another kernel than the mma.sync GEMV, the push is a
 * second launch; the result is the same.  ex may be NULL; a second output (d2) is not supported here.  With world > 1, D's base, its
 * column pitch (ldd elements) and one shard row (m, or m / 2 with SwiGLU, elements) must be multiples of 16 bytes: anything else
 * is NVFP4A_INVALID_VALUE before a kernel is launched. */
nvfp4a_status nvfp4a_b200_gemv_tc_tp(int m, int n, int k, float alpha, const nvfp4a_tensor *A, const nvfp4a_tensor *B, int ldb,
                                     const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias, const nvfp4a_epilogue *ex,
                                     void *const *buffers, void *const *flags, int world, int rank, cudaStream_t stream);

/* The DEFERRED form of the tensor-parallel decode step (1 to 8 BF16 activation vectors; no counterpart in the reference): nobody
 * waits at the END of a gather.  A rank copies its outputs into the peers' buffers and posts its epoch to them -- by a
 * nvfp4a_b200_tp_gather_post launch after the GEMV (push = 0; the GEMV may then be the FP4 tensor-core one), or by the mma.sync
 * GEMV's last CTA (push != 0) -- and goes on.  Instead every nvfp4a_b200_gemv_tc_tp_deferred call waits at the START of its kernel
 * until every peer has posted the epoch this rank has reached, i.e. until the previous gather is complete here and every peer has
 * finished the kernel that read the buffer this call overwrites; there the wait hides behind the launch and the kernel's set-up.
 * A sequence of such calls on alternating buffers (two suffice) needs no other synchronisation between them; it is closed by
 * nvfp4a_b200_tp_wait, after which the last gathered buffer is complete.  Same buffers / flags / layout rules and the same bounded
 * wait (0x401) as nvfp4a_b200_gemv_tc_tp; calls of both forms and of nvfp4a_b200_tp_gather may be mixed on one flag array. */
nvfp4a_status nvfp4a_b200_gemv_tc_tp_deferred(int m, int n, int k, float alpha, const nvfp4a_tensor *A, const nvfp4a_tensor *B, int ldb,
                                              const nvfp4a_tensor *D, int ldd, const nvfp4a_tensor *bias, const nvfp4a_epilogue *ex,
                                              void *const *buffers, void *const *flags, int world, int rank, int push, cudaStream_t stream);
nvfp4a_status nvfp4a_b200_tp_gather_post(void *const *buffers, void *const *flags, int world, int rank, int rows, long long row_pitch_bytes,
                                         long long col_offset_bytes, long long shard_bytes, cudaStream_t stream);
nvfp4a_status nvfp4a_b200_tp_wait(void *const *flags, int world, int rank, cudaStream_t stream);

/* nvfp4a_gemm_tc / nvfp4a_gemm_tc_ex (beta = 0) with the tensor-parallel all-gather fused in (no counterpart in the reference):
 * as nvfp4a_b200_gemv_tc_tp, for more than 8 tokens.  With BF16 activations the tcgen05 GEMM's epilogue stores every tile of
 * D by TMA into the local buffer and into every peer's (plain TMA stores to peer memory; no multicast, no peer loads), so the
 * gather overlaps the GEMM; a barrier launch follows.  Other operand types copy after the GEMM. */
nvfp4a_status nvfp4a_b200_gemm_tc_tp(int m, int n, int k, float alpha, const nvfp4a_tensor *A, const nvfp4a_tensor *B, const nvfp4a_tensor *D,
                                     int ldd, const nvfp4a_tensor *bias, const nvfp4a_epilogue *ex, void *workspace, void *const *buffers,
                                     void *const *flags, int world, int rank, cudaStream_t stream);

/* nvfp4a_gemm_ex that allocates nothing and still computes the RMSNorm column scales once per call: they are staged in a
 * 64 KiB device array inside the library image instead of a workspace.  No counterpart in the reference (its
 * nvfp4a_gemm_ex needs no scratch; its tensor-core entries take a caller workspace).  Same arguments and the same results,
 * bit for bit, as nvfp4a_gemm_ex.  For callers that cannot hand over or allocate scratch at the call: inside stream
 * capture, or where a framework allocator holds all device memory.
 *   - n is limited to nvfp4a_b200_static_scratch_tokens() (16384); a larger n returns NVFP4A_INVALID_VALUE.
 *   - The first call on a device looks the array's address up (cudaGetSymbolAddress): make it before capturing a stream.
 *   - Nothing needs zeroing: every call writes the entries it reads.
 *   - One array per device: calls that overlap in time on a device (two streams, two threads) race on it; serialise them. */
nvfp4a_status nvfp4a_b200_gemm_ex_static(int m, int n, int k, float alpha, const nvfp4a_tensor *A, int lda, const nvfp4a_tensor *B, int ldb,
                                         float beta, const nvfp4a_tensor *C, int ldc, const nvfp4a_tensor *D, int ldd,
                                         const nvfp4a_tensor *bias, const nvfp4a_epilogue *ex, cudaStream_t stream);
int nvfp4a_b200_static_scratch_tokens(void);

#ifdef __cplusplus
}
#endif
#endif
