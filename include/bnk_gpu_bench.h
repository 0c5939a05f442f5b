/*
 * bnk_gpu_bench.h -- measurement helpers around libbnkgpu.so, exported by libbnkgpu_bench.so.
 *
 * Nothing here is part of the drop-in boundary (that is bnk_gpu.h) and nothing here has a counterpart
 * in the reference: these calls exist for the benchmark and the tests, which need device-side timing
 * across several batches, the integer issue-rate probe
 * that gives the seal/open kernels their ALU roofline denominator, a seeded device-side fill for
 * synthetic payloads, and a copy-only pass over a batch's buffers that measures what the host link can
 * carry.  The library reaches into the handles of libbnkgpu.so, so both must come from the same build.
 */
#ifndef BNK_GPU_BENCH_H
#define BNK_GPU_BENCH_H

#include "bnk_gpu.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- timers (CUDA events on the batches' own streams) ----
 * bnk_timer_start records a start event on batches[0]'s stream and makes the other batches' streams
 * wait for it; bnk_timer_stop records an end event on every batch, waits, and returns the longest
 * start-to-end span in milliseconds. */
int bnk_timer_start(bnk_ctx *ctx, bnk_batch *const *batches, uint32_t n);
int bnk_timer_stop(bnk_ctx *ctx, bnk_batch *const *batches, uint32_t n, float *ms);
/* Measures the 32-bit integer issue rate of the device (dependent chains of add/xor/funnel-shift on the
 * ALU pipe, optionally mixed with multiply-adds on the FMA pipe); result in 10^12 operations/s. */
int bnk_probe_int_throughput(bnk_ctx *ctx, int mix, double *tera_ops_per_s);
/* What other work costs beside ChaCha20 rounds: runs ChaCha20 double rounds at the seal/open kernels' occupancy
 * (4 warps per scheduler) with k extra operations of one kind per double round interleaved from independent chains,
 * and returns scheduler cycles per double round per warp.  kind: 0 none (k = 0), 1 = 32x32+64 multiply-add
 * (k = 8, 16), 2 = FP64 fused multiply-add (16, 32), 3 = 32-bit multiply-add (16, 32), 4 = FP32 fused multiply-add
 * (16, 32), 5 = high half of a 32x32 product (8, 16); 6 (k = 0) = no extra work but TWO cipher blocks per thread at
 * half the warps (2 per scheduler), per double round of one block.  Other (kind, k) pairs are BNK_ECUDA / invalid value. */
int bnk_probe_coissue(bnk_ctx *ctx, int kind, int k, double *cycles_per_double_round);
/* Fills the device mirror of the batch's ring with SplitMix64 output (seeded, position-dependent). */
int bnk_batch_fill_random(bnk_batch *b, uint64_t seed);

/* Queues on the batch's stream the same host<->device copies a seal or open submit of npkts packets would
 * make (pinned ring and descriptors to the device mirror when `up`, back when `down`) and no kernel: the
 * ceiling of the host link for the end-to-end numbers.  Completion is reported by bnk_wait as usual. */
int bnk_batch_copy_only(bnk_batch *b, uint32_t npkts, int up, int down);

/* What the host link gives small batches: `threads` host threads, each with a stream and pinned buffers of its
 * own, copy `bytes` to the device and `bytes` back and wait, `rounds` times in a closed loop, no kernel in
 * between (directions: 1 = up only, 2 = down only, 3 = both).  Result: copy rounds per second over all threads.
 * 190,000 bytes is one 128-packet batch of 1420-byte packets. */
int bnk_probe_copy_rounds(bnk_ctx *ctx, uint32_t threads, uint64_t bytes, uint32_t rounds, int directions,
                          double *rounds_per_s);

#ifdef __cplusplus
}
#endif
#endif
