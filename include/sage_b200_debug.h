/*
 * sage_b200_debug.h - tuning and profiling aids of libsage_b200 (sm_100a).
 *
 * Not part of the drop-in boundary (include/sage_b200.h): nothing here has a counterpart in
 * the reference's operator interface, and production callers need none of it.
 */
#ifndef SAGE_B200_DEBUG_H_
#define SAGE_B200_DEBUG_H_

#ifdef __cplusplus
extern "C" {
#endif

/*
 * How the decode kernel would share out one problem of rows <= 16 on a device of `sm_count` SMs
 * (debug; pure host arithmetic, callable without a GPU).  act_kind: the producer fused into a
 * single-row launch (0 none, 1 residual add + RMSNorm, 2 SwiGLU).  fields[8] = CTAs, K slices,
 * whole-tile mode (0/1), units per ring stage (0: the share is resident in shared memory),
 * shared-memory unit slots per CTA, warps per CTA, dynamic shared bytes, scratch needed (0/1).
 * No counterpart in the reference.
 */
int sageb200_debug_plan(int rows, int n, int k, int sm_count, int act_kind, int *fields);

/*
 * Programmatic dependent launch (on by default): the decode kernel and the decode glue are
 * launched so that they may be scheduled before the previous kernel of the stream has
 * finished; they prefetch packed weights and codebooks, then wait for the previous kernel
 * before reading activations or writing anything.  `enabled` is a bit mask: 1 the packed-linear
 * kernels, 2 every decode glue kernel, 4 the attention step alone (default 5); 0 switches to plain
 * launches (debug).  No counterpart in the reference.
 */
int sageb200_set_pdl(int enabled);

/*
 * Profiling aid, active only in a library built with -DSAGEB200_TRACE (python -m
 * sage_b200.build --trace; the default build ignores the buffer): while `device_buffer` is non-NULL every CTA of the decode kernel
 * writes 16 readings at device_buffer[(512*launch + cta)*16 ...]: SM clocks at the phases of
 * its work ([0..12], [14] = after the wait for the previous kernel) and the global
 * nanosecond timer at its start [13] and end [15].  `launch` counts the decode-kernel launches
 * since this call and stops at 63; the buffer holds 64*512*16*8 bytes (one launch only:
 * 512*16*8).  NULL switches it off.
 * No counterpart in the reference.
 */
int sageb200_debug_trace(void *device_buffer);

/*
 * The tcgen05 GEMM (rows >= 33) runs as clusters of two CTAs with cta_group::2 MMAs whenever the
 * shape allows it; 0 switches that off for A/B timing (process-wide, not thread-safe).
 * No counterpart in the reference.
 */
int sageb200_debug_gemm_pairs(int enabled);

/*
 * The tile plan the tcgen05 GEMM would use for a shape (host arithmetic, no GPU needed), rows >= 33:
 * fields[0] tokens per accumulator, [1] token blocks, [2] blocks of 128 output rows, [3]
 * accumulators per CTA, [4] CTA pairs (cta_group::2), [5] K splits, [6] 128-channel groups per
 * split, [7] pipeline stages, [8] dynamic shared memory bytes, [9] FP32 scratch of the split tiles in
 * KiB.  `allow_split` = 0 plans for a caller without that scratch.  fields holds 10 ints.
 */
int sageb200_debug_gemm_plan(int rows, int n, int k, int sm_count, int allow_split, int *fields);

#ifdef __cplusplus
}
#endif
#endif /* SAGE_B200_DEBUG_H_ */
