/*
 * znn_debug.h -- measurement aids, experiment switches and test hooks of libznn_cuda.so.
 * Nothing here is part of the drop-in boundary (include/znn_cuda.h); a host program never needs these.
 * Same conventions: 0 or a negative ZNN_ERR_* code.
 */
#ifndef ZNN_DEBUG_H
#define ZNN_DEBUG_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* ---- switches of the in-place tensor-core GEMM (all default on) ---- */
/* In-place path only: 1 (default) = the converter warps leave the raw fp32 tile as the hi operand:
 * the tensor core ignores the 13 low mantissa bits of a kind::tf32 operand (measured on B200: results
 * are bit-identical to mode 0); 0 = they also store hi = x with those bits cleared. */
int znn_gemm_set_conv_mode(int mode);
/* In-place path only: 1 (default) = persistent launch (one CTA pair per SM pair walks the output tiles, so the
 * next tile's main loop overlaps the previous tile's epilogue); 0 = one CTA pair per output tile. */
int znn_gemm_set_persistent(int enable);
/* 1 (default) = products of 8..64 rows against a wide, long matrix (N, K >= 512) are computed as the transposed product (N rows,
 * at most 64 columns: many tiles instead of a quarter-filled one per column block) and written back transposed by a small
 * kernel (znn_gemm_last_path reports 5); 0 = such products take the ordinary path. */
int znn_gemm_set_skinny(int enable);
/* In-place path only: 1 (default) = when the last round of the persistent walk would be less than 70 % full, its tiles
 * are cut into K-slices (whole accumulation chunks) run by otherwise idle CTA pairs; the slices' partial tiles are added
 * in slice order by a small second kernel (deterministic).  0 = every tile is one unit. */
int znn_gemm_set_tail_split(int enable);
/* Diagnostic: where the first bounded device-side wait of a tensor-core GEMM expired since the last call (16 ints:
 * claimed flag, role, barrier, work unit, counter, M, N, K, split-K slices, tile width, CTA rank, CTA pair, units,
 * pairs, beta*1000, batch); all zero when none did.  Reading clears the record. */
int znn_gemm_wait_record(int* out16);
/* Measurement aid: with profiling on, every tensor-core GEMM kernel launch (not its split
 * pre-pass) is bracketed by CUDA events on the launching stream; znn_gemm_profile_read waits
 * for them and returns the summed kernel time, the launch count and the algorithmic
 * floating-point operations (2*M*N*K*batch) of those launches, then clears the record. */
int znn_gemm_profile(int enable);
int znn_gemm_profile_read(double* kernel_ms, long long* launches, double* flops);

/* Role profile of the fused attention kernels, filled only by a build with -DZNN_ATTN_PROFILE (all zero otherwise):
 * cycles CTA pair 0's leader spent in each role's loop and inside each kind of wait, summed over the launches since
 * the last read: [0] MMA loop, [1] x_conv, [2] y_conv, [3] w_ready, [4] z_conv, [5] acc_empty waits; [8] transform loop,
 * [9] s_full, [10] acc_full waits; [12] TMA producer loop, [13] its waits; [14] converter loop, [15] its waits;
 * [16] converter proxy fence, [17] fence + arrival; transform: [18] score load, [19] W store + hand-off, [20] accumulator drain,
 * [21] load-to-hand-off of one block.  32 values. */
int znn_debug_attn_profile(long long* out32);
/* Fused attention, per host thread: 0 (default) = converter warps inside the kernel split every landed tile into its TF32
 * head and fp32 remainder; 1 = the remainder (lo) planes of the operands that pass through shared memory are computed once
 * by a pre-pass and loaded by TMA next to the values, straight to the MMA issuer's barrier (no converter role, no proxy
 * fence).  Bit-identical results; measured no faster (the kernels wait for the tiles' arrival either way) and the pre-pass
 * costs 16-32 us per call, hence not the default. */
int znn_debug_set_attn_planes(int enable);
/* Fused attention, per host thread: 0 (default) = while the MMA issuer waits for a block's tile it issues the previous
 * block's second product as soon as that product's own inputs are there; 1 = the fixed order first product of block g,
 * second product of block g - 1, ... whatever arrives first.  Same instructions on the same buffers either way (results
 * are bit-identical); the switch exists for A/B timing. */
int znn_debug_set_attn_issue_order(int in_order);
/* Fused attention, per host thread: 1 (default) = the work units (256 rows of one batch x head slice each) are dealt to
 * the CTA pairs by a table made on the host once per problem shape (longest unit to the least loaded pair); 0 = by the
 * kernel's own arithmetic (units dealt round by round in alternating direction).  Every unit is computed by one pair
 * with the same arithmetic either way: results are bit-identical. */
int znn_debug_set_attn_schedule(int enable);
/* Host arithmetic only (no device needed): how the fused attention kernels' work units of a problem with `nslices`
 * (batch x head) slices of T positions are dealt to `pairs` CTA pairs.  rows_first = 1: forward and dQ (the blocks of a
 * unit run up to the diagonal); 0: dK and dV.  table_form = 1: the host-made table; 0: the kernel's own dealing.
 * units_per_pair[pairs] and blocks_per_pair[pairs] receive every pair's count of units and of 64-column blocks.
 * ZNN_ERR_INVALID if the table would not hold every unit exactly once. */
int znn_debug_attn_plan(int rows_first, int nslices, int T, int pairs, int table_form, int* units_per_pair, int* blocks_per_pair);

/* Conv2D path of the calling host thread: 0 (default) = layers with Ci*KH*KW >= 64 taps, at most 64 output channels and at
 * least 4096 output pixels run as implicit-im2col GEMMs on the tensor cores; 1 = never (direct kernels and the explicit
 * im2col lowering), for A/B comparisons. */
int znn_debug_set_conv_path(int mode);
/* Role profile of the tensor-core convolution kernel, filled only by a build with -DZNN_CONV_PROFILE (all zero otherwise):
 * cycles one lane of each role of CTA 0 spent, summed over the launches since the last read: [0] producer loop, [1] gather
 * issue, [2] wait for a free stage, [3] split + store, [4] proxy fence, [5] hand-off; [6] MMA loop, [7] wait for a full
 * stage, [8] wait for a drained accumulator, [9] issue; [10] epilogue loop, [11] wait for a finished chunk, [12] drain,
 * [13] store.  16 values. */
int znn_debug_conv_profile(long long* out16);

/* ---- test hooks ---- */
/* SM cycles a GEMM role waits on an mbarrier before it gives up, sets a ZNN_DEV_*_WAIT_EXPIRED bit in the device status
 * word and leaves (default 4e9, about 2 s; 0 restores the default).  Applies to kernels launched afterwards. */
int znn_debug_set_wait_limit(unsigned long long sm_cycles);
/* Launches a one-thread kernel that waits, with the GEMM roles' own wait routine, on an mbarrier nothing arrives at, for
 * at most limit_cycles (1 .. 2e9): the wait runs out, ZNN_DEV_TMA_WAIT_EXPIRED is set in the status word and the kernel
 * returns normally.  Exercises the recovery path (status word -> later GEMMs return without work ->
 * znn_device_status(clear = 1) restores service) without hanging, trapping or faulting anything. */
int znn_debug_wait_probe(unsigned long long limit_cycles);
/* Host-side fault injection: the n-th kernel launch from now (0 = the next one), by any host thread, is reported as a
 * failed launch (ZNN_ERR_CUDA, "injected failure") although the kernel was enqueued; n < 0 disarms.  Lets tests check
 * that callers unwind cleanly from an error in the middle of a step. */
int znn_debug_fail_after(long long n);

/* Runs the data-parallel bucket schedule (when each gradient bucket's all-reduce starts during the backward sweep)
 * against a caller-supplied reduction, without a GPU: parameters at offsets[0..n_params) of a slab of `total` floats,
 * buckets of at least bucket_floats, uses[i] tape ops reading parameter i; completion_order lists, one entry per tape op
 * input, the parameter whose reader just ran backward.  fn(ctx, begin, count) is called for each bucket at the moment
 * the real schedule would start its all-reduce, and for the rest at the end in slab order; a nonzero return stops all
 * further reductions and comes back as this call's result. */
typedef int (*znn_debug_allreduce_fn)(void* ctx, size_t begin, size_t count);
int znn_debug_bucket_schedule_run(const size_t* offsets, int n_params, size_t total, size_t bucket_floats, const int* uses,
                                  const int* completion_order, int n_events, znn_debug_allreduce_fn fn, void* ctx,
                                  int* n_buckets);

#ifdef __cplusplus
}
#endif
#endif
