/*
 * Profiling hooks of librwkvq_b200.so.  NOT part of the C ABI of include/rwkvq_b200.h: unstable,
 * exported only for the package's own microbenchmarks, and free to change or vanish.
 */
#ifndef RWKVQ_PROFILING_H
#define RWKVQ_PROFILING_H
#ifdef __cplusplus
extern "C" {
#endif
/* With a device buffer of 512 uint64 set, CTA (0,0,0) of every later rwkvq_gemm launch of the calling
 * process records global-timer nanoseconds of its pipeline events (slot map in the kernel source);
 * NULL (the default) switches it off. */
void rwkvq_profiling_gemm_trace(void* buf512);
/* rwkvq_gemm with more than 128 tokens: 1 keeps 128-row tiles (one accumulator per activation slab),
 * 2 takes 256-row tiles (two accumulators) wherever the row count allows, 0 (the default) leaves the
 * choice to the launcher (256-row tiles once they alone fill the SMs). */
void rwkvq_profiling_gemm_acc_mode(int mode);
/* With a device buffer of 8 uint64 set, CTA (0,0,0) of every later small-batch launch records
 * global-timer nanoseconds: 0 start, 1 producer done, 2 activations staged, 3 products done,
 * 4 cluster barrier passed, 5 reduced and stored, 6 end.  force_ks > 0 overrides the launcher's choice:
 * low 4 bits the cluster size (0: keep the launcher's), +16 groups of 256 rows, +32 groups of 128 rows,
 * +64 half the token tile (twice the token groups), +128 half again. */
void rwkvq_profiling_batch_trace(void* buf8, int force_ks);
/* The same override for tensors of one shape only (rows = 0: every shape); 0 switches it off. */
void rwkvq_profiling_batch_force(int force_ks, int rows, int cols);
/* Small-batch linear on tcgen05: > 0 selects it at every batch size and forces the cluster size where
 * that divides the pass count (1000: every batch size, launcher's cluster size), -1 routes every
 * call to the mma.sync kernel instead, 0 restores the launcher's choice. */
void rwkvq_profiling_tcb_force(int force_ks);
/* Precision of the small-batch linears: 1 single fp16 operands (what RWKVQ_BATCH_FAST=1 selects),
 * 0 two-term operands (the default), -1 read the environment again. */
void rwkvq_profiling_batch_fast(int fast);
/* The exact zero-group skip of the single-vector GEMV (what RWKVQ_ZERO_SKIP=1 selects): 1 on, 0 off (the
 * default), -1 read the environment again. */
void rwkvq_profiling_zero_skip(int on);
/* Decode step above 32 streams in the default precision: 1 runs r / k / v, the ffn key and the head on the
 * two-term tcgen05 linear at every such batch (what RWKVQ_TCB_EXACT=1 selects), 0 keeps them on mma.sync
 * (RWKVQ_TCB_EXACT=0), -1 reads the environment again (unset: the launcher's measured choice by batch size). */
void rwkvq_profiling_tcb_exact(int on);
#ifdef __cplusplus
}
#endif
#endif
