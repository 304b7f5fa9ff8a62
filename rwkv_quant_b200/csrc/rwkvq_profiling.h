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
#ifdef __cplusplus
}
#endif
#endif
