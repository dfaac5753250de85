/* pelica_moe_diag.h - measurement and test hooks of libpelica_moe.so.
 *
 * Not part of the boundary a Pelica engine binds (include/pelica_moe.h): nothing here
 * replaces a reference interface. The benchmark, the profiles and the tests use these to
 * time phases on the device, to count launches, to see which kernel family served a call,
 * and to make a bounded device-side wait run out on purpose.
 */
#ifndef PELICA_MOE_DIAG_H
#define PELICA_MOE_DIAG_H

#include "pelica_moe.h"

#ifdef __cplusplus
extern "C" {
#endif

/* kernels launched by this context since creation */
PM_API int64_t pm_ctx_launch_count(pm_ctx *ctx);
/* launches of the expert-product kernels per family since creation: out[PM_PATH_N] */
enum {
  PM_PATH_GENERAL = 0, /* warp-per-row kernels (any type, any token count)            */
  PM_PATH_TENSOR = 1,  /* tcgen05 grouped kernels                                     */
  PM_PATH_DECODE = 2,  /* the persistent one-token stack kernel                       */
  PM_PATH_MULTI = 3,   /* weight-streaming kernels for a few tokens per expert        */
  PM_PATH_N = 4
};
PM_API int32_t pm_ctx_path_counts(pm_ctx *ctx, int64_t *out);
/* device-timed interval on the context's stream, in milliseconds */
PM_API int32_t pm_timer_start(pm_ctx *ctx);
PM_API int32_t pm_timer_stop(pm_ctx *ctx, float *ms);
/* writes a buffer larger than L2 (evicts cached weights between timed runs) */
PM_API int32_t pm_flush_l2(pm_ctx *ctx);
/* per-phase device timing (CUDA events around each phase of the operator):
 * enable, run, then read milliseconds and span counts per phase; phase names
 * by index below pm_profile_phases(). Costs two event records per phase. */
PM_API int32_t pm_profile_enable(pm_ctx *ctx, int32_t on);
PM_API int32_t pm_profile_phases(void);
PM_API const char *pm_profile_phase_name(int32_t i);
PM_API int32_t pm_profile_read(pm_ctx *ctx, float *ms, int64_t *spans);
/* phase trace of the decode kernel: called with out == NULL it switches tracing on and
 * returns the number of int64 entries; called with a buffer it copies the last call's
 * stamps. */
PM_API int32_t pm_stack_trace(pm_stack *stack, int64_t *out, int32_t capacity);

/* ---- making a bounded wait run out (tests) ------------------------------------------
 * Every device-side wait of the library (arrival counters and copy barriers of the decode
 * kernel, the product barrier of the tensor-core kernels) gives up after a time limit, sets
 * an error word and lets the kernel return; the host then reports PM_ERR_TIMEOUT. These
 * hooks make that happen without any fault: the limit is shortened and the awaited event is
 * one that cannot arrive. */
/* the limit of every bounded wait of kernels launched by this context (default 2 s) */
PM_API int32_t pm_debug_set_wait_limit_ns(pm_ctx *ctx, uint64_t ns);
/* the next decode-kernel call of this stack waits for one more arrival than its CTAs
 * make: every CTA's wait runs out in the first layer */
PM_API int32_t pm_debug_stack_fault_next_call(pm_stack *stack);
/* tensor-core kernels launched by this context issue no products from 256-value block
 * `block` on (and never signal them): the workers' wait runs out. -1 = off */
PM_API int32_t pm_debug_tc_fault_block(pm_ctx *ctx, int32_t block);

/* free device memory as the CUDA runtime reports it (a test checks that a call that must
 * not allocate leaves it unchanged) */
PM_API int32_t pm_debug_device_free_bytes(pm_ctx *ctx, uint64_t *out);

#ifdef __cplusplus
}
#endif
#endif /* PELICA_MOE_DIAG_H */
