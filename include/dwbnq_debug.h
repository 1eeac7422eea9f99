/*
 * dwbnq - test and tuning switches. Not part of the drop-in boundary: nothing the
 * reference binds has a counterpart here, and a production caller never needs them.
 *
 * All state set through this header belongs to the CALLING HOST THREAD (it lives in
 * thread-local storage): a thread that forces a kernel family or overrides the planner
 * changes only the kernels of its own later calls, never those of another thread.
 */
#ifndef DWBNQ_DEBUG_H_
#define DWBNQ_DEBUG_H_

#include "dwbnq.h"

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

/* Restricts the kernel family dwbnq_fused_fwd / dwbnq_dwconv_fwd choose for this thread's
 * calls (-1 = automatic; 0..5 as in dwbnq_fused_plan); the tests use it to cover every
 * family on shapes where the planner would pick another one. The environment variable
 * DWBNQ_FORCE_PATH=generic|coop|tma|raw|plane|planegen, read once when the library is
 * first used, sets the default for every thread. */
int dwbnq_set_forced_path(int path);
/* Planner overrides for tuning runs (0 = automatic): planes per tile, 7-row patch blocks
 * per tile, threads per CTA; the fourth value is reserved (pass 0). Values that do not fit
 * the shared-memory budget fall back to the generic kernel. */
int dwbnq_set_tuning(int planes_per_cta, int row_blocks_per_tile, int threads, int rows_per_patch);
/* Restricts the kernel dwbnq_pwconv_fwd / dwbnq_pwconv_fused_fwd choose for this thread's
 * calls: -1 automatic, 0 the plain FMA kernel, 1 the tcgen05 kernel (a shape it cannot take
 * then fails with DWBNQ_ERR_UNSUPPORTED). DWBNQ_PW_FORCE=simt|tc sets the default. */
int dwbnq_set_forced_pw_path(int path);
/* Upper bound on the CTAs of the tcgen05 pointwise kernel for this thread's calls (0 = one per
 * SM): with a few CTAs a small tensor already makes every CTA walk through many tiles, which
 * is what exercises the reuse of pipeline stages and accumulator buffers. */
int dwbnq_set_pw_max_ctas(int ctas);
/* Host only: the launch shape the tcgen05 pointwise kernel would get for `desc` with activations
 * at `x` (only its alignment is looked at) on a device of `sms` SMs. out8 receives: columns per
 * channel tile, channel tiles, activation path (0 = TMA boxes, 1 = one-element gather, 2 =
 * four-position gather), tiles, CTAs, pipeline stages, accumulator buffers in tensor memory, and
 * whether the epilogue groups share each tile's columns. DWBNQ_ERR_UNSUPPORTED for a descriptor
 * that goes to the plain FMA kernel. */
int dwbnq_debug_pwconv_tiling(const dwbnq_pwconv_desc *desc, const void *x, int sms, int *out8);
/* Launches one warp that waits, with the bounded wait every copy-engine kernel of the
 * library uses, on a shared-memory barrier that nothing ever completes, with the limit
 * shortened to `limit_us` microseconds. The wait runs out, the kernel records it in the
 * per-device flag and returns normally: a following dwbnq_check_device_flag reports
 * DWBNQ_ERR_DEVICE_FLAG. This is how the give-up path is tested without a faulting copy. */
int dwbnq_debug_expire_wait(unsigned int limit_us, int device, void *stream);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* DWBNQ_DEBUG_H_ */
