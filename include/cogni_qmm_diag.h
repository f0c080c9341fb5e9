/*
 * cogni_qmm diagnostics: A/B switches for tests and measurements.  Not part of the product ABI a
 * host runtime binds (include/cogni_qmm.h); nothing here has a counterpart in the reference.
 *
 * Every choice below leaves results VALID: it only selects among kernels and plans that the
 * automatic choice could also have taken.  The switches are process-wide and unsynchronised: set
 * them from one thread while no call of the library is in flight.
 */
#ifndef COGNI_QMM_DIAG_H
#define COGNI_QMM_DIAG_H

#ifdef __cplusplus
extern "C" {
#endif

/*
 * cogni_qmm_set_kernel_choice(choice):
 *    0        automatic: the tiled tensor-core GEMV where the shape allows it (default)
 *    1        the general row-per-warp GEMV everywhere
 *   24-26     superblocks per work item of the tiled GEMV: automatic / 1 / 2
 *   27-30     at least 1 .. 4 column ranges per row of the tiled GEMV (27 = default)
 *   48-51     prefill token-tile width: automatic / 128 / 256 / 512
 *   52-54     prefill split along K: automatic / never / wherever it is allowed
 *   55-56     prefill raw superblocks staged by TMA (default) / read directly by the dequant threads
 *   57-58     prefill 512-token tiles of Q4_K / Q5_K on CTA pairs (default) / on single CTAs
 *   59        prefill split along K: four ordered splits wherever allowed (52 returns to automatic)
 *   60-68     K slabs of the tiled GEMV (several CTAs share a row tile, partial sums meet in a
 *             workspace): 60 = off (default), 61-68 = 1 .. 8 slabs wherever a plan allows it
 * Returns COGNI_QMM_ERR_ARG for any other value.  (A library built with -DCOGNI_QMM_DIAG_TIMING
 * also accepts the timing modes 16-21 and 32-47, whose results are invalid; the shipped build
 * does not contain them.)
 */
int cogni_qmm_set_kernel_choice(int choice);

/*
 * Makes one bounded wait run out on purpose: a one-warp kernel waits on a barrier that nothing
 * ever arrives at, with a limit of `limit_us` microseconds (1 .. 100000), gives up, is counted by
 * cogni_qmm_wait_timeouts(), and returns.  Nothing faults or hangs; it exists so that the give-up
 * path and cogni_qmm_reset_wait_timeouts() can be tested.
 */
int cogni_qmm_diag_expire_wait(unsigned limit_us, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* COGNI_QMM_DIAG_H */
