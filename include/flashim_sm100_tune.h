/* Schedule overrides of libflashim_sm100.so for tests and measurements. Not part of the product ABI: nothing here is
 * needed to use the library, and a caller that never touches these gets the automatic choices. The settings are
 * process-wide and not synchronised: set them from the thread that launches.
 *
 * No counterpart in the FlashIM reference (its kernels take their tile sizes from Triton autotune configs). */
#ifndef FLASHIM_SM100_TUNE_H_
#define FLASHIM_SM100_TUNE_H_

#ifdef __cplusplus
extern "C" {
#endif

/* Overrides for the following conv launches of this process (all 0 = automatic): `block_n` forces the output-channel
 * tile (64 / 128 / 256); `max_ctas` caps the persistent grid, so that a small problem makes every CTA walk many tiles;
 * `flags` selects between schedules that all produce the same bits:
 *    16  keeps the last partial round of tiles at full width;
 *    32  lets the epilogue poll for its accumulator without sleeping between polls;
 *    64  disables CTA pairs (clusters of two CTAs on one cta_group::2 instruction stream; the default for INT8 with
 *        256-wide tiles and for large spatial block-scaled convs with 128-wide tiles);
 *   128  enables pairs for block-scaled 256-wide tiles too;
 *   256  reloads the weight scales for every tile instead of keeping the first K iterations resident in tensor memory;
 *   512  makes the four warps of an epilogue group of a 1x1 conv share one output panel and one store (as the spatial
 *        convs do) instead of one per warp;
 *  1024  sends every call through the general epilogue instead of the ones whose switches are fixed at compile time;
 *  2048  streams the weights of a layer through the stage ring even where they are kept in shared memory by default;
 *  4096  keeps them resident for every tile width where they fit (by default only 64-wide tiles do);
 * 16384  runs 128-wide block-scaled tiles as CTA pairs whatever the size of the layer.
 * A library built with -DFIM_PROBE_BUILD=1 (never shipped) also honours bits 1, 2, 4, 8 (skip activation loads / weight
 * loads / stores / scale copies), which make results invalid, and 8192 (the MMA warp of CTA 0 prints its cycle counts).
 * `max_ctas` and flag 32 also apply to fim_mxfp8_gelu_mlp_residual; in a probe build its bits are 1 (no residual loads),
 * 2 (the output warps only drain the accumulator) and 4 (no GELU / requantisation arithmetic), results invalid, and 8192
 * (two of its hidden-block warps print their cycle counts per block). */
void fim_conv_tune(int block_n, int max_ctas, int flags);

/* Depthwise launches: `variant` selects the thread layout (0 = automatic; 1: four columns per lane, four warps, three
 * CTAs per SM; 2: five warps, two CTAs; 3: two columns per lane, eight warps, two CTAs; 4: as 1 with four CTAs per SM, which
 * leaves 128 registers per thread and a four-chunk ring). A probe build also honours, in `probe_flags`,
 * 1: skip the FMAs, 2: skip the epilogue, 4: skip the loads and the waits for them (results invalid). */
void fim_dw_tune(int variant, int probe_flags);

#ifdef __cplusplus
}
#endif
#endif /* FLASHIM_SM100_TUNE_H_ */
