/*
 * mmfree_b200_experiments.h — configuration overrides of the tensor-core BitLinear kernels, for kernel experiments.
 *
 * NOT part of the product ABI: libmmfree_b200.so does not export mmf_tuning and keeps no mutable global state.  The
 * entry point below exists only in libmmfree_b200_experiments.so (the same sources built with -DMMF_EXPERIMENTS), which
 * the configuration-sweep tests load to check that every configuration the kernels can be tuned into gives the same
 * integers.  No counterpart in the reference.
 */
#ifndef MMFREE_B200_EXPERIMENTS_H
#define MMFREE_B200_EXPERIMENTS_H

#ifdef __cplusplus
extern "C" {
#endif

/* Overrides the automatic choice of the tensor-core kernel's configuration for all later mmf_bitlinear calls of this
 * process (value 0 = automatic again). */
#define MMF_TUNE_KSPLIT 0     /* K split / cluster size: 1, 2, 4 or 8                          */
#define MMF_TUNE_TOKEN_TILE 1 /* token rows per tile: 16..128 (multiple of 16) or 256           */
#define MMF_TUNE_DEEP_RING 2  /* 1 = prefer the deep-ring (no split) variant, 2 = never use it  */
#define MMF_TUNE_WEIGHT_TILES 3 /* weight tiles per CTA for large M: 1 or 2                       */
#define MMF_TUNE_B_STAGES 4   /* activation-tile ring depth (128 K per stage)                  */
#define MMF_TUNE_A_STAGES 5   /* unpacked-weight stages held in tensor memory (even)           */
#define MMF_TUNE_W_STAGES 6   /* packed-weight ring depth (even)                               */
#define MMF_TUNE_PERSISTENT 7 /* persistent large-M kernel: 1 = whenever M > 128, 2 = never, 10+v = its compiled shape v (1..4) whenever M > 128 */
#define MMF_TUNE_PROBE_COMMITS 8 /* mmf_int8_mma_peak: tcgen05.commit instructions issued per 4 MMAs */
#define MMF_TUNE_ACCUMULATORS 9 /* accumulators consecutive MMAs rotate through at few token columns: 1, 2 or 4 */
int mmf_tuning(int knob, int value);

#ifdef __cplusplus
}
#endif
#endif /* MMFREE_B200_EXPERIMENTS_H */
