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

#include <stdint.h>

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
#define MMF_TUNE_PERSISTENT 7 /* persistent large-M kernel: 1 = whenever M > 128, 2 = never, 10+v = its compiled shape v (1..12) whenever M > 128 */
#define MMF_TUNE_PROBE_COMMITS 8 /* mmf_int8_mma_peak: tcgen05.commit instructions issued per 4 MMAs */
#define MMF_TUNE_ACCUMULATORS 9 /* accumulators consecutive MMAs rotate through at few token columns: 1, 2 or 4 */
#define MMF_TUNE_PROBE_ISSUERS 11 /* mmf_int8_mma_peak: 2 = two threads issue the MMAs, each into its own accumulator (<= 128 token columns); 3 = pairs of CTAs (cta_group::2), 256-row MMAs */
#define MMF_TUNE_PREFILL_SKIP 12 /* persistent large-M kernel, timing only (results are wrong): bit 0 = no activation loads, bit 1 = no weight expansion, bit 2 = no output stores */
#define MMF_TUNE_ASYNC_REDUCE 10 /* split-K partial sums by st.async + the owner's mbarrier: 1 = on, 2 = off, 0 = library default */
int mmf_tuning(int knob, int value);

/* Timeline trace of mmf_prenorm_quant launches: buffer_dev is a device buffer of at least 8 + 8 * 1000 int64 ([0] = launch
 * counter, then one record of 8 global-timer stamps per launch, taken by thread 0 of CTA 0: start, weights staged, grid
 * dependency resolved, row loaded, first row sum done, second norm done, codes written, end); NULL switches it off. */
int mmf_row_trace(long long* buffer_dev);

/* Slab-major copy of a packed weight for mmf_bitlinear_decode (experiment; no counterpart in the reference).  The tile-major layout of mmf_pack_ternary keeps a 16-row slab as K/64 pieces of 256 bytes that lie
 * 2 KB apart; the decode kernel fetches whole slabs with one bulk copy each, so it reads a second copy in which slab
 * s (16 rows) of tile t occupies the (K/64)*256 contiguous bytes at ((t*8 + s) * (K/64)) * 256: chunk c at + c*256,
 * row r of the slab at + r*16, the 16 bytes themselves unchanged.  `slabs`: mmf_packed_bytes(N, K) bytes. */
int mmf_repack_slabs(const void* packed, int64_t N, int64_t K, void* slabs, void* stream);

/* 1 if mmf_bitlinear_decode accepts M token rows with K input features (M <= MMF_STREAM_MAX_M and the codes of at
 * least 8 rows fit in shared memory beside one slab of weights: K <= 16384 or so), else 0. */
#define MMF_STREAM_MAX_M 64
int mmf_bitlinear_decode_fits(int64_t M, int64_t K);

/* The contraction of mmf_bitlinear for a decode step (M <= MMF_STREAM_MAX_M token rows): same arithmetic, same
 * arguments and outputs, but the weights come from the slab-major copy (mmf_repack_slabs) and no workspace is needed.
 * One persistent CTA per SM keeps the activation codes resident in shared memory, streams its slabs of weights by
 * bulk TMA ahead of the grid dependency (programmatic dependent launch) and contracts them with mma.sync m16n8k32
 * (s8 x s8 -> s32).  `status` (may be NULL): one device int that is set to 1 if a bounded device-side wait gave up.
 * Replaces: F.linear(y_dequant, weight_quant(W)), mmfreelm/ops/fusedbitnet.py:456-458, for single-token forwards
 * (the cached generation step, mmfreelm/models/hgrn_bit/modeling_hgrn_bit.py:335-338). */
int mmf_bitlinear_decode(const int8_t* q, const float* dq, const int32_t* rowsum, const void* packed_slabs,
                         const float* w_scale, int groups, void* out, int out_dtype, int64_t ld_out,
                         int32_t* acc_out, int64_t M, int64_t N, int64_t K, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MMFREE_B200_EXPERIMENTS_H */
