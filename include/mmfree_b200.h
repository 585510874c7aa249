/*
 * mmfree_b200.h — C ABI of libmmfree_b200.so: the MatMul-free LM inference hot path
 * (BitLinear, HGRN recurrence, RMSNorm / swish-gate / SwiGLU) as hand-written CUDA for
 * NVIDIA B200 (sm_100a).
 *
 * The reference project (ridgerchu/matmulfreellm) has no FFI: its "plugin surface" is the
 * Python package `mmfreelm`, whose leaves are Triton kernels and torch calls.  Each entry
 * point below replaces one such leaf; the comment above it cites the reference function
 * it stands in for (path inside the reference project : line).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the name ends in `_host`;
 *   - the caller owns all memory (inputs, outputs and workspaces); unless an entry point's
 *     comment says otherwise the library allocates nothing, frees nothing, keeps no
 *     pointer after return and never synchronises the device;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - `dtype` arguments take MMF_F32 / MMF_BF16 / MMF_F16;
 *   - return value: MMF_OK (0) or a negative MMF_ERR_* code; mmf_last_error() gives text;
 *   - kernels are launched asynchronously; launch errors are caught with
 *     cudaGetLastError() right after the launch, execution errors surface at the caller's
 *     next synchronisation.
 */
#ifndef MMFREE_B200_H
#define MMFREE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MMF_ABI_VERSION 2

/* element types of activation tensors */
#define MMF_F32 0
#define MMF_BF16 1
#define MMF_F16 2

/* status codes */
#define MMF_OK 0
#define MMF_ERR_BAD_ARG (-1)     /* null pointer, negative size, unknown dtype            */
#define MMF_ERR_BAD_SHAPE (-2)   /* size violates a divisibility / range rule             */
#define MMF_ERR_ALIGN (-3)       /* pointer or leading dimension not aligned as required   */
#define MMF_ERR_CUDA (-4)        /* a CUDA runtime call or kernel launch failed            */
#define MMF_ERR_ARCH (-5)        /* device is not compute capability 10.x                  */
#define MMF_ERR_WORKSPACE (-6)   /* workspace smaller than mmf_*_workspace_bytes() says    */
#define MMF_ERR_TIMEOUT (-7)     /* a bounded device-side wait gave up (see status word)   */

/* layout constants of the packed ternary weight format (see mmf_pack_ternary) */
#define MMF_TILE_ROWS 128 /* output rows per weight tile                               */
#define MMF_TILE_K 64     /* input columns per 16-byte packed chunk                    */

/* Text of the last error raised on the calling host thread ("" if none). */
const char* mmf_last_error(void);

/* ABI version of the loaded library (== MMF_ABI_VERSION of the header it was built from). */
int mmf_abi_version(void);

/* 0 if the current CUDA device can run this library (compute capability 10.x), else
 * MMF_ERR_ARCH / MMF_ERR_CUDA. */
int mmf_check_device(void);

/* ------------------------------------------------------------------------------------
 * Offline weight ternarisation and 2-bit packing.
 * Replaces: weight_quant(), mmfreelm/ops/fusedbitnet.py:32-46, which the reference
 * re-evaluates on the full weight in every forward (fusedbitnet.py:456).
 * ------------------------------------------------------------------------------------ */

/* Number of doubles mmf_absmean_f32 needs in `partials`. */
#define MMF_ABSMEAN_PARTIALS 1024

/* mean(|w|) over n fp32 values, accumulated in fp64 in a fixed order (deterministic), then
 * rounded once to fp32 and clamped to >= 1e-5, i.e. the reciprocal of weight_quant's
 * `scale` (fusedbitnet.py:43).  `partials`: scratch of MMF_ABSMEAN_PARTIALS doubles.
 * `out_mean`: one float. */
int mmf_absmean_f32(const float* w, int64_t n, double* partials, float* out_mean, void* stream);

/* Bytes of the packed form of an [N,K] weight: ceil(N/128) * (K/64) * 128 * 16. */
int64_t mmf_packed_bytes(int64_t N, int64_t K);

/* codes = clamp(rint(w / mean), -1, 1) (rint = round-half-even, as torch.round in
 * fusedbitnet.py:45) stored as 2-bit fields (code+1).  K must be a multiple of 64.
 * Layout: tiles of 128 output rows; for tile t, chunk c (64 input columns) and row r the
 * 16 bytes at ((t*(K/64) + c)*128 + r)*16 hold that row's 64 codes: 32-bit word q covers
 * columns c*64 + q*16 .. +15, and column j of those sits in bits [2f, 2f+2) with
 * f = j/4 + 4*(j%4), so that (word >> 2*i) & 0x03030303 yields columns 4i..4i+3 as bytes.
 * Rows >= N of the last tile are filled with code 0. */
int mmf_pack_ternary(const float* w, int64_t N, int64_t K, const float* mean, void* packed,
                     void* stream);

/* Inverse of the layout above: int8 codes [N,K] in {-1,0,1} (test / debugging aid). */
int mmf_unpack_ternary(const void* packed, int64_t N, int64_t K, int8_t* codes, void* stream);

/* ------------------------------------------------------------------------------------
 * BitLinear prologue: RMSNorm + per-token int8 absmax quantisation.
 * Replaces: _layer_norm_fwd_quant_kernel, mmfreelm/ops/fusedbitnet.py:63-131 (RMS branch)
 * and activation_quant(), fusedbitnet.py:15-29.  Emits integer codes and one fp32
 * dequantisation factor per row instead of the reference's dequantised floats.
 * ------------------------------------------------------------------------------------ */

/* For each of M rows of x [M, ld_x] (first K columns used):
 *   rstd = 1/sqrt(mean(x^2) + eps)   (sum of squares in fp64, rest in fp32, no fma)
 *   y    = (x * rstd) * norm_w       (norm_w may be NULL = all ones; fp32 [K])
 *   a    = max(max|y|, 1e-5);  s = 127 / a
 *   q    = clamp(rint(y * s), -128, 127)              -> q [M,K] int8
 *   dq   = a / 127                                    -> dq [M] fp32
 *   rowsum = sum_k q                                  -> rowsum [M] int32
 * `use_norm` = 0 skips the RMSNorm (y = x), giving plain activation_quant.
 * K must be a multiple of 16 and <= 16384. */
int mmf_act_quant(const void* x, int dtype, int64_t ld_x, const float* norm_w, int use_norm,
                  float eps, int8_t* q, float* dq, int32_t* rowsum, int64_t M, int64_t K,
                  void* stream);

/* ------------------------------------------------------------------------------------
 * BitLinear contraction: int8 activation codes x 2-bit ternary weight codes -> int32,
 * then the dequantising epilogue.
 * Replaces: F.linear(y_dequant, weight_quant(W)) in LayerNormLinearQuantFn.forward,
 * mmfreelm/ops/fusedbitnet.py:456-458 (cuBLAS fp16/bf16 GEMM in the reference).
 * ------------------------------------------------------------------------------------ */

/* Which kernel mmf_bitlinear runs. AUTO: GEMV below MMF_MMA_MIN_M rows, tcgen05 above. */
#define MMF_KERNEL_AUTO 0
#define MMF_KERNEL_GEMV 1 /* CUDA-core dp4a, weight-streaming, any M (slow for large M) */
#define MMF_KERNEL_MMA 2  /* tcgen05 kind::i8 tensor-core tiles, weights unpacked into TMEM */
#define MMF_MMA_MIN_M 3

/* Bytes of int32 workspace mmf_bitlinear may need for split-K partial sums (a multiple of
 * 256; includes a 256-byte header whose first word is a status flag — 0, or 1 if a bounded
 * device-side wait gave up — and the tile counters).  The workspace must be ZERO before its first use; the
 * kernels leave it zero again, so it can be reused by the next call on the same stream.
 * Concurrent calls on different streams need separate workspaces. */
int64_t mmf_bitlinear_workspace_bytes(int64_t M, int64_t N, int64_t K);

/* out[m, n] = acc[m, n] * (dq[g][m] * w_scale[g]),  acc = sum_k q[g][m,k] * code[n,k],
 * for n in [0,N).  The N output rows may form `groups` equal slabs of N/groups rows
 * (N/groups a multiple of 128), slab g using its own activation codes q + g*M*K,
 * dq + g*M, rowsum + g*M and weight scale w_scale[g] — this is how the i/f/g projections,
 * which share an input row but not a norm weight, run as one launch.  groups = 1 is a
 * plain BitLinear.
 *   out: [M, ld_out] of `out_dtype`, or, if acc_out != NULL, the raw int32 accumulators are
 *   ALSO written to acc_out [M,N] (test hook for the bit-exactness checks).
 *   w_scale: device fp32 [groups] = mean|w| from mmf_absmean_f32.
 *   workspace: mmf_bitlinear_workspace_bytes() bytes, zeroed once by the caller. */
int mmf_bitlinear(const int8_t* q, const float* dq, const int32_t* rowsum, const void* packed,
                  const float* w_scale, int groups, void* out, int out_dtype, int64_t ld_out,
                  int32_t* acc_out, int64_t M, int64_t N, int64_t K, void* workspace,
                  int64_t workspace_bytes, int kernel, void* stream);

/* BitLinear for a few token rows WITHOUT caller-provided scratch and without any allocation.
 * (No counterpart in the reference: it exists for hosts that must not allocate.)
 *
 * Some programs that embed this library cannot call cudaMalloc at the point where they run a decode
 * step: an inference server whose device memory is one arena planned at start-up and owned by another
 * runtime, a latency-critical loop where an allocation (which may synchronise the device) is forbidden,
 * or a process running under a memory budget that leaves nothing to hand out.  mmf_bitlinear needs a
 * zeroed split-K workspace from such a caller; this entry point instead keeps that workspace inside the
 * library image, as a fixed array of MMF_STATIC_SCRATCH_BYTES in device global memory.  Every GPU that
 * loads the library holds those bytes until the process exits.
 *
 * Same arithmetic and arguments as mmf_bitlinear with kernel = MMF_KERNEL_GEMV (the CUDA-core
 * weight-streaming kernel meant for M <= 4; larger M works but is slow); there is no acc_out.  The call
 * fails with MMF_ERR_WORKSPACE, launching nothing, when mmf_bitlinear_workspace_bytes(M, N, K) exceeds
 * MMF_STATIC_SCRATCH_BYTES (e.g. M = 8 with N = 32000) — use mmf_bitlinear with your own workspace then.
 *
 * It calls no cudaMalloc / cudaFree and no allocating library routine.  The first call on each device
 * looks up the array's device address (cudaGetSymbolAddress, with that device current) and remembers it;
 * make that first call during start-up, before any stream capture.  Each call first clears the part of
 * the array it will accumulate into (cudaMemsetAsync on `stream`), because the array keeps whatever the
 * previous call left.  All calls on a device share the one array: two calls that overlap on the GPU (for
 * example on different streams) race on it — serialise them or use mmf_bitlinear with separate workspaces. */
#define MMF_STATIC_SCRATCH_BYTES (1 << 20)
int mmf_bitlinear_gemv_static(const int8_t* q, const float* dq, const int32_t* rowsum, const void* packed,
                              const float* w_scale, int groups, void* out, int out_dtype, int64_t ld_out,
                              int64_t M, int64_t N, int64_t K, void* stream);

/* Measurement aid (no counterpart in the reference): the int8 tensor-pipe peak of the current GPU in
 * TOP/s (2*M*N*K ops per MMA), measured with a bare tcgen05.mma kind::i8 loop of `iters` 128 x n_tokens x 32
 * instructions per SM, one CTA per SM, timed with CUDA events.  Unlike the other entry points this one
 * runs on the default stream and SYNCHRONISES; status_dev is one device int of scratch, tops_host a host
 * double. */
int mmf_int8_mma_peak(int n_tokens, int iters, int* status_dev, double* tops_host);

/* Measurement aid (no counterpart in the reference): the synchronisation costs that bound a chain of dependent decode
 * kernels on the current GPU, in microseconds.  barrier_us: one grid-wide barrier among one resident CTA per SM (each
 * CTA adds to a global counter with release semantics and polls it with acquire loads; cooperative launch, every wait
 * bounded).  signal_us: one hand-over of a flag between two CTAs (release store -> the other CTA's acquire poll sees
 * it).  chain_pdl_us / chain_plain_us: time per kernel of a chain of 200 dependent one-CTA-per-SM kernels replayed from
 * a CUDA graph, launched with / without the programmatic-dependent-launch attribute.  scratch_dev: 256 device uints.
 * Runs on streams of its own and SYNCHRONISES. */
int mmf_sync_probe(int iters, unsigned* scratch_dev, double* barrier_us_host, double* signal_us_host,
                   double* chain_pdl_us_host, double* chain_plain_us_host);

/* ------------------------------------------------------------------------------------
 * HGRN recurrence  h_t = f_t * h_{t-1} + x_t  (element-wise, fp32 state).
 * Replaces: fused_recurrent_hgrn (linear-domain gate), mmfreelm/ops/hgrn/recurrent_fuse.py:32-68,
 * :176-185, and chunk_hgrn (log-domain gate, f = exp(g)), mmfreelm/ops/hgrn/chunk.py:49-116,
 * :287-296.  Oracle: naive_recurrent_hgrn, mmfreelm/ops/hgrn/naive.py:8-31.
 * ------------------------------------------------------------------------------------ */

/* Scratch bytes for the chunk carries of mmf_hgrn_scan (0 when T is handled in one pass). */
int64_t mmf_hgrn_workspace_bytes(int64_t B, int64_t T, int64_t D);

/* x, g, o: [B, T, D] contiguous (the reference's [B,H,T,D] with B*H folded into B).
 * x/o have `x_dtype`, g has `g_dtype`.  h0 (may be NULL = zeros) and ht (may be NULL = not
 * wanted) are [B, D] of `state_dtype`.  gate_is_log != 0 selects chunk_hgrn's convention.
 * D must be a multiple of 8.  workspace: mmf_hgrn_workspace_bytes() bytes (no zeroing
 * needed). */
int mmf_hgrn_scan(const void* x, int x_dtype, const void* g, int g_dtype, const void* h0,
                  void* ht, int state_dtype, void* o, int64_t B, int64_t T, int64_t D,
                  int gate_is_log, void* workspace, int64_t workspace_bytes, void* stream);

/* Gated recurrence straight from the raw i/f projection outputs, i.e. the element-wise glue of
 * HGRNBitAttention.forward fused into the scan: mmfreelm/layers/hgrn_bit.py:113-125
 *   f = sigmoid(f_raw);  if lower_bound: f = lb + (1 - lb) * f;  x = silu(i_raw) * (1 - f);
 *   h_t = f_t * h_{t-1} + x_t;  o_t = h_t
 * with every intermediate rounded to `dtype` where the reference materialises a tensor.
 * i_raw, f_raw: [B, T, *] rows `ld` elements apart (two column slabs of one projection output);
 * lower_bound: [D] of `dtype` or NULL; state: fp32 [B, D], read as h_0 and overwritten with h_T
 * (decode-step update in place when T = 1); o: [B, T, D] contiguous.  D % 8 == 0.
 * workspace: mmf_hgrn_workspace_bytes(B, T, D) bytes. */
int mmf_hgrn_gated(const void* i_raw, const void* f_raw, int64_t ld, int dtype,
                   const void* lower_bound, float* state, void* o, int64_t B, int64_t T, int64_t D,
                   void* workspace, int64_t workspace_bytes, void* stream);

/* mmf_hgrn_gated with a padding mask: mask is uint8 [B, T] (device), 1 = token, 0 = padding; at a masked position
 * the input x_t is replaced by zero (the forget gate still applies), mask == NULL means no padding.
 * Replaces: `i = i.mul_(attention_mask.unsqueeze(-1))`, mmfreelm/layers/hgrn_bit.py:119-120, fused into the scan. */
int mmf_hgrn_gated_masked(const void* i_raw, const void* f_raw, int64_t ld, int dtype,
                          const void* lower_bound, const uint8_t* mask, float* state, void* o, int64_t B,
                          int64_t T, int64_t D, void* workspace, int64_t workspace_bytes, void* stream);

/* Error reporting of the scan kernels (no counterpart in the reference): the kernels wait for their TMA
 * stages with a bounded spin; *failed_host becomes 1 if any launch of this process ever gave up on such a
 * wait (its outputs are then undefined).  Synchronises with the device. */
int mmf_hgrn_status(int* failed_host);

/* ------------------------------------------------------------------------------------
 * Fused producers of BitLinear inputs: each emits the int8 codes (+ dq, rowsum, laid out
 * [groups][M][D] / [groups][M]) that mmf_bitlinear consumes, so no activation tensor is
 * written between two contractions.  D % 16 == 0, D <= 8192, rows and norm weights 16-byte aligned.
 * ------------------------------------------------------------------------------------ */

/* s = x [+ residual]; residual_out = s (optional); y = rmsnorm(s; norm_w, eps_norm) rounded to
 * `dtype` (optionally stored to y_out); then for each of `groups` (0, 1 or 3) BitLinear norm
 * weights nw_g: codes of rmsnorm(y; nw_g, eps_bl) as in mmf_act_quant.
 * round_sum_first = 1 rounds s to `dtype` before the statistics (the reference's separate
 * `residual + hidden_states` tensor add, modeling_hgrn_bit.py:109, followed by the next block's
 * attn_norm, :98); 0 normalises the fp32 sum (the fused add of mlp_norm, :107, i.e.
 * _layer_norm_fwd_1pass_kernel, modules/layernorm.py:136-153).
 * Replaces: HGRNBitBlock.forward's attn_norm / mlp_norm (modeling_hgrn_bit.py:98,107) followed by
 * the RMSNorm+quant prologue of the BitLinears they feed (ops/fusedbitnet.py:63-131). */
int mmf_prenorm_quant(const void* x, int64_t ld_x, const void* residual, int64_t ld_res, int dtype,
                      int round_sum_first, const float* norm_w, float eps_norm, void* residual_out,
                      void* y_out, int groups, const float* nw0, const float* nw1, const float* nw2,
                      float eps_bl, int8_t* q, float* dq, int32_t* rowsum, int64_t M, int64_t D,
                      void* stream);

/* y = (rmsnorm(g; gnorm_w, eps_g)) * o * sigmoid(o) rounded to `dtype`, then the BitLinear
 * prologue with norm weight nw.  Replaces: FusedRMSNormSwishGate (modules/fused_norm_gate.py:68-131)
 * + o_proj's prologue, layers/hgrn_bit.py:139-140. */
int mmf_gatenorm_quant(const void* g, int64_t ld_g, const void* o, int64_t ld_o, int dtype,
                       const float* gnorm_w, float eps_g, const float* nw, float eps_bl, int8_t* q,
                       float* dq, int32_t* rowsum, int64_t M, int64_t D, void* stream);

/* Single-token (decode) step of the token mixer in one kernel: for each of M sequences, the gate math
 * and state update of mmf_hgrn_gated with T = 1 (state fp32 [M, D], updated in place) followed by
 * mmf_gatenorm_quant on the same row.  ifg: [M, ld] rows holding the i | f | g projections as three
 * consecutive D-wide slabs (ld >= 3*D).  lower_bound, gnorm_w and nw are read before the kernel synchronises with
 * the launches preceding it on the stream: they must be complete when those launches are enqueued (model constants).
 * Replaces: mmfreelm/layers/hgrn_bit.py:113-140 for a one-token forward. */
int mmf_decode_mix(const void* ifg, int64_t ld, int dtype, const void* lower_bound, float* state,
                   const float* gnorm_w, float eps_g, const float* nw, float eps_bl, int8_t* q, float* dq,
                   int32_t* rowsum, int64_t M, int64_t D, void* stream);

/* mmf_decode_mix with a padding mask: mask is uint8 [M] (device), 1 = token, 0 = padding position; a masked row's
 * input to the recurrence is zero (its forget gate still decays the state), mask == NULL means no padding.  The mask is
 * read AFTER the kernel has synchronised with the preceding launches (it may be written by them).
 * Replaces: `i = i.mul_(attention_mask.unsqueeze(-1))`, mmfreelm/layers/hgrn_bit.py:119-120, for a one-token forward
 * (the attention_mask[:, -1:] of a cached generation step, mmfreelm/models/hgrn_bit/modeling_hgrn_bit.py:335-338). */
int mmf_decode_mix_masked(const void* ifg, int64_t ld, int dtype, const void* lower_bound, const uint8_t* mask,
                          float* state, const float* gnorm_w, float eps_g, const float* nw, float eps_bl, int8_t* q,
                          float* dq, int32_t* rowsum, int64_t M, int64_t D, void* stream);

/* z = silu(gate) * up rounded to `dtype`, then the BitLinear prologue with norm weight nw.
 * gate/up: the two halves of gate_proj's output, rows `ld` elements apart.
 * Replaces: swiglu (modules/activations.py:115-119) + down_proj's prologue, modeling_hgrn_bit.py:57-58. */
int mmf_swiglu_quant(const void* gate, const void* up, int64_t ld, int dtype, const float* nw,
                     float eps_bl, int8_t* q, float* dq, int32_t* rowsum, int64_t M, int64_t D,
                     void* stream);

/* ------------------------------------------------------------------------------------
 * Row-wise norms and activations.
 * ------------------------------------------------------------------------------------ */

/* y = rmsnorm(x [+ residual]) * w.  Replaces: _layer_norm_fwd_1pass_kernel (RMS branch),
 * mmfreelm/modules/layernorm.py:104-165; oracle rms_norm_ref, layernorm.py:73-87.
 * residual / residual_out may be NULL.  residual_out (dtype res_dtype) receives x+residual.
 * w may be NULL (= ones).  x, y: [M, D] of `dtype`; w fp32 [D]. */
int mmf_rmsnorm(const void* x, int dtype, const void* residual, int res_dtype, const float* w,
                float eps, void* y, void* residual_out, int64_t M, int64_t D, void* stream);

/* y = (rmsnorm(x) * w) * o * sigmoid(o).  Replaces: the gated kernel
 * mmfreelm/modules/fused_norm_gate.py:68-131 (formula at :123-128). */
int mmf_rmsnorm_swishgate(const void* x, const void* o, int dtype, const float* w, float eps,
                          void* y, int64_t M, int64_t D, void* stream);

/* out = x * y / (1 + exp(-x)) computed in fp32.  Replaces: swiglu_fwd jiterator kernel,
 * mmfreelm/modules/activations.py:115-119.  Rows may be strided (ld_* in elements) so the
 * two halves of gate_proj's output can be passed without a copy. */
int mmf_swiglu(const void* x, int64_t ld_x, const void* y, int64_t ld_y, void* out,
               int64_t ld_out, int dtype, int64_t M, int64_t D, void* stream);

/* Greedy sampling helper: idx[m] = first index of the maximum of logits[m, 0:V].
 * Replaces: torch.argmax in a greedy decoding loop around HGRNBitForCausalLM.forward,
 * mmfreelm/models/hgrn_bit/modeling_hgrn_bit.py:356-409. */
int mmf_argmax_rows(const void* logits, int dtype, int64_t ld, int64_t M, int64_t V,
                    int64_t* idx, void* stream);

/* Nucleus sampling helper: idx[m] = one token drawn from softmax(logits[m, 0:V] / temperature) restricted to the
 * smallest set of most probable tokens whose mass reaches top_p (top_p >= 1: no restriction; tokens tied with the
 * least probable kept one are all kept), using the caller's uniform number uniforms[m] in [0, 1): the first kept
 * token, in index order, at which the running kept mass exceeds uniforms[m] * (kept mass).  Deterministic.
 * Replaces: the sampling step of model.generate(..., do_sample=True, top_p=0.4, temperature=0.6) in the reference's
 * generate.py:11 (transformers' TemperatureLogitsWarper + TopPLogitsWarper + multinomial). */
int mmf_sample_top_p(const void* logits, int dtype, int64_t ld, float temperature, float top_p,
                     const float* uniforms, int64_t* idx, int64_t M, int64_t V, void* stream);

/* out[m, :] = table[ids[m], :].  Replaces: nn.Embedding lookup, modeling_hgrn_bit.py:211-213. */
int mmf_embedding(const void* table, int dtype, int64_t V, int64_t D, const int64_t* ids,
                  void* out, int64_t M, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MMFREE_B200_H */
