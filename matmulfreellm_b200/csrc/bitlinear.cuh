// Internal interface between the BitLinear dispatcher and its two kernels.
#pragma once
#include "common.cuh"

// Arguments shared by both BitLinear kernels (all device pointers; see mmf_bitlinear).
struct BitLinearArgs {
    const int8_t* q;        // [groups][M][K] activation codes
    const float* dq;        // [groups][M]    per-row dequantisation factor
    const int32_t* rowsum;  // [groups][M]    sum of the row's codes (weights are stored +1 biased)
    const uint4* packed;    // tile-major 2-bit weights
    const float* w_scale;   // [groups] mean|w|
    void* out;              // [M][ld_out]
    int32_t* acc_out;       // optional [M][N] raw accumulators
    int out_dtype;
    int64_t ld_out;
    int M, N, K;
    int groups;
    int32_t* ws;            // split-K workspace (zero on entry, zero on exit)
    int64_t ws_bytes;
};

// workspace geometry (in 32-bit words):
//   [header: MMF_WS_HEADER words, word 0 = status (0 = ok, 1 = a bounded device-side wait gave up)]
//   [counters: n_tiles * MMF_WS_MBLK] [acc: min(M,MMF_SPLITK_MAX_M) * n_tiles*128]
constexpr int MMF_WS_HEADER = 64;
constexpr int MMF_WS_MBLK = 64;
constexpr int MMF_SPLITK_MAX_M = 256;

int bitlinear_gemv_launch(const BitLinearArgs& a, cudaStream_t st, bool force_split_k);
int bitlinear_mma_launch(const BitLinearArgs& a, cudaStream_t st);
int bitlinear_mma_prefill_launch(const BitLinearArgs& a, cudaStream_t st, int variant);   // persistent kernel for many token rows
int bitlinear_mma_prefill_tile(const BitLinearArgs& a, int variant);                       // its token tile

// out = acc * (dq * w_scale), the one place the dequantising epilogue is defined
__device__ __forceinline__ float bitlinear_dequant(int32_t acc, float dq, float w_scale) {
    return __fmul_rn((float)acc, __fmul_rn(dq, w_scale));
}

__device__ __forceinline__ void store_out(void* out, int dt, int64_t i, float v) {
    if (dt == MMF_F32) reinterpret_cast<float*>(out)[i] = v;
    else if (dt == MMF_BF16) reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<__half*>(out)[i] = __float2half_rn(v);
}
