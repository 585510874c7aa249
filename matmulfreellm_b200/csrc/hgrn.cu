// HGRN recurrence h_t = f_t * h_{t-1} + x_t as an HBM-bound streaming scan.
//
// Work decomposition: one CTA owns 64 channels of one sequence and one chunk of the time
// axis; eight threads per channel each scan an eighth of a 64-timestep stage and are stitched
// together through shared memory (fp32 state throughout).  [64 timesteps x 64
// channels] tiles of x and g are staged in shared memory through a 4-deep cp.async ring
// (about 70-100 KB in flight per CTA) and the outputs leave through a shared-memory tile as
// 16-byte stores, so every access to HBM is a full sector and x, g, o are each touched
// once (8 B per element for bf16 x/o and fp32 g).
//
// When B*D/64 CTAs would leave most SMs idle the time axis is split into NT chunks
// ("chunked parallel scan"): pass 1 reduces every chunk but the last to its aggregate
// (prod f, local end state), pass 2 lets each chunk fold the aggregates before it into its
// carry-in and scans.  Pass 1 re-reads x and g, so it is only used when it buys occupancy.
#include "common.cuh"

namespace {

constexpr int HG_BD = 64;      // channels per CTA
constexpr int HG_SUB = 8;      // threads per channel: each scans an eighth of a stage's timesteps
constexpr int HG_THREADS = HG_BD * HG_SUB;
constexpr int HG_TS = 64;      // timesteps per stage
constexpr int HG_STAGES = 4;  // cp.async ring depth

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

template <typename T> __device__ __forceinline__ float load_state(const void* p, int64_t i) {
    return to_f32(reinterpret_cast<const T*>(p)[i]);
}
__device__ __forceinline__ float load_state_dt(const void* p, int64_t i, int dt) {
    return dt == MMF_F32 ? load_state<float>(p, i) : dt == MMF_BF16 ? load_state<__nv_bfloat16>(p, i)
                                                                     : load_state<__half>(p, i);
}
__device__ __forceinline__ void store_state_dt(void* p, int64_t i, int dt, float v) {
    if (dt == MMF_F32) reinterpret_cast<float*>(p)[i] = v;
    else if (dt == MMF_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
}

// workspace layout (floats): h0 copy [B,D] | prod_f [B,NT,D] | h_loc [B,NT,D]
struct HgrnWs {
    float* h0c;
    float* agg_a;
    float* agg_h;
};

// gate conventions
constexpr int HG_LINEAR = 0;  // g is the forget gate itself           (fused_recurrent_hgrn)
constexpr int HG_LOG = 1;     // g is its logarithm                     (chunk_hgrn)
constexpr int HG_RAW = 2;     // x, g are the raw i/f projection outputs (HGRNBitAttention's gate math fused in):
                              //   f = round(sigmoid(g)); with a lower bound lb: f = round(lb + round(round(1-lb)*f))
                              //   x = round(silu(x_raw) * round(1-f));  every round() is to the activation dtype TX

// AGG = true : pass 1, chunks 0..NT-2 -> aggregates (no o written)
// AGG = false: pass 2 (or the only pass when NT == 1) -> o, ht
// x and g rows may be strided (ld_x, ld_g elements); o is [B,T,D] contiguous.
//
// A CTA has 512 threads for its 64 channels: thread (channel, sub) scans 8 of the 64 timesteps of a stage
// from a zero state, keeping the local states and the running gate products in registers; the eight
// sub-chunk aggregates of a channel meet in shared memory, each thread folds the ones before it (and the
// carry of the previous stage) into its carry-in and fixes its eight states up: h_t = h_local_t + prod_t * carry.
// Channel-parallel alone would leave 3-4 warps per SM, which cannot hide the latency of the scan loop.
template <typename TX, typename TG, int MODE, bool AGG>
__global__ void __launch_bounds__(HG_THREADS)
hgrn_scan_kernel(const TX* __restrict__ x, int64_t ld_x, const TG* __restrict__ g, int64_t ld_g,
                 const TX* __restrict__ lb, const void* __restrict__ h0, void* __restrict__ ht,
                 int state_dt, TX* __restrict__ o, int T, int D, int NT, int chunk_len, HgrnWs ws) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) uint8_t smem_raw[];
    constexpr int XB = HG_TS * HG_BD * sizeof(TX);  // bytes of one x stage
    constexpr int GB = HG_TS * HG_BD * sizeof(TG);
    TX* sx = reinterpret_cast<TX*>(smem_raw);
    TG* sg = reinterpret_cast<TG*>(smem_raw + HG_STAGES * XB);
    TX* so = reinterpret_cast<TX*>(smem_raw + HG_STAGES * (XB + GB));
    __shared__ float s_agg_a[HG_SUB][HG_BD], s_agg_h[HG_SUB][HG_BD];
    __shared__ float s_carry[2][HG_BD];          // carry of the previous stage, double-buffered by stage parity

    const int d0 = blockIdx.x * HG_BD;
    const int c = blockIdx.y;
    const int64_t b = blockIdx.z;
    const int tid = threadIdx.x;
    const int lc = tid & (HG_BD - 1);            // channel inside the block
    const int sub = tid / HG_BD;                 // which quarter of a stage's timesteps
    const int ch = d0 + lc;
    const bool ch_ok = ch < D;
    const int t_begin = c * chunk_len;
    const int t_end = min(T, t_begin + chunk_len);
    const int nsteps = t_end - t_begin;
    const int nstage = (nsteps + HG_TS - 1) / HG_TS;
    const TX* xb = x + (b * T + t_begin) * ld_x + d0;
    const TG* gb = g + (b * T + t_begin) * ld_g + d0;
    TX* ob = AGG ? nullptr : o + (b * T + t_begin) * (int64_t)D + d0;

    constexpr int XV = 16 / sizeof(TX), GV = 16 / sizeof(TG);   // channels per 16-byte piece
    constexpr int XP = HG_BD / XV, GP = HG_BD / GV;             // pieces per tile row

    auto issue = [&](int s) {
        if (s < nstage) {
            const int buf = s % HG_STAGES;
            const int rows = min(HG_TS, nsteps - s * HG_TS);
            for (int p = tid; p < rows * XP; p += HG_THREADS) {
                const int r = p / XP, pc = (p % XP) * XV;
                if (d0 + pc < D) cp_async16(sx + (buf * HG_TS + r) * HG_BD + pc, xb + (int64_t)(s * HG_TS + r) * ld_x + pc);
            }
            for (int p = tid; p < rows * GP; p += HG_THREADS) {
                const int r = p / GP, pc = (p % GP) * GV;
                if (d0 + pc < D) cp_async16(sg + (buf * HG_TS + r) * HG_BD + pc, gb + (int64_t)(s * HG_TS + r) * ld_g + pc);
            }
        }
        cp_async_commit();  // always commit so that group counting stays uniform
    };

#pragma unroll
    for (int s = 0; s < HG_STAGES - 1; ++s) issue(s);

    const bool has_lb = MODE == HG_RAW && lb != nullptr && ch_ok;
    float lbv = 0.0f, oml = 1.0f;
    if (has_lb) {
        lbv = to_f32(lb[ch]);
        oml = round_to<TX>(__fsub_rn(1.0f, lbv));
    }
    // carry into the first stage
    if (sub == 0) {
        float h = 0.0f;
        if (!AGG && ch_ok) {
            if (NT == 1) {
                if (h0) h = load_state_dt(h0, b * D + ch, state_dt);
            } else {
                h = ws.h0c[b * D + ch];
                for (int j = 0; j < c; ++j) {
                    const int64_t i = (b * NT + j) * (int64_t)D + ch;
                    h = fmaf(ws.agg_a[i], h, ws.agg_h[i]);
                }
            }
        }
        s_carry[0][lc] = h;
        if (AGG && c == 0 && ch_ok) ws.h0c[b * D + ch] = h0 ? load_state_dt(h0, b * D + ch, state_dt) : 0.0f;
    }
    float a_run = 1.0f;   // AGG: product of all gates of this chunk

    for (int s = 0; s < nstage; ++s) {
        cp_async_wait<HG_STAGES - 2>();
        __syncthreads();                          // stage s has landed; s_carry[s&1] and `so` are free to use
        const int buf = s % HG_STAGES;
        const int rows = min(HG_TS, nsteps - s * HG_TS);
        constexpr int SUBT = HG_TS / HG_SUB;      // timesteps per thread
        float hl[SUBT], ap[SUBT];
        {
            const TX* px = sx + (buf * HG_TS + sub * SUBT) * HG_BD + lc;
            const TG* pg = sg + (buf * HG_TS + sub * SUBT) * HG_BD + lc;
            float h = 0.0f, a = 1.0f;
#pragma unroll
            for (int j = 0; j < SUBT; ++j) {
                float xv = 0.0f, f = 1.0f;        // steps past the end of the sequence are the identity
                if (ch_ok && sub * SUBT + j < rows) {
                    xv = to_f32(px[j * HG_BD]);
                    f = to_f32(pg[j * HG_BD]);
                    if (MODE == HG_LOG) f = expf(f);
                    if (MODE == HG_RAW) {
                        f = round_to<TX>(sigmoidf_(f));
                        if (has_lb) f = round_to<TX>(__fadd_rn(lbv, round_to<TX>(__fmul_rn(oml, f))));
                        xv = round_to<TX>(silu_mul(xv, round_to<TX>(__fsub_rn(1.0f, f))));
                    }
                }
                h = fmaf(f, h, xv);
                a *= f;
                hl[j] = h;
                ap[j] = a;
            }
            s_agg_a[sub][lc] = a;
            s_agg_h[sub][lc] = h;
        }
        __syncthreads();
        // carry-in of this thread's sub-chunk: previous stage's carry folded through the sub-chunks before it
        float cin = s_carry[s & 1][lc];
#pragma unroll
        for (int q = 0; q < HG_SUB; ++q)
            if (q < sub) cin = fmaf(s_agg_a[q][lc], cin, s_agg_h[q][lc]);
        if (AGG) {
#pragma unroll
            for (int q = 0; q < HG_SUB; ++q) a_run *= s_agg_a[q][lc];
        } else {
#pragma unroll
            for (int j = 0; j < SUBT; ++j) so[(sub * SUBT + j) * HG_BD + lc] = from_f32<TX>(fmaf(ap[j], cin, hl[j]));
        }
        if (sub == HG_SUB - 1) s_carry[(s + 1) & 1][lc] = fmaf(ap[SUBT - 1], cin, hl[SUBT - 1]);
        if (!AGG) {
            __syncthreads();
            for (int p = tid; p < rows * XP; p += HG_THREADS) {
                const int r = p / XP, pc = (p % XP) * XV;
                if (d0 + pc < D)
                    *reinterpret_cast<uint4*>(ob + (int64_t)(s * HG_TS + r) * D + pc) =
                        *reinterpret_cast<const uint4*>(so + r * HG_BD + pc);
            }
        }
        issue(s + HG_STAGES - 1);
    }
    cp_async_wait<0>();
    __syncthreads();

    if (ch_ok && sub == 0) {
        const float h_end = s_carry[nstage & 1][lc];
        if (AGG) {
            const int64_t i = (b * NT + c) * (int64_t)D + ch;
            ws.agg_a[i] = a_run;
            ws.agg_h[i] = h_end;
        } else if (ht && c == NT - 1) {
            store_state_dt(ht, b * D + ch, state_dt, h_end);
        }
    }
}

// number of time chunks: split only while it at least doubles the number of busy SMs and each
// chunk keeps >= 256 timesteps
int hgrn_num_chunks(int64_t B, int64_t T, int64_t D) {
    const int64_t ctas = B * ((D + HG_BD - 1) / HG_BD);
    int nt = 1;
    while (ctas * nt < 148 && T / (nt * 2) >= 256 && nt < 64) nt *= 2;
    return nt;
}

template <typename TX, typename TG>
size_t hgrn_smem_bytes() {
    return (size_t)HG_STAGES * HG_TS * HG_BD * (sizeof(TX) + sizeof(TG)) + (size_t)HG_TS * HG_BD * sizeof(TX);
}

template <typename TX, typename TG, int MODE>
int hgrn_launch(const void* x, int64_t ld_x, const void* g, int64_t ld_g, const void* lb, const void* h0, void* ht,
                int state_dt, void* o, int64_t B, int64_t T, int64_t D, int NT, HgrnWs ws, cudaStream_t st) {
    const size_t smem = hgrn_smem_bytes<TX, TG>();
    const int chunk_len = (int)((T + NT - 1) / NT);
    const dim3 grid((unsigned)((D + HG_BD - 1) / HG_BD), (unsigned)NT, (unsigned)B);
    if (NT > 1) {
        auto k1 = hgrn_scan_kernel<TX, TG, MODE, true>;
        MMF_CUDA(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        const dim3 grid1(grid.x, (unsigned)(NT - 1), grid.z);
        MMF_CUDA(mmf_launch_pdl(k1, grid1, dim3(HG_THREADS), smem, st, (const TX*)x, ld_x, (const TG*)g, ld_g, (const TX*)lb, h0,
                                (void*)nullptr, state_dt, (TX*)nullptr, (int)T, (int)D, NT, chunk_len, ws));
        MMF_LAUNCH_CHECK("hgrn_scan_kernel<aggregate>");
    }
    auto k2 = hgrn_scan_kernel<TX, TG, MODE, false>;
    MMF_CUDA(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MMF_CUDA(mmf_launch_pdl(k2, grid, dim3(HG_THREADS), smem, st, (const TX*)x, ld_x, (const TG*)g, ld_g, (const TX*)lb, h0, ht,
                            state_dt, (TX*)o, (int)T, (int)D, NT, chunk_len, ws));
    MMF_LAUNCH_CHECK("hgrn_scan_kernel<scan>");
    return MMF_OK;
}

int hgrn_setup_ws(int64_t B, int64_t T, int64_t D, void* workspace, int64_t workspace_bytes, int& NT, HgrnWs& ws,
                  const char* who) {
    NT = hgrn_num_chunks(B, T, D);
    ws = HgrnWs{nullptr, nullptr, nullptr};
    if (NT > 1) {
        const int64_t need = mmf_hgrn_workspace_bytes(B, T, D);
        MMF_REQUIRE(workspace && workspace_bytes >= need, MMF_ERR_WORKSPACE, "%s: workspace of %lld bytes needed, %lld given",
                    who, (long long)need, (long long)workspace_bytes);
        MMF_REQUIRE(mmf_aligned(workspace, 16), MMF_ERR_ALIGN, "%s: workspace must be 16-byte aligned", who);
        ws.h0c = (float*)workspace;
        ws.agg_a = ws.h0c + B * D;
        ws.agg_h = ws.agg_a + B * NT * D;
    }
    return MMF_OK;
}

}  // namespace

extern "C" int64_t mmf_hgrn_workspace_bytes(int64_t B, int64_t T, int64_t D) {
    if (B <= 0 || T <= 0 || D <= 0) return 0;
    const int nt = hgrn_num_chunks(B, T, D);
    if (nt == 1) return 0;
    return (B * D + 2 * B * nt * D) * (int64_t)sizeof(float);
}

extern "C" int mmf_hgrn_scan(const void* x, int x_dtype, const void* g, int g_dtype, const void* h0, void* ht,
                             int state_dtype, void* o, int64_t B, int64_t T, int64_t D, int gate_is_log,
                             void* workspace, int64_t workspace_bytes, void* stream) {
    MMF_REQUIRE(x && g && o, MMF_ERR_BAD_ARG, "mmf_hgrn_scan: null pointer");
    MMF_REQUIRE(mmf_dtype_ok(x_dtype) && mmf_dtype_ok(g_dtype) && mmf_dtype_ok(state_dtype), MMF_ERR_BAD_ARG,
                "mmf_hgrn_scan: unknown dtype");
    MMF_REQUIRE(B >= 0 && T >= 0 && D > 0 && D % 8 == 0, MMF_ERR_BAD_SHAPE, "mmf_hgrn_scan: D must be a multiple of 8");
    MMF_REQUIRE(B < 65536 && T < (1ll << 31) && D < (1ll << 31), MMF_ERR_BAD_SHAPE, "mmf_hgrn_scan: size too large");
    MMF_REQUIRE(mmf_aligned(x, 16) && mmf_aligned(g, 16) && mmf_aligned(o, 16), MMF_ERR_ALIGN,
                "mmf_hgrn_scan: x, g, o must be 16-byte aligned");
    if (B == 0 || T == 0) return MMF_OK;
    int NT;
    HgrnWs ws;
    const int rc0 = hgrn_setup_ws(B, T, D, workspace, workspace_bytes, NT, ws, "mmf_hgrn_scan");
    if (rc0 != MMF_OK) return rc0;
    cudaStream_t st = (cudaStream_t)stream;
    int rc = MMF_OK;
#define HG_GO(TX, TG)                                                                                                  \
    rc = gate_is_log ? hgrn_launch<TX, TG, HG_LOG>(x, D, g, D, nullptr, h0, ht, state_dtype, o, B, T, D, NT, ws, st)     \
                     : hgrn_launch<TX, TG, HG_LINEAR>(x, D, g, D, nullptr, h0, ht, state_dtype, o, B, T, D, NT, ws, st)
    if (x_dtype == MMF_F32 && g_dtype == MMF_F32) { HG_GO(float, float); }
    else if (x_dtype == MMF_BF16 && g_dtype == MMF_BF16) { HG_GO(__nv_bfloat16, __nv_bfloat16); }
    else if (x_dtype == MMF_BF16 && g_dtype == MMF_F32) { HG_GO(__nv_bfloat16, float); }
    else if (x_dtype == MMF_F16 && g_dtype == MMF_F16) { HG_GO(__half, __half); }
    else if (x_dtype == MMF_F16 && g_dtype == MMF_F32) { HG_GO(__half, float); }
    else return mmf_set_error(MMF_ERR_BAD_ARG, "mmf_hgrn_scan: unsupported dtype pair x=%d g=%d", x_dtype, g_dtype);
#undef HG_GO
    return rc;
}

extern "C" int mmf_hgrn_gated(const void* i_raw, const void* f_raw, int64_t ld, int dtype, const void* lower_bound,
                              float* state, void* o, int64_t B, int64_t T, int64_t D, void* workspace,
                              int64_t workspace_bytes, void* stream) {
    MMF_REQUIRE(i_raw && f_raw && state && o, MMF_ERR_BAD_ARG, "mmf_hgrn_gated: null pointer");
    MMF_REQUIRE(mmf_dtype_ok(dtype), MMF_ERR_BAD_ARG, "mmf_hgrn_gated: unknown dtype %d", dtype);
    MMF_REQUIRE(B >= 0 && B < 65536 && T >= 0 && T < (1ll << 31) && D > 0 && D < (1ll << 31) && D % 8 == 0 && ld >= D,
                MMF_ERR_BAD_SHAPE, "mmf_hgrn_gated: bad sizes (D must be a multiple of 8)");
    const int es = mmf_dtype_size(dtype);
    MMF_REQUIRE(mmf_aligned(i_raw, 16) && mmf_aligned(f_raw, 16) && mmf_aligned(o, 16) && (ld * es) % 16 == 0, MMF_ERR_ALIGN,
                "mmf_hgrn_gated: rows must be 16-byte aligned");
    if (B == 0 || T == 0) return MMF_OK;
    int NT;
    HgrnWs ws;
    const int rc0 = hgrn_setup_ws(B, T, D, workspace, workspace_bytes, NT, ws, "mmf_hgrn_gated");
    if (rc0 != MMF_OK) return rc0;
    int rc = MMF_OK;
    MMF_DISPATCH(dtype, Ty, {
        rc = hgrn_launch<Ty, Ty, HG_RAW>(i_raw, ld, f_raw, ld, lower_bound, state, state, MMF_F32, o, B, T, D, NT, ws,
                                         (cudaStream_t)stream);
    });
    return rc;
}
