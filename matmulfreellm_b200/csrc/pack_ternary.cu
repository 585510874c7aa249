// Offline absmean ternarisation of fp32 latent weights and 2-bit packing into the
// tile-major layout the BitLinear kernels stream (layout described in mmfree_b200.h).
#include "common.cuh"

namespace {

// stage 1: MMF_ABSMEAN_PARTIALS blocks, each sums |w| over one contiguous slice in fp64
__global__ void __launch_bounds__(256)
absmean_partial_kernel(const float* __restrict__ w, int64_t n, int64_t slice, double* __restrict__ partials) {
    __shared__ double red[33];
    const int64_t lo = blockIdx.x * slice;
    int64_t hi = lo + slice;
    if (hi > n) hi = n;
    double s = 0.0;
    for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) s += (double)fabsf(w[i]);
    s = block_sum(s, red);
    if (threadIdx.x == 0) partials[blockIdx.x] = s;
}

// stage 2: one block folds the partials in a fixed order, rounds once to fp32, clamps
__global__ void __launch_bounds__(MMF_ABSMEAN_PARTIALS)
absmean_final_kernel(const double* __restrict__ partials, int64_t n, float* __restrict__ out_mean) {
    __shared__ double red[33];
    const double s = block_sum(partials[threadIdx.x], red);
    if (threadIdx.x == 0) out_mean[0] = fmaxf((float)(s / (double)n), 1e-5f);
}

__device__ __forceinline__ uint32_t ternary_field(float w, float scale) {
    float r = rintf(__fmul_rn(w, scale));     // round half to even
    r = fminf(fmaxf(r, -1.0f), 1.0f);
    return (uint32_t)((int)r + 1);            // {-1,0,1} -> {0,1,2}
}

// one thread = one 16-byte chunk (64 codes of one row)
__global__ void __launch_bounds__(128)
pack_kernel(const float* __restrict__ w, int64_t N, int64_t K, const float* __restrict__ mean,
            uint4* __restrict__ packed) {
    const int64_t KC = K / MMF_TILE_K;
    const int64_t tile = blockIdx.x / KC, c = blockIdx.x % KC;
    const int r = threadIdx.x;
    const int64_t n = tile * MMF_TILE_ROWS + r;
    const float scale = __fdiv_rn(1.0f, mean[0]);
    uint32_t words[4];
    if (n < N) {
        const float4* src = reinterpret_cast<const float4*>(w + n * K + c * MMF_TILE_K);
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
            uint32_t word = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {  // i = j/4: which group of 4 columns inside the word
                const float4 v = src[qd * 4 + i];
                // column j = 4*i + b goes to field f = i + 4*b
                word |= ternary_field(v.x, scale) << (2 * (i + 0));
                word |= ternary_field(v.y, scale) << (2 * (i + 4));
                word |= ternary_field(v.z, scale) << (2 * (i + 8));
                word |= ternary_field(v.w, scale) << (2 * (i + 12));
            }
            words[qd] = word;
        }
    } else {
        words[0] = words[1] = words[2] = words[3] = 0x55555555u;  // code 0 everywhere
    }
    packed[(tile * KC + c) * MMF_TILE_ROWS + r] = make_uint4(words[0], words[1], words[2], words[3]);
}

__global__ void __launch_bounds__(256)
unpack_kernel(const uint32_t* __restrict__ packed, int64_t N, int64_t K, int8_t* __restrict__ codes) {
    const int64_t KC = K / MMF_TILE_K;
    const int64_t groups = N * (K / 16);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < groups; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / (K / 16);
        const int64_t k16 = i % (K / 16);
        const int64_t c = k16 / 4;
        const int qd = (int)(k16 % 4);
        const int64_t tile = n / MMF_TILE_ROWS;
        const int r = (int)(n % MMF_TILE_ROWS);
        const uint32_t word = packed[((tile * KC + c) * MMF_TILE_ROWS + r) * 4 + qd];
        uint32_t out[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const uint32_t b = (word >> (2 * g)) & 0x03030303u;   // columns 4g..4g+3, biased by +1
            out[g] = __vsub4(b, 0x01010101u);
        }
        *reinterpret_cast<uint4*>(codes + n * K + k16 * 16) = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

}  // namespace

extern "C" int64_t mmf_packed_bytes(int64_t N, int64_t K) {
    if (N <= 0 || K <= 0 || K % MMF_TILE_K != 0) return 0;
    const int64_t tiles = (N + MMF_TILE_ROWS - 1) / MMF_TILE_ROWS;
    return tiles * (K / MMF_TILE_K) * MMF_TILE_ROWS * 16;
}

extern "C" int mmf_absmean_f32(const float* w, int64_t n, double* partials, float* out_mean, void* stream) {
    MMF_REQUIRE(w && partials && out_mean, MMF_ERR_BAD_ARG, "mmf_absmean_f32: null pointer");
    MMF_REQUIRE(n > 0, MMF_ERR_BAD_SHAPE, "mmf_absmean_f32: n must be positive");
    MMF_REQUIRE(mmf_aligned(partials, 8), MMF_ERR_ALIGN, "mmf_absmean_f32: partials must be 8-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t slice = (n + MMF_ABSMEAN_PARTIALS - 1) / MMF_ABSMEAN_PARTIALS;
    absmean_partial_kernel<<<MMF_ABSMEAN_PARTIALS, 256, 0, st>>>(w, n, slice, partials);
    MMF_LAUNCH_CHECK("absmean_partial_kernel");
    absmean_final_kernel<<<1, MMF_ABSMEAN_PARTIALS, 0, st>>>(partials, n, out_mean);
    MMF_LAUNCH_CHECK("absmean_final_kernel");
    return MMF_OK;
}

extern "C" int mmf_pack_ternary(const float* w, int64_t N, int64_t K, const float* mean, void* packed, void* stream) {
    MMF_REQUIRE(w && mean && packed, MMF_ERR_BAD_ARG, "mmf_pack_ternary: null pointer");
    MMF_REQUIRE(N > 0 && K > 0 && K % MMF_TILE_K == 0, MMF_ERR_BAD_SHAPE,
                "mmf_pack_ternary: K must be a positive multiple of %d (N=%lld, K=%lld)", MMF_TILE_K, (long long)N,
                (long long)K);
    MMF_REQUIRE(mmf_aligned(w, 16) && mmf_aligned(packed, 16), MMF_ERR_ALIGN,
                "mmf_pack_ternary: w and packed must be 16-byte aligned");
    const int64_t tiles = (N + MMF_TILE_ROWS - 1) / MMF_TILE_ROWS;
    const int64_t blocks = tiles * (K / MMF_TILE_K);
    MMF_REQUIRE(blocks < (1ll << 31), MMF_ERR_BAD_SHAPE, "mmf_pack_ternary: weight too large for one launch");
    pack_kernel<<<(unsigned)blocks, MMF_TILE_ROWS, 0, (cudaStream_t)stream>>>(w, N, K, mean, (uint4*)packed);
    MMF_LAUNCH_CHECK("pack_kernel");
    return MMF_OK;
}

extern "C" int mmf_unpack_ternary(const void* packed, int64_t N, int64_t K, int8_t* codes, void* stream) {
    MMF_REQUIRE(packed && codes, MMF_ERR_BAD_ARG, "mmf_unpack_ternary: null pointer");
    MMF_REQUIRE(N > 0 && K > 0 && K % MMF_TILE_K == 0, MMF_ERR_BAD_SHAPE, "mmf_unpack_ternary: bad shape");
    MMF_REQUIRE(mmf_aligned(packed, 16) && mmf_aligned(codes, 16), MMF_ERR_ALIGN, "mmf_unpack_ternary: alignment");
    const int64_t groups = N * (K / 16);
    const unsigned grid = (unsigned)((groups + 255) / 256 < 148 * 32 ? (groups + 255) / 256 : 148 * 32);
    unpack_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint32_t*)packed, N, K, codes);
    MMF_LAUNCH_CHECK("unpack_kernel");
    return MMF_OK;
}
