// Host-side access to cuTensorMapEncodeTiled without linking libcuda: the entry point is fetched from the
// driver through the runtime once per process.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

typedef CUresult (*MmfEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                     const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline MmfEncodeTiledFn mmf_encode_tiled() {
    static MmfEncodeTiledFn fn = []() -> MmfEncodeTiledFn {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<MmfEncodeTiledFn>(ptr);
    }();
    return fn;
}
