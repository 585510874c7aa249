// Error state, version and device checks of the C ABI.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

static thread_local char g_err[512] = "";

int mmf_set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

extern "C" const char* mmf_last_error(void) { return g_err; }

extern "C" int mmf_abi_version(void) { return MMF_ABI_VERSION; }

extern "C" int mmf_check_device(void) {
    int dev = 0;
    MMF_CUDA(cudaGetDevice(&dev));
    int major = 0;
    MMF_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    MMF_REQUIRE(major == 10, MMF_ERR_ARCH,
                "libmmfree_b200 is built for sm_100a only; device %d has compute capability major %d", dev, major);
    return MMF_OK;
}
