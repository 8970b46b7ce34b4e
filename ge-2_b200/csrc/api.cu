// Library-level entry points of the C ABI: version, status strings, device check.
#include "common.cuh"

namespace ge2 {
thread_local int g_last_cuda_error = 0;
}

extern "C" const char* ge2_version(void) { return "ge2_b200 0.1 (sm_100a)"; }

extern "C" int ge2_last_cuda_error(void) { return ge2::g_last_cuda_error; }

extern "C" const char* ge2_status_string(int status) {
    switch (status) {
        case GE2_OK: return "ok";
        case GE2_ERR_INVALID_ARGUMENT: return "invalid argument";
        case GE2_ERR_CUDA: return "CUDA runtime error";
        case GE2_ERR_WORKSPACE: return "workspace missing, too small or misaligned";
        case GE2_ERR_UNSUPPORTED: return "unsupported shape or option";
        case GE2_ERR_NO_DEVICE: return "no sm_100 device";
        default: return "unknown status";
    }
}

extern "C" int ge2_check_device(int device) {
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || device < 0 || device >= count) {
        ge2::g_last_cuda_error = (int)e;
        return GE2_ERR_NO_DEVICE;
    }
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    if (e != cudaSuccess) return ge2::cuda_fail(e);
    return major == 10 ? GE2_OK : GE2_ERR_NO_DEVICE;
}
