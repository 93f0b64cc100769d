// Status plumbing shared by every entry point of the library.
#include "common.cuh"

namespace mpsbnb {

static thread_local cudaError_t g_last_error = cudaSuccess;

int record_cuda_error(cudaError_t e) {
    g_last_error = e;
    return MPSBNB_ERR_CUDA;
}

int check_launch() {
    const cudaError_t e = cudaPeekAtLastError();
    if (e == cudaSuccess) return MPSBNB_OK;
    (void)cudaGetLastError();  // clear the non-sticky launch error so later calls start clean
    return record_cuda_error(e);
}

int sm_count() {
    static thread_local int cached_dev = -1, cached = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached = n;
        cached_dev = dev;
    }
    return cached;
}

}  // namespace mpsbnb

extern "C" const char *mpsbnb_status_string(int status) {
    switch (status) {
        case MPSBNB_OK: return "ok";
        case MPSBNB_ERR_INVALID_ARG: return "invalid argument (null pointer, bad enum or bad size)";
        case MPSBNB_ERR_UNSUPPORTED: return "shape/dtype combination not supported by this entry point";
        case MPSBNB_ERR_CUDA: return "a CUDA call failed (see mpsbnb_last_cuda_error_string)";
        case MPSBNB_ERR_WORKSPACE: return "workspace too small";
        case MPSBNB_ERR_TOO_LARGE: return "size exceeds a documented fixed limit";
        case MPSBNB_ERR_NO_DEVICE: return "no sm_100 CUDA device is current";
        default: return "unknown status";
    }
}

extern "C" int mpsbnb_last_cuda_error(void) { return (int)mpsbnb::g_last_error; }
extern "C" const char *mpsbnb_last_cuda_error_string(void) { return cudaGetErrorString(mpsbnb::g_last_error); }
extern "C" int mpsbnb_abi_version(void) { return 1; }
