// Error reporting and device queries shared by the C ABI entry points.

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace leankv {

namespace {
thread_local char g_last_cuda_error[256] = "";
constexpr int kMaxDevices = 64;
int g_sm_count[kMaxDevices] = {0};
}  // namespace

int note_cuda_error(cudaError_t e, const char* what) {
    std::snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s: %s (%s)", what,
                  cudaGetErrorName(e), cudaGetErrorString(e));
    return LEANKV_ECUDA;
}

int pdl_mode() {
    static int state = -1;
    if (state < 0) {
        const char* e = std::getenv("LEANKV_PDL");
        state = (e != nullptr && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 2;
    }
    return state;
}
bool pdl_enabled() { return pdl_mode() != 0; }

int sm_count() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    int n = g_sm_count[dev];
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;   // B200; also the value used when planning without a device present
        g_sm_count[dev] = n;
    }
    return n;
}

}  // namespace leankv

extern "C" const char* leankv_strerror(int code) {
    switch (code) {
        case LEANKV_OK: return "success";
        case LEANKV_EINVAL: return "invalid argument (shape, size or null pointer)";
        case LEANKV_EALIGN: return "pointer, size or segment boundary not suitably aligned";
        case LEANKV_EWORKSPACE: return "workspace missing or too small";
        case LEANKV_ECUDA: return "CUDA runtime error (see leankv_last_cuda_error)";
        case LEANKV_EUNSUPPORTED: return "configuration not implemented by the sm_100a kernels";
        case LEANKV_ELIMIT: return "size exceeds a compiled-in maximum";
        default: return "unknown leankv error code";
    }
}

extern "C" int leankv_abi_version(void) { return 2; }

extern "C" const char* leankv_last_cuda_error(void) { return leankv::g_last_cuda_error; }

// ---- device memory shared between the ranks of one node (CUDA IPC) ----

extern "C" int leankv_ipc_alloc(size_t bytes, void** ptr, unsigned char handle[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    if (!ptr || !handle || bytes == 0) return LEANKV_EINVAL;
    void* d = nullptr;
    LEANKV_CUDA_TRY(cudaMalloc(&d, bytes));
    cudaError_t e = cudaMemset(d, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, d);
    if (e != cudaSuccess) {
        cudaFree(d);
        LEANKV_CUDA_TRY(e);
    }
    std::memcpy(handle, &h, 64);
    *ptr = d;
    return LEANKV_OK;
}

extern "C" int leankv_ipc_open(const unsigned char handle[64], void** ptr) {
    if (!ptr || !handle) return LEANKV_EINVAL;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, 64);
    void* d = nullptr;
    LEANKV_CUDA_TRY(cudaIpcOpenMemHandle(&d, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr = d;
    return LEANKV_OK;
}

extern "C" int leankv_ipc_close(void* ptr) {
    if (!ptr) return LEANKV_EINVAL;
    LEANKV_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
    return LEANKV_OK;
}

extern "C" int leankv_ipc_free(void* ptr) {
    if (!ptr) return LEANKV_EINVAL;
    LEANKV_CUDA_TRY(cudaFree(ptr));
    return LEANKV_OK;
}
