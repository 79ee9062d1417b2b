// Library-wide pieces of the C ABI: error strings, version, device check.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "sp24_common.cuh"

namespace sp24 {

int check_device() {
    // The answer is cached per device ordinal; the cache is written once per device and only ever
    // with the same value, so concurrent first calls are harmless.
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return SP24_ERR_CUDA;
    if (dev >= 0 && dev < 64 && cached[dev]) return cached[dev] == 1 ? SP24_OK : SP24_ERR_DEVICE;
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return SP24_ERR_CUDA;
    const int ok = major == 10;
    if (dev >= 0 && dev < 64) cached[dev] = ok ? 1 : 2;
    return ok ? SP24_OK : SP24_ERR_DEVICE;
}

// Number of SMs of the current device (cached per device ordinal; 148 if the query fails).
int sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

int launch_status() {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return SP24_OK;
    if (getenv("SP24_DEBUG")) fprintf(stderr, "sparse24_b200: CUDA error %d: %s\n", (int)e, cudaGetErrorString(e));
    return SP24_ERR_CUDA;
}

}  // namespace sp24

extern "C" const char *sp24_strerror(int code) {
    switch (code) {
        case SP24_OK: return "ok";
        case SP24_ERR_SHAPE: return "unsupported shape: a dimension is not a positive multiple of the required block size";
        case SP24_ERR_STRIDE: return "unsupported leading dimension: too small or not a multiple of 16 bytes";
        case SP24_ERR_DTYPE: return "unsupported element type combination";
        case SP24_ERR_ALIGN: return "pointer is not 16-byte aligned";
        case SP24_ERR_ARG: return "invalid argument: null pointer, contradictory flags or value out of range";
        case SP24_ERR_CUDA: return "the CUDA runtime reported an error";
        case SP24_ERR_DEVICE: return "the current device is not a compute capability 10.x GPU";
        case SP24_ERR_TOO_LARGE: return "size exceeds a fixed capacity of this entry point";
        default: return "unknown sparse24_b200 error code";
    }
}

extern "C" int sp24_abi_version(void) { return 2; }

// Peer memory for exchanges that run on the copy engines: a buffer exported by its owner (cudaIpcGetMemHandle, or a
// framework's equivalent) is mapped into this process; copies from the returned address are ordinary device-to-device
// copies on a stream of the current device.
extern "C" int sp24_ipc_open(const void *handle, int handle_bytes, void **ptr) {
    if (!handle || !ptr || handle_bytes != (int)sizeof(cudaIpcMemHandle_t)) return SP24_ERR_ARG;
    if (int rc = sp24::check_device()) return rc;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    *ptr = nullptr;
    if (cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        sp24::launch_status();     // clears (and with SP24_DEBUG prints) the runtime's error
        return SP24_ERR_CUDA;
    }
    return SP24_OK;
}

extern "C" int sp24_ipc_close(void *ptr) {
    if (!ptr) return SP24_ERR_ARG;
    return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? SP24_OK : SP24_ERR_CUDA;
}
