// Host-side runtime shared by the entry points: per-thread error text, launch checks,
// device properties and the device status word of the bounded waits.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "runtime.h"

namespace vtp {

static thread_local char t_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
    return code;
}

int check_launch(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return VTP_OK;
    set_error("%s: %s", what, cudaGetErrorString(e));
    return (int)e;
}

static const int kMaxDevices = 64;

int sm_count() {
    static int cached[kMaxDevices];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

bool pdl_enabled() {
    static int cached = -1;
    if (cached < 0) cached = getenv("VTP_PDL") ? 1 : 0;
    return cached == 1;
}

__device__ int g_status_word = 0;

int* device_status_ptr() {
    static int* cached[kMaxDevices];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (!cached[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        cached[dev] = static_cast<int*>(p);
    }
    return cached[dev];
}

}  // namespace vtp

extern "C" int vtp_version(void) { return 1000; }

extern "C" const char* vtp_last_error_string(void) { return vtp::t_error; }

extern "C" int vtp_device_status(int* value, int reset) {
    if (!value) return vtp::fail(VTP_ERR_NULL, "device status: null pointer");
    int* p = vtp::device_status_ptr();
    if (!p) return vtp::fail(VTP_ERR_DRIVER, "device status: no current CUDA device");
    cudaError_t e = cudaMemcpy(value, p, sizeof(int), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && reset) e = cudaMemset(p, 0, sizeof(int));
    if (e != cudaSuccess) {
        vtp::set_error("device status: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return VTP_OK;
}
