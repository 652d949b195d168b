// Error reporting shared by every C-ABI entry point: integer return codes plus a
// thread-local message (no exceptions cross the ABI).
#include <cstdio>
#include <string>

#include "internal.h"

namespace uep {
namespace {
thread_local std::string g_last_error;
}
void set_error(const std::string& msg) { g_last_error = msg; }
int fail(int code, const std::string& msg) {
    g_last_error = msg;
    return code;
}
int fail_cuda(cudaError_t e, const char* what) {
    g_last_error = std::string("CUDA error ") + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ") in " + what;
    return UEP_ERR_CUDA;
}

// SM count of the current device (asked once per device; 0 if the device cannot be queried).
int device_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess) cached[dev] = n;
    }
    return cached[dev];
}
}  // namespace uep

extern "C" {
const char* uep_last_error(void) { return uep::g_last_error.c_str(); }
const char* uep_version(void) { return "uep_b200 0.1 (sm_100a)"; }
}
