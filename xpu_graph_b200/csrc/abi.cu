// Library identity and error reporting for the xg_sm100 C ABI.
#include "common.cuh"

namespace xg {

char* last_error_buf() {
    static thread_local char buf[512] = {0};
    return buf;
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buf(), 512, fmt, ap);
    va_end(ap);
    return code;
}

}  // namespace xg

extern "C" int xg_version(void) { return 1000; }

extern "C" const char* xg_last_error(void) { return xg::last_error_buf(); }

extern "C" int xg_device_arch_ok(int device) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) {
        cudaGetLastError();
        xg::fail(XG_ERR_DEVICE, "xg_device_arch_ok: cannot query device %d", device);
        return 0;
    }
    return major == 10 ? 1 : 0;
}
