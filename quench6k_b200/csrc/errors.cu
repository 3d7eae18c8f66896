// Error text of the exported launchers (one message per host thread).
#include <cstdlib>

#include "common.cuh"

static thread_local char g_msg[512] = "";

int q6k_fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_msg, sizeof g_msg, fmt, ap);
    va_end(ap);
    return 1;
}

int q6k_check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return 0;
    return q6k_fail("%s: %s", what, cudaGetErrorString(e));
}

int q6k_pdl_mode() {
    static const int mode = [] {
        const char* v = getenv("Q6K_PDL");
        if (!v || !v[0]) return 2;
        return v[0] == '0' ? 0 : v[0] == '1' ? 1 : 2;
    }();
    return mode;
}

Q6K_API const char* q6k_last_error() { return g_msg; }
Q6K_API int q6k_abi_version() { return 1; }
