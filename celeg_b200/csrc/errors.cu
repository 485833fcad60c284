// Error reporting of the kernel library: every entry point returns 0 or a negative code and
// leaves a message that celeg_last_error() returns.
#include "common.cuh"

#include <cstdarg>
#include <cstdio>

namespace celeg_b200 {

static thread_local char g_error[512] = "";

void set_error(const char* format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(g_error, sizeof(g_error), format, args);
    va_end(args);
}

int check_launch(const char* what) {
    const cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) {
        set_error("%s: %s", what, cudaGetErrorString(status));
        return -2;
    }
    return 0;
}

}  // namespace celeg_b200

CELEG_API const char* celeg_last_error() { return celeg_b200::g_error; }

CELEG_API int celeg_kernels_abi_version() { return 1; }
