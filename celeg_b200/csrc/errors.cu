// Error reporting of the kernel library: every entry point returns 0 or a negative code and
// leaves a message that celeg_last_error() returns.
#include "common.cuh"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>

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

static int g_chaining = 7;

// bit 0: small-batch products, bit 1: norms, bit 2: every other chained kernel (default: all)
bool chaining_enabled(int kernel_class) { return (g_chaining >> kernel_class) & 1; }

}  // namespace celeg_b200

// A bit per class of kernels (see chaining_enabled): set = launched with programmatic stream serialization.
// One setting for the whole process (for measurements); every kernel launched that way waits with
// griddepcontrol.wait before its first access to memory that an earlier kernel writes, so both settings
// compute the same.
CELEG_API void celeg_set_chained_launch(int mask) { celeg_b200::g_chaining = mask & 7; }

CELEG_API const char* celeg_last_error() { return celeg_b200::g_error; }

CELEG_API int celeg_kernels_abi_version() { return 1; }
