// Error text behind the C ABI: every entry point returns an int status and
// leaves a message here (per host thread) when it is non-zero.
#include <stdarg.h>

#include "common.cuh"
#include "fold_b200.h"

namespace fold {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: %s", what, cudaGetErrorString(e));
        return FOLD_ERR_LAUNCH;
    }
    return FOLD_OK;
}

}  // namespace fold

extern "C" const char* fold_last_error(void) { return fold::g_error; }

extern "C" int fold_abi_version(void) { return FOLD_B200_ABI_VERSION; }
