// Error channel and library identity of the kernel library.
#include "common.cuh"

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

namespace qi {

static thread_local char g_error[1024] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return 1;
}

bool pdl_enabled() {
    static int state = -1;
    if (state < 0) {
        const char* v = getenv("QUANTINFER_B200_PDL");
        state = (v && strcmp(v, "0") == 0) ? 0 : 1;
    }
    return state == 1;
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail("%s: launch failed: %s", what, cudaGetErrorString(e));
    return 0;
}

}  // namespace qi

extern "C" const char* qi_last_error() { return qi::g_error; }

// Bumped whenever an entry point's signature changes; the Python side checks it.
extern "C" int qi_abi_version() { return 6; }
