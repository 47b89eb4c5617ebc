// Last refusal text of this thread, for the Python side to raise.
#include "common.cuh"
#include <stdarg.h>

static thread_local char g_last_error[512] = "";

void braid_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}

extern "C" const char* braid_last_error(void) { return g_last_error; }

// Build stamp: lets the loader check that the library it opened is the one it built.
extern "C" int braid_abi_version(void) { return 1; }
