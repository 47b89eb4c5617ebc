// Last refusal text of this thread, for the Python side to raise.
#include "common.cuh"
#include <stdarg.h>
#include <stdlib.h>

static thread_local char g_last_error[512] = "";

void braid_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}

extern "C" const char* braid_last_error(void) { return g_last_error; }

int braid_pdl_enabled(void) {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("BRAIDINFER_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on;
}

// Build stamp: lets the loader check that the library it opened is the one it built.
extern "C" int braid_abi_version(void) { return 1; }
