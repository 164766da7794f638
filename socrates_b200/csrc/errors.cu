// Last-error text of the library (host side only).
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

void sb_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

extern "C" const char* sb_last_error() { return g_error; }

// Programmatic dependent launch: on unless SOCRATES_PDL=0; a model may switch it off for its own steps
// (sb_set_dependent_launch), which the environment variable overrides only towards "off".
static int g_pdl_wanted = 1;

namespace sb {
bool pdl_enabled() {
    static const bool allowed = [] {
        const char* e = getenv("SOCRATES_PDL");
        return !(e && e[0] == '0');
    }();
    return allowed && g_pdl_wanted != 0;
}
}  // namespace sb

extern "C" int sb_set_dependent_launch(int on) {
    g_pdl_wanted = on ? 1 : 0;
    return 0;
}

extern "C" int sb_abi_version() { return 1; }
