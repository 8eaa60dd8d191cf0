// Error text and version of the C ABI.
#include <stdarg.h>

#include "tpk_common.cuh"

namespace tpk
{
static thread_local char g_last_error[512] = "";

void set_error(const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}
}  // namespace tpk

extern "C" int tpk_version(void) { return 100; }

extern "C" const char* tpk_last_error(void) { return tpk::g_last_error; }
