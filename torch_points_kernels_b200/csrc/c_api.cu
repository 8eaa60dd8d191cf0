// Error text, version and launch counter of the C ABI.
#include <stdarg.h>

#include <atomic>

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

static std::atomic<long long> g_kernel_launches{0};

void count_launches(int k) { g_kernel_launches.fetch_add(k, std::memory_order_relaxed); }
}  // namespace tpk

extern "C" int tpk_version(void) { return 100; }

extern "C" int64_t tpk_kernel_launches(void) { return tpk::g_kernel_launches.load(std::memory_order_relaxed); }

extern "C" const char* tpk_last_error(void) { return tpk::g_last_error; }
