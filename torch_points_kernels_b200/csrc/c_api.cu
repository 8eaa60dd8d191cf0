// Error text, version, launch counter, device status word and test hook of the C ABI.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

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

// The one environment variable the library reads: TPK_B200_TEST, a comma-separated list of
// `name` or `name=value` tokens that steer a call onto a kernel the size heuristics would
// not pick (the index-order scans behind the grids, the global-memory fallbacks of the
// row-resident gather kernels, another FPS cluster shape), so that tests can compare every
// kernel family on the same inputs.  Read on every call; unset in normal use.
static const char* find_token(const char* name, size_t* value_len)
{
    const char* env = getenv("TPK_B200_TEST");
    if (env == nullptr) return nullptr;
    const size_t len = strlen(name);
    for (const char* p = env; *p;)
    {
        const char* end = strchr(p, ',');
        const size_t tok = end ? static_cast<size_t>(end - p) : strlen(p);
        if (tok >= len && strncmp(p, name, len) == 0 && (tok == len || p[len] == '='))
        {
            if (value_len) *value_len = tok == len ? 0 : tok - len - 1;
            return tok == len ? p + len : p + len + 1;
        }
        if (!end) break;
        p = end + 1;
    }
    return nullptr;
}

bool test_path(const char* name) { return find_token(name, nullptr) != nullptr; }

bool test_value(const char* name, char* out, size_t cap)
{
    size_t n = 0;
    const char* v = find_token(name, &n);
    if (v == nullptr || cap == 0) return false;
    if (n >= cap) n = cap - 1;
    memcpy(out, v, n);
    out[n] = 0;
    return true;
}

// Every translation unit with kernels that can raise the sticky status keeps its own device
// word (no relocatable device code is needed that way) and registers a reader here.
static StatusReader g_status_readers[16];
static int g_num_status_readers = 0;

StatusRegistrar::StatusRegistrar(StatusReader r)
{
    if (g_num_status_readers < 16) g_status_readers[g_num_status_readers++] = r;
}
}  // namespace tpk

extern "C" int tpk_version(void) { return 100; }

extern "C" int64_t tpk_kernel_launches(void) { return tpk::g_kernel_launches.load(std::memory_order_relaxed); }

extern "C" const char* tpk_last_error(void) { return tpk::g_last_error; }

extern "C" int tpk_device_status(int* status_out, int reset)
{
    int all = 0;
    for (int i = 0; i < tpk::g_num_status_readers; ++i)
    {
        int v = 0;
        const cudaError_t err = tpk::g_status_readers[i](&v, reset);
        if (err != cudaSuccess)
        {
            tpk::set_error("device status: %s", cudaGetErrorString(err));
            return TPK_ERR_CUDA;
        }
        all |= v;
    }
    if (status_out) *status_out = all;
    return TPK_OK;
}
