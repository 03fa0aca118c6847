#include "common.cuh"
#include <stdarg.h>
#include <atomic>
#include "../../include/ptv3_b200.h"

namespace ptv3 {

static thread_local char g_err[512] = "";
static std::atomic<long long> g_launches{0};

void count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launches() { return g_launches.load(std::memory_order_relaxed); }

void set_error(const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int check_launch(const char* what)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: %s", what, cudaGetErrorString(e));
        return PTV3_ERR_CUDA;
    }
    return PTV3_OK;
}

}  // namespace ptv3

extern "C" const char* ptv3_last_error(void) { return ptv3::g_err; }
extern "C" int ptv3_version(void) { return 1; }
extern "C" long long ptv3_launch_count(void) { return ptv3::launches(); }
extern "C" int ptv3_status_reset(uint32_t* status, void* stream)
{
    PTV3_REQUIRE(status != nullptr, PTV3_ERR_INVALID_ARGUMENT, "ptv3_status_reset: null pointer");
    if (cudaMemsetAsync(status, 0, sizeof(uint32_t), (cudaStream_t)stream) != cudaSuccess)
        return ptv3::check_launch("ptv3_status_reset");
    return PTV3_OK;
}
