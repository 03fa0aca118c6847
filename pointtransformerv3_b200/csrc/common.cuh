// Shared helpers of the sm_100a kernel library: status codes, the thread-local
// error string behind ptv3_last_error(), launch checking and small device
// utilities.  The library never allocates device memory (one documented entry
// point uses a static device array instead); callers pass outputs and
// workspaces.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/ptv3_b200.h"

namespace ptv3 {

void set_error(const char* fmt, ...);
int check_launch(const char* what);
// Adds to the process-wide count of kernels this library has launched
// (read through ptv3_launch_count()).
void count_launches(int n);

#define PTV3_REQUIRE(cond, code, ...)            \
    do {                                         \
        if (!(cond)) {                           \
            ::ptv3::set_error(__VA_ARGS__);      \
            return (code);                       \
        }                                        \
    } while (0)

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Carves a caller-provided workspace into 256-byte aligned pieces.
struct Carver {
    char* base;
    size_t off;
    explicit Carver(void* p) : base(static_cast<char*>(p)), off(0) {}
    template <typename T>
    T* take(size_t count) {
        T* p = reinterpret_cast<T*>(base + off);
        off += align_up(count * sizeof(T), 256);
        return p;
    }
};

static inline int ceil_div(int64_t a, int64_t b) { return static_cast<int>((a + b - 1) / b); }

// ---- programmatic dependent launch -------------------------------------------------------------
// A forward is a chain of a few hundred kernels on one stream, many of them a few microseconds
// long.  A kernel launched with launch_dependent() may be scheduled while the kernel before it in
// the stream still runs; it must call pdl_wait() before it touches anything that kernel wrote (all
// such kernels here call it first thing), and pdl_launch_next() tells the scheduler that the
// kernel after it may be brought up.  The launch latency and the start-up of a kernel then overlap
// the tail of its predecessor.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_next() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_dependent(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                           cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
#endif

}  // namespace ptv3
