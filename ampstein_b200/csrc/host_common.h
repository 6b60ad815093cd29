// Host-side helpers of the C-ABI launch layer: return-code convention and error text.
//
// Return codes follow the reference's launcher convention (src/torch/amp_torch.cpp:238-256):
//   0        launched
//   negative unsupported configuration / bad argument (text via amp_b200_last_error())
//   positive a cudaError_t
#pragma once
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdio>

namespace amp {

void set_error(const char* fmt, ...);

inline int fail(int code, const char* fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    set_error("%s", buf);
    return code;
}

inline int cuda_rc(cudaError_t e, const char* what)
{
    if (e == cudaSuccess) return 0;
    set_error("%s: %s", what, cudaGetErrorString(e));
    return (int) e;
}

// Raise a kernel's dynamic shared-memory limit; remembered per (kernel, device) so that
// repeated launches (and launches during stream capture) make no runtime call.
cudaError_t ensure_smem_impl(const void* kernel, int bytes, int dev);

template <typename Kern>
inline cudaError_t ensure_smem(Kern kernel, int bytes, int dev)
{
    return ensure_smem_impl((const void*) kernel, bytes, dev);
}

constexpr int AMP_E_ARG = -1;          // bad pointer / size / alignment
constexpr int AMP_E_UNSUPPORTED = -2;  // configuration the kernels do not cover

}  // namespace amp

#define AMP_API extern "C" __attribute__((visibility("default")))

#define AMP_REQUIRE(cond, ...) do { if (!(cond)) return amp::fail(amp::AMP_E_ARG, __VA_ARGS__); } while (0)
