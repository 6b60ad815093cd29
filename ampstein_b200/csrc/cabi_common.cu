// Library-wide pieces of the C-ABI: version, last-error text, cached kernel attributes.
#include "host_common.h"
#include <map>
#include <mutex>
#include <utility>

namespace amp {

static thread_local char t_error[512] = "";

void set_error(const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
}

cudaError_t ensure_smem_impl(const void* kernel, int bytes, int dev)
{
    static std::map<std::pair<const void*, int>, int> seen;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    int& have = seen[std::make_pair(kernel, dev)];
    if (have >= bytes) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) have = bytes;
    return e;
}

}  // namespace amp

AMP_API int amp_b200_version(void) { return 1; }

// Text of the last error reported on the calling thread ("" when none)
AMP_API const char* amp_b200_last_error(void) { return amp::t_error; }
