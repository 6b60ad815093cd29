// Host side of the trellis-decode GEMV: argument checks, split / stage selection, cluster launch.
// C-ABI entry points amp_exl3_gemv and amp_exl3_gemm (the launcher the reference's exl3_gemm,
// vendor/exl3/exllamav3_ext/quant/exl3_gemm.cu:114-349, maps onto).
#include "exl3_gemv_kernel.cuh"
#include "host_common.h"
#include <mutex>

namespace amp {

__device__ int g_gemv_status;     // non-zero after a bounded wait inside the kernel ran out

struct DevInfo { int sms = 0; int smem_optin = 0; bool ok = false; };

static DevInfo& dev_info(int dev)
{
    static DevInfo info[64];
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    DevInfo& d = info[dev & 63];
    if (!d.ok)
    {
        cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        d.ok = true;
    }
    return d;
}

static gemv_fn gemv_kernel_for(int K, int cb, int MB)
{
    switch (K)
    {
        case 1: return gemv_kernel_k1(cb, MB);
        case 2: return gemv_kernel_k2(cb, MB);
        case 3: return gemv_kernel_k3(cb, MB);
        case 4: return gemv_kernel_k4(cb, MB);
        case 5: return gemv_kernel_k5(cb, MB);
        case 6: return gemv_kernel_k6(cb, MB);
        case 7: return gemv_kernel_k7(cb, MB);
        case 8: return gemv_kernel_k8(cb, MB);
    }
    return nullptr;
}

// k-split (= cluster size along y). CTAs spread round-robin over the SMs; an SM's time is the
// rows it decodes divided by its issue efficiency, which is poor with a single resident CTA
// (8 warps). Pick the split whose busiest SM finishes first.
static int choose_split(int k, int n, int sms, int ctas_per_sm)
{
    const int nb = n / 128, B2 = k / 128;
    int best = 1;
    double best_cost = 1e30;
    for (int S = 1; S <= 8; ++S)
    {
        if (S > B2) break;
        const long ctas = (long) nb * S;
        const long per_sm = (ctas + sms - 1) / sms;                   // CTAs on the busiest SM
        const int rows = ((B2 + S - 1) / S) * 128;
        const double eff = (per_sm >= 2 && ctas_per_sm >= 2) ? 1.0 : 0.7;
        const double cost = (double) per_sm * (rows + 256.0) / eff;
        if (cost < best_cost - 1e-9) { best_cost = cost; best = S; }
    }
    return best;
}

int launch_gemv(const void* x, const void* trellis, void* c, const void* suh, const void* svh,
                int m, int k, int n, int K, int cb, int c_fp32, int force_split, int force_stages,
                cudaStream_t stream)
{
    AMP_REQUIRE(x && trellis && c && suh && svh, "exl3_gemv: null pointer (suh and svh are required)");
    AMP_REQUIRE(K >= 1 && K <= 8, "exl3_gemv: unsupported EXL3 bitrate %d (integer 1..8)", K);
    AMP_REQUIRE(cb >= 0 && cb <= 2, "exl3_gemv: codebook index %d out of range", cb);
    AMP_REQUIRE(m >= 1 && m <= 16, "exl3_gemv: m must be 1..16 (got %d)", m);
    AMP_REQUIRE(k > 0 && n > 0 && k % 128 == 0 && n % 128 == 0, "exl3_gemv: k and n must be multiples of 128");
    AMP_REQUIRE(((uintptr_t) trellis & 15) == 0, "exl3_gemv: trellis must be 16-byte aligned");
    AMP_REQUIRE(((uintptr_t) x & 7) == 0 && ((uintptr_t) suh & 7) == 0 && ((uintptr_t) svh & 7) == 0,
                "exl3_gemv: x, suh, svh must be 8-byte aligned");
    AMP_REQUIRE(((uintptr_t) c & (c_fp32 ? 15 : 7)) == 0, "exl3_gemv: output misaligned");
    AMP_REQUIRE(n / 128 <= 0x7fffffff, "exl3_gemv: n too large");

    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev)) return cuda_rc(e, "cudaGetDevice");
    const DevInfo& D = dev_info(dev);

    const int MB = m <= 8 ? 1 : 2;
    gemv_fn fn = gemv_kernel_for(K, cb, MB);
    if (!fn) return fail(AMP_E_UNSUPPORTED, "exl3_gemv: no kernel for K=%d cb=%d", K, cb);

    // ring depth: two stages per warp cover the refill latency; fall back to one if that is all
    // that fits. CTAs per SM follow from shared memory (registers allow two for m <= 8).
    int stages = force_stages > 0 ? force_stages : 2;
    while (stages > 1 && gemv_smem_layout(K, m, stages).total > D.smem_optin) --stages;
    AMP_REQUIRE(stages >= 1 && stages <= GEMV_MAX_STAGES, "exl3_gemv: stages out of range");
    const GemvSmem L = gemv_smem_layout(K, m, stages);
    AMP_REQUIRE(L.total <= D.smem_optin, "exl3_gemv: shared memory layout does not fit (%d bytes)", L.total);
    const int smem_per_sm = D.smem_optin + 1024;                       // opt-in limit excludes 1 KB per CTA
    int ctas_per_sm = smem_per_sm / (L.total + 1024);
    if (ctas_per_sm > (MB == 1 ? 2 : 1)) ctas_per_sm = (MB == 1 ? 2 : 1);
    if (ctas_per_sm < 1) ctas_per_sm = 1;

    int S = force_split > 0 ? force_split : choose_split(k, n, D.sms, ctas_per_sm);
    AMP_REQUIRE(S >= 1 && S <= 8, "exl3_gemv: split out of range");

    if (cudaError_t e = ensure_smem(fn, L.total, dev)) return cuda_rc(e, "exl3_gemv smem attribute");

    GemvParams P;
    P.x = (const __half*) x; P.trellis = (const uint16_t*) trellis;
    P.suh = (const __half*) suh; P.svh = (const __half*) svh; P.c = c;
    P.m = m; P.k = k; P.n = n; P.c_fp32 = c_fp32; P.stages = stages;
    {
        // address of the status word, looked up once per device
        static int* status_ptr[64] = {};
        int*& sp = status_ptr[dev & 63];
        if (!sp)
            if (cudaError_t e = cudaGetSymbolAddress((void**) &sp, g_gemv_status)) return cuda_rc(e, "status symbol");
        P.status = sp;
    }

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n / 128, S, 1);
    cfg.blockDim = dim3(GEMV_THREADS, 1, 1);
    cfg.dynamicSmemBytes = L.total;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = S;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cuda_rc(cudaLaunchKernelEx(&cfg, fn, P), "exl3_gemv launch");
}

}  // namespace amp

using namespace amp;

AMP_API int amp_exl3_gemv(const void* x, const void* trellis, void* c, const void* suh, const void* svh,
                             int m, int k, int n, int K, int cb, int c_fp32, cudaStream_t stream)
{
    return launch_gemv(x, trellis, c, suh, svh, m, k, n, K, cb, c_fp32, 0, 0, stream);
}

// tuning / test hook: fixed k-split and ring depth
AMP_API int amp_exl3_gemv_cfg(const void* x, const void* trellis, void* c, const void* suh, const void* svh,
                                 int m, int k, int n, int K, int cb, int c_fp32, int split, int stages,
                                 cudaStream_t stream)
{
    return launch_gemv(x, trellis, c, suh, svh, m, k, n, K, cb, c_fp32, split, stages, stream);
}

// Reads and clears the GEMV status word of the current device (synchronises the device).
AMP_API int amp_exl3_gemv_status(int* out)
{
    int v = 0, zero = 0;
    if (cudaError_t e = cudaMemcpyFromSymbol(&v, g_gemv_status, sizeof(int))) return cuda_rc(e, "status read");
    if (cudaError_t e = cudaMemcpyToSymbol(g_gemv_status, &zero, sizeof(int))) return cuda_rc(e, "status clear");
    if (out) *out = v;
    return 0;
}

// C = had(A*suh) @ W_hat -> had(.)*svh for any m. A_had (scratch of A's size in the reference's
// signature) is accepted for drop-in compatibility and not used: the input transform lives in
// each CTA's prologue. Rows are processed in slabs of 16 by the GEMV kernel.
AMP_API int amp_exl3_gemm(const void* A, const void* trellis, void* C, const void* suh, void* A_had,
                          const void* svh, int m, int k, int n, int K, int cb, int c_fp32,
                          cudaStream_t stream)
{
    (void) A_had;
    AMP_REQUIRE(m >= 0, "exl3_gemm: negative m");
    for (int r = 0; r < m; r += 16)
    {
        const int rows = m - r < 16 ? m - r : 16;
        const char* a = (const char*) A + (size_t) r * k * 2;
        char* c = (char*) C + (size_t) r * n * (c_fp32 ? 4 : 2);
        if (int rc = launch_gemv(a, trellis, c, suh, svh, rows, k, n, K, cb, c_fp32, 0, 0, stream)) return rc;
    }
    return 0;
}
