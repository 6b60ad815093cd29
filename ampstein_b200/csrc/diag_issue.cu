// Issue-rate microbenchmark behind `python bench.py --workload issue`: how many cycles a scheduler
// needs per 8 decoded weights and lane for the decode GEMV's instruction mix, with the dot product
// fed (a) through two mma.sync m16n8k16 as in exl3_gemv_kernel, (b) through one tcgen05.st into
// tensor memory as in exl3_gemv_tc_kernel, (c) not at all (decoded words folded into a checksum),
// and (d) the two mma.sync alone. Measurement infrastructure, not part of the hot path: it backs the
// statement that on sm_100 a legacy mma.sync keeps its scheduler from issuing other instructions
// for most of the eight cycles the tensor pipe works on it. No counterpart in the reference.
#include "exl3_common.cuh"
#include "host_common.h"
#include <vector>

namespace amp {

constexpr int DIAG_ITERS = 1024;

__device__ __forceinline__ uint32_t diag_lo16(uint32_t r) { uint32_t d; asm("dp2a.lo.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(r), "r"(0x00000001u), "r"(0u)); return d; }
__device__ __forceinline__ uint32_t diag_hi16(uint32_t r) { uint32_t d; asm("dp2a.lo.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(r), "r"(0x00000100u), "r"(0u)); return d; }

// V: 0 decode + two mma.sync, 1 decode + tcgen05.st (8 registers), 2 decode + checksum (four lop3),
// 3 two mma.sync on undecoded words
template <int V>
__global__ void __launch_bounds__(128) diag_issue_kernel(uint32_t* out, long long* clk, uint32_t seed)
{
    __shared__ uint32_t s_tmem;
    uint32_t tmem = 0;
    const int warp = threadIdx.x >> 5;
    if (V == 1)
    {
        if (warp == 0)
        {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&s_tmem)), "r"(32u) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        tmem = s_tmem + ((uint32_t) (warp * 32) << 16);
    }
    uint32_t cur = seed * (threadIdx.x + 1) + blockIdx.x, prev = cur ^ 0x9e3779b9u, sink = 0;
    float d0[4] = {0, 0, 0, 0}, d1[4] = {0, 0, 0, 0};
    const uint32_t b0 = seed | 0x3c003c00u, b1 = b0 + 1;
    __syncthreads();
    const long long t0 = clock64();
    #pragma unroll 4
    for (int it = 0; it < DIAG_ITERS; ++it)
    {
        uint32_t a[8];
        if (V == 3)
        {
            #pragma unroll
            for (int j = 0; j < 8; ++j) a[j] = cur + j;
        }
        else
        {
            // the kernel's K = 4 decode: three funnel shifts, eight 16-bit extractions split between
            // the ALU and the FMA-heavy pipe, eight multiply-adds, eight lop3
            #pragma unroll
            for (int c = 0; c < 4; ++c)
            {
                const uint32_t r = c ? __funnelshift_r(cur, prev, 4 * c) : cur;
                const uint32_t h = (c == 1 || c == 2) ? diag_hi16(r) : (r >> 16);
                const uint32_t l = diag_lo16(r);
                a[3 - c] = cb_halves<0>(h);
                a[7 - c] = cb_halves<0>(l);
            }
        }
        if (V == 0 || V == 3)
        {
            mma_16816(d0, a[0], a[4], a[1], a[5], b0, b1);
            mma_16816(d1, a[2], a[6], a[3], a[7], b1, b0);
        }
        if (V == 1)
        {
            asm volatile("tcgen05.st.sync.aligned.16x256b.x2.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                :: "r"(tmem + (uint32_t) ((it & 1) * 16)), "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]) : "memory");
            if ((it & 7) == 7) asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
        if (V == 2)
        {
            asm volatile("lop3.b32 %0, %0, %1, %2, 0x96;" : "+r"(sink) : "r"(a[0]), "r"(a[1]));
            asm volatile("lop3.b32 %0, %0, %1, %2, 0x96;" : "+r"(sink) : "r"(a[2]), "r"(a[3]));
            asm volatile("lop3.b32 %0, %0, %1, %2, 0x96;" : "+r"(sink) : "r"(a[4]), "r"(a[5]));
            asm volatile("lop3.b32 %0, %0, %1, %2, 0x96;" : "+r"(sink) : "r"(a[6]), "r"(a[7]));
        }
        prev = cur;
        cur = cur * 1664525u + 1013904223u;
    }
    const long long t1 = clock64();
    out[blockIdx.x * blockDim.x + threadIdx.x] = __float_as_uint(d0[0] + d0[1] + d0[2] + d0[3] + d1[0] + d1[1] + d1[2] + d1[3]) + cur + sink;
    if (threadIdx.x == 0) clk[blockIdx.x] = t1 - t0;
    if (V == 1)
    {
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(s_tmem), "r"(32u) : "memory");
    }
}

}  // namespace amp

using namespace amp;

// variant 0..3 (see the kernel), warps_per_scheduler 1..8 (= CTAs of four warps per SM). Writes the
// average cycles one scheduler needs per iteration (8 weights per lane) to *cycles_per_iter.
// Synchronises; allocates and frees its own small buffers.
AMP_API int amp_diag_issue_cycles(int variant, int warps_per_scheduler, float* cycles_per_iter)
{
    AMP_REQUIRE(variant >= 0 && variant <= 3 && warps_per_scheduler >= 1 && warps_per_scheduler <= 8 && cycles_per_iter,
                "diag_issue: variant 0..3, 1..8 warps per scheduler");
    int dev = 0, sms = 0;
    if (cudaError_t e = cudaGetDevice(&dev)) return cuda_rc(e, "cudaGetDevice");
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int blocks = sms * warps_per_scheduler;
    uint32_t* out = nullptr; long long* clk = nullptr;
    if (cudaError_t e = cudaMalloc(&out, (size_t) blocks * 128 * 4)) return cuda_rc(e, "diag_issue alloc");
    if (cudaError_t e = cudaMalloc(&clk, (size_t) blocks * 8)) { cudaFree(out); return cuda_rc(e, "diag_issue alloc"); }
    for (int rep = 0; rep < 2; ++rep)
    {
        switch (variant)
        {
            case 0: diag_issue_kernel<0><<<blocks, 128>>>(out, clk, 12345u); break;
            case 1: diag_issue_kernel<1><<<blocks, 128>>>(out, clk, 12345u); break;
            case 2: diag_issue_kernel<2><<<blocks, 128>>>(out, clk, 12345u); break;
            default: diag_issue_kernel<3><<<blocks, 128>>>(out, clk, 12345u); break;
        }
        if (cudaError_t e = cudaDeviceSynchronize()) { cudaFree(out); cudaFree(clk); return cuda_rc(e, "diag_issue run"); }
    }
    std::vector<long long> h(blocks);
    cudaError_t e = cudaMemcpy(h.data(), clk, (size_t) blocks * 8, cudaMemcpyDeviceToHost);
    cudaFree(out); cudaFree(clk);
    if (e) return cuda_rc(e, "diag_issue copy");
    double avg = 0;
    for (long long v : h) avg += (double) v;
    avg /= blocks;
    *cycles_per_iter = (float) (avg / ((double) DIAG_ITERS * warps_per_scheduler));
    return 0;
}
