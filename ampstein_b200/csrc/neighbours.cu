// Stand-alone forms of the element-wise kernels that sit between the linears of the decode step:
// residual add + RMSNorm, gated activation, greedy pick + state advance. The library's product for
// these is the FUSED form (the prologue / epilogue instances of the decode GEMV); the kernels here
// exist so that the fused forms can be tested and timed against the same arithmetic as separate
// launches inside one CUDA graph (the reference keeps its own kernels for them:
// src/torch/amp_kernels.cu:235-251, 279-360, 823-901). Each takes part in programmatic dependent
// launch like the GEMV kernels do.
#include "exl3_common.cuh"
#include "exl3_gemv_host.h"
#include "host_common.h"
#include "../../include/ampstein_b200.h"

namespace amp {

// y = fp16(x + r); n = fp16(y * rsqrt(mean(y^2) + eps)) * w (fp16 multiply). One CTA per row. The norm
// weight does not depend on the producer: it is loaded before the wait for it, and the sum y stays in
// registers between the two passes (rows up to 4096 wide; wider rows re-read y), so one L2 round trip
// follows the wait.
__global__ __launch_bounds__(256)
void rms_norm_res_kernel(const __half* __restrict__ x, const __half* __restrict__ r, const __half* __restrict__ w,
                         __half* __restrict__ y, __half* __restrict__ n, int dim, float eps, int pdl)
{
    __shared__ float s_red[8];
    __shared__ float s_scale;
    const int t = threadIdx.x, cnt = dim >> 2;
    const size_t row = (size_t) blockIdx.x * dim;
    constexpr int KEEP = 4;                                  // chunks per thread held in registers
    half4 wv[KEEP], h[KEEP];
    if (pdl) pdl_launch_dependents();
    #pragma unroll
    for (int j = 0; j < KEEP; ++j)
        if (t + j * 256 < cnt) wv[j] = reinterpret_cast<const half4*>(w)[t + j * 256];
    if (pdl) pdl_wait();
    float acc = 0.0f;
    {
        half4 xv[KEEP], rv[KEEP];
        #pragma unroll
        for (int j = 0; j < KEEP; ++j)
            if (t + j * 256 < cnt) { xv[j] = reinterpret_cast<const half4*>(x + row)[t + j * 256]; rv[j] = reinterpret_cast<const half4*>(r + row)[t + j * 256]; }
        #pragma unroll
        for (int j = 0; j < KEEP; ++j)
        {
            if (t + j * 256 >= cnt) continue;
            h[j].x = __floats2half2_rn(__low2float(xv[j].x) + __low2float(rv[j].x), __high2float(xv[j].x) + __high2float(rv[j].x));
            h[j].y = __floats2half2_rn(__low2float(xv[j].y) + __low2float(rv[j].y), __high2float(xv[j].y) + __high2float(rv[j].y));
            reinterpret_cast<half4*>(y + row)[t + j * 256] = h[j];
            const float2 a = __half22float2(h[j].x), b = __half22float2(h[j].y);
            acc += a.x * a.x + a.y * a.y;
            acc += b.x * b.x + b.y * b.y;
        }
    }
    for (int c = t + KEEP * 256; c < cnt; c += 256)             // rows wider than 4096
    {
        const half4 xv = reinterpret_cast<const half4*>(x + row)[c], rv = reinterpret_cast<const half4*>(r + row)[c];
        half4 hh;
        hh.x = __floats2half2_rn(__low2float(xv.x) + __low2float(rv.x), __high2float(xv.x) + __high2float(rv.x));
        hh.y = __floats2half2_rn(__low2float(xv.y) + __low2float(rv.y), __high2float(xv.y) + __high2float(rv.y));
        reinterpret_cast<half4*>(y + row)[c] = hh;
        const float2 a = __half22float2(hh.x), b = __half22float2(hh.y);
        acc += a.x * a.x + a.y * a.y;
        acc += b.x * b.x + b.y * b.y;
    }
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((t & 31) == 0) s_red[t >> 5] = acc;
    __syncthreads();
    if (t == 0)
    {
        float total = 0.0f;
        for (int i = 0; i < 8; ++i) total += s_red[i];
        s_scale = rsqrtf(total / (float) dim + eps);
    }
    __syncthreads();
    const float sc = s_scale;
    #pragma unroll
    for (int j = 0; j < KEEP; ++j)
    {
        if (t + j * 256 >= cnt) continue;
        half4 o;
        o.x = __hmul2(__floats2half2_rn(__low2float(h[j].x) * sc, __high2float(h[j].x) * sc), wv[j].x);
        o.y = __hmul2(__floats2half2_rn(__low2float(h[j].y) * sc, __high2float(h[j].y) * sc), wv[j].y);
        reinterpret_cast<half4*>(n + row)[t + j * 256] = o;
    }
    for (int c = t + KEEP * 256; c < cnt; c += 256)
    {
        const half4 hh = reinterpret_cast<const half4*>(y + row)[c], w1 = reinterpret_cast<const half4*>(w)[c];
        half4 o;
        o.x = __hmul2(__floats2half2_rn(__low2float(hh.x) * sc, __high2float(hh.x) * sc), w1.x);
        o.y = __hmul2(__floats2half2_rn(__low2float(hh.y) * sc, __high2float(hh.y) * sc), w1.y);
        reinterpret_cast<half4*>(n + row)[c] = o;
    }
}

// out = fp16(silu(g) * u), fp32 math
__global__ __launch_bounds__(256)
void silu_mul_kernel(const __half* __restrict__ g, const __half* __restrict__ u, __half* __restrict__ out, long count4, int pdl)
{
    if (pdl) { pdl_launch_dependents(); pdl_wait(); }
    for (long c = (long) blockIdx.x * 256 + threadIdx.x; c < count4; c += (long) gridDim.x * 256)
    {
        const half4 gv = reinterpret_cast<const half4*>(g)[c], uv = reinterpret_cast<const half4*>(u)[c];
        auto f = [](float gf, float uf) { return (gf / (1.0f + __expf(-gf))) * uf; };
        half4 o;
        o.x = __floats2half2_rn(f(__low2float(gv.x), __low2float(uv.x)), f(__high2float(gv.x), __high2float(uv.x)));
        o.y = __floats2half2_rn(f(__low2float(gv.y), __low2float(uv.y)), f(__high2float(gv.y), __high2float(uv.y)));
        reinterpret_cast<half4*>(out)[c] = o;
    }
}

// greedy pick over fp16 logits (largest value, ties to the lowest index, NaN skipped) and the state
// advance log[pos] = ids; ids = pick; pos += 1, by the block that arrives last. key / count: zero
// between launches.
__global__ __launch_bounds__(256)
void argmax_advance_kernel(const __half* __restrict__ logits, int n, long long* ids, long long* pos, long long* log,
                           long long log_cap, unsigned long long* key_out, unsigned int* count, int pdl)
{
    if (pdl) { pdl_launch_dependents(); pdl_wait(); }
    unsigned long long key = 0ull;
    for (int i = blockIdx.x * 256 + threadIdx.x; i < n; i += gridDim.x * 256)
    {
        const float v = __half2float(logits[i]);
        if (!(v == v)) continue;
        const uint32_t u = v == 0.0f ? 0u : __float_as_uint(v);
        const uint32_t ord = u ^ ((u >> 31) ? 0xffffffffu : 0x80000000u);
        const unsigned long long k = ((unsigned long long) ord << 32) | (0xffffffffu - (uint32_t) i);
        key = k > key ? k : key;
    }
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1)
    {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
        key = other > key ? other : key;
    }
    __shared__ unsigned long long s_key[8];
    if ((threadIdx.x & 31) == 0) s_key[threadIdx.x >> 5] = key;
    __syncthreads();
    if (threadIdx.x == 0)
    {
        for (int i = 1; i < 8; ++i) key = s_key[i] > key ? s_key[i] : key;
        if (key) atomicMax(key_out, key);
        __threadfence();
        if (atomicAdd(count, 1u) + 1u == gridDim.x)
        {
            __threadfence();
            const unsigned long long best = *(volatile unsigned long long*) key_out;
            const long long p = pos[0];
            if (p >= 0 && p < log_cap) log[p] = ids[0];
            ids[0] = best ? (long long) (0xffffffffu - (uint32_t) (best & 0xffffffffull)) : 0;
            pos[0] = p + 1;
            *key_out = 0ull;
            *count = 0u;
        }
    }
}

template <typename... Args>
static cudaError_t launch_pdl(void (*kernel)(Args...), int grid, cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

}  // namespace amp

using namespace amp;

AMP_API int amp_b200_rms_norm_res(const void* x, const void* r, const void* w, void* y, void* n, long rows, int dim, float eps,
                                  cudaStream_t stream)
{
    if (rows <= 0 || dim <= 0) return 0;
    AMP_REQUIRE(x && r && w && y && n && dim % 4 == 0 && rows <= 65535, "rms_norm_res: null pointer, dim not a multiple of 4, or too many rows");
    AMP_REQUIRE((((uintptr_t) x | (uintptr_t) r | (uintptr_t) w | (uintptr_t) y | (uintptr_t) n) & 7) == 0, "rms_norm_res: pointers must be 8-byte aligned");
    return cuda_rc(launch_pdl(rms_norm_res_kernel, (int) rows, stream, (const __half*) x, (const __half*) r, (const __half*) w,
                              (__half*) y, (__half*) n, dim, eps, g_pdl), "rms_norm_res launch");
}

AMP_API int amp_b200_silu_mul(const void* g, const void* u, void* out, long count, cudaStream_t stream)
{
    if (count <= 0) return 0;
    AMP_REQUIRE(g && u && out && count % 4 == 0, "silu_mul: null pointer or count not a multiple of 4");
    AMP_REQUIRE((((uintptr_t) g | (uintptr_t) u | (uintptr_t) out) & 7) == 0, "silu_mul: pointers must be 8-byte aligned");
    const long c4 = count / 4;
    const int grid = (int) (c4 + 255) / 256 > 1024 ? 1024 : (int) ((c4 + 255) / 256);
    return cuda_rc(launch_pdl(silu_mul_kernel, grid, stream, (const __half*) g, (const __half*) u, (__half*) out, c4, g_pdl), "silu_mul launch");
}

AMP_API int amp_b200_argmax_advance(const void* logits, int n, void* ids, void* pos, void* log, long long log_cap, void* ws,
                                    cudaStream_t stream)
{
    AMP_REQUIRE(logits && ids && pos && log && ws && n > 0 && ((uintptr_t) ws & 7) == 0, "argmax_advance: null or misaligned pointer");
    return cuda_rc(launch_pdl(argmax_advance_kernel, 64, stream, (const __half*) logits, n, (long long*) ids, (long long*) pos,
                              (long long*) log, log_cap, (unsigned long long*) ws, (unsigned int*) ((char*) ws + 8), g_pdl),
                   "argmax_advance launch");
}
