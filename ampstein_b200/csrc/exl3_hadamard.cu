// Blockwise 128-point Hadamard with optional pre / post scale vectors, as its own launch.
// Replaces the reference's had_r_128 (vendor/exl3/exllamav3_ext/quant/hadamard.cu:125-207;
// arithmetic of hadamard_inner.cuh:93-279): fp16 data is scaled in fp16 before the transform,
// transformed in fp32, multiplied by scale/sqrt(128), rounded once, post-scaled in fp16; fp32
// data stays fp32 throughout. Works in place.
#include "exl3_common.cuh"
#include <cuda_bf16.h>
#include "host_common.h"

namespace amp {

// bf16 rows in, fp16 rows out (prefill activations arrive as bf16): fp32 scale and transform, one
// rounding to fp16
__global__ __launch_bounds__(256)
void had_r_128_bf16_kernel(const __nv_bfloat16* __restrict__ in, __half* __restrict__ out,
                           const __half* __restrict__ pre, const __half* __restrict__ post,
                           long chunks, int chunks_per_row, float r_scale)
{
    const int lane = threadIdx.x & 31;
    const long chunk = (long) blockIdx.x * 8 + (threadIdx.x >> 5);
    if (chunk >= chunks) return;
    const int cb = (int) (chunk % chunks_per_row);
    const uint2 raw = reinterpret_cast<const uint2*>(in)[chunk * 32 + lane];
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    float h0 = __low2float(a), h1 = __high2float(a), h2 = __low2float(b), h3 = __high2float(b);
    if (pre)
    {
        half4 s = reinterpret_cast<const half4*>(pre)[cb * 32 + lane];
        h0 *= __low2float(s.x); h1 *= __high2float(s.x); h2 *= __low2float(s.y); h3 *= __high2float(s.y);
    }
    warp_had128(h0, h1, h2, h3, lane);
    half4 o;
    o.x = __floats2half2_rn(h0 * r_scale, h1 * r_scale);
    o.y = __floats2half2_rn(h2 * r_scale, h3 * r_scale);
    if (post)
    {
        half4 s = reinterpret_cast<const half4*>(post)[cb * 32 + lane];
        o.x = __hmul2(o.x, s.x);
        o.y = __hmul2(o.y, s.y);
    }
    reinterpret_cast<half4*>(out)[chunk * 32 + lane] = o;
}

// fp32 rows in, fp16 rows out (the form the reference's GEMM epilogue uses on its fp32
// accumulators, had_fh_r_128_inner, vendor/exl3/exllamav3_ext/quant/hadamard_inner.cuh:216-279):
// fp32 pre-scale and transform, one rounding to fp16, fp16 post-scale
__global__ __launch_bounds__(256)
void had_r_128_fh_kernel(const float* __restrict__ in, __half* __restrict__ out,
                         const __half* __restrict__ pre, const __half* __restrict__ post,
                         long chunks, int chunks_per_row, float r_scale)
{
    const int lane = threadIdx.x & 31;
    const long chunk = (long) blockIdx.x * 8 + (threadIdx.x >> 5);
    if (chunk >= chunks) return;
    const int cb = (int) (chunk % chunks_per_row);
    const float4 v = reinterpret_cast<const float4*>(in)[chunk * 32 + lane];
    float h0 = v.x, h1 = v.y, h2 = v.z, h3 = v.w;
    if (pre)
    {
        half4 s = reinterpret_cast<const half4*>(pre)[cb * 32 + lane];
        h0 *= __low2float(s.x); h1 *= __high2float(s.x); h2 *= __low2float(s.y); h3 *= __high2float(s.y);
    }
    warp_had128(h0, h1, h2, h3, lane);
    half4 o;
    o.x = __floats2half2_rn(h0 * r_scale, h1 * r_scale);
    o.y = __floats2half2_rn(h2 * r_scale, h3 * r_scale);
    if (post)
    {
        half4 s = reinterpret_cast<const half4*>(post)[cb * 32 + lane];
        o.x = __hmul2(o.x, s.x);
        o.y = __hmul2(o.y, s.y);
    }
    reinterpret_cast<half4*>(out)[chunk * 32 + lane] = o;
}

template <bool F32>
__global__ __launch_bounds__(256)
void had_r_128_kernel(const void* __restrict__ in, void* __restrict__ out,
                      const __half* __restrict__ pre, const __half* __restrict__ post,
                      long chunks, int chunks_per_row, float r_scale)
{
    const int lane = threadIdx.x & 31;
    const long chunk = (long) blockIdx.x * 8 + (threadIdx.x >> 5);
    if (chunk >= chunks) return;
    const int cb = (int) (chunk % chunks_per_row);       // which 128-block of the row

    float h0, h1, h2, h3;
    if constexpr (F32)
    {
        float4 v = reinterpret_cast<const float4*>(in)[chunk * 32 + lane];
        h0 = v.x; h1 = v.y; h2 = v.z; h3 = v.w;
        if (pre)
        {
            half4 s = reinterpret_cast<const half4*>(pre)[cb * 32 + lane];
            h0 *= __low2float(s.x); h1 *= __high2float(s.x);
            h2 *= __low2float(s.y); h3 *= __high2float(s.y);
        }
    }
    else
    {
        half4 v = reinterpret_cast<const half4*>(in)[chunk * 32 + lane];
        if (pre)
        {
            half4 s = reinterpret_cast<const half4*>(pre)[cb * 32 + lane];
            v.x = __hmul2(v.x, s.x);
            v.y = __hmul2(v.y, s.y);
        }
        h0 = __low2float(v.x); h1 = __high2float(v.x);
        h2 = __low2float(v.y); h3 = __high2float(v.y);
    }

    warp_had128(h0, h1, h2, h3, lane);
    h0 *= r_scale; h1 *= r_scale; h2 *= r_scale; h3 *= r_scale;

    if constexpr (F32)
    {
        if (post)
        {
            half4 s = reinterpret_cast<const half4*>(post)[cb * 32 + lane];
            h0 *= __low2float(s.x); h1 *= __high2float(s.x);
            h2 *= __low2float(s.y); h3 *= __high2float(s.y);
        }
        reinterpret_cast<float4*>(out)[chunk * 32 + lane] = make_float4(h0, h1, h2, h3);
    }
    else
    {
        half4 o;
        o.x = __floats2half2_rn(h0, h1);
        o.y = __floats2half2_rn(h2, h3);
        if (post)
        {
            half4 s = reinterpret_cast<const half4*>(post)[cb * 32 + lane];
            o.x = __hmul2(o.x, s.x);
            o.y = __hmul2(o.y, s.y);
        }
        reinterpret_cast<half4*>(out)[chunk * 32 + lane] = o;
    }
}

// Rotated prefill activations in the layout the tensor-core GEMM fetches them in: x~ =
// fp16(H(x * suh) / sqrt(128)) of an (M, k) matrix, stored k-step-major -- [k / 64][M] rows of 64
// halves (128 bytes) -- with the 16-byte pieces of a row already XOR-swizzled by (row & 7). A
// 128-token x 64-k box is then 16 KB of contiguous global memory that one bulk copy drops into
// shared memory in the K-major 128-byte-swizzled form the MMA descriptors expect. Same arithmetic
// as the plain kernels above (fp16 input: scaled in fp16; bf16 input: scaled in fp32).
template <bool BF16>
__global__ __launch_bounds__(256)
void had_tiled_kernel(const void* __restrict__ in, __half* __restrict__ out, const __half* __restrict__ pre,
                      const long long* __restrict__ pre_table, long chunks, int chunks_per_row, long M, float r_scale)
{
    // bundle: blockIdx.y = source; each source has its own scale vector and its own x~
    if (pre_table)
    {
        pre = reinterpret_cast<const __half*>(pre_table[blockIdx.y]);
        out += (size_t) blockIdx.y * (size_t) chunks * 128;
    }
    // the GEMM that consumes this kernel's output may be scheduled from now on: it allocates its
    // tensor memory and starts its weight stream under this kernel, and waits (griddepcontrol.wait
    // in its fetch thread) before it reads the first rotated row
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const long chunk = (long) blockIdx.x * 8 + (threadIdx.x >> 5);
    if (chunk >= chunks) return;
    const long row = chunk / chunks_per_row;
    const int cb = (int) (chunk - row * chunks_per_row);
    const half4 s = reinterpret_cast<const half4*>(pre)[cb * 32 + lane];
    float h0, h1, h2, h3;
    if constexpr (BF16)
    {
        const uint2 raw = reinterpret_cast<const uint2*>(in)[chunk * 32 + lane];
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        h0 = __low2float(a) * __low2float(s.x); h1 = __high2float(a) * __high2float(s.x);
        h2 = __low2float(b) * __low2float(s.y); h3 = __high2float(b) * __high2float(s.y);
    }
    else
    {
        half4 v = reinterpret_cast<const half4*>(in)[chunk * 32 + lane];
        v.x = __hmul2(v.x, s.x);
        v.y = __hmul2(v.y, s.y);
        h0 = __low2float(v.x); h1 = __high2float(v.x); h2 = __low2float(v.y); h3 = __high2float(v.y);
    }
    warp_had128(h0, h1, h2, h3, lane);
    half4 o;
    o.x = __floats2half2_rn(h0 * r_scale, h1 * r_scale);
    o.y = __floats2half2_rn(h2 * r_scale, h3 * r_scale);
    // lane l holds k = 128 cb + 4l .. +3: k step 2 cb + l / 16, 16-byte piece (l % 16) / 2, half of the piece l % 2
    const long kstep = 2 * cb + (lane >> 4);
    const int piece = ((lane & 15) >> 1) ^ (int) (row & 7);
    unsigned char* dst = reinterpret_cast<unsigned char*>(out) + ((kstep * M + row) << 7) + (piece << 4) + ((lane & 1) << 3);
    *reinterpret_cast<half4*>(dst) = o;
}

// (M, k) fp16 or bf16 -> tiled x~ (M * k halves). Internal to the prefill path.
int launch_had_tiled(const void* in, void* out, const void* pre, long M, int k, int bf16, cudaStream_t stream,
                     const long long* pre_table, int sources)
{
    AMP_REQUIRE(in && out && (pre || pre_table) && M > 0 && k > 0 && k % 128 == 0, "exl3_gemm: bad arguments to the input rotation");
    AMP_REQUIRE(((uintptr_t) in & 7) == 0 && ((uintptr_t) out & 15) == 0 && ((uintptr_t) pre & 7) == 0, "exl3_gemm: misaligned pointer");
    AMP_REQUIRE(sources >= 1 && sources <= 65535, "exl3_mgemm: source count out of range");
    const long chunks = M * (k / 128);
    const long blocks = (chunks + 7) / 8;
    AMP_REQUIRE(blocks <= 0x7fffffffL, "exl3_gemm: too many rows");
    const dim3 grid((unsigned) blocks, pre_table ? (unsigned) sources : 1u);
    if (bf16) had_tiled_kernel<true><<<grid, 256, 0, stream>>>(in, (__half*) out, (const __half*) pre, pre_table, chunks, k / 128, M, kRScale);
    else had_tiled_kernel<false><<<grid, 256, 0, stream>>>(in, (__half*) out, (const __half*) pre, pre_table, chunks, k / 128, M, kRScale);
    return cuda_rc(cudaGetLastError(), "exl3_gemm input rotation");
}

}  // namespace amp

using namespace amp;

// dtype: 0 = fp16 in/out, 1 = fp32 in/out, 2 = bf16 in / fp16 out, 3 = fp32 in / fp16 out. pre / post: fp16 vectors of
// `cols` values or null.
AMP_API int amp_had_r_128(const void* in, void* out, const void* pre, const void* post,
                             long rows, int cols, int dtype, float scale, cudaStream_t stream)
{
    AMP_REQUIRE(dtype >= 0 && dtype <= 3, "had_r_128: unsupported datatype");
    AMP_REQUIRE(rows >= 0 && cols >= 0 && cols % 128 == 0, "had_r_128: columns must be divisible by 128");
    if (rows == 0 || cols == 0) return 0;
    AMP_REQUIRE(in && out, "had_r_128: null pointer");
    const uintptr_t imask = (dtype == 1 || dtype == 3) ? 15 : 7, omask = dtype == 1 ? 15 : 7;
    AMP_REQUIRE(((uintptr_t) in & imask) == 0 && ((uintptr_t) out & omask) == 0, "had_r_128: misaligned pointer");
    AMP_REQUIRE(((uintptr_t) pre & 7) == 0 && ((uintptr_t) post & 7) == 0, "had_r_128: misaligned scale vector");
    const long chunks = rows * (cols / 128);
    const long blocks = (chunks + 7) / 8;
    AMP_REQUIRE(blocks <= 0x7fffffffL, "had_r_128: too many rows");
    const float rs = scale * kRScale;
    if (dtype == 3)
        had_r_128_fh_kernel<<<(unsigned) blocks, 256, 0, stream>>>((const float*) in, (__half*) out, (const __half*) pre, (const __half*) post, chunks, cols / 128, rs);
    else if (dtype == 2)
        had_r_128_bf16_kernel<<<(unsigned) blocks, 256, 0, stream>>>((const __nv_bfloat16*) in, (__half*) out, (const __half*) pre, (const __half*) post, chunks, cols / 128, rs);
    else if (dtype)
        had_r_128_kernel<true><<<(unsigned) blocks, 256, 0, stream>>>(in, out, (const __half*) pre, (const __half*) post, chunks, cols / 128, rs);
    else
        had_r_128_kernel<false><<<(unsigned) blocks, 256, 0, stream>>>(in, out, (const __half*) pre, (const __half*) post, chunks, cols / 128, rs);
    return cuda_rc(cudaGetLastError(), "amp_had_r_128");
}
