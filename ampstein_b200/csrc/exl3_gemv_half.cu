// Decode GEMV for the half-integer bitrates 1.5 / 2.5 / 3.5 (mul1 codebook): c (m, n) = had(x * suh) @
// W_hat -> had(.) * svh for up to 16 rows, as one CTA per 128 output columns.
//
// Replaces the half_k instances of the reference's kernels for this format (exl3_gemv_half_inst,
// comp_unit_h1..h3, vendor/exl3/exllamav3_ext/quant/exl3_dq.cuh:254-284 for the decode). A first,
// plain form: positions alternate KA and KA + 1 bits, so a lane's 32-weight piece is not a whole
// number of words and the word-per-lane streaming of the tuned integer-rate kernel does not carry
// over; here a warp stages one tile (4 * (2 KA + 1) words) at a time in shared memory and every lane
// cuts its eight windows with run-time shifts. fp32 accumulation over k in tile order, the four
// lanes that share a column are added by shuffles, then the same Hadamard / svh epilogue as the
// other kernels. Correct and deterministic; lightly tuned (words requested four tiles ahead; one CTA
// per 128 columns and k slice, the slices' partial sums added in slice order by the last to arrive).
#include "exl3_common.cuh"
#include "host_common.h"

namespace amp {

constexpr int GH_XROWS = 1024;          // rows of x~ staged in shared memory at a time (m * 2 KB)

template <int KA>
__global__ __launch_bounds__(256)
void exl3_gemv_half_kernel(const __half* __restrict__ xt, const uint16_t* __restrict__ trellis, const __half* __restrict__ svh,
                           void* __restrict__ c, int m, int k, int n, int c_fp32, int* __restrict__ counters, float* __restrict__ scratch)
{
    constexpr int TW = 4 * (2 * KA + 1);                   // words per tile
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* xs = reinterpret_cast<__half*>(smem_raw);       // [m][GH_XROWS] rotated input rows of the chunk
    float* outs = reinterpret_cast<float*>(smem_raw);       // [m][128] after the k loop (reuses xs)
    __shared__ uint32_t s_tile[8][4][TW];                   // per warp: the four tiles of one pass
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int nb = blockIdx.x, tiles_n = n >> 4;
    const int S = gridDim.y, z = blockIdx.y;                // k split: this CTA takes tile rows [z, z + 1) * (k / 16) / S
    __shared__ int s_last;
    const int r0 = 2 * (lane & 3), ca = lane >> 2;          // this lane's rows r0, r0+1, r0+8, r0+9 of columns ca and ca+8

    float acc[16][2];
    #pragma unroll
    for (int b = 0; b < 16; ++b) acc[b][0] = acc[b][1] = 0.0f;

    // a lane's word of a tile is requested four tiles ahead (the tiles of a column come from HBM
    // 4 TW bytes at a time, one latency each if asked for only when needed)
    const int ktiles = k >> 4, kt_begin = z * (ktiles / S), kt_end = kt_begin + ktiles / S;
    const uint32_t* base = reinterpret_cast<const uint32_t*>(trellis) + ((size_t) nb * 8 + warp) * TW;
    const size_t kstride = (size_t) tiles_n * TW;
    auto fetch = [&](int kt) { return (lane < TW && kt < kt_end) ? __ldg(base + (size_t) kt * kstride + lane) : 0u; };
    uint32_t pf[4];
    #pragma unroll
    for (int j = 0; j < 4; ++j) pf[j] = fetch(kt_begin + j);

    for (int kt0 = kt_begin; kt0 < kt_end; kt0 += 4)
    {
        if (kt0 == kt_begin || (kt0 & (GH_XROWS / 16 - 1)) == 0)
        {
            // the chunk of rotated input rows this tile row lies in
            const int k0 = (kt0 & ~(GH_XROWS / 16 - 1)) << 4, rows = min(GH_XROWS, k - k0);
            __syncthreads();
            for (int i = t; i < m * (rows >> 3); i += 256)
            {
                const int b = i / (rows >> 3), j = i - b * (rows >> 3);
                reinterpret_cast<uint4*>(xs + b * GH_XROWS)[j] = reinterpret_cast<const uint4*>(xt + (size_t) b * k + k0)[j];
            }
            __syncthreads();
        }
        // four tiles per pass: staged together, so that their decode chains overlap
        __syncwarp();
        #pragma unroll
        for (int j = 0; j < 4; ++j)
        {
            if (lane < TW) s_tile[warp][j][lane] = pf[j];
            pf[j] = fetch(kt0 + j + 4);                    // (k is a multiple of 128: the tile count is a multiple of 8)
        }
        __syncwarp();
        #pragma unroll
        for (int j = 0; j < 4; ++j)
        {
            const int kt = kt0 + j;
            float w[8];
            #pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = __half2float(decode_state<2>(window_rt_half<KA>(s_tile[warp][j], lane * 8 + i)));
            // position i of the lane: row r0 + (i & 1) + 8 * ((i >> 1) & 1), column ca + 8 * (i >> 2)
            const int xoff = (kt & (GH_XROWS / 16 - 1)) * 16 + r0;
            #pragma unroll
            for (int b = 0; b < 16; ++b)
                if (b < m)
                {
                    const __half* xr = xs + b * GH_XROWS + xoff;
                    const float x0 = __half2float(xr[0]), x1 = __half2float(xr[1]), x8 = __half2float(xr[8]), x9 = __half2float(xr[9]);
                    acc[b][0] = fmaf(w[0], x0, fmaf(w[1], x1, fmaf(w[2], x8, fmaf(w[3], x9, acc[b][0]))));
                    acc[b][1] = fmaf(w[4], x0, fmaf(w[5], x1, fmaf(w[6], x8, fmaf(w[7], x9, acc[b][1]))));
                }
        }
    }
    __syncthreads();
    // the four lanes of a column hold the sums of their rows
    #pragma unroll
    for (int b = 0; b < 16; ++b)
        if (b < m)
        {
            #pragma unroll
            for (int e = 0; e < 2; ++e)
            {
                float v = acc[b][e];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                if ((lane & 3) == 0) outs[b * 128 + warp * 16 + ca + 8 * e] = v;
            }
        }
    __syncthreads();
    if (S > 1)
    {
        // k split: partial sums to global memory; the CTA that arrives last at the block's counter
        // adds the S partials in split order (fixed, so the result does not depend on timing),
        // resets the counter and finishes the block
        float* mine = scratch + ((size_t) nb * S + z) * (size_t) m * 128;
        for (int i = t; i < m * 128; i += 256) mine[i] = outs[i];
        __threadfence();
        __syncthreads();
        if (t == 0)
        {
            const int old = atomicAdd(&counters[nb], 1);
            s_last = old == S - 1;
            if (s_last) counters[nb] = 0;
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        for (int i = t; i < m * 128; i += 256)
        {
            float v = 0.0f;
            for (int q = 0; q < S; ++q) v += __ldcg(scratch + ((size_t) nb * S + q) * (size_t) m * 128 + i);
            outs[i] = v;
        }
        __syncthreads();
    }
    const half4 sv = reinterpret_cast<const half4*>(svh + (size_t) nb * 128)[lane];
    for (int b = warp; b < m; b += 8)
    {
        const float4 v = *reinterpret_cast<const float4*>(outs + b * 128 + lane * 4);
        float h0 = v.x, h1 = v.y, h2 = v.z, h3 = v.w;
        warp_had128(h0, h1, h2, h3, lane);
        h0 *= kRScale; h1 *= kRScale; h2 *= kRScale; h3 *= kRScale;
        if (c_fp32)
            reinterpret_cast<float4*>(reinterpret_cast<float*>(c) + (size_t) b * n + (size_t) nb * 128)[lane] =
                make_float4(h0 * __low2float(sv.x), h1 * __high2float(sv.x), h2 * __low2float(sv.y), h3 * __high2float(sv.y));
        else
        {
            half4 o;
            o.x = __hmul2(__floats2half2_rn(h0, h1), sv.x);
            o.y = __hmul2(__floats2half2_rn(h2, h3), sv.y);
            reinterpret_cast<half4*>(reinterpret_cast<__half*>(c) + (size_t) b * n + (size_t) nb * 128)[lane] = o;
        }
    }
}

typedef void (*gemv_half_fn)(const __half*, const uint16_t*, const __half*, void*, int, int, int, int, int*, float*);
static const gemv_half_fn k_gemv_half[3] = { exl3_gemv_half_kernel<1>, exl3_gemv_half_kernel<2>, exl3_gemv_half_kernel<3> };

// xt: the rotated input fp16(had(x * suh) / sqrt(128)), (m, k), written by the caller (amp_had_r_128)
// counters / scratch: the decode kernels' per-stream workspace (arrival counters, zero between
// launches; scratch_bytes of partial-sum space) for the k split; counters may be null (no split)
int launch_gemv_half(const void* xt, const void* trellis, const void* svh, void* c, int m, int k, int n, int KA, int c_fp32,
                     int* counters, float* scratch, size_t scratch_bytes, int max_blocks, int sms, cudaStream_t stream)
{
    AMP_REQUIRE(xt && trellis && svh && c, "exl3_gemv: null pointer");
    AMP_REQUIRE(KA >= 1 && KA <= 3 && m >= 1 && m <= 16 && k > 0 && n > 0 && k % 128 == 0 && n % 128 == 0,
                "exl3_gemv: half-integer bitrates take 1..16 rows, k and n multiples of 128");
    AMP_REQUIRE(((uintptr_t) xt & 15) == 0 && ((uintptr_t) trellis & 3) == 0 && ((uintptr_t) svh & 7) == 0 && ((uintptr_t) c & 15) == 0,
                "exl3_gemv: misaligned pointer");
    const int smem = m * GH_XROWS * 2 > m * 128 * 4 ? m * GH_XROWS * 2 : m * 128 * 4;
    gemv_half_fn fn = k_gemv_half[KA - 1];
    // k split so that about two CTAs per SM are in flight: a CTA walks its tile rows one after the
    // other, so a narrow weight on few CTAs is bound by that walk (4096 x 4096: 32 CTAs of 256 tile rows)
    int S = 1;
    const int blocks = n / 128, ktiles = k / 16;
    if (counters && scratch && blocks <= max_blocks)
        while (S < 16 && blocks * S * 2 <= 2 * sms && ktiles % (8 * S) == 0 && ktiles / (2 * S) >= 8 &&
               (size_t) blocks * (2 * S) * m * 128 * sizeof(float) <= scratch_bytes) S *= 2;
    fn<<<dim3(blocks, S), 256, smem, stream>>>((const __half*) xt, (const uint16_t*) trellis, (const __half*) svh, c, m, k, n, c_fp32,
                                                counters, scratch);
    return cuda_rc(cudaGetLastError(), "exl3_gemv half-rate launch");
}

}  // namespace amp
