// EXL3 trellis -> fp16 weight, two forms:
//   amp_exl3_reconstruct      W_hat (rotated basis), bit-exact decode
//   amp_exl3_reconstruct_had  W = diag(suh) . H128 . W_hat . H128 . diag(svh) / 128 (original basis)
//
// Replaces the reference's reconstruct / reconstruct_slice / reconstruct_had_slice
// (vendor/exl3/exllamav3_ext/quant/reconstruct.cu:141-197, 431-503). The decode is integer work
// plus one fp16 add, so results are bit-identical; the original-basis form performs the same
// sequence of fp16 / fp32 operations per element as the reference (:300-377) and is bit-identical
// too.
#include "exl3_common.cuh"
#include "host_common.h"

namespace amp {

// ------------------------------------------------------------------------------------------
// Rotated-basis reconstruct: one CTA = 16 rows x 128 columns (eight tiles), one warp per tile.
// HBM-bound: K/8 bytes in, 2 bytes out per weight.
// ------------------------------------------------------------------------------------------

// HALF: K is the integer part KA of a half-integer rate KA + 0.5 (a tile is 4 * (2 KA + 1) words)
template <int K, int CB, bool HALF = false>
__global__ __launch_bounds__(256)
void reconstruct_kernel(__half* __restrict__ out, const uint16_t* __restrict__ trellis,
                        int tiles_n, int tile_n_offset, int n_out, const long long* __restrict__ t_trellis, size_t mat_elems)
{
    // batch form: blockIdx.z = matrix; the trellis comes from a device pointer table and the
    // outputs are stacked
    if (t_trellis)
    {
        trellis = reinterpret_cast<const uint16_t*>(t_trellis[blockIdx.z]);
        out += (size_t) blockIdx.z * mat_elems;
    }
    constexpr int TW = HALF ? 4 * (2 * K + 1) : 8 * K;     // uint32 words per tile
    __shared__ __align__(16) uint32_t s_packed[8 * TW];
    __shared__ __align__(16) __half s_tile[16][128 + 8];

    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int kt = blockIdx.y, nb = blockIdx.x;

    const uint16_t* src = trellis + ((size_t) kt * tiles_n + tile_n_offset + nb * 8) * (2 * TW);
    if (t < 2 * TW)                            // 8 tiles * 4 TW bytes = 2*TW int4
        reinterpret_cast<int4*>(s_packed)[t] = reinterpret_cast<const int4*>(src)[t];
    __syncthreads();

    const uint32_t* ring = s_packed + warp * TW;
    #pragma unroll
    for (int j = 0; j < 8; ++j)
    {
        uint32_t s;
        if constexpr (HALF) s = window_rt_half<K>(ring, lane * 8 + j);
        else s = window_rt<K>(ring, lane * 8 + j);
        int row = 2 * (lane & 3) + (j & 1) + 8 * ((j >> 1) & 1);
        int col = (lane >> 2) + 8 * (j >> 2);
        s_tile[row][warp * 16 + col] = decode_state<CB>(s);
    }
    __syncthreads();

    const int r = t >> 4, c = t & 15;          // 16 rows x 16 int4
    int4 v = *reinterpret_cast<const int4*>(&s_tile[r][c * 8]);
    *reinterpret_cast<int4*>(out + (size_t) (kt * 16 + r) * n_out + nb * 128 + c * 8) = v;
}

// ------------------------------------------------------------------------------------------
// Original-basis reconstruct: one CTA = one 128x128 block held in shared memory (32 KB) with
// an XOR swizzle on 4-column chunks so that both transform directions are conflict-free.
// ------------------------------------------------------------------------------------------

__device__ __forceinline__ __half2 had_tail_h2(__half2 v, int lane)
{
    #pragma unroll
    for (int i = 1; i < 32; i <<= 1)
    {
        __half2 p = __shfl_xor_sync(0xffffffffu, v, i);
        v = (lane & i) ? __hsub2(p, v) : __hadd2(v, p);
    }
    return v;
}

template <int K, int CB, bool HALF = false>
__global__ __launch_bounds__(256)
void reconstruct_had_kernel(__half* __restrict__ out, const uint16_t* __restrict__ trellis,
                            const __half* __restrict__ suh, const __half* __restrict__ svh,
                            int tiles_n, int tile_n_offset, int n_out, const long long* __restrict__ t_trellis,
                            const long long* __restrict__ t_suh, const long long* __restrict__ t_svh, size_t mat_elems)
{
    if (t_trellis)
    {
        trellis = reinterpret_cast<const uint16_t*>(t_trellis[blockIdx.z]);
        suh = reinterpret_cast<const __half*>(t_suh[blockIdx.z]);
        svh = reinterpret_cast<const __half*>(t_svh[blockIdx.z]);
        out += (size_t) blockIdx.z * mat_elems;
    }
    constexpr int TW = HALF ? 4 * (2 * K + 1) : 8 * K;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* st = reinterpret_cast<__half*>(smem_raw);                       // [128][128] swizzled
    uint32_t* s_packed = reinterpret_cast<uint32_t*>(smem_raw + 128 * 128 * 2);   // [8][8][TW]

    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int kb = blockIdx.y, nb = blockIdx.x;

    auto at = [&](int R, int c) -> int {       // half index of element (R, c)
        return R * 128 + ((((c >> 2) ^ (R >> 2)) & 31) << 2) + (c & 3);
    };

    // 8 tile rows x (8 tiles contiguous = 2*TW int4)
    for (int u = t; u < 8 * 2 * TW; u += 256)
    {
        int j = u / (2 * TW), r = u % (2 * TW);
        const uint16_t* src = trellis + ((size_t) (kb * 8 + j) * tiles_n + tile_n_offset + nb * 8) * (2 * TW);
        reinterpret_cast<int4*>(s_packed + j * 8 * TW)[r] = reinterpret_cast<const int4*>(src)[r];
    }
    __syncthreads();

    for (int j = 0; j < 8; ++j)                // warp = tile column, j = tile row
    {
        const uint32_t* ring = s_packed + (j * 8 + warp) * TW;
        #pragma unroll
        for (int i = 0; i < 8; ++i)
        {
            uint32_t s;
            if constexpr (HALF) s = window_rt_half<K>(ring, lane * 8 + i);
            else s = window_rt<K>(ring, lane * 8 + i);
            int row = j * 16 + 2 * (lane & 3) + (i & 1) + 8 * ((i >> 1) & 1);
            int col = warp * 16 + (lane >> 2) + 8 * (i >> 2);
            st[at(row, col)] = decode_state<CB>(s);
        }
    }
    __syncthreads();

    const __half2 rs2 = __float2half2_rn(0.08838834764831845f);

    // columns: lane l owns rows 4l..4l+3, four columns (one chunk) at a time, all fp16
    #pragma unroll
    for (int qq = 0; qq < 4; ++qq)
    {
        const int q = warp * 4 + qq;
        __half2 a[4], b[4];
        #pragma unroll
        for (int i = 0; i < 4; ++i)
        {
            half4 v = *reinterpret_cast<const half4*>(st + at(lane * 4 + i, q * 4));
            a[i] = v.x; b[i] = v.y;
        }
        #pragma unroll
        for (int x = 0; x < 2; ++x)
        {
            __half2* v = x ? b : a;
            __half2 s0 = __hadd2(v[0], v[1]), d0 = __hsub2(v[0], v[1]);
            __half2 s1 = __hadd2(v[2], v[3]), d1 = __hsub2(v[2], v[3]);
            v[0] = had_tail_h2(__hmul2(__hadd2(s0, s1), rs2), lane);
            v[1] = had_tail_h2(__hmul2(__hadd2(d0, d1), rs2), lane);
            v[2] = had_tail_h2(__hmul2(__hsub2(s0, s1), rs2), lane);
            v[3] = had_tail_h2(__hmul2(__hsub2(d0, d1), rs2), lane);
        }
        #pragma unroll
        for (int i = 0; i < 4; ++i)
        {
            half4 v; v.x = a[i]; v.y = b[i];
            *reinterpret_cast<half4*>(st + at(lane * 4 + i, q * 4)) = v;
        }
    }
    __syncthreads();

    // rows: lane l owns columns 4l..4l+3; fp32 in-lane butterfly, one rounding, fp16 tail
    const half4 sv4 = reinterpret_cast<const half4*>(svh)[nb * 32 + lane];
    #pragma unroll 4
    for (int rr = 0; rr < 16; ++rr)
    {
        const int R = warp * 16 + rr;
        half4 in = *reinterpret_cast<const half4*>(st + at(R, lane * 4));
        float v0 = __low2float(in.x), v1 = __high2float(in.x);
        float v2 = __low2float(in.y), v3 = __high2float(in.y);
        float s0 = v0 + v1, d0 = v0 - v1, s1 = v2 + v3, d1 = v2 - v3;
        __half2 h01 = had_tail_h2(__hmul2(__floats2half2_rn(s0 + s1, d0 + d1), rs2), lane);
        __half2 h23 = had_tail_h2(__hmul2(__floats2half2_rn(s0 - s1, d0 - d1), rs2), lane);
        const __half2 su2 = __half2half2(suh[kb * 128 + R]);
        half4 o;
        o.x = __hmul2(__hmul2(h01, su2), sv4.x);
        o.y = __hmul2(__hmul2(h23, su2), sv4.y);
        *reinterpret_cast<half4*>(out + (size_t) (kb * 128 + R) * n_out + nb * 128 + lane * 4) = o;
    }
}

typedef void (*recon_fn)(__half*, const uint16_t*, int, int, int, const long long*, size_t);
typedef void (*recon_had_fn)(__half*, const uint16_t*, const __half*, const __half*, int, int, int,
                             const long long*, const long long*, const long long*, size_t);

#define AMP_ROW(T, cb) { T<1, cb>, T<2, cb>, T<3, cb>, T<4, cb>, T<5, cb>, T<6, cb>, T<7, cb>, T<8, cb> }
static const recon_fn k_recon[3][8] = { AMP_ROW(reconstruct_kernel, 0), AMP_ROW(reconstruct_kernel, 1), AMP_ROW(reconstruct_kernel, 2) };
static const recon_had_fn k_recon_had[3][8] = { AMP_ROW(reconstruct_had_kernel, 0), AMP_ROW(reconstruct_had_kernel, 1), AMP_ROW(reconstruct_had_kernel, 2) };
#undef AMP_ROW
// half-integer rates 1.5 / 2.5 / 3.5: mul1 codebook only, as in the reference (Q/reconstruct.cu:116-127)
static const recon_fn k_recon_half[3] = { reconstruct_kernel<1, 2, true>, reconstruct_kernel<2, 2, true>, reconstruct_kernel<3, 2, true> };
static const recon_had_fn k_recon_had_half[3] = { reconstruct_had_kernel<1, 2, true>, reconstruct_had_kernel<2, 2, true>,
                                                  reconstruct_had_kernel<3, 2, true> };

// K as the C ABI passes it: 1..8, or AMP_EXL3_HALF_RATE(KA) = 256 + KA for KA + 0.5 bits per weight
static inline bool k_is_half(int K) { return K > 256 && K <= 256 + 3; }

static int check_common(const void* out, const void* trellis, int k, int n, int K, int cb, int n_offset, int n_out)
{
    AMP_REQUIRE(out && trellis, "reconstruct: null pointer");
    AMP_REQUIRE((K >= 1 && K <= 8) || k_is_half(K), "reconstruct: unsupported EXL3 bitrate %d (integer 1..8, or 1.5 / 2.5 / 3.5)", K);
    AMP_REQUIRE(!k_is_half(K) || cb == 2, "reconstruct: half-integer bitrates require the mul1 codebook");
    AMP_REQUIRE(cb >= 0 && cb <= 2, "reconstruct: codebook index %d out of range", cb);
    AMP_REQUIRE(k >= 0 && n >= 0 && k % 16 == 0 && n % 16 == 0, "reconstruct: k and n must be multiples of 16");
    AMP_REQUIRE(n_out % 128 == 0, "unpacked N dimension must be divisible by 128");
    AMP_REQUIRE(n_offset % 128 == 0 && n_offset >= 0, "n_offset must be a non-negative multiple of 128");
    AMP_REQUIRE(n_offset + n_out <= n, "reconstruct slice exceeds packed tensor bounds");
    AMP_REQUIRE(((uintptr_t) out & 15) == 0 && ((uintptr_t) trellis & 15) == 0, "reconstruct: pointers must be 16-byte aligned");
    return 0;
}

}  // namespace amp

using namespace amp;

AMP_API int amp_exl3_reconstruct(void* unpacked, const void* trellis, int k, int n, int K, int cb,
                                    int n_offset, int n_out, cudaStream_t stream)
{
    if (k == 0 || n_out == 0) return 0;
    if (int rc = check_common(unpacked, trellis, k, n, K, cb, n_offset, n_out)) return rc;
    AMP_REQUIRE(k / 16 <= 65535, "reconstruct: k too large");
    dim3 grid(n_out / 128, k / 16);
    const recon_fn fn = k_is_half(K) ? k_recon_half[K - 257] : k_recon[cb][K - 1];
    fn<<<grid, 256, 0, stream>>>((__half*) unpacked, (const uint16_t*) trellis, n / 16, n_offset / 16, n_out, nullptr, 0);
    return cuda_rc(cudaGetLastError(), "amp_exl3_reconstruct");
}

// `batch` whole matrices of one shape in one launch: unpacked (batch, k, n) fp16 contiguous,
// packed_ptrs a DEVICE array of int64 trellis addresses (rotated basis, as amp_exl3_reconstruct)
AMP_API int amp_exl3_reconstruct_batch(void* unpacked, const void* packed_ptrs, int batch, int k, int n, int K, int cb,
                                       cudaStream_t stream)
{
    AMP_REQUIRE(batch >= 0 && batch <= 65535, "reconstruct_batch: batch out of range");
    if (batch == 0 || k == 0 || n == 0) return 0;
    AMP_REQUIRE(packed_ptrs, "reconstruct_batch: null pointer table");
    if (int rc = check_common(unpacked, unpacked, k, n, K, cb, 0, n)) return rc;
    AMP_REQUIRE(!k_is_half(K), "reconstruct_batch: integer bitrates only");
    AMP_REQUIRE(k / 16 <= 65535, "reconstruct: k too large");
    dim3 grid(n / 128, k / 16, batch);
    k_recon[cb][K - 1]<<<grid, 256, 0, stream>>>((__half*) unpacked, nullptr, n / 16, 0, n,
                                                 (const long long*) packed_ptrs, (size_t) k * n);
    return cuda_rc(cudaGetLastError(), "amp_exl3_reconstruct_batch");
}

AMP_API int amp_exl3_reconstruct_had(void* unpacked, const void* trellis, const void* suh, const void* svh,
                                        int k, int n, int K, int cb, int n_offset, int n_out,
                                        cudaStream_t stream)
{
    if (k == 0 || n_out == 0) return 0;
    if (int rc = check_common(unpacked, trellis, k, n, K, cb, n_offset, n_out)) return rc;
    AMP_REQUIRE(suh && svh, "reconstruct_had: null scale vector");
    AMP_REQUIRE(k % 128 == 0, "reconstruct_had: K dimension must be divisible by 128");
    AMP_REQUIRE(((uintptr_t) svh & 7) == 0, "reconstruct_had: svh must be 8-byte aligned");
    AMP_REQUIRE(k / 128 <= 65535, "reconstruct_had: k too large");
    const bool half = k_is_half(K);
    const int smem = 128 * 128 * 2 + 64 * (half ? 4 * (2 * (K - 256) + 1) : 8 * K) * 4;
    recon_had_fn fn = half ? k_recon_had_half[K - 257] : k_recon_had[cb][K - 1];
    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev)) return cuda_rc(e, "cudaGetDevice");
    if (cudaError_t e = ensure_smem(fn, smem, dev)) return cuda_rc(e, "reconstruct_had smem");
    dim3 grid(n_out / 128, k / 128);
    fn<<<grid, 256, smem, stream>>>((__half*) unpacked, (const uint16_t*) trellis, (const __half*) suh,
                                    (const __half*) svh, n / 16, n_offset / 16, n_out, nullptr, nullptr, nullptr, 0);
    return cuda_rc(cudaGetLastError(), "amp_exl3_reconstruct_had");
}

// `batch` whole matrices of one shape into the original basis in one launch; packed_ptrs / suh_ptrs
// / svh_ptrs are DEVICE arrays of int64 addresses (trellis, k-length suh, n-length svh per matrix)
AMP_API int amp_exl3_reconstruct_had_batch(void* unpacked, const void* packed_ptrs, const void* suh_ptrs, const void* svh_ptrs,
                                           int batch, int k, int n, int K, int cb, cudaStream_t stream)
{
    AMP_REQUIRE(batch >= 0 && batch <= 65535, "reconstruct_had_batch: batch out of range");
    if (batch == 0 || k == 0 || n == 0) return 0;
    AMP_REQUIRE(packed_ptrs && suh_ptrs && svh_ptrs, "reconstruct_had_batch: null pointer table");
    if (int rc = check_common(unpacked, unpacked, k, n, K, cb, 0, n)) return rc;
    AMP_REQUIRE(!k_is_half(K), "reconstruct_had_batch: integer bitrates only");
    AMP_REQUIRE(k % 128 == 0, "reconstruct_had_batch: K dimension must be divisible by 128");
    AMP_REQUIRE(k / 128 <= 65535, "reconstruct_had: k too large");
    const int smem = 128 * 128 * 2 + 64 * 8 * K * 4;
    recon_had_fn fn = k_recon_had[cb][K - 1];
    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev)) return cuda_rc(e, "cudaGetDevice");
    if (cudaError_t e = ensure_smem(fn, smem, dev)) return cuda_rc(e, "reconstruct_had smem");
    dim3 grid(n / 128, k / 128, batch);
    fn<<<grid, 256, smem, stream>>>((__half*) unpacked, nullptr, nullptr, nullptr, n / 16, 0, n,
                                    (const long long*) packed_ptrs, (const long long*) suh_ptrs, (const long long*) svh_ptrs, (size_t) k * n);
    return cuda_rc(cudaGetLastError(), "amp_exl3_reconstruct_had_batch");
}
