// Prefill GEMM: C (M, n) = x~ (M, k) @ W_hat (k, n) -> Hadamard -> * svh, with W_hat decoded from
// the trellis on the fly into shared memory and multiplied on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory). x~ = fp16(H(x * suh) / sqrt(128)) is produced by
// the Hadamard kernel into the caller's A_had scratch first.
//
// Replaces, for m > 16, the reference's trellis-decode GEMM (exl3_gemm_kernel,
// vendor/exl3/exllamav3_ext/quant/exl3_gemm_kernel.cuh:8-80, mma.sync, re-decoding the weights for
// every 16-row slab) and its reconstruct + cuBLAS path (torch_exl3_gemm_recon,
// src/torch/amp_torch.cpp:11148-11230, which writes the whole fp16 weight to global memory first).
//
// One CTA = 512 tokens x 128 output columns. Per 64-row k step:
//   * all eight warps copy the x~ tile (512 x 64 fp16, four 128-row sub-tiles) with cp.async
//     into the canonical K-major 128-byte-swizzled layout, and the step's packed trellis words
//     (4 tile rows x 8 tiles) into a staging area;
//   * they decode the 8192 weights (bit-exact codebook values) straight into the swizzled
//     K-major B tile (128 columns x 64 k): each decoded weight is used for 512 tokens;
//   * one thread issues 16 tcgen05.mma (M128 x N128 x K16, fp16 in, fp32 accumulate) into four
//     128-column accumulators in tensor memory and commits them to an mbarrier that frees the
//     stage. Two stages: the copies and the decode of step i+1 run under the MMAs of step i.
// Epilogue: accumulators -> registers (tcgen05.ld) -> shared memory, then the same warp-level
// 128-point Hadamard, svh scale and rounding as the decode kernels, coalesced stores.
//
// Tensor-pipe bound by design (2 * M * k * n flops); the decode costs about a sixteenth of an
// instruction per MAC at 512 tokens per decoded weight. Every wait on an mbarrier is bounded;
// on expiry the status word is set and the CTA still frees its tensor memory.
#include "exl3_common.cuh"
#include "host_common.h"

namespace amp {

constexpr int TC_THREADS = 256;
constexpr int TC_BM = 128;            // tokens per sub-tile (UMMA M)
constexpr int TC_SUB = 4;             // sub-tiles per CTA
constexpr int TC_BN = 128;            // output columns per CTA (UMMA N)
constexpr int TC_BK = 64;             // k per step (one 128-byte swizzle row)
constexpr int TC_A_BYTES = TC_SUB * TC_BM * TC_BK * 2;     // 65536
constexpr int TC_B_BYTES = TC_BN * TC_BK * 2;              // 16384
constexpr int TC_STAGES = 2;
constexpr unsigned TC_SPIN_LIMIT = 1u << 22;   // try_wait polls before a wait is declared lost

__host__ __device__ constexpr int tc_packed_bytes(int K) { return 4 * 8 * 32 * K; }      // 4 tile rows x 8 tiles
__host__ __device__ constexpr int tc_stage_bytes(int K) { return TC_A_BYTES + TC_B_BYTES + tc_packed_bytes(K); }
__host__ __device__ constexpr int tc_smem_bytes(int K) { return 1024 + TC_STAGES * tc_stage_bytes(K); }

__device__ int g_tc_status;

struct TcParams
{
    const __half* xh;           // (M, k) rotated input
    const uint16_t* trellis;    // (k/16, n/16, 16K)
    const __half* svh;          // (n)
    void* c;                    // (M, n) fp16 or fp32
    int M, k, n, c_fp32;
    int* status;
};

// K-major, 128-byte swizzle, rows of 128 bytes: byte offset of (row, 16-byte chunk)
__device__ __forceinline__ uint32_t sw128(int row, int chunk)
{
    return (uint32_t) (row * 128 + ((chunk ^ (row & 7)) << 4));
}

__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr)
{
    // start address >> 4 [0,14), LBO (1, unused for swizzled K-major) [16,30), SBO = 1024 B >> 4
    // [32,46), descriptor version 1 [46,48), layout SWIZZLE_128B (2) [61,64)
    return (uint64_t) ((smem_addr & 0x3ffff) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        :: "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 :: "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void cp_async16_zfill(void* dst, const void* src, int src_bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(smem_u32(dst)), "l"(src), "r"(src_bytes) : "memory");
}

template <int K, int CB>
__global__ __launch_bounds__(TC_THREADS, 1)
void exl3_gemm_tc_kernel(const TcParams P)
{
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte alignment is required by the swizzled layout
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    __shared__ uint64_t bar_free[TC_STAGES];
    __shared__ uint64_t bar_done;
    __shared__ uint32_t s_tmem;
    __shared__ int s_bad;

    constexpr int STAGE = tc_stage_bytes(K);
    constexpr int TW = 8 * K;                          // words per trellis tile
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int nb = blockIdx.x, mb = blockIdx.y;
    const int m0 = mb * (TC_SUB * TC_BM);
    const int rows = min(TC_SUB * TC_BM, P.M - m0);    // valid token rows of this CTA
    const int ksteps = P.k / TC_BK;
    const size_t tiles_n = (size_t) P.n >> 4;

    if (t == 0)
    {
        mbar_init(&bar_free[0], 1);
        mbar_init(&bar_free[1], 1);
        mbar_init(&bar_done, 1);
        fence_mbar_init();
        s_bad = 0;
    }
    __syncwarp();
    if (warp == 0)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&s_tmem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    auto stage_a = [&](int s) { return smem + s * STAGE; };
    auto stage_b = [&](int s) { return smem + s * STAGE + TC_A_BYTES; };
    auto stage_p = [&](int s) { return smem + s * STAGE + TC_A_BYTES + TC_B_BYTES; };

    // x~ tile (rows beyond M read as zero) and packed trellis words of k step i into stage s
    auto issue_loads = [&](int i, int s)
    {
        unsigned char* a = stage_a(s);
        for (int c = t; c < TC_SUB * TC_BM * 8; c += TC_THREADS)
        {
            const int r = c >> 3, ch = c & 7;                 // row inside the CTA tile, 16-byte chunk
            const int sub = r >> 7, rr = r & 127;
            const int ok = (r < rows) ? 16 : 0;
            const __half* src = P.xh + (size_t) (m0 + (ok ? r : 0)) * P.k + (size_t) i * TC_BK + ch * 8;
            cp_async16_zfill(a + sub * (TC_BM * 128) + sw128(rr, ch), src, ok);
        }
        unsigned char* p = stage_p(s);
        constexpr int ROWP = 8 * 32 * K;                        // bytes of one tile row (8 tiles)
        for (int c = t; c < 4 * ROWP / 16; c += TC_THREADS)
        {
            const int row = c / (ROWP / 16), off = (c - row * (ROWP / 16)) * 16;
            const unsigned char* src = reinterpret_cast<const unsigned char*>(P.trellis)
                                     + ((size_t) (4 * i + row) * tiles_n + (size_t) nb * 8) * (32 * K) + off;
            cp_async16_zfill(p + row * ROWP + off, src, 16);
        }
        cp_async_commit();
    };

    bool ok = true;
    auto wait_bar = [&](uint64_t* bar, uint32_t parity)
    {
        if (!ok) return;
        bool done = false;
        for (unsigned spin = 0; spin < TC_SPIN_LIMIT && !done; ++spin) done = mbar_try_wait(bar, parity);
        if (!done) { ok = false; s_bad = 1; }
    };

    // instruction descriptor: D fp32, A/B fp16, both K-major, N = 128, M = 128
    constexpr uint32_t IDESC = (1u << 4) | ((uint32_t) (TC_BN >> 3) << 17) | ((uint32_t) (TC_BM >> 4) << 24);

    issue_loads(0, 0);
    for (int i = 0; i < ksteps; ++i)
    {
        const int s = i & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                 // stage s holds x~ and the packed words of step i

        // decode 4 x 8 trellis tiles into the B tile: warp w takes tile column w, rows 0..3
        {
            const uint32_t* packed = reinterpret_cast<const uint32_t*>(stage_p(s));
            unsigned char* b = stage_b(s);
            #pragma unroll
            for (int kt = 0; kt < 4; ++kt)
            {
                const uint32_t* ring = packed + (kt * 8 + warp) * TW;
                uint32_t st[8];
                #pragma unroll
                for (int j = 0; j < 8; ++j) st[j] = window_rt<K>(ring, lane * 8 + j);
                // positions (0,1) rows (2p, 2p+1), (2,3) rows (2p+8, 2p+9) of column c; (4..7) the same for column c+8
                const int p2 = (lane & 3) * 2, cc = lane >> 2;
                #pragma unroll
                for (int h = 0; h < 4; ++h)
                {
                    const __half w0 = decode_state<CB>(st[2 * h]), w1 = decode_state<CB>(st[2 * h + 1]);
                    const int ncol = warp * 16 + cc + 8 * (h >> 1);
                    const int kk = kt * 16 + p2 + 8 * (h & 1);
                    *reinterpret_cast<__half2*>(b + sw128(ncol, kk >> 3) + (kk & 7) * 2) = __halves2half2(w0, w1);
                }
            }
        }
        // make the generic-proxy writes (cp.async data, decoded tile) visible to the tensor core
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();

        if (t == 0)
        {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a0 = smem_u32(stage_a(s)), b0 = smem_u32(stage_b(s));
            #pragma unroll
            for (int sub = 0; sub < TC_SUB; ++sub)
                #pragma unroll
                for (int kk = 0; kk < TC_BK / 16; ++kk)
                    umma_f16(tmem + sub * TC_BN, make_desc(a0 + sub * (TC_BM * 128) + kk * 32),
                             make_desc(b0 + kk * 32), IDESC, (i > 0 || kk > 0) ? 1u : 0u);
            umma_commit(&bar_free[s]);                  // arrives when these MMAs have read the stage
            if (i == ksteps - 1) umma_commit(&bar_done);
        }

        // the other stage is free once the MMAs of step i-1 have completed: refill it for step i+1
        if (i + 1 < ksteps)
        {
            if (i >= 1) wait_bar(&bar_free[s ^ 1], (uint32_t) (((i - 1) >> 1) & 1));
            issue_loads(i + 1, s ^ 1);
        }
    }

    // ---- epilogue ----
    wait_bar(&bar_done, 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    const bool all_ok = ok && !s_bad;

    float* tile = reinterpret_cast<float*>(smem);        // [128][132] fp32, reuses the pipeline stages
    constexpr int TP = 132;
    for (int sub = 0; sub < TC_SUB; ++sub)
    {
        if (sub * TC_BM >= rows) break;
        if (all_ok)
        {
            // warp w reads tensor-memory lanes 32*(w%4).. (token rows), columns 64*(w/4)..+63 of this accumulator
            const int lrow = 32 * (warp & 3) + lane;
            #pragma unroll
            for (int half = 0; half < 2; ++half)
            {
                const int col0 = 64 * (warp >> 2) + 32 * half;
                const uint32_t taddr = tmem + ((uint32_t) (32 * (warp & 3)) << 16) + (uint32_t) (sub * TC_BN + col0);
                uint32_t v[32];
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                      "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                      "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                #pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<uint4*>(tile + lrow * TP + col0 + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            }
        }
        __syncthreads();
        if (all_ok)
        {
            const half4 sv = reinterpret_cast<const half4*>(P.svh + (size_t) nb * 128)[lane];
            for (int r = warp; r < TC_BM; r += TC_THREADS / 32)
            {
                const int grow = m0 + sub * TC_BM + r;
                if (grow >= P.M) break;
                const float4 v = *reinterpret_cast<const float4*>(tile + r * TP + lane * 4);
                float h0 = v.x, h1 = v.y, h2 = v.z, h3 = v.w;
                warp_had128(h0, h1, h2, h3, lane);
                h0 *= kRScale; h1 *= kRScale; h2 *= kRScale; h3 *= kRScale;
                if (P.c_fp32)
                {
                    float4 o = make_float4(h0 * __low2float(sv.x), h1 * __high2float(sv.x),
                                           h2 * __low2float(sv.y), h3 * __high2float(sv.y));
                    reinterpret_cast<float4*>(reinterpret_cast<float*>(P.c) + (size_t) grow * P.n + (size_t) nb * 128)[lane] = o;
                }
                else
                {
                    half4 o;
                    o.x = __hmul2(__floats2half2_rn(h0, h1), sv.x);
                    o.y = __hmul2(__floats2half2_rn(h2, h3), sv.y);
                    reinterpret_cast<half4*>(reinterpret_cast<__half*>(P.c) + (size_t) grow * P.n + (size_t) nb * 128)[lane] = o;
                }
            }
        }
        __syncthreads();
    }

    if (t == 0 && !all_ok) atomicExch(P.status, 1);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(512u) : "memory");
}

typedef void (*tc_fn)(const TcParams);

#define AMP_TC_ROW(cb) { exl3_gemm_tc_kernel<1, cb>, exl3_gemm_tc_kernel<2, cb>, exl3_gemm_tc_kernel<3, cb>, exl3_gemm_tc_kernel<4, cb>, \
                         exl3_gemm_tc_kernel<5, cb>, exl3_gemm_tc_kernel<6, cb>, exl3_gemm_tc_kernel<7, cb>, exl3_gemm_tc_kernel<8, cb> }
static const tc_fn k_tc[3][8] = { AMP_TC_ROW(0), AMP_TC_ROW(1), AMP_TC_ROW(2) };
#undef AMP_TC_ROW

// x~ (M, k) fp16 already rotated -> C. Called by amp_exl3_gemm for m > 16.
int launch_gemm_tc(const void* xh, const void* trellis, void* c, const void* svh, int M, int k, int n,
                   int K, int cb, int c_fp32, cudaStream_t stream)
{
    AMP_REQUIRE(xh && trellis && c && svh, "exl3_gemm: null pointer");
    AMP_REQUIRE(K >= 1 && K <= 8 && cb >= 0 && cb <= 2, "exl3_gemm: unsupported bitrate / codebook");
    AMP_REQUIRE(M >= 1 && k % 128 == 0 && n % 128 == 0 && k > 0 && n > 0, "exl3_gemm: k and n must be multiples of 128");
    AMP_REQUIRE(((uintptr_t) xh & 15) == 0 && ((uintptr_t) trellis & 15) == 0 && ((uintptr_t) c & 15) == 0 &&
                ((uintptr_t) svh & 7) == 0, "exl3_gemm: misaligned pointer");
    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev)) return cuda_rc(e, "cudaGetDevice");
    tc_fn fn = k_tc[cb][K - 1];
    const int smem = tc_smem_bytes(K);
    if (cudaError_t e = ensure_smem(fn, smem, dev)) return cuda_rc(e, "exl3_gemm smem attribute");
    TcParams P;
    P.xh = (const __half*) xh; P.trellis = (const uint16_t*) trellis; P.svh = (const __half*) svh; P.c = c;
    P.M = M; P.k = k; P.n = n; P.c_fp32 = c_fp32;
    {
        static int* status_ptr[64] = {};
        int*& sp = status_ptr[dev & 63];
        if (!sp)
            if (cudaError_t e = cudaGetSymbolAddress((void**) &sp, g_tc_status)) return cuda_rc(e, "status symbol");
        P.status = sp;
    }
    const long mblocks = ((long) M + TC_SUB * TC_BM - 1) / (TC_SUB * TC_BM);
    AMP_REQUIRE(mblocks <= 65535, "exl3_gemm: too many rows");
    dim3 grid(n / 128, (unsigned) mblocks);
    fn<<<grid, TC_THREADS, smem, stream>>>(P);
    return cuda_rc(cudaGetLastError(), "exl3_gemm_tc launch");
}

}  // namespace amp

using namespace amp;

// Reads and clears the prefill GEMM's status word on the current device (non-zero: a bounded
// wait on a tensor-core completion barrier ran out). Synchronises.
AMP_API int amp_exl3_gemm_status(int* out)
{
    int v = 0, zero = 0;
    if (cudaError_t e = cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int))) return cuda_rc(e, "status read");
    if (v) if (cudaError_t e = cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int))) return cuda_rc(e, "status clear");
    if (out) *out = v;
    return 0;
}
