// Trellis-decode GEMV for decode batches (m <= 16): C = had(A*suh) @ W_hat -> had(.)*svh.
//
// Replaces the reference's exl3_gemv_kernel / exl3_gemm_kernel at small m
// (vendor/exl3/exllamav3_ext/quant/exl3_gemv_kernel.cuh:186-482, exl3_gemm_kernel.cuh:8-80) with
// a different organisation for B200:
//
//  * One CTA owns a 128-column block of the output and a contiguous range of 128-row blocks of
//    k. The k-splits of one column block form a thread-block cluster; partial sums are
//    reduced through distributed shared memory, so the kernel needs no global scratch, no
//    locks and no grid-wide barrier (the reference needs two grid.sync()s and a lock buffer).
//  * Packed trellis words are streamed global -> shared by bulk async copies (TMA, untiled
//    form) into per-warp multi-stage rings, each copy a contiguous 256*K-byte run of one tile
//    row. A stage is four tile rows (64 rows of k) by 128 columns.
//  * Decode stays in registers. The decoded weights are the A operand of mma.sync.m16n8k16
//    (16 output columns x 16 k-slots) and the activations the B operand (k-slots x 8 batch
//    rows), so a batch of up to 8 costs one MMA per 128 weights. For codebooks 0/1 the final
//    fp16 add of the codebook is done BY the tensor core: the two fp16 halves of the masked
//    product sit in adjacent k-slots against a duplicated activation, which removes the
//    byte-permute and half-add per weight from the instruction stream (fp32 accumulation of
//    x*lo + x*hi is at least as accurate as x*fp16(lo+hi)).
//  * The input Hadamard runs in each CTA's prologue per 1024-row chunk (x is tiny and L2
//    resident); the output Hadamard, svh scale and store run in the cluster leader.
//
// HBM-bound by design (K/8 bytes per weight, read once); in practice limited by integer
// issue rate: about three integer instructions per weight (window, multiply-add, lop3).
#pragma once
#include "exl3_common.cuh"
#include <cooperative_groups.h>

namespace amp {

namespace cg = cooperative_groups;

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = 8;
constexpr int GEMV_XCHUNK = 1024;              // rows of x~ held in shared memory at a time
constexpr int GEMV_XPITCH = GEMV_XCHUNK + 8;   // halves; +16 bytes keeps B-fragment loads conflict-free
constexpr int GEMV_RPITCH = 132;               // floats; cross-warp reduction rows
constexpr int GEMV_MAX_STAGES = 4;

struct GemvParams
{
    const __half* x;            // (m, k)
    const uint16_t* trellis;    // (k/16, n/16, 16K)
    const __half* suh;          // (k)
    const __half* svh;          // (n)
    void* c;                    // (m, n) fp16 or fp32
    int m, k, n;
    int c_fp32;
    int stages;                 // ring depth per warp, 1..GEMV_MAX_STAGES
    int* status;                // device word, set non-zero when a bounded wait ran out
};

__host__ __device__ constexpr int gemv_row_pitch(int K) { return 256 * K + 32; }     // bytes per tile row in a stage
__host__ __device__ constexpr int gemv_stage_bytes(int K) { return 4 * gemv_row_pitch(K); }

// byte offsets inside dynamic shared memory
struct GemvSmem
{
    int bars, part, ytot, xh, ring, total;
};

// xrows: rows of x~ / partial sums kept (the batch size m, at most 8*MB)
__host__ __device__ inline GemvSmem gemv_smem_layout(int K, int xrows, int stages)
{
    GemvSmem L;
    L.bars = 0;                                             // 8 warps x 4 stages x 8 bytes
    L.part = 512;                                           // [xrows][128] fp32, read by the cluster leader
    L.ytot = L.part + xrows * 128 * 4;                      // [xrows][128] fp32
    L.xh = L.ytot + xrows * 128 * 4;                        // [xrows][XPITCH] fp16
    L.ring = L.xh + xrows * GEMV_XPITCH * 2;
    L.ring = (L.ring + 127) & ~127;
    int ring_bytes = GEMV_WARPS * stages * gemv_stage_bytes(K);
    int red_bytes = GEMV_WARPS * xrows * GEMV_RPITCH * 4;   // overlays the ring after the main loop
    L.total = L.ring + (ring_bytes > red_bytes ? ring_bytes : red_bytes);
    return L;
}

// K words of one lane's chunk, widest loads the alignment allows
template <int K>
__device__ __forceinline__ void load_chunk(const uint32_t* p, uint32_t (&w)[K])
{
    if constexpr (K % 4 == 0)
    {
        #pragma unroll
        for (int i = 0; i < K / 4; ++i)
        {
            uint4 v = reinterpret_cast<const uint4*>(p)[i];
            w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
        }
    }
    else if constexpr (K % 2 == 0)
    {
        #pragma unroll
        for (int i = 0; i < K / 2; ++i)
        {
            uint2 v = reinterpret_cast<const uint2*>(p)[i];
            w[2 * i] = v.x; w[2 * i + 1] = v.y;
        }
    }
    else
    {
        #pragma unroll
        for (int i = 0; i < K; ++i) w[i] = p[i];
    }
}

// A-operand word of one weight: codebooks 0/1 give (lo, hi) halves, codebook 2 the raw
// 1024+bytesum pattern with a zero upper half (affine part applied in the epilogue)
template <int CB>
__device__ __forceinline__ uint32_t a_word(uint32_t s)
{
    if constexpr (CB == 2) return cb2_raw(s);
    else return cb_halves<CB>(s);
}

// The eight 16-bit states of virtual lane R (positions 8R..8R+7 of the lane's chunk).
// When K divides 16, windows 16/K positions apart are exactly 16 bits apart, so one 32-bit
// word cut from the stream holds two states (high and low half): one funnel shift serves two
// weights. Other bitrates cut each window on its own.
template <int K, int R>
__device__ __forceinline__ void states8(const uint32_t (&w)[K], uint32_t prev, uint32_t (&s)[8])
{
    if constexpr (K == 4 || K == 8)
    {
        constexpr int D = 16 / K;                       // pair distance in positions
        #pragma unroll
        for (int j = 0; j < 8; ++j)
        {
            if ((j / D) % 2 != 0) continue;             // j is the earlier (high-half) member of its pair
            const int i_lo = R * 8 + j + D;             // later member: its window ends the 32-bit word
            const int last = (i_lo + 1) * K - 1;
            const int j1 = last / 32, sh = 31 - (last % 32);
            uint32_t r;
            if (sh == 0) r = w[j1];
            else r = __funnelshift_r(w[j1], j1 == 0 ? prev : w[j1 > 0 ? j1 - 1 : 0], sh);
            s[j] = r >> 16;
            s[j + D] = r & 0xffffu;
        }
    }
    else
    {
        s[0] = window_ct<K, R * 8 + 0, K>(w, prev); s[1] = window_ct<K, R * 8 + 1, K>(w, prev);
        s[2] = window_ct<K, R * 8 + 2, K>(w, prev); s[3] = window_ct<K, R * 8 + 3, K>(w, prev);
        s[4] = window_ct<K, R * 8 + 4, K>(w, prev); s[5] = window_ct<K, R * 8 + 5, K>(w, prev);
        s[6] = window_ct<K, R * 8 + 6, K>(w, prev); s[7] = window_ct<K, R * 8 + 7, K>(w, prev);
    }
}

// Decode the lane's 8 weights of virtual lane R of one tile and issue the two MMAs. w/prev: the
// lane's K words and the word before them. xb: duplicated activations of the tile's 16 rows for
// this lane's batch row(s).
template <int K, int CB, int MB, int R>
__device__ __forceinline__ void decode_mma_r(const uint32_t (&w)[K], uint32_t prev,
                                             const uint32_t (&xb)[MB][16], float (&acc)[MB][4])
{
    uint32_t s[8], a[8];
    states8<K, R>(w, prev, s);
    #pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = a_word<CB>(s[j]);
    #pragma unroll
    for (int mb = 0; mb < MB; ++mb)
    {
        // positions j and j+4 are the same row in columns c and c+8 -> MMA rows g and g+8;
        // positions (0,1) are tile rows (2R, 2R+1), positions (2,3) rows (2R+8, 2R+9)
        mma_16816(acc[mb], a[0], a[4], a[1], a[5], xb[mb][2 * R], xb[mb][2 * R + 1]);
        mma_16816(acc[mb], a[2], a[6], a[3], a[7], xb[mb][2 * R + 8], xb[mb][2 * R + 9]);
    }
}

template <int K, int CB, int MB>
__global__ __launch_bounds__(GEMV_THREADS, (MB == 1 ? 2 : 1))
void exl3_gemv_kernel(const GemvParams P)
{
    extern __shared__ __align__(128) unsigned char smem[];
    const GemvSmem L = gemv_smem_layout(K, P.m, P.stages);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L.bars);
    float* part = reinterpret_cast<float*>(smem + L.part);
    float* ytot = reinterpret_cast<float*>(smem + L.ytot);
    __half* xh = reinterpret_cast<__half*>(smem + L.xh);
    unsigned char* ring = smem + L.ring;

    constexpr int ROWB = 256 * K;                      // bytes of one tile row of this column block
    constexpr int PITCH = gemv_row_pitch(K);
    constexpr int STAGE = gemv_stage_bytes(K);

    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int gq = lane >> 2, pq = lane & 3;
    const int nb = blockIdx.x;
    const int S = gridDim.y, split = blockIdx.y;
    const int stages = P.stages;
    const int m = P.m, k = P.k, n = P.n;

    // this CTA's k range in 64-row groups (128-row aligned so Hadamard blocks stay whole)
    const int B2 = k >> 7;
    const int g_begin = 2 * (int) ((long) B2 * split / S);
    const int g_end = 2 * (int) ((long) B2 * (split + 1) / S);
    const int my_groups = (g_end - g_begin - warp + GEMV_WARPS - 1) / GEMV_WARPS;   // groups of this warp (may be <= 0)

    uint64_t* my_bars = bars + warp * GEMV_MAX_STAGES;
    unsigned char* my_ring = ring + (size_t) warp * stages * STAGE;
    const size_t tiles_n = (size_t) n >> 4;

    auto issue = [&](int q)                            // lane 0 only
    {
        const int g = g_begin + warp + GEMV_WARPS * q;
        const int s = q % stages;
        uint64_t* bar = my_bars + s;
        mbar_expect_tx(bar, 4 * ROWB);
        const unsigned char* src = reinterpret_cast<const unsigned char*>(P.trellis)
                                 + ((size_t) (4 * g) * tiles_n + (size_t) nb * 8) * (32 * K);
        unsigned char* dst = my_ring + (size_t) s * STAGE;
        #pragma unroll
        for (int p = 0; p < 4; ++p)
            bulk_g2s(dst + p * PITCH, src + (size_t) p * tiles_n * (32 * K), ROWB, bar);
    };

    if (lane == 0)
    {
        for (int s = 0; s < stages; ++s) mbar_init(my_bars + s, 1);
        fence_mbar_init();
        // the weight stream does not depend on the previous kernel: start it before anything else
        for (int q = 0; q < stages && q < my_groups; ++q) issue(q);
    }

    float acc[MB][8][4];
    #pragma unroll
    for (int mb = 0; mb < MB; ++mb)
        #pragma unroll
        for (int nt = 0; nt < 8; ++nt)
            acc[mb][nt][0] = acc[mb][nt][1] = acc[mb][nt][2] = acc[mb][nt][3] = 0.f;
    float acc1[MB][4];                                 // cb 2 only: sum of activations (all-ones weights)
    #pragma unroll
    for (int mb = 0; mb < MB; ++mb) acc1[mb][0] = acc1[mb][1] = acc1[mb][2] = acc1[mb][3] = 0.f;

    bool ok = true;
    int q = 0;                                          // index of this warp's next group
    int q_fail = 0;                                     // first group whose data never arrived
    const int n_chunks = (g_end - g_begin + 15) >> 4;

    for (int c = 0; c < n_chunks; ++c)
    {
        const int cg0 = g_begin + 16 * c;
        const int cg1 = min(cg0 + 16, g_end);
        const int nblk = (cg1 - cg0) >> 1;              // 128-row blocks in this chunk
        __syncthreads();                                // previous chunk's x~ fully consumed (and zero fill done)

        for (int idx = warp; idx < m * nblk; idx += GEMV_WARPS)
        {
            const int b = idx / nblk, j = idx - b * nblk;
            const size_t col = (size_t) cg0 * 64 + (size_t) j * 128 + lane * 4;
            half4 v = *reinterpret_cast<const half4*>(P.x + (size_t) b * k + col);
            half4 sc = *reinterpret_cast<const half4*>(P.suh + col);
            v.x = __hmul2(v.x, sc.x);
            v.y = __hmul2(v.y, sc.y);
            float h0 = __low2float(v.x), h1 = __high2float(v.x), h2 = __low2float(v.y), h3 = __high2float(v.y);
            warp_had128(h0, h1, h2, h3, lane);
            half4 o;
            o.x = __floats2half2_rn(h0 * kRScale, h1 * kRScale);
            o.y = __floats2half2_rn(h2 * kRScale, h3 * kRScale);
            *reinterpret_cast<half4*>(xh + b * GEMV_XPITCH + j * 128 + lane * 4) = o;
        }
        __syncthreads();

        for (int g = cg0 + warp; g < cg1; g += GEMV_WARPS, ++q)
        {
            const int s = q % stages;
            const uint32_t parity = (uint32_t) (q / stages) & 1u;
            if (!ok) continue;
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(my_bars + s, parity)))
            {
                ok = false;
                q_fail = q;
                if (lane == 0) atomicExch(P.status, 1);
                continue;
            }

            // activations of this lane's tile row block: rows (g - cg0)*64 + 16*pq .. +15
            uint32_t xb[MB][16];
            #pragma unroll
            for (int mb = 0; mb < MB; ++mb)
            {
                // batch rows >= m do not exist: read row m-1 instead (their MMA columns are never stored)
                const uint4* xp = reinterpret_cast<const uint4*>(
                    xh + min(mb * 8 + gq, m - 1) * GEMV_XPITCH + (g - cg0) * 64 + 16 * pq);
                uint4 v0 = xp[0], v1 = xp[1];
                const uint32_t r[8] = { v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w };
                #pragma unroll
                for (int i = 0; i < 8; ++i)
                {
                    xb[mb][2 * i] = __byte_perm(r[i], r[i], 0x1010);
                    xb[mb][2 * i + 1] = __byte_perm(r[i], r[i], 0x3232);
                }
            }

            const unsigned char* st = my_ring + (size_t) s * STAGE + pq * PITCH;
            #pragma unroll
            for (int nt = 0; nt < 8; ++nt)
            {
                const uint32_t* tile = reinterpret_cast<const uint32_t*>(st + nt * (32 * K));
                uint32_t w[K];
                load_chunk<K>(tile + gq * K, w);
                const uint32_t prev = tile[(gq * K + 8 * K - 1) % (8 * K)];
                float a4[MB][4];
                #pragma unroll
                for (int mb = 0; mb < MB; ++mb)
                {
                    a4[mb][0] = acc[mb][nt][0]; a4[mb][1] = acc[mb][nt][1];
                    a4[mb][2] = acc[mb][nt][2]; a4[mb][3] = acc[mb][nt][3];
                }
                decode_mma_r<K, CB, MB, 0>(w, prev, xb, a4);
                decode_mma_r<K, CB, MB, 1>(w, prev, xb, a4);
                decode_mma_r<K, CB, MB, 2>(w, prev, xb, a4);
                decode_mma_r<K, CB, MB, 3>(w, prev, xb, a4);
                #pragma unroll
                for (int mb = 0; mb < MB; ++mb)
                {
                    acc[mb][nt][0] = a4[mb][0]; acc[mb][nt][1] = a4[mb][1];
                    acc[mb][nt][2] = a4[mb][2]; acc[mb][nt][3] = a4[mb][3];
                }
            }
            if constexpr (CB == 2)
            {
                // sum of x~ over the 64 rows of this group: weights of 1.0 in the low half
                #pragma unroll
                for (int mb = 0; mb < MB; ++mb)
                    #pragma unroll
                    for (int i = 0; i < 8; ++i)
                        mma_16816(acc1[mb], 0x3c00u, 0x3c00u, 0x3c00u, 0x3c00u, xb[mb][2 * i], xb[mb][2 * i + 1]);
            }

            __syncwarp();                               // every lane has its words in registers
            if (lane == 0 && q + stages < my_groups) issue(q + stages);
        }
    }

    // drain copies that were issued but never consumed (only possible after a failed wait)
    if (!ok)
        for (int qq = q_fail; qq < q_fail + stages && qq < my_groups; ++qq)
            mbar_wait_bounded(my_bars + (qq % stages), (uint32_t) (qq / stages) & 1u);

    __syncthreads();                                    // ring is free: reuse it for the cross-warp reduction

    float* red = reinterpret_cast<float*>(ring);        // [warp][m][RPITCH]
    #pragma unroll
    for (int mb = 0; mb < MB; ++mb)
    {
        const int b0 = mb * 8 + 2 * pq;
        #pragma unroll
        for (int nt = 0; nt < 8; ++nt)
        {
            float d0 = acc[mb][nt][0], d1 = acc[mb][nt][1], d2 = acc[mb][nt][2], d3 = acc[mb][nt][3];
            if constexpr (CB == 2)
            {
                // w = raw * k_inv + k_bias  ->  sum x*w = k_inv * sum x*raw + k_bias * sum x
                const float kinv = __half2float(__ushort_as_half((unsigned short) 0x1eee));
                const float kbias = __half2float(__ushort_as_half((unsigned short) 0xc931));
                d0 = d0 * kinv + acc1[mb][0] * kbias; d1 = d1 * kinv + acc1[mb][1] * kbias;
                d2 = d2 * kinv + acc1[mb][2] * kbias; d3 = d3 * kinv + acc1[mb][3] * kbias;
            }
            float* r0 = red + ((size_t) warp * m + b0) * GEMV_RPITCH + nt * 16 + gq;
            if (b0 < m) { r0[0] = d0; r0[8] = d2; }
            if (b0 + 1 < m) { r0[GEMV_RPITCH] = d1; r0[GEMV_RPITCH + 8] = d3; }
        }
    }
    __syncthreads();

    for (int idx = t; idx < m * 128; idx += GEMV_THREADS)
    {
        const int b = idx >> 7, col = idx & 127;
        float sum = 0.f;
        #pragma unroll
        for (int w8 = 0; w8 < GEMV_WARPS; ++w8)
            sum += red[((size_t) w8 * m + b) * GEMV_RPITCH + col];
        part[b * 128 + col] = sum;
    }

    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();                                     // partial sums of every split are in place

    if (split == 0)
    {
        for (int idx = t; idx < m * 128; idx += GEMV_THREADS)
        {
            float sum = 0.f;
            for (int r = 0; r < S; ++r)                 // rank order: deterministic
                sum += cluster.map_shared_rank(part, r)[idx];
            ytot[idx] = sum;
        }
    }
    cluster.sync();                                     // peers may exit; ytot visible to the leader's warps
    if (split != 0) return;

    for (int b = warp; b < m; b += GEMV_WARPS)
    {
        float4 v = reinterpret_cast<const float4*>(ytot + b * 128)[lane];
        float h0 = v.x, h1 = v.y, h2 = v.z, h3 = v.w;
        warp_had128(h0, h1, h2, h3, lane);
        h0 *= kRScale; h1 *= kRScale; h2 *= kRScale; h3 *= kRScale;
        const half4 sv = reinterpret_cast<const half4*>(P.svh + (size_t) nb * 128)[lane];
        if (P.c_fp32)
        {
            float4 o = make_float4(h0 * __low2float(sv.x), h1 * __high2float(sv.x),
                                   h2 * __low2float(sv.y), h3 * __high2float(sv.y));
            reinterpret_cast<float4*>(reinterpret_cast<float*>(P.c) + (size_t) b * n + (size_t) nb * 128)[lane] = o;
        }
        else
        {
            half4 o;
            o.x = __hmul2(__floats2half2_rn(h0, h1), sv.x);
            o.y = __hmul2(__floats2half2_rn(h2, h3), sv.y);
            reinterpret_cast<half4*>(reinterpret_cast<__half*>(P.c) + (size_t) b * n + (size_t) nb * 128)[lane] = o;
        }
    }
}

typedef void (*gemv_fn)(const GemvParams);

// one lookup function per K, defined by the per-K translation units: (cb, MB) -> kernel
#define AMP_GEMV_LOOKUP_DECL(K) gemv_fn gemv_kernel_k##K(int cb, int MB);
AMP_GEMV_LOOKUP_DECL(1) AMP_GEMV_LOOKUP_DECL(2) AMP_GEMV_LOOKUP_DECL(3) AMP_GEMV_LOOKUP_DECL(4)
AMP_GEMV_LOOKUP_DECL(5) AMP_GEMV_LOOKUP_DECL(6) AMP_GEMV_LOOKUP_DECL(7) AMP_GEMV_LOOKUP_DECL(8)
#undef AMP_GEMV_LOOKUP_DECL

}  // namespace amp
