// Prefill GEMM: C (M, n) = x~ (M, k) @ W_hat (k, n) -> Hadamard -> * svh, with W_hat decoded from
// the trellis on the fly into shared memory and multiplied on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory). x~ = fp16(H(x * suh) / sqrt(128)) is produced by
// the rotation kernel (had_tiled_kernel) into the caller's A_had scratch first.
//
// Replaces, for m > 16, the reference's trellis-decode GEMM (exl3_gemm_kernel,
// vendor/exl3/exllamav3_ext/quant/exl3_gemm_kernel.cuh:8-80, mma.sync, re-decoding the weights for
// every 16-row slab) and its reconstruct + cuBLAS path (torch_exl3_gemm_recon,
// src/torch/amp_torch.cpp:11148-11230, which writes the whole fp16 weight to global memory first).
//
// Two kernels. The pair form (exl3_gemm_tc2_kernel, second half of this file: two SMs per 512 x 256
// tile with cta_group::2) runs wherever n is a multiple of 256 and the grid fills the device; the
// single-CTA form below covers narrow weights and short batches.
//
// One CTA = 512 tokens x 128 output columns, k walked in steps of 64. Three roles, 18 warps:
//   * warp 0, one thread: fetches the x~ tile of a step with four bulk (TMA) copies of 16 KB. The
//     rotation kernel has already written x~ k-step-major with the 128-byte swizzle applied, so a
//     128-token x 64-k box is contiguous in global memory and lands in the canonical K-major
//     layout as it is (two stages); a stage is refilled the moment the MMAs that read it have
//     completed.
//   * warp 1, one thread: issues the step's 16 tcgen05.mma (M128 x N128 x K16, fp16 in, fp32
//     accumulate) into four 128-column accumulators in tensor memory as soon as the x~ tile has
//     landed and the weight tile is decoded, and commits them to the barriers that free the
//     stages. It does nothing else: with fetch and issue in one thread the tensor pipe idled
//     two thirds of the time.
//   * warps 2-17 decode, in two groups of eight that take alternate k steps: warp w of a group
//     owns tile column w of the 128-column block; a lane streams its 32 weights' packed words
//     through its own cp.async ring (several k steps deep: the words come from HBM exactly once
//     and a step lasts about half a microsecond), cuts the windows with compile-time shifts,
//     forms the exact fp16 codebook values and writes them as 16-byte pieces into the swizzled
//     K-major B tile (three stages): each decoded weight serves 512 tokens.
//   * mbarriers tie the roles together: TMA completion (bytes), "B tile decoded" (one arrival per
//     decode warp of the group), and tcgen05.commit arrivals that free an A stage and a B stage.
// Epilogue: accumulators -> registers (tcgen05.ld) -> shared memory, then the same warp-level
// 128-point Hadamard, svh scale and rounding as the decode kernels, coalesced stores.
//
// Tensor-pipe bound by design (2 * M * k * n flops). Every wait on an mbarrier is bounded; on
// expiry the status word is set, every role leaves its loop and the CTA still frees its tensor
// memory.
#include "exl3_gemv_kernel.cuh"
#include "exl3_gemv_host.h"
#include "host_common.h"
#include <mutex>

namespace amp {

constexpr int TC_DECODE_WARPS = 16;           // two groups of eight that take alternate k steps
constexpr int TC_THREADS = 32 * (2 + TC_DECODE_WARPS);     // warp 0 fetches, warp 1 issues the MMAs, the rest decode
constexpr int TC_BM = 128;            // tokens per sub-tile (UMMA M)
constexpr int TC_SUB = 4;             // sub-tiles per CTA
constexpr int TC_BN = 128;            // output columns per CTA (UMMA N)
constexpr int TC_BK = 64;             // k per step (one 128-byte swizzle row)
constexpr int TC_A_SLOTS = 2, TC_B_STAGES = 3;
constexpr int TC_A_BYTES = TC_SUB * TC_BM * TC_BK * 2;     // one slot = the x~ tile of one k step: 65536
constexpr int TC_B_BYTES = TC_BN * TC_BK * 2;              // 16384
// packed trellis words travel through per-lane cp.async rings this many k steps deep (the words
// come from HBM exactly once: the ring must cover the HBM latency, a step is ~0.5 us)
__host__ __device__ constexpr int tc_p_stages(int K) { return K <= 4 ? 4 : 3; }        // per decode group: every other step
__host__ __device__ constexpr int tc_smem_bytes(int K)
{
    return 1024 + TC_A_SLOTS * TC_A_BYTES + TC_B_STAGES * TC_B_BYTES + TC_DECODE_WARPS * tc_p_stages(K) * 128 * K;
}
constexpr unsigned TC_SPIN_LIMIT = 1u << 22;   // try_wait polls before a wait is declared lost

__device__ int g_tc_status;

struct TcParams
{
    const unsigned char* xt;    // rotated input, k-step-major and pre-swizzled (had_tiled_kernel): [k/64][M][128 bytes]
    const uint16_t* trellis;    // (k/16, n/16, 16K)
    const __half* svh;          // (n)
    void* c;                    // (M, n) fp16 or fp32
    int M, k, n, c_fp32;        // n: row width of the trellis / output (bundle: columns per slice)
    int sub;                    // 128-token sub-tiles per CTA: 4, or fewer when the grid would leave SMs idle
    int* status;
    int relay_release;          // pair form: the relay's remote arrival releases at cluster scope (slower; default relaxed)
    // bundle (tables == 1): several matrices or equal-width column slices in one grid, identified
    // by device pointer tables with one entry per slice, exactly as the decode kernel's table mode
    int tables;
    const long long* t_trellis;
    const long long* t_svh;
    const long long* t_c;       // may be null: outputs stacked in c as (slices, M, n)
    const int* t_stride;        // may be null: row width = n
    const int* t_src;           // may be null: rotated input of slice i is source i
    // expert groups (grouped instances of the single-CTA kernel): blockIdx.y walks a tile table
    // that a kernel in front of this one built from the routing, blockIdx.x = projection * (n / 128)
    // + column block. A tile is up to sub * 128 consecutive rows of ONE expert in the padded,
    // expert-sorted row space of xt / c (M = its capacity); t_trellis / t_svh hold g_kinds *
    // g_experts entries, projection-major; projection p reads xt + p * M * k halves and writes
    // c + p * M * n elements.
    const int* g_ntiles;        // device: tiles in use (CTAs beyond it return at once)
    const int* g_tile_e;        // device: expert of a tile
    const int* g_tile_row0;     // device: first padded row of a tile (a multiple of 8)
    const int* g_tile_rows;     // device: valid rows of a tile (1 .. sub * 128)
    int g_experts;
    // experts of different bit widths: per projection a device table of the experts' widths (null:
    // all of this launch's width); a CTA whose expert has another width than this instance returns
    const unsigned char* g_bits[2];
};

// What one CTA (pair) works on: its weight, scales, output, rotated input and column block
struct TcSlice
{
    const unsigned char* trellis;
    const __half* svh;
    unsigned char* c;
    const unsigned char* xt;
    int n_row;                  // row width of trellis and output
    int nb;                     // column block (of BW columns) inside the slice
};

template <int BW>
__device__ __forceinline__ TcSlice tc_slice(const TcParams& P, int nbg)
{
    TcSlice s;
    s.trellis = reinterpret_cast<const unsigned char*>(P.trellis);
    s.svh = P.svh; s.c = reinterpret_cast<unsigned char*>(P.c); s.xt = P.xt; s.n_row = P.n; s.nb = nbg;
    if (P.tables)
    {
        const int bps = P.n / BW, slice = nbg / bps;
        s.nb = nbg - slice * bps;
        s.trellis = reinterpret_cast<const unsigned char*>(P.t_trellis[slice]);
        s.svh = reinterpret_cast<const __half*>(P.t_svh[slice]);
        s.n_row = P.t_stride ? P.t_stride[slice] : P.n;
        s.c = P.t_c ? reinterpret_cast<unsigned char*>(P.t_c[slice])
                    : reinterpret_cast<unsigned char*>(P.c) + (size_t) slice * P.M * P.n * (P.c_fp32 ? 4 : 2);
        const int src = P.t_src ? P.t_src[slice] : slice;
        s.xt = P.xt + (size_t) src * P.M * P.k * 2;
    }
    return s;
}

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

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}

// 4K bytes of one lane, global -> this lane's ring slot, widest cp.async the alignment allows
template <int K>
__device__ __forceinline__ void cp_async_chunk(uint32_t dst, const unsigned char* src)
{
    if constexpr (K % 4 == 0)
    {
        #pragma unroll
        for (int i = 0; i < K / 4; ++i)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst + 16 * i), "l"(src + 16 * i) : "memory");
    }
    else if constexpr (K % 2 == 0)
    {
        #pragma unroll
        for (int i = 0; i < K / 2; ++i)
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" :: "r"(dst + 8 * i), "l"(src + 8 * i) : "memory");
    }
    else
    {
        #pragma unroll
        for (int i = 0; i < K; ++i)
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"(dst + 4 * i), "l"(src + 4 * i) : "memory");
    }
}

// two states -> two exact fp16 weights packed (a in the low half), bit-identical to the reference
template <int CB>
__device__ __forceinline__ uint32_t weights2(uint32_t sa, uint32_t sb)
{
    if constexpr (CB == 2)
    {
        const uint32_t raw = __byte_perm(cb2_raw(sa), cb2_raw(sb), 0x5410);
        const __half2 kinv = __half2half2(__ushort_as_half((unsigned short) 0x1eee));
        const __half2 kbias = __half2half2(__ushort_as_half((unsigned short) 0xc931));
        const __half2 w = __hfma2(*reinterpret_cast<const __half2*>(&raw), kinv, kbias);
        return *reinterpret_cast<const uint32_t*>(&w);
    }
    else
    {
        const uint32_t ya = cb_halves<CB>(sa), yb = cb_halves<CB>(sb);
        const uint32_t lo = __byte_perm(ya, yb, 0x5410), hi = __byte_perm(ya, yb, 0x7632);
        const __half2 w = __hadd2(*reinterpret_cast<const __half2*>(&lo), *reinterpret_cast<const __half2*>(&hi));
        return *reinterpret_cast<const uint32_t*>(&w);
    }
}

template <int K, int CB, bool GROUPED = false>
__global__ __launch_bounds__(TC_THREADS, GROUPED ? 2 : 1)
void exl3_gemm_tc_kernel(const TcParams P)
{
    if constexpr (GROUPED)
    {
        // the whole CTA leaves, before any barrier or allocation
        if ((int) blockIdx.y >= *P.g_ntiles || P.g_tile_rows[blockIdx.y] <= 0) return;
        const unsigned char* bits = P.g_bits[(int) blockIdx.x / (P.n / TC_BN)];
        if (bits && bits[P.g_tile_e[blockIdx.y]] != K) return;
    }
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte alignment is required by the swizzled layout
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    __shared__ uint64_t a_full[TC_A_SLOTS], a_free[TC_A_SLOTS], b_full[TC_B_STAGES], b_free[TC_B_STAGES], bar_done;
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_bad;

    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    // grouped instances size an x~ slot and the tensor-memory allocation by the launch's rows per
    // tile: with 128-row tiles two CTAs share an SM (shared memory, 2 x 128 accumulator columns)
    const int a_bytes = GROUPED ? P.sub * (TC_BM * TC_BK * 2) : TC_A_BYTES;
    const uint32_t tmem_cols = GROUPED ? (P.sub == 1 ? 128u : (P.sub == 2 ? 256u : 512u)) : 512u;
    TcSlice W;
    int m0, rows;                                       // first row and valid token rows of this CTA
    if constexpr (GROUPED)
    {
        const int tile = blockIdx.y, bpk = P.n / TC_BN, kind = (int) blockIdx.x / bpk;
        const size_t idx = (size_t) kind * P.g_experts + P.g_tile_e[tile];
        W.trellis = reinterpret_cast<const unsigned char*>(P.t_trellis[idx]);
        W.svh = reinterpret_cast<const __half*>(P.t_svh[idx]);
        W.c = reinterpret_cast<unsigned char*>(P.c) + (size_t) kind * P.M * P.n * (P.c_fp32 ? 4 : 2);
        W.xt = P.xt + (size_t) kind * P.M * P.k * 2;
        W.n_row = P.n;
        W.nb = (int) blockIdx.x - kind * bpk;
        m0 = P.g_tile_row0[tile];
        rows = min(P.g_tile_rows[tile], P.sub * TC_BM);
    }
    else
    {
        W = tc_slice<TC_BN>(P, blockIdx.x);
        m0 = (int) blockIdx.y * (P.sub * TC_BM);
        rows = min(P.sub * TC_BM, P.M - m0);
    }
    const int nb = W.nb;
    const int nsub = (rows + TC_BM - 1) / TC_BM;        // sub-tiles that hold any of them
    const int ksteps = P.k / TC_BK;
    const size_t tiles_n = (size_t) W.n_row >> 4;

    if (t == 0)
    {
        for (int i = 0; i < TC_A_SLOTS; ++i) { mbar_init(&a_full[i], 1); mbar_init(&a_free[i], 1); }
        for (int i = 0; i < TC_B_STAGES; ++i) { mbar_init(&b_full[i], TC_DECODE_WARPS / 2); mbar_init(&b_free[i], 1); }
        mbar_init(&bar_done, 1);
        fence_mbar_init();
        s_bad = 0;
    }
    __syncwarp();
    if (warp == 0)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&s_tmem)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    unsigned char* a_base = smem;
    unsigned char* b_base = smem + TC_A_SLOTS * a_bytes;

    bool ok = true;
    auto wait_bar = [&](uint64_t* bar, uint32_t parity)
    {
        if (!ok) return;
        bool done = false;
        for (unsigned spin = 0; spin < TC_SPIN_LIMIT && !done; ++spin)
        {
            done = mbar_try_wait(bar, parity);
            if (!done && (spin & 1023) == 1023 && s_bad) break;      // another role gave up: leave too
        }
        if (!done) { ok = false; s_bad = 1; }
    };
    // a whole warp waits: one lane polls (32 lanes polling one mbarrier word serialise in the
    // shared-memory pipe and delay every other thread's barrier operations), the rest take its word
    auto wait_bar_warp = [&](uint64_t* bar, uint32_t parity)
    {
        if (lane == 0) wait_bar(bar, parity);
        __syncwarp();
        ok = __shfl_sync(0xffffffffu, (int) ok, 0) != 0;
    };

    if (warp == 0)
    {
        // ---- fetch: one thread keeps both x~ stages full ----
        if (lane == 0)
        {
            for (int i = 0; i < ksteps && ok; ++i)
            {
                const int s = i % TC_A_SLOTS;
                // the stage is free once the MMAs of step i - 2 have read it
                if (i >= TC_A_SLOTS) wait_bar(&a_free[s], (uint32_t) (((i / TC_A_SLOTS) - 1) & 1));
                if (!ok) break;
                // a 128-token box of this k step is one contiguous run of 128-byte rows: one bulk copy
                // each (the rows of a ragged last box that do not exist are not copied; their
                // accumulator rows are never stored)
                mbar_expect_tx(&a_full[s], (uint32_t) rows * 128);
                const unsigned char* src = W.xt + (((size_t) i * P.M + m0) << 7);
                for (int sub = 0; sub < nsub; ++sub)
                    bulk_g2s(a_base + s * a_bytes + sub * (TC_BM * 128), src + ((size_t) sub * TC_BM << 7),
                             (uint32_t) min(TC_BM, rows - sub * TC_BM) * 128, &a_full[s]);
            }
        }
        __syncwarp();
    }
    else if (warp == 1)
    {
        // ---- MMA issue: one thread, nothing else on its plate ----
        if (lane == 0)
        {
            // instruction descriptor: D fp32, A/B fp16, both K-major, N = 128, M = 128
            constexpr uint32_t IDESC = (1u << 4) | ((uint32_t) (TC_BN >> 3) << 17) | ((uint32_t) (TC_BM >> 4) << 24);
            const uint64_t da0 = make_desc(smem_u32(a_base)), db0 = make_desc(smem_u32(b_base));
            for (int i = 0; i < ksteps && ok; ++i)
            {
                const int sa = i % TC_A_SLOTS, sb = i % TC_B_STAGES;
                wait_bar(&a_full[sa], (uint32_t) ((i / TC_A_SLOTS) & 1));
                wait_bar(&b_full[sb], (uint32_t) ((i / TC_B_STAGES) & 1));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // descriptors advance by byte offset >> 4 in their low (address) field
                const uint64_t da = da0 + (uint64_t) ((sa * a_bytes) >> 4), db = db0 + (uint64_t) ((sb * TC_B_BYTES) >> 4);
                for (int sub = 0; sub < nsub; ++sub)
                    #pragma unroll
                    for (int kk = 0; kk < TC_BK / 16; ++kk)
                        umma_f16(tmem + sub * TC_BN, da + (uint64_t) ((sub * (TC_BM * 128) + kk * 32) >> 4),
                                 db + (uint64_t) ((kk * 32) >> 4), IDESC, (i > 0 || kk > 0) ? 1u : 0u);
                umma_commit(&a_free[sa]);                   // arrive when these MMAs have read their operands
                umma_commit(&b_free[sb]);
                if (i == ksteps - 1) umma_commit(&bar_done);
            }
        }
        __syncwarp();
    }
    else
    {
        // ---- decode warps ----
        const int dw = (warp - 2) & 7;                     // tile column of the 128-column block
        const int grp = (warp - 2) >> 3;                   // this warp's steps: grp, grp + 2, ...
        const int gq = lane >> 2, pq = lane & 3;           // 32-weight piece of the tile, tile row of the step
        const unsigned char* src = W.trellis + ((size_t) pq * tiles_n + (size_t) nb * 8 + dw) * (32 * K) + gq * (4 * K);
        const size_t step_bytes = (size_t) 4 * tiles_n * (32 * K);
        // this lane's ring: slot s at pring + s * SLOT (a warp's lanes side by side inside a slot); a
        // lane only ever reads what it copied itself
        constexpr int PS = tc_p_stages(K);
        constexpr int SLOT = 32 * 4 * K;
        const uint32_t pring = smem_u32(smem + TC_A_SLOTS * a_bytes + TC_B_STAGES * TC_B_BYTES)
                             + (uint32_t) ((warp - 2) * PS * SLOT + lane * 4 * K);
        #pragma unroll
        for (int j = 0; j < PS - 1; ++j)
        {
            if (grp + 2 * j < ksteps) cp_async_chunk<K>(pring + j * SLOT, src + (size_t) (grp + 2 * j) * step_bytes);
            cp_async_commit();
        }
        int pslot = 0;
        for (int i = grp; i < ksteps && ok; i += 2)
        {
            cp_async_wait_n<PS - 2>();                  // this lane's words of step i have landed
            uint32_t w[K];
            load_chunk_s<K>(pring + pslot * SLOT, w);
            {
                // refill the slot read in this warp's previous step with the words of its step PS - 1 ahead
                const int nxt = i + 2 * (PS - 1), nslot = (pslot == 0) ? PS - 1 : pslot - 1;
                if (nxt < ksteps) cp_async_chunk<K>(pring + nslot * SLOT, src + (size_t) nxt * step_bytes);
                cp_async_commit();
                if (++pslot == PS) pslot = 0;
            }
            // the word in front of this lane's piece: the last word of the lane four below (ring)
            const uint32_t prev = __shfl_sync(0xffffffffu, w[K - 1], (lane + 28) & 31);

            // 32 weights: columns gq and gq+8 of the tile, k rows 0..15 of tile row pq
            uint32_t colA[8], colB[8];                     // packed pairs (k, k+1): words 0-3 = k 0..7, 4-7 = k 8..15
            auto decode_r = [&](auto rtag)
            {
                constexpr int R = decltype(rtag)::value;
                uint32_t s[8];
                states8<K, R>(w, prev, s);
                colA[R] = weights2<CB>(s[0], s[1]);     colA[4 + R] = weights2<CB>(s[2], s[3]);
                colB[R] = weights2<CB>(s[4], s[5]);     colB[4 + R] = weights2<CB>(s[6], s[7]);
            };
            decode_r(std::integral_constant<int, 0>()); decode_r(std::integral_constant<int, 1>());
            decode_r(std::integral_constant<int, 2>()); decode_r(std::integral_constant<int, 3>());

            const int sb = i % TC_B_STAGES;
            if (i >= TC_B_STAGES) wait_bar_warp(&b_free[sb], (uint32_t) (((i / TC_B_STAGES) - 1) & 1));
            if (!ok) break;
            unsigned char* b = b_base + sb * TC_B_BYTES;
            const int ncol = dw * 16 + gq;
            *reinterpret_cast<uint4*>(b + sw128(ncol, 2 * pq)) = make_uint4(colA[0], colA[1], colA[2], colA[3]);
            *reinterpret_cast<uint4*>(b + sw128(ncol, 2 * pq + 1)) = make_uint4(colA[4], colA[5], colA[6], colA[7]);
            *reinterpret_cast<uint4*>(b + sw128(ncol + 8, 2 * pq)) = make_uint4(colB[0], colB[1], colB[2], colB[3]);
            *reinterpret_cast<uint4*>(b + sw128(ncol + 8, 2 * pq + 1)) = make_uint4(colB[4], colB[5], colB[6], colB[7]);
            // make the generic-proxy writes visible to the tensor core, then one arrival per warp
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&b_full[sb]);
        }
    }

    // ---- epilogue ----
    if (warp >= 2 && lane == 0) wait_bar(&bar_done, 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    const bool all_ok = !s_bad;

    float* tile = reinterpret_cast<float*>(smem);        // [128][132] fp32, reuses the pipeline stages
    constexpr int TP = 132;
    const int ew = warp - 2;                             // epilogue warp 0..15 (warps 0 and 1 only keep the barriers company)
    for (int sub = 0; sub < nsub; ++sub)
    {
        if (all_ok && warp >= 2)
        {
            // a warp may read the tensor-memory lanes 32*(warp%4)..+31 (token rows); the two warps
            // of a lane group split the 128 columns of this accumulator
            const int lg = warp & 3, ch = ew >> 2;          // lane group, 32-column quarter of this accumulator
            const int lrow = 32 * lg + lane;
            {
                const int col0 = 32 * ch;
                const uint32_t taddr = tmem + ((uint32_t) (32 * lg) << 16) + (uint32_t) (sub * TC_BN + col0);
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
        if (all_ok && warp >= 2)
        {
            const half4 sv = reinterpret_cast<const half4*>(W.svh + (size_t) nb * 128)[lane];
            for (int r = ew; r < TC_BM; r += TC_DECODE_WARPS)
            {
                const int grow = m0 + sub * TC_BM + r;
                if (sub * TC_BM + r >= rows) break;
                const float4 v = *reinterpret_cast<const float4*>(tile + r * TP + lane * 4);
                float h0 = v.x, h1 = v.y, h2 = v.z, h3 = v.w;
                warp_had128(h0, h1, h2, h3, lane);
                h0 *= kRScale; h1 *= kRScale; h2 *= kRScale; h3 *= kRScale;
                if (P.c_fp32)
                {
                    float4 o = make_float4(h0 * __low2float(sv.x), h1 * __high2float(sv.x),
                                           h2 * __low2float(sv.y), h3 * __high2float(sv.y));
                    reinterpret_cast<float4*>(reinterpret_cast<float*>(W.c) + (size_t) grow * W.n_row + (size_t) nb * 128)[lane] = o;
                }
                else
                {
                    half4 o;
                    o.x = __hmul2(__floats2half2_rn(h0, h1), sv.x);
                    o.y = __hmul2(__floats2half2_rn(h2, h3), sv.y);
                    reinterpret_cast<half4*>(reinterpret_cast<__half*>(W.c) + (size_t) grow * W.n_row + (size_t) nb * 128)[lane] = o;
                }
            }
        }
        __syncthreads();
    }

    if (t == 0 && !all_ok) atomicExch(P.status, 1);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(tmem_cols) : "memory");
}

// ------------------------------------------------------------------------------------------
// Pair form: two CTAs of a cluster (two SMs) work on 512 tokens x 256 columns with
// tcgen05.mma.cta_group::2 (M = 256: 128 token rows per CTA and sub-tile; N = 256: each CTA decodes
// 128 of the columns into its own shared memory and the tensor cores of both SMs read both
// halves). Per flop a CTA fetches half the x~ bytes and decodes half the weights of the single-CTA
// kernel above, and one issuing thread feeds two SMs.
//
// Roles per CTA as above. What a cycle-stamped lab build showed, and the structure that follows:
//   * the thread that issues the MMAs is the critical resource: every barrier operation of that
//     thread costs a few hundred cycles through the busy shared-memory pipe. So a stage holds the
//     x~ tile AND the weight tile of a k step and is freed by ONE tcgen05.commit that arrives in
//     both CTAs; the thread waits on two local barriers per step and polls the next step's
//     barriers (non-blocking) before it issues this step's MMAs, so that the answer is there by
//     the time it reaches that step;
//   * decode warps arrive on a barrier of their own CTA. A remote arrival with cluster-scope
//     release took 1000-2000 cycles (it waits for what the SM has in flight); one relay thread per
//     pair (the peer's warp 1) tells the first CTA "my x~ and my columns are ready" with a single,
//     relaxed remote arrival per step (see mbar_arrive_cluster);
//   * one lane of a decode warp polls for the free stage, the other 31 take its word;
//   * two threads issue the MMAs, one per 128-token sub-tile (each sub-tile has its own
//     accumulator, so the two streams need no order between them); both commit on the stage's
//     barrier, which therefore counts two arrivals where a CTA has two sub-tiles;
//   * tensor memory is allocated and freed by warp 0 of both CTAs with the cta_group::2 forms.
// ------------------------------------------------------------------------------------------
constexpr int T2_SUB = 2;                                  // 128-token sub-tiles per CTA
constexpr int T2_A_BYTES = T2_SUB * TC_BM * TC_BK * 2;     // x~ of one k step, this CTA's 256 tokens: 32768
constexpr int T2_B_BYTES = 128 * TC_BK * 2;                // this CTA's half of the 256-column B tile: 16384
// A stage holds the x~ tile and the decoded weight tile of one k step and is freed by ONE commit.
// Four stages where the packed-word rings leave room, three above 5 bits per weight.
__host__ __device__ constexpr int t2_stages(int K) { return K <= 5 ? 4 : 3; }
__host__ __device__ constexpr int t2_p_stages(int K) { return K <= 4 ? 4 : 3; }
__host__ __device__ constexpr int tc2_smem_bytes(int K)
{
    return 1024 + t2_stages(K) * (T2_A_BYTES + T2_B_BYTES) + TC_DECODE_WARPS * t2_p_stages(K) * 128 * K;
}
static_assert(tc2_smem_bytes(5) <= 232448 && tc2_smem_bytes(8) <= 232448 && tc2_smem_bytes(4) <= 232448, "pair kernel stages must fit 227 KB");
constexpr int T2_MAX_STAGES = 4;
// MMA-issuing threads in the first CTA: one per 128-token sub-tile (each with its own accumulator),
// in warps 1 and 18, so that the two instruction streams run on different schedulers
#ifndef AMP_T2_ISSUERS
#define AMP_T2_ISSUERS 2
#endif
constexpr int T2_ISSUERS = AMP_T2_ISSUERS;
constexpr int T2_THREADS = TC_THREADS + (T2_ISSUERS > 1 ? 32 : 0);

__device__ __forceinline__ uint32_t cluster_addr(const void* p, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
    return r;
}

// The relay's arrival on the first CTA's barrier. Relaxed on purpose: with release semantics at
// cluster scope this one instruction took well over a thousand cycles (it waits for everything the
// SM has in flight), and since the relay thread sends one per k step, in order, it set the pace of
// the whole pair: 690 -> 793 TFLOP/s on a 4096 x 4096 weight when it was relaxed. What the arrival
// publishes is already in place when it is sent: the x~ bytes were written by the bulk copy whose
// completion the relay observed with an acquire, the weight tile by warps that each ran
// fence.proxy.async and a releasing arrive on the barrier the relay acquired; both live in this
// SM's shared memory, which is read in place by the pair's tensor cores and cached nowhere.
// This leans on a property of the hardware, not on a rule of the PTX memory model: on paper the
// relay's acquire of its own barriers and the first CTA's acquire of this arrival are only
// chained into one causality order if the arrival releases (or a fence.acq_rel.cluster stands in
// front of it). `release` selects that form at run time (amp_exl3_set_gemm_relay_release); a test
// runs the benchmark's shapes in both forms, twelve launches each, and requires identical bits.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar, int release)
{
    if (release) asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(cluster_bar) : "memory");
    else asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" :: "r"(cluster_bar) : "memory");
}

// Arrives, once every tcgen05.mma issued so far by this thread has completed, on the barrier at
// this shared-memory offset in BOTH CTAs of the pair. One instruction (an arrival multicast, not a
// load); AMP_T2_TWO_COMMITS selects two unicast commits instead (measured 4-5 % slower: the
// issuing thread's instruction stream is the critical resource of this kernel).
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar)
{
#ifndef AMP_T2_TWO_COMMITS
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 :: "r"(smem_u32(bar)), "h"((unsigned short) 3) : "memory");
#else
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(cluster_addr(bar, 0)) : "memory");
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(cluster_addr(bar, 1)) : "memory");
#endif
}

// One k step of one sub-tile as a single instruction sequence: the non-blocking polls of the NEXT
// step's two barriers go out first, then the four MMAs of the 128-token sub-tile (k = 16 each:
// the descriptors advance by 32 bytes = 2 units), and only then are the polls' predicates turned
// into values. Written as one asm block because a predicate cannot leave one:
// with the polls in blocks of their own the thread sat out each poll's latency through the
// shared-memory pipe before it issued the first MMA.
#define AMP_UMMA2(d, a, b, p) "tcgen05.mma.cta_group::2.kind::f16 [" d "], " a ", " b ", %5, {%10, %10, %10, %10, %10, %10, %10, %10}, " p ";\n\t"
#define AMP_UMMA2_HEAD \
        "{\n\t" \
        ".reg .pred pa, pb, pacc, pone;\n\t" \
        ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t" \
        "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 pa, [%7], %9;\n\t" \
        "mbarrier.test_wait.parity.shared::cta.b64 pb, [%8], %9;\n\t" \
        "setp.ne.b32 pacc, %6, 0;\n\t" \
        "setp.eq.b32 pone, %10, 0;\n\t" \
        "add.u64 a1, %3, 2;\n\t"  "add.u64 a2, %3, 4;\n\t"  "add.u64 a3, %3, 6;\n\t" \
        "add.u64 b1, %4, 2;\n\t"  "add.u64 b2, %4, 4;\n\t"  "add.u64 b3, %4, 6;\n\t" \
        AMP_UMMA2("%2", "%3", "%4", "pacc") AMP_UMMA2("%2", "a1", "b1", "pone") \
        AMP_UMMA2("%2", "a2", "b2", "pone") AMP_UMMA2("%2", "a3", "b3", "pone")
#define AMP_UMMA2_TAIL \
        "selp.u32 %0, 1, 0, pa;\n\t" \
        "selp.u32 %1, 1, 0, pb;\n\t" \
        "}"
__device__ __forceinline__ void umma2_step(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate,
                                           uint32_t next_a_bar, uint32_t next_b_bar, uint32_t next_parity,
                                           uint32_t& next_a_ready, uint32_t& next_b_ready)
{
    asm volatile(AMP_UMMA2_HEAD AMP_UMMA2_TAIL
        : "=r"(next_a_ready), "=r"(next_b_ready)
        : "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(next_a_bar), "r"(next_b_bar), "r"(next_parity), "r"(0u)
        : "memory");
}
#undef AMP_UMMA2
#undef AMP_UMMA2_HEAD
#undef AMP_UMMA2_TAIL

__device__ __forceinline__ void cluster_barrier()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int K, int CB>
__global__ __launch_bounds__(T2_THREADS, 1)
void exl3_gemm_tc2_kernel(const TcParams P)
{
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    // a_land: this CTA's x~ bytes of a stage have landed; b_full: this CTA's eight decode warps of
    // the step have published their columns. In the first CTA a_land also counts one arrival from
    // the peer's relay thread, sent when BOTH of the peer's barriers have completed, so the issuing
    // thread learns about all four operand pieces from two local barriers and the pair exchanges
    // one remote arrival per step. st_free: the MMAs that read the stage have completed (one
    // commit, both CTAs).
    __shared__ uint64_t a_land[T2_MAX_STAGES], b_full[T2_MAX_STAGES], st_free[T2_MAX_STAGES], bar_done;
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_bad;
    constexpr int S = t2_stages(K);

    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    uint32_t crank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
    const bool leader = crank == 0;
    const TcSlice W = tc_slice<256>(P, blockIdx.x >> 1);
    const int nb = W.nb, mb = blockIdx.y;                  // 256-column block, 512-token block of the pair
    const int cta_rows = P.sub * TC_BM;                    // token rows per CTA: 256, or 128 for short grids
    const int m0 = mb * (2 * cta_rows) + (int) crank * cta_rows;
    const int rows = max(0, min(cta_rows, P.M - m0));               // valid token rows of this CTA (the peer may have none)
    const int nsub = (rows + TC_BM - 1) / TC_BM;
    const int rows_lead = min(cta_rows, P.M - mb * (2 * cta_rows));
    const int nsub_mma = (rows_lead + TC_BM - 1) / TC_BM;           // sub-tiles the pair multiplies (the first CTA's count)
    const int n_issuers = (T2_ISSUERS > 1 && nsub_mma > 1) ? 2 : 1;   // threads that issue MMAs and commit (same value in both CTAs)
    const int ksteps = P.k / TC_BK;
    const size_t tiles_n = (size_t) W.n_row >> 4;

    if (t == 0)
    {
        for (int i = 0; i < S; ++i)
        {
            mbar_init(&a_land[i], leader ? 2 : 1);
            mbar_init(&b_full[i], TC_DECODE_WARPS / 2);
            mbar_init(&st_free[i], n_issuers);
        }
        mbar_init(&bar_done, n_issuers);
        fence_mbar_init();
        s_bad = 0;
    }
    __syncwarp();
    if (warp == 0)
    {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&s_tmem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_barrier();                                     // both CTAs' barriers exist before anyone arrives remotely
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    unsigned char* a_base = smem;
    unsigned char* b_base = smem + S * T2_A_BYTES;

    bool ok = true;
    auto wait_bar = [&](uint64_t* bar, uint32_t parity)
    {
        if (!ok) return;
        bool done = false;
        for (unsigned spin = 0; spin < TC_SPIN_LIMIT && !done; ++spin)
        {
            done = mbar_try_wait(bar, parity);
            if (!done && (spin & 1023) == 1023 && s_bad) break;
        }
        if (!done) { ok = false; s_bad = 1; }
    };
    // a whole warp waits: one lane polls (32 lanes polling one mbarrier word serialise in the
    // shared-memory pipe and delay every other thread's barrier operations), the rest take its word
    auto wait_bar_warp = [&](uint64_t* bar, uint32_t parity)
    {
        if (lane == 0) wait_bar(bar, parity);
        __syncwarp();
        ok = __shfl_sync(0xffffffffu, (int) ok, 0) != 0;
    };
    // The three single threads that drive the pipeline (fetch, MMA issue, relay) poll without
    // parking: a thread parked in try_wait was seen to sleep on for up to ~1000 cycles after an
    // arrival that came from the tensor core, a bulk copy or the other CTA. Cluster-scope acquire,
    // since those arrivals may come from the peer.
    auto wait_bar_spin = [&](uint64_t* bar, uint32_t parity)
    {
        if (!ok) return;
        bool done = false;
        for (unsigned spin = 0; spin < TC_SPIN_LIMIT && !done; ++spin)
        {
            uint32_t r;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(r) : "r"(smem_u32(bar)), "r"(parity) : "memory");
            done = r != 0;
            if (!done && (spin & 1023) == 1023 && s_bad) break;
        }
        if (!done) { ok = false; s_bad = 1; }
    };

    if (warp == 0)
    {
        // ---- fetch ----
        if (lane == 0)
        {
            int s = 0; uint32_t ph = 1;                    // stage, parity of "freed for the (use)-th time" - first pass needs no wait
            // launched as a programmatic dependent of the rotation kernel: everything up to here
            // (tensor-memory allocation, barriers, the decode warps' first weight copies) ran under
            // that kernel; its output is read from here on
            // (only this thread waits: every other role consumes what it fetches. Any new read of
            // the rotation kernel's output by another thread must come after a wait of its own.)
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int i = 0; i < ksteps && ok; ++i)
            {
                if (i >= S) wait_bar_spin(&st_free[s], ph);
                if (!ok) break;
                mbar_expect_tx(&a_land[s], (uint32_t) rows * 128);
                const unsigned char* src = W.xt + (((size_t) i * P.M + m0) << 7);
                for (int sub = 0; sub < nsub; ++sub)
                    bulk_g2s(a_base + s * T2_A_BYTES + sub * (TC_BM * 128), src + ((size_t) sub * TC_BM << 7),
                             (uint32_t) min(TC_BM, rows - sub * TC_BM) * 128, &a_land[s]);
                if (++s == S) { s = 0; ph ^= 1; }
            }
        }
        __syncwarp();
    }
    else if (warp == 1 || warp == 18)
    {
        // ---- MMA issue for the pair: per k step two waits, four MMAs per sub-tile, one commit ----
        // `which` = the sub-tile (and accumulator) this thread owns; with one issuer it owns both
        auto issue_loop = [&](const int which)
        {
            // instruction descriptor: D fp32, A/B fp16, both K-major, N = 256, M = 256 (pair)
            constexpr uint32_t IDESC = (1u << 4) | ((uint32_t) (256 >> 3) << 17) | ((uint32_t) (256 >> 4) << 24);
            constexpr uint32_t SUB_DESC = (TC_BM * 128) >> 4;
            const uint64_t da0 = make_desc(smem_u32(a_base)), db0 = make_desc(smem_u32(b_base));
            const bool has0 = which == 0;                                          // this thread multiplies sub-tile 0
            const bool has1 = (n_issuers == 1 || which == 1) && nsub_mma > 1;      // ... sub-tile 1
            int s = 0; uint32_t ph = 0;
            uint32_t ra = 0, rb = 0;                       // this step's barriers were seen complete by the look-ahead poll
            for (int i = 0; i < ksteps && ok; ++i)
            {
                if (!ra) wait_bar_spin(&a_land[s], ph);
                if (!rb) wait_bar_spin(&b_full[s], ph);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // Look-ahead: the NEXT step's barriers are polled (non-blocking) in the same
                // instruction sequence as this step's MMAs. The decode warps and the fetch run
                // stages ahead, so the answer is almost always yes and the waits above are skipped.
                const int s2 = (s + 1 == S) ? 0 : s + 1;
                const uint32_t ph2 = (s + 1 == S) ? ph ^ 1 : ph;
                const uint64_t da = da0 + (uint64_t) ((s * T2_A_BYTES) >> 4), db = db0 + (uint64_t) ((s * T2_B_BYTES) >> 4);
                const uint32_t acc = i > 0 ? 1u : 0u;
                const uint32_t na = smem_u32(&a_land[s2]), nbar = smem_u32(&b_full[s2]);
                ra = rb = 0;
                if (has0) umma2_step(tmem, da, db, IDESC, acc, na, nbar, ph2, ra, rb);
                if (has1) umma2_step(tmem + 256, da + SUB_DESC, db, IDESC, acc, na, nbar, ph2, ra, rb);
                umma2_commit_both(&st_free[s]);            // the stage is free in BOTH CTAs once every issuer's MMAs have read it
                if (i == ksteps - 1) umma2_commit_both(&bar_done);
                if (++s == S) { s = 0; ph ^= 1; }
            }
        };
        if (lane == 0)
        {
            if (leader)
            {
                if (warp == 1) issue_loop(0);
                else if (n_issuers > 1) issue_loop(1);
            }
            else if (warp == 1)
            {
                // ---- relay: tell the first CTA that this CTA's halves of the stage are ready ----
                int s = 0; uint32_t ph = 0;
                for (int i = 0; i < ksteps && ok; ++i)
                {
                    wait_bar_spin(&a_land[s], ph);
                    wait_bar_spin(&b_full[s], ph);
                    if (!ok) break;
                    mbar_arrive_cluster(cluster_addr(&a_land[s], 0), P.relay_release);
                    if (++s == S) { s = 0; ph ^= 1; }
                }
            }
        }
        __syncwarp();
    }
    else
    {
        // ---- decode warps: this CTA's 128 columns of the pair's 256 ----
        const int dw = (warp - 2) & 7;
        const int grp = (warp - 2) >> 3;
        const int gq = lane >> 2, pq = lane & 3;
        const unsigned char* src = W.trellis + ((size_t) pq * tiles_n + (size_t) nb * 16 + crank * 8 + dw) * (32 * K) + gq * (4 * K);
        const size_t step_bytes = (size_t) 4 * tiles_n * (32 * K);
        constexpr int PS = t2_p_stages(K);
        constexpr int SLOT = 32 * 4 * K;
        const uint32_t pring = smem_u32(smem + S * (T2_A_BYTES + T2_B_BYTES)) + (uint32_t) ((warp - 2) * PS * SLOT + lane * 4 * K);
        #pragma unroll
        for (int j = 0; j < PS - 1; ++j)
        {
            if (grp + 2 * j < ksteps) cp_async_chunk<K>(pring + j * SLOT, src + (size_t) (grp + 2 * j) * step_bytes);
            cp_async_commit();
        }
        int pslot = 0;
        for (int i = grp; i < ksteps && ok; i += 2)
        {
            uint32_t w[K];
            cp_async_wait_n<PS - 2>();
            load_chunk_s<K>(pring + pslot * SLOT, w);
            const uint32_t prev = __shfl_sync(0xffffffffu, w[K - 1], (lane + 28) & 31);
            uint32_t colA[8], colB[8];
            auto decode_r = [&](auto rtag)
            {
                constexpr int R = decltype(rtag)::value;
                uint32_t s[8];
                states8<K, R>(w, prev, s);
                colA[R] = weights2<CB>(s[0], s[1]);     colA[4 + R] = weights2<CB>(s[2], s[3]);
                colB[R] = weights2<CB>(s[4], s[5]);     colB[4 + R] = weights2<CB>(s[6], s[7]);
            };
            decode_r(std::integral_constant<int, 0>()); decode_r(std::integral_constant<int, 1>());
            decode_r(std::integral_constant<int, 2>()); decode_r(std::integral_constant<int, 3>());

            const int sb = i % S;
            if (i >= S) wait_bar_warp(&st_free[sb], (uint32_t) (((i / S) - 1) & 1));
            if (!ok) break;
            unsigned char* b = b_base + sb * T2_B_BYTES;
            const int ncol = dw * 16 + gq;
            *reinterpret_cast<uint4*>(b + sw128(ncol, 2 * pq)) = make_uint4(colA[0], colA[1], colA[2], colA[3]);
            *reinterpret_cast<uint4*>(b + sw128(ncol, 2 * pq + 1)) = make_uint4(colA[4], colA[5], colA[6], colA[7]);
            *reinterpret_cast<uint4*>(b + sw128(ncol + 8, 2 * pq)) = make_uint4(colB[0], colB[1], colB[2], colB[3]);
            *reinterpret_cast<uint4*>(b + sw128(ncol + 8, 2 * pq + 1)) = make_uint4(colB[4], colB[5], colB[6], colB[7]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&b_full[sb]);
            {
                // refill the slot read in this warp's previous step with the words of its step PS - 1
                // ahead. Issued after the arrival: the arrival's release must not find this warp's
                // newest copies still on their way from HBM.
                const int nxt = i + 2 * (PS - 1), nslot = (pslot == 0) ? PS - 1 : pslot - 1;
                if (nxt < ksteps) cp_async_chunk<K>(pring + nslot * SLOT, src + (size_t) nxt * step_bytes);
                cp_async_commit();
                if (++pslot == PS) pslot = 0;
            }
        }
    }

    // ---- epilogue: each CTA stores its own 256 tokens x 256 columns ----
    const bool dec_warp = warp >= 2 && warp < 2 + TC_DECODE_WARPS;
    if (dec_warp && lane == 0) wait_bar(&bar_done, 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    const bool all_ok = !s_bad;

    // two [128][132] fp32 tiles in the pipeline's stages, used alternately: a warp that has
    // finished the rows of one pass goes straight on to unload the next accumulator block into
    // the other tile, one block-wide barrier per pass
    constexpr int TP = 132;
    const int ew = warp - 2;
    int pass = 0;
    for (int sub = 0; sub < nsub; ++sub)
    for (int hb = 0; hb < 2; ++hb, ++pass)               // the two 128-column Hadamard blocks of the pair's 256 columns
    {
        float* tile = reinterpret_cast<float*>(smem) + (pass & 1) * (TC_BM * TP);
        if (all_ok && dec_warp)
        {
            const int lg = warp & 3, ch = ew >> 2;
            const int lrow = 32 * lg + lane;
            const int col0 = 32 * ch;
            const uint32_t taddr = tmem + ((uint32_t) (32 * lg) << 16) + (uint32_t) (sub * 256 + hb * 128 + col0);
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
        __syncthreads();
        if (all_ok && dec_warp)
        {
            const size_t cblk = (size_t) nb * 256 + (size_t) hb * 128;
            const half4 sv = reinterpret_cast<const half4*>(W.svh + cblk)[lane];
            for (int r = ew; r < TC_BM; r += TC_DECODE_WARPS)
            {
                const int grow = m0 + sub * TC_BM + r;
                if (sub * TC_BM + r >= rows) break;
                const float4 v = *reinterpret_cast<const float4*>(tile + r * TP + lane * 4);
                float h0 = v.x, h1 = v.y, h2 = v.z, h3 = v.w;
                warp_had128(h0, h1, h2, h3, lane);
                h0 *= kRScale; h1 *= kRScale; h2 *= kRScale; h3 *= kRScale;
                if (P.c_fp32)
                {
                    float4 o = make_float4(h0 * __low2float(sv.x), h1 * __high2float(sv.x),
                                           h2 * __low2float(sv.y), h3 * __high2float(sv.y));
                    reinterpret_cast<float4*>(reinterpret_cast<float*>(W.c) + (size_t) grow * W.n_row + cblk)[lane] = o;
                }
                else
                {
                    half4 o;
                    o.x = __hmul2(__floats2half2_rn(h0, h1), sv.x);
                    o.y = __hmul2(__floats2half2_rn(h2, h3), sv.y);
                    reinterpret_cast<half4*>(reinterpret_cast<__half*>(W.c) + (size_t) grow * W.n_row + cblk)[lane] = o;
                }
            }
        }
    }

    if (t == 0 && !all_ok) atomicExch(P.status, 1);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_barrier();                                     // neither CTA leaves while the other may still use its memory
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(512u) : "memory");
}

typedef void (*tc_fn)(const TcParams);

#define AMP_TC_ROW(cb) { exl3_gemm_tc_kernel<1, cb>, exl3_gemm_tc_kernel<2, cb>, exl3_gemm_tc_kernel<3, cb>, exl3_gemm_tc_kernel<4, cb>, \
                         exl3_gemm_tc_kernel<5, cb>, exl3_gemm_tc_kernel<6, cb>, exl3_gemm_tc_kernel<7, cb>, exl3_gemm_tc_kernel<8, cb> }
static const tc_fn k_tc[3][8] = { AMP_TC_ROW(0), AMP_TC_ROW(1), AMP_TC_ROW(2) };
#undef AMP_TC_ROW
#define AMP_TCG_ROW(cb) { exl3_gemm_tc_kernel<1, cb, true>, exl3_gemm_tc_kernel<2, cb, true>, exl3_gemm_tc_kernel<3, cb, true>, \
                          exl3_gemm_tc_kernel<4, cb, true>, exl3_gemm_tc_kernel<5, cb, true>, exl3_gemm_tc_kernel<6, cb, true>, \
                          exl3_gemm_tc_kernel<7, cb, true>, exl3_gemm_tc_kernel<8, cb, true> }
static const tc_fn k_tcg[3][8] = { AMP_TCG_ROW(0), AMP_TCG_ROW(1), AMP_TCG_ROW(2) };
#undef AMP_TCG_ROW
#define AMP_TC2_ROW(cb) { exl3_gemm_tc2_kernel<1, cb>, exl3_gemm_tc2_kernel<2, cb>, exl3_gemm_tc2_kernel<3, cb>, exl3_gemm_tc2_kernel<4, cb>, \
                          exl3_gemm_tc2_kernel<5, cb>, exl3_gemm_tc2_kernel<6, cb>, exl3_gemm_tc2_kernel<7, cb>, exl3_gemm_tc2_kernel<8, cb> }
static const tc_fn k_tc2[3][8] = { AMP_TC2_ROW(0), AMP_TC2_ROW(1), AMP_TC2_ROW(2) };
#undef AMP_TC2_ROW
int g_tc_relay_release = 0;
int g_tc_pair = 1;        // pair (cta_group::2) form: 0 never, 1 where it fills the device, 2 whenever n % 256 == 0

// tiled x~ (launch_had_tiled) -> C. Called by amp_exl3_gemm for m > 16, and by amp_exl3_mgemm
// with T set: then `n` is the width of one slice, the grid covers T->num slices, and trellis / svh
// (and c when T->c is given) are ignored in favour of the tables.
int launch_gemm_tc(const void* xh, const void* trellis, void* c, const void* svh, int M, int k, int n,
                   int K, int cb, int c_fp32, cudaStream_t stream, const TcTables* T)
{
    AMP_REQUIRE(xh && (T || (trellis && c && svh)), "exl3_gemm: null pointer");
    AMP_REQUIRE(!T || (T->num >= 1 && T->trellis && T->svh && (T->c || c)), "exl3_mgemm: pointer tables are required");
    AMP_REQUIRE(K >= 1 && K <= 8 && cb >= 0 && cb <= 2, "exl3_gemm: unsupported bitrate / codebook");
    AMP_REQUIRE(M >= 1 && k % 128 == 0 && n % 128 == 0 && k > 0 && n > 0, "exl3_gemm: k and n must be multiples of 128");
    AMP_REQUIRE(((uintptr_t) xh & 15) == 0 && ((uintptr_t) trellis & 15) == 0 && ((uintptr_t) c & 15) == 0 &&
                ((uintptr_t) svh & 7) == 0, "exl3_gemm: misaligned pointer");
    const long slices = T ? T->num : 1;
    AMP_REQUIRE(slices * (n / 128) <= 0x3fffffffL, "exl3_gemm: too many column blocks");
    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev)) return cuda_rc(e, "cudaGetDevice");
    tc_fn fn = k_tc[cb][K - 1];
    const int smem_bytes = tc_smem_bytes(K);
    if (cudaError_t e = ensure_smem(fn, smem_bytes, dev)) return cuda_rc(e, "exl3_gemm smem attribute");

    TcParams P;
    P.xt = (const unsigned char*) xh; P.trellis = (const uint16_t*) trellis; P.svh = (const __half*) svh; P.c = c;
    P.M = M; P.k = k; P.n = n; P.c_fp32 = c_fp32;
    P.tables = T ? 1 : 0;
    P.relay_release = g_tc_relay_release;
    P.t_trellis = T ? T->trellis : nullptr; P.t_svh = T ? T->svh : nullptr; P.t_c = T ? T->c : nullptr;
    P.t_stride = T ? T->stride : nullptr; P.t_src = T ? T->src : nullptr;
    {
        // address of the status word, looked up once per device (under a lock: two host threads
        // may make their first launch on a device at the same time)
        static int* status_ptr[64] = {};
        static std::mutex status_mu;
        std::lock_guard<std::mutex> lock(status_mu);
        int*& sp = status_ptr[dev & 63];
        if (!sp)
            if (cudaError_t e = cudaGetSymbolAddress((void**) &sp, g_tc_status)) return cuda_rc(e, "status symbol");
        P.status = sp;
    }
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // pair form (two CTAs per 256-column block) for every weight it can tile. That includes
    // batches of 17..256 tokens, where the second CTA of a pair may hold no token at all and only
    // contributes its half of the decode: 64 tokens x 14336 x 4096 0.198 -> 0.134 ms, 256 tokens x
    // 4096 x 14336 0.128 -> 0.059 ms against the single-CTA form.
    if (g_tc_pair && n % 256 == 0)
    {
        // 256 token rows per CTA amortise the decode best, but a pair's k loop takes about as long
        // with 128: where the 128-row grid still fits one wave of CTA pairs it halves the time
        // (measured: 2048 x 4096 x 1024 0.080 -> 0.068 ms, 1024 x 4096 x 4096 0.073 -> 0.060 ms,
        // against 0.082 / 0.084 ms for the single-CTA form), beyond one wave it doubles the waves.
        const long pairs128 = slices * (n / 256) * (((long) M + 255) / 256);
        const int psub = g_tc_pair == 3 ? 1 : (g_tc_pair == 2 ? T2_SUB : (pairs128 <= sms / 2 ? 1 : T2_SUB));
        const long mblk = ((long) M + 256 * psub - 1) / (256 * psub);
        if (mblk <= 65535)
        {
            tc_fn fn2 = k_tc2[cb][K - 1];
            const int smem2 = tc2_smem_bytes(K);
            if (cudaError_t e = ensure_smem(fn2, smem2, dev)) return cuda_rc(e, "exl3_gemm smem attribute");
            P.sub = psub;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned) (2 * slices * (n / 256)), (unsigned) mblk, 1);
            cfg.blockDim = dim3(T2_THREADS, 1, 1);
            cfg.dynamicSmemBytes = smem2;
            cfg.stream = stream;
            cudaLaunchAttribute attr[2];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
            attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[1].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = g_pdl ? 2 : 1;
            return cuda_rc(cudaLaunchKernelEx(&cfg, fn2, P), "exl3_gemm_tc2 launch");
        }
    }
    // single-CTA form: 512 tokens per CTA amortise the decode best; with few column blocks that
    // leaves most SMs idle, so the token tile shrinks until the grid covers the device
    int sub = TC_SUB;
    while (sub > 1 && slices * (n / 128) * (((long) M + sub * TC_BM - 1) / (sub * TC_BM)) < (long) sms * 4 / 5) sub >>= 1;
    P.sub = sub;
    const long mblocks = ((long) M + sub * TC_BM - 1) / (sub * TC_BM);
    AMP_REQUIRE(mblocks <= 65535, "exl3_gemm: too many rows");
    dim3 grid((unsigned) (slices * (n / 128)), (unsigned) mblocks);
    fn<<<grid, TC_THREADS, smem_bytes, stream>>>(P);
    return cuda_rc(cudaGetLastError(), "exl3_gemm_tc launch");
}

// Expert-grouped form for token-sorted MoE prefill: xt / c are (kinds, Mcap, k / n) in the padded,
// expert-sorted row space, the tile table lives in device memory (see TcParams). One CTA per
// (tile, projection, 128-column block); the grid is sized for G.max_tiles and the surplus returns.
int launch_gemm_tc_grouped(const void* xt, void* c, long Mcap, int k, int n, int K, int cb, int c_fp32,
                           const long long* t_trellis, const long long* t_svh, const TcGroups& G, cudaStream_t stream)
{
    AMP_REQUIRE(xt && c && t_trellis && t_svh && G.ntiles && G.tile_e && G.tile_row0 && G.tile_rows, "exl3_moe_sorted: null pointer");
    AMP_REQUIRE(K >= 1 && K <= 8 && cb >= 0 && cb <= 2, "exl3_moe_sorted: unsupported bitrate / codebook");
    AMP_REQUIRE(Mcap >= 1 && Mcap <= 0x7fffffffL && k % 128 == 0 && n % 128 == 0 && k > 0 && n > 0, "exl3_moe_sorted: k and n must be multiples of 128");
    AMP_REQUIRE(((uintptr_t) xt & 15) == 0 && ((uintptr_t) c & 15) == 0, "exl3_moe_sorted: misaligned pointer");
    AMP_REQUIRE(G.kinds >= 1 && G.kinds <= 2 && G.sub >= 1 && G.sub <= TC_SUB && G.experts >= 1, "exl3_moe_sorted: bad grouping");
    AMP_REQUIRE(G.max_tiles >= 1 && G.max_tiles <= 65535, "exl3_moe_sorted: too many row tiles");
    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev)) return cuda_rc(e, "cudaGetDevice");
    tc_fn fn = k_tcg[cb][K - 1];
    // x~ slots sized by the rows per tile; never below the epilogue's 128 x 132 fp32 staging tile
    int smem_bytes = 1024 + TC_A_SLOTS * G.sub * (TC_BM * TC_BK * 2) + TC_B_STAGES * TC_B_BYTES + TC_DECODE_WARPS * tc_p_stages(K) * 128 * K;
    if (smem_bytes < 1024 + 128 * 132 * 4) smem_bytes = 1024 + 128 * 132 * 4;
    if (cudaError_t e = ensure_smem(fn, smem_bytes, dev)) return cuda_rc(e, "exl3_moe_sorted smem attribute");
    TcParams P = {};
    P.xt = (const unsigned char*) xt; P.c = c;
    P.M = (int) Mcap; P.k = k; P.n = n; P.c_fp32 = c_fp32; P.sub = G.sub;
    P.t_trellis = t_trellis; P.t_svh = t_svh;
    P.g_ntiles = G.ntiles; P.g_tile_e = G.tile_e; P.g_tile_row0 = G.tile_row0; P.g_tile_rows = G.tile_rows;
    P.g_experts = G.experts;
    P.g_bits[0] = G.bits[0]; P.g_bits[1] = G.bits[1];
    {
        static int* status_ptr[64] = {};
        static std::mutex status_mu;
        std::lock_guard<std::mutex> lock(status_mu);
        int*& sp = status_ptr[dev & 63];
        if (!sp)
            if (cudaError_t e = cudaGetSymbolAddress((void**) &sp, g_tc_status)) return cuda_rc(e, "status symbol");
        P.status = sp;
    }
    dim3 grid((unsigned) (G.kinds * (n / 128)), (unsigned) G.max_tiles);
    fn<<<grid, TC_THREADS, smem_bytes, stream>>>(P);
    return cuda_rc(cudaGetLastError(), "exl3_moe_sorted gemm launch");
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


// Chooses between the single-CTA and the pair (cta_group::2) form of the prefill GEMM: 0 = never
// the pair form, 1 = by shape (default: pairs whenever n is a multiple of 256, 128-token CTAs while
// that grid fits one wave, 256-token CTAs beyond), 2 / 3 = pairs of 256- / 128-token CTAs whenever
// n is a multiple of 256 (tests). Returns the previous setting.
// The pair form's remote arrival: 0 = relaxed (default), 1 = release at cluster scope (what the PTX
// memory model asks for on paper; measured 10-15 % slower). Returns the previous setting.
AMP_API int amp_exl3_set_gemm_relay_release(int enable)
{
    const int old = g_tc_relay_release;
    g_tc_relay_release = enable ? 1 : 0;
    return old;
}

AMP_API int amp_exl3_set_gemm_pair(int mode)
{
    const int old = g_tc_pair;
    g_tc_pair = mode < 0 ? 0 : (mode > 3 ? 3 : mode);
    return old;
}
