// Trellis-decode GEMV for decode batches of up to 8 rows on the 5th-generation tensor cores.
//
// Same job, work split and partial-sum exchange as exl3_gemv_kernel (exl3_gemv_kernel.cuh; the
// reference's exl3_gemv_kernel / exl3_gemm_kernel at small m / exl3_mgemm_kernel,
// vendor/exl3/exllamav3_ext/quant/exl3_gemv_kernel.cuh:186-482, exl3_gemm_kernel.cuh:8-343), but
// the dot product no longer goes through mma.sync. On sm_100 a legacy mma.sync m16n8k16 keeps the
// scheduler from issuing for about eight cycles, and at a quarter MMA per weight that was a
// third of the decode kernel's time (the decode itself is about 3.4 integer instructions per
// weight). Here
//
//   * the four warps write the decoded (lo, hi) fp16 words straight from registers into tensor
//     memory with tcgen05.st (shape 16x256b: exactly the fragment a lane holds after decoding a
//     16x16 tile): TMEM lane = output column, TMEM column = one weight row, so the decoded block
//     is the A operand (M = 128 output columns) of tcgen05.mma;
//   * a fifth warp's elected thread issues tcgen05.mma (M128 x N16 x K16, A from tensor memory, B =
//     the rotated activations from shared memory, fp32 accumulators in tensor memory): one
//     instruction per 1024 weights, asynchronous, no issue slot of the decode warps; it sleeps
//     in mbarrier.try_wait between stages;
//   * the codebook's final add still happens in the tensor core: the two halves of a word are
//     adjacent K elements against a duplicated activation.
//
// Tensor memory per CTA: 128 columns = 16 accumulator columns + three 32-column stages of A (a
// stage = half a unit = 32 weight rows x 128 columns). Stages are handed over with mbarriers
// (decode warps -> issuer: `full`; tcgen05.commit -> decode warps: `free`); every wait is bounded.
// A warp's tcgen05.st of one stage are only waited for (tcgen05.wait::st) after half of the next
// stage has been decoded, so their latency is covered by arithmetic.
// The rotated input x~ lives in shared memory in the K-major no-swizzle operand layout for eight
// batch rows (rows 8-15 of N alias rows 0-7), XG 64-row groups at a time in two buffers, so the
// next chunk is written while the MMAs of the current one still read theirs.
#pragma once
#include "exl3_gemv_kernel.cuh"

namespace amp {

constexpr int TCV_WARPS = 4;                   // decode warps; one more warp issues the MMAs
constexpr int TCV_THREADS = 32 * (TCV_WARPS + 1);
constexpr int TCV_NST = 3;                     // A stages in tensor memory
constexpr int TCV_TMEM_COLS = 128;
constexpr int TCV_D_COL = 0, TCV_A_COL = 16;   // accumulators, then the stages
constexpr int TCV_TB = 4;                      // x~ tasks (batch row, 128-row block) per warp and chunk
constexpr unsigned TCV_SPIN_LIMIT = 1u << 16;  // try_wait calls (each may sleep up to 16 us) before a wait is declared lost: about a second
constexpr int TCV_MAX_M = 8;
#ifndef TCV_MINBLOCKS
#define TCV_MINBLOCKS 4
#endif

__host__ __device__ constexpr int tcv_stages(int K) { return K <= 4 ? 7 : (K <= 6 ? 5 : 4); }

struct TcvSmem { int part, xb, gsum, ring, xchg, total; };

// xgroups: 64-row groups of x~ per chunk (even). One group of x~ is 2 KB: [8 MMAs][2 core
// matrices][8 batch rows][16 bytes].
__host__ __device__ inline TcvSmem tcv_smem_layout(int K, int m, int xgroups, int cluster = 0)
{
    TcvSmem L;
    L.part = 0;
    L.xb = (L.part + m * 128 * 4 + 127) & ~127;
    L.gsum = L.xb + 2 * xgroups * 2048;
    L.ring = (L.gsum + 2 * m * xgroups * 4 + 127) & ~127;
    L.xchg = L.ring + TCV_WARPS * tcv_stages(K) * gemv_slot_bytes(K);
    L.total = L.xchg + cluster * m * 128 * 4;
    return L;
}

__device__ __forceinline__ uint64_t tcv_bdesc(uint32_t saddr)
{
    // K-major, no swizzle: start address >> 4; leading (K direction) core-matrix stride 128 B;
    // stride between 8-row groups of N = 0 (batch rows 8-15 alias rows 0-7); descriptor version 1
    return (uint64_t) ((saddr & 0x3ffff) >> 4) | ((uint64_t) (128 >> 4) << 16) | (1ull << 46);
}

__device__ __forceinline__ void tcv_mma(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t accumulate)
{
    // D fp32, A/B fp16, both K-major, N = 16, M = 128
    constexpr uint32_t IDESC = (1u << 4) | ((uint32_t) (16 >> 3) << 17) | ((uint32_t) (128 >> 4) << 24);
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        :: "r"(tmem_d), "r"(tmem_a), "l"(db), "r"(IDESC), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void tcv_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}

__device__ __forceinline__ void tcv_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}

// Bounded wait for the phase of parity `parity` of an mbarrier: the already-complete case costs a
// try_wait and a branch. Returns false when the limit ran out.
__device__ __forceinline__ bool tcv_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .u32 n;\n\t"
        "mov.u32 n, %3;\n\t"
        "TCV_WAIT_LOOP:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 0x4000;\n\t"
        "@p bra TCV_WAIT_DONE;\n\t"
        "sub.u32 n, n, 1;\n\t"
        "setp.ne.u32 p, n, 0;\n\t"
        "@p bra TCV_WAIT_LOOP;\n\t"
        "setp.ne.u32 p, n, 0;\n\t"
        "TCV_WAIT_DONE:\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "n"(TCV_SPIN_LIMIT) : "memory");
    return ok != 0;
}

// one decoded tile fragment (this lane's eight words) -> tensor memory, 16 lanes x 16 columns
__device__ __forceinline__ void tcv_st_tile(uint32_t taddr, const uint32_t (&a)[8])
{
    // registers 0,1 / 2,3: lanes g, g+8 at columns 2p, 2p+1; registers 4,5 / 6,7: the same lanes at
    // columns 8+2p, 9+2p. Decoded positions 0..3 belong to tile column g (rows 2R, 2R+1, 2R+8,
    // 2R+9), positions 4..7 to tile column g+8.
    asm volatile("tcgen05.st.sync.aligned.16x256b.x2.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
        :: "r"(taddr), "r"(a[0]), "r"(a[1]), "r"(a[4]), "r"(a[5]), "r"(a[2]), "r"(a[3]), "r"(a[6]), "r"(a[7]) : "memory");
}

__device__ __forceinline__ void tcv_bar_decode()
{
    asm volatile("bar.sync 1, %0;" :: "n"(32 * TCV_WARPS) : "memory");
}

// AR: instance with the fused tensor-parallel all-reduce in the epilogue (P.ar)
template <int K, int CB, int AR>
__global__ __launch_bounds__(TCV_THREADS, TCV_MINBLOCKS)
void exl3_gemv_tc_kernel(const GemvParams P)
{
    extern __shared__ __align__(128) unsigned char smem[];
    const TcvSmem L = tcv_smem_layout(K, P.m, P.xgroups, P.cluster);
    const int XG = P.xgroups;
    float* part = reinterpret_cast<float*>(smem + L.part);
    unsigned char* xb = smem + L.xb;
    float* gsum = reinterpret_cast<float*>(smem + L.gsum);
    __shared__ uint64_t bar_full[TCV_NST], bar_free[TCV_NST], bar_d, bar_x[2];
    __shared__ uint32_t s_tmem;
    __shared__ int s_last;

    constexpr int S = tcv_stages(K);
    constexpr int RP = gemv_row_pitch(K);
    constexpr int SLOT = gemv_slot_bytes(K);
    constexpr int TILE_BYTES = 32 * K;
    constexpr int NT = GEMV_NT;
    constexpr int ROWP = NT * 2 * K;
    constexpr int PIECES = 4 * ROWP;
    constexpr int NP = (PIECES + 31) / 32;

    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int gq = lane >> 2, pq = lane & 3;
    const int m = P.m, k = P.k;
    const int G = k >> 6;
    const int nbw = P.width >> 7;

    const int U = P.blocks * G;
    const int cta = blockIdx.x, ncta = min((int) gridDim.x, U);
    if (cta >= ncta) return;
    GemvSplit split;
    split.q = U / ncta;
    split.r = U - split.q * ncta;
    const int u0 = split.begin(cta), u1 = split.begin(cta + 1);

    if (t == 0)
    {
        for (int i = 0; i < TCV_NST; ++i) { mbar_init(&bar_full[i], TCV_WARPS); mbar_init(&bar_free[i], 1); }
        mbar_init(&bar_d, 1);
        mbar_init(&bar_x[0], TCV_WARPS); mbar_init(&bar_x[1], TCV_WARPS);
        fence_mbar_init();
    }
    if (warp == TCV_WARPS)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&s_tmem)), "r"((uint32_t) TCV_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    // Dependent launch: only now, with this CTA's tensor memory in hand, may CTAs of the next
    // kernel be scheduled (they wait for this grid while holding theirs).
    if (P.pdl) pdl_launch_dependents();

    bool ok = true;                                  // false once a bounded wait ran out: no more waits
    auto wait_bar = [&](uint32_t bar, uint32_t parity)
    {
        if (ok && !tcv_wait(bar, parity)) { ok = false; atomicExch(P.status, 1); }
    };
    const uint32_t full_s = smem_u32(&bar_full[0]), free_s = smem_u32(&bar_free[0]), d_s = smem_u32(&bar_d), x_s = smem_u32(&bar_x[0]);

    // slice-dependent pointers of a column block
    auto slice_of = [&](int blk, const __half*& suh) -> int
    {
        const int slice = blk / nbw;
        suh = P.suh;
        if (P.tables) suh = reinterpret_cast<const __half*>(P.t_suh[P.t_src ? P.t_src[slice] : slice]);
        return slice;
    };


    if (warp == TCV_WARPS)
    {
        // ---------------- MMA issue: one thread mirrors the decode warps' walk ----------------
        if (lane == 0)
        {
            int st = 0; uint32_t wrap = 0; int ev = 0;
            int useg = u0;
            while (useg < u1 && ok)
            {
                const int blk = useg / G;
                const int g0 = useg - blk * G;
                const int g1 = min(G, g0 + (u1 - useg));
                uint32_t acc_flag = 0;
                for (int cg0 = (g0 / XG) * XG; cg0 < g1 && ok; cg0 += XG)
                {
                    const int cg1 = min(cg0 + XG, g1);
                    const int buf = ev & 1;
                    wait_bar(x_s + 8 * buf, (uint32_t) ((ev >> 1) & 1));
                    ++ev;
                    uint32_t xs = smem_u32(xb + buf * (XG * 2048)) + (max(cg0, g0) - cg0) * 2048;
                    for (int n = 2 * (cg1 - max(cg0, g0)); n > 0 && ok; --n, xs += 1024)
                    {
                        wait_bar(full_s + 8 * st, wrap & 1);
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t ta = tmem + TCV_A_COL + 32 * st;
                        const uint64_t db = tcv_bdesc(xs);
                        tcv_mma(tmem + TCV_D_COL, ta, db, acc_flag);
                        tcv_mma(tmem + TCV_D_COL, ta + 8, db + (256 >> 4), 1u);
                        tcv_mma(tmem + TCV_D_COL, ta + 16, db + (512 >> 4), 1u);
                        tcv_mma(tmem + TCV_D_COL, ta + 24, db + (768 >> 4), 1u);
                        tcv_commit(free_s + 8 * st);
                        acc_flag = 1u;
                        if (++st == TCV_NST) { st = 0; ++wrap; }
                    }
                }
                if (ok) tcv_commit(d_s);
                useg += g1 - g0;
            }
        }
        __syncwarp();
    }
    else
    {
        // ---- weight stream: a cursor walks the range's units; piece p = lane + 32 j of a unit is
        // 16 bytes of tile row p / ROWP ----
        const uint32_t ring_s = smem_u32(smem + L.ring) + warp * (S * SLOT);
        int iu = u0;
        int iblk = iu / G, ig = iu - iblk * G;
        uint32_t islot = 0;
        const unsigned char* isrc[NP];
        size_t istep = 0;
        uint32_t idst[NP];
        #pragma unroll
        for (int j = 0; j < NP; ++j)
        {
            const int p = lane + 32 * j, row = p / ROWP;
            idst[j] = ring_s + row * RP + (p - row * ROWP) * 16;
            isrc[j] = nullptr;
        }
        auto set_block = [&](int blk, int g)
        {
            const int slice = blk / nbw, nb = blk - slice * nbw;
            const unsigned char* tr = reinterpret_cast<const unsigned char*>(P.trellis);
            int stride = P.stride;
            if (P.tables)
            {
                tr = reinterpret_cast<const unsigned char*>(P.t_trellis[slice]);
                stride = P.t_stride ? P.t_stride[slice] : P.width;
            }
            const size_t irow = (size_t) (stride >> 4) * TILE_BYTES;
            const unsigned char* base = tr + (size_t) (nb * 8 + warp * NT) * TILE_BYTES + (size_t) (4 * g) * irow;
            istep = 4 * irow;
            #pragma unroll
            for (int j = 0; j < NP; ++j)
            {
                const int p = lane + 32 * j, row = p / ROWP;
                isrc[j] = base + (size_t) row * irow + (p - row * ROWP) * 16;
            }
        };
        auto issue = [&]()
        {
            if (iu < u1)
            {
                #pragma unroll
                for (int j = 0; j < NP; ++j)
                {
                    if (NP * 32 == PIECES || lane + 32 * j < PIECES) cp_async16_s(idst[j] + islot, isrc[j]);
                    isrc[j] += istep;
                }
                ++iu;
                if (++ig == G)
                {
                    ig = 0;
                    ++iblk;
                    if (iu < u1) set_block(iblk, 0);
                }
            }
            cp_async_commit();
            islot += SLOT;
            if (islot == S * SLOT) islot = 0;
        };

        if (t < 2)
        {
            const int slice0 = iblk / nbw;
            const __half* svh0 = P.tables ? reinterpret_cast<const __half*>(P.t_svh[slice0]) : P.svh;
            asm volatile("prefetch.global.L2 [%0];" :: "l"(svh0 + (size_t) (iblk - slice0 * nbw) * 128 + t * 64));
        }
        // the weight stream does not depend on the previous kernel: start it before waiting for it
        set_block(iblk, ig);
        #pragma unroll
        for (int j = 0; j < S - 1; ++j) issue();

        const uint32_t w_off = ring_s + pq * RP + gq * K * 4;
        const uint32_t p_off = ring_s + pq * RP + ((gq * K + 8 * K - 1) % (8 * K)) * 4;
        const uint32_t t_lane = tmem + ((uint32_t) (32 * warp) << 16) + TCV_A_COL;

        // x~ of one chunk: tasks (batch row b, 128-row block jb) go round the warps. Each warp's first
        // task of the NEXT chunk is loaded one chunk ahead (batches of one or two rows have no other
        // task), so that a chunk boundary costs no trip to L2.
        half4 vx[TCV_TB], vs[TCV_TB];
        auto x_fetch = [&](const __half* suh, int cg0, int nblk, int i_from, int i_to)
        {
            #pragma unroll
            for (int i = 0; i < TCV_TB; ++i)
            {
                if (i < i_from || i >= i_to) continue;
                const int tt = warp + TCV_WARPS * i;
                if (tt < m * nblk)
                {
                    const int b = tt / nblk, jb = tt - b * nblk;
                    const size_t col = (size_t) cg0 * 64 + (size_t) jb * 128 + lane * 4;
                    vs[i] = *reinterpret_cast<const half4*>(suh + col);
                    vx[i] = *reinterpret_cast<const half4*>(P.x + (size_t) b * k + col);
                }
            }
        };
        auto x_store = [&](int buf, int nblk)
        {
            unsigned char* xs = xb + buf * (XG * 2048);
            #pragma unroll
            for (int i = 0; i < TCV_TB; ++i)
            {
                const int tt = warp + TCV_WARPS * i;
                if (tt < m * nblk)
                {
                    const int b = tt / nblk, jb = tt - b * nblk;
                    half4 v = vx[i];
                    v.x = __hmul2(v.x, vs[i].x);
                    v.y = __hmul2(v.y, vs[i].y);
                    float h0 = __low2float(v.x), h1 = __high2float(v.x), h2 = __low2float(v.y), h3 = __high2float(v.y);
                    warp_had128(h0, h1, h2, h3, lane);
                    const __half2 o01 = __floats2half2_rn(h0 * kRScale, h1 * kRScale);
                    const __half2 o23 = __floats2half2_rn(h2 * kRScale, h3 * kRScale);
                    const uint32_t u01 = *reinterpret_cast<const uint32_t*>(&o01);
                    const uint32_t u23 = *reinterpret_cast<const uint32_t*>(&o23);
                    // rows 4*lane .. +3 of the block: group jb*2 + lane/16; inside the group tile row
                    // p4 = (lane%16)/4, and rows 4*(lane%4) + i of the tile: MMA q = 2*R + f with
                    // R = 2*(lane%2) + i/2, f = (lane%4)/2; slot pair 2*p4 + i%2 of the MMA
                    const int g = jb * 2 + (lane >> 4), p4 = (lane & 15) >> 2;
                    const int q0 = 4 * (lane & 1) + ((lane & 3) >> 1);
                    unsigned char* dst = xs + ((g * 8 + q0) * 2 + (p4 >> 1)) * 128 + b * 16 + 8 * (p4 & 1);
                    uint2 d0, d1;
                    d0.x = __byte_perm(u01, u01, 0x1010); d0.y = __byte_perm(u01, u01, 0x3232);
                    d1.x = __byte_perm(u23, u23, 0x1010); d1.y = __byte_perm(u23, u23, 0x3232);
                    *reinterpret_cast<uint2*>(dst) = d0;
                    *reinterpret_cast<uint2*>(dst + 2 * 256) = d1;
                    if constexpr (CB == 2)
                    {
                        float sg = (__low2float(o01) + __high2float(o01)) + (__low2float(o23) + __high2float(o23));
                        #pragma unroll
                        for (int s2 = 1; s2 < 16; s2 <<= 1) sg += __shfl_xor_sync(0xffffffffu, sg, s2);
                        if ((lane & 15) == 0) gsum[(buf * m + b) * XG + 2 * jb + (lane >> 4)] = sg;
                    }
                }
            }
        };

        uint32_t cslot = 0;
        int st = 0;                                      // next stage's slot in the ring
        uint32_t wrap = 0;                               // how many times the ring has gone round
        int nstage = 0;                                  // stages produced so far
        int ev = 0;                                      // x~ chunk counter
        int done_upto = -1;                              // stages whose MMAs are known to be complete
        int ev_last[2] = { -1, -1 };                     // last stage that reads each x~ buffer
        uint32_t nseg = 0;
        bool waited = false, prefetched = false;
        int pend = -1;                                   // stage whose stores are issued but not yet handed over
        int useg = u0;
        while (useg < u1)
        {
            // ---- one segment: the part of this CTA's range that lies in one column block ----
            const int blk = useg / G;
            const int g0 = useg - blk * G;
            const int g1 = min(G, g0 + (u1 - useg));
            const __half* suh;
            const int slice = slice_of(blk, suh);
            const int nb = blk - slice * nbw;
            const __half* svh = P.svh;
            unsigned char* cbase = reinterpret_cast<unsigned char*>(P.c);
            int stride = P.stride;
            if (P.tables)
            {
                svh = reinterpret_cast<const __half*>(P.t_svh[slice]);
                stride = P.t_stride ? P.t_stride[slice] : P.width;
                if (P.t_c) cbase = reinterpret_cast<unsigned char*>(P.t_c[slice]);
                else cbase += (size_t) slice * m * P.width * (P.c_fp32 ? 4 : 2);
            }
            float xsum[TCV_MAX_M];
            #pragma unroll
            for (int b = 0; b < TCV_MAX_M; ++b) xsum[b] = 0.f;

            for (int cg0 = (g0 / XG) * XG; cg0 < g1; cg0 += XG)
            {
                const int cg1 = min(cg0 + XG, g1);
                const int cend = min(cg0 + XG, G);       // x~ is made for the whole chunk
                const int nblk = (cend - cg0) >> 1;
                const int buf = ev & 1;
                // the buffer's previous readers (two chunks ago) must be done
                if (ev_last[buf] > done_upto)
                {
                    wait_bar(free_s + 8 * (ev_last[buf] % TCV_NST), (uint32_t) ((ev_last[buf] / TCV_NST) & 1));
                    done_upto = ev_last[buf];
                }
                // suh belongs to the weights; x is the previous kernel's output
                if (!waited) { if (P.pdl) pdl_wait(); waited = true; }
                x_fetch(suh, cg0, nblk, prefetched ? 1 : 0, TCV_TB);
                x_store(buf, nblk);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) tcv_arrive(x_s + 8 * buf);
                ++ev;
                // first task of the next chunk (this block's, or the first of the next block)
                prefetched = false;
                if (cg0 + XG < g1)
                {
                    x_fetch(suh, cg0 + XG, (min(cg0 + 2 * XG, G) - (cg0 + XG)) >> 1, 0, 1);
                    prefetched = true;
                }
                else if (useg + (g1 - g0) < u1)
                {
                    const __half* suh_n;
                    slice_of(blk + 1, suh_n);
                    x_fetch(suh_n, 0, (min(XG, G)) >> 1, 0, 1);
                    prefetched = true;
                }

                const int c0 = max(cg0, g0);
                for (int g = c0; g < cg1; ++g)
                {
                    cp_async_wait_n<S - 2>();
                    __syncwarp();
                    issue();
                    if constexpr (CB == 2)
                    {
                        #pragma unroll
                        for (int b = 0; b < TCV_MAX_M; ++b)
                            if (b < m) xsum[b] += gsum[(buf * m + b) * XG + (g - cg0)];
                    }
                    uint32_t w[NT][K], prev[NT];
                    #pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
                    {
                        load_chunk_s<K>(w_off + cslot + nt * TILE_BYTES, w[nt]);
                        prev[nt] = lds32(p_off + cslot + nt * TILE_BYTES);
                    }
                    #pragma unroll
                    for (int h = 0; h < 2; ++h)
                    {
                        uint32_t st8[8], a0[8], a1[8];
                        if (h == 0) states8<K, 0>(w[0], prev[0], st8); else states8<K, 2>(w[0], prev[0], st8);
                        #pragma unroll
                        for (int j = 0; j < 8; ++j) a0[j] = a_word<CB>(st8[j]);
                        if (h == 0) states8<K, 1>(w[0], prev[0], st8); else states8<K, 3>(w[0], prev[0], st8);
                        #pragma unroll
                        for (int j = 0; j < 8; ++j) a1[j] = a_word<CB>(st8[j]);
                        // the previous stage's stores have had half a stage of arithmetic to land
                        if (pend >= 0)
                        {
                            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                            __syncwarp();
                            if (lane == 0) tcv_arrive(full_s + 8 * pend);
                        }
                        if (wrap)
                        {
                            // the MMAs that read this slot one round ago must be done
                            wait_bar(free_s + 8 * st, (wrap & 1) ^ 1);
                            done_upto = nstage - TCV_NST;
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        }
                        const uint32_t t_st = t_lane + 32 * st;
                        tcv_st_tile(t_st, a0);
                        tcv_st_tile(t_st + 16, a1);
                        if (h == 0) states8<K, 0>(w[1], prev[1], st8); else states8<K, 2>(w[1], prev[1], st8);
                        #pragma unroll
                        for (int j = 0; j < 8; ++j) a0[j] = a_word<CB>(st8[j]);
                        tcv_st_tile(t_st + (16u << 16), a0);
                        if (h == 0) states8<K, 1>(w[1], prev[1], st8); else states8<K, 3>(w[1], prev[1], st8);
                        #pragma unroll
                        for (int j = 0; j < 8; ++j) a1[j] = a_word<CB>(st8[j]);
                        tcv_st_tile(t_st + (16u << 16) + 16, a1);
                        pend = st;
                        ++nstage;
                        if (++st == TCV_NST) { st = 0; ++wrap; }
                    }
                    cslot += SLOT;
                    if (cslot == S * SLOT) cslot = 0;
                }
                ev_last[buf] = nstage - 1;
            }

            // ---- segment done: hand over the last stage, then the accumulators hold this CTA's rows ----
            if (pend >= 0)
            {
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) tcv_arrive(full_s + 8 * pend);
                pend = -1;
            }
            wait_bar(d_s, nseg & 1);
            ++nseg;
            done_upto = nstage - 1;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t dv[8];
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                : "=r"(dv[0]), "=r"(dv[1]), "=r"(dv[2]), "=r"(dv[3]), "=r"(dv[4]), "=r"(dv[5]), "=r"(dv[6]), "=r"(dv[7])
                : "r"(tmem + ((uint32_t) (32 * warp) << 16) + TCV_D_COL) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");

            const bool whole = (g0 == 0 && g1 == G);
            const int i_first = split.owner(blk * G);
            const int i_last = split.owner((blk + 1) * G - 1);
            float* slots = P.scratch;
            const int my_slot = 2 * cta + (blk * G > u0 ? 1 : 0);
            float* dst = whole ? part : slots + (size_t) my_slot * m * 128;
            const bool clustered = P.cluster > 0;
            uint32_t xdst = 0;
            if (clustered) xdst = cluster_map(smem_u32(smem + L.xchg), 0) + cluster_rank() * (m * 128 * 4);
            const int col = 32 * warp + lane;
            #pragma unroll
            for (int b = 0; b < TCV_MAX_M; ++b)
            {
                if (b >= m) continue;
                float d = __uint_as_float(dv[b]);
                if constexpr (CB == 2)
                {
                    const float kinv = __half2float(__ushort_as_half((unsigned short) 0x1eee));
                    const float kbias = __half2float(__ushort_as_half((unsigned short) 0xc931));
                    d = d * kinv + xsum[b] * kbias;
                }
                if (clustered) cluster_st_f32(xdst + (b * 128 + col) * 4, d);
                else dst[b * 128 + col] = d;
            }

            bool finish = whole;
            if (clustered)
            {
                cluster_sync_all();
                finish = cluster_rank() == 0;
                if (finish)
                {
                    const float* xc = reinterpret_cast<const float*>(smem + L.xchg);
                    for (int idx = t; idx < m * 128; idx += 32 * TCV_WARPS)
                    {
                        float sum = xc[idx];
                        for (int r = 1; r < P.cluster; ++r) sum += xc[r * m * 128 + idx];
                        part[idx] = sum;
                    }
                }
            }
            else if (!whole)
            {
                tcv_bar_decode();
                if (t == 0)
                {
                    __threadfence();
                    const int prevc = atomicAdd(P.counters + blk, 1);
                    s_last = (prevc == i_last - i_first);
                    if (s_last)
                    {
                        P.counters[blk] = 0;
                        __threadfence();
                    }
                }
                tcv_bar_decode();
                finish = s_last != 0;
                if (finish)
                {
                    const int first_slot = 2 * i_first + (blk * G > split.begin(i_first) ? 1 : 0);
                    for (int idx = t; idx < m * 128; idx += 32 * TCV_WARPS)
                    {
                        float sum = __ldcg(slots + (size_t) first_slot * m * 128 + idx);
                        for (int ii = i_first + 1; ii <= i_last; ++ii)
                            sum += __ldcg(slots + (size_t) (2 * ii) * m * 128 + idx);
                        part[idx] = sum;
                    }
                }
            }
            tcv_bar_decode();

            if (finish)
            {
                for (int b = warp; b < m; b += TCV_WARPS)
                {
                    float4 v = reinterpret_cast<const float4*>(part + b * 128)[lane];
                    float h0 = v.x, h1 = v.y, h2 = v.z, h3 = v.w;
                    warp_had128(h0, h1, h2, h3, lane);
                    h0 *= kRScale; h1 *= kRScale; h2 *= kRScale; h3 *= kRScale;
                    const half4 sv = reinterpret_cast<const half4*>(svh + (size_t) nb * 128)[lane];
                    if (P.c_fp32)
                    {
                        float4 o = make_float4(h0 * __low2float(sv.x), h1 * __high2float(sv.x),
                                               h2 * __low2float(sv.y), h3 * __high2float(sv.y));
                        reinterpret_cast<float4*>(reinterpret_cast<float*>(cbase) + (size_t) b * stride + (size_t) nb * 128)[lane] = o;
                    }
                    else
                    {
                        half4 o;
                        o.x = __hmul2(__floats2half2_rn(h0, h1), sv.x);
                        o.y = __hmul2(__floats2half2_rn(h2, h3), sv.y);
                        if constexpr (AR)
                        if (P.ar.N)
                        {
                            // this lane's four halves are one unit of the all-reduce payload (m, stride):
                            // push it to every peer, then add up the peers' units in rank order
                            const uint32_t seq = (uint32_t) (*(volatile int*) &P.ar.ctl[0] + 1);
                            const long unit = ((long) b * stride + (long) nb * 128 + lane * 4) >> 2;
                            const long slot_off = (long) (seq & 1) * P.ar.N * P.ar.wcap;
                            const uint2 mine = *reinterpret_cast<const uint2*>(&o);
                            for (int p = 0; p < P.ar.N; ++p)
                                if (p != P.ar.rank)
                                    st_ll2(P.ar.buf[p] + slot_off + (long) P.ar.rank * P.ar.wcap + 2 * unit, mine.x, mine.y, seq);
                            uint2* srcs[COMM_MAXN];
                            #pragma unroll
                            for (int p = 0; p < COMM_MAXN; ++p)
                                srcs[p] = (p < P.ar.N) ? P.ar.buf[P.ar.rank] + slot_off + (long) p * P.ar.wcap + 2 * unit : nullptr;
                            uint32_t d[COMM_MAXN][2];
                            unsigned budget = COMM_SPIN_LIMIT;
                            if (!gather_unit(srcs, &mine, P.ar.rank, P.ar.N, seq, d, budget)) atomicExch(P.ar.ctl + COMM_MAXB, 1);
                            float acc[4] = { 0.f, 0.f, 0.f, 0.f };
                            #pragma unroll
                            for (int p = 0; p < COMM_MAXN; ++p)
                                if (p < P.ar.N) acc4(acc, d[p][0], d[p][1]);
                            o.x = __floats2half2_rn(acc[0], acc[1]);
                            o.y = __floats2half2_rn(acc[2], acc[3]);
                        }
                        reinterpret_cast<half4*>(reinterpret_cast<__half*>(cbase) + (size_t) b * stride + (size_t) nb * 128)[lane] = o;
                    }
                }
                if (AR && P.ar.N)
                {
                    tcv_bar_decode();
                    if (t == 0)
                    {
                        const int seq = *(volatile int*) &P.ar.ctl[0] + 1;
                        __threadfence();
                        if (atomicAdd(&P.ar.ctl[1], 1) == P.blocks - 1)
                        {
                            P.ar.ctl[1] = 0;
                            __threadfence();
                            *(volatile int*) &P.ar.ctl[0] = seq;
                        }
                    }
                }
            }
            useg += g1 - g0;
            if (useg < u1) tcv_bar_decode();              // `part` and the partial slots are reused
        }
        cp_async_wait_n<0>();
    }
    // the cluster barrier is a whole-CTA affair: the issuing warp joins it here
    if (warp == TCV_WARPS && P.cluster > 0) cluster_sync_all();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == TCV_WARPS)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"((uint32_t) TCV_TMEM_COLS) : "memory");
}

#define AMP_GEMV_TC_LOOKUP_DECL(K) gemv_fn gemv_tc_kernel_k##K(int cb, int ar);
AMP_GEMV_TC_LOOKUP_DECL(1) AMP_GEMV_TC_LOOKUP_DECL(2) AMP_GEMV_TC_LOOKUP_DECL(3) AMP_GEMV_TC_LOOKUP_DECL(4)
AMP_GEMV_TC_LOOKUP_DECL(5) AMP_GEMV_TC_LOOKUP_DECL(6) AMP_GEMV_TC_LOOKUP_DECL(7) AMP_GEMV_TC_LOOKUP_DECL(8)
#undef AMP_GEMV_TC_LOOKUP_DECL

}  // namespace amp
