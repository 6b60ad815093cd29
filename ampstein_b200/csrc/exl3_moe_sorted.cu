// Token-sorted MoE for prefill chunks: every routed expert's gate / up GEMM, activation and down
// GEMM over the rows the router gave it, and the routing-weighted sum per token, for hundreds to
// thousands of tokens. Routing (counts, sorted token list, weights) is read from device memory; no
// host synchronisation.
//
// Replaces the reference's exl3_moe (vendor/exl3/exllamav3_ext/quant/exl3_moe.cu:139-531, kernel
// exl3_moe_kernel.cuh:61-313: one persistent kernel, groups of SMs walk the experts, 16/32/64-row
// mma.sync tiles that decode an expert's weights once per row tile) and exl3_moe_gather, the
// fixed-order sum of its per-assignment slots. Organisation here, six launches on one stream:
//   1. moe_sorted_prep_kernel    one block: scans the per-expert counts into (a) each active
//                                expert's first row in a padded row space (every expert starts on a
//                                multiple of 8 rows: the swizzle phase of the rotated layout), (b) a
//                                tile table -- up to 512 consecutive rows of one expert per tile --
//                                for the GEMMs, (c) the projection-major pointer tables.
//   2. moe_sorted_rotate_in      gathers each assignment's token row and writes its two rotated
//                                forms (gate's and up's input scales) in the k-step-major swizzled
//                                layout the tensor-core GEMM fetches with bulk copies; notes, per
//                                token, which padded rows belong to it.
//   3. grouped tcgen05 GEMM      gate and up in one grid (exl3_gemm_tc_kernel<K, CB, true>): one CTA
//                                per (tile, projection, 128 columns) decodes its weight block ONCE
//                                for up to 512 rows; fp16 outputs as exl3_gemm gives them.
//   4. moe_sorted_rotate_act     act(gate, up) * down's input scales, rotated, same layout.
//   5. grouped tcgen05 GEMM      down, fp32 outputs into per-assignment rows.
//   6. moe_sorted_combine        per token: its rows in ascending expert order, weight * row summed in
//                                fp32 and ADDED to the output row (the reference accumulates into a
//                                zero-initialised output too). Fixed order: bit-reproducible.
// The element arithmetic is that of the decode-shaped fused MoE in exl3_gemv_kernel.cuh (fp16
// scale multiply on the gathered input, fp32 activation and scale in front of the down
// projection, one rounding to fp16 at each GEMM input).
#include "exl3_gemv_host.h"
#include "host_common.h"
#include "../../include/ampstein_b200.h"

namespace amp {

constexpr int MS_TILE_SUB = 4;                     // 128-row sub-tiles per GEMM tile
constexpr int MS_TILE_ROWS = MS_TILE_SUB * 128;
constexpr int MS_GROUP_ROWS = 32;                  // rows per task of the rotation kernels
constexpr int MS_GROUPS = MS_TILE_ROWS / MS_GROUP_ROWS;
constexpr int MS_MAX_TOPK = 64;

// status bits (header word 2)
constexpr int MS_E_TILES = 1;                      // more row tiles than the table holds (counts exceed the list length)
constexpr int MS_E_ROWS = 2;                       // padded rows exceed the workspace
constexpr int MS_E_TOKEN = 4;                      // a sorted entry names a token outside [0, T)
constexpr int MS_E_TOPK = 8;                       // a token occurs more often than A / T times

struct MsLayout
{
    long mcap; int max_tiles, topk;
    size_t hdr, pstart, sstart, tile_e, tile_row0, tile_rows, fill, list, tab, xt_gu, gu, xt_d, dout, total;
};

static inline size_t up256(size_t v) { return (v + 255) & ~(size_t) 255; }

static MsLayout ms_layout(long T, long A, long E, long H, long I)
{
    MsLayout L;
    const long act = A < E ? A : E;
    L.mcap = ((A + 7 * act) + 7) & ~7L;
    if (L.mcap < 8) L.mcap = 8;
    L.max_tiles = (int) (act + A / MS_TILE_ROWS);
    if (L.max_tiles < 1) L.max_tiles = 1;
    L.topk = (int) (T > 0 ? (A + T - 1) / T : 1);
    size_t o = 0;
    L.hdr = o;       o = up256(o + 4 * sizeof(int));
    L.pstart = o;    o = up256(o + (size_t) E * sizeof(int));
    L.sstart = o;    o = up256(o + (size_t) E * sizeof(int));
    L.tile_e = o;    o = up256(o + (size_t) L.max_tiles * sizeof(int));
    L.tile_row0 = o; o = up256(o + (size_t) L.max_tiles * sizeof(int));
    L.tile_rows = o; o = up256(o + (size_t) L.max_tiles * sizeof(int));
    L.fill = o;      o = up256(o + (size_t) T * sizeof(int));
    L.list = o;      o = up256(o + (size_t) T * L.topk * sizeof(int2));
    L.tab = o;       o = up256(o + (size_t) 6 * E * sizeof(long long));       // trellis | svh of gate, up; of down
    // the per-assignment fp32 down outputs take the place of the rotated gate / up inputs, which
    // are dead by then: both are 4 * mcap * H bytes
    L.xt_gu = o;     L.dout = o; o = up256(o + (size_t) 4 * L.mcap * H);
    L.gu = o;        o = up256(o + (size_t) 2 * L.mcap * I * 2);
    L.xt_d = o;      o = up256(o + (size_t) L.mcap * I * 2);
    L.total = o;
    return L;
}

struct MsPrep
{
    const long long* count; int E, lo, hi, T; long A; int mcap, max_tiles;
    int* hdr; int* pstart; int* sstart; int* tile_e; int* tile_row0; int* tile_rows; int* fill;
    const long long* src[6];        // g_trellis, u_trellis, g_svh, u_svh, d_trellis, d_svh (g_* null when not gated)
    long long* tab;                 // [trellis: gate E, up E][svh: gate E, up E][down trellis E][down svh E]
};

__device__ __forceinline__ int block_excl_scan_1024(int v, int* s_warp, int& total)
{
    // exclusive prefix over the 1024 threads of the block; total = sum over all
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
    #pragma unroll
    for (int d = 1; d < 32; d <<= 1)
    {
        const int o = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += o;
    }
    __syncthreads();                                   // s_warp may still be read from the previous scan
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    int wsum = s_warp[lane];                           // 32 warps
    int winc = wsum;
    #pragma unroll
    for (int d = 1; d < 32; d <<= 1)
    {
        const int o = __shfl_up_sync(0xffffffffu, winc, d);
        if (lane >= d) winc += o;
    }
    total = __shfl_sync(0xffffffffu, winc, 31);
    const int wbase = __shfl_sync(0xffffffffu, winc - wsum, warp);
    return wbase + inc - v;
}

__global__ __launch_bounds__(1024)
void moe_sorted_prep_kernel(const MsPrep P)
{
    __shared__ int s_warp[32];
    const int t = threadIdx.x;
    for (int i = t; i < P.T; i += 1024) P.fill[i] = 0;
    for (int i = t; i < P.E; i += 1024)
    {
        P.tab[i] = P.src[0] ? P.src[0][i] : 0;             P.tab[P.E + i] = P.src[1][i];
        P.tab[2 * P.E + i] = P.src[2] ? P.src[2][i] : 0;   P.tab[3 * P.E + i] = P.src[3][i];
        P.tab[4 * P.E + i] = P.src[4][i];                  P.tab[5 * P.E + i] = P.src[5][i];
    }
    int carry_s = 0, carry_p = 0, carry_t = 0, status = 0;
    for (int base = 0; base < P.E; base += 1024)
    {
        const int e = base + t;
        long long cl = e < P.E ? P.count[e] : 0;
        if (cl < 0) cl = 0;
        if (cl > P.A) cl = P.A + 1;                        // inconsistent count: runs into the checks below
        const int c = (int) (cl > 0x3fffffff ? 0x3fffffff : cl);
        const bool active = c > 0 && c >= P.lo && c <= P.hi;
        const int pad = active ? ((c + 7) & ~7) : 0;
        const int nt = active ? (c + MS_TILE_ROWS - 1) / MS_TILE_ROWS : 0;
        int tot_s, tot_p, tot_t;
        const int s0 = carry_s + block_excl_scan_1024(c, s_warp, tot_s);
        const int p0 = carry_p + block_excl_scan_1024(pad, s_warp, tot_p);
        const int t0 = carry_t + block_excl_scan_1024(nt, s_warp, tot_t);
        if (e < P.E)
        {
            bool ok = active;
            if (active && ((long) s0 + c > P.A || p0 + pad > P.mcap)) { ok = false; status |= MS_E_ROWS; }
            if (ok && t0 + nt > P.max_tiles) { ok = false; status |= MS_E_TILES; }
            P.sstart[e] = s0;
            P.pstart[e] = ok ? p0 : -1;
            if (ok)
                for (int j = 0; j < nt; ++j)
                {
                    P.tile_e[t0 + j] = e;
                    P.tile_row0[t0 + j] = p0 + j * MS_TILE_ROWS;
                    P.tile_rows[t0 + j] = min(MS_TILE_ROWS, c - j * MS_TILE_ROWS);
                }
            else
                for (int j = 0; j < nt && t0 + j < P.max_tiles; ++j)
                {
                    P.tile_e[t0 + j] = 0; P.tile_row0[t0 + j] = 0; P.tile_rows[t0 + j] = 0;    // a tile without rows
                }
        }
        carry_s += tot_s; carry_p += tot_p; carry_t += tot_t;
    }
    status = __syncthreads_or(status);
    if (t == 0)
    {
        P.hdr[0] = min(carry_t, P.max_tiles);
        P.hdr[1] = min(carry_p, P.mcap);
        P.hdr[2] = status;
    }
}

struct MsRot
{
    const int* hdr; const int* pstart; const int* sstart;
    const int* tile_e; const int* tile_row0; const int* tile_rows;
    int* status;
    const long long* tok_sorted; long A; int T, topk;
    const __half* y; int H;                          // gather source (T, H)
    const long long* g_suh; const long long* u_suh;  // g_suh null: not gated
    unsigned char* xt;                               // (kinds, k / 64, mcap, 128 bytes)
    int mcap;
    int* fill; int2* list;
    // activation stage
    const __half* gu; int I; const long long* d_suh; int act, gated; float act_limit;
};

// rotated chunk -> its place in the k-step-major, swizzled layout (see had_tiled_kernel)
__device__ __forceinline__ void ms_store_tiled(unsigned char* xt, int mcap, int p, int cb, int lane, float h0, float h1, float h2, float h3)
{
    half4 o;
    o.x = __floats2half2_rn(h0 * kRScale, h1 * kRScale);
    o.y = __floats2half2_rn(h2 * kRScale, h3 * kRScale);
    const size_t kstep = (size_t) (2 * cb + (lane >> 4));
    const int piece = ((lane & 15) >> 1) ^ (p & 7);
    *reinterpret_cast<half4*>(xt + ((kstep * (size_t) mcap + (size_t) p) << 7) + (piece << 4) + ((lane & 1) << 3)) = o;
}

// task = (tile, group of 32 rows); a warp takes rows w, w + 8, ... of the group
__global__ __launch_bounds__(256)
void moe_sorted_rotate_in_kernel(const MsRot P)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ntasks = P.hdr[0] * MS_GROUPS, chunks = P.H >> 7;
    for (int task = blockIdx.x; task < ntasks; task += gridDim.x)
    {
        const int tile = task / MS_GROUPS, rg = task - tile * MS_GROUPS;
        const int rows = P.tile_rows[tile];
        if (rg * MS_GROUP_ROWS >= rows) continue;
        const int e = P.tile_e[tile], row0 = P.tile_row0[tile];
        const __half* gs = P.g_suh ? reinterpret_cast<const __half*>(P.g_suh[e]) : nullptr;
        const __half* us = reinterpret_cast<const __half*>(P.u_suh[e]);
        const int sbase = P.sstart[e] + (row0 - P.pstart[e]);
        for (int r = rg * MS_GROUP_ROWS + warp; r < min(rows, (rg + 1) * MS_GROUP_ROWS); r += 8)
        {
            const int p = row0 + r, s = sbase + r;
            long long tok = (s >= 0 && s < P.A) ? P.tok_sorted[s] : -1;
            if (tok < 0 || tok >= P.T)
            {
                if (lane == 0) atomicOr(P.status, MS_E_TOKEN);
                continue;                                  // the row keeps whatever it held; it is never summed
            }
            if (lane == 0)
            {
                const int j = atomicAdd(&P.fill[tok], 1);
                if (j < P.topk) P.list[(size_t) tok * P.topk + j] = make_int2(p, s);
                else atomicOr(P.status, MS_E_TOPK);
            }
            const half4* src = reinterpret_cast<const half4*>(P.y + (size_t) tok * P.H);
            #pragma unroll 4
            for (int cb = 0; cb < chunks; ++cb)
            {
                const half4 v = src[cb * 32 + lane];
                const half4 su = reinterpret_cast<const half4*>(us)[cb * 32 + lane];
                {
                    const __half2 a = __hmul2(v.x, su.x), b = __hmul2(v.y, su.y);
                    float h0 = __low2float(a), h1 = __high2float(a), h2 = __low2float(b), h3 = __high2float(b);
                    warp_had128(h0, h1, h2, h3, lane);
                    ms_store_tiled(P.xt + (gs ? (size_t) P.mcap * P.H * 2 : 0), P.mcap, p, cb, lane, h0, h1, h2, h3);
                }
                if (gs)
                {
                    const half4 sg = reinterpret_cast<const half4*>(gs)[cb * 32 + lane];
                    const __half2 a = __hmul2(v.x, sg.x), b = __hmul2(v.y, sg.y);
                    float h0 = __low2float(a), h1 = __high2float(a), h2 = __low2float(b), h3 = __high2float(b);
                    warp_had128(h0, h1, h2, h3, lane);
                    ms_store_tiled(P.xt, P.mcap, p, cb, lane, h0, h1, h2, h3);
                }
            }
        }
    }
}

__global__ __launch_bounds__(256)
void moe_sorted_rotate_act_kernel(const MsRot P)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ntasks = P.hdr[0] * MS_GROUPS, chunks = P.I >> 7;
    const __half* gbase = P.gu;                                                     // gate outputs (projection 0)
    const __half* ubase = P.gu + (P.gated ? (size_t) P.mcap * P.I : 0);              // up outputs
    for (int task = blockIdx.x; task < ntasks; task += gridDim.x)
    {
        const int tile = task / MS_GROUPS, rg = task - tile * MS_GROUPS;
        const int rows = P.tile_rows[tile];
        if (rg * MS_GROUP_ROWS >= rows) continue;
        const int e = P.tile_e[tile], row0 = P.tile_row0[tile];
        const __half* ds = reinterpret_cast<const __half*>(P.d_suh[e]);
        for (int r = rg * MS_GROUP_ROWS + warp; r < min(rows, (rg + 1) * MS_GROUP_ROWS); r += 8)
        {
            const int p = row0 + r;
            const half4* ur = reinterpret_cast<const half4*>(ubase + (size_t) p * P.I);
            const half4* gr = reinterpret_cast<const half4*>(gbase + (size_t) p * P.I);
            #pragma unroll 2
            for (int cb = 0; cb < chunks; ++cb)
            {
                const half4 u = ur[cb * 32 + lane];
                const half4 g = P.gated ? gr[cb * 32 + lane] : u;
                const half4 sc = reinterpret_cast<const half4*>(ds)[cb * 32 + lane];
                float h0 = moe_act_gate(P.act, P.gated, __low2float(g.x), __low2float(u.x), P.act_limit);
                float h1 = moe_act_gate(P.act, P.gated, __high2float(g.x), __high2float(u.x), P.act_limit);
                float h2 = moe_act_gate(P.act, P.gated, __low2float(g.y), __low2float(u.y), P.act_limit);
                float h3 = moe_act_gate(P.act, P.gated, __high2float(g.y), __high2float(u.y), P.act_limit);
                h0 *= __low2float(sc.x); h1 *= __high2float(sc.x); h2 *= __low2float(sc.y); h3 *= __high2float(sc.y);
                warp_had128(h0, h1, h2, h3, lane);
                ms_store_tiled(P.xt, P.mcap, p, cb, lane, h0, h1, h2, h3);
            }
        }
    }
}

// One block per token: its (row, sorted position) entries in ascending row order (= ascending
// expert), weight * row summed in fp32, added to the output row.
__global__ __launch_bounds__(256)
void moe_sorted_combine_kernel(const int* __restrict__ fill, const int2* __restrict__ list, int topk,
                               const __half* __restrict__ w_sorted, const float* __restrict__ dout,
                               float* __restrict__ out, int H)
{
    __shared__ int s_row[MS_MAX_TOPK];
    __shared__ float s_w[MS_MAX_TOPK];
    const int tok = blockIdx.x, t = threadIdx.x;
    const int n = min(fill[tok], topk);
    if (n == 0) return;
    if (t < n)
    {
        const int2 me = list[(size_t) tok * topk + t];
        int rank = 0;
        for (int j = 0; j < n; ++j)
        {
            const int pj = list[(size_t) tok * topk + j].x;
            rank += (pj < me.x || (pj == me.x && j < t)) ? 1 : 0;
        }
        s_row[rank] = me.x;
        s_w[rank] = __half2float(w_sorted[me.y]);
    }
    __syncthreads();
    for (int c = t; c < (H >> 2); c += 256)
    {
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        #pragma unroll 4
        for (int j = 0; j < n; ++j)
        {
            const float4 v = __ldcs(reinterpret_cast<const float4*>(dout + (size_t) s_row[j] * H) + c);
            const float w = s_w[j];
            acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
        }
        float4* o = reinterpret_cast<float4*>(out + (size_t) tok * H) + c;
        float4 cur = *o;
        cur.x += acc.x; cur.y += acc.y; cur.z += acc.z; cur.w += acc.w;
        *o = cur;
    }
}

}  // namespace amp

using namespace amp;

AMP_API long amp_exl3_moe_sorted_workspace(long T, long A, long E, long H, long I)
{
    if (T < 1 || A < 1 || E < 1 || H < 128 || I < 128) return 0;
    return (long) ms_layout(T, A, E, H, I).total;
}

AMP_API int amp_exl3_moe_sorted(const amp_moe_sorted_args* a, cudaStream_t stream)
{
    AMP_REQUIRE(a, "exl3_moe_sorted: null argument block");
    AMP_REQUIRE(a->T >= 0 && a->A >= 0 && a->E >= 1, "exl3_moe_sorted: sizes");
    if (a->T == 0 || a->A == 0) return 0;
    AMP_REQUIRE(a->y && a->out && a->count && a->tok_sorted && a->w_sorted, "exl3_moe_sorted: null tensor");
    AMP_REQUIRE(a->H % 128 == 0 && a->I % 128 == 0 && a->H > 0 && a->I > 0, "exl3_moe_sorted: hidden and intermediate widths must be multiples of 128");
    AMP_REQUIRE(a->A % a->T == 0 && a->A / a->T <= MS_MAX_TOPK, "exl3_moe_sorted: the sorted list must hold the same number of picks (<= 64) for every token");
    AMP_REQUIRE(a->A <= 0x3fffffffL && a->T <= 0x3fffffffL && a->E <= (1 << 20), "exl3_moe_sorted: sizes out of range");
    AMP_REQUIRE(a->u_trellis && a->u_suh && a->u_svh && a->d_trellis && a->d_suh && a->d_svh, "exl3_moe_sorted: pointer tables missing");
    AMP_REQUIRE(!a->gated || (a->g_trellis && a->g_suh && a->g_svh), "exl3_moe_sorted: gate tables missing");
    AMP_REQUIRE(a->Ku >= 1 && a->Ku <= 8 && a->Kd >= 1 && a->Kd <= 8 && (!a->gated || (a->Kg >= 1 && a->Kg <= 8)), "exl3_moe_sorted: K out of range");
    AMP_REQUIRE(a->cb >= 0 && a->cb <= 2, "exl3_moe_sorted: codebook index out of range");
    AMP_REQUIRE(a->act >= 0 && a->act <= 3, "exl3_moe_sorted: unknown activation");
    AMP_REQUIRE(((uintptr_t) a->y & 7) == 0 && ((uintptr_t) a->out & 15) == 0, "exl3_moe_sorted: misaligned tensor");
    const MsLayout L = ms_layout(a->T, a->A, a->E, a->H, a->I);
    AMP_REQUIRE(a->workspace && ((uintptr_t) a->workspace & 255) == 0 && a->workspace_bytes >= (long) L.total,
                "exl3_moe_sorted: workspace missing, misaligned (256) or smaller than amp_exl3_moe_sorted_workspace()");
    AMP_REQUIRE(L.mcap <= 0x7ffffff0L && L.max_tiles <= 65535, "exl3_moe_sorted: chunk too large");
    unsigned char* ws = (unsigned char*) a->workspace;
    const bool gated = a->gated != 0;
    const int E = a->E;

    MsPrep Pp = {};
    Pp.count = (const long long*) a->count; Pp.E = E; Pp.T = a->T; Pp.A = a->A;
    Pp.lo = a->count_lo < 1 ? 1 : a->count_lo;
    Pp.hi = a->count_hi <= 0 ? 0x3fffffff : a->count_hi;
    Pp.mcap = (int) L.mcap; Pp.max_tiles = L.max_tiles;
    Pp.hdr = (int*) (ws + L.hdr); Pp.pstart = (int*) (ws + L.pstart); Pp.sstart = (int*) (ws + L.sstart);
    Pp.tile_e = (int*) (ws + L.tile_e); Pp.tile_row0 = (int*) (ws + L.tile_row0); Pp.tile_rows = (int*) (ws + L.tile_rows);
    Pp.fill = (int*) (ws + L.fill);
    Pp.src[0] = gated ? (const long long*) a->g_trellis : nullptr; Pp.src[1] = (const long long*) a->u_trellis;
    Pp.src[2] = gated ? (const long long*) a->g_svh : nullptr;     Pp.src[3] = (const long long*) a->u_svh;
    Pp.src[4] = (const long long*) a->d_trellis;                   Pp.src[5] = (const long long*) a->d_svh;
    Pp.tab = (long long*) (ws + L.tab);
    moe_sorted_prep_kernel<<<1, 1024, 0, stream>>>(Pp);
    if (cudaError_t e = cudaGetLastError()) return cuda_rc(e, "exl3_moe_sorted prep launch");

    int dev = 0, sms = 148;
    if (cudaError_t e = cudaGetDevice(&dev)) return cuda_rc(e, "cudaGetDevice");
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long tasks_max = (long) L.max_tiles * MS_GROUPS;
    const int rot_blocks = (int) (tasks_max < (long) sms * 8 ? tasks_max : (long) sms * 8);

    MsRot R = {};
    R.hdr = Pp.hdr; R.pstart = Pp.pstart; R.sstart = Pp.sstart;
    R.tile_e = Pp.tile_e; R.tile_row0 = Pp.tile_row0; R.tile_rows = Pp.tile_rows;
    R.status = Pp.hdr + 2;
    R.tok_sorted = (const long long*) a->tok_sorted; R.A = a->A; R.T = a->T; R.topk = (int) (a->A / a->T);
    R.y = (const __half*) a->y; R.H = a->H;
    R.g_suh = gated ? (const long long*) a->g_suh : nullptr; R.u_suh = (const long long*) a->u_suh;
    R.xt = ws + L.xt_gu; R.mcap = (int) L.mcap;
    R.fill = Pp.fill; R.list = (int2*) (ws + L.list);
    moe_sorted_rotate_in_kernel<<<rot_blocks, 256, 0, stream>>>(R);
    if (cudaError_t e = cudaGetLastError()) return cuda_rc(e, "exl3_moe_sorted input rotation launch");

    TcGroups G = {};
    G.ntiles = Pp.hdr; G.tile_e = Pp.tile_e; G.tile_row0 = Pp.tile_row0; G.tile_rows = Pp.tile_rows;
    G.experts = E; G.max_tiles = L.max_tiles; G.sub = MS_TILE_SUB;
    const long long* tab = Pp.tab;
    __half* gu = (__half*) (ws + L.gu);
    if (gated && a->Kg == a->Ku)
    {
        G.kinds = 2;
        if (int rc = launch_gemm_tc_grouped(ws + L.xt_gu, gu, L.mcap, a->H, a->I, a->Ku, a->cb, 0, tab, tab + 2 * E, G, stream)) return rc;
    }
    else
    {
        G.kinds = 1;
        if (gated)
            if (int rc = launch_gemm_tc_grouped(ws + L.xt_gu, gu, L.mcap, a->H, a->I, a->Kg, a->cb, 0, tab, tab + 2 * E, G, stream)) return rc;
        const size_t po = gated ? (size_t) L.mcap : 0;       // up is projection 1 when gated
        if (int rc = launch_gemm_tc_grouped(ws + L.xt_gu + po * a->H * 2, gu + po * a->I, L.mcap, a->H, a->I, a->Ku, a->cb, 0,
                                            tab + E, tab + 3 * E, G, stream)) return rc;
    }

    MsRot D = R;
    D.gu = gu; D.I = a->I; D.d_suh = (const long long*) a->d_suh; D.act = a->act; D.gated = gated ? 1 : 0; D.act_limit = a->act_limit;
    D.xt = ws + L.xt_d;
    moe_sorted_rotate_act_kernel<<<rot_blocks, 256, 0, stream>>>(D);
    if (cudaError_t e = cudaGetLastError()) return cuda_rc(e, "exl3_moe_sorted activation launch");

    G.kinds = 1;
    if (int rc = launch_gemm_tc_grouped(ws + L.xt_d, ws + L.dout, L.mcap, a->I, a->H, a->Kd, a->cb, 1, tab + 4 * E, tab + 5 * E, G, stream)) return rc;

    moe_sorted_combine_kernel<<<a->T, 256, 0, stream>>>(Pp.fill, (const int2*) (ws + L.list), R.topk, (const __half*) a->w_sorted,
                                                        (const float*) (ws + L.dout), (float*) a->out, a->H);
    return cuda_rc(cudaGetLastError(), "exl3_moe_sorted combine launch");
}

// Reads the status word a call of amp_exl3_moe_sorted left in its workspace (0 = clean; bit 0 / 1:
// the counts describe more rows than the sorted list holds, bit 2: a token index outside [0, T),
// bit 3: a token with more entries than A / T). Synchronises the stream.
AMP_API int amp_exl3_moe_sorted_status(const void* workspace, int* out, cudaStream_t stream)
{
    AMP_REQUIRE(workspace && out, "exl3_moe_sorted_status: null pointer");
    if (cudaError_t e = cudaMemcpyAsync(out, (const unsigned char*) workspace + 2 * sizeof(int), sizeof(int), cudaMemcpyDeviceToHost, stream))
        return cuda_rc(e, "exl3_moe_sorted_status copy");
    return cuda_rc(cudaStreamSynchronize(stream), "exl3_moe_sorted_status sync");
}
