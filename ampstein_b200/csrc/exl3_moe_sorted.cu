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
//                                tile table -- up to 128 / 256 / 512 consecutive rows of one expert
//                                per tile (ms_pick_sub) -- for the GEMMs, (c) the projection-major
//                                pointer tables.
//   2. moe_sorted_rotate_in      gathers each assignment's token row and writes its two rotated
//                                forms (gate's and up's input scales) in the k-step-major swizzled
//                                layout the tensor-core GEMM fetches with bulk copies; notes, per
//                                token, which padded rows belong to it.
//   3. grouped tcgen05 GEMM      gate and up in one grid (exl3_gemm_tc_kernel<K, CB, true>): one CTA
//                                per (tile, projection, 128 columns) decodes its weight block ONCE
//                                for all rows of the tile; fp16 outputs as exl3_gemm gives them.
//   4. moe_sorted_rotate_act     act(gate, up) * down's input scales, rotated, same layout.
//   5. grouped tcgen05 GEMM      down, fp32 outputs into per-assignment rows.
//   6. moe_sorted_combine        per token: its rows in ascending expert order, weight * row summed in
//                                fp32 and ADDED to the output row (the reference accumulates into a
//                                zero-initialised output too). Fixed order: bit-reproducible.
//      or moe_sorted_to_slots    with the caller's slot scratch (the reference's deferred mode):
//                                weight * row copied to slot_base[expert] + row; the sum is then
//                                amp_exl3_moe_gather's (k order, other tiers' slots included).
// The element arithmetic is that of the decode-shaped fused MoE in exl3_gemv_kernel.cuh (fp16
// scale multiply on the gathered input, fp32 activation and scale in front of the down
// projection, one rounding to fp16 at each GEMM input).
#include "exl3_gemv_host.h"
#include "host_common.h"
#include "../../include/ampstein_b200.h"

namespace amp {

constexpr int MS_GROUP_ROWS = 8;                   // rows per task of the rotation kernels: one per warp
constexpr int MS_MAX_TOPK = 64;
// 128-row sub-tiles per GEMM tile: 0 = chosen from the average rows per expert, 1..4 forced (A/B)
int g_ms_tile_sub = 0;

// status bits (header word 2)
constexpr int MS_E_TILES = 1;                      // more row tiles than the table holds (counts exceed the list length)
constexpr int MS_E_ROWS = 2;                       // padded rows exceed the workspace
constexpr int MS_E_TOKEN = 4;                      // a sorted entry names a token outside [0, T)
constexpr int MS_E_TOPK = 8;                       // a token occurs more often than A / T times
constexpr int MS_E_SLOT = 16;                      // deferred sum: a slot index outside the caller's scratch

struct MsLayout
{
    long mcap; int max_tiles, topk, sub;
    size_t hdr, pstart, sstart, tile_e, tile_row0, tile_rows, fill, list, tab, xt_gu, gu, xt_d, dout, total;
};

static inline size_t up256(size_t v) { return (v + 255) & ~(size_t) 255; }

// Rows per tile. A tile's weight block is decoded once for all its rows, so large tiles decode
// least; but only the 128-row form leaves room for two CTAs per SM (shared memory and 2 x 128
// accumulator columns), which hides one CTA's prologue and epilogue behind the other's main loop.
static int ms_pick_sub(long A, long E)
{
    if (g_ms_tile_sub >= 1 && g_ms_tile_sub <= 4) return g_ms_tile_sub;
    const long avg = A / (E > 0 ? E : 1);
    return avg <= 192 ? 1 : 4;         // (256-row tiles lost to one of the two at every chunk size measured)
}

static MsLayout ms_layout(long T, long A, long E, long H, long I, int sub)
{
    MsLayout L;
    const long act = A < E ? A : E;
    L.sub = sub;
    L.mcap = ((A + 7 * act) + 7) & ~7L;
    if (L.mcap < 8) L.mcap = 8;
    L.max_tiles = (int) (act + A / (128 * sub));
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
    const long long* count; int E, lo, hi, T; long A; int mcap, max_tiles, tile_cap;
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
        const int nt = active ? (c + P.tile_cap - 1) / P.tile_cap : 0;
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
                    P.tile_row0[t0 + j] = p0 + j * P.tile_cap;
                    P.tile_rows[t0 + j] = min(P.tile_cap, c - j * P.tile_cap);
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
    int mcap, groups;                                // groups: 8-row groups per tile
    int* fill; int2* list;
    // activation stage
    const __half* gu; int I; const long long* d_suh; int act, gated; float act_limit;
};

// 128-point Hadamard with eight lanes per 128-value chunk: lane piece pc (0..7) holds the two 16-byte
// pieces (eight values each) at elements 8 pc .. and 64 + 8 pc .. . Same butterflies in the same
// order as warp_had128 (index bits 0..6 in turn; lower = a + b, upper = a - b), hence the same bits
// out: bits 0-2 and 6 inside the lane, bits 3-5 across the eight lanes. 3 shuffles per value
// instead of 5, and both the loads and the stores of a chunk are whole 128-byte lines per eight lanes.
__device__ __forceinline__ void oct_had128(float (&h)[16], int pc)
{
    #pragma unroll
    for (int b = 1; b < 8; b <<= 1)
        #pragma unroll
        for (int i = 0; i < 16; ++i)
            if (!(i & b))
            {
                const float lo = h[i], hi = h[i | b];
                h[i] = lo + hi;
                h[i | b] = lo - hi;
            }
    #pragma unroll
    for (int m = 1; m <= 4; m <<= 1)
    {
        const bool up = (pc & m) != 0;
        #pragma unroll
        for (int i = 0; i < 16; ++i)
        {
            const float p = __shfl_xor_sync(0xffffffffu, h[i], m);
            h[i] = up ? p - h[i] : h[i] + p;
        }
    }
    #pragma unroll
    for (int i = 0; i < 8; ++i)
    {
        const float lo = h[i], hi = h[i + 8];
        h[i] = lo + hi;
        h[i + 8] = lo - hi;
    }
}

// a lane's 16 rotated values -> their place in the k-step-major, swizzled layout (see
// had_tiled_kernel): k steps 2 * chunk and 2 * chunk + 1, 16-byte piece pc ^ (row & 7) of each
__device__ __forceinline__ void ms_store_pieces(unsigned char* xt, int mcap, int p, int cb, int pc, const float (&h)[16])
{
    #pragma unroll
    for (int j = 0; j < 2; ++j)
    {
        const __half2 a = __floats2half2_rn(h[8 * j + 0] * kRScale, h[8 * j + 1] * kRScale);
        const __half2 b = __floats2half2_rn(h[8 * j + 2] * kRScale, h[8 * j + 3] * kRScale);
        const __half2 c = __floats2half2_rn(h[8 * j + 4] * kRScale, h[8 * j + 5] * kRScale);
        const __half2 d = __floats2half2_rn(h[8 * j + 6] * kRScale, h[8 * j + 7] * kRScale);
        uint4 o;
        o.x = *reinterpret_cast<const uint32_t*>(&a); o.y = *reinterpret_cast<const uint32_t*>(&b);
        o.z = *reinterpret_cast<const uint32_t*>(&c); o.w = *reinterpret_cast<const uint32_t*>(&d);
        unsigned char* row = xt + (((size_t) (2 * cb + j) * (size_t) mcap + (size_t) p) << 7);
        *reinterpret_cast<uint4*>(row + ((pc ^ (p & 7)) << 4)) = o;
    }
}

// the lane's two pieces of a chunk (src = first value of the chunk): elements 8 pc .. and 64 + 8 pc ..
__device__ __forceinline__ void ms_load_pieces(const __half* src, int pc, __half2 (&v)[8])
{
    #pragma unroll
    for (int j = 0; j < 2; ++j)
    {
        const uint4 r = *reinterpret_cast<const uint4*>(src + 64 * j + 8 * pc);
        v[4 * j + 0] = *reinterpret_cast<const __half2*>(&r.x); v[4 * j + 1] = *reinterpret_cast<const __half2*>(&r.y);
        v[4 * j + 2] = *reinterpret_cast<const __half2*>(&r.z); v[4 * j + 3] = *reinterpret_cast<const __half2*>(&r.w);
    }
}

// task = (tile, group of 8 rows): one row per warp; a warp takes four 128-value chunks of its row
// per pass, eight lanes each.
__global__ __launch_bounds__(256)
void moe_sorted_rotate_in_kernel(const MsRot P)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, pc = lane & 7, cl = lane >> 3;
    const int ntasks = P.hdr[0] * P.groups, chunks = P.H >> 7;
    for (int task = blockIdx.x; task < ntasks; task += gridDim.x)
    {
        const int tile = task / P.groups, rg = task - tile * P.groups;
        const int rows = P.tile_rows[tile];
        const int r = rg * MS_GROUP_ROWS + warp;
        if (r >= rows) continue;
        const int e = P.tile_e[tile], row0 = P.tile_row0[tile];
        const __half* gs = P.g_suh ? reinterpret_cast<const __half*>(P.g_suh[e]) : nullptr;
        const __half* us = reinterpret_cast<const __half*>(P.u_suh[e]);
        const int p = row0 + r, s = P.sstart[e] + (row0 - P.pstart[e]) + r;
        const long long tok = (s >= 0 && s < P.A) ? P.tok_sorted[s] : -1;
        if (tok < 0 || tok >= P.T)
        {
            if (lane == 0) atomicOr(P.status, MS_E_TOKEN);
            continue;                                      // the row keeps whatever it held; it is never summed
        }
        if (lane == 0)
        {
            const int j = atomicAdd(&P.fill[tok], 1);
            if (j < P.topk) P.list[(size_t) tok * P.topk + j] = make_int2(p, s);
            else atomicOr(P.status, MS_E_TOPK);
        }
        const __half* src = P.y + (size_t) tok * P.H;
        unsigned char* xu = P.xt + (gs ? (size_t) P.mcap * P.H * 2 : 0);
        for (int c0 = 0; c0 < chunks; c0 += 4)
        {
            const int cb = c0 + cl;
            const bool live = cb < chunks;                 // (idle lanes still take part in the shuffles)
            const int off = (live ? cb : 0) * 128;
            __half2 v[8], su[8], sg[8];
            float h[16];
            ms_load_pieces(src + off, pc, v);
            ms_load_pieces(us + off, pc, su);
            if (gs) ms_load_pieces(gs + off, pc, sg);
            #pragma unroll
            for (int i = 0; i < 8; ++i)
            {
                const __half2 a = __hmul2(v[i], su[i]);
                h[2 * i] = __low2float(a); h[2 * i + 1] = __high2float(a);
            }
            oct_had128(h, pc);
            if (live) ms_store_pieces(xu, P.mcap, p, cb, pc, h);
            if (gs)
            {
                #pragma unroll
                for (int i = 0; i < 8; ++i)
                {
                    const __half2 a = __hmul2(v[i], sg[i]);
                    h[2 * i] = __low2float(a); h[2 * i + 1] = __high2float(a);
                }
                oct_had128(h, pc);
                if (live) ms_store_pieces(P.xt, P.mcap, p, cb, pc, h);
            }
        }
    }
}

__global__ __launch_bounds__(256)
void moe_sorted_rotate_act_kernel(const MsRot P)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, pc = lane & 7, cl = lane >> 3;
    const int ntasks = P.hdr[0] * P.groups, chunks = P.I >> 7;
    const __half* gbase = P.gu;                                                     // gate outputs (projection 0)
    const __half* ubase = P.gu + (P.gated ? (size_t) P.mcap * P.I : 0);              // up outputs
    for (int task = blockIdx.x; task < ntasks; task += gridDim.x)
    {
        const int tile = task / P.groups, rg = task - tile * P.groups;
        const int rows = P.tile_rows[tile];
        const int r = rg * MS_GROUP_ROWS + warp;
        if (r >= rows) continue;
        const int e = P.tile_e[tile], p = P.tile_row0[tile] + r;
        const __half* ds = reinterpret_cast<const __half*>(P.d_suh[e]);
        const __half* ur = ubase + (size_t) p * P.I;
        const __half* gr = gbase + (size_t) p * P.I;
        for (int c0 = 0; c0 < chunks; c0 += 4)
        {
            const int cb = c0 + cl;
            const bool live = cb < chunks;
            const int off = (live ? cb : 0) * 128;
            __half2 u[8], g[8], sc[8];
            float h[16];
            ms_load_pieces(ur + off, pc, u);
            ms_load_pieces((P.gated ? gr : ur) + off, pc, g);
            ms_load_pieces(ds + off, pc, sc);
            #pragma unroll
            for (int i = 0; i < 8; ++i)
            {
                h[2 * i] = moe_act_gate(P.act, P.gated, __low2float(g[i]), __low2float(u[i]), P.act_limit) * __low2float(sc[i]);
                h[2 * i + 1] = moe_act_gate(P.act, P.gated, __high2float(g[i]), __high2float(u[i]), P.act_limit) * __high2float(sc[i]);
            }
            oct_had128(h, pc);
            if (live) ms_store_pieces(P.xt, P.mcap, p, cb, pc, h);
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

// Deferred sum (the reference's slot mode): weight * down output of every assignment goes to the
// caller's slot row slot_base[expert] + (row within the expert); amp_exl3_moe_gather adds the slots
// up later. One row per warp.
__global__ __launch_bounds__(256)
void moe_sorted_to_slots_kernel(const MsRot P, const float* __restrict__ dout, const __half* __restrict__ w_sorted,
                                float* __restrict__ scratch, const long long* __restrict__ slot_base, long scratch_rows)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ntasks = P.hdr[0] * P.groups;
    for (int task = blockIdx.x; task < ntasks; task += gridDim.x)
    {
        const int tile = task / P.groups, rg = task - tile * P.groups;
        const int rows = P.tile_rows[tile];
        const int r = rg * MS_GROUP_ROWS + warp;
        if (r >= rows) continue;
        const int e = P.tile_e[tile], row0 = P.tile_row0[tile];
        const int in_expert = (row0 - P.pstart[e]) + r, p = row0 + r, s = P.sstart[e] + in_expert;
        const long long slot = slot_base[e] + in_expert;
        if (slot < 0 || slot >= scratch_rows || s < 0 || s >= P.A)
        {
            if (lane == 0) atomicOr(P.status, MS_E_SLOT);
            continue;
        }
        const float w = __half2float(w_sorted[s]);
        const float4* src = reinterpret_cast<const float4*>(dout + (size_t) p * P.H);
        float4* dst = reinterpret_cast<float4*>(scratch + (size_t) slot * P.H);
        for (int c = lane; c < (P.H >> 2); c += 32)
        {
            float4 v = __ldcs(src + c);
            v.x *= w; v.y *= w; v.z *= w; v.w *= w;
            dst[c] = v;
        }
    }
}

// The fixed-order sum over per-assignment slots, as the reference defines it (exl3_moe_gather_kernel,
// vendor/exl3/exllamav3_ext/quant/exl3_moe.cu:420-470): one block per token; assignment a = token *
// topk + k of local expert e = flat_expert[a] (outside [0, E): none) owns slot slot_base[e] +
// inv_order[a] - expert_start[e] when slot_kind[e] != 0; kind 2 slots hold unweighted rows and are
// multiplied by weight_sorted[inv_order[a]] here. Summed in k order in fp32, added to the output row.
__global__ __launch_bounds__(256)
void moe_gather_kernel(float* __restrict__ out, const float* __restrict__ scratch, const long long* __restrict__ flat_expert,
                       const long long* __restrict__ inv_order, const long long* __restrict__ expert_start,
                       const long long* __restrict__ slot_base, const long long* __restrict__ slot_kind,
                       const __half* __restrict__ w_sorted, int H, int topk, int E, long scratch_rows, long A)
{
    __shared__ long long s_slot[MS_MAX_TOPK];
    __shared__ float s_w[MS_MAX_TOPK];
    __shared__ int s_n;
    const int tok = blockIdx.x, t = threadIdx.x;
    if (t == 0)
    {
        int n = 0;
        for (int k = 0; k < topk; ++k)
        {
            const long long a = (long long) tok * topk + k, e = flat_expert[a];
            if (e < 0 || e >= E) continue;
            const long long kind = slot_kind[e];
            if (!kind) continue;
            const long long pos = inv_order[a], slot = slot_base[e] + (pos - expert_start[e]);
            if (slot < 0 || slot >= scratch_rows || pos < 0 || pos >= A) continue;      // (never read out of bounds)
            s_slot[n] = slot;
            s_w[n] = kind == 2 ? __half2float(w_sorted[pos]) : 1.0f;
            ++n;
        }
        s_n = n;
    }
    __syncthreads();
    const int n = s_n;
    if (n == 0) return;
    for (int c = t; c < (H >> 2); c += 256)
    {
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int j = 0; j < n; ++j)
        {
            const float4 v = __ldcs(reinterpret_cast<const float4*>(scratch + (size_t) s_slot[j] * H) + c);
            const float w = s_w[j];
            acc.x += v.x * w; acc.y += v.y * w; acc.z += v.z * w; acc.w += v.w * w;
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
    // the largest over the tile sizes a call may pick (the tile table shrinks as tiles grow)
    return (long) ms_layout(T, A, E, H, I, 1).total;
}

AMP_API int amp_exl3_moe_sorted(const amp_moe_sorted_args* a, cudaStream_t stream)
{
    AMP_REQUIRE(a, "exl3_moe_sorted: null argument block");
    AMP_REQUIRE(a->T >= 0 && a->A >= 0 && a->E >= 1, "exl3_moe_sorted: sizes");
    if (a->T == 0 || a->A == 0) return 0;
    AMP_REQUIRE(a->y && a->out && a->count && a->tok_sorted && a->w_sorted, "exl3_moe_sorted: null tensor");
    AMP_REQUIRE(!a->scratch || (a->slot_base && a->scratch_rows > 0 && ((uintptr_t) a->scratch & 15) == 0),
                "exl3_moe_sorted: the slot scratch needs slot_base, its row count and 16-byte alignment");
    AMP_REQUIRE(a->H % 128 == 0 && a->I % 128 == 0 && a->H > 0 && a->I > 0, "exl3_moe_sorted: hidden and intermediate widths must be multiples of 128");
    AMP_REQUIRE(a->A % a->T == 0 && a->A / a->T <= MS_MAX_TOPK, "exl3_moe_sorted: the sorted list must hold the same number of picks (<= 64) for every token");
    AMP_REQUIRE(a->A <= 0x3fffffffL && a->T <= 0x3fffffffL && a->E <= (1 << 20), "exl3_moe_sorted: sizes out of range");
    AMP_REQUIRE(a->u_trellis && a->u_suh && a->u_svh && a->d_trellis && a->d_suh && a->d_svh, "exl3_moe_sorted: pointer tables missing");
    AMP_REQUIRE(!a->gated || (a->g_trellis && a->g_suh && a->g_svh), "exl3_moe_sorted: gate tables missing");
    if (a->g_bits || a->u_bits || a->d_bits)
    {
        AMP_REQUIRE(a->u_bits && a->d_bits && (!a->gated || a->g_bits), "exl3_moe_sorted: give all bit width tables or none");
        AMP_REQUIRE(a->kmask_gu > 0 && a->kmask_gu < 256 && a->kmask_d > 0 && a->kmask_d < 256,
                    "exl3_moe_sorted: kmask_gu / kmask_d must name the bit widths (1..8) that occur in the tables");
    }
    else
        AMP_REQUIRE(a->Ku >= 1 && a->Ku <= 8 && a->Kd >= 1 && a->Kd <= 8 && (!a->gated || (a->Kg >= 1 && a->Kg <= 8)), "exl3_moe_sorted: K out of range");
    AMP_REQUIRE(a->cb >= 0 && a->cb <= 2, "exl3_moe_sorted: codebook index out of range");
    AMP_REQUIRE(a->act >= 0 && a->act <= 3, "exl3_moe_sorted: unknown activation");
    // (16 bytes also for every scale vector the tables point to: the rotation kernels load them in 16-byte pieces)
    AMP_REQUIRE(((uintptr_t) a->y & 15) == 0 && ((uintptr_t) a->out & 15) == 0, "exl3_moe_sorted: misaligned tensor");
    const MsLayout L = ms_layout(a->T, a->A, a->E, a->H, a->I, ms_pick_sub(a->A, a->E));
    AMP_REQUIRE(a->workspace && ((uintptr_t) a->workspace & 255) == 0 &&
                a->workspace_bytes >= amp_exl3_moe_sorted_workspace(a->T, a->A, a->E, a->H, a->I),
                "exl3_moe_sorted: workspace missing, misaligned (256) or smaller than amp_exl3_moe_sorted_workspace()");
    AMP_REQUIRE(L.mcap <= 0x7ffffff0L && L.max_tiles <= 65535, "exl3_moe_sorted: chunk too large");
    unsigned char* ws = (unsigned char*) a->workspace;
    const bool gated = a->gated != 0;
    const int E = a->E;

    MsPrep Pp = {};
    Pp.count = (const long long*) a->count; Pp.E = E; Pp.T = a->T; Pp.A = a->A;
    Pp.lo = a->count_lo < 1 ? 1 : a->count_lo;
    Pp.hi = a->count_hi <= 0 ? 0x3fffffff : a->count_hi;
    Pp.mcap = (int) L.mcap; Pp.max_tiles = L.max_tiles; Pp.tile_cap = 128 * L.sub;
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
    const int groups = 128 * L.sub / MS_GROUP_ROWS;
    const long tasks_max = (long) L.max_tiles * groups;
    const int rot_blocks = (int) (tasks_max < (long) sms * 8 ? tasks_max : (long) sms * 8);

    MsRot R = {};
    R.hdr = Pp.hdr; R.pstart = Pp.pstart; R.sstart = Pp.sstart;
    R.tile_e = Pp.tile_e; R.tile_row0 = Pp.tile_row0; R.tile_rows = Pp.tile_rows;
    R.status = Pp.hdr + 2;
    R.tok_sorted = (const long long*) a->tok_sorted; R.A = a->A; R.T = a->T; R.topk = (int) (a->A / a->T);
    R.y = (const __half*) a->y; R.H = a->H;
    R.g_suh = gated ? (const long long*) a->g_suh : nullptr; R.u_suh = (const long long*) a->u_suh;
    R.xt = ws + L.xt_gu; R.mcap = (int) L.mcap; R.groups = groups;
    R.fill = Pp.fill; R.list = (int2*) (ws + L.list);
    moe_sorted_rotate_in_kernel<<<rot_blocks, 256, 0, stream>>>(R);
    if (cudaError_t e = cudaGetLastError()) return cuda_rc(e, "exl3_moe_sorted input rotation launch");

    TcGroups G = {};
    G.ntiles = Pp.hdr; G.tile_e = Pp.tile_e; G.tile_row0 = Pp.tile_row0; G.tile_rows = Pp.tile_rows;
    G.experts = E; G.max_tiles = L.max_tiles; G.sub = L.sub;
    const long long* tab = Pp.tab;
    __half* gu = (__half*) (ws + L.gu);
    const bool mixed = a->g_bits || a->u_bits || a->d_bits;
    if (mixed)
    {
        // one launch per width that occurs; each CTA works only if its expert has the launch's width
        const unsigned char* ub = (const unsigned char*) a->u_bits;
        G.kinds = gated ? 2 : 1;
        G.bits[0] = gated ? (const unsigned char*) a->g_bits : ub; G.bits[1] = ub;
        for (int K = 1; K <= 8; ++K)
            if (a->kmask_gu & (1 << (K - 1)))
                if (int rc = launch_gemm_tc_grouped(ws + L.xt_gu, gu, L.mcap, a->H, a->I, K, a->cb, 0,
                                                    gated ? tab : tab + E, gated ? tab + 2 * E : tab + 3 * E, G, stream)) return rc;
    }
    else if (gated && a->Kg == a->Ku)
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
    G.bits[0] = G.bits[1] = mixed ? (const unsigned char*) a->d_bits : nullptr;
    for (int K = 1; K <= 8; ++K)
        if (mixed ? (a->kmask_d & (1 << (K - 1))) != 0 : K == a->Kd)
            if (int rc = launch_gemm_tc_grouped(ws + L.xt_d, ws + L.dout, L.mcap, a->I, a->H, K, a->cb, 1, tab + 4 * E, tab + 5 * E, G, stream)) return rc;

    if (a->scratch)
    {
        moe_sorted_to_slots_kernel<<<rot_blocks, 256, 0, stream>>>(R, (const float*) (ws + L.dout), (const __half*) a->w_sorted,
                                                                 (float*) a->scratch, (const long long*) a->slot_base, a->scratch_rows);
        return cuda_rc(cudaGetLastError(), "exl3_moe_sorted slot launch");
    }
    moe_sorted_combine_kernel<<<a->T, 256, 0, stream>>>(Pp.fill, (const int2*) (ws + L.list), R.topk, (const __half*) a->w_sorted,
                                                        (const float*) (ws + L.dout), (float*) a->out, a->H);
    return cuda_rc(cudaGetLastError(), "exl3_moe_sorted combine launch");
}

AMP_API int amp_exl3_moe_gather(float* out, const float* scratch, const void* flat_expert, const void* inv_order,
                                const void* expert_start, const void* slot_base, const void* slot_kind, const void* w_sorted,
                                int T, int H, int topk, int E, long scratch_rows, cudaStream_t stream)
{
    AMP_REQUIRE(T >= 0 && H > 0 && H % 4 == 0 && E >= 0, "exl3_moe_gather: sizes");
    if (T == 0 || E == 0) return 0;
    AMP_REQUIRE(out && scratch && flat_expert && inv_order && expert_start && slot_base && slot_kind && w_sorted, "exl3_moe_gather: null tensor");
    AMP_REQUIRE(topk >= 1 && topk <= MS_MAX_TOPK, "exl3_moe_gather: top-k too large");
    AMP_REQUIRE(((uintptr_t) out & 15) == 0 && ((uintptr_t) scratch & 15) == 0, "exl3_moe_gather: misaligned tensor");
    moe_gather_kernel<<<T, 256, 0, stream>>>(out, scratch, (const long long*) flat_expert, (const long long*) inv_order,
                                             (const long long*) expert_start, (const long long*) slot_base,
                                             (const long long*) slot_kind, (const __half*) w_sorted, H, topk, E, scratch_rows,
                                             (long) T * topk);
    return cuda_rc(cudaGetLastError(), "exl3_moe_gather launch");
}

// Rows per GEMM tile of amp_exl3_moe_sorted in units of 128: 0 (default) = chosen per call from the
// average rows per expert, 1..4 = forced. For A/B measurements. Returns the previous setting.
AMP_API int amp_exl3_set_moe_sorted_tile(int sub)
{
    const int prev = g_ms_tile_sub;
    g_ms_tile_sub = (sub >= 0 && sub <= 4) ? sub : 0;
    return prev;
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
