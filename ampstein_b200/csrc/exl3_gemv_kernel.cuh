// Trellis-decode GEMV for decode batches (m <= 16): C = had(A*suh) @ W_hat -> had(.)*svh, for
// one matrix or a bundle of matrices / column slices that share one input.
//
// Replaces the reference's exl3_gemv_kernel, exl3_gemm_kernel at small m and exl3_mgemm_kernel
// (vendor/exl3/exllamav3_ext/quant/exl3_gemv_kernel.cuh:186-482, exl3_gemm_kernel.cuh:8-343)
// with a different organisation for B200:
//
//  * The work -- (128-column block, 64-row group) units in block-major order -- is cut into as
//    many equal contiguous ranges as the device holds CTAs at once, so every SM decodes the
//    same number of weights whatever the shape (no wave quantisation, no tail). A range
//    touches one to three column blocks; a block whose rows are shared between CTAs is
//    finished by whichever contributor arrives last (per-block arrival counter, partial sums
//    in a small global scratch area, summed in ascending-k order so results are bitwise
//    reproducible). Nobody waits: there is no spin, no lock and no grid-wide barrier (the
//    reference needs two grid.sync()s, an A_had scratch tensor and a lock buffer).
//  * A CTA is four warps; each owns two adjacent 16-column tile columns of the block and walks
//    every unit of the range: the warps stay in step (no imbalance inside a CTA, nothing to
//    reduce between warps), a warp's unit is only 2048 weights, so small matrices still spread
//    evenly, and the per-unit bookkeeping (ring, cursors, activations) is shared by two tiles.
//    The decode is bound by the issue rate of the integer pipes (about 0.72 instructions per
//    clock and scheduler whatever the occupancy), so three such CTAs per SM are enough.
//  * Packed trellis words are streamed global -> shared with 16-byte cp.async copies into
//    per-warp rings (a slot = one unit = four tile rows of two tiles, 256*K bytes). Bulk
//    (TMA) copies were measured and rejected for this access pattern: one warp sustains only
//    about one bulk copy per 1000 cycles whatever the ring depth, so the small row pieces of
//    a column block cap the kernel near 1.4 TB/s, while cp.async streams at the full HBM
//    rate. With programmatic dependent launch (optional) the copies are issued before the
//    kernel waits for its predecessor, and a CTA releases the dependents when its decode is
//    done.
//  * Decode stays in registers. The decoded weights are the A operand of mma.sync.m16n8k16
//    (16 output columns x 16 k-slots) and the activations the B operand (k-slots x 8 batch
//    rows), so a batch of up to 8 costs one MMA per 128 weights. For codebooks 0/1 the final
//    fp16 add of the codebook is done BY the tensor core: the two fp16 halves of the masked
//    product sit in adjacent k-slots against a duplicated activation, which removes the
//    byte-permute and half-add per weight from the instruction stream (fp32 accumulation of
//    x*lo + x*hi is at least as accurate as x*fp16(lo+hi)).
//  * The input Hadamard runs in each CTA per column-block segment (x is tiny and L2 resident)
//    and leaves x~ in shared memory already duplicated and in fragment order; the output
//    Hadamard, svh scale and store run in the CTA that finishes the block.
//
// HBM-bound by design (K/8 bytes per weight, read once); in practice limited by instruction
// issue: window cut, multiply-add, lop3 per weight plus a quarter MMA (about four issue slots
// per weight, i.e. ~30 weights per clock per SM).
#pragma once
#include "exl3_common.cuh"
#include "comm_ll.cuh"

namespace amp {

constexpr int GEMV_NT = 2;                     // 16-column tile columns per warp
constexpr int GEMV_WARPS = 8 / GEMV_NT;        // the warps of a CTA cover one 128-column block
constexpr int GEMV_THREADS = 32 * GEMV_WARPS;
constexpr int GEMV_XCHUNK_MAX = 8192;          // most rows of x~ held in shared memory at a time

// Grouped expert GEMV (fused decode MoE): the kernel's slices are expert runs described by a
// device-side run table, the input rows are gathered per run, outputs scatter to slot rows.
constexpr int MOE_RUN_INTS = 4;                 // per run: local expert, row count, eight slot indices as bytes
constexpr int MOE_ACT_SILU = 0, MOE_ACT_GELU = 1, MOE_ACT_RELU2 = 2, MOE_ACT_SILU_OAI = 3;

struct GemvMoe
{
    const int* runs;            // [0] run count, [1] active slots, then MOE_RUN_INTS per run
    const __half* x;            // (tokens, H) input rows, row stride x_stride (gate/up stage)
    int x_stride, H, topk;
    const long long* trellis[3];   // per-expert pointer tables: gate, up, down
    const long long* suh[3];
    const long long* svh[3];
    const long long* bias[3];      // nullable
    void* gu[2];                // (slots, I) gate / up outputs (un-activated, after svh and bias), fp32 or fp16
    int gu_f32;
    float* d_out;               // (slots, Ho) fp32 down outputs (after svh and bias)
    int Hi, I, Ho;
    int act; float act_limit; int gated;
    // routing, read on the device
    const long long* sel; const __half* rw; int bsz;
    int min_expert, max_expert, n_local;
    int inline_runs;            // one token: every CTA derives the run table from sel / rw itself
    // routing-weighted sum of a token's slot outputs, done by whichever CTA delivers the last of the
    // token's picks for a 128-column chunk (MODE 2)
    const int* need;            // [bsz] active local picks per token (inline_runs: derived in the kernel)
    int* done;                  // [bsz][Ho / 128] arrivals, zero between calls
    float* out; int out_stride, H_out;
    const float* sh_out; const __half* sh_gate_w;
    // mixed bit widths: per-expert widths of gate / up / down (uint8, indexed by local expert), or
    // null for one width. A launch then works on the runs whose expert has the launch's width.
    const unsigned char* bits[3];
    int first_down;             // MODE 2: this launch also writes the row of a single token without any pick
};

struct MoeSlot { int row, local; float w; bool active; };

// one (token, pick) slot of the routing: the local expert index and weight, or inactive (weight
// zero, expert outside this shard's range or tables)
__device__ __forceinline__ MoeSlot moe_slot(const long long* sel, const __half* rw, int topk,
                                            int min_expert, int max_expert, int n_local, int s)
{
    MoeSlot si;
    si.row = s / topk;
    long long e = sel[s];
    si.w = __half2float(rw[s]);
    bool ok = si.w != 0.0f;
    if (min_expert >= 0)
    {
        ok = ok && e >= min_expert && e < max_expert;
        e -= min_expert;
    }
    ok = ok && e >= 0 && e < n_local;
    si.local = ok ? (int) e : 0;
    si.active = ok;
    return si;
}

// out[row, chunk] = sum over the row's active picks, in pick order, of weight * d_out[slot] (+ the
// shared expert's output, optionally gated by sigmoid(x . w)): one warp, four columns per lane.
// Reference: exl3_moe_coop_b_kernel's last-arrival epilogue, exl3_moe_coop_kernel.cuh:848-999.
__device__ __forceinline__ void moe_combine_chunk(const GemvMoe& M, int row, int chunk, int lane)
{
    const int col = chunk * 128 + lane * 4;
    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
    for (int k0 = 0; k0 < M.topk; k0 += 8)               // pick order: deterministic
    {
        // lane i < 8 reads pick k0 + i of the routing; then all eight slot rows are requested
        // before the first is added (the loads would otherwise form a chain of L2 round trips)
        MoeSlot mine; mine.active = false; mine.w = 0.f;
        if (lane < 8 && k0 + lane < M.topk)
            mine = moe_slot(M.sel, M.rw, M.topk, M.min_expert, M.max_expert, M.n_local, row * M.topk + k0 + lane);
        const unsigned act = __ballot_sync(0xffffffffu, mine.active);
        float4 v[8];
        #pragma unroll
        for (int i = 0; i < 8; ++i)
            if ((act >> i) & 1)
                v[i] = __ldcg(reinterpret_cast<const float4*>(M.d_out + (size_t) (row * M.topk + k0 + i) * M.Ho + col));
        #pragma unroll
        for (int i = 0; i < 8; ++i)
        {
            const float w = __shfl_sync(0xffffffffu, mine.w, i);
            if (!((act >> i) & 1)) continue;
            o0 = __fadd_rn(o0, __fmul_rn(w, v[i].x)); o1 = __fadd_rn(o1, __fmul_rn(w, v[i].y));
            o2 = __fadd_rn(o2, __fmul_rn(w, v[i].z)); o3 = __fadd_rn(o3, __fmul_rn(w, v[i].w));
        }
    }
    if (M.sh_out)
    {
        float gv = 1.0f;
        if (M.sh_gate_w)
        {
            const __half* xr = M.x + (size_t) row * M.x_stride;
            float dot = 0.0f;
            for (int i = lane * 2; i < M.H; i += 64)
            {
                const __half2 xv = *reinterpret_cast<const __half2*>(xr + i);
                const __half2 wv = *reinterpret_cast<const __half2*>(M.sh_gate_w + i);
                dot += __low2float(xv) * __low2float(wv) + __high2float(xv) * __high2float(wv);
            }
            #pragma unroll
            for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            gv = 1.0f / (1.0f + __expf(-dot));
        }
        const float* sh = M.sh_out + (size_t) row * M.H + col;
        if (col + 0 < M.H) o0 += gv * sh[0];
        if (col + 1 < M.H) o1 += gv * sh[1];
        if (col + 2 < M.H) o2 += gv * sh[2];
        if (col + 3 < M.H) o3 += gv * sh[3];
    }
    float* dst = M.out + (size_t) row * M.out_stride + col;
    if (col + 3 < M.H_out) *reinterpret_cast<float4*>(dst) = make_float4(o0, o1, o2, o3);
    else
    {
        if (col + 0 < M.H_out) dst[0] = o0;
        if (col + 1 < M.H_out) dst[1] = o1;
        if (col + 2 < M.H_out) dst[2] = o2;
    }
}

// Fused tensor-parallel all-reduce (row-parallel linears): the CTA that finishes a column block
// pushes the block's fp16 partial straight into every peer's all-reduce buffer and gathers the
// peers' partials of the same block, so the exchange starts while other blocks still decode and
// needs no launch of its own. Same buffers, layout and sequence protocol as the stand-alone kernel.
struct GemvAr
{
    uint2* buf[COMM_MAXN];      // every rank's buffer as this process addresses it
    int* ctl;                   // this rank's control block
    int rank, N;                // N == 0: no exchange
    long wcap;                  // LL words per (slot, sender) = cap / 2
    int push_only;              // 1: push the partial to every rank (this one included) and do not
                                // gather: the consumer adds the ranks' partials up (GemvArIn)
};

// Input side of the split exchange: the (m, k) input of this launch is the all-reduce of the
// partials that the ranks' previous launches pushed (GemvAr::push_only): every x value is
// gathered from this rank's own buffer (N flag-in-data words per unit of four values), added up in
// fp32 in rank order and rounded once -- the bits the stand-alone all-reduce would have written --
// inside the x~ prologue, while this launch's weight stream is already in flight.
struct GemvArIn
{
    const uint2* buf;           // this rank's buffer
    int* ctl;                   // this rank's control block
    int N;                      // N == 0: plain input
    long wcap;
};

struct GemvParams
{
    // direct mode (tables == 0): one matrix
    const __half* x;            // (m, k), shared by every slice
    const uint16_t* trellis;    // (k/16, stride/16, 16K)
    const __half* suh;          // (k)
    const __half* svh;          // (width)
    void* c;                    // (m, stride) fp16 or fp32; stacked (num, m, width) in table mode without t_c
    // table mode (tables == 1): device pointer tables, one entry per slice (suh: per source)
    const long long* t_trellis;
    const long long* t_suh;
    const long long* t_svh;
    const long long* t_c;       // may be null: outputs stacked in c
    const int* t_stride;        // may be null: stride = width
    const int* t_src;           // may be null: source = slice
    int tables;
    int width;                  // columns per slice (multiple of 128)
    int stride;                 // row width of trellis / output in direct mode
    int m, k;
    int c_fp32;
    int xgroups;                // 64-row groups of x~ held in shared memory at a time (multiple of 4)
    int pdl;                    // launched with programmatic stream serialization
    int cluster;                // 0, or CTAs per thread-block cluster: one cluster = one column block
    int blocks;                 // column blocks in total (slices * width / 128)
    float* scratch;             // [gridDim.x][2][m][128] partial sums of blocks shared between CTAs
    int* counters;              // [blocks] arrival counters, zero between launches
    int* status;                // device status word (the kernel has no waits that can run out; kept for the ABI)
    GemvMoe moe;                // grouped-expert modes only
    GemvAr ar;                  // MODE 0, fp16 output only
    GemvArIn arin;              // MODE 0: x is gathered from the communicator's buffer
    const __half* x2;           // GIN == 3: the input is act(x, x2) = silu(x) * x2 (x = gate, x2 = up), rounded to fp16
                                // GIN == 4: the residual contribution added to x before the norm
    const __half* norm_w;       // GIN == 4: RMSNorm weight (k)
    __half* y;                  // GIN == 4: updated residual stream fp16(x + x2), (m, k), written by the first CTA
    float eps;
    // GIN == 5 (producer side of the split norm): the fp16 output o of this launch is added to the
    // residual stream: y = fp16(h + o) is written instead of o, and every finished 128-column block
    // leaves the sum of squares of its y values in ssq[row][block] (fp32).
    // GIN == 6 (consumer side): the input is fp16(x * rsqrt(sum(ssq[row][*]) / k + eps)) * norm_w, x = the
    // residual stream a GIN == 5 launch wrote.
    const __half* h_in;         // GIN == 5: (m, n) residual stream before the add
    float* ssq;                 // GIN == 5: (m, n / 128) out; GIN == 6: (m, k / 128) in
    int rowbuf;                 // GIN == 4: 4 k bytes of shared memory for y and norm_w of one row (m == 1), or 0
    // GIN == 4, one row, fp16 output: greedy next-token pick over the output (the lm_head's logits)
    // and the decode-state advance, done by the CTAs that finish the column blocks
    unsigned long long* am_key; // best (ordered value << 32 | ~index) so far; zero between launches
    unsigned int* am_count;     // finished column blocks; zero between launches
    long long* am_ids; long long* am_pos; long long* am_log; long long am_log_cap;
    int am_vocab;               // columns that take part (<= n)
};

// A ring slot holds one unit of one warp: four tile rows (the 64-row group) of GEMV_NT adjacent
// tiles, each row padded by 32 bytes so that the four rows start in different banks.
__host__ __device__ constexpr int gemv_row_pitch(int K) { return GEMV_NT * 32 * K + 32; }   // bytes per tile row inside a slot
__host__ __device__ constexpr int gemv_slot_bytes(int K) { return 4 * gemv_row_pitch(K); }
// ring depth per warp: deep enough that a layer-sized matrix is requested almost whole when the
// grid starts (a CTA's range is then 4-30 units), so HBM streams from the first microsecond on
__host__ __device__ constexpr int gemv_stages(int K) { return K <= 4 ? 8 : (K <= 6 ? 6 : 5); }

// byte offsets inside dynamic shared memory
struct GemvSmem
{
    int part, xd, gsum, qs, ring, xchg, stage, total;
};

// 32-bit words per batch row of the duplicated x~ (+16 keeps fragment loads conflict-free)
__host__ __device__ constexpr int gemv_xpitch(int xgroups) { return xgroups * 64 + 16; }

// xrows: rows of x~ / partial sums kept (the batch size m)
// stage: reserve room for the gathered input of one chunk (split exchange), fp16 [xrows][xgroups * 64]
__host__ __device__ inline GemvSmem gemv_smem_layout(int K, int xrows, int xgroups, int cluster = 0, int stage = 0, int extra = 0)
{
    GemvSmem L;
    L.part = 0;                                             // [xrows][128] fp32: the finished block
    L.xd = L.part + xrows * 128 * 4;                        // [xrows][XPITCH] duplicated fp16 pairs
    L.gsum = L.xd + xrows * gemv_xpitch(xgroups) * 4;       // [xrows][xgroups] fp32 (codebook 2: sum of x~ per group)
    L.qs = L.gsum + xrows * xgroups * 4;                    // [xrows][xgroups] fp32 (int8 activations: scale of the group's 128-row block)
    L.ring = L.qs + xrows * xgroups * 4;
    L.ring = (L.ring + 127) & ~127;
    L.xchg = L.ring + GEMV_WARPS * gemv_stages(K) * gemv_slot_bytes(K);   // [cluster][xrows][128] fp32, filled by the cluster's CTAs
    L.stage = L.xchg + cluster * xrows * 128 * 4;
    L.total = L.stage + (stage ? xrows * xgroups * 128 : 0) + extra;     // extra: row-resident vectors of the fused norm
    return L;
}

__device__ __forceinline__ void lds128(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d)
{
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr) : "memory");
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}

// K words of one lane's chunk from shared memory, widest loads the alignment allows
template <int K>
__device__ __forceinline__ void load_chunk_s(uint32_t addr, uint32_t (&w)[K])
{
    if constexpr (K % 4 == 0)
    {
        #pragma unroll
        for (int i = 0; i < K / 4; ++i)
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(w[4 * i]), "=r"(w[4 * i + 1]), "=r"(w[4 * i + 2]), "=r"(w[4 * i + 3]) : "r"(addr + 16 * i) : "memory");
    }
    else if constexpr (K % 2 == 0)
    {
        #pragma unroll
        for (int i = 0; i < K / 2; ++i)
            asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(w[2 * i]), "=r"(w[2 * i + 1]) : "r"(addr + 8 * i) : "memory");
    }
    else
    {
        #pragma unroll
        for (int i = 0; i < K; ++i) w[i] = lds32(addr + 4 * i);
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

// 16-bit field extraction on the FMA-heavy pipe: dp2a with a one-hot byte vector is
// (x & 0xffff) + 0 or (x >> 16) + 0. The integer ALU and the FMA-heavy pipe each accept one warp
// instruction every two cycles on sm_100, and everything else in the decode except the
// multiply-add is ALU work (funnel shifts, lop3), so splitting the field extraction between the
// two pipes is what keeps either from becoming the only bottleneck.
__device__ __forceinline__ uint32_t lo16_fma(uint32_t r)
{
    uint32_t d;
    asm("dp2a.lo.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(r), "r"(0x00000001u), "r"(0u));
    return d;
}

__device__ __forceinline__ uint32_t hi16_fma(uint32_t r)
{
    uint32_t d;
    asm("dp2a.lo.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(r), "r"(0x00000100u), "r"(0u));
    return d;
}

#ifndef AMP_GEMV_HI_FMA_MASK
#define AMP_GEMV_HI_FMA_MASK 0x6      // which of a word's (up to four) pairs take their high state on the FMA pipe
#endif
#ifndef AMP_GEMV_LO_FMA_MASK
#define AMP_GEMV_LO_FMA_MASK 0xf      // ... and their low state
#endif

// The eight 16-bit states of virtual lane R (positions 8R..8R+7 of the lane's chunk).
// When K divides 16, windows 16/K positions apart are exactly 16 bits apart, so one 32-bit
// word cut from the stream holds two states (high and low half): one funnel shift serves two
// weights. Other bitrates cut each window on its own (shift on the ALU, mask on the FMA pipe).
template <int K, int R, bool FMA = true>
__device__ __forceinline__ void states8(const uint32_t (&w)[K], uint32_t prev, uint32_t (&s)[8])
{
    if constexpr (K == 4 || K == 8)
    {
        constexpr int D = 16 / K;                       // pair distance in positions
        int pair = 0;
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
            s[j] = (FMA && ((AMP_GEMV_HI_FMA_MASK >> pair) & 1)) ? hi16_fma(r) : (r >> 16);
            s[j + D] = (FMA && ((AMP_GEMV_LO_FMA_MASK >> pair) & 1)) ? lo16_fma(r) : (r & 0xffffu);
            ++pair;
        }
    }
    else
    {
        s[0] = window_ct<K, R * 8 + 0, K, FMA>(w, prev); s[1] = window_ct<K, R * 8 + 1, K, FMA>(w, prev);
        s[2] = window_ct<K, R * 8 + 2, K, FMA>(w, prev); s[3] = window_ct<K, R * 8 + 3, K, FMA>(w, prev);
        s[4] = window_ct<K, R * 8 + 4, K, FMA>(w, prev); s[5] = window_ct<K, R * 8 + 5, K, FMA>(w, prev);
        s[6] = window_ct<K, R * 8 + 6, K, FMA>(w, prev); s[7] = window_ct<K, R * 8 + 7, K, FMA>(w, prev);
    }
}

// Decode the lane's 8 weights of virtual lane R of one tile and issue the two MMAs (into two
// accumulators, so that they do not wait for each other). w/prev: the lane's K words and the
// word before them. xb: duplicated activations of the tile's 16 rows for this lane's batch
// row(s), xb[r] = row r.
template <int K, int CB, int MB, int R>
__device__ __forceinline__ void decode_mma_r(const uint32_t (&w)[K], uint32_t prev, const uint32_t (&xb)[MB][16],
                                             float (&acc0)[MB][4], float (&acc1)[MB][4])
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
        mma_16816(acc0[mb], a[0], a[4], a[1], a[5], xb[mb][2 * R], xb[mb][2 * R + 1]);
        mma_16816(acc1[mb], a[2], a[6], a[3], a[7], xb[mb][2 * R + 8], xb[mb][2 * R + 9]);
    }
}

// u8 x s8 dot product with int32 accumulation
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Int8-activation form for the mul1 codebook (reference: exl3_gemv_int8_kernel.cuh:19-47): the
// weight is affine in the byte sum of s * M, so dp4a of the product against the activation's int8
// code replicated into four bytes is bytesum * code, accumulated exactly. xs[r] = the replicated
// code of tile row r; a0 / a1: columns gq and gq + 8 of the tile (two chains each). The multiply
// and the dp4a both run on the FMA-heavy pipe, so the field extraction stays on the ALU.
template <int K, int R>
__device__ __forceinline__ void decode_dp4a_r(const uint32_t (&w)[K], uint32_t prev, const uint32_t (&xs)[16],
                                              int (&a0)[2], int (&a1)[2])
{
    uint32_t s[8];
    states8<K, R, false>(w, prev, s);
    a0[0] = dp4a_us(s[0] * 0x83DCD12Du, xs[2 * R], a0[0]);
    a0[1] = dp4a_us(s[2] * 0x83DCD12Du, xs[2 * R + 8], a0[1]);
    a1[0] = dp4a_us(s[4] * 0x83DCD12Du, xs[2 * R], a1[0]);
    a1[1] = dp4a_us(s[6] * 0x83DCD12Du, xs[2 * R + 8], a1[1]);
    a0[0] = dp4a_us(s[1] * 0x83DCD12Du, xs[2 * R + 1], a0[0]);
    a0[1] = dp4a_us(s[3] * 0x83DCD12Du, xs[2 * R + 9], a0[1]);
    a1[0] = dp4a_us(s[5] * 0x83DCD12Du, xs[2 * R + 1], a1[0]);
    a1[1] = dp4a_us(s[7] * 0x83DCD12Du, xs[2 * R + 9], a1[1]);
}

// The same with a second set of activation codes (the int8 rounding error of the first set, quantised
// again): the decoded products are shared, each costs one more dp4a.
template <int K, int R>
__device__ __forceinline__ void decode_dp4a2_r(const uint32_t (&w)[K], uint32_t prev, const uint32_t (&xs)[16], const uint32_t (&xr)[16],
                                               int (&a0)[2], int (&a1)[2], int (&b0)[2], int (&b1)[2])
{
    uint32_t s[8];
    states8<K, R, false>(w, prev, s);
    #pragma unroll
    for (int i = 0; i < 8; ++i) s[i] *= 0x83DCD12Du;
    a0[0] = dp4a_us(s[0], xs[2 * R], a0[0]);         b0[0] = dp4a_us(s[0], xr[2 * R], b0[0]);
    a0[1] = dp4a_us(s[2], xs[2 * R + 8], a0[1]);     b0[1] = dp4a_us(s[2], xr[2 * R + 8], b0[1]);
    a1[0] = dp4a_us(s[4], xs[2 * R], a1[0]);         b1[0] = dp4a_us(s[4], xr[2 * R], b1[0]);
    a1[1] = dp4a_us(s[6], xs[2 * R + 8], a1[1]);     b1[1] = dp4a_us(s[6], xr[2 * R + 8], b1[1]);
    a0[0] = dp4a_us(s[1], xs[2 * R + 1], a0[0]);     b0[0] = dp4a_us(s[1], xr[2 * R + 1], b0[0]);
    a0[1] = dp4a_us(s[3], xs[2 * R + 9], a0[1]);     b0[1] = dp4a_us(s[3], xr[2 * R + 9], b0[1]);
    a1[0] = dp4a_us(s[5], xs[2 * R + 1], a1[0]);     b1[0] = dp4a_us(s[5], xr[2 * R + 1], b1[0]);
    a1[1] = dp4a_us(s[7], xs[2 * R + 9], a1[1]);     b1[1] = dp4a_us(s[7], xr[2 * R + 9], b1[1]);
}

// thread-block cluster helpers: rank of this CTA, address of a shared-memory location in another
// CTA of the cluster, a store there, and the cluster-wide barrier (release / acquire)
__device__ __forceinline__ uint32_t cluster_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ uint32_t cluster_map(uint32_t saddr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}

__device__ __forceinline__ void cluster_st_f32(uint32_t addr, float v)
{
    asm volatile("st.shared::cluster.f32 [%0], %1;" :: "r"(addr), "f"(v) : "memory");
}

__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}


__device__ __forceinline__ void pdl_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void pdl_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Gated activations of the fused MoE (reference: exl3_moe_coop_kernel.cuh:79-132)
__device__ __forceinline__ float moe_act_gate(int act, bool gated, float g, float u, float limit)
{
    if (act == MOE_ACT_SILU_OAI)
    {
        if (limit != 0.0f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
        const float glu = g * (1.0f / (1.0f + __expf(-1.702f * g)));
        return (u + 1.0f) * glu;
    }
    float x;
    if (!gated) x = fmaxf(0.0f, u);
    else if (act == MOE_ACT_SILU) x = g * __fdividef(1.0f, 1.0f + __expf(-g));
    else if (act == MOE_ACT_GELU)
    {
        const float t = 0.797884560803f * (g + 0.044715f * g * g * g);
        x = 0.5f * g * (1.0f + tanhf(t));
    }
    else { x = fmaxf(0.0f, g); x = x * x; }
    if (limit != 0.0f) { u = fminf(fmaxf(u, -limit), limit); x = fminf(x, limit); }
    return x * u;
}

#ifndef AMP_GEMV_TB
#define AMP_GEMV_TB 6               // x~ tasks whose loads are in flight together (per warp and pass)
#endif
#ifndef AMP_GEMV_MINBLOCKS
#define AMP_GEMV_MINBLOCKS 3
#endif

__device__ __forceinline__ void cp_async16_s(uint32_t dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst), "l"(src) : "memory");
}

template <int N>
__device__ __forceinline__ void cp_async_wait_n()
{
    asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory");
}

// The CTAs' ranges: U units over ncta CTAs, the first r ranges one unit longer (q = U / ncta,
// r = U % ncta). All 32-bit, no division on the way from a CTA to its range.
struct GemvSplit
{
    int q, r;
    __device__ __forceinline__ int begin(int i) const { return i * q + min(i, r); }
    __device__ __forceinline__ int owner(int u) const
    {
        const int edge = r * (q + 1);
        return u < edge ? u / (q + 1) : r + (u - edge) / q;
    }
};

// All-reduced input of one x~ chunk (split exchange) into a staging area: `total` units of four
// values, `upr` units per batch row starting at unit `first` of each row. A unit is the N ranks'
// flag-in-data words; U units per thread are in flight at a time: all their words are loaded at
// once, the ones not yet there are polled with a bound, then fp32 sum in rank order and one
// rounding -- the stand-alone all-reduce's arithmetic.
template <int U, int NMAX>
__device__ __forceinline__ void gather_chunk(half4* stage, const uint2* gbase, int N, long wcap, uint32_t seq, int* ctl,
                                             int total, int upr, long row_units, long first, int t)
{
    for (int u = t; u < total; u += U * GEMV_THREADS)
    {
        uint32_t v[U][NMAX][4];
        const uint2* src[U];
        #pragma unroll
        for (int i = 0; i < U; ++i)
        {
            const int ui = u + i * GEMV_THREADS;
            if (ui >= total) continue;
            const int b = ui / upr;
            src[i] = gbase + 2 * ((long) b * row_units + first + (ui - b * upr));
            #pragma unroll
            for (int p = 0; p < NMAX; ++p)
                if (p < N) ld_ll2_once(src[i] + (long) p * wcap, v[i][p]);
        }
        #pragma unroll
        for (int i = 0; i < U; ++i)
        {
            const int ui = u + i * GEMV_THREADS;
            if (ui >= total) continue;
            unsigned budget = COMM_SPIN_LIMIT;
            float acc[4] = { 0.f, 0.f, 0.f, 0.f };
            #pragma unroll
            for (int p = 0; p < NMAX; ++p)
            {
                if (p >= N) continue;
                uint32_t d0 = v[i][p][0], d1 = v[i][p][2];
                if (v[i][p][1] != seq || v[i][p][3] != seq)
                    if (!ld_ll2(src[i] + (long) p * wcap, seq, &d0, &d1, budget)) { atomicExch(ctl + COMM_MAXB, 1); d0 = d1 = 0; }
                acc4(acc, d0, d1);
            }
            half4 r;
            r.x = __floats2half2_rn(acc[0], acc[1]);
            r.y = __floats2half2_rn(acc[2], acc[3]);
            stage[ui] = r;
        }
    }
}

// The last arriver's sum of a column block's partials (slots [cta][2][m][128] fp32; contributor i's
// partial sits in slot 2 i, the first contributor's in first_slot), added in ascending k order into
// part: deterministic. Kept out of line so that its registers are not the main loop's. One batch row:
// four contributors' loads in flight per thread (one after the other they are a chain of L2 round
// trips on the critical path of the launch). Several rows: a thread would walk rows x contributors
// round trips, so the partials are staged through the x~ area (free at this point) with 16-byte
// asynchronous copies, as many contributors per batch as it holds, all in flight at once, and the
// adds run from shared memory in the same order.
static __device__ __forceinline__ void gemv_reduce_partials_body(float* part, const float* slots, const float* stage, uint32_t stage_s, int stage_bytes,
                                                                 int m, int nrows, int i_first, int i_last, int first_slot, int t)
{
    if (nrows >= 2)
    {
        const int pieces = nrows * 32;                         // 16-byte pieces of one partial
        const int cap = stage_bytes / (pieces * 16);           // contributors per batch (>= 2)
        for (int c0 = i_first; c0 <= i_last; c0 += cap)
        {
            const int nb = min(cap, i_last - c0 + 1);
            for (int e = t; e < nb * pieces; e += GEMV_THREADS)
            {
                const int ci = e / pieces, pc = e - ci * pieces, i = c0 + ci;
                cp_async16_s(stage_s + e * 16, slots + (size_t) (i == i_first ? first_slot : 2 * i) * m * 128 + pc * 4);
            }
            cp_async_commit();
            cp_async_wait_n<0>();
            __syncthreads();
            for (int idx = t; idx < nrows * 128; idx += GEMV_THREADS)
            {
                float sum = (c0 == i_first) ? stage[idx] : part[idx];
                for (int ci = (c0 == i_first) ? 1 : 0; ci < nb; ++ci) sum += stage[ci * nrows * 128 + idx];
                part[idx] = sum;
            }
            __syncthreads();
        }
        return;
    }
    const size_t pitch = (size_t) 2 * m * 128;                 // floats between consecutive contributors' slots
    for (int idx = t; idx < nrows * 128; idx += GEMV_THREADS)
    {
        float sum = __ldcg(slots + (size_t) first_slot * m * 128 + idx);
        const float* src = slots + (size_t) (i_first + 1) * pitch + idx;
        for (int i = i_first + 1; i <= i_last; i += 8, src += 8 * pitch)
        {
            float v[8];
            #pragma unroll
            for (int j = 0; j < 8; ++j)
                if (i + j <= i_last) v[j] = __ldcg(src + j * pitch);
            #pragma unroll
            for (int j = 0; j < 8; ++j)
                if (i + j <= i_last) sum += v[j];
        }
        part[idx] = sum;
    }
}

// (used by the instance that serves five rows and more; out of line so that it does not shape the
// main loop's code. The other instances keep a plain in-line form: their code shape is what the
// one-row step and the single-token MoE were tuned on, and any change to it costs them 1-12 %.)
static __device__ __noinline__ void gemv_reduce_partials(float* part, const float* slots, const float* stage, uint32_t stage_s, int stage_bytes,
                                                         int m, int nrows, int i_first, int i_last, int first_slot, int t)
{
    gemv_reduce_partials_body(part, slots, stage, stage_s, stage_bytes, m, nrows, i_first, i_last, first_slot, t);
}

// MODE 0: one matrix or a bundle sharing one input.  MODE 1: grouped expert gate/up (slice = expert
// run x projection, input rows gathered by token).  MODE 2: grouped expert down (input = the
// activation of the run's gate/up rows, computed on the fly).
// GIN: MODE 0 instances with another input side. 1: the input is gathered from the all-reduce
// buffers (GemvArIn). 2: the input arrives already rotated (several batch rows, gemv_prerotate_kernel).
// 3: the input is silu(x) * x2 of two vectors (the gated activation in front of a down projection).
// 4: the input is RMSNorm(x + x2) * norm_w (residual add and norm in front of q|k|v, gate|up, lm_head).
// 5 / 6: the same norm split between the producer of the residual contribution (its epilogue adds it to
// the stream and leaves per-block sums of squares) and the consumer (its prologue only scales).
template <int K, int CB, int MB, int MODE = 0, int GIN = 0>
__global__ __launch_bounds__(GEMV_THREADS, (MB == 1 ? AMP_GEMV_MINBLOCKS : 3))
void exl3_gemv_kernel(const GemvParams P)
{
    extern __shared__ __align__(128) unsigned char smem[];
    const GemvSmem L = gemv_smem_layout(K, P.m, P.xgroups, P.cluster, GIN == 1, (GIN == 4 || CB == 4) ? P.rowbuf : 0);
    const int XPITCH = gemv_xpitch(P.xgroups);
    const int XG = P.xgroups;
    float* part = reinterpret_cast<float*>(smem + L.part);
    uint32_t* xd = reinterpret_cast<uint32_t*>(smem + L.xd);
    float* gsum = reinterpret_cast<float*>(smem + L.gsum);
    float* qs = reinterpret_cast<float*>(smem + L.qs);
    uint32_t* xd2 = reinterpret_cast<uint32_t*>(smem + L.total - (CB == 4 ? P.rowbuf : 0));   // CB 4: second set of int8 codes
    (void) xd2;
    __shared__ int s_last;

    constexpr int S = gemv_stages(K);
    constexpr int RP = gemv_row_pitch(K);
    constexpr int SLOT = gemv_slot_bytes(K);
    constexpr int TILE_BYTES = 32 * K;
    constexpr int NT = GEMV_NT;
    constexpr int ROWP = NT * 2 * K;                   // 16-byte pieces per tile row of a unit
    constexpr int PIECES = 4 * ROWP;                   // ... and per unit
    constexpr int NP = (PIECES + 31) / 32;             // copy instructions per unit and lane

    // Dependent launch: the next kernel's CTAs may be scheduled from now on. The launch asks for
    // so much shared memory that an SM holds exactly this grid's share of CTAs, so they only move
    // in as CTAs of this grid leave -- one for one, which keeps the next grid evenly spread --
    // and start their weight stream under this grid's partial-sum exchange.
    // The gate/up launch of the grouped mode (MODE 1) needs the routing (or the run table built from
    // it) before anything else and releases its dependents only once that has arrived, so that
    // the down launch (MODE 2), which starts under it, may read the same without a wait of its own.
    if constexpr (MODE == 1) { if (P.pdl) { pdl_wait(); pdl_launch_dependents(); } }
    else if (P.pdl) pdl_launch_dependents();
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int gq = lane >> 2, pq = lane & 3;
    const int m = P.m, k = P.k;
    const int G = k >> 6;                              // 64-row groups per column block
    const int nbw = P.width >> 7;                      // column blocks per slice

    // Work = (column block, group) units in block-major order, cut into equal contiguous ranges:
    // every CTA decodes the same number of weights (+-1 group) whatever the shape.
    const int nproj = (MODE == 1 && P.moe.gated) ? 2 : 1;
    const int* runs = P.moe.runs;                      // [0] run count, [1] active slots, then the runs
    __shared__ int s_runs[2 + 16 * MOE_RUN_INTS];
    int inline_active = 0;
    if constexpr (MODE != 0)
    {
        if (P.moe.inline_runs)
        {
            // one token: its active picks, in pick order, are the runs (one row each); lane i of
            // the first warp reads pick i
            if (t < 32)
            {
                MoeSlot si; si.active = false; si.local = 0;
                if (t < P.moe.topk)
                    si = moe_slot(P.moe.sel, P.moe.rw, P.moe.topk, P.moe.min_expert, P.moe.max_expert, P.moe.n_local, t);
                const unsigned act = __ballot_sync(0xffffffffu, si.active);
                if (si.active)
                {
                    int* rec = s_runs + 2 + __popc(act & ((1u << t) - 1u)) * MOE_RUN_INTS;
                    rec[0] = si.local; rec[1] = 1; rec[2] = t; rec[3] = 0;
                }
                if (t == 0) s_runs[0] = s_runs[1] = __popc(act);
            }
            __syncthreads();
            runs = s_runs;
            inline_active = s_runs[0];
        }
    }
    // mixed bit widths: the runs this launch works on (those whose expert has this instance's width)
    __shared__ unsigned char s_sel[256];
    __shared__ int s_nsel;
    bool filtered = false;
    int nruns = 0;
    if constexpr (MODE != 0)
    {
        nruns = runs[0];
        const unsigned char* bits = P.moe.bits[MODE == 2 ? 2 : 1];
        if (bits)
        {
            filtered = true;
            if (t < 32)
            {
                int count = 0;
                for (int base = 0; base < nruns; base += 32)
                {
                    const int r = base + t;
                    const bool hit = r < nruns && bits[runs[2 + r * MOE_RUN_INTS]] == K;
                    const unsigned m32 = __ballot_sync(0xffffffffu, hit);
                    if (hit) s_sel[count + __popc(m32 & ((1u << t) - 1u))] = (unsigned char) r;
                    count += __popc(m32);
                }
                if (t == 0) s_nsel = count;
            }
            __syncthreads();
            nruns = s_nsel;
        }
    }
    const int U = (MODE == 0 ? P.blocks : nruns * nproj * nbw) * G;
    const int cta = blockIdx.x, ncta = min((int) gridDim.x, U);    // never more ranges than units
    if constexpr (MODE == 2)
    {
        // a single token without any local pick: nobody will deliver a slot, the row is still due
        if (P.moe.inline_runs && inline_active == 0 && cta == 0 && P.moe.first_down)
            for (int c = warp; c < (P.moe.Ho >> 7); c += GEMV_WARPS) moe_combine_chunk(P.moe, 0, c, lane);
    }
    if (cta >= ncta) return;                           // an exited CTA counts as having released its dependents
    GemvSplit split;
    split.q = U / ncta;
    split.r = U - split.q * ncta;
    int u0 = split.begin(cta), u1 = split.begin(cta + 1);
    if constexpr (MODE != 0)
    {
        if (P.cluster)
        {
            // cluster form of a grouped launch (one token): the grid holds a cluster per column
            // block of every pick; the clusters of picks that turn out inactive leave as a whole
            const int cblk = cta / P.cluster, per = G / P.cluster;
            if (cblk * G >= U) return;
            u0 = cblk * G + (cta - cblk * P.cluster) * per;
            u1 = u0 + per;
        }
    }

    const uint32_t ring_s = smem_u32(smem + L.ring) + warp * (S * SLOT);      // this warp's ring

    // ---- weight stream: a cursor walks the range's units; piece p = lane + 32 j of a unit is
    // 16 bytes of tile row p / ROWP ----
    int iu = u0;                                       // next unit to fetch
    int iblk = iu / G, ig = iu - iblk * G;
    uint32_t islot = 0;                                // byte offset of the next slot to fill
    const unsigned char* isrc[NP];                     // this lane's pieces of the cursor's unit
    size_t istep = 0;                                  // bytes from one unit to the next (four tile rows)
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
        if constexpr (MODE != 0)
        {
            const int srun = slice / nproj, proj = (MODE == 2) ? 2 : (P.moe.gated ? slice - srun * nproj : 1);
            const int run = filtered ? s_sel[srun] : srun;
            const int expert = runs[2 + run * MOE_RUN_INTS];
            tr = reinterpret_cast<const unsigned char*>(P.moe.trellis[proj][expert]);
            stride = P.width;
        }
        else if (P.tables)
        {
            tr = reinterpret_cast<const unsigned char*>(P.t_trellis[slice]);
            stride = P.t_stride ? P.t_stride[slice] : P.width;
        }
        const size_t irow = (size_t) (stride >> 4) * TILE_BYTES;          // bytes between tile rows
        const unsigned char* base = tr + (size_t) (nb * 8 + warp * NT) * TILE_BYTES + (size_t) (4 * g) * irow;
        istep = 4 * irow;
        #pragma unroll
        for (int j = 0; j < NP; ++j)
        {
            const int p = lane + 32 * j, row = p / ROWP;
            isrc[j] = base + (size_t) row * irow + (p - row * ROWP) * 16;
        }
    };

    // A group is committed even when nothing is left to copy so that the group count stays in
    // step with the unit index.
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

    // the two lines of svh this CTA may need at the very end are pulled into L2 now
    if constexpr (MODE == 0)
    {
        if (t < 2)
        {
            const int slice0 = iblk / nbw;
            const __half* svh0 = P.tables ? reinterpret_cast<const __half*>(P.t_svh[slice0]) : P.svh;
            asm volatile("prefetch.global.L2 [%0];" :: "l"(svh0 + (size_t) (iblk - slice0 * nbw) * 128 + t * 64));
        }
    }

    // The weight stream does not depend on the previous kernel. With dependent launch it starts
    // before the wait for that kernel; otherwise right behind the loads of the first x~ pass
    // (those are tiny and must not queue behind the weight burst of the whole grid).
    if (iu < u1) set_block(iblk, ig);
    bool started = false;
    if (MODE != 0 || P.pdl)
    {
        #pragma unroll
        for (int j = 0; j < S - 1; ++j) issue();
        started = true;
    }
    bool waited = (MODE == 1);                         // MODE 0 / 2 wait for their predecessor inside the first x~ pass

    // GIN == 4: the input is RMSNorm(x + x2) * norm_w (reference: amp_rms_norm_res_kernel,
    // src/torch/amp_kernels.cu:279-360: y = fp16(x + r); n = fp16(y * rsqrt(mean(y^2) + eps)) * w in
    // fp16). Every CTA needs the row's sum of squares, so every CTA reads the whole row once (it is
    // L2 resident) while its weight stream is in flight; the first CTA also writes y.
    __shared__ float s_scale[16];
    if constexpr (GIN == 4)
    {
        __shared__ float s_red[16][GEMV_WARPS];
        if (!started)
        {
            #pragma unroll
            for (int j = 0; j < S - 1; ++j) issue();
            started = true;
        }
        const int cnt = k >> 2;
        if (P.rowbuf)
        {
            // One row, short enough to sit in shared memory: the static vectors (norm weight, suh of
            // the first source) are copied in BEFORE the wait for the producer, the row itself takes a
            // single batch of loads after it, and the x~ passes then read everything from shared
            // memory: one L2 round trip on the critical path, like the plain kernel.
            half4* s_y = reinterpret_cast<half4*>(smem + L.total - P.rowbuf);
            const uint32_t s_w = smem_u32(s_y) + k * 2;
            for (int c = t; c < cnt / 2; c += GEMV_THREADS) cp_async16_s(s_w + c * 16, P.norm_w + c * 8);
            cp_async_commit();
            if (!waited) { if (P.pdl) pdl_wait(); waited = true; }
            float acc = 0.0f;
            for (int c0 = t; c0 < cnt; c0 += 8 * GEMV_THREADS)
            {
                half4 xv[8], rv[8];
                #pragma unroll
                for (int j = 0; j < 8; ++j)
                {
                    const int c = c0 + j * GEMV_THREADS;
                    if (c < cnt) { xv[j] = reinterpret_cast<const half4*>(P.x)[c]; rv[j] = reinterpret_cast<const half4*>(P.x2)[c]; }
                }
                #pragma unroll
                for (int j = 0; j < 8; ++j)
                {
                    const int c = c0 + j * GEMV_THREADS;
                    if (c >= cnt) continue;
                    half4 h;
                    h.x = __floats2half2_rn(__low2float(xv[j].x) + __low2float(rv[j].x), __high2float(xv[j].x) + __high2float(rv[j].x));
                    h.y = __floats2half2_rn(__low2float(xv[j].y) + __low2float(rv[j].y), __high2float(xv[j].y) + __high2float(rv[j].y));
                    s_y[c] = h;
                    if (cta == 0) reinterpret_cast<half4*>(P.y)[c] = h;
                    const float2 v0 = __half22float2(h.x), v1 = __half22float2(h.y);
                    acc += v0.x * v0.x + v0.y * v0.y;
                    acc += v1.x * v1.x + v1.y * v1.y;
                }
            }
            #pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0) s_red[0][warp] = acc;
            cp_async_wait_n<0>();                       // the norm weight (and the first weights: long since there)
        }
        else
        {
        if (!waited) { if (P.pdl) pdl_wait(); waited = true; }
        for (int b = 0; b < m; ++b)
        {
            const __half* xr = P.x + (size_t) b * k;
            const __half* rr = P.x2 + (size_t) b * k;
            float acc = 0.0f;
            for (int c0 = t; c0 < cnt; c0 += 4 * GEMV_THREADS)
            {
                // four chunks per thread in flight: one after the other they are a chain of L2 round trips
                half4 xv[4], rv[4];
                #pragma unroll
                for (int j = 0; j < 4; ++j)
                {
                    const int c = c0 + j * GEMV_THREADS;
                    if (c < cnt) { xv[j] = reinterpret_cast<const half4*>(xr)[c]; rv[j] = reinterpret_cast<const half4*>(rr)[c]; }
                }
                #pragma unroll
                for (int j = 0; j < 4; ++j)
                {
                    const int c = c0 + j * GEMV_THREADS;
                    if (c >= cnt) continue;
                    half4 h;
                    h.x = __floats2half2_rn(__low2float(xv[j].x) + __low2float(rv[j].x), __high2float(xv[j].x) + __high2float(rv[j].x));
                    h.y = __floats2half2_rn(__low2float(xv[j].y) + __low2float(rv[j].y), __high2float(xv[j].y) + __high2float(rv[j].y));
                    if (cta == 0) reinterpret_cast<half4*>(P.y + (size_t) b * k)[c] = h;
                    const float2 v0 = __half22float2(h.x), v1 = __half22float2(h.y);
                    acc += v0.x * v0.x + v0.y * v0.y;
                    acc += v1.x * v1.x + v1.y * v1.y;
                }
            }
            #pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0) s_red[b][warp] = acc;
        }
        }
        __syncthreads();
        if (t < m)
        {
            float total = 0.0f;
            #pragma unroll
            for (int i = 0; i < GEMV_WARPS; ++i) total += s_red[t][i];
            s_scale[t] = rsqrtf(total / (float) k + P.eps);
        }
        __syncthreads();
    }

    // per-lane constants of the consume side
    int xrow[MB];                                      // word offset of this lane's batch row in xd
    #pragma unroll
    for (int mb = 0; mb < MB; ++mb) xrow[mb] = min(mb * 8 + gq, m - 1) * XPITCH + pq * 4;
    const uint32_t w_off = ring_s + pq * RP + gq * K * 4;                             // this lane's K words of the first tile
    const uint32_t p_off = ring_s + pq * RP + ((gq * K + 8 * K - 1) % (8 * K)) * 4;   // the word before them (ring)
    const uint32_t xd_s = smem_u32(xd);

    uint32_t cslot = 0;                                // byte offset of the next slot to consume
    int useg = u0;
    while (useg < u1)
    {
        // ---- one segment: the part of this CTA's range that lies in one column block ----
        const int blk = useg / G;
        const int g0 = useg - blk * G;
        const int g1 = min(G, g0 + (u1 - useg));
        const int slice = blk / nbw, nb = blk - slice * nbw;
        const __half* suh = P.suh;
        const __half* svh = P.svh;
        const __half* bias = nullptr;
        unsigned char* cbase = reinterpret_cast<unsigned char*>(P.c);
        int stride = P.stride;
        int nrows = m;                                 // batch rows of this segment
        const unsigned char* run_slots = nullptr;      // grouped modes: the run's slot indices
        const __half* xrot = P.x;                      // GIN == 2: this slice's rotated input
        if constexpr (MODE != 0)
        {
            const int srun = slice / nproj, proj = (MODE == 2) ? 2 : (P.moe.gated ? slice - srun * nproj : 1);
            const int run = filtered ? s_sel[srun] : srun;
            const int* rec = runs + 2 + run * MOE_RUN_INTS;
            const int expert = rec[0];
            nrows = rec[1];
            run_slots = reinterpret_cast<const unsigned char*>(rec + 2);
            suh = reinterpret_cast<const __half*>(P.moe.suh[proj][expert]);
            svh = reinterpret_cast<const __half*>(P.moe.svh[proj][expert]);
            if (P.moe.bias[proj]) bias = reinterpret_cast<const __half*>(P.moe.bias[proj][expert]);
            cbase = reinterpret_cast<unsigned char*>(MODE == 2 ? P.moe.d_out : P.moe.gu[proj]);
            stride = P.width;
            // the expert's output scales are needed at the very end: pull their lines into L2 now
            if (t < 2) asm volatile("prefetch.global.L2 [%0];" :: "l"(svh + (size_t) nb * 128 + t * 64));
            #pragma unroll
            for (int mb = 0; mb < MB; ++mb) xrow[mb] = min(mb * 8 + gq, nrows - 1) * XPITCH + pq * 4;
        }
        else if (P.tables)
        {
            const int src = P.t_src ? P.t_src[slice] : slice;
            if constexpr (GIN == 2) xrot = P.x + (size_t) src * m * k;
            suh = reinterpret_cast<const __half*>(P.t_suh[src]);
            svh = reinterpret_cast<const __half*>(P.t_svh[slice]);
            stride = P.t_stride ? P.t_stride[slice] : P.width;
            if (P.t_c) cbase = reinterpret_cast<unsigned char*>(P.t_c[slice]);
            else cbase += (size_t) slice * m * P.width * (P.c_fp32 ? 4 : 2);
        }

        float acc0[NT][MB][4], acc1[NT][MB][4];        // this warp's tile columns x this lane's batch rows
        #pragma unroll
        for (int nt = 0; nt < NT; ++nt)
            #pragma unroll
            for (int mb = 0; mb < MB; ++mb)
            {
                acc0[nt][mb][0] = acc0[nt][mb][1] = acc0[nt][mb][2] = acc0[nt][mb][3] = 0.f;
                acc1[nt][mb][0] = acc1[nt][mb][1] = acc1[nt][mb][2] = acc1[nt][mb][3] = 0.f;
            }
        float xsum[MB][2];                             // cb 2 only: sum of x~ over the segment's rows, batch rows 2pq, 2pq+1
        #pragma unroll
        for (int mb = 0; mb < MB; ++mb) xsum[mb][0] = xsum[mb][1] = 0.f;

        // x~ is needed in whole 128-row blocks: chunks start at an even group
        for (int cg0 = g0 & ~1; cg0 < g1; cg0 += XG)
        {
            const int cg1 = min(cg0 + XG, g1);
            const int nblk = (cg1 - cg0 + 1) >> 1;      // 128-row blocks in this chunk
            __syncthreads();                            // previous x~ fully consumed

            // x~ = fp16(H(x * suh) / sqrt(128)), stored duplicated ((v, v) per word) and in the
            // order the B fragments are read: word = group*64 + (row%16 / 4)*16 + (row%64 / 16)*4 + row%4.
            // Tasks (batch row b, 128-row block jb) go round the warps.
            // store one task's four rotated values per lane; b, jb name the task
            auto frag_store = [&](int b, int jb, const __half2 o01, const __half2 o23)
            {
                if constexpr (CB == 3 || CB == 4)
                {
                    // int8 activations: one scale per 128-row block (this warp's task), codes
                    // replicated into the four bytes of the word the fp16 pair would occupy
                    const float v0 = __low2float(o01), v1 = __high2float(o01), v2 = __low2float(o23), v3 = __high2float(o23);
                    float mx = fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)));
                    #pragma unroll
                    for (int i = 16; i > 0; i >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, i));
                    const float inv = mx > 0.0f ? __fdiv_rn(127.0f, mx) : 0.0f;
                    const int i0 = __float2int_rn(v0 * inv), i1 = __float2int_rn(v1 * inv);
                    const int i2 = __float2int_rn(v2 * inv), i3 = __float2int_rn(v3 * inv);
                    uint4 d;
                    d.x = (uint32_t) (i0 & 0xff) * 0x01010101u; d.y = (uint32_t) (i1 & 0xff) * 0x01010101u;
                    d.z = (uint32_t) (i2 & 0xff) * 0x01010101u; d.w = (uint32_t) (i3 & 0xff) * 0x01010101u;
                    const int r = jb * 128 + lane * 4;
                    const int word = (r >> 6) * 64 + ((r & 15) >> 2) * 16 + ((r & 63) >> 4) * 4;
                    *reinterpret_cast<uint4*>(xd + b * XPITCH + word) = d;
                    const float q = __fdiv_rn(mx, 127.0f);
                    // per 64-row group (lanes 0-15 / 16-31): the dequantised sum of the codes and the scale
                    int si = (i0 + i1) + (i2 + i3);
                    #pragma unroll
                    for (int i = 1; i < 16; i <<= 1) si += __shfl_xor_sync(0xffffffffu, si, i);
                    float gs = q * (float) si;
                    if constexpr (CB == 4)
                    {
                        // error feedback: the rounding error of the first code (within +- q / 2) quantised with
                        // the fixed scale q / 254 (reference: gemv_int8_stage_splats, exl3_gemv_int8_kernel.cuh:251-280)
                        const float inv2 = mx > 0.0f ? 254.0f * inv : 0.0f;
                        auto code2 = [&](float v, int c) { return max(-127, min(127, __float2int_rn(fmaf(-q, (float) c, v) * inv2))); };
                        const int j0 = code2(v0, i0), j1 = code2(v1, i1), j2 = code2(v2, i2), j3 = code2(v3, i3);
                        uint4 e;
                        e.x = (uint32_t) (j0 & 0xff) * 0x01010101u; e.y = (uint32_t) (j1 & 0xff) * 0x01010101u;
                        e.z = (uint32_t) (j2 & 0xff) * 0x01010101u; e.w = (uint32_t) (j3 & 0xff) * 0x01010101u;
                        *reinterpret_cast<uint4*>(xd2 + b * XPITCH + word) = e;
                        int sj = (j0 + j1) + (j2 + j3);
                        #pragma unroll
                        for (int i = 1; i < 16; i <<= 1) sj += __shfl_xor_sync(0xffffffffu, sj, i);
                        gs = fmaf(q * (1.0f / 254.0f), (float) sj, gs);
                    }
                    if ((lane & 15) == 0)
                    {
                        gsum[b * XG + 2 * jb + (lane >> 4)] = gs;
                        qs[b * XG + 2 * jb + (lane >> 4)] = q;
                    }
                    return;
                }
                const uint32_t u01 = *reinterpret_cast<const uint32_t*>(&o01);
                const uint32_t u23 = *reinterpret_cast<const uint32_t*>(&o23);
                uint4 d;
                d.x = __byte_perm(u01, u01, 0x1010); d.y = __byte_perm(u01, u01, 0x3232);
                d.z = __byte_perm(u23, u23, 0x1010); d.w = __byte_perm(u23, u23, 0x3232);
                const int r = jb * 128 + lane * 4;      // row inside the chunk
                const int word = (r >> 6) * 64 + ((r & 15) >> 2) * 16 + ((r & 63) >> 4) * 4;
                *reinterpret_cast<uint4*>(xd + b * XPITCH + word) = d;
                if constexpr (CB == 2)
                {
                    // sum of the rounded x~ over each 64-row group (lanes 0-15 / 16-31), fixed order
                    float sg = (__low2float(o01) + __high2float(o01)) + (__low2float(o23) + __high2float(o23));
                    #pragma unroll
                    for (int i = 1; i < 16; i <<= 1) sg += __shfl_xor_sync(0xffffffffu, sg, i);
                    if ((lane & 15) == 0) gsum[b * XG + 2 * jb + (lane >> 4)] = sg;
                }
            };
            auto had_store = [&](int b, int jb, float h0, float h1, float h2, float h3)
            {
                warp_had128(h0, h1, h2, h3, lane);
                frag_store(b, jb, __floats2half2_rn(h0 * kRScale, h1 * kRScale), __floats2half2_rn(h2 * kRScale, h3 * kRScale));
            };
            if constexpr (MODE == 0 && GIN == 2)
            {
                // The input arrives rotated (fp16 x~ of every source, written by gemv_prerotate_kernel
                // right before this launch): only the copy into fragment order is left, eight tasks
                // per pass. With several batch rows the rotation would otherwise be repeated by every
                // CTA for all rows of its range.
                if (!waited) { if (P.pdl) pdl_wait(); waited = true; }
                int b = 0, jb = warp;
                while (jb >= nblk && b < nrows) { jb -= nblk; ++b; }
                do
                {
                    constexpr int TB = 8;
                    half4 vx[TB];
                    int tb[TB], tj[TB];
                    #pragma unroll
                    for (int i = 0; i < TB; ++i)
                    {
                        tb[i] = b; tj[i] = jb;
                        if (b < nrows)
                        {
                            vx[i] = *reinterpret_cast<const half4*>(xrot + (size_t) b * k + (size_t) cg0 * 64 + (size_t) jb * 128 + lane * 4);
                            jb += GEMV_WARPS;
                            while (jb >= nblk && b < nrows) { jb -= nblk; ++b; }
                        }
                        else tb[i] = -1;
                    }
                    if (!started)
                    {
                        #pragma unroll
                        for (int j = 0; j < S - 1; ++j) issue();
                        started = true;
                    }
                    #pragma unroll
                    for (int i = 0; i < TB; ++i)
                        if (tb[i] >= 0) frag_store(tb[i], tj[i], vx[i].x, vx[i].y);
                } while (b < nrows);
            }
            else if constexpr (MODE == 0 && GIN == 3)
            {
                // The input is the gated activation of two vectors, computed here instead of by a
                // kernel of its own between the gate|up bundle and this launch: a = fp16(silu(g) * u)
                // in fp32 exactly as the stand-alone kernel forms it (reference: amp_silu_mul_kernel,
                // src/torch/amp_kernels.cu:235-251), then the usual fp16 scale and rotation.
                int b = 0, jb = warp;
                while (jb >= nblk && b < nrows) { jb -= nblk; ++b; }
                do
                {
                    constexpr int TB = 4;
                    half4 vg[TB], vu[TB], vs[TB];
                    int tb[TB], tj[TB];
                    #pragma unroll
                    for (int i = 0; i < TB; ++i)
                    {
                        tb[i] = b; tj[i] = jb;
                        if (b < nrows)
                        {
                            vs[i] = *reinterpret_cast<const half4*>(suh + (size_t) cg0 * 64 + (size_t) jb * 128 + lane * 4);
                            jb += GEMV_WARPS;
                            while (jb >= nblk && b < nrows) { jb -= nblk; ++b; }
                        }
                        else tb[i] = -1;
                    }
                    if (!waited) { if (P.pdl) pdl_wait(); waited = true; }
                    #pragma unroll
                    for (int i = 0; i < TB; ++i)
                        if (tb[i] >= 0)
                        {
                            const size_t off = (size_t) tb[i] * k + (size_t) cg0 * 64 + (size_t) tj[i] * 128 + lane * 4;
                            vg[i] = *reinterpret_cast<const half4*>(P.x + off);
                            vu[i] = *reinterpret_cast<const half4*>(P.x2 + off);
                        }
                    if (!started)
                    {
                        #pragma unroll
                        for (int j = 0; j < S - 1; ++j) issue();
                        started = true;
                    }
                    #pragma unroll
                    for (int i = 0; i < TB; ++i)
                    {
                        if (tb[i] < 0) continue;
                        auto act1 = [](float gf, float uf) { return (gf / (1.0f + __expf(-gf))) * uf; };
                        half4 v;
                        v.x = __floats2half2_rn(act1(__low2float(vg[i].x), __low2float(vu[i].x)), act1(__high2float(vg[i].x), __high2float(vu[i].x)));
                        v.y = __floats2half2_rn(act1(__low2float(vg[i].y), __low2float(vu[i].y)), act1(__high2float(vg[i].y), __high2float(vu[i].y)));
                        v.x = __hmul2(v.x, vs[i].x);
                        v.y = __hmul2(v.y, vs[i].y);
                        had_store(tb[i], tj[i], __low2float(v.x), __high2float(v.x), __low2float(v.y), __high2float(v.y));
                    }
                } while (b < nrows);
            }
            else if constexpr (MODE == 0 && GIN == 4)
            {
                // normalised input: n = fp16(fp16(x + r) * scale) * w (fp16), then the usual scale and rotation
                int b = 0, jb = warp;
                while (jb >= nblk && b < nrows) { jb -= nblk; ++b; }
                if (P.rowbuf)
                {
                    // y and the norm weight come from shared memory; only suh (this source's) is loaded
                    const half4* s_y = reinterpret_cast<const half4*>(smem + L.total - P.rowbuf);
                    const half4* s_wv = s_y + (k >> 2);
                    const float sc = s_scale[0];
                    for (; jb < nblk; jb += GEMV_WARPS)
                    {
                        const int c = cg0 * 16 + jb * 32 + lane;               // 4-half chunk of the row
                        const half4 vs1 = *reinterpret_cast<const half4*>(suh + (size_t) c * 4);
                        const half4 h = s_y[c], wv = s_wv[c];
                        half4 v;
                        v.x = __hmul2(__floats2half2_rn(__low2float(h.x) * sc, __high2float(h.x) * sc), wv.x);
                        v.y = __hmul2(__floats2half2_rn(__low2float(h.y) * sc, __high2float(h.y) * sc), wv.y);
                        v.x = __hmul2(v.x, vs1.x);
                        v.y = __hmul2(v.y, vs1.y);
                        had_store(0, jb, __low2float(v.x), __high2float(v.x), __low2float(v.y), __high2float(v.y));
                    }
                }
                else
                do
                {
                    constexpr int TB = 3;
                    half4 vg[TB], vu[TB], vs[TB], vw[TB];
                    int tb[TB], tj[TB];
                    #pragma unroll
                    for (int i = 0; i < TB; ++i)
                    {
                        tb[i] = b; tj[i] = jb;
                        if (b < nrows)
                        {
                            const size_t col = (size_t) cg0 * 64 + (size_t) jb * 128 + lane * 4;
                            vs[i] = *reinterpret_cast<const half4*>(suh + col);
                            vw[i] = *reinterpret_cast<const half4*>(P.norm_w + col);
                            vg[i] = *reinterpret_cast<const half4*>(P.x + (size_t) b * k + col);
                            vu[i] = *reinterpret_cast<const half4*>(P.x2 + (size_t) b * k + col);
                            jb += GEMV_WARPS;
                            while (jb >= nblk && b < nrows) { jb -= nblk; ++b; }
                        }
                        else tb[i] = -1;
                    }
                    #pragma unroll
                    for (int i = 0; i < TB; ++i)
                    {
                        if (tb[i] < 0) continue;
                        const float sc = s_scale[tb[i]];
                        half4 h, v;
                        h.x = __floats2half2_rn(__low2float(vg[i].x) + __low2float(vu[i].x), __high2float(vg[i].x) + __high2float(vu[i].x));
                        h.y = __floats2half2_rn(__low2float(vg[i].y) + __low2float(vu[i].y), __high2float(vg[i].y) + __high2float(vu[i].y));
                        v.x = __hmul2(__floats2half2_rn(__low2float(h.x) * sc, __high2float(h.x) * sc), vw[i].x);
                        v.y = __hmul2(__floats2half2_rn(__low2float(h.y) * sc, __high2float(h.y) * sc), vw[i].y);
                        v.x = __hmul2(v.x, vs[i].x);
                        v.y = __hmul2(v.y, vs[i].y);
                        had_store(tb[i], tj[i], __low2float(v.x), __high2float(v.x), __low2float(v.y), __high2float(v.y));
                    }
                } while (b < nrows);
            }
            else if constexpr (MODE == 0 && GIN == 6)
            {
                // Normalised input whose sum of squares the producer already left per 128-column block:
                // the warp adds the row's block sums up (fixed order), scale = rsqrt(mean + eps), and the
                // task is n = fp16(x * scale) * w (fp16), then the usual scale and rotation. The block
                // sums travel in the same batch of loads as the row itself: one round trip after the wait.
                const int kb = k >> 7;                                  // 128-column blocks of the input row
                int b = 0, jb = warp;
                while (jb >= nblk && b < nrows) { jb -= nblk; ++b; }
                do
                {
                    constexpr int TB = 4;
                    half4 vx[TB], vs[TB], vw[TB];
                    float q[TB];
                    int tb[TB], tj[TB];
                    #pragma unroll
                    for (int i = 0; i < TB; ++i)
                    {
                        tb[i] = b; tj[i] = jb;
                        if (b < nrows)
                        {
                            const size_t col = (size_t) cg0 * 64 + (size_t) jb * 128 + lane * 4;
                            vs[i] = *reinterpret_cast<const half4*>(suh + col);
                            vw[i] = *reinterpret_cast<const half4*>(P.norm_w + col);
                            jb += GEMV_WARPS;
                            while (jb >= nblk && b < nrows) { jb -= nblk; ++b; }
                        }
                        else tb[i] = -1;
                    }
                    if (!waited) { if (P.pdl) pdl_wait(); waited = true; }
                    #pragma unroll
                    for (int i = 0; i < TB; ++i)
                        if (tb[i] >= 0)
                        {
                            vx[i] = *reinterpret_cast<const half4*>(P.x + (size_t) tb[i] * k + (size_t) cg0 * 64 + (size_t) tj[i] * 128 + lane * 4);
                            float acc = 0.0f;
                            for (int j = lane; j < kb; j += 32) acc += __ldcg(P.ssq + (size_t) tb[i] * kb + j);
                            q[i] = acc;
                        }
                    if (!started)
                    {
                        #pragma unroll
                        for (int j = 0; j < S - 1; ++j) issue();
                        started = true;
                    }
                    #pragma unroll
                    for (int i = 0; i < TB; ++i)
                    {
                        if (tb[i] < 0) continue;
                        float tot = q[i];
                        #pragma unroll
                        for (int o2 = 16; o2 > 0; o2 >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o2);
                        const float sc = rsqrtf(tot / (float) k + P.eps);
                        half4 v;
                        v.x = __hmul2(__floats2half2_rn(__low2float(vx[i].x) * sc, __high2float(vx[i].x) * sc), vw[i].x);
                        v.y = __hmul2(__floats2half2_rn(__low2float(vx[i].y) * sc, __high2float(vx[i].y) * sc), vw[i].y);
                        v.x = __hmul2(v.x, vs[i].x);
                        v.y = __hmul2(v.y, vs[i].y);
                        had_store(tb[i], tj[i], __low2float(v.x), __high2float(v.x), __low2float(v.y), __high2float(v.y));
                    }
                } while (b < nrows);
            }
            else if constexpr (MODE == 0 && (GIN == 0 || GIN == 5))
            {
                // up to six tasks per pass: all their loads are in flight before the first
                // transform (at grid start a load takes a microsecond), and the weight stream is
                // started right behind the first pass's loads
                int b = 0, jb = warp;
                while (jb >= nblk && b < nrows) { jb -= nblk; ++b; }
                do
                {
                    constexpr int TB = AMP_GEMV_TB;
                    half4 vx[TB], vs[TB];
                    int tb[TB], tj[TB];
                    #pragma unroll
                    for (int i = 0; i < TB; ++i)
                    {
                        tb[i] = b; tj[i] = jb;
                        if (b < nrows)
                        {
                            vs[i] = *reinterpret_cast<const half4*>(suh + (size_t) cg0 * 64 + (size_t) jb * 128 + lane * 4);
                            jb += GEMV_WARPS;
                            while (jb >= nblk && b < nrows) { jb -= nblk; ++b; }
                        }
                        else tb[i] = -1;
                    }
                    // suh belongs to the weights; x is the previous kernel's output
                    if (!waited) { if (P.pdl) pdl_wait(); waited = true; }
                    #pragma unroll
                    for (int i = 0; i < TB; ++i)
                        if (tb[i] >= 0)
                            vx[i] = *reinterpret_cast<const half4*>(P.x + (size_t) tb[i] * k + (size_t) cg0 * 64 + (size_t) tj[i] * 128 + lane * 4);
                    if (!started)
                    {
                        #pragma unroll
                        for (int j = 0; j < S - 1; ++j) issue();
                        started = true;
                    }
                    #pragma unroll
                    for (int i = 0; i < TB; ++i)
                    {
                        if (tb[i] < 0) continue;
                        half4 v = vx[i];
                        v.x = __hmul2(v.x, vs[i].x);
                        v.y = __hmul2(v.y, vs[i].y);
                        had_store(tb[i], tj[i], __low2float(v.x), __high2float(v.x), __low2float(v.y), __high2float(v.y));
                    }
                } while (b < nrows);
            }
            else
            {
                if constexpr (MODE == 0)
                {
                    // (GIN == 1) Gathered input (split exchange): the whole CTA adds up the ranks' partials of this
                    // chunk's rows, two units per thread in flight, into a staging area. The local
                    // producer has completed (stream order / the wait for the predecessor), so its
                    // sequence number is final; the peers' words may still be on their way.
                    if (!waited) { if (P.pdl) pdl_wait(); waited = true; }
                    const uint32_t seq_in = (uint32_t) *(volatile int*) &P.arin.ctl[0];
                    const uint2* gbase = P.arin.buf + (long) (seq_in & 1) * P.arin.N * P.arin.wcap;
                    half4* stage = reinterpret_cast<half4*>(smem + L.stage);
                    const int upr = nblk * 32;                      // units per batch row in this chunk
                    const long first = (long) cg0 * 16, row_units = k >> 2;
                    if (P.arin.N <= 2) gather_chunk<4, 2>(stage, gbase, P.arin.N, P.arin.wcap, seq_in, P.arin.ctl, nrows * upr, upr, row_units, first, t);
                    else if (P.arin.N <= 4) gather_chunk<2, 4>(stage, gbase, P.arin.N, P.arin.wcap, seq_in, P.arin.ctl, nrows * upr, upr, row_units, first, t);
                    else gather_chunk<1, COMM_MAXN>(stage, gbase, P.arin.N, P.arin.wcap, seq_in, P.arin.ctl, nrows * upr, upr, row_units, first, t);
                    if (!started)
                    {
                        #pragma unroll
                        for (int j = 0; j < S - 1; ++j) issue();
                        started = true;
                    }
                    __syncthreads();
                }
                int b = 0, jb = warp;
                while (jb >= nblk && b < nrows) { jb -= nblk; ++b; }
                while (b < nrows)
                {
                    const size_t col = (size_t) cg0 * 64 + (size_t) jb * 128 + lane * 4;
                    float h0, h1, h2, h3;
                    if constexpr (MODE == 0)
                    {
                        half4 sc = *reinterpret_cast<const half4*>(suh + col);
                        half4 v = reinterpret_cast<const half4*>(smem + L.stage)[b * (nblk * 32) + jb * 32 + lane];
                        v.x = __hmul2(v.x, sc.x);
                        v.y = __hmul2(v.y, sc.y);
                        h0 = __low2float(v.x); h1 = __high2float(v.x); h2 = __low2float(v.y); h3 = __high2float(v.y);
                    }
                    else
                    {
                        // grouped modes scale in fp32 (reference: exl3_moe_coop_kernel.cuh:643-660, 826-838)
                        const int slot = run_slots[b];
                        if constexpr (MODE == 1)
                        {
                            const __half* xr = P.moe.x + (size_t) (slot / P.moe.topk) * P.moe.x_stride;
                            h0 = h1 = h2 = h3 = 0.f;                  // zero padding from H to Hi
                            if ((int) col + 3 < P.moe.H)
                            {
                                half4 v = *reinterpret_cast<const half4*>(xr + col);
                                h0 = __low2float(v.x); h1 = __high2float(v.x); h2 = __low2float(v.y); h3 = __high2float(v.y);
                            }
                            else
                            {
                                if ((int) col + 0 < P.moe.H) h0 = __half2float(xr[col + 0]);
                                if ((int) col + 1 < P.moe.H) h1 = __half2float(xr[col + 1]);
                                if ((int) col + 2 < P.moe.H) h2 = __half2float(xr[col + 2]);
                            }
                        }
                        else
                        {
                            // the gate / up outputs are the previous launch's
                            if (!waited) { if (P.pdl) pdl_wait(); waited = true; }
                            float4 u4, g4;
                            if (P.moe.gu_f32)
                            {
                                u4 = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(P.moe.gu[1]) + (size_t) slot * P.moe.I + col));
                                g4 = u4;
                                if (P.moe.gated) g4 = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(P.moe.gu[0]) + (size_t) slot * P.moe.I + col));
                            }
                            else
                            {
                                auto ld = [&](const void* base) {
                                    const uint2 r = __ldcg(reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(base) + (size_t) slot * P.moe.I + col));
                                    const __half2 a = *reinterpret_cast<const __half2*>(&r.x), b2 = *reinterpret_cast<const __half2*>(&r.y);
                                    return make_float4(__low2float(a), __high2float(a), __low2float(b2), __high2float(b2));
                                };
                                u4 = ld(P.moe.gu[1]);
                                g4 = P.moe.gated ? ld(P.moe.gu[0]) : u4;
                            }
                            h0 = moe_act_gate(P.moe.act, P.moe.gated, g4.x, u4.x, P.moe.act_limit);
                            h1 = moe_act_gate(P.moe.act, P.moe.gated, g4.y, u4.y, P.moe.act_limit);
                            h2 = moe_act_gate(P.moe.act, P.moe.gated, g4.z, u4.z, P.moe.act_limit);
                            h3 = moe_act_gate(P.moe.act, P.moe.gated, g4.w, u4.w, P.moe.act_limit);
                        }
                        half4 sc = *reinterpret_cast<const half4*>(suh + col);
                        h0 *= __low2float(sc.x); h1 *= __high2float(sc.x); h2 *= __low2float(sc.y); h3 *= __high2float(sc.y);
                    }
                    had_store(b, jb, h0, h1, h2, h3);
                    jb += GEMV_WARPS;
                    while (jb >= nblk && b < nrows) { jb -= nblk; ++b; }
                }
            }
            __syncthreads();

            const int c0 = max(cg0, g0);                // first group of the chunk that belongs to the range
            if constexpr (CB == 2 || CB == 3 || CB == 4)
            {
                #pragma unroll
                for (int mb = 0; mb < MB; ++mb)
                    #pragma unroll
                    for (int e = 0; e < 2; ++e)
                    {
                        const int b = min(mb * 8 + 2 * pq + e, nrows - 1);
                        float sacc = xsum[mb][e];
                        for (int g = c0; g < cg1; ++g) sacc += gsum[b * XG + (g - cg0)];
                        xsum[mb][e] = sacc;
                    }
            }

            // every warp walks the chunk's units c0 .. cg1-1
            uint32_t xaddr = xd_s + (c0 - cg0) * 256;   // shared address of the unit's x~ (64 words a group)
            for (int n = cg1 - c0; n > 0; --n, xaddr += 256)
            {
                cp_async_wait_n<S - 2>();               // the unit has landed (this lane's pieces)
                __syncwarp();                           // ... and every other lane's; the slot consumed last is free
                issue();

                // duplicated activations of this lane's tile row (rows 16*pq .. +15 of the group): four
                // 16-byte loads. Batch rows >= m do not exist: row m-1 is read instead (their MMA
                // columns are never stored).
                uint32_t xb[MB][16];
                #pragma unroll
                for (int mb = 0; mb < MB; ++mb)
                    #pragma unroll
                    for (int i = 0; i < 4; ++i)
                        lds128(xaddr + xrow[mb] * 4 + i * 64, xb[mb][4 * i], xb[mb][4 * i + 1], xb[mb][4 * i + 2], xb[mb][4 * i + 3]);

                uint32_t w[NT][K], prev[NT];
                #pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                {
                    load_chunk_s<K>(w_off + cslot + nt * TILE_BYTES, w[nt]);
                    prev[nt] = lds32(p_off + cslot + nt * TILE_BYTES);
                }
                if constexpr (CB == 4)
                {
                    // int8 activations with the error-feedback codes: two exact integer sums per unit
                    uint32_t xr[16];
                    #pragma unroll
                    for (int i = 0; i < 4; ++i)
                        lds128(xaddr + (uint32_t) ((xd2 - xd) * 4) + xrow[0] * 4 + i * 64, xr[4 * i], xr[4 * i + 1], xr[4 * i + 2], xr[4 * i + 3]);
                    const float q = qs[(c0 - cg0) + (cg1 - c0 - n)], q2 = q * (1.0f / 254.0f);
                    #pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
                    {
                        int a0[2] = { 0, 0 }, a1[2] = { 0, 0 }, b0[2] = { 0, 0 }, b1[2] = { 0, 0 };
                        decode_dp4a2_r<K, 0>(w[nt], prev[nt], xb[0], xr, a0, a1, b0, b1);
                        decode_dp4a2_r<K, 1>(w[nt], prev[nt], xb[0], xr, a0, a1, b0, b1);
                        decode_dp4a2_r<K, 2>(w[nt], prev[nt], xb[0], xr, a0, a1, b0, b1);
                        decode_dp4a2_r<K, 3>(w[nt], prev[nt], xb[0], xr, a0, a1, b0, b1);
                        acc0[nt][0][0] = fmaf(q, (float) (a0[0] + a0[1]), acc0[nt][0][0]);
                        acc0[nt][0][2] = fmaf(q, (float) (a1[0] + a1[1]), acc0[nt][0][2]);
                        acc1[nt][0][0] = fmaf(q2, (float) (b0[0] + b0[1]), acc1[nt][0][0]);
                        acc1[nt][0][2] = fmaf(q2, (float) (b1[0] + b1[1]), acc1[nt][0][2]);
                    }
                }
                else if constexpr (CB == 3)
                {
                    // int8 activations (one batch row): exact integer sums over the unit, scaled by
                    // the unit's block scale into the fp32 sums of the segment
                    const float q = qs[(c0 - cg0) + (cg1 - c0 - n)];
                    #pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
                    {
                        int a0[2] = { 0, 0 }, a1[2] = { 0, 0 };
                        decode_dp4a_r<K, 0>(w[nt], prev[nt], xb[0], a0, a1);
                        decode_dp4a_r<K, 1>(w[nt], prev[nt], xb[0], a0, a1);
                        decode_dp4a_r<K, 2>(w[nt], prev[nt], xb[0], a0, a1);
                        decode_dp4a_r<K, 3>(w[nt], prev[nt], xb[0], a0, a1);
                        acc0[nt][0][0] = fmaf(q, (float) (a0[0] + a0[1]), acc0[nt][0][0]);
                        acc0[nt][0][2] = fmaf(q, (float) (a1[0] + a1[1]), acc0[nt][0][2]);
                    }
                }
                else
                {
                    #pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
                    {
                        decode_mma_r<K, CB, MB, 0>(w[nt], prev[nt], xb, acc0[nt], acc1[nt]);
                        decode_mma_r<K, CB, MB, 1>(w[nt], prev[nt], xb, acc0[nt], acc1[nt]);
                        decode_mma_r<K, CB, MB, 2>(w[nt], prev[nt], xb, acc0[nt], acc1[nt]);
                        decode_mma_r<K, CB, MB, 3>(w[nt], prev[nt], xb, acc0[nt], acc1[nt]);
                    }
                }

                cslot += SLOT;
                if (cslot == S * SLOT) cslot = 0;
            }
        }



        // ---- segment done: every lane holds final sums of this CTA's rows for its columns ----
        const bool whole = (g0 == 0 && g1 == G);       // this CTA owns every row of the block
        // contributors of this block: the CTAs whose ranges meet [blk*G, (blk+1)*G)
        const int i_first = split.owner(blk * G);
        const int i_last = split.owner((blk + 1) * G - 1);
        float* slots = P.scratch;                      // [cta][2][m][128]
        const int my_slot = 2 * cta + (blk * G > u0 ? 1 : 0);
        float* dst = whole ? part : slots + (size_t) my_slot * m * 128;
        // cluster form: the partial goes straight into the shared memory of the cluster's first CTA
        const bool clustered = P.cluster > 0;
        uint32_t xdst = 0;
        if (clustered) xdst = cluster_map(smem_u32(smem + L.xchg), 0) + cluster_rank() * (m * 128 * 4);
        #pragma unroll
        for (int nt = 0; nt < NT; ++nt)
        #pragma unroll
        for (int mb = 0; mb < MB; ++mb)
        {
            float d0 = acc0[nt][mb][0] + acc1[nt][mb][0], d1 = acc0[nt][mb][1] + acc1[nt][mb][1];
            float d2 = acc0[nt][mb][2] + acc1[nt][mb][2], d3 = acc0[nt][mb][3] + acc1[nt][mb][3];
            if constexpr (CB == 2)
            {
                // w = raw * k_inv + k_bias  ->  sum x*w = k_inv * sum x*raw + k_bias * sum x
                const float kinv = __half2float(__ushort_as_half((unsigned short) 0x1eee));
                const float kbias = __half2float(__ushort_as_half((unsigned short) 0xc931));
                d0 = d0 * kinv + xsum[mb][0] * kbias; d1 = d1 * kinv + xsum[mb][1] * kbias;
                d2 = d2 * kinv + xsum[mb][0] * kbias; d3 = d3 * kinv + xsum[mb][1] * kbias;
            }
            if constexpr (CB == 3 || CB == 4)
            {
                // the four lanes of a column hold the sums of their tile rows: add them up (fixed
                // order), then sum x*w = k_inv * sum x*bytesum + (1024 k_inv + k_bias) * sum x
                const float kinv = __half2float(__ushort_as_half((unsigned short) 0x1eee));
                const float kbias = __half2float(__ushort_as_half((unsigned short) 0xc931));
                d0 += __shfl_xor_sync(0xffffffffu, d0, 1); d2 += __shfl_xor_sync(0xffffffffu, d2, 1);
                d0 += __shfl_xor_sync(0xffffffffu, d0, 2); d2 += __shfl_xor_sync(0xffffffffu, d2, 2);
                const float aff = fmaf(1024.0f, kinv, kbias);
                d0 = d0 * kinv + xsum[mb][0] * aff; d2 = d2 * kinv + xsum[mb][0] * aff;
                d1 = d3 = 0.0f;
            }
            const int b0 = mb * 8 + 2 * pq;
            if (clustered)
            {
                const uint32_t r0 = xdst + (b0 * 128 + (warp * NT + nt) * 16 + gq) * 4;
                if (b0 < nrows) { cluster_st_f32(r0, d0); cluster_st_f32(r0 + 32, d2); }
                if (b0 + 1 < nrows) { cluster_st_f32(r0 + 512, d1); cluster_st_f32(r0 + 512 + 32, d3); }
                continue;
            }
            float* r0 = dst + b0 * 128 + (warp * NT + nt) * 16 + gq;
            if (b0 < nrows) { r0[0] = d0; r0[8] = d2; }
            if (b0 + 1 < nrows) { r0[128] = d1; r0[128 + 8] = d3; }
        }

        bool finish = whole;
        if (clustered)
        {
            // every CTA of the cluster has delivered its partial when the barrier completes; the
            // first CTA adds them in rank order (= ascending k) and finishes the block
            cluster_sync_all();
            finish = cluster_rank() == 0;
            if (finish)
            {
                const float* xc = reinterpret_cast<const float*>(smem + L.xchg);
                for (int idx = t; idx < nrows * 128; idx += GEMV_THREADS)
                {
                    float sum = xc[idx];
                    for (int r = 1; r < P.cluster; ++r) sum += xc[r * m * 128 + idx];
                    part[idx] = sum;
                }
            }
        }
        else if (!whole)
        {
            // publish the partial, then count arrivals: the last contributor finishes the block.
            // One thread fences after the block-wide barrier (the fence is cumulative over the
            // stores the barrier ordered before it).
            __syncthreads();
            if (t == 0)
            {
                __threadfence();
                const int prev = atomicAdd(P.counters + blk, 1);
                s_last = (prev == i_last - i_first);
                if (s_last)
                {
                    P.counters[blk] = 0;                // self-reset for the next launch
                    __threadfence();                    // acquire side: the other partials are visible
                }
            }
            __syncthreads();
            finish = s_last != 0;
            if (finish)
            {
                // only the first contributor can have started before this block (its second slot)
                const int first_slot = 2 * i_first + (blk * G > split.begin(i_first) ? 1 : 0);
                if constexpr (MODE == 0 && GIN == 2)
                    gemv_reduce_partials(part, slots, reinterpret_cast<const float*>(xd), xd_s, m * XPITCH * 4, m, nrows,
                                         i_first, i_last, first_slot, t);
                else
                {
                    // every other instance: the plain form (one to four rows, or runs that mostly hold
                    // one or two); the instance for five rows and more stages through shared memory
                    const size_t pitch = (size_t) 2 * m * 128;
                    for (int idx = t; idx < nrows * 128; idx += GEMV_THREADS)
                    {
                        float sum = __ldcg(slots + (size_t) first_slot * m * 128 + idx);
                        const float* src = slots + (size_t) (i_first + 1) * pitch + idx;
                        for (int i = i_first + 1; i <= i_last; i += 4, src += 4 * pitch)
                        {
                            float v[4];
                            #pragma unroll
                            for (int j = 0; j < 4; ++j)
                                if (i + j <= i_last) v[j] = __ldcg(src + j * pitch);
                            #pragma unroll
                            for (int j = 0; j < 4; ++j)
                                if (i + j <= i_last) sum += v[j];
                        }
                        part[idx] = sum;
                    }
                }
            }
        }
        __syncthreads();

        if (finish)
        {
            for (int b = warp; b < nrows; b += GEMV_WARPS)
            {
                float4 v = reinterpret_cast<const float4*>(part + b * 128)[lane];
                float h0 = v.x, h1 = v.y, h2 = v.z, h3 = v.w;
                warp_had128(h0, h1, h2, h3, lane);
                h0 *= kRScale; h1 *= kRScale; h2 *= kRScale; h3 *= kRScale;
                const half4 sv = reinterpret_cast<const half4*>(svh + (size_t) nb * 128)[lane];
                if constexpr (MODE != 0)
                {
                    // fp32 scale, optional bias, scattered to the slot's row
                    float4 o = make_float4(h0 * __low2float(sv.x), h1 * __high2float(sv.x),
                                           h2 * __low2float(sv.y), h3 * __high2float(sv.y));
                    if (bias)
                    {
                        const half4 bv = reinterpret_cast<const half4*>(bias + (size_t) nb * 128)[lane];
                        o.x += __low2float(bv.x); o.y += __high2float(bv.x); o.z += __low2float(bv.y); o.w += __high2float(bv.y);
                    }
                    if (MODE == 2 || P.moe.gu_f32)
                        reinterpret_cast<float4*>(reinterpret_cast<float*>(cbase) + (size_t) run_slots[b] * stride + (size_t) nb * 128)[lane] = o;
                    else
                    {
                        half4 oh;
                        oh.x = __floats2half2_rn(o.x, o.y);
                        oh.y = __floats2half2_rn(o.z, o.w);
                        reinterpret_cast<half4*>(reinterpret_cast<__half*>(cbase) + (size_t) run_slots[b] * stride + (size_t) nb * 128)[lane] = oh;
                    }
                    if constexpr (MODE == 2)
                    {
                        // this slot's part of the token's output chunk is delivered: whoever delivers
                        // the last of the token's picks adds them up (pick order) and writes the row
                        const int row = run_slots[b] / P.moe.topk;
                        int* cnt = P.moe.done + row * (P.moe.Ho >> 7) + nb;
                        __syncwarp();
                        int last = 0;
                        if (lane == 0)
                        {
                            __threadfence();
                            const int need = P.moe.inline_runs ? inline_active : P.moe.need[row];
                            if (atomicAdd(cnt, 1) == need - 1)
                            {
                                *cnt = 0;                            // zero again for the next call
                                __threadfence();
                                last = 1;
                            }
                        }
                        last = __shfl_sync(0xffffffffu, last, 0);
                        if (last) moe_combine_chunk(P.moe, row, nb, lane);
                    }
                }
                else if (P.c_fp32)
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
                    if constexpr (MODE == 0)
                    {
                        if (P.ar.N)
                        {
                            // this lane's four halves are one unit of the all-reduce payload (m, stride):
                            // push it to every peer, then add up the peers' units in rank order
                            const uint32_t seq = (uint32_t) (*(volatile int*) &P.ar.ctl[0] + 1);
                            const long unit = ((long) b * stride + (long) nb * 128 + lane * 4) >> 2;
                            const long slot_off = (long) (seq & 1) * P.ar.N * P.ar.wcap;
                            const uint2 mine = *reinterpret_cast<const uint2*>(&o);
                            for (int p = 0; p < P.ar.N; ++p)
                                if (p != P.ar.rank || P.ar.push_only)
                                    st_ll2(P.ar.buf[p] + slot_off + (long) P.ar.rank * P.ar.wcap + 2 * unit, mine.x, mine.y, seq);
                            if (P.ar.push_only) continue;           // the consumer adds the partials up
                            uint2* srcs[COMM_MAXN];
                            #pragma unroll
                            for (int p = 0; p < COMM_MAXN; ++p)
                                srcs[p] = (p < P.ar.N) ? P.ar.buf[P.ar.rank] + slot_off + (long) p * P.ar.wcap + 2 * unit : nullptr;
                            uint32_t d[COMM_MAXN][2];
                            unsigned budget = COMM_SPIN_LIMIT;
                            if (!gather_unit(srcs, &mine, P.ar.rank, P.ar.N, seq, d, budget)) atomicExch(P.ar.ctl + COMM_MAXB, 1);
                            float acc[4] = { 0.f, 0.f, 0.f, 0.f };
                            #pragma unroll
                            for (int p = 0; p < COMM_MAXN; ++p)         // rank order, fp32, one rounding
                                if (p < P.ar.N) acc4(acc, d[p][0], d[p][1]);
                            o.x = __floats2half2_rn(acc[0], acc[1]);
                            o.y = __floats2half2_rn(acc[2], acc[3]);
                        }
                    }
                    if constexpr (GIN == 5)
                    {
                        // producer side of the split norm: y = fp16(h + o) replaces the output, and the
                        // block's sum of squares of y goes to ssq[row][block] (warp sum, fixed order)
                        const size_t at = ((size_t) b * stride + (size_t) nb * 128) / 4 + lane;
                        const half4 hv = reinterpret_cast<const half4*>(P.h_in)[at];
                        half4 yv;
                        yv.x = __floats2half2_rn(__low2float(hv.x) + __low2float(o.x), __high2float(hv.x) + __high2float(o.x));
                        yv.y = __floats2half2_rn(__low2float(hv.y) + __low2float(o.y), __high2float(hv.y) + __high2float(o.y));
                        reinterpret_cast<half4*>(P.y)[at] = yv;
                        const float2 a0 = __half22float2(yv.x), a1 = __half22float2(yv.y);
                        float qs2 = (a0.x * a0.x + a0.y * a0.y) + (a1.x * a1.x + a1.y * a1.y);
                        #pragma unroll
                        for (int o2 = 16; o2 > 0; o2 >>= 1) qs2 += __shfl_xor_sync(0xffffffffu, qs2, o2);
                        if (lane == 0) P.ssq[(size_t) b * P.blocks + blk] = qs2;
                        continue;
                    }
                    reinterpret_cast<half4*>(reinterpret_cast<__half*>(cbase) + (size_t) b * stride + (size_t) nb * 128)[lane] = o;
                    if constexpr (GIN == 4)
                    {
                        if (P.am_key && b == 0)
                        {
                            // argmax over the logits just stored (reference: amp_argmax_advance_kernel,
                            // src/torch/amp_kernels.cu:823-901: largest value, ties to the lowest index,
                            // NaN skipped): the value goes into the high half of a 64-bit key in an order
                            // preserving form, the complemented index into the low half, so one atomic
                            // maximum per column block keeps the winner whatever the arrival order
                            const int col0 = blk * 128 + lane * 4;
                            const float v[4] = { __low2float(o.x), __high2float(o.x), __low2float(o.y), __high2float(o.y) };
                            unsigned long long key = 0ull;
                            #pragma unroll
                            for (int j = 3; j >= 0; --j)
                            {
                                if (!(v[j] == v[j]) || col0 + j >= P.am_vocab) continue;
                                const uint32_t u = v[j] == 0.0f ? 0u : __float_as_uint(v[j]);     // -0 and +0 compare equal
                                const uint32_t ord = u ^ ((u >> 31) ? 0xffffffffu : 0x80000000u);
                                const unsigned long long kj = ((unsigned long long) ord << 32) | (0xffffffffu - (uint32_t) (col0 + j));
                                key = kj > key ? kj : key;
                            }
                            #pragma unroll
                            for (int sft = 16; sft > 0; sft >>= 1)
                            {
                                const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, sft);
                                key = other > key ? other : key;
                            }
                            if (lane == 0)
                            {
                                if (key) atomicMax(P.am_key, key);
                                __threadfence();
                                if (atomicAdd(P.am_count, 1u) + 1u == (unsigned) P.blocks)
                                {
                                    // last block: every candidate has been merged; advance the decode state
                                    __threadfence();
                                    const unsigned long long best = *(volatile unsigned long long*) P.am_key;
                                    const long long p = P.am_pos[0];
                                    if (p >= 0 && p < P.am_log_cap) P.am_log[p] = P.am_ids[0];
                                    P.am_ids[0] = best ? (long long) (0xffffffffu - (uint32_t) (best & 0xffffffffull)) : 0;
                                    P.am_pos[0] = p + 1;
                                    *P.am_key = 0ull;
                                    *P.am_count = 0u;
                                }
                            }
                        }
                    }
                }
            }
            if constexpr (MODE == 0)
            {
                if (P.ar.N)
                {
                    // one arrival per finished column block; the last one closes the call (the
                    // sequence number advances once every block of this rank has been gathered)
                    __syncthreads();
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
        }
        useg += g1 - g0;
    }
    cp_async_wait_n<0>();
}

typedef void (*gemv_fn)(const GemvParams);

// one lookup function per K, defined by the per-K translation units: (cb, MB, mode) -> kernel
// (grouped-expert modes exist for MB == 1 only: a run holds at most eight rows)
#define AMP_GEMV_LOOKUP_DECL(K) gemv_fn gemv_kernel_k##K(int cb, int MB, int mode, int gin);
AMP_GEMV_LOOKUP_DECL(1) AMP_GEMV_LOOKUP_DECL(2) AMP_GEMV_LOOKUP_DECL(3) AMP_GEMV_LOOKUP_DECL(4)
AMP_GEMV_LOOKUP_DECL(5) AMP_GEMV_LOOKUP_DECL(6) AMP_GEMV_LOOKUP_DECL(7) AMP_GEMV_LOOKUP_DECL(8)
#undef AMP_GEMV_LOOKUP_DECL

}  // namespace amp
