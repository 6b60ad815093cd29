// Fused decode-shaped MoE ("coop"): routed experts' gate/up GEMV, activation, down GEMV and the
// routing-weighted sum, for 1..32 tokens, entirely on the device (routing is read from device
// memory; no host synchronisation, capturable in a CUDA graph).
//
// Replaces the reference's exl3_moe_coop (vendor/exl3/exllamav3_ext/quant/exl3_moe_coop.cu:119-371,
// kernels exl3_moe_coop_kernel.cuh:667-999). Organisation here:
//   1. moe_prep_kernel     sorts the active (token, pick) slots by expert and cuts them into runs
//                          of at most eight slots of one expert (a run's slots are the batch rows
//                          of one MMA, so an expert's weights are decoded once per run), and counts
//                          every token's active picks. Skipped for a single token: the two GEMV
//                          launches then derive the (one row per pick) table from the routing.
//   2. grouped GEMV mode 1 gate and up of every run through the decode GEMV kernel (input rows
//                          gathered by token, rotated in the prologue), fp32 outputs per slot
//   3. grouped GEMV mode 2 down of every run; its prologue computes act(gate, up) * d_suh on the
//                          fly; the warp that delivers the last of a token's picks for a 128-column
//                          chunk adds them up (routing weight * slot output in pick order, plus the
//                          shared expert, optionally sigmoid-gated) and writes the fp32 output row
// All counters live in the caller's ctr scratch (zero before the first call, left zero by every
// call), so calls on different streams with different scratch do not interfere.
// The arithmetic per element follows the reference's epilogues (fp32 scales, fp32 Hadamard,
// one rounding to fp16 at each GEMV input).
#include "exl3_gemv_host.h"
#include "host_common.h"
#include "../../include/ampstein_b200.h"

namespace amp {

// One block. Active slots ranked by (local expert, slot), then cut into runs; per token the
// number of active picks (the down launch counts arrivals against it); a token without any local
// pick gets its output row here (nobody else will write it).
__global__ __launch_bounds__(256)
void moe_prep_kernel(const GemvMoe M, int* runs, int* need, int pdl)
{
    __shared__ int s_local[256];
    __shared__ short s_order[256];
    __shared__ int s_need[256];
    __shared__ int s_active;
    const int t = threadIdx.x, slots = M.bsz * M.topk;
    if (pdl) { pdl_wait(); pdl_launch_dependents(); }
    if (t == 0) s_active = 0;
    if (t < M.bsz) s_need[t] = 0;
    __syncthreads();
    if (t < slots)
    {
        const MoeSlot si = moe_slot(M.sel, M.rw, M.topk, M.min_expert, M.max_expert, M.n_local, t);
        s_local[t] = si.active ? si.local : -1;
        if (si.active) atomicAdd(&s_need[si.row], 1);
    }
    __syncthreads();
    const int my_e = t < slots ? s_local[t] : -1;
    if (my_e >= 0)
    {
        const int key = (my_e << 8) | t;
        int rank = 0;
        for (int u = 0; u < slots; ++u)
        {
            const int eu = s_local[u];
            rank += (eu >= 0 && ((eu << 8) | u) < key) ? 1 : 0;
        }
        s_order[rank] = (short) t;
        atomicAdd(&s_active, 1);
    }
    __syncthreads();
    if (t < M.bsz) need[t] = s_need[t];
    if (t == 0)
    {
        const int n_active = s_active;
        int n_runs = 0, prev_e = -1, rows = 0;
        for (int i = 0; i < n_active; ++i)
        {
            const int slot = s_order[i], e = s_local[slot];
            if (e != prev_e || rows == 8)
            {
                ++n_runs;
                rows = 0;
                prev_e = e;
                runs[2 + (n_runs - 1) * MOE_RUN_INTS] = e;
            }
            int* rec = runs + 2 + (n_runs - 1) * MOE_RUN_INTS;
            reinterpret_cast<unsigned char*>(rec + 2)[rows] = (unsigned char) slot;
            rec[1] = ++rows;
        }
        runs[0] = n_runs;
        runs[1] = n_active;
    }
    // rows nobody will deliver a slot for
    const int lane = t & 31, chunks = M.Ho >> 7;
    for (int item = t >> 5; item < M.bsz * chunks; item += 8)
    {
        const int row = item / chunks;
        if (s_need[row] == 0) moe_combine_chunk(M, row, item - row * chunks, lane);
    }
}

template <typename... Args>
static cudaError_t launch_small(void (*kernel)(Args...), int grid, cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

}  // namespace amp

using namespace amp;

// run table (2 + 4 ints per slot), active picks per token, arrivals per (token, 128-column chunk
// of the down output)
AMP_API long amp_exl3_moe_coop_ctr_len(long slots_max, long rows_max, long I, long Ho)
{
    (void) I;
    return 2 + slots_max * MOE_RUN_INTS + rows_max * (1 + Ho / 128);
}

AMP_API int amp_exl3_moe_coop(const amp_moe_coop_args* a, cudaStream_t stream)
{
    AMP_REQUIRE(a, "exl3_moe_coop: null argument block");
    AMP_REQUIRE(a->x && a->sel && a->rw && a->out, "exl3_moe_coop: null tensor");
    AMP_REQUIRE(a->bsz >= 0 && a->topk >= 1, "exl3_moe_coop: sel/rw must be (bsz, topk)");
    if (a->bsz == 0) return 0;
    const int slots = a->bsz * a->topk;
    AMP_REQUIRE(slots <= 256 && slots <= a->slots_max, "exl3_moe_coop: batch exceeds the scratch");
    AMP_REQUIRE(a->Hi % 128 == 0 && a->I % 128 == 0 && a->Ho % 128 == 0 && a->H_out <= a->Ho,
                "exl3_moe_coop: Hi/I/Ho shape");
    AMP_REQUIRE(a->H % 4 == 0 && a->H <= a->Hi, "exl3_moe_coop: H/Hi shape");
    AMP_REQUIRE((a->g_bits && a->u_bits && a->d_bits) || (a->Kgu >= 1 && a->Kgu <= 8 && a->Kd >= 1 && a->Kd <= 8), "exl3_moe_coop: K out of range");
    AMP_REQUIRE(a->cb >= 0 && a->cb <= 2, "exl3_moe_coop: codebook index out of range");
    AMP_REQUIRE(a->act >= 0 && a->act <= 3, "exl3_moe_coop: unknown activation");
    AMP_REQUIRE(a->u_trellis && a->u_suh && a->u_svh && a->d_trellis && a->d_suh && a->d_svh,
                "exl3_moe_coop: pointer tables missing");
    AMP_REQUIRE(!a->gated || (a->g_trellis && a->g_suh && a->g_svh), "exl3_moe_coop: gate tables missing");
    AMP_REQUIRE(a->gu_g && a->gu_u && a->d_out && a->ctr, "exl3_moe_coop: scratch missing");
    AMP_REQUIRE(a->ctr_len >= amp_exl3_moe_coop_ctr_len(a->slots_max, a->bsz, a->I, a->Ho), "exl3_moe_coop: counter scratch too small");
    AMP_REQUIRE(a->min_expert < 0 || a->max_expert - a->min_expert <= a->n_local, "exl3_moe_coop: expert range exceeds tables");
    AMP_REQUIRE(!a->sh_out || a->H_out == a->H, "exl3_moe_coop: shared expert output width must match the routed output");
    AMP_REQUIRE(!a->sh_gate_w || a->H % 2 == 0, "exl3_moe_coop: shared gate width");

    int* runs = a->ctr;
    int* need = a->ctr + 2 + a->slots_max * MOE_RUN_INTS;
    int* done = need + a->bsz;

    GemvLaunch L = {};
    L.moe.runs = runs;
    L.moe.x = (const __half*) a->x; L.moe.x_stride = a->x_stride; L.moe.H = a->H; L.moe.topk = a->topk;
    L.moe.trellis[0] = (const long long*) a->g_trellis; L.moe.trellis[1] = (const long long*) a->u_trellis; L.moe.trellis[2] = (const long long*) a->d_trellis;
    L.moe.suh[0] = (const long long*) a->g_suh; L.moe.suh[1] = (const long long*) a->u_suh; L.moe.suh[2] = (const long long*) a->d_suh;
    L.moe.svh[0] = (const long long*) a->g_svh; L.moe.svh[1] = (const long long*) a->u_svh; L.moe.svh[2] = (const long long*) a->d_svh;
    L.moe.bias[0] = (const long long*) a->g_bias; L.moe.bias[1] = (const long long*) a->u_bias; L.moe.bias[2] = (const long long*) a->d_bias;
    L.moe.gu[0] = a->gu_g; L.moe.gu[1] = a->gu_u; L.moe.gu_f32 = a->gu_f32 ? 1 : 0; L.moe.d_out = (float*) a->d_out;
    L.moe.Hi = a->Hi; L.moe.I = a->I; L.moe.Ho = a->Ho;
    L.moe.act = a->act; L.moe.act_limit = a->act_limit; L.moe.gated = a->gated ? 1 : 0;
    L.moe.sel = (const long long*) a->sel; L.moe.rw = (const __half*) a->rw; L.moe.bsz = a->bsz;
    L.moe.min_expert = a->min_expert; L.moe.max_expert = a->max_expert; L.moe.n_local = a->n_local;
    L.moe.need = need; L.moe.done = done;
    L.moe.out = (float*) a->out; L.moe.out_stride = a->out_stride; L.moe.H_out = a->H_out;
    L.moe.sh_out = (const float*) a->sh_out; L.moe.sh_gate_w = a->sh_out ? (const __half*) a->sh_gate_w : nullptr;
    // one token with at most 16 picks: the kernels derive the (trivial) run table themselves and
    // the sorting launch is not needed
    L.moe.inline_runs = (a->bsz == 1 && a->topk <= 16) ? 1 : 0;
    L.m = 8; L.cb = a->cb; L.c_fp32 = 1;
    const bool mixed = a->g_bits || a->u_bits || a->d_bits;
    if (mixed)
    {
        AMP_REQUIRE(a->g_bits && a->u_bits && a->d_bits, "exl3_moe_coop: give all three bit width tables or none");
        AMP_REQUIRE(a->kmask_gu > 0 && a->kmask_gu < 256 && a->kmask_d > 0 && a->kmask_d < 256,
                    "exl3_moe_coop: kmask_gu / kmask_d must name the bit widths (1..8) that occur in the tables");
        L.moe.bits[0] = (const unsigned char*) a->g_bits; L.moe.bits[1] = (const unsigned char*) a->u_bits;
        L.moe.bits[2] = (const unsigned char*) a->d_bits;
    }
    const int mask_gu = mixed ? a->kmask_gu : (1 << (a->Kgu - 1));
    const int mask_d = mixed ? a->kmask_d : (1 << (a->Kd - 1));

    if (!L.moe.inline_runs)
        if (cudaError_t e = launch_small(moe_prep_kernel, 1, stream, L.moe, runs, need, g_pdl))
            return cuda_rc(e, "moe_prep launch");

    // gate + up: slices = runs x projections, k = Hi, width = I
    const int nproj = a->gated ? 2 : 1;
    // (mixed bit widths: one launch per width that occurs; each works on the runs of its width)
    L.mode = 1; L.k = a->Hi; L.width = a->I; L.stride = a->I;
    L.slices = slots * nproj; L.max_slices = slots * nproj;          // at most one run per slot
    for (int K = 1; K <= 8; ++K)
        if (mask_gu & (1 << (K - 1)))
        {
            L.K = K;
            if (int rc = launch_gemv(L, stream)) return rc;
        }

    // down: slices = runs, k = I, width = Ho; its finishing CTAs also do the routing-weighted sum
    L.mode = 2; L.k = a->I; L.width = a->Ho; L.stride = a->Ho;
    L.slices = slots; L.max_slices = slots;
    L.moe.first_down = 1;
    for (int K = 1; K <= 8; ++K)
        if (mask_d & (1 << (K - 1)))
        {
            L.K = K;
            if (int rc = launch_gemv(L, stream)) return rc;
            L.moe.first_down = 0;
        }
    return 0;
}
