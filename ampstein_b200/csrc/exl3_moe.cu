// Fused decode-shaped MoE ("coop"): routed experts' gate/up GEMV, activation, down GEMV and the
// routing-weighted sum, for 1..32 tokens, entirely on the device (routing is read from device
// memory; no host synchronisation, capturable in a CUDA graph).
//
// Replaces the reference's exl3_moe_coop (vendor/exl3/exllamav3_ext/quant/exl3_moe_coop.cu:119-371,
// kernels exl3_moe_coop_kernel.cuh:667-999). Organisation here:
//   1. moe_prep_kernel     sorts the active (token, pick) slots by expert and cuts them into runs
//                          of at most eight slots of one expert (a run's slots are the batch rows
//                          of one MMA, so an expert's weights are decoded once per run)
//   2. grouped GEMV mode 1 gate and up of every run through the decode GEMV kernel (input rows
//                          gathered by token, rotated in the prologue), fp32 outputs per slot
//   3. grouped GEMV mode 2 down of every run; its prologue computes act(gate, up) * d_suh on the fly
//   4. moe_combine_kernel  per token: sum of routing weight * slot output in pick order, plus the
//                          shared expert (optionally sigmoid-gated), fp32 output row
// The arithmetic per element follows the reference's epilogues (fp32 scales, fp32 Hadamard,
// one rounding to fp16 at each GEMV input).
#include "exl3_gemv_host.h"
#include "host_common.h"
#include "../../include/ampstein_b200.h"

namespace amp {

struct SlotInfo { int row, local; float w; bool active; };

__device__ __forceinline__ SlotInfo moe_slot(const long long* sel, const __half* rw, int topk,
                                             int min_expert, int max_expert, int s)
{
    SlotInfo si;
    si.row = s / topk;
    long long e = sel[s];
    si.w = __half2float(rw[s]);
    bool ok = si.w != 0.0f;
    if (min_expert >= 0)
    {
        ok = ok && e >= min_expert && e < max_expert;
        e -= min_expert;
    }
    si.local = ok ? (int) e : 0;
    si.active = ok;
    return si;
}

// One block. Active slots ranked by (local expert, slot), then cut into runs.
__global__ __launch_bounds__(256)
void moe_prep_kernel(const long long* sel, const __half* rw, int bsz, int topk, int min_expert,
                     int max_expert, int n_local, int* runs, int pdl)
{
    __shared__ int s_local[256];
    __shared__ short s_order[256];
    __shared__ int s_active;
    const int t = threadIdx.x, slots = bsz * topk;
    if (pdl) { pdl_launch_dependents(); pdl_wait(); }
    if (t == 0) s_active = 0;
    if (t < slots)
    {
        SlotInfo si = moe_slot(sel, rw, topk, min_expert, max_expert, t);
        s_local[t] = (si.active && si.local < n_local) ? si.local : -1;
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
}

struct CombineParams
{
    const __half* x; int x_stride, H;
    const long long* sel; const __half* rw; int bsz, topk, min_expert, max_expert, n_local;
    const float* d_out; int Ho, H_out;
    float* out; int out_stride;
    const float* sh_out; const __half* sh_gate_w;
    int pdl;
};

// one warp per (token row, 128-column chunk)
__global__ __launch_bounds__(256)
void moe_combine_kernel(const CombineParams p)
{
    if (p.pdl) { pdl_launch_dependents(); pdl_wait(); }
    const int lane = threadIdx.x & 31;
    const int item = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int chunks = p.Ho / 128;
    if (item >= p.bsz * chunks) return;
    const int row = item / chunks, chunk = item - row * chunks;
    const int col = chunk * 128 + lane * 4;

    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
    for (int k = 0; k < p.topk; ++k)                      // pick order: deterministic
    {
        const int s = row * p.topk + k;
        const SlotInfo si = moe_slot(p.sel, p.rw, p.topk, p.min_expert, p.max_expert, s);
        if (!si.active || si.local >= p.n_local) continue;
        const float4 v = __ldcg(reinterpret_cast<const float4*>(p.d_out + (size_t) s * p.Ho + col));
        o0 = __fadd_rn(o0, __fmul_rn(si.w, v.x)); o1 = __fadd_rn(o1, __fmul_rn(si.w, v.y));
        o2 = __fadd_rn(o2, __fmul_rn(si.w, v.z)); o3 = __fadd_rn(o3, __fmul_rn(si.w, v.w));
    }
    if (p.sh_out)
    {
        float gv = 1.0f;
        if (p.sh_gate_w)
        {
            const __half* xr = p.x + (size_t) row * p.x_stride;
            float dot = 0.0f;
            for (int i = lane * 2; i < p.H; i += 64)
            {
                const __half2 xv = *reinterpret_cast<const __half2*>(xr + i);
                const __half2 wv = *reinterpret_cast<const __half2*>(p.sh_gate_w + i);
                dot += __low2float(xv) * __low2float(wv) + __high2float(xv) * __high2float(wv);
            }
            #pragma unroll
            for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            gv = 1.0f / (1.0f + __expf(-dot));
        }
        const float* sh = p.sh_out + (size_t) row * p.H + col;
        if (col + 0 < p.H) o0 += gv * sh[0];
        if (col + 1 < p.H) o1 += gv * sh[1];
        if (col + 2 < p.H) o2 += gv * sh[2];
        if (col + 3 < p.H) o3 += gv * sh[3];
    }
    float* dst = p.out + (size_t) row * p.out_stride + col;
    if (col + 3 < p.H_out) *reinterpret_cast<float4*>(dst) = make_float4(o0, o1, o2, o3);
    else
    {
        if (col + 0 < p.H_out) dst[0] = o0;
        if (col + 1 < p.H_out) dst[1] = o1;
        if (col + 2 < p.H_out) dst[2] = o2;
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

AMP_API long amp_exl3_moe_coop_ctr_len(long slots_max)
{
    return 2 + slots_max * MOE_RUN_INTS;
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
    AMP_REQUIRE(a->Kgu >= 1 && a->Kgu <= 8 && a->Kd >= 1 && a->Kd <= 8, "exl3_moe_coop: K out of range");
    AMP_REQUIRE(a->cb >= 0 && a->cb <= 2, "exl3_moe_coop: codebook index out of range");
    AMP_REQUIRE(a->act >= 0 && a->act <= 3, "exl3_moe_coop: unknown activation");
    AMP_REQUIRE(a->u_trellis && a->u_suh && a->u_svh && a->d_trellis && a->d_suh && a->d_svh,
                "exl3_moe_coop: pointer tables missing");
    AMP_REQUIRE(!a->gated || (a->g_trellis && a->g_suh && a->g_svh), "exl3_moe_coop: gate tables missing");
    AMP_REQUIRE(a->gu_g && a->gu_u && a->d_out && a->ctr, "exl3_moe_coop: scratch missing");
    AMP_REQUIRE(a->min_expert < 0 || a->max_expert - a->min_expert <= a->n_local, "exl3_moe_coop: expert range exceeds tables");
    AMP_REQUIRE(!a->sh_out || a->H_out == a->H, "exl3_moe_coop: shared expert output width must match the routed output");
    AMP_REQUIRE(!a->sh_gate_w || a->H % 2 == 0, "exl3_moe_coop: shared gate width");

    int* runs = a->ctr;
    if (cudaError_t e = launch_small(moe_prep_kernel, 1, stream, (const long long*) a->sel, (const __half*) a->rw,
                                     a->bsz, a->topk, a->min_expert, a->max_expert, a->n_local, runs, g_pdl))
        return cuda_rc(e, "moe_prep launch");

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
    L.m = 8; L.cb = a->cb; L.c_fp32 = 1;

    // gate + up: slices = runs x projections, k = Hi, width = I
    const int nproj = a->gated ? 2 : 1;
    L.mode = 1; L.k = a->Hi; L.width = a->I; L.stride = a->I; L.K = a->Kgu;
    L.slices = slots * nproj; L.max_slices = slots * nproj;          // at most one run per slot
    if (int rc = launch_gemv(L, stream)) return rc;

    // down: slices = runs, k = I, width = Ho
    L.mode = 2; L.k = a->I; L.width = a->Ho; L.stride = a->Ho; L.K = a->Kd;
    L.slices = slots; L.max_slices = slots;
    if (int rc = launch_gemv(L, stream)) return rc;

    CombineParams C;
    C.x = (const __half*) a->x; C.x_stride = a->x_stride; C.H = a->H;
    C.sel = (const long long*) a->sel; C.rw = (const __half*) a->rw; C.bsz = a->bsz; C.topk = a->topk;
    C.min_expert = a->min_expert; C.max_expert = a->max_expert; C.n_local = a->n_local;
    C.d_out = (const float*) a->d_out; C.Ho = a->Ho; C.H_out = a->H_out;
    C.out = (float*) a->out; C.out_stride = a->out_stride;
    C.sh_out = (const float*) a->sh_out; C.sh_gate_w = a->sh_out ? (const __half*) a->sh_gate_w : nullptr;
    C.pdl = g_pdl;
    const int items = a->bsz * (a->Ho / 128);
    if (cudaError_t e = launch_small(moe_combine_kernel, (items + 7) / 8, stream, C)) return cuda_rc(e, "moe_combine launch");
    return 0;
}
