// Kernel instances of the trellis-decode GEMV for one bitrate; compiled once per K with
// -DAMP_GEMV_K=<1..8> so the eight translation units build in parallel.
#include "exl3_gemv_kernel.cuh"
#include "exl3_gemv_tc.cuh"

#ifndef AMP_GEMV_K
#error "compile with -DAMP_GEMV_K=<bits>"
#endif

#define AMP_CAT_(a, b) a##b
#define AMP_CAT(a, b) AMP_CAT_(a, b)

namespace amp {

gemv_fn AMP_CAT(gemv_kernel_k, AMP_GEMV_K)(int cb, int MB, int mode, int gin)
{
    // input gathered from the all-reduce buffers (split exchange)
    static const gemv_fn fng[3][2] =
    {
        { exl3_gemv_kernel<AMP_GEMV_K, 0, 1, 0, 1>, exl3_gemv_kernel<AMP_GEMV_K, 0, 2, 0, 1> },
        { exl3_gemv_kernel<AMP_GEMV_K, 1, 1, 0, 1>, exl3_gemv_kernel<AMP_GEMV_K, 1, 2, 0, 1> },
        { exl3_gemv_kernel<AMP_GEMV_K, 2, 1, 0, 1>, exl3_gemv_kernel<AMP_GEMV_K, 2, 2, 0, 1> },
    };
    // input already rotated (batches of five rows and more)
    static const gemv_fn fnr[3][2] =
    {
        { exl3_gemv_kernel<AMP_GEMV_K, 0, 1, 0, 2>, exl3_gemv_kernel<AMP_GEMV_K, 0, 2, 0, 2> },
        { exl3_gemv_kernel<AMP_GEMV_K, 1, 1, 0, 2>, exl3_gemv_kernel<AMP_GEMV_K, 1, 2, 0, 2> },
        { exl3_gemv_kernel<AMP_GEMV_K, 2, 1, 0, 2>, exl3_gemv_kernel<AMP_GEMV_K, 2, 2, 0, 2> },
    };
    // input = silu(gate) * up, formed in the prologue
    static const gemv_fn fna[3][2] =
    {
        { exl3_gemv_kernel<AMP_GEMV_K, 0, 1, 0, 3>, exl3_gemv_kernel<AMP_GEMV_K, 0, 2, 0, 3> },
        { exl3_gemv_kernel<AMP_GEMV_K, 1, 1, 0, 3>, exl3_gemv_kernel<AMP_GEMV_K, 1, 2, 0, 3> },
        { exl3_gemv_kernel<AMP_GEMV_K, 2, 1, 0, 3>, exl3_gemv_kernel<AMP_GEMV_K, 2, 2, 0, 3> },
    };
    // input = RMSNorm(x + residual) * w, formed in the prologue
    static const gemv_fn fnn[3][2] =
    {
        { exl3_gemv_kernel<AMP_GEMV_K, 0, 1, 0, 4>, exl3_gemv_kernel<AMP_GEMV_K, 0, 2, 0, 4> },
        { exl3_gemv_kernel<AMP_GEMV_K, 1, 1, 0, 4>, exl3_gemv_kernel<AMP_GEMV_K, 1, 2, 0, 4> },
        { exl3_gemv_kernel<AMP_GEMV_K, 2, 1, 0, 4>, exl3_gemv_kernel<AMP_GEMV_K, 2, 2, 0, 4> },
    };
    // split norm: producer epilogue (5) and consumer prologue (6)
    static const gemv_fn fnp[3][2] =
    {
        { exl3_gemv_kernel<AMP_GEMV_K, 0, 1, 0, 5>, exl3_gemv_kernel<AMP_GEMV_K, 0, 2, 0, 5> },
        { exl3_gemv_kernel<AMP_GEMV_K, 1, 1, 0, 5>, exl3_gemv_kernel<AMP_GEMV_K, 1, 2, 0, 5> },
        { exl3_gemv_kernel<AMP_GEMV_K, 2, 1, 0, 5>, exl3_gemv_kernel<AMP_GEMV_K, 2, 2, 0, 5> },
    };
    static const gemv_fn fnc[3][2] =
    {
        { exl3_gemv_kernel<AMP_GEMV_K, 0, 1, 0, 6>, exl3_gemv_kernel<AMP_GEMV_K, 0, 2, 0, 6> },
        { exl3_gemv_kernel<AMP_GEMV_K, 1, 1, 0, 6>, exl3_gemv_kernel<AMP_GEMV_K, 1, 2, 0, 6> },
        { exl3_gemv_kernel<AMP_GEMV_K, 2, 1, 0, 6>, exl3_gemv_kernel<AMP_GEMV_K, 2, 2, 0, 6> },
    };
    static const gemv_fn fn[3][2] =
    {
        { exl3_gemv_kernel<AMP_GEMV_K, 0, 1>, exl3_gemv_kernel<AMP_GEMV_K, 0, 2> },
        { exl3_gemv_kernel<AMP_GEMV_K, 1, 1>, exl3_gemv_kernel<AMP_GEMV_K, 1, 2> },
        { exl3_gemv_kernel<AMP_GEMV_K, 2, 1>, exl3_gemv_kernel<AMP_GEMV_K, 2, 2> },
    };
    static const gemv_fn moe[3][2] =
    {
        { exl3_gemv_kernel<AMP_GEMV_K, 0, 1, 1>, exl3_gemv_kernel<AMP_GEMV_K, 0, 1, 2> },
        { exl3_gemv_kernel<AMP_GEMV_K, 1, 1, 1>, exl3_gemv_kernel<AMP_GEMV_K, 1, 1, 2> },
        { exl3_gemv_kernel<AMP_GEMV_K, 2, 1, 1>, exl3_gemv_kernel<AMP_GEMV_K, 2, 1, 2> },
    };
    // cb 3 = the mul1 codebook with int8 activations: one batch row, plain launches only
    if (cb == 3) return (MB == 1 && !mode && !gin) ? exl3_gemv_kernel<AMP_GEMV_K, 3, 1> : nullptr;
    if (cb == 4) return (MB == 1 && !mode && !gin) ? exl3_gemv_kernel<AMP_GEMV_K, 4, 1> : nullptr;
    if (cb < 0 || cb > 2 || MB < 1 || MB > 2 || mode < 0 || mode > 2) return nullptr;
    if (mode) return (MB == 1 && !gin) ? moe[cb][mode - 1] : nullptr;
    if (gin == 4) return fnn[cb][MB - 1];
    if (gin == 5) return fnp[cb][MB - 1];
    if (gin == 6) return fnc[cb][MB - 1];
    return gin == 3 ? fna[cb][MB - 1] : (gin == 2 ? fnr[cb][MB - 1] : (gin ? fng[cb][MB - 1] : fn[cb][MB - 1]));
}

// tensor-memory form (dense / bundle launches of up to eight rows)
gemv_fn AMP_CAT(gemv_tc_kernel_k, AMP_GEMV_K)(int cb, int ar)
{
    static const gemv_fn fn[3][2] =
    {
        { exl3_gemv_tc_kernel<AMP_GEMV_K, 0, 0>, exl3_gemv_tc_kernel<AMP_GEMV_K, 0, 1> },
        { exl3_gemv_tc_kernel<AMP_GEMV_K, 1, 0>, exl3_gemv_tc_kernel<AMP_GEMV_K, 1, 1> },
        { exl3_gemv_tc_kernel<AMP_GEMV_K, 2, 0>, exl3_gemv_tc_kernel<AMP_GEMV_K, 2, 1> },
    };
    if (cb < 0 || cb > 2) return nullptr;
    return fn[cb][ar ? 1 : 0];
}

}  // namespace amp
