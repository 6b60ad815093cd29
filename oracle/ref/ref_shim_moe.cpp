// C-callable doors into the reference's token-sorted prefill MoE (exl3_moe and exl3_moe_gather,
// vendor/exl3/exllamav3_ext/quant/exl3_moe.cu), compiled unmodified from the reference tree by
// Makefile.ref (target `moe`) into oracle/_ref/libexl3_ref_moe.so. Test infrastructure: used only by
// the tests that time and compare the reference's kernel beside this library's on the same GPU.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <cstdio>
#include <exception>

void exl3_moe(const at::Tensor& hidden_state, const at::Tensor& output_state, const at::Tensor& expert_count,
              const at::Tensor& token_sorted, const at::Tensor& weight_sorted,
              const at::Tensor& temp_state_g, const at::Tensor& temp_state_u,
              const at::Tensor& temp_intermediate_g, const at::Tensor& temp_intermediate_u,
              const int act_function, const float K_gate, const float K_up, const float K_down,
              const at::Tensor& gate_ptrs_trellis, const at::Tensor& gate_ptrs_suh, const at::Tensor& gate_ptrs_svh,
              const at::Tensor& up_ptrs_trellis, const at::Tensor& up_ptrs_suh, const at::Tensor& up_ptrs_svh,
              const at::Tensor& down_ptrs_trellis, const at::Tensor& down_ptrs_suh, const at::Tensor& down_ptrs_svh,
              const bool gate_mcg, const bool gate_mul1, const bool up_mcg, const bool up_mul1,
              const bool down_mcg, const bool down_mul1, const float act_limit, const int num_active,
              const c10::optional<at::Tensor>& output_scratch, const c10::optional<at::Tensor>& fused_base,
              const int count_lo, const int count_hi, const int m_tile,
              const c10::optional<at::Tensor>& bits_g, const c10::optional<at::Tensor>& bits_u,
              const c10::optional<at::Tensor>& bits_d);
int exl3_moe_max_concurrency(int device);

static at::Tensor view(void* p, at::IntArrayRef shape, at::ScalarType t, int dev)
{
    return at::from_blob(p, shape, at::TensorOptions().dtype(t).device(at::kCUDA, dev));
}

struct ref_moe_sorted_args
{
    void* y; void* out; void* count; void* tok; void* w;
    int T, H, I, E; long A;
    void* tables[9];            // g_trellis, g_suh, g_svh, u_*, d_* : int64 device arrays (E entries)
    int K; int cb; int act; float act_limit;
    void* ts_g; void* ts_u; void* ti_g; void* ti_u;     // (conc, cap, H) / (conc, cap, I) fp16
    int conc, cap;
    int lo, hi, m_tile, num_active;
};

extern "C" int ref_exl3_moe_concurrency(int dev)
{
    try { c10::cuda::CUDAGuard guard(dev); return exl3_moe_max_concurrency(dev); }
    catch (const std::exception& e) { fprintf(stderr, "ref_shim: %s\n", e.what()); return -1; }
}

// One launch of the reference kernel in its arrival-order (atomic) summation mode: experts with
// lo <= rows <= hi, weight * result added into out.
extern "C" int ref_exl3_moe_sorted(const ref_moe_sorted_args* a, int dev)
{
    try
    {
        c10::cuda::CUDAGuard guard(dev);
        auto y = view(a->y, {a->T, a->H}, at::kHalf, dev);
        auto out = view(a->out, {a->T, a->H}, at::kFloat, dev);
        auto count = view(a->count, {a->E + 1}, at::kLong, dev);
        auto tok = view(a->tok, {a->A}, at::kLong, dev);
        auto w = view(a->w, {a->A}, at::kHalf, dev);
        at::Tensor t[9];
        for (int i = 0; i < 9; ++i) t[i] = view(a->tables[i], {a->E}, at::kLong, dev);
        auto ts_g = view(a->ts_g, {a->conc, a->cap, a->H}, at::kHalf, dev);
        auto ts_u = view(a->ts_u, {a->conc, a->cap, a->H}, at::kHalf, dev);
        auto ti_g = view(a->ti_g, {a->conc, a->cap, a->I}, at::kHalf, dev);
        auto ti_u = view(a->ti_u, {a->conc, a->cap, a->I}, at::kHalf, dev);
        c10::optional<at::Tensor> none;
        const bool mcg = a->cb == 1, mul1 = a->cb == 2;
        exl3_moe(y, out, count, tok, w, ts_g, ts_u, ti_g, ti_u, a->act, (float) a->K, (float) a->K, (float) a->K,
                 t[0], t[1], t[2], t[3], t[4], t[5], t[6], t[7], t[8], mcg, mul1, mcg, mul1, mcg, mul1,
                 a->act_limit, a->num_active, none, none, a->lo, a->hi, a->m_tile, none, none, none);
        return 0;
    }
    catch (const std::exception& e) { fprintf(stderr, "ref_shim: %s\n", e.what()); return -1; }
}
