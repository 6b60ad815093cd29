// libtorch host layer over the C ABI: the functions the reference's binding file links against,
// with the reference's own C++ signatures (global namespace, at::Tensor arguments), implemented by
// unpacking the tensors and calling libampstein_b200.so. Linking this object in place of the
// reference's exl3 kernel library leaves src/torch/amp_torch.cpp unchanged.
//
// Signatures replaced (declarations in the reference at src/torch/amp_torch.cpp):
//   exl3_gemm              :3775-3787      exl3_mgemm            :3841-3864
//   reconstruct            :3832-3839      reconstruct_had_slice :11071-11081
//   had_r_128              :11062-11069    exl3_moe_coop         :3739-3771
//   exl3_moe               :7796-7836      exl3_moe_gather, exl3_moe_max_concurrency (same block)
// Error convention: argument and launch errors throw c10::Error (TORCH_CHECK), which every
// binding of the reference catches and turns into a script exception (:224-236).
//
// The same functions are exposed as the Python module ampstein_b200._torch_glue so that the tests
// can drive this layer with torch tensors (compile with -DAMP_NO_PYBIND to leave the module out).
#ifndef AMP_NO_PYBIND
#include <torch/extension.h>
#else
#include <ATen/ATen.h>
#endif
#include <map>
#include <mutex>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>

#include "../../include/ampstein_b200.h"

namespace {

void check_rc(int rc, const char* what)
{
    if (rc == 0) return;
    if (rc < 0) TORCH_CHECK(false, what, ": ", amp_b200_last_error());
    TORCH_CHECK(false, what, ": CUDA error ", rc, " (", cudaGetErrorString((cudaError_t) rc), ") ", amp_b200_last_error());
}

int codebook(bool mcg, bool mul1)
{
    TORCH_CHECK(!(mcg && mul1), "mcg and mul1 are exclusive");
    return mul1 ? 2 : (mcg ? 1 : 0);
}

int bits_of(const at::Tensor& trellis, const char* who)
{
    TORCH_CHECK(trellis.dim() == 3 && trellis.scalar_type() == at::kShort, who, ": trellis must be int16 (k/16, n/16, 16K)");
    TORCH_CHECK(trellis.is_contiguous(), who, ": trellis must be contiguous");
    const int64_t w = trellis.size(2);
    TORCH_CHECK(w % 16 == 0 && w / 16 >= 1 && w / 16 <= 8, who, ": unsupported EXL3 bitrate");
    return (int) (w / 16);
}

int bits_of(float K, const char* who)
{
    TORCH_CHECK(K == (float) (int) K && K >= 1.f && K <= 8.f, who, ": unsupported EXL3 bitrate ", K, " (integer 1..8)");
    return (int) K;
}

// the same for the entries that also take the half-integer rates 1.5 / 2.5 / 3.5 (third dimension
// 16 KA + 8, mul1 only): the C ABI's code AMP_EXL3_HALF_RATE(KA) comes back for those
int bits_or_half(const at::Tensor& trellis, bool mul1, const char* who)
{
    TORCH_CHECK(trellis.dim() == 3, who, ": trellis must be int16 (k/16, n/16, 16K)");
    const int64_t w = trellis.size(2);
    if (w % 16 != 8) return bits_of(trellis, who);
    TORCH_CHECK(trellis.scalar_type() == at::kShort && trellis.is_contiguous(), who, ": trellis must be contiguous int16");
    TORCH_CHECK(w / 16 >= 1 && w / 16 <= 3, who, ": unsupported EXL3 bitrate");
    TORCH_CHECK(mul1, who, ": half-integer bitrates require the mul1 codebook");
    return AMP_EXL3_HALF_RATE((int) (w / 16));
}

int bits_or_half(float K, const char* who)
{
    const int b = (int) K;
    if (K - (float) b == 0.5f && b >= 1 && b <= 3) return AMP_EXL3_HALF_RATE(b);
    return bits_of(K, who);
}

const void* opt_ptr(const c10::optional<at::Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }

cudaStream_t stream_of(const at::Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

// Mixed bit widths: the C ABI wants to know which widths occur in a per-expert uint8 table (bit K-1
// of the mask per width K). The tables are static, so each is read back once (keyed by address and
// length) and remembered.
int bit_mask_of(const at::Tensor& t, int n, const char* who)
{
    TORCH_CHECK(t.scalar_type() == at::kByte && t.is_cuda() && t.is_contiguous() && t.numel() >= n,
                who, ": bit width tables must be contiguous uint8 device tensors with one entry per expert");
    static std::mutex mu;
    static std::map<std::pair<const void*, int>, int> masks;
    std::lock_guard<std::mutex> lock(mu);
    const auto key = std::make_pair((const void*) t.data_ptr(), n);
    auto it = masks.find(key);
    if (it != masks.end()) return it->second;
    const at::Tensor h = t.narrow(0, 0, n).cpu();
    int m = 0;
    for (int i = 0; i < n; ++i)
    {
        const int K = h.data_ptr<uint8_t>()[i];
        TORCH_CHECK(K >= 1 && K <= 8, who, ": bit widths must be 1..8");
        m |= 1 << (K - 1);
    }
    masks[key] = m;
    return m;
}

void same_device(const at::Tensor& a, const at::Tensor& b, const char* who)
{
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.get_device() == b.get_device(), who, ": tensors must live on one CUDA device");
}

}  // namespace

// C (m, n) = A (m, k) through the quantized weight B. Returns the kernel family used: 90 for the
// decode kernel (the reference's GEMV index), 100 for the tensor-core prefill kernel.
int exl3_gemm(const at::Tensor& A, const at::Tensor& B, at::Tensor& C, const c10::optional<at::Tensor>& suh,
              const c10::optional<at::Tensor>& A_had, const c10::optional<at::Tensor>& svh, int force_shape_idx,
              bool mcg, bool mul1, int force_num_sms)
{
    (void) force_shape_idx; (void) force_num_sms;
    const c10::cuda::CUDAGuard guard(A.device());
    same_device(A, B, "exl3_gemm"); same_device(A, C, "exl3_gemm");
    const int K = bits_or_half(B, mul1, "exl3_gemm");
    TORCH_CHECK(A.dim() == 2 && C.dim() == 2 && A.is_contiguous() && C.is_contiguous(), "exl3_gemm: A and C must be contiguous 2-D");
    TORCH_CHECK(A.scalar_type() == at::kHalf || A.scalar_type() == at::kBFloat16, "exl3_gemm: A must be float16 (or bfloat16)");
    TORCH_CHECK(C.scalar_type() == at::kHalf || C.scalar_type() == at::kFloat, "exl3_gemm: C must be float16 or float32");
    TORCH_CHECK(suh.has_value() && svh.has_value(), "exl3_gemm: suh and svh are required");
    TORCH_CHECK(suh->scalar_type() == at::kHalf && svh->scalar_type() == at::kHalf, "exl3_gemm: suh, svh must be float16");
    const int64_t m = A.size(0), k = A.size(1), n = C.size(1);
    TORCH_CHECK(B.size(0) * 16 == k && B.size(1) * 16 == n && C.size(0) == m, "exl3_gemm: shape mismatch");
    TORCH_CHECK(suh->numel() == k && svh->numel() == n, "exl3_gemm: suh / svh length mismatch");
    if (A_had.has_value() && A_had->defined())
        TORCH_CHECK(A_had->scalar_type() == at::kHalf && A_had->numel() >= A.numel() && A_had->is_contiguous(),
                    "exl3_gemm: A_had must be contiguous float16 of A's size");
    if (m == 0 || n == 0) return 0;
    const bool bf16 = A.scalar_type() == at::kBFloat16;
    if (K > 256 && (m > 16 || bf16 || !(A_had.has_value() && A_had->defined())))
    {
        // half-integer bitrate beyond the decode kernel's reach (more than 16 rows, or no scratch
        // for the rotated input): the weight is decoded once into the original basis and
        // multiplied by a library GEMM, as the reference's torch_exl3_gemm_recon does
        at::Tensor w = at::empty({k, n}, A.options().dtype(at::kHalf));
        check_rc(amp_exl3_reconstruct_had(w.data_ptr(), B.data_ptr(), suh->data_ptr(), svh->data_ptr(), (int) k, (int) n, K, 2, 0, (int) n,
                                          stream_of(A)), "exl3_gemm");
        C.copy_(at::mm(A.to(at::kHalf), w));
        return 100;
    }
    auto fn = bf16 ? amp_exl3_gemm_bf16 : amp_exl3_gemm;
    check_rc(fn(A.data_ptr(), B.data_ptr(), C.data_ptr(), suh->data_ptr(), const_cast<void*>(opt_ptr(A_had)), svh->data_ptr(),
                (int) m, (int) k, (int) n, K, codebook(mcg, mul1), C.scalar_type() == at::kFloat ? 1 : 0, stream_of(A)),
             "exl3_gemm");
    return m <= 16 ? 90 : 100;
}

// Several weights (or equal-width column slices) against one shared input. B / suh / svh are int64
// device pointer tables. The routed forms of the reference (indices / weights) belong to its
// token-sorted MoE path and are not part of this library.
int exl3_mgemm(const at::Tensor& A, const at::Tensor& B, at::Tensor& C, const at::Tensor& suh, const at::Tensor& A_had,
               const at::Tensor& svh, const c10::optional<at::Tensor>& indices, const c10::optional<at::Tensor>& weights,
               float K, int force_shape_idx, uint32_t mcg_mult, uint32_t mul1_mult, int min_index, int max_index,
               int force_num_sms, int num_tokens, const c10::optional<at::Tensor>& size_n_list,
               const c10::optional<at::Tensor>& c_ptrs, const c10::optional<at::Tensor>& n_stride_list,
               const c10::optional<at::Tensor>& had_src_list, int num_had_src)
{
    (void) force_shape_idx; (void) force_num_sms; (void) min_index; (void) max_index; (void) num_tokens;
    const c10::cuda::CUDAGuard guard(A.device());
    TORCH_CHECK(!indices.has_value() && !weights.has_value(), "exl3_mgemm: routed (indices / weights) form is not supported");
    same_device(A, B, "exl3_mgemm"); same_device(A, C, "exl3_mgemm");
    TORCH_CHECK(B.scalar_type() == at::kLong && suh.scalar_type() == at::kLong && svh.scalar_type() == at::kLong,
                "exl3_mgemm: B, suh, svh must be int64 pointer tables");
    TORCH_CHECK(A.scalar_type() == at::kHalf && A.is_contiguous() && A.dim() == 3 && A.size(0) == 1, "exl3_mgemm: A must be contiguous float16 (1, m, k)");
    TORCH_CHECK(C.dim() == 3 && C.is_contiguous() && (C.scalar_type() == at::kHalf || C.scalar_type() == at::kFloat),
                "exl3_mgemm: C must be contiguous (num, m, n) float16 or float32");
    const int bits = bits_of(K, "exl3_mgemm");
    const int64_t num = C.size(0), m = C.size(1), width = C.size(2), k = A.size(2);
    TORCH_CHECK(A.size(1) == m, "exl3_mgemm: row count of A and C differ");
    TORCH_CHECK(B.numel() >= num && svh.numel() >= num, "exl3_mgemm: pointer tables shorter than the matrix count");
    const void* cp = nullptr; const void* ns = nullptr; const void* hs = nullptr;
    if (size_n_list.has_value())
    {
        // every entry must equal C.size(2): the slices of one launch share one width
        TORCH_CHECK(c_ptrs.has_value(), "exl3_mgemm: size_n_list requires c_ptrs");
        TORCH_CHECK(size_n_list->scalar_type() == at::kInt && c_ptrs->scalar_type() == at::kLong, "exl3_mgemm: size_n_list int32, c_ptrs int64");
        TORCH_CHECK(c_ptrs->numel() == num && size_n_list->numel() == num, "exl3_mgemm: slice tables do not match C");
        cp = c_ptrs->data_ptr();
    }
    if (had_src_list.has_value())
    {
        TORCH_CHECK(size_n_list.has_value() && c_ptrs.has_value() && n_stride_list.has_value(),
                    "exl3_mgemm: sliced mode requires size_n_list, c_ptrs and n_stride_list");
        TORCH_CHECK(had_src_list->scalar_type() == at::kInt && n_stride_list->scalar_type() == at::kInt, "exl3_mgemm: had_src_list / n_stride_list must be int32");
        TORCH_CHECK(had_src_list->numel() >= num && n_stride_list->numel() >= num, "exl3_mgemm: had_src_list / n_stride_list must have one entry per slice");
        TORCH_CHECK(num_had_src > 0 && suh.numel() >= num_had_src, "exl3_mgemm: suh must hold one entry per source");
        ns = n_stride_list->data_ptr();
        hs = had_src_list->data_ptr();
    }
    else
    {
        TORCH_CHECK(!n_stride_list.has_value(), "exl3_mgemm: n_stride_list requires had_src_list");
        TORCH_CHECK(suh.numel() >= num, "exl3_mgemm: suh table shorter than the matrix count");
    }
    const int cb = mul1_mult ? 2 : (mcg_mult ? 1 : 0);
    check_rc(amp_exl3_mgemm(A.data_ptr(), B.data_ptr(), C.data_ptr(), suh.data_ptr(), A_had.defined() ? A_had.data_ptr() : nullptr,
                            svh.data_ptr(), (int) num, (int) m, (int) k, (int) width, bits, cb, C.scalar_type() == at::kFloat ? 1 : 0,
                            cp, ns, hs, num_had_src, stream_of(A)),
             "exl3_mgemm");
    return 90;
}

void reconstruct(at::Tensor unpacked, at::Tensor packed, float K_, bool mcg, bool mul1)
{
    const c10::cuda::CUDAGuard guard(unpacked.device());
    same_device(unpacked, packed, "reconstruct");
    const int K = bits_or_half(packed, mul1, "reconstruct");
    TORCH_CHECK(bits_or_half(K_, "reconstruct") == K, "reconstruct: K does not match the trellis");
    TORCH_CHECK(unpacked.scalar_type() == at::kHalf && unpacked.dim() == 2 && unpacked.is_contiguous(), "reconstruct: unpacked must be contiguous float16 (k, n)");
    const int64_t k = packed.size(0) * 16, n = packed.size(1) * 16;
    TORCH_CHECK(unpacked.size(0) == k && unpacked.size(1) == n, "reconstruct: shape mismatch");
    if (k == 0 || n == 0) return;
    check_rc(amp_exl3_reconstruct(unpacked.data_ptr(), packed.data_ptr(), (int) k, (int) n, K, codebook(mcg, mul1), 0, (int) n, stream_of(unpacked)),
             "reconstruct");
}

void reconstruct_had_slice(at::Tensor unpacked, at::Tensor packed, at::Tensor suh, at::Tensor svh, float K_, bool mcg, bool mul1,
                           int64_t n_offset)
{
    const c10::cuda::CUDAGuard guard(unpacked.device());
    same_device(unpacked, packed, "reconstruct_had_slice");
    const int K = bits_or_half(packed, mul1, "reconstruct_had_slice");
    TORCH_CHECK(bits_or_half(K_, "reconstruct_had_slice") == K, "reconstruct_had_slice: K does not match the trellis");
    TORCH_CHECK(unpacked.scalar_type() == at::kHalf && unpacked.dim() == 2 && unpacked.is_contiguous(), "reconstruct_had_slice: unpacked must be contiguous float16");
    TORCH_CHECK(suh.scalar_type() == at::kHalf && svh.scalar_type() == at::kHalf, "reconstruct_had_slice: suh, svh must be float16");
    const int64_t k = packed.size(0) * 16, n = packed.size(1) * 16, n_out = unpacked.size(1);
    TORCH_CHECK(unpacked.size(0) == k && n_offset >= 0 && n_offset + n_out <= n, "reconstruct_had_slice: slice outside the weight");
    TORCH_CHECK(suh.numel() == k && svh.numel() >= n_out, "reconstruct_had_slice: suh / svh length mismatch");
    if (k == 0 || n_out == 0) return;
    check_rc(amp_exl3_reconstruct_had(unpacked.data_ptr(), packed.data_ptr(), suh.data_ptr(), svh.data_ptr(), (int) k, (int) n, K,
                                      codebook(mcg, mul1), (int) n_offset, (int) n_out, stream_of(unpacked)),
             "reconstruct_had_slice");
}

void had_r_128(const at::Tensor& input, const at::Tensor& output, const c10::optional<at::Tensor>& pre_scale,
               const c10::optional<at::Tensor>& post_scale, const float scale)
{
    const c10::cuda::CUDAGuard guard(input.device());
    same_device(input, output, "had_r_128");
    TORCH_CHECK(input.dim() >= 1 && input.is_contiguous() && output.is_contiguous() && input.numel() == output.numel(), "had_r_128: contiguous tensors of one size");
    TORCH_CHECK(input.scalar_type() == output.scalar_type() && (input.scalar_type() == at::kHalf || input.scalar_type() == at::kFloat),
                "had_r_128: float16 or float32, same type in and out");
    const int64_t cols = input.size(-1), rows = cols ? input.numel() / cols : 0;
    TORCH_CHECK(cols % 128 == 0, "had_r_128: last dimension must be a multiple of 128");
    for (const auto* s : { &pre_scale, &post_scale })
        if (s->has_value() && (*s)->defined())
            TORCH_CHECK((*s)->scalar_type() == at::kHalf && (*s)->numel() == cols, "had_r_128: scales must be float16 of the row length");
    if (rows == 0) return;
    check_rc(amp_had_r_128(input.data_ptr(), output.data_ptr(), opt_ptr(pre_scale), opt_ptr(post_scale), rows, (int) cols,
                           input.scalar_type() == at::kFloat ? 1 : 0, scale, stream_of(input)),
             "had_r_128");
}

// Fused decode MoE. had_g / had_u / act_out are scratch of the reference's kernels that this
// implementation does not need (accepted, untouched); per-expert bit tables are not supported.
void exl3_moe_coop(const at::Tensor& x, const at::Tensor& sel, const at::Tensor& rw, int min_expert, int max_expert, int Hi,
                   const at::Tensor& g_trellis, const at::Tensor& g_suh, const at::Tensor& g_svh,
                   const at::Tensor& u_trellis, const at::Tensor& u_suh, const at::Tensor& u_svh,
                   const at::Tensor& d_trellis, const at::Tensor& d_suh, const at::Tensor& d_svh,
                   const c10::optional<at::Tensor>& g_bias, const c10::optional<at::Tensor>& u_bias, const c10::optional<at::Tensor>& d_bias,
                   float Kg, float Ku, float Kd, bool mcg, bool mul1, int act, float act_limit, bool gated,
                   at::Tensor& had_g, at::Tensor& had_u, at::Tensor& gu_g, at::Tensor& gu_u, at::Tensor& act_out, at::Tensor& d_out,
                   at::Tensor& ctr, at::Tensor& out, const c10::optional<at::Tensor>& sh_out, const c10::optional<at::Tensor>& sh_gate_w,
                   const c10::optional<at::Tensor>& bits_g, const c10::optional<at::Tensor>& bits_u, const c10::optional<at::Tensor>& bits_d)
{
    (void) had_g; (void) had_u; (void) act_out;
    const c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(x.dim() == 2 && x.scalar_type() == at::kHalf && x.stride(1) == 1, "exl3_moe_coop: x must be float16 (bsz, H)");
    TORCH_CHECK(sel.scalar_type() == at::kLong && rw.scalar_type() == at::kHalf && sel.is_contiguous() && rw.is_contiguous() &&
                sel.dim() == 2 && sel.sizes() == rw.sizes() && sel.size(0) == x.size(0), "exl3_moe_coop: sel int64 / rw float16 (bsz, topk)");
    for (const at::Tensor* t : { &g_trellis, &g_suh, &g_svh, &u_trellis, &u_suh, &u_svh, &d_trellis, &d_suh, &d_svh })
        TORCH_CHECK(t->scalar_type() == at::kLong && t->is_cuda(), "exl3_moe_coop: expert tables must be int64 device pointer tables");
    TORCH_CHECK(!gated || Kg == Ku, "exl3_moe_coop: gate and up must share one bitrate");
    TORCH_CHECK(d_out.scalar_type() == at::kFloat && d_out.dim() >= 1 && out.scalar_type() == at::kFloat && out.dim() >= 2 && out.stride(-1) == 1,
                "exl3_moe_coop: d_out and out must be float32");
    TORCH_CHECK(gu_g.scalar_type() == gu_u.scalar_type() && (gu_g.scalar_type() == at::kFloat || gu_g.scalar_type() == at::kHalf) && gu_g.dim() >= 1,
                "exl3_moe_coop: gu scratch must be float32 or float16 (slots, I)");
    TORCH_CHECK(ctr.scalar_type() == at::kInt, "exl3_moe_coop: ctr must be int32");

    amp_moe_coop_args a = {};
    a.x = x.data_ptr(); a.x_stride = (int) x.stride(0);
    a.sel = sel.data_ptr(); a.rw = rw.data_ptr();
    a.bsz = (int) x.size(0); a.topk = (int) sel.size(1);
    a.H = (int) x.size(1); a.Hi = Hi; a.I = (int) gu_u.size(-1); a.Ho = (int) d_out.size(-1); a.H_out = (int) out.size(-1);
    a.min_expert = min_expert; a.max_expert = max_expert; a.n_local = (int) u_trellis.numel();
    a.g_trellis = g_trellis.data_ptr(); a.g_suh = g_suh.data_ptr(); a.g_svh = g_svh.data_ptr();
    a.u_trellis = u_trellis.data_ptr(); a.u_suh = u_suh.data_ptr(); a.u_svh = u_svh.data_ptr();
    a.d_trellis = d_trellis.data_ptr(); a.d_suh = d_suh.data_ptr(); a.d_svh = d_svh.data_ptr();
    a.g_bias = opt_ptr(g_bias); a.u_bias = opt_ptr(u_bias); a.d_bias = opt_ptr(d_bias);
    a.Kgu = bits_of(Ku, "exl3_moe_coop"); a.Kd = bits_of(Kd, "exl3_moe_coop");
    a.cb = codebook(mcg, mul1); a.act = act; a.act_limit = act_limit; a.gated = gated ? 1 : 0;
    a.gu_g = gu_g.data_ptr(); a.gu_u = gu_u.data_ptr(); a.gu_f32 = gu_g.scalar_type() == at::kFloat ? 1 : 0;
    a.d_out = d_out.data_ptr(); a.ctr = (int*) ctr.data_ptr(); a.ctr_len = (long) ctr.numel();
    a.slots_max = (int) std::min(std::min(gu_g.numel(), gu_u.numel()) / std::max(a.I, 1), d_out.numel() / std::max(a.Ho, 1));
    TORCH_CHECK(a.bsz <= out.size(-2), "exl3_moe_coop: batch exceeds the output tensor");
    TORCH_CHECK(ctr.numel() >= amp_exl3_moe_coop_ctr_len(a.slots_max, a.bsz, a.I, a.Ho), "exl3_moe_coop: ctr too short for the scratch's slot count");
    a.out = out.data_ptr(); a.out_stride = (int) out.stride(-2);
    a.sh_out = opt_ptr(sh_out); a.sh_gate_w = opt_ptr(sh_gate_w);
    if (bits_g.has_value() || bits_u.has_value() || bits_d.has_value())
    {
        TORCH_CHECK(bits_g.has_value() && bits_u.has_value() && bits_d.has_value(), "exl3_moe_coop: give all three bit width tables or none");
        a.g_bits = bits_g->data_ptr(); a.u_bits = bits_u->data_ptr(); a.d_bits = bits_d->data_ptr();
        a.kmask_gu = bit_mask_of(*bits_u, a.n_local, "exl3_moe_coop"); a.kmask_d = bit_mask_of(*bits_d, a.n_local, "exl3_moe_coop");
        if (gated) TORCH_CHECK(bit_mask_of(*bits_g, a.n_local, "exl3_moe_coop") == a.kmask_gu, "exl3_moe_coop: gate and up of an expert must share a bit width");
    }
    check_rc(amp_exl3_moe_coop(&a, stream_of(x)), "exl3_moe_coop");
}

// Token-sorted prefill MoE with the reference's signature (vendor/exl3/exllamav3_ext/quant/exl3_moe.cuh:8-53).
// The reference's temps (temp_state_*, temp_intermediate_*) are accepted and not used: the kernels
// here work in one workspace per device and stream that this layer allocates on first use and grows
// when a larger chunk arrives (no allocation after that). num_active and m_tile only tune the
// reference's launch and are ignored; experts with more rows than the reference's temps hold
// (max_tokens_per_expert = temp_state_g.size(1)) are skipped exactly as the reference skips them,
// so that a caller who routes those through another tier does not get them twice. Per-expert bit
// tables are served for every codebook.
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
              const c10::optional<at::Tensor>& bits_d)
{
    (void) temp_state_u; (void) temp_intermediate_u; (void) m_tile;
    if (num_active == 0) return;
    const c10::cuda::CUDAGuard guard(hidden_state.device());
    TORCH_CHECK(hidden_state.dim() == 2 && hidden_state.scalar_type() == at::kHalf && hidden_state.is_contiguous(),
                "exl3_moe: hidden_state must be contiguous float16 (bsz, hidden)");
    TORCH_CHECK(output_state.scalar_type() == at::kFloat && output_state.is_contiguous() && output_state.sizes() == hidden_state.sizes(),
                "exl3_moe: output_state must be float32 of hidden_state's shape");
    TORCH_CHECK(expert_count.scalar_type() == at::kLong && expert_count.dim() == 1 && expert_count.is_contiguous(), "exl3_moe: expert_count int64");
    TORCH_CHECK(token_sorted.scalar_type() == at::kLong && token_sorted.dim() == 1 && token_sorted.is_contiguous() &&
                weight_sorted.scalar_type() == at::kHalf && weight_sorted.is_contiguous() && weight_sorted.numel() == token_sorted.numel(),
                "exl3_moe: token_sorted int64 / weight_sorted float16, one entry per pick");
    TORCH_CHECK(gate_mcg == up_mcg && up_mcg == down_mcg && gate_mul1 == up_mul1 && up_mul1 == down_mul1,
                "MoE kernel: gate/up/down must share the same codebook");
    TORCH_CHECK(temp_state_g.dim() == 3 && temp_intermediate_g.dim() == 3, "exl3_moe: temps must be 3-D");
    const int64_t E = expert_count.numel() - 1;
    for (const at::Tensor* t : { &gate_ptrs_trellis, &gate_ptrs_suh, &gate_ptrs_svh, &up_ptrs_trellis, &up_ptrs_suh, &up_ptrs_svh,
                                 &down_ptrs_trellis, &down_ptrs_suh, &down_ptrs_svh })
        TORCH_CHECK(t->scalar_type() == at::kLong && t->is_cuda() && t->is_contiguous() && t->numel() == E,
                    "exl3_moe: expert tables must be int64 device pointer tables, one entry per expert");

    amp_moe_sorted_args a = {};
    a.y = hidden_state.data_ptr(); a.out = output_state.data_ptr(); a.count = expert_count.data_ptr();
    a.tok_sorted = token_sorted.data_ptr(); a.w_sorted = weight_sorted.data_ptr();
    a.T = (int) hidden_state.size(0); a.H = (int) hidden_state.size(1); a.I = (int) temp_intermediate_g.size(2); a.E = (int) E;
    a.A = (long) token_sorted.numel();
    a.g_trellis = gate_ptrs_trellis.data_ptr(); a.g_suh = gate_ptrs_suh.data_ptr(); a.g_svh = gate_ptrs_svh.data_ptr();
    a.u_trellis = up_ptrs_trellis.data_ptr(); a.u_suh = up_ptrs_suh.data_ptr(); a.u_svh = up_ptrs_svh.data_ptr();
    a.d_trellis = down_ptrs_trellis.data_ptr(); a.d_suh = down_ptrs_suh.data_ptr(); a.d_svh = down_ptrs_svh.data_ptr();
    a.cb = codebook(gate_mcg, gate_mul1);
    // the reference's activation codes (quant/exl3_moe_common.cuh:6-8): 0 silu, 1 gelu, 2 = relu^2 without a gate projection
    a.gated = act_function == 2 ? 0 : 1;
    a.act = act_function == 2 ? 2 : act_function;
    a.act_limit = act_limit;
    const int cap = (int) temp_state_g.size(1);
    a.count_lo = count_lo;
    a.count_hi = count_hi > 0 ? std::min(count_hi, cap) : cap;
    if (bits_g.has_value() || bits_u.has_value() || bits_d.has_value())
    {
        TORCH_CHECK(bits_g.has_value() && bits_u.has_value() && bits_d.has_value(), "exl3_moe: give all three bit width tables or none");
        a.g_bits = a.gated ? bits_g->data_ptr() : nullptr; a.u_bits = bits_u->data_ptr(); a.d_bits = bits_d->data_ptr();
        a.kmask_gu = bit_mask_of(*bits_u, a.E, "exl3_moe"); a.kmask_d = bit_mask_of(*bits_d, a.E, "exl3_moe");
        if (a.gated) TORCH_CHECK(bit_mask_of(*bits_g, a.E, "exl3_moe") == a.kmask_gu, "exl3_moe: gate and up of an expert must share a bit width");
    }
    else
    {
        a.Kg = bits_of(K_gate, "exl3_moe"); a.Ku = bits_of(K_up, "exl3_moe"); a.Kd = bits_of(K_down, "exl3_moe");
    }
    if (output_scratch.has_value())
    {
        TORCH_CHECK(fused_base.has_value(), "exl3_moe: output_scratch needs fused_base");
        TORCH_CHECK(output_scratch->scalar_type() == at::kFloat && output_scratch->is_contiguous() && output_scratch->dim() == 2 &&
                    output_scratch->size(1) == hidden_state.size(1), "exl3_moe: output_scratch must be [slots, hidden]");
        TORCH_CHECK(fused_base->scalar_type() == at::kLong && fused_base->is_contiguous() && fused_base->numel() >= E, "exl3_moe: fused_base int64 per expert");
        a.scratch = output_scratch->data_ptr(); a.slot_base = fused_base->data_ptr(); a.scratch_rows = (long) output_scratch->size(0);
    }
    if (a.T == 0 || a.A == 0) return;
    const long need = amp_exl3_moe_sorted_workspace(a.T, a.A, a.E, a.H, a.I);
    TORCH_CHECK(need > 0, "exl3_moe: unsupported sizes");
    {
        // one workspace per (device, stream): calls on different streams may overlap on the GPU
        static std::map<std::pair<int, const void*>, at::Tensor> ws;
        static std::mutex mu;
        std::lock_guard<std::mutex> lock(mu);
        at::Tensor& w = ws[std::make_pair((int) hidden_state.get_device(), (const void*) stream_of(hidden_state))];
        if (!w.defined() || w.numel() < need)
            w = at::empty({need}, at::TensorOptions().dtype(at::kByte).device(hidden_state.device()));
        a.workspace = w.data_ptr(); a.workspace_bytes = (long) w.numel();
    }
    check_rc(amp_exl3_moe_sorted(&a, stream_of(hidden_state)), "exl3_moe");
}

// reference: exl3_moe_gather, vendor/exl3/exllamav3_ext/quant/exl3_moe.cu:472-531
void exl3_moe_gather(at::Tensor output_state, const at::Tensor& output_scratch, const at::Tensor& flat_expert,
                     const at::Tensor& inv_order, const at::Tensor& expert_start, const at::Tensor& slot_base,
                     const at::Tensor& slot_kind, const at::Tensor& weight_sorted)
{
    const c10::cuda::CUDAGuard guard(output_state.device());
    TORCH_CHECK(output_state.scalar_type() == at::kFloat && output_scratch.scalar_type() == at::kFloat && weight_sorted.scalar_type() == at::kHalf,
                "exl3_moe_gather: output_state / output_scratch float32, weight_sorted float16");
    for (const at::Tensor* t : { &flat_expert, &inv_order, &expert_start, &slot_base, &slot_kind })
        TORCH_CHECK(t->scalar_type() == at::kLong && t->is_contiguous(), "exl3_moe_gather: index tensors must be contiguous int64");
    TORCH_CHECK(output_state.is_contiguous() && output_state.dim() == 2, "exl3_moe_gather: output_state");
    TORCH_CHECK(output_scratch.is_contiguous() && output_scratch.dim() == 2 && output_scratch.size(1) == output_state.size(1),
                "exl3_moe_gather: output_scratch must be [slots, hidden]");
    const int64_t tokens = output_state.size(0), assign = flat_expert.numel(), E = slot_kind.numel();
    if (!tokens) return;
    TORCH_CHECK(assign % tokens == 0 && inv_order.numel() == assign, "exl3_moe_gather: assignments / tokens");
    TORCH_CHECK(slot_base.numel() >= E && expert_start.numel() >= E, "exl3_moe_gather: table sizes");
    check_rc(amp_exl3_moe_gather((float*) output_state.data_ptr(), (const float*) output_scratch.data_ptr(), flat_expert.data_ptr(),
                                 inv_order.data_ptr(), expert_start.data_ptr(), slot_base.data_ptr(), slot_kind.data_ptr(),
                                 weight_sorted.data_ptr(), (int) tokens, (int) output_state.size(1), (int) (assign / tokens), (int) E,
                                 (long) output_scratch.size(0), stream_of(output_state)),
             "exl3_moe_gather");
}

// The reference sizes its temps by this (SMs / 8 expert groups, quant/exl3_moe.cu:15-19); callers
// keep working, the temps they allocate from it are simply not used here.
int exl3_moe_max_concurrency(int device)
{
    int sms = 0;
    TORCH_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) == cudaSuccess, "exl3_moe_max_concurrency: bad device");
    return sms / 8;
}

// same arguments as the reference's exl3_moe_coop_ctr_len (vendor/exl3/exllamav3_ext/quant/exl3_moe_coop.cuh:164-167)
int64_t exl3_moe_coop_ctr_len(int64_t slots_max, int64_t bsz_max, int64_t I, int64_t Ho)
{
    return amp_exl3_moe_coop_ctr_len(slots_max, bsz_max, I, Ho);
}

#ifndef AMP_NO_PYBIND
PYBIND11_MODULE(_torch_glue, m)
{
    m.doc() = "reference-signature C++ layer of ampstein_b200 (for tests)";
    m.def("exl3_gemm", &exl3_gemm);
    m.def("exl3_mgemm", &exl3_mgemm);
    m.def("reconstruct", &reconstruct);
    m.def("reconstruct_had_slice", &reconstruct_had_slice);
    m.def("had_r_128", &had_r_128);
    m.def("exl3_moe_coop", &exl3_moe_coop);
    m.def("exl3_moe_coop_ctr_len", &exl3_moe_coop_ctr_len);
    m.def("exl3_moe", &exl3_moe);
    m.def("exl3_moe_gather", &exl3_moe_gather);
    m.def("exl3_moe_max_concurrency", &exl3_moe_max_concurrency);
}
#endif
