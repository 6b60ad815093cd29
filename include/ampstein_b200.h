/*
 * ampstein_b200 -- C ABI of the B200-native EXL3 quantized-linear path.
 *
 * This is the drop-in boundary: plain pointers and sizes, no C++ or torch types. Every entry
 * point launches on the given stream of the CURRENT device and returns immediately; none
 * synchronises, allocates or frees device memory unless its comment says so, which keeps
 * them capturable in CUDA graphs once warmed up.
 *
 * Return codes (the convention of the reference's own launchers,
 * src/torch/amp_torch.cpp:238-256): 0 = launched; negative = bad argument / unsupported
 * configuration (text in amp_b200_last_error()); positive = a cudaError_t.
 *
 * "Reference" citations below are paths inside the jow-/ampstein tree; Q/ abbreviates
 * vendor/exl3/exllamav3_ext/quant/.
 *
 * Data layout shared by all entry points:
 *   trellis  int16/uint16 (k/16, n/16, 16*K): one 16x16 tile = 256*K bits, K = 1..8
 *   suh      fp16 (k) input sign/scale vector,  svh  fp16 (n) output sign/scale vector
 *   cb       codebook: 0 = default ("3INST"), 1 = mcg, 2 = mul1
 *   the linear is  C = had128(A * suh) @ W_hat  ->  had128(.) * svh,   W_hat = decoded tiles (k, n)
 */
#ifndef AMPSTEIN_B200_H
#define AMPSTEIN_B200_H

#ifdef __cplusplus
extern "C" {
#endif

#ifndef __CUDA_RUNTIME_API_H__
typedef struct CUstream_st* cudaStream_t;
#endif

/* Library version (bumped on ABI changes). */
int amp_b200_version(void);

/* Text of the last error reported on the calling thread ("" when none). */
const char* amp_b200_last_error(void);

/*
 * Bitrate argument K of the entry points below: 1..8 bits per weight, or, where an entry says so,
 * AMP_EXL3_HALF_RATE(KA) for the half-integer rates KA + 0.5 = 1.5 / 2.5 / 3.5 (mul1 codebook only;
 * the trellis tensor's third dimension is then 16 KA + 8). The reference passes these rates as a
 * float K (Q/bits_k.cuh:14-29). Entries that accept them: amp_exl3_reconstruct,
 * amp_exl3_reconstruct_had, amp_exl3_gemm (up to 16 rows, A_had required), amp_exl3_shard_cols /
 * amp_exl3_shard_rows. The fused / bundle / grouped entries and the int8 form take integer rates only.
 */
#define AMP_EXL3_HALF_RATE(KA) (256 + (KA))

/*
 * Dequantize a trellis into fp16 W_hat (rotated basis). Bit-exact with the reference.
 * Replaces: reconstruct / reconstruct_slice, Q/reconstruct.cu:141-197, 512-523
 *           (binding torch.exl3_reconstruct, src/torch/amp_torch.cpp:11015-11060).
 * unpacked: fp16 (k, n_out) receiving columns [n_offset, n_offset + n_out) of the (k, n) weight.
 * n_out and n_offset multiples of 128, k a multiple of 16. Empty tensors are a no-op.
 */
int amp_exl3_reconstruct(void* unpacked, const void* trellis, int k, int n, int K, int cb,
                         int n_offset, int n_out, cudaStream_t stream);

/*
 * Dequantize into the ORIGINAL basis: diag(suh) . H128 . W_hat . H128 . diag(svh) / 128, with
 * the reference's per-element operation order (bit-exact with it).
 * Replaces: reconstruct_had_slice, Q/reconstruct.cu:431-503.
 * k, n_out, n_offset multiples of 128; svh points at the slice's first column.
 */
int amp_exl3_reconstruct_had(void* unpacked, const void* trellis, const void* suh, const void* svh,
                             int k, int n, int K, int cb, int n_offset, int n_out,
                             cudaStream_t stream);

/*
 * Batch forms: `batch` whole matrices of one shape in one launch. unpacked (batch, k, n) fp16
 * contiguous; packed_ptrs (and suh_ptrs / svh_ptrs) are DEVICE arrays of int64 addresses, one per
 * matrix. n a multiple of 128; k a multiple of 16 (rotated basis) or 128 (original basis).
 * Replaces: reconstruct_batch / reconstruct_had_batch, Q/reconstruct.cu:512-626 (kernels :102-139,
 * :381-429).
 */
int amp_exl3_reconstruct_batch(void* unpacked, const void* packed_ptrs, int batch, int k, int n, int K, int cb,
                               cudaStream_t stream);
int amp_exl3_reconstruct_had_batch(void* unpacked, const void* packed_ptrs, const void* suh_ptrs, const void* svh_ptrs,
                                   int batch, int k, int n, int K, int cb, cudaStream_t stream);

/*
 * Blockwise 128-point Hadamard of a (rows, cols) matrix, out = H(in [* pre]) * scale/sqrt(128)
 * [* post]; in place allowed. dtype 0 = fp16, 1 = fp32, 2 = bf16 in / fp16 out, 3 = fp32 in / fp16
 * out (2 and 3 not in place; 3 is the form the reference applies to fp32 accumulators,
 * had_fh_r_128_inner, Q/hadamard_inner.cuh:216-279). pre / post: fp16 (cols) or NULL.
 * Replaces: had_r_128, Q/hadamard.cu:125-207.
 */
int amp_had_r_128(const void* in, void* out, const void* pre, const void* post,
                  long rows, int cols, int dtype, float scale, cudaStream_t stream);

/*
 * EXL3 linear, any m: C (m, n) fp16 (c_fp32 = 0) or fp32 (c_fp32 = 1) = A (m, k) fp16 through
 * the quantized weight. suh and svh are required. k and n multiples of 128. Up to 16 rows run on
 * the decode kernel; more rows on the tensor-core (tcgen05) prefill kernel, which needs A_had:
 * the reference's scratch argument, m * k halves, 16-byte aligned (it receives the rotated input
 * in an internal order; its contents mean nothing to the caller). With 5..16 rows A_had is optional:
 * when given, the input is rotated into it once by a small launch of its own instead of by every
 * CTA of the decode kernel (about 10 % faster at eight rows); NULL keeps the single launch.
 * Replaces: exl3_gemm, Q/exl3_gemm.cu:114-349 (binding torch.exl3_gemm,
 * src/torch/amp_torch.cpp:11250-11293), including its GEMV dispatch Q/exl3_gemv.cu:92-184, and,
 * above 144 rows, the reconstruct + cuBLAS path of torch.exl3_gemm_recon
 * (src/torch/amp_torch.cpp:11148-11230).
 */
int amp_exl3_gemm(const void* A, const void* trellis, void* C, const void* suh, void* A_had,
                  const void* svh, int m, int k, int n, int K, int cb, int c_fp32,
                  cudaStream_t stream);

/*
 * Same with bf16 activations (A is (m, k) bf16; A_had (m, k) fp16 is required at every m). The
 * reference has no counterpart: its exl3_gemm accepts fp16 only (Q/exl3_gemm.cu:136).
 */
int amp_exl3_gemm_bf16(const void* A, const void* trellis, void* C, const void* suh, void* A_had,
                       const void* svh, int m, int k, int n, int K, int cb, int c_fp32,
                       cudaStream_t stream);

/*
 * Form of the prefill GEMM: 0 = one CTA per tile only, 1 = by shape (default: CTA pairs with
 * tcgen05 cta_group::2 whenever n is a multiple of 256: 256 tokens x 256 columns per pair while
 * that grid fits one wave, 512 tokens beyond; single CTAs otherwise), 2 / 3 = pairs of
 * 512 / 256 tokens whenever n is a multiple of 256 (for tests). Returns the previous setting. No
 * counterpart in the reference.
 */
int amp_exl3_set_gemm_pair(int mode);
/*
 * Int8-activation form of the one-row GEMV for mul1 (codebook 2) tensors up to max_k bits: the
 * rotated input is quantised to int8 with one scale per 128 rows of k and the dot product runs as
 * dp4a on the byte sum of the codebook's product, exact in int32 (about 6e-3 relative rms against
 * the fp16 form). mode: 0 off, 2 on (default), 1 on with the error-feedback pass (the rounding error of
 * the codes quantised again at 1/254 of the scale and accumulated by a second dp4a: about 2e-4
 * relative rms, at the speed of the fp16 kernel) -- the reference's EXL3_INT8_GEMV modes, whose
 * value this library also reads from the environment at load, with EXL3_INT8_GEMV_MAX_K, default 6.
 * max_k <= 0 leaves the bit-width limit as it is. Returns the previous mode.
 * Replaces: the dispatch of exl3_gemm to exl3_gemv_int8, Q/exl3_gemm.cu:188-196,
 * Q/exl3_gemv_int8.cu:20-52, kernel Q/exl3_gemv_int8_kernel.cuh (m == 1 only; half-integer
 * bitrates are not supported).
 */
int amp_exl3_set_int8_gemv(int mode, int max_k);
/*
 * Pair form only: the one remote mbarrier arrival per k step that tells the first CTA of a pair that
 * the second CTA's operands are ready is `relaxed` by default; 1 selects `release.cluster`, the form
 * the PTX memory model asks for on paper (slower; results are identical, which a test checks).
 * Returns the previous setting. No counterpart in the reference.
 */
int amp_exl3_set_gemm_relay_release(int enable);

/* Reads and clears the prefill GEMM's status word (non-zero: a bounded wait on a tensor-core
 * completion barrier ran out). Synchronises; diagnostics only. */
int amp_exl3_gemm_status(int* out);

/*
 * The decode-batch kernel on its own, m = 1..16. The first call on a device allocates a
 * workspace for the stream it is issued on (16 MB + 64 KB of arrival counters and partial-sum slots per
 * stream and device, so that launches overlapping on different streams never share counters) and must
 * therefore come before any capture on that stream; later calls on the stream allocate nothing.
 * Replaces: exl3_gemv_kernel / exl3_gemv_try_launch, Q/exl3_gemv_kernel.cuh:186-482,
 * Q/exl3_gemv.cu:92-184.
 */
int amp_exl3_gemv(const void* x, const void* trellis, void* c, const void* suh, const void* svh,
                  int m, int k, int n, int K, int cb, int c_fp32, cudaStream_t stream);

/*
 * The decode kernel without any device allocation, ever: its arrival counters and partial-sum
 * slots live in a fixed 2 MB array inside the library instead of the lazily allocated workspace.
 * This entry point has no counterpart in the reference. Limits: m = 1..4, n <= 131072 (a multiple
 * of 128), k a multiple of 128; anything larger is refused with a negative return and a message.
 * The first call on a device looks up the array's address (cudaGetSymbolAddress), so it should
 * come before any stream capture; later calls only launch. Every call on a device uses the same
 * array: calls that overlap on the GPU (other streams, parallel graph branches) race on it and
 * must be serialised by the caller. The counters in the array are zero when the library is
 * loaded and each launch leaves them zero; nothing else needs initialising.
 */
int amp_exl3_gemv_static(const void* x, const void* trellis, void* c, const void* suh, const void* svh,
                         int m, int k, int n, int K, int cb, int c_fp32, cudaStream_t stream);

/*
 * Same with a fixed number of CTAs (split, 1..1024: the work is cut into that many equal
 * ranges) and number of 64-row groups of the transformed input held in shared memory at a time
 * (xgroups, a multiple of 4 up to 128; smaller values force more chunks); 0 = choose. The counterpart of the
 * reference's force_shape_idx / force_num_sms arguments (Q/exl3_gemm.cu:114-127), used by
 * tuning and tests.
 */
int amp_exl3_gemv_cfg(const void* x, const void* trellis, void* c, const void* suh, const void* svh,
                      int m, int k, int n, int K, int cb, int c_fp32, int split, int xgroups,
                      cudaStream_t stream);

/*
 * Down projection with the gated activation folded into its input side: C (m, n) = the linear of
 * a = fp16(silu(gate) * up), gate / up (m, k) fp16 (e.g. the two slabs of the gate|up bundle's stacked
 * output). One launch instead of two; fp32 activation math and one rounding as the stand-alone kernel.
 * m <= 16.
 * Replaces: the pair torch.silu_mul + torch.exl3_gemm of the decode step,
 * src/ucode/ampstein/graphdec.uc:205-217 (kernel amp_silu_mul_kernel, src/torch/amp_kernels.cu:235-251);
 * the reference has no fused form for dense layers (its fused MoE does the same for experts).
 */
int amp_exl3_gemv_silu_mul(const void* gate, const void* up, const void* trellis, void* C, const void* suh, const void* svh,
                           int m, int k, int n, int K, int cb, int c_fp32, cudaStream_t stream);

/*
 * Linear (or bundle) behind the fused residual add + RMSNorm of the decode step, in ONE launch:
 *   y (m, k)  = fp16(x + res)                                   the updated residual stream
 *   C         = the linear(s) of  fp16(y * rsqrt(mean(y^2) + eps)) * norm_w   (fp16 multiply)
 * x, res, y (m, k) fp16, norm_w (k) fp16; y must not alias x or res (every CTA re-reads x while the
 * first one writes y). The sum of squares is formed per CTA (fp32, a fixed order that differs from
 * the stand-alone kernel's, so the scale may differ in its last bit). m <= 16. The bundle form
 * takes amp_exl3_mgemm's tables.
 * Replaces: torch.rms_norm_res followed by the q|k|v / gate|up bundle or the lm_head,
 * src/ucode/ampstein/graphdec.uc:163-225 (kernel amp_rms_norm_res_kernel,
 * src/torch/amp_kernels.cu:279-360); the reference has no fused form.
 */
int amp_exl3_gemv_rms_norm_res(const void* x, const void* res, const void* norm_w, float eps, void* y,
                               const void* trellis, void* C, const void* suh, const void* svh,
                               int m, int k, int n, int K, int cb, int c_fp32, cudaStream_t stream);
/*
 * Stand-alone forms of the three element-wise kernels the fused entry points above absorb (residual
 * add + RMSNorm, gated activation, greedy pick + state advance), with the arithmetic of the fused
 * forms. Provided so that fused and unfused sequences can be compared inside one CUDA graph; an
 * integrator keeps the reference's own kernels (amp_rms_norm_res_fp16, amp_silu_mul_fp16,
 * amp_argmax_advance_fp16, src/torch/amp_kernels.cu:253-271, 362-390, 903-960) or switches to the
 * fused entries. y may alias x here (one CTA per row). ws of argmax_advance: 16 bytes, zero before the
 * first call.
 */
int amp_b200_rms_norm_res(const void* x, const void* r, const void* w, void* y, void* n, long rows, int dim, float eps,
                          cudaStream_t stream);
int amp_b200_silu_mul(const void* g, const void* u, void* out, long count, cudaStream_t stream);
int amp_b200_argmax_advance(const void* logits, int n, void* ids, void* pos, void* log, long long log_cap, void* ws,
                            cudaStream_t stream);
/*
 * The residual norm split between the launches on either side of it (the form that pays: nothing
 * reads a whole row on a CTA's critical path).
 *   amp_exl3_gemv_add_res   y (m, n) = fp16(h + linear(x)), the updated residual stream (the linear's own
 *                           output is not stored), and ssq (m, n / 128) fp32 = the sum of squares of y per
 *                           128-column block, written by the warps that finish the blocks. y must not
 *                           alias h. Replaces exl3_gemm (o_proj / down_proj) + the add of rms_norm_res.
 *   amp_exl3_gemv_normed /  the linear / bundle of fp16(y * rsqrt(sum(ssq row) / k + eps)) * norm_w: the
 *   amp_exl3_mgemm_normed   prologue adds the k / 128 block sums up and scales. Replaces the norm of
 *                           rms_norm_res + the q|k|v / gate|up bundle or the lm_head.
 * m <= 16; fp16 y. Same rounding points as amp_rms_norm_res_kernel (src/torch/amp_kernels.cu:279-360);
 * the sum of squares is added in another (fixed) order. The reference has no such entry points.
 */
int amp_exl3_gemv_add_res(const void* x, const void* trellis, const void* suh, const void* svh,
                          const void* h, void* y, void* ssq, int m, int k, int n, int K, int cb, cudaStream_t stream);
int amp_exl3_gemv_normed(const void* y, const void* ssq, const void* norm_w, float eps,
                         const void* trellis, void* C, const void* suh, const void* svh,
                         int m, int k, int n, int K, int cb, int c_fp32, cudaStream_t stream);
int amp_exl3_mgemm_normed(const void* y, const void* ssq, const void* norm_w, float eps,
                          const void* trellis_ptrs, void* C, const void* suh_ptrs, const void* svh_ptrs,
                          int num, int m, int k, int width, int K, int cb, int c_fp32,
                          const void* c_ptrs, const void* n_stride_list, const void* had_src_list, cudaStream_t stream);
/*
 * The last three launches of a greedy decode step in one: y = fp16(x + res), logits (1, n) fp16 = the
 * lm_head of RMSNorm(y) * norm_w, then argmax over the first `vocab` logits and the state advance
 * log[pos] = ids; ids = argmax; pos += 1 (ids, pos: one int64 each; log: int64 array of log_cap
 * entries, the write is skipped when pos is outside it). Ties go to the lowest index, NaN logits are
 * skipped, no valid logit gives 0. ws: 16 bytes, 8-byte aligned, zero before the first call (every
 * call leaves it zero); one ws per decoder that may run concurrently.
 * Replaces: torch.rms_norm_res + torch.exl3_gemm + torch.argmax_advance,
 * src/ucode/ampstein/graphdec.uc:219-240 (kernel amp_argmax_advance_kernel,
 * src/torch/amp_kernels.cu:823-901, same tie and NaN rules); the reference has no fused form.
 */
int amp_exl3_lm_head_argmax(const void* x, const void* res, const void* norm_w, float eps, void* y,
                            const void* trellis, void* logits, const void* suh, const void* svh,
                            int k, int n, int K, int cb, int vocab,
                            void* ids, void* pos, void* log, long long log_cap, void* ws, cudaStream_t stream);
int amp_exl3_mgemm_rms_norm_res(const void* x, const void* res, const void* norm_w, float eps, void* y,
                                const void* trellis_ptrs, void* C, const void* suh_ptrs, const void* svh_ptrs,
                                int num, int m, int k, int width, int K, int cb, int c_fp32,
                                const void* c_ptrs, const void* n_stride_list, const void* had_src_list, cudaStream_t stream);

/*
 * Several EXL3 matrices -- or equal-width column slices of matrices -- against ONE shared input
 * x (m, k) in a single launch, m <= 16. Matrices are named by DEVICE pointer tables (int64
 * device arrays), exactly as the reference takes them, so no host synchronisation is needed:
 *   trellis_ptrs[num], svh_ptrs[num]  per slice (already offset to the slice's first column)
 *   suh_ptrs[num_had_src]             per source matrix; had_src_list[num] (int32) maps a slice
 *                                     to its source, NULL = identity
 *   c_ptrs[num] + n_stride_list[num]  per-slice output pointer and row width of the matrix it
 *                                     belongs to; both NULL = outputs stacked in C (num, m, width)
 * All slices share k, K, the codebook and the width (a multiple of 128). Up to 16 rows run on the
 * decode kernel (A_had, when given, receives the rotated input of every source from five rows up,
 * as for amp_exl3_gemm); more rows run as ONE tensor-core grid over all slices and A_had
 * ((sources, m, k) fp16, sources = num_had_src or num) is required.
 * Replaces: exl3_mgemm, Q/exl3_gemm.cu:351-735 (binding torch.mgemm,
 * src/torch/amp_torch.cpp:10193-10322; bundle builders src/ucode/ampstein/models.uc:338-432).
 * size_n_list of the reference's signature has no counterpart here: every slice is `width` columns
 * wide (the reference's caller cuts matrices into equal slices, src/ucode/ampstein/models.uc:373-398).
 */
int amp_exl3_mgemm(const void* x, const void* trellis_ptrs, void* C, const void* suh_ptrs,
                   void* A_had, const void* svh_ptrs, int num, int m, int k, int width,
                   int K, int cb, int c_fp32, const void* c_ptrs, const void* n_stride_list,
                   const void* had_src_list, int num_had_src, cudaStream_t stream);
/* The same with bf16 activations (any row count takes the tensor-core path). No counterpart in the
 * reference, whose bundle checks for fp16 (Q/exl3_gemm.cu:429). */
int amp_exl3_mgemm_bf16(const void* x, const void* trellis_ptrs, void* C, const void* suh_ptrs,
                        void* A_had, const void* svh_ptrs, int num, int m, int k, int width,
                        int K, int cb, int c_fp32, const void* c_ptrs, const void* n_stride_list,
                        const void* had_src_list, int num_had_src, cudaStream_t stream);

/*
 * Fused decode-shaped MoE: out[row] = sum over the row's active picks of rw * expert(x[row]),
 * expert = down(act(gate(x), up(x))), plus an optional shared-expert term. Up to 256
 * (token, pick) slots per call. Routing (sel, rw) is read on the device; nothing synchronises.
 * Three launches (run table, gate|up, down: the CTA that delivers the last of a token's picks for
 * an output chunk also does the routing-weighted sum), two for a single token.
 * Replaces: exl3_moe_coop, Q/exl3_moe_coop.cu:309-371 and its parameter block MoeCoopParams,
 * Q/exl3_moe_coop.cuh:21-83 (binding torch.moe_coop, src/torch/amp_torch.cpp:7852-7934). Fields
 * keep the reference's names and meaning; scratch the new kernels do not need (had_g, had_u,
 * act_out) has no field.
 */
typedef struct amp_moe_coop_args
{
    const void* x;              /* (bsz, H) fp16, row stride x_stride */
    int x_stride;
    const void* sel;            /* (bsz, topk) int64 global expert indices */
    const void* rw;             /* (bsz, topk) fp16 routing weights (0 = inactive pick) */
    int bsz, topk;
    int H;                      /* x width (<= Hi, multiple of 4) */
    int Hi, I, Ho;              /* padded gate/up input, intermediate, down output widths (x128) */
    int H_out;                  /* output width (<= Ho) */
    int min_expert, max_expert; /* min_expert < 0: no range filter; else sel in [min, max) is local */
    int n_local;                /* entries in the pointer tables */
    /* per-expert int64 device pointer tables, indexed by local expert */
    const void* g_trellis; const void* g_suh; const void* g_svh;
    const void* u_trellis; const void* u_suh; const void* u_svh;
    const void* d_trellis; const void* d_suh; const void* d_svh;
    const void* g_bias; const void* u_bias; const void* d_bias;   /* nullable */
    int Kgu, Kd;                /* bit widths of gate/up and down */
    int cb;                     /* codebook, uniform across the three projections */
    int act;                    /* 0 silu, 1 gelu, 2 relu2, 3 gpt-oss clamped swiglu */
    float act_limit;
    int gated;                  /* 0: no gate projection, activation is relu(u) * u */
    /* scratch, leading dimension >= slots_max */
    void* gu_g; void* gu_u;     /* (slots_max, I) fp32 (gu_f32 = 1) or fp16 (gu_f32 = 0) */
    int gu_f32;
    void* d_out;                /* (slots_max, Ho) fp32 */
    int* ctr;                   /* int32 scratch, zero-filled once: run table, active picks per token, arrivals per
                                   (token, 128-column output chunk); the kernels leave the arrivals zero */
    long ctr_len;               /* entries in ctr, >= amp_exl3_moe_coop_ctr_len(slots_max, bsz, I, Ho) */
    int slots_max;
    void* out;                  /* (bsz, H_out) fp32, row stride out_stride */
    int out_stride;
    const void* sh_out;         /* nullable: (bsz, H) fp32 shared-expert output */
    const void* sh_gate_w;      /* nullable: (H) fp16, gate = sigmoid(x . w) */
    /* mixed bit widths (nullable, all three or none): uint8 device tables indexed by local expert;
     * gate and up of an expert share one width (g_bits[e] == u_bits[e]). kmask_gu / kmask_d: bit K-1
     * set for every width K that occurs in u_bits / d_bits (host values: the tables are static, the
     * caller reads them once); Kgu / Kd are ignored then. One pair of launches per width.
     * Reference: g_bits / u_bits / d_bits of MoeCoopParams, Q/exl3_moe_coop.cuh:46-50. */
    const void* g_bits; const void* u_bits; const void* d_bits;
    int kmask_gu, kmask_d;
} amp_moe_coop_args;

int amp_exl3_moe_coop(const amp_moe_coop_args* args, cudaStream_t stream);

/* Length (int32 entries) of the ctr scratch for up to slots_max (token, pick) slots and rows_max
 * tokens: 2 + 4 * slots_max + rows_max * (1 + Ho / 128). Same arguments as the reference's
 * exl3_moe_coop_ctr_len, Q/exl3_moe_coop.cuh:164-167 (I is not needed here); never longer than
 * the reference's figure when I >= 384. */
long amp_exl3_moe_coop_ctr_len(long slots_max, long rows_max, long I, long Ho);

/*
 * Token-sorted MoE for prefill chunks: for every expert e whose row count lies in
 * [count_lo, count_hi], the rows tok_sorted[start_e .. start_e + count[e]) of y go through gate / up,
 * the activation and down, and weight * result is summed per token, in ascending expert order,
 * and ADDED to out (fp32; the caller zero-fills it, as for the reference). start_e is the running
 * sum of count[0..e); the sentinel bin count[E] (picks that belong to nobody here) is ignored.
 * Every token must own the same number of entries of the sorted list (A = T * picks, picks <= 64).
 * Routing stays on the device; the call enqueues six launches on `stream` and returns (no
 * allocation, no host read-back: capturable in a CUDA graph and replayable with other routing in the
 * same tensors). Calls that share a workspace must be ordered on one stream.
 * Replaces: exl3_moe, Q/exl3_moe.cu:139-531 (kernel Q/exl3_moe_kernel.cuh:61-313) together with
 * exl3_moe_gather, its fixed-order slot sum; bindings torch.moe_fused / torch.moe_gather,
 * src/torch/amp_torch.cpp:9257-9378. Differences: one call covers every row count (the reference
 * needs one launch per row tier 1-16 / 17-32 / 33+ and leaves experts above its temp capacity to
 * the caller), all three codebooks are served (the reference instantiates mcg and mul1 only,
 * Q/exl3_moe.cu:33-46), the temps ts_g ts_u ti_g ti_u, the slot scratch and slot_base are one
 * caller-provided workspace, and without a slot scratch the sum is a fixed-order one made by the
 * call itself (the reference adds atomically in arrival order then). Per-expert bit width
 * tables are served for every codebook (the reference: mul1 only).
 */
typedef struct amp_moe_sorted_args
{
    const void* y;              /* (T, H) fp16, contiguous */
    void* out;                  /* (T, H) fp32, contiguous; accumulated into */
    const void* count;          /* (E + 1) int64: rows per expert, last entry ignored */
    const void* tok_sorted;     /* (A) int64 token index of every pick, sorted by expert */
    const void* w_sorted;       /* (A) fp16 routing weight of every pick, same order */
    int T, H, I, E;
    long A;
    /* per-expert int64 device pointer tables (E entries); every tensor they name 16-byte aligned */
    const void* g_trellis; const void* g_suh; const void* g_svh;
    const void* u_trellis; const void* u_suh; const void* u_svh;
    const void* d_trellis; const void* d_suh; const void* d_svh;
    int Kg, Ku, Kd;             /* bit widths */
    int cb;                     /* codebook, uniform across the three projections */
    int act;                    /* as amp_moe_coop_args */
    float act_limit;
    int gated;                  /* 0: no gate projection (g_* ignored), activation relu(u) * u */
    int count_lo, count_hi;     /* experts with row counts outside are skipped; <= 0: no bound */
    void* workspace;            /* 256-byte aligned device scratch */
    long workspace_bytes;       /* >= amp_exl3_moe_sorted_workspace(T, A, E, H, I) */
    /* deferred sum (nullable; the reference's output_scratch / fused_base): with scratch set, out is
     * left alone and weight * result of the r-th row of expert e is stored in scratch row
     * slot_base[e] + r, for amp_exl3_moe_gather to add up */
    void* scratch;              /* (scratch_rows, H) fp32 */
    const void* slot_base;      /* (E) int64 */
    long scratch_rows;
    /* experts of different bit widths (nullable, all or none; g_bits only when gated): uint8 device
     * tables indexed by expert, gate and up of an expert sharing one width; kmask_gu / kmask_d as in
     * amp_moe_coop_args (host values); Kg / Ku / Kd are ignored then. One GEMM launch per width that
     * occurs. Reference: bits_g / bits_u / bits_d of exl3_moe, Q/exl3_moe.cuh:50-52 (there mul1 only). */
    const void* g_bits; const void* u_bits; const void* d_bits;
    int kmask_gu, kmask_d;
} amp_moe_sorted_args;

int amp_exl3_moe_sorted(const amp_moe_sorted_args* args, cudaStream_t stream);
/*
 * Tensor-parallel shards cut on the device (load path). amp_exl3_shard_cols: the output columns of
 * `ranges` (nranges <= 16 host pairs [start, length], multiples of 128, in order) of a trellis
 * (k/16, n/16, 16K) concatenated into out_trellis (k/16, total/16, 16K), and the same slices of svh (n)
 * into out_svh (total) (both null: trellis only), one launch; the destinations may live on another
 * GPU when peer access is enabled. amp_exl3_shard_rows: input rows [k0, k0 + klen) (multiples of
 * 128) of the trellis and of suh, two contiguous copies. Byte moves, bit-exact. Replace the
 * narrow / torch.cat / contiguous / .cuda(dev) chains of sub_columns, cols and rows,
 * src/ucode/ampstein/models.uc:440-562 (same alignment rules and error cases).
 */
int amp_exl3_shard_cols(const void* trellis, const void* svh, void* out_trellis, void* out_svh, int k, int n, int K,
                        const int* ranges, int nranges, cudaStream_t stream);
int amp_exl3_shard_rows(const void* trellis, const void* suh, void* out_trellis, void* out_suh, int k, int n, int K,
                        int k0, int klen, cudaStream_t stream);
/*
 * Token-sorted MoE dispatch in one launch: idx (A = T * K) int64 global expert ids and w (A) fp32
 * router weights become, for the experts [e0, e0 + E) of this rank (foreign picks in the sentinel
 * bucket E): fe (A) bucket per assignment, order (A) the assignment at every sorted position (a
 * stable sort by bucket), tok (A) its token, wts (A) fp16 its weight, count / start (E + 1) sizes
 * and first positions of the buckets, inv (A) the sorted position of every assignment, kind (E) =
 * count > 0. All index tensors int64 on the device; 1 <= E <= 4096. Returns a cudaError_t.
 * Same name, signature and meaning as the reference's amp_moe_prep, src/torch/amp_kernels.cu:7024-7043
 * (binding torch.moe_prep, src/torch/amp_torch.cpp:8164-8215).
 */
int amp_moe_prep(const long long* idx, const float* w, int A, int K, int E, long long e0, long long* fe,
                 long long* order, long long* tok, void* wts, long long* count, long long* start,
                 long long* inv, long long* kind, cudaStream_t stream);
/*
 * Fixed-order sum of per-assignment slots: for every token, the slots of its picks k = 0 .. topk - 1
 * are added in that order (fp32) and the sum is added to out (T, H). Pick a = token * topk + k of
 * local expert e = flat_expert[a] (outside [0, E): no slot) owns slot slot_base[e] + inv_order[a] -
 * expert_start[e] when slot_kind[e] != 0; kind 1 slots hold weighted rows, kind 2 unweighted ones,
 * multiplied here by w_sorted[inv_order[a]]. All index tensors int64 on the device. Same arguments
 * and meaning as the reference's exl3_moe_gather, Q/exl3_moe.cu:472-531; slots outside
 * [0, scratch_rows) are skipped instead of read.
 */
int amp_exl3_moe_gather(float* out, const float* scratch, const void* flat_expert, const void* inv_order,
                        const void* expert_start, const void* slot_base, const void* slot_kind, const void* w_sorted,
                        int T, int H, int topk, int E, long scratch_rows, cudaStream_t stream);
/* bytes of workspace for a chunk of T tokens with A picks over E experts (0: bad sizes) */
long amp_exl3_moe_sorted_workspace(long T, long A, long E, long H, long I);
/* Rows per GEMM tile of amp_exl3_moe_sorted in units of 128 (one tile = rows of one expert whose
 * weight block a CTA decodes once): 0 (default) = chosen per call from the average rows per expert,
 * 1..4 forced; for A/B measurements. Returns the previous setting. No reference counterpart (its
 * row tiers are the caller's m_tile argument). */
int amp_exl3_set_moe_sorted_tile(int sub);
/* Reads the status word the last call left in its workspace: 0 = clean, bits 0 / 1 = count[]
 * describes more rows than the sorted list holds, bit 2 = a token index outside [0, T), bit 3 = a
 * token with more than A / T entries. Entries in error are left out of the sum; nothing is read
 * or written out of bounds. Synchronises the stream; not for the hot path. */
int amp_exl3_moe_sorted_status(const void* workspace, int* out, cudaStream_t stream);

/*
 * Programmatic dependent launch of the decode kernels (default on): each kernel starts its
 * weight stream before waiting for the kernel in front of it. Returns the previous setting.
 * The reference has no counterpart (it launches cooperative kernels back to back).
 */
int amp_exl3_set_pdl(int enable);

/*
 * Which kernel serves dense and bundle GEMV launches of up to eight rows: 0 (default) the
 * register-operand mma.sync kernel, 1 the tensor-memory kernel (decoded weights written to tensor
 * memory with tcgen05.st, dot products by tcgen05.mma with the weights as the A operand). Both
 * give the same results to rounding; the mma.sync kernel is the faster one on B200 and always
 * serves 9..16 rows and the grouped expert modes. For A/B measurements. Returns the previous
 * setting. The reference has no counterpart (its kernels use mma.sync only,
 * Q/exl3_gemv_kernel.cuh:396-397).
 */
int amp_exl3_set_gemv_tc(int enable);

/*
 * Measurement aid behind `python bench.py --workload issue` (not part of the hot path): cycles one
 * SM scheduler needs per 8 decoded weights and lane for the decode kernel's K = 4 instruction mix
 * when the dot product is fed by two mma.sync (variant 0), by one tcgen05.st into tensor memory
 * (1), not at all (2: checksum), or for the two mma.sync alone (3), at 1..8 resident warps per
 * scheduler. Synchronises and allocates its own buffers. The reference has no counterpart.
 */
int amp_diag_issue_cycles(int variant, int warps_per_scheduler, float* cycles_per_iter);

/*
 * Reads and clears the current device's GEMV status word (non-zero = a kernel reported an
 * internal error: a bounded wait on one of the tensor-memory kernel's hand-over barriers ran out).
 * Synchronises; not for the hot path.
 */
int amp_exl3_gemv_status(int* out);

/*
 * ---- tensor-parallel decode: fp16 all-reduce over peer-mapped memory (NVLink) ----
 *
 * rank's part of an N-way (2..8) all-reduce of the ranks' contiguous fp16 partials: x and out are
 * n halves on this rank's device (n % 8 == 0, n <= cap); bufs[p] / ctls[p] are every rank's buffer
 * and control block as THIS process addresses them (peer access or IPC mappings), each
 * zero-filled once before the first call and sized by amp_comm_buffer_bytes / amp_comm_ctl_bytes.
 * All ranks must issue the same sequence of calls with the same n, mode and blocks. mode 0 =
 * one-shot, 1 = two-phase (reduce-scatter + all-gather); blocks 1..16 (amp_comm_blocks gives the
 * value every rank should use). The sum accumulates in fp32 in rank order and rounds once:
 * bit-identical on every rank. Graph-capturable; waits on peers are bounded (a rank that never
 * arrives makes the call return with the status word set, it does not trap).
 * Same signature and return convention (a cudaError_t) as the reference:
 * amp_comm_allreduce_fp16, src/torch/amp_kernels.cu:2966-2986 (binding comm.allreduce,
 * src/torch/amp_torch.cpp:7710-7759). The buffer layout differs from the reference's (the flags
 * travel inside the data), hence the sizing functions below; the reference sizes its buffers
 * in torch_p2p_comm, src/torch/amp_torch.cpp:7682-7689.
 */
int amp_comm_allreduce_fp16(const void* x, void* out, void* const* bufs, int* const* ctls,
                            int rank, int N, long n, long cap, int mode, int blocks,
                            cudaStream_t stream);
/*
 * Row-parallel EXL3 linear of tensor-parallel decode with the all-reduce fused into the kernel:
 * out (m, n) fp16 on every rank = sum over ranks of (this rank's x (m, k) through its row shard of
 * the weight), m <= 16, m * n <= cap. The CTA that finishes a 128-column block pushes the block's
 * fp16 partial into every peer's buffer and adds up the peers' partials of that block (fp32, rank
 * order, one rounding: bit-identical on all ranks, and identical to amp_exl3_gemv followed by
 * amp_comm_allreduce_fp16), so the exchange overlaps the rest of the decode and costs no launch.
 * bufs / ctls, rank, N, cap: exactly as for amp_comm_allreduce_fp16, whose buffers, layout and
 * sequence protocol it shares (calls of both kinds may be mixed; all ranks must issue the same
 * sequence). Waits on peers are bounded (amp_comm_status).
 * Replaces the pair exl3_gemm + comm.allreduce after o_proj / down_proj,
 * src/ucode/ampstein/qwen35_tp.uc:356,368; the reference has no fused form.
 */
int amp_exl3_gemv_allreduce(const void* x, const void* trellis, void* out, const void* suh, const void* svh,
                            int m, int k, int n, int K, int cb, void* const* bufs, int* const* ctls,
                            int rank, int N, long cap, cudaStream_t stream);
/* The same with an optional scratch for the rotated input ((m, k) fp16 or NULL), used from five rows
 * on exactly as amp_exl3_gemm uses A_had. */
int amp_exl3_gemv_allreduce_rot(const void* x, const void* trellis, void* out, const void* suh, const void* svh,
                                int m, int k, int n, int K, int cb, void* const* bufs, int* const* ctls,
                                int rank, int N, long cap, void* x_rot, cudaStream_t stream);
/*
 * The same exchange split between producer and consumer, so that no kernel waits for a peer
 * while its own rank could move on: amp_exl3_gemv_push is the row-parallel linear whose finished
 * 128-column blocks are pushed as fp16 partials into EVERY rank's buffer (its own included) and
 * which writes no output tensor; the launch that consumes the all-reduced hidden state
 * (amp_exl3_gemv_gathered, or amp_exl3_mgemm_gathered for a q|k|v or gate|up bundle) has no x
 * argument: it adds the ranks' partials up (fp32, rank order, one rounding: the bits
 * amp_comm_allreduce_fp16 would give) while it rotates its input, with its weight stream already
 * in flight. buf / ctl of the gathered forms are THIS rank's buffer and control block; the
 * payload is (m, k) of the consumer = (m, n) of the producer, m * k <= cap. A push must be
 * followed by exactly one gathering launch on every rank before the next call on the
 * communicator. Waits are bounded (amp_comm_status). The reference has no counterpart: its
 * all-reduce is a kernel of its own between the two (src/ucode/ampstein/qwen35_tp.uc:356,368).
 */
int amp_exl3_gemv_push(const void* x, const void* trellis, const void* suh, const void* svh,
                       int m, int k, int n, int K, int cb, void* const* bufs, int* const* ctls,
                       int rank, int N, long cap, cudaStream_t stream);
int amp_exl3_gemv_gathered(const void* trellis, void* c, const void* suh, const void* svh,
                           int m, int k, int n, int K, int cb, int c_fp32,
                           const void* buf, int* ctl, int N, long cap, cudaStream_t stream);
int amp_exl3_mgemm_gathered(const void* trellis_ptrs, void* C, const void* suh_ptrs, const void* svh_ptrs,
                            int num, int m, int k, int width, int K, int cb, int c_fp32,
                            const void* c_ptrs, const void* n_stride_list, const void* had_src_list,
                            const void* buf, int* ctl, int N, long cap, cudaStream_t stream);
long amp_comm_buffer_bytes(int N, long cap);
long amp_comm_ctl_bytes(void);
int amp_comm_blocks(int N, long n);

/* Reads and clears the status word of a LOCAL control block (non-zero: a wait for a peer ran
 * out). Synchronises; diagnostics only. The reference has no counterpart (its kernel traps,
 * src/torch/amp_kernels.cu:2835-2839). */
int amp_comm_status(int* ctl, int* out);

/* Set-up helpers for communicator construction (allocate; never on the hot path). The
 * reference builds its communicator inside one process (torch_p2p_comm,
 * src/torch/amp_torch.cpp:7606-7708); these cover both that case (enable_peer) and one process
 * per GPU (CUDA IPC: alloc exports a 64-byte handle, open maps a peer's). */
int amp_comm_enable_peer(int peer);
int amp_comm_ipc_alloc(long bytes, void** ptr, void* handle64);
int amp_comm_ipc_open(const void* handle64, void** ptr);
int amp_comm_ipc_close(void* ptr);
int amp_comm_free(void* ptr);

#ifdef __cplusplus
}
#endif

#endif /* AMPSTEIN_B200_H */
