// Host-side launch descriptor of the decode GEMV kernel, shared by the dense / bundle entry points
// (exl3_gemv.cu) and the grouped-expert entry point (exl3_moe.cu).
#pragma once
#include "exl3_gemv_kernel.cuh"

namespace amp {

struct GemvLaunch
{
    const void* x; const void* trellis; const void* suh; const void* svh; void* c;
    const long long* t_trellis; const long long* t_suh; const long long* t_svh; const long long* t_c;
    const int* t_stride; const int* t_src;
    int tables, slices, width, stride, m, k, K, cb, c_fp32;
    int force_split, force_xgroups;
    int mode;            // 0 dense / bundle, 1 grouped gate+up, 2 grouped down
    int max_slices;      // grouped modes: most slices the run table can describe (slices = the expected count)
    GemvMoe moe;
    int* ws_counters;    // caller-provided arrival counters / partial-sum slots instead of the
    float* ws_scratch;   // per-device workspace (both or neither); ws_max_ctas bounds the CTA count
    int ws_max_ctas;
    GemvAr ar;           // fused tensor-parallel all-reduce of the output (ar.N == 0: none)
    GemvArIn arin;       // the input is gathered from the communicator's buffer (arin.N == 0: plain x)
    const void* x2;      // non-null: the input is silu(x) * x2 (x = gate, x2 = up), formed in the kernel's prologue;
                         // with norm_w: the residual contribution, input = RMSNorm(x + x2) * norm_w
    const void* norm_w;  // RMSNorm weight (k) fp16
    void* y;             // (m, k) fp16: receives fp16(x + x2), the updated residual stream (must not alias x)
    float eps;
    // split norm. Producer (h_in, y, ssq set; norm_w null): y = fp16(h_in + output), ssq (m, n / 128) block
    // sums of squares. Consumer (ssq and norm_w set, x2 null): input = fp16(x * rsqrt(sum ssq / k + eps)) * norm_w
    const void* h_in; float* ssq;
    // with norm_w, one row, fp16 output: argmax over the output + decode-state advance (all or none)
    void* am_ws;         // >= 16 bytes, 8-byte aligned, zero before the first launch (key + block counter)
    void* am_ids; void* am_pos; void* am_log; long long am_log_cap;
    int am_vocab;
    void* x_rot;         // optional scratch, (sources, m, k) fp16: with five rows or more the input is rotated
    int num_src;         // once by a launch of its own instead of by every CTA (sources: 1, or the bundle's)
};

int launch_gemv(const GemvLaunch& A, cudaStream_t stream);

// Device pointer tables of a bundle for the prefill GEMM (one entry per slice, as exl3_mgemm takes them)
struct TcTables
{
    int num;
    const long long* trellis; const long long* svh;
    const long long* c;          // may be null: outputs stacked (num, M, width)
    const int* stride;           // may be null: row width = slice width
    const int* src;              // may be null: rotated input i belongs to slice i
};

// rotated inputs -> outputs on the tensor cores (m > 16); T: bundle form
int launch_gemm_tc(const void* xh, const void* trellis, void* c, const void* svh, int M, int k, int n,
                   int K, int cb, int c_fp32, cudaStream_t stream, const TcTables* T = nullptr);
// (M, k) fp16 / bf16 -> rotated, k-step-major, swizzled x~; pre_table: `sources` device pointers to
// the scale vectors, one x~ of M * k halves per source written back to back
int launch_had_tiled(const void* in, void* out, const void* pre, long M, int k, int bf16, cudaStream_t stream,
                     const long long* pre_table = nullptr, int sources = 1);

// Tile table of the expert-grouped prefill GEMM (device arrays written by moe_sorted_prep_kernel)
struct TcGroups
{
    const int* ntiles; const int* tile_e; const int* tile_row0; const int* tile_rows;
    int experts;         // entries per projection in the pointer tables
    int max_tiles;       // grid height: an upper bound of *ntiles
    int sub;             // 128-row sub-tiles per tile (1..4)
    int kinds;           // projections in one launch (gate and up: 2)
    const unsigned char* bits[2];   // per projection: device table of per-expert bit widths, or null (uniform)
};
int launch_gemm_tc_grouped(const void* xt, void* c, long Mcap, int k, int n, int K, int cb, int c_fp32,
                           const long long* t_trellis, const long long* t_svh, const TcGroups& G, cudaStream_t stream);

// decode kernel of the half-integer bitrates (exl3_gemv_half.cu); xt = the rotated input, (m, k) fp16
int launch_gemv_half(const void* xt, const void* trellis, const void* svh, void* c, int m, int k, int n, int KA, int c_fp32,
                     int* counters, float* scratch, size_t scratch_bytes, int max_blocks, int sms, cudaStream_t stream);

extern int g_pdl;

}  // namespace amp
