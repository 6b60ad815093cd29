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
};

int launch_gemv(const GemvLaunch& A, cudaStream_t stream);

extern int g_pdl;

}  // namespace amp
