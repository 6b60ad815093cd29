// Host side of the trellis-decode GEMV: argument checks, split / stage selection, cluster launch.
// C-ABI entry points amp_exl3_gemv and amp_exl3_gemm (the launcher the reference's exl3_gemm,
// vendor/exl3/exllamav3_ext/quant/exl3_gemm.cu:114-349, maps onto).
#include "exl3_gemv_kernel.cuh"
#include "exl3_gemv_tc.cuh"
#include "host_common.h"
#include "exl3_gemv_host.h"
#include <cstdlib>
#include <mutex>

namespace amp {

__device__ int g_gemv_status;     // non-zero after a bounded wait inside the kernel ran out

struct DevInfo { int sms = 0; int smem_optin = 0; bool ok = false; };

static DevInfo& dev_info(int dev)
{
    static DevInfo info[64];
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    DevInfo& d = info[dev & 63];
    if (!d.ok)
    {
        cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        d.ok = true;
    }
    return d;
}

static gemv_fn gemv_kernel_for(int K, int cb, int MB, int mode, int gin)
{
    switch (K)
    {
        case 1: return gemv_kernel_k1(cb, MB, mode, gin);
        case 2: return gemv_kernel_k2(cb, MB, mode, gin);
        case 3: return gemv_kernel_k3(cb, MB, mode, gin);
        case 4: return gemv_kernel_k4(cb, MB, mode, gin);
        case 5: return gemv_kernel_k5(cb, MB, mode, gin);
        case 6: return gemv_kernel_k6(cb, MB, mode, gin);
        case 7: return gemv_kernel_k7(cb, MB, mode, gin);
        case 8: return gemv_kernel_k8(cb, MB, mode, gin);
    }
    return nullptr;
}

static gemv_fn gemv_tc_kernel_for(int K, int cb, int ar)
{
    switch (K)
    {
        case 1: return gemv_tc_kernel_k1(cb, ar);
        case 2: return gemv_tc_kernel_k2(cb, ar);
        case 3: return gemv_tc_kernel_k3(cb, ar);
        case 4: return gemv_tc_kernel_k4(cb, ar);
        case 5: return gemv_tc_kernel_k5(cb, ar);
        case 6: return gemv_tc_kernel_k6(cb, ar);
        case 7: return gemv_tc_kernel_k7(cb, ar);
        case 8: return gemv_tc_kernel_k8(cb, ar);
    }
    return nullptr;
}

// Workspace of the decode kernels: arrival counters and partial-sum slots for column blocks whose
// rows are shared between CTAs. One region per (device, stream), allocated on the first launch on
// that stream (like the reference's DevCtx lock buffer,
// vendor/exl3/exllamav3_ext/quant/exl3_devctx.cu:81-94), so the first call on a stream must come
// before any capture on it. Launches on one stream never use their region at the same time (a
// launch touches it only after its predecessor has completed), and launches that overlap on the
// GPU run on different streams (a side stream for the shared expert, parallel graph branches), so
// they never share counters. Beyond GEMV_MAX_STREAMS streams per device regions are shared again.
constexpr int GEMV_MAX_STREAMS = 16;
constexpr int GEMV_MAX_BLOCKS = 16384;                       // column blocks per launch
constexpr int GEMV_MAX_CTAS = 1024;
constexpr size_t GEMV_COUNTER_BYTES = GEMV_MAX_BLOCKS * sizeof(int);
constexpr size_t GEMV_SCRATCH_BYTES = (size_t) GEMV_MAX_CTAS * 2 * 16 * 128 * sizeof(float);
constexpr size_t GEMV_REGION_BYTES = GEMV_COUNTER_BYTES + GEMV_SCRATCH_BYTES;

struct Workspace { cudaStream_t stream[GEMV_MAX_STREAMS]; unsigned char* base[GEMV_MAX_STREAMS]; int n = 0; };

static int workspace_region(int dev, cudaStream_t stream, int** counters, float** scratch)
{
    static Workspace ws[64];
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    Workspace& W = ws[dev & 63];
    int idx = -1;
    for (int i = 0; i < W.n; ++i)
        if (W.stream[i] == stream) { idx = i; break; }
    if (idx < 0 && W.n == GEMV_MAX_STREAMS) idx = (int) (((uintptr_t) stream >> 4) % GEMV_MAX_STREAMS);
    if (idx < 0 && W.n > 0)
    {
        // a stream that is being captured cannot allocate: it borrows the first region (its launches
        // then share counters with that stream's; warm the stream up before capture to avoid it)
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone) idx = 0;
    }
    if (idx < 0)
    {
        void* p = nullptr;
        if (cudaError_t e = cudaMalloc(&p, GEMV_REGION_BYTES)) return cuda_rc(e, "exl3_gemv workspace");
        if (cudaError_t e = cudaMemset(p, 0, GEMV_COUNTER_BYTES)) return cuda_rc(e, "exl3_gemv workspace clear");
        if (cudaError_t e = cudaDeviceSynchronize()) return cuda_rc(e, "exl3_gemv workspace sync");
        idx = W.n++;
        W.stream[idx] = stream;
        W.base[idx] = (unsigned char*) p;
    }
    unsigned char* r = W.base[idx];
    *counters = (int*) r;
    *scratch = (float*) (r + GEMV_COUNTER_BYTES);
    return 0;
}

// Programmatic dependent launch, on by default. It only pays together with the shared-memory
// padding in launch_gemv: when an SM could take one CTA more than the grid plans for, the
// dependent grid piles up on the SMs that drain first and the chain runs 10 % slower than
// without dependent launch; with the padding it runs 3 % faster (B200, inside CUDA graphs).
int g_pdl = 1;
int g_cluster = 1;        // cluster form of the partial-sum exchange
// 1: dense / bundle launches of up to eight rows run on the tensor-memory kernel
// (exl3_gemv_tc.cuh) instead of the mma.sync kernel. Off by default: measured slower on B200 (its
// hand-over of decoded weights to the tensor core costs more instructions than the eight issue
// cycles per mma.sync it saves); kept for A/B runs (amp_exl3_set_gemv_tc).
int g_gemv_tc = 0;
// (with more than 16 units per CTA the grid of 8 x blocks CTAs is too coarse: measured slower)
constexpr int GEMV_CLUSTER = 8, GEMV_CLUSTER_MAX_M = 4, GEMV_CLUSTER_MAX_UNITS = 16;

// x~ = fp16(H(x * suh) / sqrt(128)) of every source, (sources, m, k) fp16 row-major: one warp per
// 128 values, the arithmetic of the GEMV kernel's own prologue (fp16 scale, fp32 butterfly, one
// rounding). Runs right before a GEMV of five or more rows, which then only copies x~ into
// fragment order instead of rotating all rows of its range in every CTA.
__global__ __launch_bounds__(256)
void gemv_prerotate_kernel(const __half* __restrict__ x, __half* __restrict__ out, const __half* __restrict__ suh,
                           const long long* __restrict__ t_suh, int m, int k, int pdl)
{
    // the GEMV behind this launch may start its weight stream now; it waits for this grid before it
    // reads x~, and this grid waits for the producer of x
    if (pdl) pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int per_row = k >> 7;
    const int task = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (task >= m * per_row) return;
    const int b = task / per_row, jb = task - b * per_row;
    if (t_suh) suh = reinterpret_cast<const __half*>(t_suh[blockIdx.y]);
    const half4 sc = *reinterpret_cast<const half4*>(suh + (size_t) jb * 128 + lane * 4);
    if (pdl) pdl_wait();
    half4 v = *reinterpret_cast<const half4*>(x + (size_t) b * k + (size_t) jb * 128 + lane * 4);
    v.x = __hmul2(v.x, sc.x);
    v.y = __hmul2(v.y, sc.y);
    float h0 = __low2float(v.x), h1 = __high2float(v.x), h2 = __low2float(v.y), h3 = __high2float(v.y);
    warp_had128(h0, h1, h2, h3, lane);
    half4 o;
    o.x = __floats2half2_rn(h0 * kRScale, h1 * kRScale);
    o.y = __floats2half2_rn(h2 * kRScale, h3 * kRScale);
    *reinterpret_cast<half4*>(out + ((size_t) blockIdx.y * m + b) * k + (size_t) jb * 128 + lane * 4) = o;
}

constexpr int GEMV_PREROTATE_MIN_M = 5;

// Int8-activation form of the one-row GEMV for mul1 (codebook 2) tensors, as the reference's
// EXL3_INT8_GEMV switch (vendor/exl3/exllamav3_ext/quant/exl3_gemv_int8.cu:20-52): 0 = off, 2 = plain
// int8 (the reference's default), 1 = int8 with the error-feedback pass. The environment variables
// are read once.
static int int8_env(const char* name, int fallback)
{
    const char* e = getenv(name);
    return e ? atoi(e) : fallback;
}
int g_int8_gemv = int8_env("EXL3_INT8_GEMV", 2);
int g_int8_max_k = int8_env("EXL3_INT8_GEMV_MAX_K", 6);

int launch_gemv(const GemvLaunch& A, cudaStream_t stream)
{
    const int m = A.m, k = A.k, K = A.K;
    AMP_REQUIRE(K >= 1 && K <= 8, "exl3_gemv: unsupported EXL3 bitrate %d (integer 1..8)", K);
    AMP_REQUIRE(A.cb >= 0 && A.cb <= 2, "exl3_gemv: codebook index %d out of range", A.cb);
    AMP_REQUIRE(m >= 1 && m <= 16, "exl3_gemv: m must be 1..16 (got %d)", m);
    AMP_REQUIRE(k > 0 && A.width > 0 && k % 128 == 0 && A.width % 128 == 0 && A.stride % 128 == 0,
                "exl3_gemv: k and n must be multiples of 128");
    AMP_REQUIRE(A.slices >= 1 && (long) A.slices * (A.width / 128) <= 0x7fffffffL, "exl3_gemv: bad slice count");
    AMP_REQUIRE(A.mode || A.arin.N || (A.x && ((uintptr_t) A.x & 7) == 0), "exl3_gemv: x must be a non-null 8-byte aligned pointer");
    if (A.mode)
    {
        AMP_REQUIRE(A.moe.runs && A.max_slices >= 1, "exl3_moe: run table missing");
    }
    else if (A.tables)
    {
        AMP_REQUIRE(A.t_trellis && A.t_suh && A.t_svh, "exl3_mgemm: pointer tables are required");
        AMP_REQUIRE(A.t_c || A.c, "exl3_mgemm: no output");
    }
    else
    {
        AMP_REQUIRE(A.trellis && A.c && A.suh && A.svh, "exl3_gemv: null pointer (suh and svh are required)");
        AMP_REQUIRE(((uintptr_t) A.trellis & 15) == 0, "exl3_gemv: trellis must be 16-byte aligned");
        AMP_REQUIRE(((uintptr_t) A.suh & 7) == 0 && ((uintptr_t) A.svh & 7) == 0, "exl3_gemv: suh, svh must be 8-byte aligned");
        AMP_REQUIRE(((uintptr_t) A.c & (A.c_fp32 ? 15 : 7)) == 0, "exl3_gemv: output misaligned");
    }

    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev)) return cuda_rc(e, "cudaGetDevice");
    const DevInfo& D = dev_info(dev);

    const int MB = m <= 8 ? 1 : 2;
    const bool tc = !A.mode && m <= TCV_MAX_M && g_gemv_tc && !A.arin.N && !A.ar.push_only && !A.x2 && !A.h_in && !A.norm_w;
    // five rows or more with a scratch for the rotated input: rotate once, in a launch of its own
    const bool norm_producer = A.h_in != nullptr;                       // split norm, producer side
    const bool norm_consumer = A.norm_w != nullptr && A.ssq != nullptr && !A.x2;   // ... consumer side
    AMP_REQUIRE(!norm_producer || (!A.mode && !A.arin.N && !A.ar.N && !A.tables && !A.c_fp32 && A.y && A.ssq && !A.norm_w && !A.x2 &&
                                   (((uintptr_t) A.h_in | (uintptr_t) A.y) & 7) == 0),
                "exl3_gemv: the residual-adding form takes a plain launch with fp16 output, h, y and ssq");
    AMP_REQUIRE(!norm_consumer || (!A.mode && !A.arin.N && A.x && ((uintptr_t) A.norm_w & 7) == 0),
                "exl3_gemv: the scaled-norm form takes a plain or bundle launch with x, ssq and norm_w");
    const bool fused_norm = A.norm_w != nullptr && !norm_consumer;
    const bool fused_act = A.x2 != nullptr && !fused_norm;
    AMP_REQUIRE(!fused_act || (!A.mode && !A.arin.N && !A.tables && ((uintptr_t) A.x2 & 7) == 0),
                "exl3_gemv: the fused activation takes two plain 8-byte aligned inputs");
    AMP_REQUIRE(!fused_norm || (!A.mode && !A.arin.N && A.x && A.x2 && A.y && A.y != A.x && A.y != A.x2 &&
                                (((uintptr_t) A.x2 | (uintptr_t) A.norm_w | (uintptr_t) A.y) & 7) == 0),
                "exl3_gemv: the fused norm takes x, residual, weight and a separate output for the residual stream, 8-byte aligned");
    const bool special_in = fused_act || fused_norm || norm_producer || norm_consumer;
    const bool prerot = !tc && !A.mode && !A.arin.N && !special_in && m >= GEMV_PREROTATE_MIN_M && A.x_rot && A.x;
    // mul1, one row: int8 activations (kernel instance 3), or int8 with error-feedback codes (instance 4)
    const int i8 = (!tc && !A.mode && !A.arin.N && !special_in && A.cb == 2 && m == 1 && K <= g_int8_max_k)
                       ? (g_int8_gemv == 2 ? 3 : (g_int8_gemv == 1 ? 4 : 0)) : 0;
    gemv_fn fn = tc ? gemv_tc_kernel_for(K, A.cb, A.ar.N != 0)
                    : gemv_kernel_for(K, i8 ? i8 : A.cb, MB, A.mode, A.arin.N ? 1 : (norm_producer ? 5 : (norm_consumer ? 6 : (fused_norm ? 4 : (fused_act ? 3 : (prerot ? 2 : 0))))));
    if (!fn) return fail(AMP_E_UNSUPPORTED, "exl3_gemv: no kernel for K=%d cb=%d", K, A.cb);

    // x~ rows resident at a time: at most 16 KB of shared memory (whole segments for small
    // batches, so the main loop rarely meets a block-wide barrier); shrunk below to what a
    // CTA's range needs
    const int G = k / 64;
    const int smem_per_sm = D.smem_optin + 1024;                       // opt-in limit excludes 1 KB per CTA
    const int reg_ctas = tc ? 4 : (m <= 8 ? 3 : 4);                    // CTAs per SM the register budget allows
    auto xcap_for = [&](int kb)
    {
        int c = (kb * 1024 / (m * 4)) / 64;
        c &= ~3;
        if (c > GEMV_XCHUNK_MAX / 64) c = GEMV_XCHUNK_MAX / 64;
        if (c > (G + 3) / 4 * 4) c = (G + 3) / 4 * 4;
        return c < 4 ? 4 : c;
    };
    int xcap = xcap_for(16);
    if (m > 4 && !A.mode)
    {
        // several batch rows: twice the x~ budget (half as many block-wide x~ passes per range)
        // where that does not cost a resident CTA (not for the grouped modes: their runs mostly hold
        // one or two rows, and the single-token form also needs room for the cluster exchange)
        const int big = xcap_for(32);
        if (smem_per_sm / (gemv_smem_layout(K, m, big).total + 1024) >= reg_ctas) xcap = big;
    }
    if (A.force_xgroups > 0)
    {
        AMP_REQUIRE(A.force_xgroups % 4 == 0 && A.force_xgroups <= GEMV_XCHUNK_MAX / 64,
                    "exl3_gemv: xgroups must be a multiple of 4, at most %d", GEMV_XCHUNK_MAX / 64);
        xcap = A.force_xgroups;
    }
    // tensor-memory kernel: x~ in chunks of four 64-row groups (two 128-row transforms), two buffers
    const int tc_xg = G < 4 ? G : 4;
    GemvSmem L = gemv_smem_layout(K, m, xcap, 0, 0, i8 == 4 ? gemv_xpitch(xcap) * 4 : 0);     // (instance 4: a second x~ area for the error codes)
    if (tc) L.total = tcv_smem_layout(K, m, tc_xg).total;
    AMP_REQUIRE(L.total <= D.smem_optin, "exl3_gemv: shared memory layout does not fit (%d bytes)", L.total);
    // CTAs per SM: the decode is bound by the rate of the integer pipes, not by latency, so
    // three 4-warp CTAs per SM run as fast as six (measured) and halve the partial sums that
    // have to be exchanged
    // (the tensor-memory kernel: four CTAs of 128 tensor-memory columns fill an SM's 512)
    int ctas_per_sm = smem_per_sm / (L.total + 1024);
    if (ctas_per_sm > reg_ctas) ctas_per_sm = reg_ctas;
    if (ctas_per_sm < 1) ctas_per_sm = 1;

    // one contiguous range of (column block, 64-row group) units per CTA; as many CTAs as the
    // device holds at once, fewer when that would leave a CTA with less than four units
    const long col_blocks = (long) (A.mode ? A.max_slices : A.slices) * (A.width / 128);
    AMP_REQUIRE(col_blocks <= GEMV_MAX_BLOCKS, "exl3_gemv: too many column blocks (%ld)", col_blocks);
    const long units = col_blocks * (k / 64);
    AMP_REQUIRE(units < (1L << 30), "exl3_gemv: problem too large (%ld work units)", units);
    long ncta = (long) D.sms * ctas_per_sm;
    if (A.mode)
    {
        // the run count is only known on the device: size the grid for the expected load
        const long expect = (long) A.slices * (A.width / 128) * G;
        while (ncta > D.sms && expect / ncta < 8) ncta -= D.sms;
    }
    else if (units / ncta < 16)
    {
        // small problem: give every column block the same whole number of CTAs, so that a CTA
        // works on one block only (one partial-sum exchange per CTA instead of two or three)
        long S = ncta / col_blocks;
        while (S > 1 && G / S < 4) --S;
        if (S >= 1) ncta = col_blocks * S;
        else { ncta = (long) D.sms * ctas_per_sm; while (ncta > D.sms && units / ncta < 4) ncta -= D.sms; }
    }
    // Layer-sized single matrices at small batch: one cluster of eight CTAs per column block. The
    // partial sums then travel through distributed shared memory and a cluster barrier (about a
    // microsecond) instead of global memory, a fence, an atomic and a read-back (about three).
    int cluster = 0;
    if (!A.mode && !A.ws_counters && A.force_split == 0 && A.force_xgroups == 0 && m <= GEMV_CLUSTER_MAX_M && G % GEMV_CLUSTER == 0 &&
        G / GEMV_CLUSTER >= 2 && G / GEMV_CLUSTER <= GEMV_CLUSTER_MAX_UNITS && col_blocks * GEMV_CLUSTER <= (long) D.sms * ctas_per_sm && g_cluster)
    {
        cluster = GEMV_CLUSTER;
        ncta = col_blocks * GEMV_CLUSTER;
    }
    // Grouped launch for one token: the picks are known to be at most max_slices one-row runs, so
    // the same form applies with the largest cluster that divides the row groups and fits the device
    if (A.mode && A.moe.inline_runs && g_cluster)
        for (int c = GEMV_CLUSTER; c >= 2 && !cluster; --c)
            if (G % c == 0 && G / c >= 2 && col_blocks * c <= (long) D.sms * ctas_per_sm)
            {
                cluster = c;
                ncta = col_blocks * c;
            }
    if (A.force_split > 0) ncta = A.force_split;
    if (ncta > units) ncta = units;
    if (ncta > GEMV_MAX_CTAS) ncta = GEMV_MAX_CTAS;
    if (A.ws_counters && ncta > A.ws_max_ctas) ncta = A.ws_max_ctas;
    AMP_REQUIRE(ncta >= 1, "exl3_gemv: empty problem");

    // a range of `per` units starting anywhere needs per + 1 groups of x~ (chunks start at an
    // even group); the grouped modes learn their unit count on the device and keep the cap
    int xgroups = xcap;
    if (!A.mode && A.force_xgroups <= 0)
    {
        const long per = (units + ncta - 1) / ncta;
        const long need = (per + 1 + 3) / 4 * 4;
        if (need < xgroups) xgroups = (int) need;
    }
    // fused norm, one row that fits: y and the norm weight of the row stay in shared memory (4 k bytes),
    // as long as that keeps the planned number of CTAs on an SM
    int rowbuf = 0;
    if (fused_norm && m == 1 && !tc && ((uintptr_t) A.norm_w & 15) == 0)
    {
        const int want = 4 * k;
        if (smem_per_sm / (gemv_smem_layout(K, m, xgroups, cluster, 0, want).total + 1024) >= ctas_per_sm) rowbuf = want;
    }
    if (i8 == 4) rowbuf = gemv_xpitch(xgroups) * 4;
    L = gemv_smem_layout(K, m, xgroups, cluster, A.arin.N != 0, rowbuf);
    if (tc)
    {
        xgroups = tc_xg;
        L.total = tcv_smem_layout(K, m, tc_xg, cluster).total;
    }
    // Ask for enough shared memory that exactly ctas_per_sm CTAs fit on an SM. The grid is sized
    // for that many; if an SM could take one more, a dependent grid that starts while this one
    // drains would pile four CTAs on the SMs that free up first and leave others with two.
    int smem_bytes = L.total;
    {
        const int fit_one_more = smem_per_sm / (ctas_per_sm + 1) - 1024;      // largest size of which ctas_per_sm + 1 fit
        if (smem_bytes <= fit_one_more) smem_bytes = fit_one_more + 16;
        if (smem_bytes > D.smem_optin) smem_bytes = D.smem_optin;
    }
    if (cudaError_t e = ensure_smem(fn, smem_bytes, dev)) return cuda_rc(e, "exl3_gemv smem attribute");

    GemvParams P;
    P.x = (const __half*) A.x; P.trellis = (const uint16_t*) A.trellis;
    P.suh = (const __half*) A.suh; P.svh = (const __half*) A.svh; P.c = A.c;
    P.t_trellis = A.t_trellis; P.t_suh = A.t_suh; P.t_svh = A.t_svh; P.t_c = A.t_c;
    P.t_stride = A.t_stride; P.t_src = A.t_src;
    P.tables = A.tables; P.width = A.width; P.stride = A.stride;
    P.m = m; P.k = k; P.c_fp32 = A.c_fp32; P.xgroups = xgroups; P.pdl = g_pdl; P.cluster = cluster;
    P.blocks = (int) col_blocks;
    P.moe = A.moe;
    P.ar = A.ar;
    P.arin = A.arin;
    P.x2 = (const __half*) A.x2;
    P.norm_w = (const __half*) A.norm_w; P.y = (__half*) A.y; P.eps = A.eps; P.rowbuf = rowbuf;
    P.h_in = (const __half*) A.h_in; P.ssq = A.ssq;
    P.am_key = nullptr; P.am_count = nullptr; P.am_ids = P.am_pos = P.am_log = nullptr; P.am_log_cap = 0; P.am_vocab = 0;
    if (A.am_ws)
    {
        AMP_REQUIRE(fused_norm && m == 1 && !A.c_fp32 && !A.tables && !A.ar.N, "exl3_gemv: the fused argmax needs the norm form, one row and fp16 logits");
        AMP_REQUIRE(A.am_ids && A.am_pos && A.am_log && ((uintptr_t) A.am_ws & 7) == 0, "exl3_gemv: argmax state pointers missing or misaligned");
        AMP_REQUIRE(A.am_vocab >= 1 && A.am_vocab <= A.width, "exl3_gemv: vocabulary size out of range");
        P.am_key = (unsigned long long*) A.am_ws; P.am_count = (unsigned int*) ((char*) A.am_ws + 8);
        P.am_ids = (long long*) A.am_ids; P.am_pos = (long long*) A.am_pos; P.am_log = (long long*) A.am_log;
        P.am_log_cap = A.am_log_cap; P.am_vocab = A.am_vocab;
    }
    if (A.ws_counters) { P.counters = A.ws_counters; P.scratch = A.ws_scratch; }
    else if (int rc = workspace_region(dev, stream, &P.counters, &P.scratch)) return rc;
    {
        // address of the status word, looked up once per device (under a lock: two host threads
        // may make their first launch on a device at the same time)
        static int* status_ptr[64] = {};
        static std::mutex status_mu;
        std::lock_guard<std::mutex> lock(status_mu);
        int*& sp = status_ptr[dev & 63];
        if (!sp)
            if (cudaError_t e = cudaGetSymbolAddress((void**) &sp, g_gemv_status)) return cuda_rc(e, "status symbol");
        P.status = sp;
    }

    if (prerot)
    {
        const int sources = A.tables ? (A.num_src > 0 ? A.num_src : A.slices) : 1;
        AMP_REQUIRE(sources >= 1 && sources <= 65535, "exl3_gemv: source count out of range");
        AMP_REQUIRE(((uintptr_t) A.x_rot & 7) == 0, "exl3_gemv: A_had must be 8-byte aligned");
        cudaLaunchConfig_t pc = {};
        pc.gridDim = dim3((unsigned) (((long) m * (k / 128) + 7) / 8), (unsigned) sources, 1);
        pc.blockDim = dim3(256, 1, 1);
        pc.stream = stream;
        cudaLaunchAttribute pa[1];
        pa[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        pa[0].val.programmaticStreamSerializationAllowed = 1;
        pc.attrs = pa;
        pc.numAttrs = g_pdl ? 1 : 0;
        if (cudaError_t e = cudaLaunchKernelEx(&pc, gemv_prerotate_kernel, (const __half*) A.x, (__half*) A.x_rot, (const __half*) A.suh,
                                               A.tables ? A.t_suh : (const long long*) nullptr, m, k, g_pdl))
            return cuda_rc(e, "exl3_gemv input rotation launch");
        P.x = (const __half*) A.x_rot;
    }

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned) ncta, 1, 1);
    cfg.blockDim = dim3(tc ? TCV_THREADS : GEMV_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int nattr = 0;
    if (g_pdl)
    {
        attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[nattr].val.programmaticStreamSerializationAllowed = 1;
        ++nattr;
    }
    if (cluster)
    {
        attr[nattr].id = cudaLaunchAttributeClusterDimension;
        attr[nattr].val.clusterDim.x = cluster; attr[nattr].val.clusterDim.y = 1; attr[nattr].val.clusterDim.z = 1;
        ++nattr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = nattr;
    return cuda_rc(cudaLaunchKernelEx(&cfg, fn, P), "exl3_gemv launch");
}

static GemvLaunch direct(const void* x, const void* trellis, void* c, const void* suh, const void* svh,
                         int m, int k, int n, int K, int cb, int c_fp32, int split, int xgroups)
{
    GemvLaunch A = {};
    A.x = x; A.trellis = trellis; A.suh = suh; A.svh = svh; A.c = c;
    A.tables = 0; A.slices = 1; A.width = n; A.stride = n;
    A.m = m; A.k = k; A.K = K; A.cb = cb; A.c_fp32 = c_fp32;
    A.force_split = split; A.force_xgroups = xgroups;
    return A;
}

}  // namespace amp

using namespace amp;

AMP_API int amp_exl3_gemv(const void* x, const void* trellis, void* c, const void* suh, const void* svh,
                          int m, int k, int n, int K, int cb, int c_fp32, cudaStream_t stream)
{
    return launch_gemv(direct(x, trellis, c, suh, svh, m, k, n, K, cb, c_fp32, 0, 0), stream);
}

// 0 = the mul1 one-row GEMV runs the fp16 kernel, 2 = int8 activations, 1 = int8 activations with an
// error-feedback pass (the rounding error of the codes quantised again and accumulated by a second
// dp4a: ~15 bits of effective activation precision) -- the reference's EXL3_INT8_GEMV modes.
// max_k > 0 also sets the highest bit width that takes the int8 forms (EXL3_INT8_GEMV_MAX_K).
// Returns the previous mode.
AMP_API int amp_exl3_set_int8_gemv(int mode, int max_k)
{
    const int old = g_int8_gemv;
    g_int8_gemv = (mode == 1 || mode == 2) ? mode : 0;
    if (max_k > 0) g_int8_max_k = max_k > 8 ? 8 : max_k;
    return old;
}

// Down projection with the gated activation in its prologue: c (m, n) = linear(silu(gate) * up),
// gate / up (m, k) fp16. One launch instead of silu_mul followed by exl3_gemm; the activation is
// formed in fp32 and rounded to fp16 exactly as the stand-alone kernel does it, so the result is
// that of the two-step sequence. m <= 16.
AMP_API int amp_exl3_gemv_silu_mul(const void* gate, const void* up, const void* trellis, void* c, const void* suh, const void* svh,
                                   int m, int k, int n, int K, int cb, int c_fp32, cudaStream_t stream)
{
    AMP_REQUIRE(gate && up, "exl3_gemv_silu_mul: null input");
    GemvLaunch A = direct(gate, trellis, c, suh, svh, m, k, n, K, cb, c_fp32, 0, 0);
    A.x2 = up;
    return launch_gemv(A, stream);
}

// Linear behind the fused residual add + RMSNorm of the decode step: y (m, k) = fp16(x + res) (the
// updated residual stream), c (m, n) = linear(fp16(y * rsqrt(mean(y^2) + eps)) * norm_w). One launch
// instead of rms_norm_res followed by exl3_gemm (the final norm in front of the lm_head). y must not
// alias x or res. m <= 16.
AMP_API int amp_exl3_gemv_rms_norm_res(const void* x, const void* res, const void* norm_w, float eps, void* y,
                                       const void* trellis, void* c, const void* suh, const void* svh,
                                       int m, int k, int n, int K, int cb, int c_fp32, cudaStream_t stream)
{
    AMP_REQUIRE(x && res && norm_w && y, "exl3_gemv_rms_norm_res: null input");
    GemvLaunch A = direct(x, trellis, c, suh, svh, m, k, n, K, cb, c_fp32, 0, 0);
    A.x2 = res; A.norm_w = norm_w; A.y = y; A.eps = eps;
    return launch_gemv(A, stream);
}

// The split form of the residual norm. Producer: y (m, n) = fp16(h + linear(x)) (the updated residual
// stream; the linear's own output is not stored) and ssq (m, n / 128) = per-block sums of squares of y.
// Consumer: c = linear(s) of fp16(y * rsqrt(sum(ssq row) / k + eps)) * norm_w. Unlike the one-launch
// form nothing reads a whole row on a CTA's critical path: the producer's finishing warps hold the
// values anyway, the consumer adds k / 128 floats. m <= 16. y may not alias h.
AMP_API int amp_exl3_gemv_add_res(const void* x, const void* trellis, const void* suh, const void* svh,
                                  const void* h, void* y, void* ssq, int m, int k, int n, int K, int cb, cudaStream_t stream)
{
    AMP_REQUIRE(h && y && ssq && h != y, "exl3_gemv_add_res: null pointer, or y aliases h");
    GemvLaunch A = direct(x, trellis, y, suh, svh, m, k, n, K, cb, 0, 0, 0);
    A.h_in = h; A.y = y; A.ssq = (float*) ssq;
    return launch_gemv(A, stream);
}

AMP_API int amp_exl3_gemv_normed(const void* y, const void* ssq, const void* norm_w, float eps,
                                 const void* trellis, void* c, const void* suh, const void* svh,
                                 int m, int k, int n, int K, int cb, int c_fp32, cudaStream_t stream)
{
    AMP_REQUIRE(y && ssq && norm_w, "exl3_gemv_normed: null input");
    GemvLaunch A = direct(y, trellis, c, suh, svh, m, k, n, K, cb, c_fp32, 0, 0);
    A.ssq = (float*) ssq; A.norm_w = norm_w; A.eps = eps;
    return launch_gemv(A, stream);
}

AMP_API int amp_exl3_mgemm_normed(const void* y, const void* ssq, const void* norm_w, float eps,
                                  const void* trellis_ptrs, void* C, const void* suh_ptrs, const void* svh_ptrs,
                                  int num, int m, int k, int width, int K, int cb, int c_fp32,
                                  const void* c_ptrs, const void* n_stride_list, const void* had_src_list, cudaStream_t stream)
{
    if (num == 0 || m == 0) return 0;
    AMP_REQUIRE(num > 0 && m >= 1 && m <= 16, "exl3_mgemm_normed: 1..16 rows");
    AMP_REQUIRE(y && ssq && norm_w, "exl3_mgemm_normed: null input");
    GemvLaunch A = {};
    A.x = y; A.c = C;
    A.t_trellis = (const long long*) trellis_ptrs; A.t_suh = (const long long*) suh_ptrs;
    A.t_svh = (const long long*) svh_ptrs; A.t_c = (const long long*) c_ptrs;
    A.t_stride = (const int*) n_stride_list; A.t_src = (const int*) had_src_list;
    A.tables = 1; A.slices = num; A.width = width; A.stride = width;
    A.m = m; A.k = k; A.K = K; A.cb = cb; A.c_fp32 = c_fp32;
    A.ssq = (float*) ssq; A.norm_w = norm_w; A.eps = eps;
    return launch_gemv(A, stream);
}

// The last three launches of a greedy decode step in one: final residual add + RMSNorm, lm_head (one
// row, fp16 logits (1, n)), argmax over the first `vocab` logits and the state advance
// log[pos] = ids; ids = argmax; pos += 1 (log write skipped when pos is outside [0, log_cap)). Ties go
// to the lowest index, NaN logits are skipped, no valid logit gives 0. ws: 16 bytes, 8-byte aligned,
// zero before the first call; every call leaves it zero.
AMP_API int amp_exl3_lm_head_argmax(const void* x, const void* res, const void* norm_w, float eps, void* y,
                                    const void* trellis, void* logits, const void* suh, const void* svh,
                                    int k, int n, int K, int cb, int vocab,
                                    void* ids, void* pos, void* log, long long log_cap, void* ws, cudaStream_t stream)
{
    AMP_REQUIRE(x && res && norm_w && y && ws, "exl3_lm_head_argmax: null input");
    GemvLaunch A = direct(x, trellis, logits, suh, svh, 1, k, n, K, cb, 0, 0, 0);
    A.x2 = res; A.norm_w = norm_w; A.y = y; A.eps = eps;
    A.am_ws = ws; A.am_ids = ids; A.am_pos = pos; A.am_log = log; A.am_log_cap = log_cap; A.am_vocab = vocab;
    return launch_gemv(A, stream);
}

// The bundle form (amp_exl3_mgemm's tables; q|k|v or gate|up behind rms_norm_res), m <= 16
AMP_API int amp_exl3_mgemm_rms_norm_res(const void* x, const void* res, const void* norm_w, float eps, void* y,
                                        const void* trellis_ptrs, void* C, const void* suh_ptrs, const void* svh_ptrs,
                                        int num, int m, int k, int width, int K, int cb, int c_fp32,
                                        const void* c_ptrs, const void* n_stride_list, const void* had_src_list, cudaStream_t stream)
{
    if (num == 0 || m == 0) return 0;
    AMP_REQUIRE(num > 0 && m >= 1 && m <= 16, "exl3_mgemm_rms_norm_res: 1..16 rows");
    AMP_REQUIRE(x && res && norm_w && y, "exl3_mgemm_rms_norm_res: null input");
    GemvLaunch A = {};
    A.x = x; A.c = C;
    A.t_trellis = (const long long*) trellis_ptrs; A.t_suh = (const long long*) suh_ptrs;
    A.t_svh = (const long long*) svh_ptrs; A.t_c = (const long long*) c_ptrs;
    A.t_stride = (const int*) n_stride_list; A.t_src = (const int*) had_src_list;
    A.tables = 1; A.slices = num; A.width = width; A.stride = width;
    A.m = m; A.k = k; A.K = K; A.cb = cb; A.c_fp32 = c_fp32;
    A.x2 = res; A.norm_w = norm_w; A.y = y; A.eps = eps;
    return launch_gemv(A, stream);
}

// tuning / test hook: fixed CTA count (split) and x~ chunk size (xgroups); 0 = choose
AMP_API int amp_exl3_gemv_cfg(const void* x, const void* trellis, void* c, const void* suh, const void* svh,
                              int m, int k, int n, int K, int cb, int c_fp32, int split, int xgroups,
                              cudaStream_t stream)
{
    return launch_gemv(direct(x, trellis, c, suh, svh, m, k, n, K, cb, c_fp32, split, xgroups), stream);
}

// ---- row-parallel linear with the tensor-parallel all-reduce fused into its epilogue ----
// out (m, n) fp16 = sum over the N ranks of this rank's x (m, k_local) through its row shard of
// the weight. bufs / ctls: the communicator's buffers exactly as amp_comm_allreduce_fp16 takes
// them (zero-filled once, sized by amp_comm_buffer_bytes(N, cap)); m * n <= cap. All ranks must
// issue the same sequence of all-reduce and fused calls.
AMP_API int amp_exl3_gemv_allreduce(const void* x, const void* trellis, void* out, const void* suh, const void* svh,
                                    int m, int k, int n, int K, int cb, void* const* bufs, int* const* ctls,
                                    int rank, int N, long cap, cudaStream_t stream)
{
    AMP_REQUIRE(N >= 2 && N <= COMM_MAXN && rank >= 0 && rank < N, "exl3_gemv_allreduce: bad rank / world size (2..%d ranks)", COMM_MAXN);
    AMP_REQUIRE(bufs && ctls, "exl3_gemv_allreduce: null buffer table");
    AMP_REQUIRE(cap > 0 && cap % 8 == 0 && (long) m * n <= cap, "exl3_gemv_allreduce: m * n exceeds the communicator's capacity");
    GemvLaunch A = direct(x, trellis, out, suh, svh, m, k, n, K, cb, 0, 0, 0);
    for (int p = 0; p < N; ++p)
    {
        AMP_REQUIRE(bufs[p] && ctls[p], "exl3_gemv_allreduce: null buffer of rank %d", p);
        A.ar.buf[p] = (uint2*) bufs[p];
    }
    A.ar.ctl = ctls[rank];
    A.ar.rank = rank; A.ar.N = N; A.ar.wcap = cap / 2;
    return launch_gemv(A, stream);
}

// The same with a scratch for the rotated input ((m, k) fp16, nullable): from five rows on the input
// is then rotated once by a small launch of its own instead of by every CTA (as amp_exl3_gemm's A_had).
AMP_API int amp_exl3_gemv_allreduce_rot(const void* x, const void* trellis, void* out, const void* suh, const void* svh,
                                        int m, int k, int n, int K, int cb, void* const* bufs, int* const* ctls,
                                        int rank, int N, long cap, void* x_rot, cudaStream_t stream)
{
    AMP_REQUIRE(N >= 2 && N <= COMM_MAXN && rank >= 0 && rank < N, "exl3_gemv_allreduce: bad rank / world size (2..%d ranks)", COMM_MAXN);
    AMP_REQUIRE(bufs && ctls, "exl3_gemv_allreduce: null buffer table");
    AMP_REQUIRE(cap > 0 && cap % 8 == 0 && (long) m * n <= cap, "exl3_gemv_allreduce: m * n exceeds the communicator's capacity");
    GemvLaunch A = direct(x, trellis, out, suh, svh, m, k, n, K, cb, 0, 0, 0);
    for (int p = 0; p < N; ++p)
    {
        AMP_REQUIRE(bufs[p] && ctls[p], "exl3_gemv_allreduce: null buffer of rank %d", p);
        A.ar.buf[p] = (uint2*) bufs[p];
    }
    A.ar.ctl = ctls[rank];
    A.ar.rank = rank; A.ar.N = N; A.ar.wcap = cap / 2;
    A.x_rot = x_rot;
    return launch_gemv(A, stream);
}

// ---- split exchange: the producer only pushes, the consumer gathers in its x~ prologue ----
// amp_exl3_gemv_push: a row-parallel linear whose finished column blocks are pushed, as fp16
// partials, into every rank's all-reduce buffer (this rank's included); nothing waits and no output
// tensor is written. The launch that consumes the sum (amp_exl3_gemv_gathered /
// amp_exl3_mgemm_gathered) adds the ranks' partials up while it rotates its input.
AMP_API int amp_exl3_gemv_push(const void* x, const void* trellis, const void* suh, const void* svh,
                               int m, int k, int n, int K, int cb, void* const* bufs, int* const* ctls,
                               int rank, int N, long cap, cudaStream_t stream)
{
    AMP_REQUIRE(N >= 2 && N <= COMM_MAXN && rank >= 0 && rank < N, "exl3_gemv_push: bad rank / world size (2..%d ranks)", COMM_MAXN);
    AMP_REQUIRE(bufs && ctls, "exl3_gemv_push: null buffer table");
    AMP_REQUIRE(cap > 0 && cap % 8 == 0 && (long) m * n <= cap, "exl3_gemv_push: m * n exceeds the communicator's capacity");
    // the kernel never writes through `c` in this mode; the pointer only has to pass the checks
    GemvLaunch A = direct(x, trellis, (void*) x, suh, svh, m, k, n, K, cb, 0, 0, 0);
    for (int p = 0; p < N; ++p)
    {
        AMP_REQUIRE(bufs[p] && ctls[p], "exl3_gemv_push: null buffer of rank %d", p);
        A.ar.buf[p] = (uint2*) bufs[p];
    }
    A.ar.ctl = ctls[rank];
    A.ar.rank = rank; A.ar.N = N; A.ar.wcap = cap / 2; A.ar.push_only = 1;
    return launch_gemv(A, stream);
}

static int arin_fill(GemvLaunch& A, const void* buf, int* ctl, int N, long cap, int m, int k)
{
    AMP_REQUIRE(N >= 2 && N <= COMM_MAXN && buf && ctl, "exl3_gemv_gathered: bad communicator arguments (2..%d ranks)", COMM_MAXN);
    AMP_REQUIRE(cap > 0 && cap % 8 == 0 && (long) m * k <= cap, "exl3_gemv_gathered: m * k exceeds the communicator's capacity");
    A.arin.buf = (const uint2*) buf; A.arin.ctl = ctl; A.arin.N = N; A.arin.wcap = cap / 2;
    return 0;
}

// c (m, n) = the linear of the all-reduced input: x (m, k) is the sum of the partials the ranks
// pushed with their last amp_exl3_gemv_push on this communicator (payload (m, k)); buf / ctl are
// THIS rank's buffer and control block.
AMP_API int amp_exl3_gemv_gathered(const void* trellis, void* c, const void* suh, const void* svh,
                                   int m, int k, int n, int K, int cb, int c_fp32,
                                   const void* buf, int* ctl, int N, long cap, cudaStream_t stream)
{
    GemvLaunch A = direct(nullptr, trellis, c, suh, svh, m, k, n, K, cb, c_fp32, 0, 0);
    if (int rc = arin_fill(A, buf, ctl, N, cap, m, k)) return rc;
    return launch_gemv(A, stream);
}

// the bundle form (amp_exl3_mgemm's tables) with the gathered input
AMP_API int amp_exl3_mgemm_gathered(const void* trellis_ptrs, void* C, const void* suh_ptrs, const void* svh_ptrs,
                                    int num, int m, int k, int width, int K, int cb, int c_fp32,
                                    const void* c_ptrs, const void* n_stride_list, const void* had_src_list,
                                    const void* buf, int* ctl, int N, long cap, cudaStream_t stream)
{
    if (num == 0 || m == 0) return 0;
    AMP_REQUIRE(num > 0, "exl3_mgemm_gathered: negative matrix count");
    GemvLaunch A = {};
    A.c = C;
    A.t_trellis = (const long long*) trellis_ptrs; A.t_suh = (const long long*) suh_ptrs;
    A.t_svh = (const long long*) svh_ptrs; A.t_c = (const long long*) c_ptrs;
    A.t_stride = (const int*) n_stride_list; A.t_src = (const int*) had_src_list;
    A.tables = 1; A.slices = num; A.width = width; A.stride = width;
    A.m = m; A.k = k; A.K = K; A.cb = cb; A.c_fp32 = c_fp32;
    if (int rc = arin_fill(A, buf, ctl, N, cap, m, k)) return rc;
    return launch_gemv(A, stream);
}

// ---- allocation-free variant ----------------------------------------------------------------
// The decode GEMV with its arrival counters and partial-sum slots in a fixed array of the module
// instead of the lazily allocated per-device workspace. Limits: m <= 4, n <= 131072 (1024 column
// blocks), at most 512 CTAs. The counters must be zero when a call starts: they are zero when the
// module is loaded and every launch leaves them zero; the slots need no initial value. All calls
// on a device share the one array, so two calls that overlap on the GPU (different streams, graph
// branches) race on it.
constexpr int GEMV_STATIC_MAX_BLOCKS = 1024;
constexpr int GEMV_STATIC_MAX_CTAS = 512;
constexpr int GEMV_STATIC_MAX_M = 4;
constexpr size_t GEMV_STATIC_COUNTER_BYTES = GEMV_STATIC_MAX_BLOCKS * sizeof(int);
constexpr size_t GEMV_STATIC_SLOT_BYTES = (size_t) GEMV_STATIC_MAX_CTAS * 2 * GEMV_STATIC_MAX_M * 128 * sizeof(float);
static __device__ __align__(256) unsigned char g_gemv_static_ws[GEMV_STATIC_COUNTER_BYTES + GEMV_STATIC_SLOT_BYTES];   // 2 MB + 4 KB

AMP_API int amp_exl3_gemv_static(const void* x, const void* trellis, void* c, const void* suh, const void* svh,
                                 int m, int k, int n, int K, int cb, int c_fp32, cudaStream_t stream)
{
    AMP_REQUIRE(m >= 1 && m <= GEMV_STATIC_MAX_M, "exl3_gemv_static: m must be 1..%d (got %d); larger batches need amp_exl3_gemv",
                GEMV_STATIC_MAX_M, m);
    AMP_REQUIRE(n > 0 && n % 128 == 0 && n / 128 <= GEMV_STATIC_MAX_BLOCKS,
                "exl3_gemv_static: n must be a multiple of 128 up to %d (got %d); wider matrices need amp_exl3_gemv",
                GEMV_STATIC_MAX_BLOCKS * 128, n);
    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev)) return cuda_rc(e, "cudaGetDevice");
    // set-up, once per device: the address of this device's copy of the array
    static unsigned char* ws_ptr[64] = {};
    static std::mutex mu;
    unsigned char* ws;
    {
        std::lock_guard<std::mutex> lock(mu);
        unsigned char*& slot = ws_ptr[dev & 63];
        if (!slot)
        {
            unsigned char* ptr = nullptr;
            if (cudaError_t e = cudaGetSymbolAddress((void**) &ptr, g_gemv_static_ws)) return cuda_rc(e, "exl3_gemv_static: symbol address");
            slot = ptr;
        }
        ws = slot;
    }
    GemvLaunch A = direct(x, trellis, c, suh, svh, m, k, n, K, cb, c_fp32, 0, 0);
    A.ws_counters = (int*) ws;
    A.ws_scratch = (float*) (ws + GEMV_STATIC_COUNTER_BYTES);
    A.ws_max_ctas = GEMV_STATIC_MAX_CTAS;
    return launch_gemv(A, stream);
}

// Reads and clears the GEMV status word of the current device (synchronises the device).
AMP_API int amp_exl3_gemv_status(int* out)
{
    int v = 0, zero = 0;
    if (cudaError_t e = cudaMemcpyFromSymbol(&v, g_gemv_status, sizeof(int))) return cuda_rc(e, "status read");
    if (cudaError_t e = cudaMemcpyToSymbol(g_gemv_status, &zero, sizeof(int))) return cuda_rc(e, "status clear");
    if (out) *out = v;
    return 0;
}

// Tensor-memory form of the decode GEMV for dense / bundle launches of up to eight rows (off by
// default: the mma.sync kernel is faster). Returns the old setting.
AMP_API int amp_exl3_set_gemv_tc(int enable)
{
    const int old = g_gemv_tc;
    g_gemv_tc = enable ? 1 : 0;
    return old;
}

// Programmatic dependent launch of the decode kernels (on by default): returns the old setting.
AMP_API int amp_exl3_set_pdl(int enable)
{
    const int old = g_pdl;
    g_pdl = enable ? 1 : 0;
    return old;
}

extern "C" int amp_had_r_128(const void* in, void* out, const void* pre, const void* post,
                             long rows, int cols, int dtype, float scale, cudaStream_t stream);

// C = had(A*suh) @ W_hat -> had(.)*svh for any m. Up to 16 rows run on the decode kernel (the input
// transform lives in the kernel's prologue up to four rows; from five rows on, when A_had is given,
// a small launch of its own rotates the input into A_had once); more rows take the
// tensor-core path: x~ is written into A_had (same shape as A, fp16: required) by the Hadamard
// kernel and the tcgen05 GEMM consumes it. a_bf16: A holds bf16 instead of fp16 (m > 16 only).
static int gemm_any(const void* A, int a_bf16, const void* trellis, void* C, const void* suh, void* A_had,
                    const void* svh, int m, int k, int n, int K, int cb, int c_fp32, cudaStream_t stream)
{
    AMP_REQUIRE(m >= 0, "exl3_gemm: negative m");
    if (m == 0) return 0;
    if (K > 256)
    {
        // half-integer bitrate KA + 0.5 (K = AMP_EXL3_HALF_RATE(KA)), mul1 codebook: the input is rotated into
        // A_had by the Hadamard kernel, then the half-rate decode kernel runs (up to 16 rows; the
        // many-rows operator reconstructs the weight once instead, see exl3_gemm_recon)
        AMP_REQUIRE(K <= 256 + 3 && cb == 2, "exl3_gemm: half-integer bitrates are 1.5 / 2.5 / 3.5 with the mul1 codebook");
        AMP_REQUIRE(m <= 16 && !a_bf16, "exl3_gemm: half-integer bitrates take up to 16 fp16 rows here");
        AMP_REQUIRE(A && suh && A_had && k > 0 && k % 128 == 0, "exl3_gemm: half-integer bitrates need the A_had scratch (same shape as A)");
        if (int rc = amp_had_r_128(A, A_had, suh, nullptr, m, k, 0, 1.0f, stream)) return rc;
        int dev = 0;
        if (cudaError_t e = cudaGetDevice(&dev)) return cuda_rc(e, "cudaGetDevice");
        int* counters = nullptr; float* scratch = nullptr;
        if (int rc = workspace_region(dev, stream, &counters, &scratch)) return rc;
        return launch_gemv_half(A_had, trellis, svh, C, m, k, n, K - 256, c_fp32, counters, scratch, GEMV_SCRATCH_BYTES,
                                GEMV_MAX_BLOCKS, dev_info(dev).sms, stream);
    }
    if (m <= 16 && !a_bf16)
    {
        GemvLaunch L = direct(A, trellis, C, suh, svh, m, k, n, K, cb, c_fp32, 0, 0);
        L.x_rot = A_had;                               // optional: used from five rows up
        return launch_gemv(L, stream);
    }
    AMP_REQUIRE(A_had, "exl3_gemm: A_had scratch (same shape as A, fp16) is required above 16 rows");
    AMP_REQUIRE(A && suh && k > 0 && k % 128 == 0, "exl3_gemm: bad input");
    if (int rc = launch_had_tiled(A, A_had, suh, m, k, a_bf16, stream)) return rc;
    return launch_gemm_tc(A_had, trellis, C, svh, m, k, n, K, cb, c_fp32, stream);
}

AMP_API int amp_exl3_gemm(const void* A, const void* trellis, void* C, const void* suh, void* A_had,
                          const void* svh, int m, int k, int n, int K, int cb, int c_fp32,
                          cudaStream_t stream)
{
    return gemm_any(A, 0, trellis, C, suh, A_had, svh, m, k, n, K, cb, c_fp32, stream);
}

// Same with bf16 activations (prefill). The reference has no bf16 form (exl3_gemm checks for
// fp16, vendor/exl3/exllamav3_ext/quant/exl3_gemm.cu:136); the conversion is folded into the
// input rotation: fp32 scale, fp32 Hadamard, one rounding to fp16.
AMP_API int amp_exl3_gemm_bf16(const void* A, const void* trellis, void* C, const void* suh, void* A_had,
                               const void* svh, int m, int k, int n, int K, int cb, int c_fp32,
                               cudaStream_t stream)
{
    return gemm_any(A, 1, trellis, C, suh, A_had, svh, m, k, n, K, cb, c_fp32, stream);
}

// Several EXL3 matrices (or equal-width column slices of matrices) against ONE shared input in a
// single launch, identified by DEVICE pointer tables exactly as the reference's exl3_mgemm takes
// them (int64 device arrays). num entries in trellis_ptrs / svh_ptrs (and c_ptrs, n_stride_list,
// had_src_list when given); suh_ptrs has one entry per source (num_had_src, or num when
// had_src_list is null). Outputs go to c_ptrs[i] with row width n_stride_list[i], or stacked
// into C as (num, m, width) when c_ptrs is null. Up to 16 rows run on the decode kernel (A_had
// unused); more rows take the tensor-core path as ONE grid over all slices: the rotated input of
// every source is written into A_had ((sources, m, k) fp16, required), then the bundle form of the
// prefill GEMM runs over num * width columns.
static int mgemm_any(const void* x, int x_bf16, const void* trellis_ptrs, void* C, const void* suh_ptrs,
                     void* A_had, const void* svh_ptrs, int num, int m, int k, int width,
                     int K, int cb, int c_fp32, const void* c_ptrs, const void* n_stride_list,
                     const void* had_src_list, int num_had_src, cudaStream_t stream)
{
    if (num == 0 || m == 0) return 0;
    AMP_REQUIRE(num > 0 && m > 0, "exl3_mgemm: negative matrix or row count");
    if (m > 16 || x_bf16)
    {
        AMP_REQUIRE(x && trellis_ptrs && suh_ptrs && svh_ptrs && (C || c_ptrs), "exl3_mgemm: pointer tables are required");
        AMP_REQUIRE(A_had, "exl3_mgemm: A_had scratch ((sources, m, k) fp16) is required above 16 rows");
        AMP_REQUIRE(!had_src_list || num_had_src >= 1, "exl3_mgemm: num_had_src missing");
        const int sources = had_src_list ? num_had_src : num;
        if (int rc = launch_had_tiled(x, A_had, nullptr, m, k, x_bf16, stream, (const long long*) suh_ptrs, sources)) return rc;
        TcTables T;
        T.num = num; T.trellis = (const long long*) trellis_ptrs; T.svh = (const long long*) svh_ptrs;
        T.c = (const long long*) c_ptrs; T.stride = (const int*) n_stride_list; T.src = (const int*) had_src_list;
        return launch_gemm_tc(A_had, nullptr, C, nullptr, m, k, width, K, cb, c_fp32, stream, &T);
    }
    GemvLaunch A = {};
    A.x = x; A.c = C;
    A.t_trellis = (const long long*) trellis_ptrs; A.t_suh = (const long long*) suh_ptrs;
    A.t_svh = (const long long*) svh_ptrs; A.t_c = (const long long*) c_ptrs;
    A.t_stride = (const int*) n_stride_list; A.t_src = (const int*) had_src_list;
    A.tables = 1; A.slices = num; A.width = width; A.stride = width;
    A.m = m; A.k = k; A.K = K; A.cb = cb; A.c_fp32 = c_fp32;
    A.num_src = had_src_list ? num_had_src : num;
    A.x_rot = A.num_src >= 1 ? A_had : nullptr;                     // optional: used from five rows up
    return launch_gemv(A, stream);
}

AMP_API int amp_exl3_mgemm(const void* x, const void* trellis_ptrs, void* C, const void* suh_ptrs,
                           void* A_had, const void* svh_ptrs, int num, int m, int k, int width,
                           int K, int cb, int c_fp32, const void* c_ptrs, const void* n_stride_list,
                           const void* had_src_list, int num_had_src, cudaStream_t stream)
{
    return mgemm_any(x, 0, trellis_ptrs, C, suh_ptrs, A_had, svh_ptrs, num, m, k, width, K, cb, c_fp32,
                     c_ptrs, n_stride_list, had_src_list, num_had_src, stream);
}

// Same with bf16 activations (any row count takes the tensor-core path; the reference's bundle is
// fp16 only, vendor/exl3/exllamav3_ext/quant/exl3_gemm.cu:429).
AMP_API int amp_exl3_mgemm_bf16(const void* x, const void* trellis_ptrs, void* C, const void* suh_ptrs,
                                void* A_had, const void* svh_ptrs, int num, int m, int k, int width,
                                int K, int cb, int c_fp32, const void* c_ptrs, const void* n_stride_list,
                                const void* had_src_list, int num_had_src, cudaStream_t stream)
{
    return mgemm_any(x, 1, trellis_ptrs, C, suh_ptrs, A_had, svh_ptrs, num, m, k, width, K, cb, c_fp32,
                     c_ptrs, n_stride_list, had_src_list, num_had_src, stream);
}
