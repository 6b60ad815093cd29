// N-way (2..8) fp16 all-reduce of the tensor-parallel decode path over peer-mapped memory
// (NVLink 5 / NVSwitch). Every rank runs this kernel on its own stream with its partial x; all
// ranks must issue the same sequence of calls.
//
// Replaces the reference's amp_comm_allreduce_kernel / amp_comm_allreduce_fp16
// (src/torch/amp_kernels.cu:2742-2986) and keeps its contract: sums accumulate in fp32 in rank
// order starting from 0.0f and round once, so every rank gets bit-identical values; two buffer
// slots by call parity; the call sequence number lives on the device, so the launch is
// graph-capturable; no host synchronisation.
//
// What is different on B200:
//  * Transport is a flag-in-data ("LL") push: every 8-byte store carries 4 bytes of payload and
//    the 4-byte sequence number, so a receiver sees data and flag arrive together and the
//    sender needs no system-scope fence and no separate flag round trip (the reference does
//    store -> __threadfence_system -> atomicMax flag -> poll -> fence). One NVLink traversal
//    per all-reduce instead of two plus two fences. Over NVSwitch every peer is one hop away at
//    full bandwidth, so the one-shot form (each rank pushes its whole partial to every peer)
//    is used for every N at decode payloads (10-160 KB); the two-phase form (reduce-scatter +
//    all-gather, mode 1) is kept for callers that ask for it.
//  * Every wait is bounded: after ~2^22 polls (about a second) the block records an error in the
//    status word of its control block and returns without the result, instead of trapping
//    (the reference __trap()s, which kills the context for every user of the GPU).
//  * No cluster-multicast loads: peers' data always lands in this GPU's own buffer by the
//    producers' stores and is read locally.
//
// Buffer per rank (amp_comm_buffer_bytes): LL words (uint2: payload, seq)
//   A[2 slots][N senders][cap/2 words]   phase 1 (one-shot: the whole partial; two-phase: my chunk)
//   G[2 slots][cap/2 words]              phase 2 of the two-phase form
// Control block per rank (amp_comm_ctl_bytes): ints [0] call sequence number, [1] blocks done in
// the current call, [16] status.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "host_common.h"
#include "comm_ll.cuh"
#include <cstring>

namespace amp {

constexpr int COMM_THREADS = 512;

struct CommPeers
{
    uint2* buf[COMM_MAXN];
    int* ctl[COMM_MAXN];
};

// [u0, u1) of a [0, units) range cut into `parts` pieces, piece i
__device__ __forceinline__ void comm_part(long units, int parts, int i, long* u0, long* u1)
{
    *u0 = units * i / parts;
    *u1 = units * (i + 1) / parts;
}

// n halves, n % 8 == 0. Work unit = 4 halves = 2 LL words = one 16-byte LL store.
__global__ __launch_bounds__(COMM_THREADS)
void comm_allreduce_kernel(const __half* __restrict__ x, __half* __restrict__ out, CommPeers P,
                           int rank, int N, long n, long cap, int mode)
{
    __shared__ int s_seq;
    __shared__ int s_bad;
    const int b = blockIdx.x, nb = gridDim.x;
    int* ctl = P.ctl[rank];
    int* status = ctl + COMM_MAXB;
    // One sequence number per call for every block (the flags travel inside the data, so a
    // stale word must never carry the current number): the counter only advances when the
    // last block of a call has finished, and every block reads it before it finishes.
    if (threadIdx.x == 0)
    {
        s_seq = *(volatile int*) &ctl[0] + 1;
        s_bad = 0;
    }
    __syncthreads();
    const uint32_t seq = (uint32_t) s_seq;
    const int sl = seq & 1;
    const long units = n / 4;                          // 4-half units
    const long wcap = cap / 2;                         // LL words per (slot, sender)
    const uint2* xv = reinterpret_cast<const uint2*>(x);        // one unit = one uint2 of payload
    uint2* ov = reinterpret_cast<uint2*>(out);
    bool bad = false;
    unsigned budget = COMM_SPIN_LIMIT;

    auto A_of = [&](int p, int s) { return P.buf[p] + ((long) sl * N + s) * wcap; };
    auto G_of = [&](int p) { return P.buf[p] + 2L * N * wcap + (long) sl * wcap; };

    if (mode == 0)
    {
        long u0, u1;
        comm_part(units, nb, b, &u0, &u1);
        for (int p = 0; p < N; ++p)
        {
            if (p == rank) continue;
            uint2* dst = A_of(p, rank);
            for (long i = u0 + threadIdx.x; i < u1; i += blockDim.x)
            {
                const uint2 v = xv[i];
                st_ll2(dst + 2 * i, v.x, v.y, seq);
            }
        }
        for (long i = u0 + threadIdx.x; i < u1; i += blockDim.x)
        {
            uint2* srcs[COMM_MAXN];
            #pragma unroll
            for (int p = 0; p < COMM_MAXN; ++p) srcs[p] = (p < N) ? A_of(rank, p) + 2 * i : nullptr;
            uint32_t d[COMM_MAXN][2];
            if (!gather_unit(srcs, xv + i, rank, N, seq, d, budget)) bad = true;
            float acc[4] = { 0.f, 0.f, 0.f, 0.f };
            #pragma unroll
            for (int p = 0; p < COMM_MAXN; ++p)         // rank order, fp32
                if (p < N) acc4(acc, d[p][0], d[p][1]);
            const __half2 h0 = __floats2half2_rn(acc[0], acc[1]), h1 = __floats2half2_rn(acc[2], acc[3]);
            uint2 o;
            o.x = *reinterpret_cast<const uint32_t*>(&h0);
            o.y = *reinterpret_cast<const uint32_t*>(&h1);
            ov[i] = o;
        }
    }
    else
    {
        // phase 1: my slice of chunk c goes to its owner c
        for (int c = 0; c < N; ++c)
        {
            if (c == rank) continue;
            long c0, c1, u0, u1;
            comm_part(units, N, c, &c0, &c1);
            comm_part(c1 - c0, nb, b, &u0, &u1);
            uint2* dst = A_of(c, rank);
            for (long i = c0 + u0 + threadIdx.x; i < c0 + u1; i += blockDim.x)
            {
                const uint2 v = xv[i];
                st_ll2(dst + 2 * i, v.x, v.y, seq);
            }
        }
        // reduce my chunk slice, push the result into every rank's G
        long c0, c1, u0, u1;
        comm_part(units, N, rank, &c0, &c1);
        comm_part(c1 - c0, nb, b, &u0, &u1);
        for (long i = c0 + u0 + threadIdx.x; i < c0 + u1; i += blockDim.x)
        {
            uint2* srcs[COMM_MAXN];
            #pragma unroll
            for (int p = 0; p < COMM_MAXN; ++p) srcs[p] = (p < N) ? A_of(rank, p) + 2 * i : nullptr;
            uint32_t d[COMM_MAXN][2];
            if (!gather_unit(srcs, xv + i, rank, N, seq, d, budget)) bad = true;
            float acc[4] = { 0.f, 0.f, 0.f, 0.f };
            #pragma unroll
            for (int p = 0; p < COMM_MAXN; ++p)         // rank order, fp32
                if (p < N) acc4(acc, d[p][0], d[p][1]);
            const __half2 h0 = __floats2half2_rn(acc[0], acc[1]), h1 = __floats2half2_rn(acc[2], acc[3]);
            uint2 o;
            o.x = *reinterpret_cast<const uint32_t*>(&h0);
            o.y = *reinterpret_cast<const uint32_t*>(&h1);
            for (int p = 0; p < N; ++p)
                if (p != rank) st_ll2(G_of(p) + 2 * i, o.x, o.y, seq);
            ov[i] = o;
        }
        // gather the other owners' chunk slices
        for (int c = 0; c < N; ++c)
        {
            if (c == rank) continue;
            comm_part(units, N, c, &c0, &c1);
            comm_part(c1 - c0, nb, b, &u0, &u1);
            for (long i = c0 + u0 + threadIdx.x; i < c0 + u1; i += blockDim.x)
            {
                uint2 o;
                if (!ld_ll2(G_of(rank) + 2 * i, seq, &o.x, &o.y, budget)) { bad = true; o.x = o.y = 0; }
                ov[i] = o;
            }
        }
    }

    if (bad) s_bad = 1;
    __syncthreads();
    if (threadIdx.x == 0)
    {
        if (s_bad) atomicExch(status, 1);
        __threadfence();
        if (atomicAdd(&ctl[1], 1) == nb - 1)
        {
            ctl[1] = 0;
            __threadfence();
            *(volatile int*) &ctl[0] = (int) seq;
        }
    }
}

}  // namespace amp

using namespace amp;

// Bytes of the peer-visible buffer / control block every rank must allocate (zero-filled before
// the first call) for payloads of up to `cap` halves among N ranks.
AMP_API long amp_comm_buffer_bytes(int N, long cap)
{
    if (N < 2 || N > COMM_MAXN || cap <= 0 || cap % 8) return -1;
    return (2L * N + 2) * (cap / 2) * (long) sizeof(uint2);
}

AMP_API long amp_comm_ctl_bytes(void)
{
    return (COMM_MAXB + 16) * (long) sizeof(int);
}

// Blocks the launch should use for n halves among N ranks (the same value on every rank).
AMP_API int amp_comm_blocks(int N, long n)
{
    long b = (n / 4 + COMM_THREADS - 1) / COMM_THREADS;  // one 4-half unit per thread where possible
    (void) N;
    return (int) (b < 1 ? 1 : (b > COMM_MAXB ? COMM_MAXB : b));
}

AMP_API int amp_comm_allreduce_fp16(const void* x, void* out, void* const* bufs, int* const* ctls,
                                    int rank, int N, long n, long cap, int mode, int blocks,
                                    cudaStream_t stream)
{
    if (N < 2 || N > COMM_MAXN || n <= 0 || n % 8 || n > cap || cap % 8 || blocks < 1 ||
        blocks > COMM_MAXB || rank < 0 || rank >= N || (mode != 0 && mode != 1) || !x || !out || !bufs || !ctls)
    {
        set_error("amp_comm_allreduce_fp16: invalid argument (2..8 ranks, n %% 8 == 0, n <= cap, 1..16 blocks)");
        return (int) cudaErrorInvalidValue;
    }
    CommPeers P;
    for (int p = 0; p < N; ++p)
    {
        P.buf[p] = (uint2*) bufs[p];
        P.ctl[p] = ctls[p];
        if (!bufs[p] || !ctls[p]) { set_error("amp_comm_allreduce_fp16: null peer pointer"); return (int) cudaErrorInvalidValue; }
    }
    comm_allreduce_kernel<<<blocks, COMM_THREADS, 0, stream>>>((const __half*) x, (__half*) out, P, rank, N, n, cap, mode);
    return cuda_rc(cudaGetLastError(), "amp_comm_allreduce_fp16");
}

// Reads and clears the status word of a rank's (local) control block; non-zero = a wait for a
// peer ran out. Synchronises the device.
AMP_API int amp_comm_status(int* ctl, int* out)
{
    int v = 0, zero = 0;
    if (cudaError_t e = cudaMemcpy(&v, ctl + COMM_MAXB, sizeof(int), cudaMemcpyDeviceToHost)) return cuda_rc(e, "comm status read");
    if (v) if (cudaError_t e = cudaMemcpy(ctl + COMM_MAXB, &zero, sizeof(int), cudaMemcpyHostToDevice)) return cuda_rc(e, "comm status clear");
    if (out) *out = v;
    return 0;
}

// ---- inter-process plumbing for one-process-per-GPU callers: CUDA IPC ------------------------

// Allocates `bytes` of zero-filled device memory on the current device and exports its IPC
// handle (64 bytes). Set-up time only.
AMP_API int amp_comm_ipc_alloc(long bytes, void** ptr, void* handle64)
{
    AMP_REQUIRE(bytes > 0 && ptr && handle64, "amp_comm_ipc_alloc: bad argument");
    void* p = nullptr;
    if (cudaError_t e = cudaMalloc(&p, (size_t) bytes)) return cuda_rc(e, "comm alloc");
    if (cudaError_t e = cudaMemset(p, 0, (size_t) bytes)) return cuda_rc(e, "comm clear");
    if (cudaError_t e = cudaDeviceSynchronize()) return cuda_rc(e, "comm sync");
    cudaIpcMemHandle_t h;
    if (cudaError_t e = cudaIpcGetMemHandle(&h, p)) return cuda_rc(e, "cudaIpcGetMemHandle");
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(handle64, &h, 64);
    *ptr = p;
    return 0;
}

AMP_API int amp_comm_ipc_open(const void* handle64, void** ptr)
{
    AMP_REQUIRE(handle64 && ptr, "amp_comm_ipc_open: bad argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    return cuda_rc(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
}

AMP_API int amp_comm_ipc_close(void* ptr)
{
    return cuda_rc(cudaIpcCloseMemHandle(ptr), "cudaIpcCloseMemHandle");
}

AMP_API int amp_comm_free(void* ptr)
{
    return cuda_rc(cudaFree(ptr), "cudaFree");
}

// Single-process callers (one host thread driving every GPU, as the reference does): enable
// peer access from the current device to `peer`. Already-enabled is not an error.
AMP_API int amp_comm_enable_peer(int peer)
{
    cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) { (void) cudaGetLastError(); return 0; }
    return cuda_rc(e, "cudaDeviceEnablePeerAccess");
}
