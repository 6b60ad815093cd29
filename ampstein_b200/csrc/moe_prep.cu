// Token-sorted MoE dispatch in one launch: the router's picks become the expert-sorted lists that
// amp_exl3_moe_sorted (and the reference's exl3_moe) take. Integer work, bit-exact by definition:
// a stable counting sort of the assignments by local expert.
//
// Replaces, with the same name, signature and return convention (a cudaError_t), the reference's
// amp_moe_prep (src/torch/amp_kernels.cu:7024-7043, kernels :6849-7022; binding torch.moe_prep,
// src/torch/amp_torch.cpp:8164-8215). For the experts [e0, e0 + E) of this rank, with foreign picks
// in the sentinel bucket E:
//   fe[a]     bucket of assignment a = token * K + pick            order[j]  assignment at sorted position j
//   tok[j]    its token   wts[j] its weight, fp16                  inv[a]    sorted position of assignment a
//   count[b]  assignments per bucket (E + 1)   start[b] exclusive prefix sum   kind[e] = count[e] > 0
//
// One block. The assignments are cut into one contiguous segment per warp. A warp walks its segment
// 32 assignments at a time; __match_any_sync groups the lanes of one bucket, so a bucket's counter
// of the segment takes one update per group. Pass 1 counts, a prefix over the segments and a scan
// over the buckets give every (segment, bucket) its first position, pass 2 walks the segments again
// and hands out positions in assignment order: earlier segments first, then earlier steps, then
// lower lanes. The number of warps is chosen so that warps * (E + 1) counters fit in shared memory
// (32 warps up to about 1500 experts, 8 at 4096), so every E up to 4096 takes the same path.
#include "host_common.h"
#include <cuda_fp16.h>

namespace amp {

__global__ void moe_dispatch_kernel(const long long* __restrict__ idx, const float* __restrict__ w, int A, int K, int E, long long e0,
                                    long long* __restrict__ fe, long long* __restrict__ order, long long* __restrict__ tok,
                                    __half* __restrict__ wts, long long* __restrict__ count, long long* __restrict__ start,
                                    long long* __restrict__ inv, long long* __restrict__ kind)
{
    extern __shared__ int sh[];
    const int nb = E + 1, nw = blockDim.x >> 5;
    int* tot = sh;                      // [nb] assignments per bucket
    int* first = sh + nb;               // [nb] first sorted position of a bucket
    int* seg = sh + 2 * nb;             // [nw][nb] pass 1: count of (segment, bucket); then its running offset inside the bucket
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int per = (A + nw - 1) / nw;
    const int a0 = min(warp * per, A), a1 = min(a0 + per, A);
    const unsigned below = (1u << lane) - 1u;

    for (int i = t; i < nw * nb; i += blockDim.x) seg[i] = 0;
    __syncthreads();

    auto bucket_of = [&](int a) {
        const long long loc = idx[a] - e0;
        return (loc >= 0 && loc < E) ? (int) loc : E;
    };

    for (int base = a0; base < a1; base += 32)
    {
        const int a = base + lane;
        const bool live = a < a1;
        const int b = live ? bucket_of(a) : E;
        if (live) fe[a] = b;
        const unsigned peers = __match_any_sync(0xffffffffu, b) & __ballot_sync(0xffffffffu, live);
        if (live && (peers & below) == 0) seg[warp * nb + b] += __popc(peers);       // the group's lowest lane
    }
    __syncthreads();

    // per bucket: offsets of the segments inside the bucket, and the bucket's total
    for (int b = t; b < nb; b += blockDim.x)
    {
        int acc = 0;
        for (int s = 0; s < nw; ++s)
        {
            const int c = seg[s * nb + b];
            seg[s * nb + b] = acc;
            acc += c;
        }
        tot[b] = acc;
    }
    __syncthreads();

    // exclusive scan over the buckets (warp 0: a contiguous run of buckets per lane)
    if (warp == 0)
    {
        const int run = (nb + 31) / 32, b0 = min(lane * run, nb), b1 = min(b0 + run, nb);
        int sum = 0;
        for (int b = b0; b < b1; ++b) sum += tot[b];
        int inc = sum;
        #pragma unroll
        for (int d = 1; d < 32; d <<= 1)
        {
            const int o = __shfl_up_sync(0xffffffffu, inc, d);
            if (lane >= d) inc += o;
        }
        int acc = inc - sum;
        for (int b = b0; b < b1; ++b) { first[b] = acc; acc += tot[b]; }
    }
    __syncthreads();

    for (int b = t; b < nb; b += blockDim.x)
    {
        count[b] = tot[b];
        start[b] = first[b];
        if (b < E) kind[b] = tot[b] > 0 ? 1 : 0;
    }

    for (int base = a0; base < a1; base += 32)
    {
        const int a = base + lane;
        const bool live = a < a1;
        const int b = live ? bucket_of(a) : E;
        const unsigned peers = __match_any_sync(0xffffffffu, b) & __ballot_sync(0xffffffffu, live);
        int pos = 0;
        if (live) pos = first[b] + seg[warp * nb + b] + __popc(peers & below);
        __syncwarp();                                          // every lane has read the offset before the group moves it
        if (live && (peers & below) == 0) seg[warp * nb + b] += __popc(peers);
        __syncwarp();
        if (live)
        {
            order[pos] = a;
            tok[pos] = a / K;
            wts[pos] = __float2half(w[a]);
            inv[a] = pos;
        }
    }
}

}  // namespace amp

AMP_API int amp_moe_prep(const long long* idx, const float* w, int A, int K, int E, long long e0, long long* fe,
                         long long* order, long long* tok, void* wts, long long* count, long long* start,
                         long long* inv, long long* kind, cudaStream_t stream)
{
    if (A < 1 || K < 1 || E < 1 || E > 4096 || !idx || !w || !fe || !order || !tok || !wts || !count || !start || !inv || !kind)
        return (int) cudaErrorInvalidValue;
    const size_t nb = (size_t) E + 1;
    int nw = 32;
    while (nw > 1 && (2 + nw) * nb * sizeof(int) > 200 * 1024) nw >>= 1;
    const size_t smem = (2 + nw) * nb * sizeof(int);
    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev)) return (int) e;
    if (smem > 48 * 1024)
        if (cudaError_t e = amp::ensure_smem(amp::moe_dispatch_kernel, (int) smem, dev)) return (int) e;
    amp::moe_dispatch_kernel<<<1, nw * 32, smem, stream>>>(idx, w, A, K, E, e0, fe, order, tok, (__half*) wts, count, start, inv, kind);
    return (int) cudaGetLastError();
}
