// Flag-in-data ("LL") words of the tensor-parallel all-reduce: an 8-byte word carries 4 bytes of
// payload and the 4-byte sequence number of the call, so data and flag arrive together. Shared by
// the stand-alone all-reduce kernel (comm_allreduce.cu) and the decode GEMV's fused epilogue
// (exl3_gemv_kernel.cuh); both follow the same buffer layout and sequence protocol, so calls of
// either kind can be mixed on one communicator.
//
// Buffer per rank: A[2 slots by call parity][N senders][cap/2 words] (+ the two-phase area).
// Control block per rank: ints [0] call sequence number, [1] blocks done in the current call,
// [16] status (non-zero: a bounded wait ran out).
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace amp {

constexpr int COMM_MAXN = 8;
constexpr int COMM_MAXB = 16;
constexpr unsigned COMM_SPIN_LIMIT = 1u << 22;    // polls of an L2-resident word: on the order of a second

__device__ __forceinline__ void st_ll2(uint2* dst, uint32_t d0, uint32_t d1, uint32_t seq)
{
    // two LL words in one 16-byte store; each 8-byte half is self-validating
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};"
                 :: "l"(dst), "r"(d0), "r"(seq), "r"(d1), "r"(seq) : "memory");
}

__device__ __forceinline__ void ld_ll2_once(const uint2* src, uint32_t (&v)[4])
{
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "l"(src) : "memory");
}

// Poll two LL words until both carry `seq`; false when the budget ran out. `budget` is the
// thread's remaining polls for the whole call, so a dead peer costs one limit, not one per word.
__device__ __forceinline__ bool ld_ll2(const uint2* src, uint32_t seq, uint32_t* d0, uint32_t* d1, unsigned& budget)
{
    for (; budget > 0; --budget)
    {
        uint32_t v[4];
        ld_ll2_once(src, v);
        if (v[1] == seq && v[3] == seq) { *d0 = v[0]; *d1 = v[2]; return true; }
    }
    return false;
}

// One unit from every sender: all loads are issued before any flag is looked at, so a unit costs
// one memory round trip when the data is already there (polling sender after sender would cost
// one per sender); only the senders still missing are polled again.
__device__ __forceinline__ bool gather_unit(uint2* const* srcs, const uint2* xv_unit, int rank, int N, uint32_t seq,
                                            uint32_t (&d)[COMM_MAXN][2], unsigned& budget)
{
    uint32_t v[COMM_MAXN][4];
    unsigned missing = 0;
    #pragma unroll
    for (int p = 0; p < COMM_MAXN; ++p)
        if (p < N && p != rank) ld_ll2_once(srcs[p], v[p]);
    #pragma unroll
    for (int p = 0; p < COMM_MAXN; ++p)
    {
        if (p >= N) continue;
        if (p == rank) { const uint2 x = *xv_unit; d[p][0] = x.x; d[p][1] = x.y; continue; }
        if (v[p][1] == seq && v[p][3] == seq) { d[p][0] = v[p][0]; d[p][1] = v[p][2]; }
        else missing |= 1u << p;
    }
    bool ok = true;
    #pragma unroll
    for (int p = 0; p < COMM_MAXN; ++p)
        if (missing & (1u << p))
            if (!ld_ll2(srcs[p], seq, &d[p][0], &d[p][1], budget)) { ok = false; d[p][0] = d[p][1] = 0; }
    return ok;
}

__device__ __forceinline__ void acc4(float (&acc)[4], uint32_t d0, uint32_t d1)
{
    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&d0));
    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&d1));
    acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
}

}  // namespace amp
