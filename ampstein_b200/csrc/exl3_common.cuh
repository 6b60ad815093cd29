// Shared device helpers for the EXL3 path on sm_100a: codebooks, bit-window extraction,
// the 128-point Hadamard across one warp, bounded mbarrier waits, bulk-copy issue.
//
// Reference behaviour this restates (paths inside the reference project):
//   codebooks        vendor/exl3/exllamav3_ext/quant/codebook.cuh:56-90
//   bitstream        vendor/exl3/exllamav3_ext/quant/exl3_dq.cuh:14-29
//   tile permutation vendor/exl3/exllamav3_ext/quant/reconstruct.cu:40-84
//   Hadamard         vendor/exl3/exllamav3_ext/quant/hadamard_inner.cuh:17-44,93-279
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace amp {

constexpr float kRScale = 0.088388347648f;   // 1/sqrt(128), spelled as the reference spells it

// ------------------------------------------------------------------------------------------
// Codebooks
// ------------------------------------------------------------------------------------------

// cb 0 / cb 1: the 32-bit word whose two fp16 halves SUM to the weight. Keeping the halves
// apart lets a tensor-core k-pair do the final add (see exl3_gemv.cu).
template <int CB>
__device__ __forceinline__ uint32_t cb_halves(uint32_t s)
{
    static_assert(CB == 0 || CB == 1, "cb_halves: cb 0 or 1");
    uint32_t x = (CB == 0) ? s * 89226354u + 64248484u : s * 0xCBAC1FEDu;
    uint32_t y;
    // (x & 0x8fff8fff) ^ 0x3b603b60 in one LOP3: f(a,b,c) = (a & b) ^ c  -> LUT 0x6a
    asm("lop3.b32 %0, %1, 0x8fff8fff, 0x3b603b60, 0x6a;" : "=r"(y) : "r"(x));
    return y;
}

// cb 2: fp16 bit pattern of 1024 + bytesum(s * M) (upper half of the word is zero); the weight
// is that value * k_inv + k_bias
__device__ __forceinline__ uint32_t cb2_raw(uint32_t s)
{
    return __dp4a(s * 0x83DCD12Du, 0x01010101u, 0x6400u);
}

// Exact fp16 weight of a state, bit-identical to the reference's decode_3inst<cb>
template <int CB>
__device__ __forceinline__ __half decode_state(uint32_t s)
{
    if constexpr (CB == 2)
    {
        const __half kinv = __ushort_as_half((unsigned short) 0x1eee);
        const __half kbias = __ushort_as_half((unsigned short) 0xc931);
        return __hfma(__ushort_as_half((unsigned short) cb2_raw(s)), kinv, kbias);
    }
    else
    {
        uint32_t y = cb_halves<CB>(s);
        __half2 h = *reinterpret_cast<__half2*>(&y);
        return __hadd(__low2half(h), __high2half(h));
    }
}

// ------------------------------------------------------------------------------------------
// Bit windows. A tile is a ring of 8*K uint32 words, MSB-first inside each word; position t
// owns the 16 bits ending at stream bit (t+1)*K.
// ------------------------------------------------------------------------------------------

// runtime position, words in (shared) memory
template <int K>
__device__ __forceinline__ uint32_t window_rt(const uint32_t* ring, int t)
{
    constexpr int W = 8 * K;
    const int last = (t + 1) * K - 1;            // index of the window's last bit
    const int j1 = last >> 5;                    // word holding it
    const int j0 = (j1 + W - 1) % W;             // the word before (ring)
    const int sh = 31 - (last & 31);
    return __funnelshift_r(ring[j1], ring[j0], sh) & 0xffffu;
}

// Half-integer bitrates KA + 0.5 (reference: dq8_half, vendor/exl3/exllamav3_ext/quant/exl3_dq.cuh:254-284):
// positions alternate KA and KA + 1 bits, the odd ones carrying the extra bit; with B2 = 2 KA + 1 the
// window of position t ends (exclusive) at bit (t / 2) * B2 + KA for even t, (t / 2 + 1) * B2 for
// odd t, in a ring of 4 * B2 words per tile.
template <int KA>
__device__ __forceinline__ uint32_t window_rt_half(const uint32_t* ring, int t)
{
    constexpr int B2 = 2 * KA + 1, W = 4 * B2;
    const int last = ((t & 1) ? ((t >> 1) + 1) * B2 : (t >> 1) * B2 + KA) - 1;
    const int j1 = last >> 5;
    const int j0 = (j1 + W - 1) % W;
    const int sh = 31 - (last & 31);
    return __funnelshift_r(ring[j1], ring[j0], sh) & 0xffffu;
}

// (x & 0xffff) on the FMA-heavy pipe (dp2a with a one-hot byte vector), leaving the integer ALU
// to the shifts
__device__ __forceinline__ uint32_t mask16_fma(uint32_t x)
{
    uint32_t d;
    asm("dp2a.lo.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(x), "r"(0x00000001u), "r"(0u));
    return d;
}

// compile-time position inside a register chunk w[0..NW) preceded by `prev`; bit 0 of the chunk
// is the MSB of w[0]. I = index of the weight inside the chunk. FMA: do the 16-bit mask on the
// FMA-heavy pipe instead of the ALU.
template <int K, int I, int NW, bool FMA = true>
__device__ __forceinline__ uint32_t window_ct(const uint32_t (&w)[NW], uint32_t prev)
{
    constexpr int last = (I + 1) * K - 1;
    constexpr int j1 = last / 32;
    constexpr int sh = 31 - (last % 32);
    static_assert(j1 < NW, "window outside the chunk");
    if constexpr (sh + 16 <= 32)
    {
        if constexpr (sh == 16) return w[j1] >> 16;
        else if constexpr (sh == 0) return FMA ? mask16_fma(w[j1]) : (w[j1] & 0xffffu);
        else return FMA ? mask16_fma(w[j1] >> sh) : ((w[j1] >> sh) & 0xffffu);
    }
    else
    {
        const uint32_t hi = (j1 == 0) ? prev : w[j1 > 0 ? j1 - 1 : 0];
        const uint32_t v = __funnelshift_r(w[j1], hi, sh);
        return FMA ? mask16_fma(v) : (v & 0xffffu);
    }
}

// ------------------------------------------------------------------------------------------
// 128-point Hadamard over one warp: lane l holds elements 4l..4l+3. fp32, natural order,
// additions in the reference's order (index bits 0,1 inside the lane, then lane bits 0..4).
// ------------------------------------------------------------------------------------------

__device__ __forceinline__ void warp_had128(float& h0, float& h1, float& h2, float& h3, int lane)
{
    float s0 = h0 + h1, d0 = h0 - h1, s1 = h2 + h3, d1 = h2 - h3;
    h0 = s0 + s1; h1 = d0 + d1; h2 = s0 - s1; h3 = d0 - d1;
    #pragma unroll
    for (int i = 1; i < 32; i <<= 1)
    {
        float p0 = __shfl_xor_sync(0xffffffffu, h0, i);
        float p1 = __shfl_xor_sync(0xffffffffu, h1, i);
        float p2 = __shfl_xor_sync(0xffffffffu, h2, i);
        float p3 = __shfl_xor_sync(0xffffffffu, h3, i);
        const bool up = (lane & i) != 0;
        h0 = up ? p0 - h0 : h0 + p0;
        h1 = up ? p1 - h1 : h1 + p1;
        h2 = up ? p2 - h2 : h2 + p2;
        h3 = up ? p3 - h3 : h3 + p3;
    }
}

struct alignas(8) half4 { __half2 x, y; };

// ------------------------------------------------------------------------------------------
// mbarrier + bulk copy (TMA, untiled form), all waits bounded
// ------------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return (uint32_t) __cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                 :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}

// Spin with an iteration limit; returns false when the limit ran out (the caller records an
// error status and leaves without touching the data)
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 24))
{
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// global -> this CTA's shared memory, completion counted on `bar`. dst/src 16-byte aligned,
// bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        :: "r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// ------------------------------------------------------------------------------------------
// cp.async (16-byte global -> shared copies, per-thread commit groups)
// ------------------------------------------------------------------------------------------

__device__ __forceinline__ void cp_async16(void* dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(smem_u32(dst)), "l"(src) : "memory");
}

__device__ __forceinline__ void cp_async_commit()
{
    asm volatile("cp.async.commit_group;" ::: "memory");
}

// wait until at most `pending` of this thread's committed groups are still in flight
__device__ __forceinline__ void cp_async_wait(int pending)
{
    switch (pending)
    {
        case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
        case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
        case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
        default: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    }
}

// ------------------------------------------------------------------------------------------
// mma.sync m16n8k16, fp16 operands, fp32 accumulate (register operands: the decoded weights
// never touch shared memory)
// ------------------------------------------------------------------------------------------

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1)
{
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

}  // namespace amp
