// C-ABI shim around the UNMODIFIED reference kernels (vendored exllamav3 under the reference
// tree's vendor/exl3/exllamav3_ext/quant/), compiled from where they lie by Makefile.ref into
// oracle/_ref/. Test infrastructure: lets the GPU tests and the fixture generator run the
// reference's own reconstruct / Hadamard on a B200 next to this repository's kernels.
// Raw device pointers in, wrapped into at::Tensor views without copying.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <cstdint>
#include <cstdio>
#include <exception>

// reference entry points (global namespace), quant/reconstruct.cuh and quant/hadamard.cuh
void reconstruct(at::Tensor unpacked, at::Tensor packed, float K, bool mcg, bool mul1);
void reconstruct_had_slice(at::Tensor unpacked, at::Tensor packed, at::Tensor suh, at::Tensor svh,
                           float K, bool mcg, bool mul1, int64_t n_offset);
void had_r_128(const at::Tensor& input, const at::Tensor& output,
               const c10::optional<at::Tensor>& pre_scale,
               const c10::optional<at::Tensor>& post_scale, const float scale);

static at::Tensor view(void* p, at::IntArrayRef shape, at::ScalarType t, int dev)
{
    return at::from_blob(p, shape, at::TensorOptions().dtype(t).device(at::kCUDA, dev));
}

#define GUARDED(...) \
    try { __VA_ARGS__; return 0; } \
    catch (const std::exception& e) { fprintf(stderr, "ref_shim: %s\n", e.what()); return -1; }

extern "C" int ref_reconstruct(void* unpacked, void* trellis, int k, int n, int K, int cb, int dev)
{
    GUARDED(
        auto u = view(unpacked, {k, n}, at::kHalf, dev);
        auto p = view(trellis, {k / 16, n / 16, 16 * K}, at::kShort, dev);
        reconstruct(u, p, (float) K, cb == 1, cb == 2);
    )
}

extern "C" int ref_reconstruct_had(void* unpacked, void* trellis, void* suh, void* svh,
                                   int k, int n, int K, int cb, int dev)
{
    GUARDED(
        auto u = view(unpacked, {k, n}, at::kHalf, dev);
        auto p = view(trellis, {k / 16, n / 16, 16 * K}, at::kShort, dev);
        auto su = view(suh, {k}, at::kHalf, dev);
        auto sv = view(svh, {n}, at::kHalf, dev);
        reconstruct_had_slice(u, p, su, sv, (float) K, cb == 1, cb == 2, 0);
    )
}

// half-integer bitrates KA + 0.5 (mul1 codebook only): the trellis' third dimension is 16 KA + 8
extern "C" int ref_reconstruct_half(void* unpacked, void* trellis, int k, int n, int KA, int dev)
{
    GUARDED(
        auto u = view(unpacked, {k, n}, at::kHalf, dev);
        auto p = view(trellis, {k / 16, n / 16, 16 * KA + 8}, at::kShort, dev);
        reconstruct(u, p, (float) KA + 0.5f, false, true);
    )
}

extern "C" int ref_reconstruct_had_half(void* unpacked, void* trellis, void* suh, void* svh, int k, int n, int KA, int dev)
{
    GUARDED(
        auto u = view(unpacked, {k, n}, at::kHalf, dev);
        auto p = view(trellis, {k / 16, n / 16, 16 * KA + 8}, at::kShort, dev);
        auto su = view(suh, {k}, at::kHalf, dev);
        auto sv = view(svh, {n}, at::kHalf, dev);
        reconstruct_had_slice(u, p, su, sv, (float) KA + 0.5f, false, true, 0);
    )
}

// dtype: 0 = fp16 in/out, 1 = fp32 in/out; pre/post may be null
extern "C" int ref_had_r_128(void* in, void* out, void* pre, void* post, int rows, int cols,
                             int dtype, float scale, int dev)
{
    GUARDED(
        auto t = dtype ? at::kFloat : at::kHalf;
        auto i = view(in, {rows, cols}, t, dev);
        auto o = view(out, {rows, cols}, t, dev);
        c10::optional<at::Tensor> pr, po;
        if (pre) pr = view(pre, {cols}, at::kHalf, dev);
        if (post) po = view(post, {cols}, at::kHalf, dev);
        had_r_128(i, o, pr, po, scale);
    )
}
