"""Writes tests/golden/ref_*.npz: outputs of the REFERENCE's own CUDA kernels (reconstruct,
reconstruct_had_slice, had_r_128 of the vendored exllamav3 tree, compiled unmodified for
sm_100a by oracle/ref/Makefile.ref into oracle/_ref/libexl3_ref.so) on seeded inputs. Needs a
GPU; run once on a B200:

    python tests/golden/make_reference_fixtures.py <output dir>            # all fixtures
    python tests/golden/make_reference_fixtures.py <output dir> --half     # only the half-integer bitrates

The CPU tests then pin the oracle against these files (tests/test_oracle.py), so the oracle's
parity does not rest on a restatement alone.
"""
import ctypes
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def vp(t):
    return ctypes.c_void_p(t.data_ptr())


def half_rates(R, out_dir, cuda):
    """Half-integer bitrates 1.5 / 2.5 / 3.5 (mul1 codebook): reconstruct for each, the original-basis
    form for 2.5. Own seed, so that the other fixtures do not depend on this section."""
    rng = np.random.default_rng(20241)
    for KA in (1, 2, 3):
        trellis = rng.integers(0, 65536, size=(2, 8, 16 * KA + 8), dtype=np.uint16)
        out = torch.empty((32, 128), dtype=torch.float16, device="cuda")
        assert R.ref_reconstruct_half(vp(out), vp(cuda(trellis)), 32, 128, KA, 0) == 0
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(out_dir, "ref_reconstruct_K%d5_cb2.npz" % KA),
                            kind="reconstruct", trellis=trellis, cb=2, out=out.cpu().numpy())
    KA = 2
    trellis = rng.integers(0, 65536, size=(8, 8, 16 * KA + 8), dtype=np.uint16)
    suh = (rng.choice([-1.0, 1.0], 128) * rng.uniform(0.5, 2.0, 128)).astype(np.float16)
    svh = (rng.choice([-1.0, 1.0], 128) * rng.uniform(0.5, 2.0, 128)).astype(np.float16)
    out = torch.empty((128, 128), dtype=torch.float16, device="cuda")
    assert R.ref_reconstruct_had_half(vp(out), vp(cuda(trellis)), vp(cuda(suh)), vp(cuda(svh)), 128, 128, KA, 0) == 0
    torch.cuda.synchronize()
    np.savez_compressed(os.path.join(out_dir, "ref_reconstruct_had_K25_cb2.npz"), kind="reconstruct_had",
                        trellis=trellis, suh=suh, svh=svh, cb=2, out=out.cpu().numpy())


def main(out_dir, half_only=False):
    R = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libexl3_ref.so"))
    os.makedirs(out_dir, exist_ok=True)
    rng = np.random.default_rng(20240)

    keep = []      # device tensors stay referenced until their kernels have run

    def cuda(a):
        t = torch.from_numpy(np.ascontiguousarray(a.view(np.int16) if a.dtype == np.uint16 else a)).cuda()
        keep.append(t)
        return t

    half_rates(R, out_dir, cuda)
    if half_only:
        print("wrote the half-integer bitrate fixtures to", out_dir)
        return

    # reconstruct: every bitrate and codebook, one 32 x 128 slab each (4 KB of fp16 per case)
    for cb in range(3):
        for K in range(1, 9):
            trellis = rng.integers(0, 65536, size=(2, 8, 16 * K), dtype=np.uint16)
            out = torch.empty((32, 128), dtype=torch.float16, device="cuda")
            assert R.ref_reconstruct(vp(out), vp(cuda(trellis)), 32, 128, K, cb, 0) == 0
            torch.cuda.synchronize()
            np.savez_compressed(os.path.join(out_dir, "ref_reconstruct_K%d_cb%d.npz" % (K, cb)),
                                kind="reconstruct", trellis=trellis, cb=cb, out=out.cpu().numpy())

    # original-basis reconstruct: one 128 x 128 block per (K, cb) sample, non-trivial scales
    for K, cb in [(2, 1), (3, 2), (4, 0), (5, 0), (6, 2), (8, 1)]:
        trellis = rng.integers(0, 65536, size=(8, 8, 16 * K), dtype=np.uint16)
        suh = (rng.choice([-1.0, 1.0], 128) * rng.uniform(0.5, 2.0, 128)).astype(np.float16)
        svh = (rng.choice([-1.0, 1.0], 128) * rng.uniform(0.5, 2.0, 128)).astype(np.float16)
        out = torch.empty((128, 128), dtype=torch.float16, device="cuda")
        assert R.ref_reconstruct_had(vp(out), vp(cuda(trellis)), vp(cuda(suh)), vp(cuda(svh)), 128, 128, K, cb, 0) == 0
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(out_dir, "ref_reconstruct_had_K%d_cb%d.npz" % (K, cb)),
                            kind="reconstruct_had", trellis=trellis, suh=suh, svh=svh, cb=cb,
                            out=out.cpu().numpy())

    # Hadamard, fp16 (pre / post / none) and fp32
    x = rng.standard_normal((6, 256)).astype(np.float16)
    sc = (rng.choice([-1.0, 1.0], 256) * rng.uniform(0.5, 2.0, 256)).astype(np.float16)
    empty = np.zeros(0, np.float16)
    for name, pre, post in [("pre", sc, None), ("post", None, sc), ("none", None, None)]:
        out = torch.empty((6, 256), dtype=torch.float16, device="cuda")
        assert R.ref_had_r_128(vp(cuda(x)), vp(out), vp(cuda(pre)) if pre is not None else None,
                               vp(cuda(post)) if post is not None else None, 6, 256, 0,
                               ctypes.c_float(1.0), 0) == 0
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(out_dir, "ref_had_hf_%s.npz" % name), kind="had_hf", x=x,
                            pre=pre if pre is not None else empty, post=post if post is not None else empty,
                            out=out.cpu().numpy())
    xf = rng.standard_normal((4, 256)).astype(np.float32)
    out = torch.empty((4, 256), dtype=torch.float32, device="cuda")
    assert R.ref_had_r_128(vp(cuda(xf)), vp(out), None, vp(cuda(sc)), 4, 256, 1, ctypes.c_float(1.0), 0) == 0
    torch.cuda.synchronize()
    np.savez_compressed(os.path.join(out_dir, "ref_had_ff_post.npz"), kind="had_ff", x=xf, post=sc,
                        out=out.cpu().numpy())
    print("wrote", len(os.listdir(out_dir)), "files to", out_dir)


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    main(args[0] if args else HERE, half_only="--half" in sys.argv)
