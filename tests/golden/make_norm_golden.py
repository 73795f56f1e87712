"""Generate golden vectors for the RMSNorm producer / backward by running the REFERENCE's own kernels.

Run once, in a container that has the reference checkout:

    python tests/golden/make_norm_golden.py /path/to/reference

It imports the reference's NumPy emulator of triton.language (dev/tl_emu.py) and its Triton kernels
(solution/k_norm.py: rms_fwd_kernel, rms_bwd_kernel), executes them program by program on the CPU on seeded
inputs (the shapes and value ranges of the reference's own emulator test, dev/test_emu.py:72-143, plus a narrow
case) and writes tests/golden/norm_golden.npz with inputs and outputs. The reference tree is not needed to
*use* the vectors.
"""

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("NF4LL_REFERENCE")
    if not ref or not os.path.isdir(ref):
        raise SystemExit("usage: make_norm_golden.py /path/to/reference")
    sys.dont_write_bytecode = True
    sys.path.insert(0, os.path.join(ref, "dev"))
    import tl_emu

    tl_emu.install()
    sys.path.insert(0, ref)
    from solution import k_norm

    f16, f32 = np.float16, np.float32
    gold = {}
    for tag, n, d, seed in (("a", 6, 1536, 11), ("b", 3, 256, 12)):
        rng = np.random.default_rng(seed)
        eps, p, ks = 1e-6, 0.05, f32(1.0) / f32(0.95)
        x = rng.standard_normal((n, d)).astype(f32)
        delta = (rng.standard_normal((n, d)) * 0.5).astype(f16)
        w = rng.uniform(0.5, 1.5, d).astype(f32)
        mq = (rng.uniform(size=(n, d)) >= p).astype(np.uint8)
        mv = (rng.uniform(size=(n, d)) >= p).astype(np.uint8)
        y, xout, rstd = np.zeros((n, d), f16), np.zeros((n, d), f32), np.zeros(n, f32)
        xq, xv = np.zeros((n, d), f16), np.zeros((n, d), f16)
        k_norm.rms_fwd_kernel[(n,)](x, delta, xout, w, y, rstd, xq, xv, mq, mv, n, eps, float(ks), 1, 1, 1, 1,
                                    D=d, BLOCK=2048)
        y_nd, rstd_nd = np.zeros((n, d), f16), np.zeros(n, f32)
        k_norm.rms_fwd_kernel[(n,)](x, delta, xout.copy(), w, y_nd, rstd_nd, xq.copy(), xv.copy(), mq, mv, n, eps, float(ks),
                                    0, 0, 0, 1, D=d, BLOCK=2048)
        dy16 = rng.standard_normal((n, d)).astype(f16)
        lq = (rng.standard_normal((n, d)) * 0.3).astype(f16)
        lv = (rng.standard_normal((n, d)) * 0.3).astype(f16)
        dres = rng.standard_normal((n, d)).astype(f32)
        gscale = np.array([0.75], f32)
        out, out16 = dres.copy(), np.zeros((n, d), f16)
        k_norm.rms_bwd_kernel[(n,)](dy16, gscale, x, delta, w, rstd, out, out, lq, lv, out16, mq, mv, n, float(ks),
                                    1, 1, 1, 1, D=d, BLOCK=2048)
        out_plain, out16_plain = np.zeros((n, d), f32), np.zeros((n, d), f16)
        k_norm.rms_bwd_kernel[(n,)](dy16, gscale, xout, delta, w, rstd, dres, out_plain, lq, lv, out16_plain, mq, mv, n,
                                    float(ks), 0, 0, 1, 0, D=d, BLOCK=2048)
        for name, val in dict(x=x, delta=delta, w=w, mq=mq, mv=mv, eps=np.array(eps), ks=np.array(ks), y=y, xout=xout, rstd=rstd,
                              xq=xq, xv=xv, y_nodelta=y_nd, rstd_nodelta=rstd_nd, dy16=dy16, lq=lq, lv=lv, dres=dres, gscale=gscale,
                              bwd_out=out, bwd_out16=out16, bwd_plain=out_plain, bwd_plain16=out16_plain).items():
            gold[f"{tag}_{name}"] = val
    path = os.path.join(HERE, "norm_golden.npz")
    np.savez_compressed(path, **gold)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
