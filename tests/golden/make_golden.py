"""Generate the golden dequantisation vectors by running the REFERENCE's own kernel body.

Run once, in a container that has the reference checkout (path given as argv[1] or $NF4LL_REFERENCE):

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's NumPy emulator of triton.language (dev/tl_emu.py) and its Triton kernel
(solution/k_nf4.py: nf4_layer_dequant_kernel), executes the kernel program by program on CPU, and
writes tests/golden/nf4_dequant_golden.npz. The reference tree is not needed to *use* the vectors.

Cases (inputs are either stored or rebuilt by tests from the recipe below):
  emu3        three second-level blocks of random bytes / absmax codes / sorted random code2, like the
              reference's dev/test_emu.py:34-56; inputs AND output stored.
  emu3_prefix the first 512 blocks launched alone (partial last program, dev/test_emu.py:58-62).
  emu3_range  blocks [256, 768) launched on sliced pointers (dev/test_emu.py:64-70).
  exhaustive  every byte value under every absmax code: 2048 blocks; inputs by formula; output hash
              plus a strided sample.
  toy_layer   the seven weights of the reference's GPU test layer (solution/test_kernels.py:48-49),
              N(0, 0.05) fp16 quantised by this repository's quantiser, repacked, whole layer
              dequantised by the reference kernel; hashes of the flat buffer and of the output.
"""

import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def exhaustive_inputs():
    """2048 blocks: block b has absmax code b % 256 and bytes (32*(b // 256) + i) for i in 0..31."""
    nq = 2048
    b = np.arange(nq)
    packed = ((32 * (b // 256))[:, None] + np.arange(32)[None, :]).astype(np.uint8).reshape(-1)
    qabs = (b % 256).astype(np.uint8)
    code2 = np.linspace(-1.0, 1.0, 256, dtype=np.float32)
    scale2 = (0.004 + 0.0015 * np.arange(nq // 256)).astype(np.float32)
    offset2 = np.full(nq // 256, 0.0213, dtype=np.float32)
    return packed, qabs, scale2, offset2, code2


TOY_SHAPES = {"q_proj": (256, 128), "k_proj": (128, 128), "v_proj": (128, 128), "o_proj": (256, 128),
              "gate_proj": (384, 128), "up_proj": (384, 128), "down_proj": (128, 384)}


def toy_layer(seed=0):
    """(PackedLayer on CPU, code2) of the toy layer; deterministic in the torch CPU generator."""
    import torch

    sys.path.insert(0, ROOT)
    from decentrik_prime_b200 import k_nf4, quantize

    linears = {}
    for i, name in enumerate(k_nf4.LAYER_WEIGHTS):
        rows, cols = TOY_SHAPES[name]
        linears[name] = quantize.random_nf4_weight(rows, cols, seed=1000 * seed + i, std=0.05)
    return k_nf4.repack_layer(linears, torch.device("cpu"))


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("NF4LL_REFERENCE")
    if not ref or not os.path.isdir(ref):
        raise SystemExit("usage: make_golden.py /path/to/reference")
    sys.dont_write_bytecode = True
    sys.path.insert(0, os.path.join(ref, "dev"))
    import tl_emu

    tri, _ = tl_emu.install()
    sys.path.insert(0, ref)
    from solution import k_nf4 as ref_nf4

    nf4 = np.array(ref_nf4.NF4_CODE, dtype=np.float32)
    QB = ref_nf4.QBLOCKS_PER_PROGRAM

    def run(packed, qabs, scale2, offset2, code2, nq):
        out = np.zeros(nq * 64, dtype=np.float16)
        ref_nf4.nf4_layer_dequant_kernel[(tri.cdiv(nq, QB),)](packed, qabs, scale2, offset2, code2, nf4,
                                                             out, nq, QB=QB)
        return out

    gold = {}
    # emu3 --------------------------------------------------------------------------------------
    rng = np.random.default_rng(20240611)
    nq = 256 * 3
    packed = rng.integers(0, 256, nq * 32, dtype=np.uint8)
    qabs = rng.integers(0, 256, nq, dtype=np.uint8)
    code2 = np.sort(rng.uniform(-1, 1, 256)).astype(np.float32)
    scale2 = rng.uniform(0.001, 0.02, nq // 256).astype(np.float32)
    offset2 = np.repeat(rng.uniform(0.01, 0.03, 1).astype(np.float32), nq // 256)
    gold.update(emu3_packed=packed, emu3_qabs=qabs, emu3_code2=code2, emu3_scale2=scale2,
                emu3_offset2=offset2, emu3_out=run(packed, qabs, scale2, offset2, code2, nq))
    gold["emu3_prefix_sha"] = np.array(sha(run(packed[:512 * 32], qabs[:512], scale2[:2], offset2[:2], code2, 512)))
    q0, q1 = 256, 768
    gold["emu3_range_sha"] = np.array(sha(run(packed[q0 * 32:q1 * 32], qabs[q0:q1], scale2[1:3], offset2[1:3],
                                              code2, q1 - q0)))
    # exhaustive --------------------------------------------------------------------------------
    p, q, s2, o2, c2 = exhaustive_inputs()
    out = run(p, q, s2, o2, c2, q.size)
    gold["exhaustive_sha"] = np.array(sha(out))
    gold["exhaustive_sample"] = out[::97].copy()
    # toy layer ---------------------------------------------------------------------------------
    layer, code2_t = toy_layer()
    out = run(layer.packed.numpy(), layer.qabs.numpy(), layer.scale2.numpy(), layer.offset2.numpy(),
              code2_t.numpy(), layer.n_qblocks)
    gold["toy_flat_sha"] = np.array(sha(layer.flat.numpy()))
    gold["toy_out_sha"] = np.array(sha(out))
    gold["toy_out_sample"] = out[::251].copy()
    gold["nf4_levels"] = nf4
    path = os.path.join(HERE, "nf4_dequant_golden.npz")
    np.savez_compressed(path, **gold)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
