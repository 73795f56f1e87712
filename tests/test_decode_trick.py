"""The register-only NF4 decode used by every kernel (csrc/nf4ll_common.cuh: make_block_table +
decode_word), restated in NumPy with an emulated byte-permute, against the oracle. This pins the
bit manipulation on CPU; the GPU tests pin the compiled code."""

import numpy as np

from oracle import nf4_oracle


def byte_perm(x, y, sel):
    """CUDA __byte_perm(x, y, s): result byte i = byte (s >> 4i) & 7 of the 8-byte pair {y:x}."""
    x = np.asarray(x, dtype=np.uint64)
    y = np.asarray(y, dtype=np.uint64)
    sel = np.asarray(sel, dtype=np.uint64)
    pool = x | (y << np.uint64(32))
    out = np.zeros(np.broadcast(x, y, sel).shape, dtype=np.uint64)
    for i in range(4):
        idx = (sel >> np.uint64(4 * i)) & np.uint64(7)
        out |= ((pool >> (idx * np.uint64(8))) & np.uint64(0xFF)) << np.uint64(8 * i)
    return out.astype(np.uint32)


def block_table(absmax):
    h = (nf4_oracle.NF4_LEVELS[None, :] * absmax[:, None]).astype(np.float32).astype(np.float16).view(np.uint16)
    h = h.astype(np.uint32)
    lo, hi = [], []
    for j in range(4):
        p0 = h[:, 4 * j] | (h[:, 4 * j + 1] << 16)
        p1 = h[:, 4 * j + 2] | (h[:, 4 * j + 3] << 16)
        lo.append(byte_perm(p0, p1, 0x6420))
        hi.append(byte_perm(p0, p1, 0x7531))
    return lo, hi


def decode_word(lo, hi, w):
    w = w.astype(np.uint32)
    sel = w & np.uint32(0x77777777)
    pick = ((w >> np.uint32(1)) & np.uint32(0x44444444)) | np.uint32(0x32103210)
    outs = []
    for shift in (0, 16):
        s, p = sel >> np.uint32(shift), pick >> np.uint32(shift)
        la, lb = byte_perm(lo[0], lo[1], s), byte_perm(lo[2], lo[3], s)
        ha, hb = byte_perm(hi[0], hi[1], s), byte_perm(hi[2], hi[3], s)
        l, h = byte_perm(la, lb, p), byte_perm(ha, hb, p)
        outs += [byte_perm(l, h, 0x4051), byte_perm(l, h, 0x6273)]
    return np.stack(outs, axis=-1)      # [..., 4] uint32 = 8 fp16 in element order


def test_permute_decode_matches_oracle(golden):
    p, q, s2, o2, c2 = (golden["emu3_" + k] for k in ("packed", "qabs", "scale2", "offset2", "code2"))
    absmax = nf4_oracle.absmax_ref(q, s2, o2, c2)
    lo, hi = block_table(absmax)
    words = p.view(np.uint32).reshape(-1, 8)                 # 8 words per block
    got = np.empty((words.shape[0], 8, 4), dtype=np.uint32)
    for j in range(8):
        got[:, j] = decode_word(lo, hi, words[:, j])
    got16 = got.reshape(-1).view(np.uint16)
    assert np.array_equal(got16, golden["emu3_out"].view(np.uint16))
