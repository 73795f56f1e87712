"""Host side of the NF4 (block-64, double-quantised absmax) weight format.

Same names, argument meaning and error behaviour as the reference's solution/k_nf4.py, so code
written against that module (fast_qwen's layer loop, its tests) reads the same here. The
dequantisation itself is a hand-written sm_100a kernel reached through the C-ABI library
(include/nf4ll.h); there is no Triton and no CPU fallback: without the library every launcher
raises.

Format (reference solution/k_nf4.py:16-21): element e of a weight lives in byte e // 2, the even
element in the high nibble, and dequantises to
    fp16( NF4[nibble] * absmax[e // 64] ),  absmax[b] = code2[absmax_u8[b]] * absmax2[b // 256] + offset
with the product and the sum rounded separately in fp32.
"""

import torch

from . import _lib

# The 16 NF4 levels (reference solution/k_nf4.py:29-34).
NF4_CODE = (
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453,
    -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
    0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
    0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0,
)

# Order of the weights inside a repacked layer (reference solution/k_nf4.py:61): Q|K|V and
# gate|up end up contiguous, so they can also be read as fused matrices.
LAYER_WEIGHTS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")

QBLOCK = 64            # weights per quantisation block
QBLOCKS2 = 256         # quantisation blocks per second-level (absmax) block
RANGE_ALIGN = 1024     # quantisation blocks (reference solution/k_nf4.py:190)


def section_layout(n_qblocks):
    """Byte offsets of the four sections [nibbles | absmax codes | scale2 f32 | offset2 f32] and
    the total size of a flat layer buffer; every section starts on a 64-byte boundary
    (reference solution/k_nf4.py:81-88)."""
    n2 = n_qblocks // QBLOCKS2
    offsets, at = [], 0
    for nbytes in (n_qblocks * 32, n_qblocks, n2 * 4, n2 * 4):
        offsets.append(at)
        at += (nbytes + 63) // 64 * 64
    return tuple(offsets), at


def section_views(flat, offsets, n_qblocks):
    """(packed u8, qabs u8, scale2 f32, offset2 f32) views of a flat layer buffer
    (reference solution/k_nf4.py:91-95)."""
    o_pk, o_qa, o_s2, o_o2 = offsets
    n2 = n_qblocks // QBLOCKS2
    return (flat[o_pk:o_pk + n_qblocks * 32],
            flat[o_qa:o_qa + n_qblocks],
            flat[o_s2:o_s2 + 4 * n2].view(torch.float32),
            flat[o_o2:o_o2 + 4 * n2].view(torch.float32))


class PackedLayer:
    """The repacked 4-bit weights of one decoder layer in one flat uint8 buffer
    (reference solution/k_nf4.py:64-78). `segments[name] = (start element, rows, cols)`."""

    def __init__(self, flat, offsets, n_qblocks, segments):
        self.flat, self.offsets = flat, offsets
        self.n_qblocks = n_qblocks
        self.segments = segments
        self.numel = n_qblocks * QBLOCK
        self.packed, self.qabs, self.scale2, self.offset2 = section_views(flat, offsets, n_qblocks)

    def weight(self, name):
        """Sub-views (packed, qabs, scale2, offset2, rows, cols) of one weight of the layer: what
        the fused linear kernels take as their NF4 operand."""
        start, rows, cols = self.segments[name]
        n = rows * cols
        b0, q0, s0 = start // 2, start // QBLOCK, start // (QBLOCK * QBLOCKS2)
        return (self.packed[b0:b0 + n // 2], self.qabs[q0:q0 + n // QBLOCK],
                self.scale2[s0:s0 + n // (QBLOCK * QBLOCKS2)],
                self.offset2[s0:s0 + n // (QBLOCK * QBLOCKS2)], rows, cols)

    def weight_group(self, names):
        """Sub-views of several consecutive weights of the layer that share their column count, seen
        as ONE matrix with the rows stacked (Q|K|V, gate|up: contiguous by construction, reference
        solution/k_nf4.py:7-10): (packed, qabs, scale2, offset2, total rows, cols, rows per weight)."""
        start0, _, cols = self.segments[names[0]]
        at, rows_each = start0, []
        for name in names:
            start, rows, c = self.segments[name]
            if start != at or c != cols:
                raise ValueError(f"{names} are not consecutive weights with equal column counts")
            rows_each.append(rows)
            at += rows * cols
        n = at - start0
        b0, q0, s0 = start0 // 2, start0 // QBLOCK, start0 // (QBLOCK * QBLOCKS2)
        return (self.packed[b0:b0 + n // 2], self.qabs[q0:q0 + n // QBLOCK],
                self.scale2[s0:s0 + n // (QBLOCK * QBLOCKS2)],
                self.offset2[s0:s0 + n // (QBLOCK * QBLOCKS2)], sum(rows_each), cols, rows_each)


def _quant_parts(linear):
    """(weight, quant state) of a bitsandbytes-style 4-bit linear, checked for the one format the
    kernels read (same gates as reference solution/k_nf4.py:98-114). Duck-typed: anything with the
    same attributes passes, bitsandbytes itself is not needed."""
    weight = linear.weight
    state = getattr(weight, "quant_state", None)
    if state is None:
        state = getattr(linear, "quant_state", None)
    if state is None:
        raise ValueError("4-bit weight without quant_state")
    if getattr(state, "quant_type", None) != "nf4" or int(state.blocksize) != QBLOCK:
        raise ValueError(f"unsupported 4-bit format {state.quant_type}/{state.blocksize}")
    if not getattr(state, "nested", False) or state.state2 is None or int(state.state2.blocksize) != QBLOCKS2:
        raise ValueError("expected double quantisation (nested absmax, blocksize 256)")
    if weight.data.dtype != torch.uint8:
        raise ValueError(f"packed storage {weight.data.dtype}, expected uint8")
    if state.dtype != torch.float16:
        raise ValueError(f"quant_state dtype {state.dtype}, expected float16")
    return weight, state


def layer_numel(linears):
    """Number of 4-bit weights of a layer (reference solution/k_nf4.py:117-123)."""
    return sum(int(s.shape[0]) * int(s.shape[1])
               for s in (_quant_parts(linears[name])[1] for name in LAYER_WEIGHTS))


def repack_layer(linears, device, host=False, out=None, names=LAYER_WEIGHTS):
    """Repack the 4-bit linears of a layer (dict name -> module) into one PackedLayer and point the
    modules' own tensors at views of it, so nothing is stored twice. With host=True the buffer is
    pinned host memory. Returns (PackedLayer, code2 fp32). Reference solution/k_nf4.py:126-173.

    `names` (an addition) lets a caller repack a subset or a single weight in the same layout."""
    parts = [(name, *_quant_parts(linears[name])) for name in names]
    segments, total, code2 = {}, 0, None
    for name, weight, state in parts:
        rows, cols = int(state.shape[0]), int(state.shape[1])
        n = rows * cols
        if n % (QBLOCK * QBLOCKS2) != 0:
            raise ValueError(f"{name}: {n} weights do not fill whole absmax blocks")
        if weight.data.numel() * 2 != n or state.absmax.numel() * QBLOCK != n:
            raise ValueError(f"{name}: unexpected packed sizes")
        if state.state2.absmax.numel() * QBLOCKS2 * QBLOCK != n:
            raise ValueError(f"{name}: unexpected second-level absmax size")
        table = state.state2.code.to(device)
        if code2 is None:
            code2 = table
        elif not torch.equal(code2, table):
            raise ValueError("second-level code tables differ between weights")
        segments[name] = (total, rows, cols)
        total += n
    n_qblocks = total // QBLOCK
    offsets, nbytes = section_layout(n_qblocks)
    if out is not None:
        if out.numel() != nbytes or out.dtype != torch.uint8:
            raise ValueError("preallocated layer buffer has the wrong size")
        flat = out
    elif host:
        flat = torch.zeros(nbytes, dtype=torch.uint8, pin_memory=torch.cuda.is_available())
    else:
        flat = torch.zeros(nbytes, dtype=torch.uint8, device=device)
    layer = PackedLayer(flat, offsets, n_qblocks, segments)
    for name, weight, state in parts:
        pk, qa, s2, o2, _, _ = layer.weight(name)
        pk.copy_(weight.data.reshape(-1))
        qa.copy_(state.absmax.reshape(-1))
        s2.copy_(state.state2.absmax.reshape(-1).float())
        o2.copy_(state.offset.float().reshape(1).expand(o2.numel()))
        weight.data = pk.view(weight.data.shape)
        state.absmax = qa.view(state.absmax.shape)
        state.state2.absmax = s2.view(state.state2.absmax.shape)
        state.offset = state.offset.to("cpu" if host else device)
    return layer, code2.float().contiguous()


def _check_nf4_table(nf4):
    """The kernels carry the NF4 levels as compile-time constants; a caller's table (the reference
    passes one to every launcher) must be that table."""
    if nf4 is None:
        return
    ref = torch.tensor(NF4_CODE, dtype=torch.float32)
    if nf4.numel() != 16 or not torch.equal(nf4.detach().float().cpu().reshape(-1), ref):
        raise ValueError("nf4 table differs from NF4_CODE")


_NF4_OK = set()


def dequant_tensors(packed, qabs, scale2, offset2, n_qblocks, code2, nf4, out):
    """Dequantise `n_qblocks` quantisation blocks into the fp16 tensor `out` on the current CUDA
    stream (reference solution/k_nf4.py:176-181)."""
    key = None if nf4 is None else (nf4.data_ptr(), nf4._version)
    if key not in _NF4_OK:
        _check_nf4_table(nf4)
        _NF4_OK.add(key)
    if out.dtype != torch.float16 or out.numel() < n_qblocks * QBLOCK:
        raise ValueError("dequant output must be fp16 with room for every block")
    for t in (packed, qabs, scale2, offset2, code2, out):
        if not t.is_cuda:
            raise ValueError("dequant operands must live on the GPU")
    _lib.check(_lib.lib().nf4ll_dequant(
        packed.data_ptr(), qabs.data_ptr(), scale2.data_ptr(), offset2.data_ptr(),
        code2.data_ptr(), int(n_qblocks), out.data_ptr(), _lib.current_stream(out.device)))
    return out


def dequant_layer(layer, code2, nf4, out):
    """Dequantise every weight of `layer` (GPU-resident) into the flat fp16 buffer `out`
    (reference solution/k_nf4.py:184-187)."""
    return dequant_tensors(layer.packed, layer.qabs, layer.scale2, layer.offset2, layer.n_qblocks,
                           code2, nf4, out)


def dequant_range(layer, q0, q1, code2, nf4, out, dst=None):
    """Dequantise quantisation blocks [q0, q1) of `layer` into the same positions of `out` (or at
    element offset `dst`). q0 and q1 must be multiples of RANGE_ALIGN (q1 may be the layer end), as
    in the reference (solution/k_nf4.py:193-205): sliced section pointers stay 16-byte aligned and
    second-level blocks are never split."""
    if q0 % RANGE_ALIGN or (q1 % RANGE_ALIGN and q1 != layer.n_qblocks):
        raise ValueError("dequant range not aligned")
    s0, s1 = q0 // QBLOCKS2, -(-q1 // QBLOCKS2)
    start = q0 * QBLOCK if dst is None else int(dst)
    if start % (RANGE_ALIGN * QBLOCK):
        raise ValueError("dequant destination not aligned")
    return dequant_tensors(layer.packed[q0 * 32:q1 * 32], layer.qabs[q0:q1], layer.scale2[s0:s1],
                           layer.offset2[s0:s1], q1 - q0, code2, nf4,
                           out[start:start + (q1 - q0) * QBLOCK])
