"""Data parallelism over token rows: the only way this path shards.

Every projection is row-independent (y[m, :] depends on x[m, :] only) and the NF4 weights are
read-only, so rank g of G takes a contiguous block of packed token rows, all weights and LoRA factors
are replicated, forward and dX need no communication, and the single exchange is the sum of the fp32
LoRA gradients (blocks.GradBucket.all_reduce). The reference itself is single-GPU
(solution/integration.py:466-467); this layer is an addition.
"""


def shard_rows(n_rows, world, rank, multiple=128):
    """[start, end) of the packed token rows rank `rank` of `world` owns. Boundaries fall on multiples
    of `multiple` (the kernels' 128-row M tile) so that no tile straddles two ranks; sequence
    boundaries need not be respected because attention is outside the path."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    units = -(-n_rows // multiple)
    lo = (units * rank) // world * multiple
    hi = (units * (rank + 1)) // world * multiple
    return min(lo, n_rows), min(hi, n_rows)


class GradSync:
    """All-reduce of gradient-bucket slices on a side stream, so that the exchange of one step's LoRA
    gradients overlaps the next step's compute. A slice is identified by a slot number; whoever writes
    the slice again calls `wait_slot` first, and `wait_all` joins everything (end of a timed region,
    before the optimiser reads the gradients)."""

    def __init__(self, device, n_slots, group=None):
        import torch
        self.stream = torch.cuda.Stream(device)
        self.done = [None] * n_slots
        self.group = group

    def launch(self, slot, tensor):
        """Sum `tensor` (a view of the bucket) over the ranks, after everything queued so far on the
        current stream."""
        import torch
        import torch.distributed as dist
        self.stream.wait_stream(torch.cuda.current_stream(tensor.device))
        with torch.cuda.stream(self.stream):
            dist.all_reduce(tensor, group=self.group)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        self.done[slot] = ev

    def wait_slot(self, slot):
        import torch
        if self.done[slot] is not None:
            torch.cuda.current_stream().wait_event(self.done[slot])
            self.done[slot] = None

    def wait_all(self):
        import torch
        torch.cuda.current_stream().wait_stream(self.stream)
        self.done = [None] * len(self.done)
