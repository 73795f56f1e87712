"""Failure detection on the device: a bounded wait that runs out must end the kernel with an error status
the host can read, leave the CUDA context usable and not disturb later calls. The failure is staged
without faulting anything: the library's test hook launches a split contraction one split short (with a
short poll limit), so the wait of every CTA on its tile's other splits can never be satisfied."""

import pytest
import torch

from decentrik_prime_b200 import _lib, linear
from tests.problem import make_problem, to_device

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("direction", ["forward", "backward"])
def test_expired_wait_is_reported_and_the_next_call_is_correct(direction):
    # 1536 x 1536 at M = 2048: 48 output tiles, so the plan splits the contraction three ways and the 144
    # CTAs share the reduction (single-CTA kernel forward, CTA-pair kernel backward)
    pr = make_problem(1536, 1536, 2048, seed=71, lora=True, dropout=0.05, bias=True)
    d = to_device(pr)
    dev = d.x.device
    h = _lib.lib()

    def run():
        if direction == "forward":
            return linear.forward(d.w, d.x, bias=d.bias, lora=d.lora, mask=d.mask, keep_scale=d.keep_scale)[0]
        return linear.backward_dx(d.w, d.dy, lora=d.lora, mask=d.mask, keep_scale=d.keep_scale)[0]

    good = run().clone()
    linear.check_status()
    h.nf4ll_test_expire_wait(2000)
    run()
    with pytest.raises(_lib.Nf4llError) as info:
        linear.check_status()
    assert "wait" in str(info.value)
    word = int(linear.status_word(dev).item())
    assert word == 0x0306, hex(word)             # "a split gave up waiting for its tile's counter"
    linear.status_word(dev).zero_()              # the library never clears the word itself
    # the hook was one-shot, the context is alive, and the tile counters left behind do no harm
    again = run()
    linear.check_status()
    assert torch.equal(again, good)
