"""nf4ll_forward_static: the forward for callers that cannot provide scratch memory (a host that
forbids device allocations after start-up, a sealed memory pool). It must give what nf4ll_forward
gives while taking its scratch from the buffer built into the library, on back-to-back calls that
reuse that buffer with different problems, and it must refuse problems that do not fit.

Collected last on purpose: a run that stops at the first failure has then already run every other test.
"""

import ctypes

import pytest
import torch

from decentrik_prime_b200 import _lib, linear
from oracle import nf4_oracle
from tests.problem import make_problem, oracle_weight, to_device

pytestmark = pytest.mark.gpu
MAX_ABS, REL_L2 = 2e-2, 1e-3


def _call(h, static, d, y, t, ws=None):
    lora = _lib.LoraArgs(d.A16.data_ptr(), d.B16.data_ptr(), 16, d.lora[2], d.mask.data_ptr(), d.mask.stride(0),
                         d.keep_scale, 0)
    st = linear.status_word(d.x.device)
    stream = _lib.current_stream(d.x.device)
    M = d.x.shape[0]
    if static:
        return h.nf4ll_forward_static(ctypes.byref(d.w._c), d.x.data_ptr(), d.x.stride(0), d.bias.data_ptr(),
                                      ctypes.byref(lora), t.data_ptr(), M, y.data_ptr(), y.stride(0), st.data_ptr(), stream)
    return h.nf4ll_forward(ctypes.byref(d.w._c), d.x.data_ptr(), d.x.stride(0), d.bias.data_ptr(), ctypes.byref(lora),
                           t.data_ptr(), M, y.data_ptr(), y.stride(0), ws.data_ptr(), ws.numel(), st.data_ptr(), stream)


def test_static_scratch_forward_matches_workspace_forward_twice():
    h = _lib.lib()
    # two different problems in a row through the same built-in buffer: the first splits its contraction
    # (partial sums and tile counters live in the scratch), the second does not
    for N, K, M, seed in ((1536, 1536, 2048, 51), (512, 256, 300, 52)):
        pr = make_problem(N, K, M, seed=seed, lora=True, dropout=0.05, bias=True)
        d = to_device(pr)
        need = h.nf4ll_workspace_bytes(M, N, K, 16)
        assert need <= 40 * 1024 * 1024
        ws = torch.empty(max(need, 256), dtype=torch.uint8, device="cuda")
        y_ref = torch.empty(M, N, dtype=torch.float16, device="cuda")
        y_new = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
        t_ref = torch.empty(M, 16, dtype=torch.float32, device="cuda")
        t_new = torch.full((M, 16), float("nan"), dtype=torch.float32, device="cuda")
        _lib.check(_call(h, False, d, y_ref, t_ref, ws))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        _lib.check(_call(h, True, d, y_new, t_new))
        linear.check_status()
        # the call took nothing from the device: not through the runtime, not through torch's allocator
        assert torch.cuda.mem_get_info()[0] == free_before
        err, rel = nf4_oracle.errors(y_new, y_ref.float())
        assert err <= MAX_ABS and rel <= REL_L2, (N, K, M, err, rel)
        err, rel = nf4_oracle.errors(t_new, t_ref)
        assert err <= MAX_ABS and rel <= REL_L2, (N, K, M, err, rel)
        # and against the CPU oracle, not only against the library's other entry point
        ref = nf4_oracle.lora_linear_o1(oracle_weight(pr), pr.x, None, pr.bias, pr.A16, pr.B16, pr.scale, pr.mask, pr.keep_scale)
        for name, got in (("y", y_new), ("t", t_new)):
            err, rel = nf4_oracle.errors(got, ref[name])
            assert err <= MAX_ABS and rel <= REL_L2, (name, N, K, M, err, rel)


def test_static_scratch_refuses_problems_that_do_not_fit():
    h = _lib.lib()
    d = to_device(make_problem(1536, 1536, 2048, seed=53, lora=True, dropout=0.05, bias=True))
    y = torch.empty(2048, 1536, dtype=torch.float16, device="cuda")
    t = torch.empty(2048, 16, dtype=torch.float32, device="cuda")
    with linear.tune_override(splits=4):      # four fp32 partial slabs of 12.6 MB each: more than the buffer holds
        assert h.nf4ll_workspace_bytes_tuned(2048, 1536, 1536, 16, 0, 0, 4) > 40 * 1024 * 1024
        rc = _call(h, True, d, y, t)
    assert rc == -14
    assert b"built-in buffer" in h.nf4ll_last_error_detail()
    with pytest.raises(ValueError):
        _lib.check(rc)
