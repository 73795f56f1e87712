"""The C-ABI library loads and exports every symbol include/nf4ll.h declares (no compute calls:
this runs without a GPU), and argument validation reports caller mistakes as error codes."""

import ctypes
import os
import re

import pytest

from decentrik_prime_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def handle():
    _lib.build()
    return _lib.lib()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "nf4ll.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nf4ll_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(handle):
    names = declared_symbols()
    assert "nf4ll_forward" in names and "nf4ll_backward_dx" in names and "nf4ll_dequant" in names
    for name in names:
        assert hasattr(handle, name), name
    assert set(names) == set(_lib.SIGNATURES), "ctypes signatures out of step with the header"


def test_nothing_undeclared_is_exported(handle):
    """The dynamic symbol table holds exactly the nf4ll_* functions the header declares (no debugging
    back doors), read from the ELF file with `nm -D`."""
    import shutil
    import subprocess
    nm = shutil.which("nm")
    if nm is None:
        pytest.skip("binutils nm not installed")
    out = subprocess.run([nm, "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = sorted({line.split()[-1] for line in out.splitlines() if " T " in line and line.split()[-1].startswith("nf4ll_")})
    assert exported == declared_symbols()


def test_workspace_query_ignores_the_thread_override(handle):
    """nf4ll_workspace_bytes is a pure function of the shape; a forced split count only shows through
    nf4ll_workspace_bytes_tuned; the plain figure covers the 128-column plan of stacked projections."""
    base = handle.nf4ll_workspace_bytes(2048, 1536, 1536, 16)
    handle.nf4ll_tune_override(0, 0, 4, 0)
    try:
        assert handle.nf4ll_workspace_bytes(2048, 1536, 1536, 16) == base
    finally:
        handle.nf4ll_tune_override(0, 0, 0, 0)
    assert handle.nf4ll_workspace_bytes_tuned(2048, 1536, 1536, 16, 0, 0, 4) > base
    assert handle.nf4ll_workspace_bytes_tuned(2048, 1536, 1536, 16, 0, 0, 0) == base
    for M in (1, 64, 128, 300, 2048):
        for N, K in ((256, 256), (1536, 1536), (2048, 1536), (512, 3584), (8960, 1536), (1536, 8960)):
            plain = handle.nf4ll_workspace_bytes(M, N, K, 16)
            assert plain % 256 == 0 and plain >= M * 16 * 4


def test_version_and_error_strings(handle):
    assert handle.nf4ll_version() == 1
    assert handle.nf4ll_error_string(0) == b"ok"
    for code in (-10, -11, -12, -13, -14, -20, -21, -22):
        assert handle.nf4ll_error_string(code) not in (b"", b"unknown nf4ll status")
    assert handle.nf4ll_error_string(-99) == b"unknown nf4ll status"


def test_validation_needs_no_gpu(handle):
    assert handle.nf4ll_dequant(None, None, None, None, None, 0, None, None) == 0      # empty range is a no-op
    assert handle.nf4ll_dequant(None, None, None, None, None, 64, None, None) == -10
    assert b"null" in handle.nf4ll_last_error_detail()
    mat = _lib.Nf4Mat(16, 16, 16, 16, 16, 100, 64)          # N not a multiple of 64
    assert handle.nf4ll_forward(ctypes.byref(mat), 16, 64, None, None, None, 4, 16, 100, None, 0, None, None) == -11
    mat = _lib.Nf4Mat(8, 16, 16, 16, 16, 256, 64)            # misaligned nibbles
    assert handle.nf4ll_forward(ctypes.byref(mat), 16, 64, None, None, None, 4, 16, 256, None, 0, None, None) == -12
    with pytest.raises(ValueError):
        _lib.check(-12)
    with pytest.raises(_lib.Nf4llError):
        _lib.check(-21)
    assert handle.nf4ll_lora_down(16, 64, None, 0, 1.0, 16, 2.0, 8, 4, 64, None, None, None) == -13


def test_workspace_bytes_plan(handle):
    # no LoRA, plenty of tiles: nothing needed
    assert handle.nf4ll_workspace_bytes(16384, 18944, 3584, 0) == 0
    # LoRA only needs the fp16 rank-16 operand
    need = handle.nf4ll_workspace_bytes(16384, 18944, 3584, 16)
    assert need >= 16384 * 16 * 2 and need % 256 == 0
    # few tiles: split-K partial sums
    assert handle.nf4ll_workspace_bytes(2048, 1536, 1536, 16) > 2048 * 1536 * 4
    assert handle.nf4ll_workspace_bytes(0, 1536, 1536, 16) == 0
