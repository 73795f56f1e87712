"""ctypes binding of the C-ABI library (include/nf4ll.h) and the nvcc recipe that builds it.

The library is built in-tree (decentrik_prime_b200/libnf4ll.so) for sm_100a only. There is no
fallback: if it is missing, or a call returns an error code, the caller gets an exception.
"""

import ctypes
import os
import shutil
import subprocess
import threading

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB_PATH = os.path.join(HERE, "libnf4ll.so")
SOURCES = ("nf4ll_api.cu", "nf4ll_dequant.cu", "nf4ll_gemm.cu", "nf4ll_gemm2.cu", "nf4ll_lora.cu", "nf4ll_swiglu.cu", "nf4ll_stream.cu", "nf4ll_swap.cu", "nf4ll_norm.cu")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "--fmad=true", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "-shared"]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return exe


def sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def needs_build():
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = sources() + _headers()
    return any(os.path.getmtime(d) > built for d in deps)


def _headers():
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    return deps + [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE) if f.endswith(".h")]


def build(force=False, verbose=False):
    """Compile csrc/*.cu into libnf4ll.so with nvcc for sm_100a (cross-compiles without a GPU).
    Every source becomes an object file under decentrik_prime_b200/build/ (compiled in parallel, only
    when it or a header is newer than its object), then the objects are linked into the library."""
    if not force and not needs_build():
        return LIB_PATH
    from concurrent.futures import ThreadPoolExecutor
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    newest_header = max(os.path.getmtime(h) for h in _headers())
    flags = [f for f in NVCC_FLAGS if f != "-shared"]

    def compile_one(src):
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(src), newest_header):
            return obj, ""
        cmd = [_nvcc(), *flags, "-I", INCLUDE, "-I", CSRC, "-c", "-o", obj, src]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
        return obj, res.stdout + res.stderr

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_one, sources()))
    link = [_nvcc(), "-shared", "-Xcompiler", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a",
            "-o", LIB_PATH + ".tmp", *[obj for obj, _ in results]]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + " ".join(link) + "\n" + res.stdout + res.stderr)
    os.replace(LIB_PATH + ".tmp", LIB_PATH)
    if verbose:
        print("".join(log for _, log in results))
    return LIB_PATH


class Nf4Mat(ctypes.Structure):
    """struct nf4ll_mat (include/nf4ll.h): device pointers to the four sections of one NF4 weight
    W[N, K] plus the shared second-level code table."""
    _fields_ = [("nib", ctypes.c_void_p), ("qabs", ctypes.c_void_p), ("scale2", ctypes.c_void_p),
                ("offset2", ctypes.c_void_p), ("code2", ctypes.c_void_p),
                ("N", ctypes.c_int64), ("K", ctypes.c_int64)]


class LoraArgs(ctypes.Structure):
    """struct nf4ll_lora (include/nf4ll.h)."""
    _fields_ = [("A", ctypes.c_void_p), ("B", ctypes.c_void_p), ("r", ctypes.c_int32),
                ("scale", ctypes.c_float), ("mask", ctypes.c_void_p), ("ld_mask", ctypes.c_int64),
                ("keep_scale", ctypes.c_float), ("Bt", ctypes.c_void_p)]


class Segment(ctypes.Structure):
    """struct nf4ll_segment (include/nf4ll.h)."""
    _fields_ = [("rows", ctypes.c_int64), ("lora", ctypes.POINTER(LoraArgs)), ("t_out", ctypes.c_void_p),
                ("t_ready", ctypes.c_int32)]


_vp, _i64, _i32, _f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_float
_MAT, _LORA, _SEG = ctypes.POINTER(Nf4Mat), ctypes.POINTER(LoraArgs), ctypes.POINTER(Segment)

# name -> (restype, argtypes); must list every symbol include/nf4ll.h declares.
SIGNATURES = {
    "nf4ll_version": (_i32, []),
    "nf4ll_error_string": (ctypes.c_char_p, [_i32]),
    "nf4ll_last_error_detail": (ctypes.c_char_p, []),
    "nf4ll_dequant": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp]),
    "nf4ll_workspace_bytes": (_i64, [_i64, _i64, _i64, _i32]),
    "nf4ll_forward": (_i32, [_MAT, _vp, _i64, _vp, _LORA, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp]),
    "nf4ll_forward_multi": (_i32, [_MAT, _vp, _i64, _vp, _SEG, _i32, _i64, _vp, _i64, _vp, _i64, _vp, _vp]),
    "nf4ll_forward_gate_up": (_i32, [_MAT, _vp, _i64, _LORA, _LORA, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64,
                                     _vp, _vp]),
    "nf4ll_forward_static": (_i32, [_MAT, _vp, _i64, _vp, _LORA, _vp, _i64, _vp, _i64, _vp, _vp]),
    "nf4ll_backward_dx": (_i32, [_MAT, _vp, _i64, _LORA, _vp, _i64, _vp, _i64, _i32, _vp, _i64, _vp, _vp]),
    "nf4ll_lora_down": (_i32, [_vp, _i64, _vp, _i64, _f32, _vp, _f32, _i32, _i64, _i64, _vp, _vp, _vp]),
    "nf4ll_lora_grads": (_i32, [_vp, _i64, _vp, _i64, _vp, _i64, _f32, _vp, _vp, _f32, _i32, _i64, _i64, _i64,
                                _vp, _vp, _i32, _vp]),
    "nf4ll_workspace_bytes_tuned": (_i64, [_i64, _i64, _i64, _i32, _i32, _i32, _i32]),
    "nf4ll_tune_override": (None, [_i32, _i32, _i32, _i32]),
    "nf4ll_test_expire_wait": (None, [ctypes.c_uint32]),
    "nf4ll_launch_count": (_i64, []),
    "nf4ll_kernel_events": (None, [_vp, _vp]),
    "nf4ll_rms_forward": (_i32, [_vp, _vp, _vp, _vp, _f32, _i64, _i64, _vp, _i64, _vp, _LORA, _vp, _LORA, _vp, _vp]),
    "nf4ll_rms_backward": (_i32, [_vp, _i64, _f32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _LORA, _vp, _LORA, _vp, _vp]),
    "nf4ll_swiglu_forward": (_i32, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _vp]),
    "nf4ll_swiglu_backward": (_i32, [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _vp]),
    "nf4ll_read_status": (_i32, [_vp, _vp]),
}

_lock = threading.Lock()
_handle = None


def lib():
    """The loaded library. Raises if it was not built: there is no other implementation."""
    global _handle
    if _handle is not None:
        return _handle
    with _lock:
        if _handle is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"{LIB_PATH} is missing: build it with decentrik_prime_b200._lib.build() "
                    "(needs nvcc); there is no CPU or Triton fallback")
            h = ctypes.CDLL(LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(h, name)
                fn.restype, fn.argtypes = res, args
            _handle = h
    return _handle


class Nf4llError(RuntimeError):
    pass


def check(code):
    """Raise for a non-zero return code: ValueError for caller mistakes (bad shape, alignment,
    null pointer), Nf4llError for device or driver failures."""
    if code == 0:
        return
    h = lib()
    msg = h.nf4ll_error_string(code).decode()
    detail = h.nf4ll_last_error_detail().decode()
    text = f"nf4ll error {code}: {msg}" + (f" ({detail})" if detail else "")
    if -19 <= code <= -10:
        raise ValueError(text)
    raise Nf4llError(text)


def current_stream(device):
    return torch.cuda.current_stream(device).cuda_stream
