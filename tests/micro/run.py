"""Stand-alone micro-benchmarks behind the design decisions of the small-batch kernels. They measure the
hardware, not the library: each is one .cu file built with nvcc for sm_100a and run on cuda:0.

  feed_bench             DRAM -> shared memory of a 27648 x 2560-byte code matrix: TMA boxes, bulk copies, cp.async
  mma_issue_bench        clocks per tcgen05.mma of 128 x N x 16 for one and for several issuing threads
  stream_variants_bench  the register-level streaming kernel: loads only / compute only / both
  tma_fed_stream_bench   the same decode + mma.sync consumer fed by a TMA ring

usage: python tests/micro/run.py [name ...]      (no name: all four)
Binaries go to tests/micro/build/ (git-ignored). Not collected by pytest."""

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
BENCHES = ("feed_bench", "mma_issue_bench", "stream_variants_bench", "tma_fed_stream_bench")


def build(name):
    out_dir = os.path.join(HERE, "build")
    os.makedirs(out_dir, exist_ok=True)
    src, exe = os.path.join(HERE, name + ".cu"), os.path.join(out_dir, name)
    if not os.path.exists(exe) or os.path.getmtime(exe) < os.path.getmtime(src):
        cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
               "-I", os.path.join(ROOT, "include"), "-o", exe, src, "-lcuda"]
        subprocess.run(cmd, check=True)
    return exe


def main(argv):
    names = argv or BENCHES
    for name in names:
        if name not in BENCHES:
            raise SystemExit(f"unknown benchmark {name!r}; one of {', '.join(BENCHES)}")
    build_only = os.environ.get("MICRO_BUILD_ONLY") == "1"
    for name in names:
        exe = build(name)
        if build_only:
            continue
        print(f"==== {name}", flush=True)
        subprocess.run([exe], check=True)


if __name__ == "__main__":
    main(sys.argv[1:])
