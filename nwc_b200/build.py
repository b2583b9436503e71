"""Builds nwc_b200/lib/nwc_ops.so from nwc_b200/csrc with nvcc for sm_100a (cross-compiles without a GPU).

    python nwc_b200/build.py [--verbose]

Run it as a script (or load it by path): importing the nwc_b200 package needs the library this step produces.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "lib", "nwc_ops.so")
SOURCES = ["nwc_abi.cu", "nwc_kernels.cu", "nwc_gather.cu", "nwc_encode.cu", "nwc_model.cu", "nwc_static.cu", "nwc_prefill.cu", "nwc_comm.cu"]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--shared", "-Xcompiler", "-fPIC",
         "-Xcompiler", "-fvisibility=hidden"]


def stale() -> bool:
    if not os.path.exists(LIB): return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(os.path.dirname(HERE), "include", "nwc_ops.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, force: bool = False) -> str:
    if not force and not stale(): return LIB
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    cmd = ["nvcc"] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES]
    env = dict(os.environ); env.pop("CXX", None); env.pop("CC", None)
    out = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if verbose or out.returncode: sys.stderr.write(out.stdout + out.stderr)
    if out.returncode: raise RuntimeError("nvcc failed building nwc_ops.so")
    return LIB


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force=True))
