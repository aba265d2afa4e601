"""Builds libitb.so (CUDA kernels + C ABI) in-tree for sm_100a with nvcc. No torch involved."""
import os
import subprocess
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
SO = PKG / "libitb.so"
SOURCES = ["itb_ctx.cu", "itb_ops.cu", "itb_engine.cu", "itb_synth.cu", "itb_noalloc.cu", "itb_gguf.cu", "itb_tc.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "--fmad=false", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-ffp-contract=off", "-Xcompiler", "-O2"]


def _stale():
    if not SO.exists():
        return True
    t = SO.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [PKG.parent / "include" / "itb.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force=False, verbose=False):
    """Compile every CUDA source for sm_100a and link libitb.so next to this file. Safe when several processes call it at once
    (the ranks of a multi-GPU run importing the package with a stale library): one of them builds under a file lock, the others
    wait and find the library fresh; the link goes to a temporary name and is moved into place, so a reader never maps half a file."""
    if not force and not _stale():
        return SO
    import fcntl
    with open(PKG / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not _stale():      # another process built it while this one waited
                return SO
            return _build_locked(verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(verbose):
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objs = []
    procs = []
    for s in SOURCES:
        src = CSRC / s
        if not src.exists():
            continue
        obj = CSRC / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((subprocess.Popen(cmd), cmd))
        objs.append(str(obj))
    for p, cmd in procs:
        if p.wait() != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    tmp = PKG / f".libitb.{os.getpid()}.tmp"
    subprocess.check_call([nvcc, "-shared", "-o", str(tmp), *objs, "-lcudart_static", "-lpthread", "-ldl", "-lrt"])
    os.replace(tmp, SO)
    return SO


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
