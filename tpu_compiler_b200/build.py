"""In-tree build of libtpucb.so (sm_100a only).

    python -m tpu_compiler_b200.build [--force]
"""
import fcntl
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libtpucb.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def _nvcc():
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC)) + [
        os.path.join(os.path.dirname(HERE), "include", "tpucb.h")]


def stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(s) > t for s in sources())


def compile_command(out, verbose=False):
    cmd = [_nvcc()] + NVCC_FLAGS + [os.path.join(CSRC, "tpucb.cu"), "-o", out]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    return cmd


def build(force=False, verbose=False, run=subprocess.run):
    """Compiles the library when it is missing or older than a source. Several processes may call this at once (one
    rank per GPU under torchrun): the compile runs under an exclusive file lock, the staleness check is repeated once
    the lock is held, and the compiler writes a temporary file that replaces the library in one rename, so no process
    ever loads a half-written file."""
    if not (force or stale()):
        return LIB
    with open(LIB + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not (force or stale()):
                return LIB  # another process built it while this one waited
            tmp = "%s.%d.tmp" % (LIB, os.getpid())
            try:
                run(compile_command(tmp, verbose), check=True)
                os.replace(tmp, LIB)
            finally:
                if os.path.exists(tmp):
                    os.unlink(tmp)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
