"""Build the CPU oracle (test infrastructure).

* ``oracle/liboracle.so``        -- this repository's restatement (oracle.cpp).
* ``oracle/_ref/libtpuc_ref.so`` -- the reference's own arithmetic sources
  (QuantizationArithmetic.cpp, core/lut_func.cpp, kld/calibration_math.cpp),
  compiled unmodified from the reference checkout with the stand-in headers in
  ``oracle/shims``. The checkout is named by the environment variable
  ``TPUC_REFERENCE_DIR``; without it (or without the sources there) the prebuilt
  file is reused, and ``build_ref`` says so when there is none.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("TPUC_REFERENCE_DIR", "")


def _run(cmd):
    subprocess.run(cmd, check=True, cwd=HERE)


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources if os.path.exists(s))


def build_oracle(force=False):
    out = os.path.join(HERE, "liboracle.so")
    src = os.path.join(HERE, "oracle.cpp")
    if force or _stale(out, [src]):
        _run(["g++", "-O2", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", src, "-o", out])
    return out


def build_ref(force=False):
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libtpuc_ref.so")
    srcs = [
        os.path.join(REF, "lib/Dialect/TPU/Quantization/QuantizationArithmetic.cpp"),
        os.path.join(REF, "lib/Dialect/TPU/Interpreter/core/lut_func.cpp"),
        os.path.join(REF, "bindings/python/kld/calibration_math.cpp"),
    ]
    if not REF or not all(os.path.exists(s) for s in srcs):
        if os.path.exists(out):
            return out
        if force:
            raise RuntimeError("oracle/_ref is not built and TPUC_REFERENCE_DIR does not name a reference checkout "
                               "(set it to the directory that holds lib/Dialect/TPU/Quantization/QuantizationArithmetic.cpp)")
        return None
    wrap = os.path.join(HERE, "ref_wrap.cpp")
    if force or _stale(out, srcs + [wrap]):
        os.makedirs(out_dir, exist_ok=True)
        _run(["g++", "-O2", "-fPIC", "-shared", "-fopenmp", "-w",
              "-I" + os.path.join(HERE, "shims"), "-I" + os.path.join(REF, "include")]
             + srcs + [wrap, "-lpthread", "-o", out])
    return out


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_oracle(force))
    print(build_ref(force))
