"""TEST INFRASTRUCTURE.  Builds the CPU oracle.

  liboracle.so        - this repository's restatement (oracle.cpp), always built
  _ref/libref_mlp.so  - the reference's own host MLP (test/mlp.h), compiled unmodified from the
                        reference checkout when one is present (environment variable TNN_REFERENCE_ROOT, else the default below);
                        on machines without the checkout the prebuilt file is used as is.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libref_mlp.so")
# the reference checkout: TNN_REFERENCE_ROOT, else a directory "reference" beside this repository
REFERENCE_ROOT = os.environ.get("TNN_REFERENCE_ROOT",
                                os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def _stale(out, srcs):
    return not os.path.exists(out) or any(os.path.getmtime(s) > os.path.getmtime(out) for s in srcs)


def build(force=False):
    src = os.path.join(HERE, "oracle.cpp")
    if force or _stale(ORACLE_SO, [src]):
        _run(["g++", "-O3", "-march=native", "-fopenmp", "-shared", "-fPIC", "-std=c++17", src, "-o", ORACLE_SO])
    mlp_h = os.path.join(REFERENCE_ROOT, "test", "mlp.h")
    if os.path.exists(mlp_h):
        harness = os.path.join(HERE, "ref_mlp_harness.cpp")
        if force or _stale(REF_SO, [harness, mlp_h, os.path.join(HERE, "shim", "common.h")]):
            os.makedirs(REF_DIR, exist_ok=True)
            _run(["g++", "-O3", "-march=native", "-shared", "-fPIC", "-std=c++20", "-I", os.path.join(HERE, "shim"),
                  "-I", os.path.join(REFERENCE_ROOT, "test"), harness, "-o", REF_SO])
    return ORACLE_SO, (REF_SO if os.path.exists(REF_SO) else None)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
