"""Build recipe for the CPU oracle (test infrastructure, not product code).

Two artefacts:

* ``oracle/liboxref.so`` -- the C restatement in ``gemm_ref.c`` (always built).
* ``oracle/_ref/run_gemm_h100_fake`` -- the reference's own host harness,
  ``test/hardware/run_gemm_h100.cu``, compiled as C *from where it lies* in a
  reference checkout and linked against ``fake_cuda_driver.c`` + ``gemm_ref.c``.
  Only built when a reference checkout is available; no reference source is
  copied.  ``tests/golden/make_golden.py`` runs it and records the outcome.

Run ``python oracle/build.py [--reference DIR]``.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboxref.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_BIN = os.path.join(REF_DIR, "run_gemm_h100_fake")
CUDA_INCLUDE = os.environ.get("CUDA_HOME", "/usr/local/cuda") + "/include"

# -ffp-contract=off: `acc += a*b` must stay a rounded multiply followed by a
# rounded add, as in the reference's plain x86-64 host build.
CFLAGS = ["-O2", "-ffp-contract=off", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wextra"]


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + proc.stdout + proc.stderr)
        raise RuntimeError("oracle build failed: " + cmd[0])


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "gemm_ref.c")
    if force or not _newer(LIB, [src]):
        _run(["gcc", *CFLAGS, "-fopenmp", "-shared", src, "-o", LIB, "-lm"])
    return LIB


def build_reference_harness(reference_root: str, force: bool = False) -> str | None:
    """Compile the reference's host harness against the fake driver."""
    harness = os.path.join(reference_root, "test", "hardware", "run_gemm_h100.cu")
    if not os.path.exists(harness):
        return None
    fake = os.path.join(HERE, "fake_cuda_driver.c")
    ref = os.path.join(HERE, "gemm_ref.c")
    if not force and _newer(REF_BIN, [harness, fake, ref]):
        return REF_BIN
    os.makedirs(REF_DIR, exist_ok=True)
    obj = os.path.join(REF_DIR, "run_gemm_h100.o")
    # The harness is plain C inside a .cu file.  fabsf is renamed so the fake
    # driver observes every C[i]-expect[i] the harness forms.
    _run(["gcc", "-x", "c", "-O2", "-ffp-contract=off", "-Dfabsf=oxpin_fabsf",
          "-I", CUDA_INCLUDE, "-c", harness, "-o", obj])
    _run(["gcc", "-O2", "-ffp-contract=off", "-I", CUDA_INCLUDE, obj, fake, ref,
          "-o", REF_BIN, "-lm"])
    return REF_BIN


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("OXGPU_REFERENCE_ROOT", ""))
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    print(build_oracle(args.force))
    if args.reference:
        print(build_reference_harness(args.reference, args.force))


if __name__ == "__main__":
    main()
