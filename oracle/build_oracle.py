"""Build recipe for the parity oracle (TEST INFRASTRUCTURE, not the product).

* ``oracle/libtgoracle.so``      — the scalar restatement, ``oracle/tg_oracle.cpp``.
  Flags matter: ``-mfma -ffp-contract=off`` so that only the ``std::fmaf`` calls
  written in the source are fused.
* ``oracle/_ref/libtgref.so``    — the UNMODIFIED reference headers compiled
  through ``oracle/ref_shim.cpp`` with the reference's own arithmetic flags
  (reference ``Makefile:5``: ``-std=c++20 -O3 -mavx2 -mfma -ffast-math``; the
  warning flags are dropped because they do not change code generation). Built
  only where the reference checkout is present; the headers are read from where
  they lie, nothing is copied.

Usage: ``python oracle/build_oracle.py [--reference /path/to/tiny-gemma]``
"""

from __future__ import annotations

import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_REFERENCE = os.environ.get("TINY_GEMMA_REFERENCE", "/root/reference")


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources if os.path.exists(s))


def build_port(force: bool = False) -> str:
    src = os.path.join(HERE, "tg_oracle.cpp")
    out = os.path.join(HERE, "libtgoracle.so")
    if force or _stale(out, [src]):
        cmd = ["g++", "-std=c++17", "-O2", "-mfma", "-ffp-contract=off", "-fPIC", "-shared", src, "-o", out]
        subprocess.check_call(cmd)
    return out


def build_ref(reference: str = DEFAULT_REFERENCE, force: bool = False) -> str | None:
    inc = os.path.join(reference, "csrc", "include")
    out = os.path.join(HERE, "_ref", "libtgref.so")
    if not os.path.isdir(inc):
        return out if os.path.exists(out) else None
    src = os.path.join(HERE, "ref_shim.cpp")
    if force or _stale(out, [src]):
        os.makedirs(os.path.dirname(out), exist_ok=True)
        cmd = ["g++", "-std=c++20", "-O3", "-mavx2", "-mfma", "-Wno-vla", "-ffast-math", "-fPIC", "-shared",
               "-I", inc, src, "-o", out, "-lpthread"]
        subprocess.check_call(cmd)
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print("port:", build_port(a.force))
    print("ref :", build_ref(a.reference, a.force))
    return 0


if __name__ == "__main__":
    sys.exit(main())
