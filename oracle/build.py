"""Build recipe for the CPU checkers (test infrastructure, never part of the product path).

  oracle/_build/libmoe_oracle.so   this repository's plain-C restatement (oracle/moe_oracle.c)
  oracle/_ref/libmoe_cpu_ref.so    the reference's own C++ CPU MoE library, compiled from its source file where
                                   it lies in the reference checkout (dsv41/cpu/moe_cpu.cpp) with the flags its
                                   own loader uses (dsv41/cpumoe.py:22).  Built only when the reference checkout is
                                   present; no reference source is copied into this repository.

Run: python oracle/build.py [--reference DIR]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "_build", "libmoe_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libmoe_cpu_ref.so")
# the reference checkout: named by the environment, else a directory "reference" beside this repository
DEFAULT_REFERENCE = os.environ.get("B200MOE_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def _newer(target: str, *sources: str) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "moe_oracle.c")
    if force or not _newer(ORACLE_SO, src):
        os.makedirs(os.path.dirname(ORACLE_SO), exist_ok=True)
        subprocess.run(["gcc", "-O2", "-fopenmp", "-fvisibility=hidden", "-shared", "-fPIC", "-o", ORACLE_SO, src, "-lm"], check=True)
    return ORACLE_SO


def build_reference(reference_dir: str = DEFAULT_REFERENCE, force: bool = False) -> str | None:
    """Compile the reference's moe_cpu.cpp in place; returns the .so path, or None when the checkout is absent."""
    src = os.path.join(reference_dir, "dsv41", "cpu", "moe_cpu.cpp")
    if not os.path.exists(src):
        return REF_SO if os.path.exists(REF_SO) else None
    if force or not _newer(REF_SO, src):
        os.makedirs(os.path.dirname(REF_SO), exist_ok=True)
        subprocess.run(["g++", "-O3", "-march=sapphirerapids", "-fopenmp", "-shared", "-fPIC", "-o", REF_SO, src], check=True)
    return REF_SO


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build_oracle(a.force))
    print(build_reference(a.reference, a.force))
    sys.exit(0)
