"""Builds lib/libflywheel_b200.so for sm_100a from csrc/*.cu with nvcc.

    python flywheel-tpu_b200/build.py [--force] [--verbose]

The library is built in-tree so it travels with the source tree; nothing is
installed.  nvcc cross-compiles without a GPU present.
"""

from __future__ import annotations

import argparse
import pathlib
import subprocess
import sys

ROOT = pathlib.Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
INCLUDE = ROOT.parent / "include"
OUTPUT = ROOT / "lib" / "libflywheel_b200.so"
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
    "-std=c++17", "--shared", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def sources():
    return sorted(CSRC.glob("*.cu"))


def is_stale() -> bool:
    if not OUTPUT.exists():
        return True
    built = OUTPUT.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return any(path.stat().st_mtime > built for path in deps)


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    if not force and not is_stale():
        return OUTPUT
    OUTPUT.parent.mkdir(parents=True, exist_ok=True)
    cmd = ["nvcc", *FLAGS, f"-I{INCLUDE}", f"-I{CSRC}", "-o", str(OUTPUT),
           *map(str, sources())]
    result = subprocess.run(cmd, capture_output=True, text=True, check=False)
    if verbose or result.returncode:
        sys.stderr.write(result.stdout + result.stderr)
    if result.returncode:
        raise RuntimeError(f"nvcc failed with exit code {result.returncode}")
    return OUTPUT


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    ns = parser.parse_args()
    print(build(ns.force, ns.verbose))
