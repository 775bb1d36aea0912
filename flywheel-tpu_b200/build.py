"""Builds lib/libflywheel_b200.so for sm_100a from csrc/*.cu with nvcc.

    python flywheel-tpu_b200/build.py [--force] [--verbose]

The library is built in-tree so it travels with the source tree; nothing is
installed.  nvcc cross-compiles without a GPU present.

Where JAX is installed (`jax.ffi.include_dir()` resolves) the XLA FFI handlers
of csrc/ffi/ are built too, into lib/libflywheel_b200_ffi.so, linked against the
library above; elsewhere that step is skipped and says so.
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
FFI_SOURCE = CSRC / "ffi" / "flywheel_xla_ffi.cc"
FFI_OUTPUT = ROOT / "lib" / "libflywheel_b200_ffi.so"
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
    build_ffi(verbose)
    return OUTPUT


def xla_ffi_include_dir():
    """Directory of xla/ffi/api/ffi.h, or None where JAX is not installed."""
    try:
        import jax.ffi  # type: ignore
        return jax.ffi.include_dir()
    except Exception:  # pylint: disable=broad-except
        return None


def build_ffi(verbose: bool = False):
    """The XLA FFI handlers, only where their header exists."""
    include_dir = xla_ffi_include_dir()
    if include_dir is None:
        if verbose:
            sys.stderr.write("XLA FFI handlers skipped: jax.ffi.include_dir() does not resolve here.\n")
        return None
    cmd = ["nvcc", "-O2", "-std=c++17", "--shared", "-Xcompiler", "-fPIC", f"-I{include_dir}", f"-I{INCLUDE}",
           "-o", str(FFI_OUTPUT), str(FFI_SOURCE), f"-L{OUTPUT.parent}", "-lflywheel_b200",
           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
    result = subprocess.run(cmd, capture_output=True, text=True, check=False)
    if verbose or result.returncode:
        sys.stderr.write(result.stdout + result.stderr)
    if result.returncode:
        raise RuntimeError(f"building the XLA FFI handlers failed with exit code {result.returncode}")
    return FFI_OUTPUT


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    ns = parser.parse_args()
    print(build(ns.force, ns.verbose))
