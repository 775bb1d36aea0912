"""Regenerates tests/golden/*.npz from the reference's own NumPy test oracle.

Run inside the build container only (the reference checkout is not available
where the GPU tests run):

    python tests/golden/make_golden.py /path/to/reference

The reference's test module imports JAX at the top, which is not installed, so
the two pure-NumPy functions this needs (append_to_pages and ragged_reference,
tests/softmax_attention/test_paged.py:80-206 of the reference) are located by
name in its syntax tree and executed as they stand with only ``numpy`` and
``math`` in scope.  No reference source is written into this repository; only
the numeric outputs on the seeded inputs of cases.py are stored.
"""

import ast
import hashlib
import math
import pathlib
import sys

import numpy as np

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import cases  # noqa: E402


def load_reference_functions(reference_root):
    path = (pathlib.Path(reference_root) / "tests" / "softmax_attention"
            / "test_paged.py")
    tree = ast.parse(path.read_text())
    wanted = {"append_to_pages", "ragged_reference"}
    body = [node for node in tree.body
            if isinstance(node, ast.FunctionDef) and node.name in wanted]
    assert {node.name for node in body} == wanted
    scope = {"np": np, "math": math}
    exec(compile(ast.Module(body=body, type_ignores=[]), str(path), "exec"),
         scope)
    return scope["ragged_reference"]


def digest(bits):
    return np.frombuffer(hashlib.sha256(bits.tobytes()).digest(), np.uint8)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/reference-checkout")
    reference_root = sys.argv[1]
    ragged_reference = load_reference_functions(reference_root)
    for name in cases.CASES:
        c = cases.build(name)
        # fp8 cases: the reference's oracle is handed stored * descale, as its own
        # fp8 tests do (tests/softmax_attention/test_prefill.py:614-625)
        k_pages, v_pages, k_new, v_new = cases.dequantized(c)
        out, lse, kc, vc, _ = ragged_reference(
            c["q"], k_pages, v_pages, k_new, v_new, c["cu"],
            c["lengths"], c["table"], causal=c["causal"],
            window_left=c["window_left"], softcap=c["softcap"],
            sinks=c["sinks"])
        np.savez_compressed(
            HERE / f"{name}.npz", out=out.astype(np.float32),
            lse=lse.astype(np.float32),
            # The appended pages are exact in the cache type; a digest of their
            # bit patterns pins them bit for bit without storing the pools.
            k_pages_sha256=digest(cases.stored_bits(kc, c, "k")),
            v_pages_sha256=digest(cases.stored_bits(vc, c, "v")))
        print(name, out.shape, float(np.abs(out).max()))


if __name__ == "__main__":
    main()
