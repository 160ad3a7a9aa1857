"""CPU oracle for the PopTransformer per-token decode path.

TEST INFRASTRUCTURE ONLY.  This package is a CPU restatement (numpy, plus a
small C file for the timed baseline) of the reference algorithms for the decode
hot path.  Only the test-suite, the smoke check and the CPU-baseline leg of the
benchmark may import it; the product package never does.

Parity status: the reference ships no tests and no golden vectors, and its
native ops need the Poplar SDK, so the custom-op restatements in
``ops_np.py`` are pinned only by reading the cited sources ("parity unpinned"
for third-party arithmetic: matmul accumulation order, transcendental ulps,
top-k tie-breaks).  The Python-level model composition is pinned by running the
reference's own unmodified model code through ``popart_cpu`` (see
``tests/golden/make_golden.py``).
"""
