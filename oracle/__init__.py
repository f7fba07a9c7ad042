"""CPU oracle for the routed E8P expert path.  TEST INFRASTRUCTURE, not product code.

Everything in this package restates, on the CPU, the algorithm of the reference's routed
VQ expert path (jackmaxwil/keep: ``src/keep/vq/e8.py``, ``src/ramp/kernels``,
``src/ramp/ops/vq_switch.py``, ``scripts/v41_build/omlx_routed.py``,
``scripts/runpod/v41_reap/local_eval.py``).  Each function cites the reference lines it follows.

Only the tests, the smoke check and the CPU-baseline leg of the benchmark may import it.  The
shipped package ``keep_b200`` never does: its operators run CUDA code or raise.

Parity status: pinned.  The codebooks are checked against the SHA-256 digests and packed words in
the reference's ``tests/test_e8_reference.py:23-34``, the decoders against the golden codewords
of ``:37-83``, and the operators, router and residency policy against vectors that
``tests/golden/make_golden.py`` produced by running the reference's own Python here.
"""
