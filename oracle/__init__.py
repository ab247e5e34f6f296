"""CPU oracle for the GCN hot path -- TEST INFRASTRUCTURE, not product code.

A plain restatement, in torch/numpy on the CPU, of what PASSIONLab/CAGNET computes on the path this
repository accelerates: the COO->CSR conversion and `C += A.B` of its native op, its block
partitioners and normalisation, its process-group layouts, and one training epoch of each of its four
algorithms.  Each function cites the reference file:line it follows.

Only the tests, the smoke check and the CPU-baseline leg of the benchmark may import this package, and
only as the checker.  Nothing under `cagnet_b200/` imports it.

Pinning: the reference ships no tests or golden vectors.  The fixtures under `tests/golden/` were
produced by running the reference's own Python sources on CPU (see `tests/golden/make_golden.py` for
exactly which absent dependencies were replaced by stand-ins); `tests/test_oracle_golden.py` checks
this oracle against them: bit-exact for indices, partition values and communicator layouts, and to
1e-5 for per-epoch activations, weights and weight gradients.
"""
