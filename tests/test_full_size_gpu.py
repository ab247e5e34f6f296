"""The benchmark workload at full size (232,965 vertices, ~114.6 M nonzeros, width 602), checked through
properties that need no CPU product of that size: a checksum that is independent of the order of summation,
linearity in B, and agreement between the all-sparse multiply and the one that sends the dense core of the
block through the tensor-core kernel."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.double() - b.double()).abs().max()) / max(float(b.double().abs().max()), 1e-30)


def test_benchmark_graph_checksum_linearity_and_core_agreement():
    from cagnet_b200 import graphs, ops, partition as PP
    n, f = 232965, 602
    edge = graphs.rmat_graph(n, target_nnz=114_600_000, seed=1, device="cuda")
    adj = graphs.add_self_loops(edge, n)
    _, blocks = PP.oned_partition(0, 1, torch.zeros(n, 1, device="cuda"), adj, True)
    blk = blocks[0]
    del edge, adj
    old = ops.configure_core(enabled=False)
    try:
        plain = ops.CsrBlock.from_coo(blk.rows, blk.cols, blk.vals, n, n)
    finally:
        ops.configure_core(**old)
    A = ops.CsrBlock.from_coo(blk.rows, blk.cols, blk.vals, n, n)
    assert plain.core is None
    assert A.core is not None, "the benchmark graph has a dense hub-by-hub core"
    dense = A.core[0]
    assert A.rest.nnz + int((dense != 0).sum()) == A.nnz == plain.nnz
    g = torch.Generator(device="cuda").manual_seed(7)
    b1 = ops.to_padded(torch.randn(n, f, device="cuda", generator=g))
    b2 = ops.to_padded(torch.randn(n, f, device="cuda", generator=g))
    c1, c2, c12, cp = (ops.zeros_padded(n, f, "cuda") for _ in range(4))
    ops.spmm(A, b1, c1, 0.0)
    ops.spmm(plain, b1, cp, 0.0)
    assert _rel(c1, cp) <= 1e-5                     # same product with and without the dense core
    if ops.integer_core_available():
        # the block with its normalisation factors: the core becomes bf16 edge multiplicities between two diagonals
        Ai = ops.CsrBlock.from_coo(blk.rows, blk.cols, blk.vals, n, n, row_scale=blk.row_scale, col_scale=blk.col_scale)
        assert Ai.core_kind() == "bf16-integer"
        cnt = Ai.core_int[0]
        assert Ai.rest.nnz + int((cnt != 0).sum()) == Ai.nnz
        assert cnt.numel() > dense.numel()          # a cheaper cell lets a larger rectangle pay
        ci = ops.zeros_padded(n, f, "cuda")
        ops.spmm(Ai, b1, ci, 0.0)
        assert _rel(ci, cp) <= 1e-5
        del Ai, ci, cnt
    # 1^T (A B) == (1^T A) B in fp64
    colsum = torch.zeros(n, dtype=torch.float64, device="cuda")
    colsum.index_add_(0, A.col.long(), A.val.double())
    assert _rel(c1.double().sum(0), colsum @ b1.double()) <= 1e-4
    # linearity in B
    ops.spmm(A, b2, c2, 0.0)
    ops.spmm(A, ops.to_padded(2 * b1 - b2), c12, 0.0)
    assert _rel(c12, 2 * c1 - c2) <= 1e-4
    # accumulate form: C += A B twice is 2 A B
    ops.spmm(A, b1, cp, 0.0)
    ops.spmm(A, b1, cp, 1.0)
    assert _rel(cp, 2 * c1) <= 1e-6
