"""Product partitioners: bit-exact against the reference-generated fixtures and against the oracle."""
import os

import numpy as np
import pytest
import torch

from cagnet_b200 import graphs, partition as PP
from oracle import partition as OP


@pytest.fixture(scope="module")
def pg(golden_dir):
    return np.load(os.path.join(golden_dir, "partition_golden.npz"))


def _t(a):
    return torch.from_numpy(np.asarray(a))


def _same_block(blk, idx, val, size=None):
    assert np.array_equal(torch.stack([blk.rows, blk.cols]).numpy(), np.asarray(idx))
    assert np.array_equal(blk.vals.numpy(), np.asarray(val))       # bit-exact fp32
    if size is not None:
        assert [blk.n_rows, blk.n_cols] == list(size)


def test_self_loops_match_reference(pg):
    assert np.array_equal(graphs.add_self_loops(_t(pg["edge_index"]), 50).numpy(), pg["adj_selfloops"])


@pytest.mark.parametrize("P", [1, 3, 4])
def test_oned_golden(pg, P):
    adj, x = _t(pg["adj_selfloops"]), _t(pg["x"])
    for rank in range(P):
        xin, blocks = PP.oned_partition(rank, P, x, adj, True)
        assert np.array_equal(xin.numpy(), pg[f"p1d_P{P}_r{rank}_inputs"])
        for b, blk in enumerate(blocks):
            _same_block(blk, pg[f"p1d_P{P}_r{rank}_b{b}_idx"], pg[f"p1d_P{P}_r{rank}_b{b}_val"],
                        pg[f"p1d_P{P}_r{rank}_b{b}_size"].tolist())


def test_oned_unnormalised_golden(pg):
    edge, x = _t(pg["edge_index"]), _t(pg["x"])
    for rank in range(3):
        _, blocks = PP.oned_partition(rank, 3, x, edge, False)
        for b, blk in enumerate(blocks):
            _same_block(blk, pg[f"p1d_nonorm_P3_r{rank}_b{b}_idx"], pg[f"p1d_nonorm_P3_r{rank}_b{b}_val"])


@pytest.mark.parametrize("P,c", [(4, 2), (8, 2)])
def test_15d_golden(pg, P, c):
    adj, x = _t(pg["adj_selfloops"]), _t(pg["x"])
    for rank in range(P):
        xin, blocks = PP.oned_partition(rank, P, x, adj, True, replication=c)
        assert np.array_equal(xin.numpy(), pg[f"p15d_P{P}c{c}_r{rank}_inputs"])
        for b, blk in enumerate(blocks):
            _same_block(blk, pg[f"p15d_P{P}c{c}_r{rank}_b{b}_idx"], pg[f"p15d_P{P}c{c}_r{rank}_b{b}_val"],
                        pg[f"p15d_P{P}c{c}_r{rank}_b{b}_size"].tolist())


@pytest.mark.parametrize("P", [4, 9])
def test_twod_golden(pg, P):
    adj, x = _t(pg["adj_selfloops51"]), _t(pg["x51"])
    for rank in range(P):
        xin, blk = PP.twod_partition(rank, P, x, adj, True)
        assert np.array_equal(xin.numpy(), pg[f"p2d_P{P}_r{rank}_inputs"])
        _same_block(blk, pg[f"p2d_P{P}_r{rank}_idx"], pg[f"p2d_P{P}_r{rank}_val"], pg[f"p2d_P{P}_r{rank}_size"].tolist())


def test_threed_golden(pg):
    edge, x = _t(pg["edge_index51"]), _t(pg["x51"])
    for rank in range(8):
        xin, blk = PP.threed_partition(rank, 8, x, edge)
        assert np.array_equal(xin.numpy(), pg[f"p3d_P8_r{rank}_inputs"])
        _same_block(blk, pg[f"p3d_P8_r{rank}_idx"], pg[f"p3d_P8_r{rank}_val"], pg[f"p3d_P8_r{rank}_size"].tolist())


def test_groups_golden(pg):
    for P, c in ((4, 2), (8, 2), (8, 4)):
        rows, cols = PP.proc_groups_15d(P, c)
        assert rows == pg[f"groups15d_P{P}c{c}_rows"].tolist() and cols == pg[f"groups15d_P{P}c{c}_cols"].tolist()
    for P in (4, 9):
        rows, cols = PP.proc_groups_2d(P)
        assert rows == pg[f"groups2d_P{P}_rows"].tolist() and cols == pg[f"groups2d_P{P}_cols"].tolist()
    rows, cols, fibers = PP.proc_groups_3d(8)
    assert (rows, cols, fibers) == (pg["groups3d_P8_rows"].tolist(), pg["groups3d_P8_cols"].tolist(),
                                    pg["groups3d_P8_c"].tolist())


@pytest.mark.parametrize("n,P,c", [(97, 4, 1), (128, 8, 2), (61, 2, 1), (200, 8, 4)])
def test_oned_vs_oracle_random(n, P, c):
    """Ragged sizes, an R-MAT graph with hubs and isolated-but-for-self-loop vertices, duplicate edges."""
    edge = graphs.rmat_graph(n, edge_factor=6, seed=n)
    edge = torch.cat([edge, edge[:, :7]], dim=1)            # duplicates must add up, as coalesce() does
    x = torch.randn(n, 3)
    for norm in (True, False):
        adj = graphs.add_self_loops(edge, n) if norm else edge
        for rank in range(P):
            xin, blocks = PP.oned_partition(rank, P, x, adj, norm, c)
            oxin, oblocks = OP.oned_partition(rank, P, x, adj, norm, c)
            assert torch.equal(xin, oxin) and len(blocks) == len(oblocks)
            for blk, (idx, val, nr, nc) in zip(blocks, oblocks):
                _same_block(blk, idx, val, [nr, nc])


@pytest.mark.parametrize("n,P", [(97, 4), (64, 9), (51, 16)])
def test_twod_vs_oracle_random(n, P):
    edge = graphs.er_graph(n, 8, seed=n)
    x = torch.randn(n, 7)
    adj = graphs.add_self_loops(edge, n)
    for rank in range(PP.grid_side_2d(P) ** 2):
        xin, blk = PP.twod_partition(rank, P, x, adj, True)
        oxin, (idx, val, nr, nc) = OP.twod_partition(rank, P, x, adj, True)
        assert torch.equal(xin, oxin)
        _same_block(blk, idx, val, [nr, nc])


@pytest.mark.parametrize("n,P", [(97, 8), (130, 27)])
def test_threed_vs_oracle_random(n, P):
    edge = graphs.er_graph(n, 8, seed=n + 1)
    x = torch.randn(n, 9)
    for rank in range(P):
        xin, blk = PP.threed_partition(rank, P, x, edge)
        oxin, (idx, val, nr, nc) = OP.threed_partition(rank, P, x, edge)
        assert torch.equal(xin, oxin)
        _same_block(blk, idx, val, [nr, nc])


def test_stages_15d_match_oracle():
    for P, c in ((8, 2), (4, 2), (16, 4), (8, 1), (16, 2)):
        for rank in range(P):
            assert PP.stages_15d(rank, P, c) == OP.stages_15d(rank, P, c)
    # with c = 1 the stage list is the 1D loop: block i from rank i
    assert PP.stages_15d(3, 8, 1) == [(i, i) for i in range(8)]


def test_generators_are_seeded_and_symmetric():
    a = graphs.rmat_graph(300, edge_factor=8, seed=4)
    b = graphs.rmat_graph(300, edge_factor=8, seed=4)
    assert torch.equal(a, b)
    assert (a[0] != a[1]).all()
    fwd = set(map(tuple, a.t().tolist()))
    assert all((v, u) in fwd for (u, v) in fwd)
    t = graphs.rmat_graph(1000, target_nnz=30000, seed=9)
    nnz = t.size(1) + 1000
    assert 0.985 * 30000 <= nnz <= 1.005 * 30000


@pytest.mark.parametrize("normalization", [True, False])
def test_transposed_blocks_are_the_exact_transpose(normalization):
    """`transposed=True` of each partitioner, assembled over all ranks, is the transpose of what the plain call
    assembles to -- bit for bit, on an edge list that is not symmetric and has duplicates."""
    g = torch.Generator().manual_seed(5)
    n, f = 37, 6
    edge = torch.randint(0, n, (2, 300), generator=g)
    edge = torch.cat([edge, edge[:, :20]], dim=1)                   # duplicates: multiplicities above one
    adj = graphs.add_self_loops(edge, n) if normalization else edge
    x = torch.randn(n, f, generator=g)

    def dense(b):
        return torch.sparse_coo_tensor(torch.stack([b.rows, b.cols]), b.vals, (b.n_rows, b.n_cols)).to_dense()

    def oned(P, c, t):
        rows = [torch.cat([dense(b) for b in PP.oned_partition(r, P, x, adj, normalization, c, transposed=t)[1]], dim=1)
                for r in range(0, P, c)]
        return torch.cat(rows, dim=0)

    def twod(P, t):
        q = PP.grid_side_2d(P)
        return torch.cat([torch.cat([dense(PP.twod_partition(i * q + j, P, x, adj, normalization, transposed=t)[1])
                                     for j in range(q)], dim=1) for i in range(q)], dim=0)

    def threed(t, q=2):
        return torch.cat([torch.cat([dense(PP.threed_partition((i * q + j) * q + k, q ** 3, x, adj, normalization,
                                                               transposed=t)[1])
                                     for j in range(q) for k in range(q)], dim=1) for i in range(q)], dim=0)

    for P, c in ((1, 1), (3, 1), (4, 2)):
        assert torch.equal(oned(P, c, True), oned(P, c, False).t())
    assert not torch.equal(oned(3, 1, False), oned(3, 1, False).t())        # the graph really is directed
    for P in (4, 9):
        assert torch.equal(twod(P, True), twod(P, False).t())
    assert torch.equal(threed(True), threed(False).t())
    if normalization:
        # the scale vectors travel with the transposed blocks (the integer dense core needs them)
        b = PP.twod_partition(1, 4, x, adj, True, transposed=True)[1]
        assert b.row_scale.numel() == b.n_rows and b.col_scale.numel() == b.n_cols
