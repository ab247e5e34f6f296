"""The partitioners with the edge list on the GPU: block indices and fp32 values must equal, bit for bit, the
reference-generated fixtures (50-vertex graph) and the CPU oracle (20,011-vertex R-MAT graph, every rank of
1D P=4, 1.5D P=8 c=2, 2D P=4 and 3D P=8)."""
import os

import numpy as np
import pytest
import torch

from cagnet_b200 import graphs, partition as PP
from oracle import partition as OP

pytestmark = pytest.mark.gpu


def _same(blk, idx, val):
    assert np.array_equal(torch.stack([blk.rows, blk.cols]).cpu().numpy(), np.asarray(idx))
    assert np.array_equal(blk.vals.cpu().numpy(), np.asarray(val))          # bit-exact fp32


def test_fixture_partitions_on_the_gpu(golden_dir):
    pg = np.load(os.path.join(golden_dir, "partition_golden.npz"))
    adj = torch.from_numpy(pg["adj_selfloops"]).cuda()
    x = torch.from_numpy(pg["x"]).cuda()
    for P in (1, 3, 4):
        for rank in range(P):
            xin, blocks = PP.oned_partition(rank, P, x, adj, True)
            assert np.array_equal(xin.cpu().numpy(), pg[f"p1d_P{P}_r{rank}_inputs"])
            for b, blk in enumerate(blocks):
                _same(blk, pg[f"p1d_P{P}_r{rank}_b{b}_idx"], pg[f"p1d_P{P}_r{rank}_b{b}_val"])
    for P, c in ((4, 2), (8, 2)):
        for rank in range(P):
            _, blocks = PP.oned_partition(rank, P, x, adj, True, replication=c)
            for b, blk in enumerate(blocks):
                _same(blk, pg[f"p15d_P{P}c{c}_r{rank}_b{b}_idx"], pg[f"p15d_P{P}c{c}_r{rank}_b{b}_val"])


@pytest.fixture(scope="module")
def rmat():
    n = 20011
    edge = graphs.rmat_graph(n, target_nnz=400000, seed=4, device="cpu")
    adj = graphs.add_self_loops(edge, n)
    x = torch.randn(n, 6, generator=torch.Generator().manual_seed(1))
    return n, adj, x


@pytest.mark.parametrize("P,c", [(4, 1), (8, 2)])
def test_oned_against_oracle(rmat, P, c):
    n, adj, x = rmat
    adj_d, x_d = adj.cuda(), x.cuda()
    for rank in range(P):
        xin, blocks = PP.oned_partition(rank, P, x_d, adj_d, True, replication=c)
        xin_o, blocks_o = OP.oned_partition(rank, P, x, adj, True, replication=c)
        assert torch.equal(xin.cpu(), xin_o)
        assert len(blocks) == len(blocks_o)
        for blk, (idx, val, nr, nc) in zip(blocks, blocks_o):
            _same(blk, idx.numpy(), val.numpy())
            assert (blk.n_rows, blk.n_cols) == (nr, nc)


def test_twod_and_threed_against_oracle(rmat):
    n, adj, x = rmat
    adj_d, x_d = adj.cuda(), x.cuda()
    for rank in range(4):
        xin, blk = PP.twod_partition(rank, 4, x_d, adj_d, True)
        xin_o, (idx, val, nr, nc) = OP.twod_partition(rank, 4, x, adj, True)
        assert torch.equal(xin.cpu(), xin_o)
        _same(blk, idx.numpy(), val.numpy())
        assert (blk.n_rows, blk.n_cols) == (nr, nc)
    for rank in range(8):
        xin, slab = PP.threed_partition(rank, 8, x_d, adj_d, False)
        xin_o, (idx, val, nr, nc) = OP.threed_partition(rank, 8, x, adj)
        assert torch.equal(xin.cpu(), xin_o)
        _same(slab, idx.numpy(), val.numpy())
        assert (slab.n_rows, slab.n_cols) == (nr, nc)
