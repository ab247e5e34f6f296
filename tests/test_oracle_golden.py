"""The oracle against fixtures produced by the reference's own code (tests/golden/make_golden.py)."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import gcn as OG
from oracle import partition as OP


@pytest.fixture(scope="module")
def pg(golden_dir):
    return np.load(os.path.join(golden_dir, "partition_golden.npz"))


def _t(a):
    return torch.from_numpy(np.asarray(a))


def test_self_loops(pg):
    got = OP.add_self_loops(_t(pg["edge_index"]), 50)
    assert np.array_equal(got.numpy(), pg["adj_selfloops"])


@pytest.mark.parametrize("dim", [0, 1])
def test_split_coo_1d(pg, dim):
    parts, vtx = OP.split_coo(_t(pg["adj_selfloops"]), 50, 13, dim)
    assert vtx == pg[f"split1d_dim{dim}_vtx"].tolist()
    for i, p in enumerate(parts):
        assert np.array_equal(p.numpy(), pg[f"split1d_dim{dim}_part{i}"])


@pytest.mark.parametrize("P", [1, 3, 4])
def test_oned_partition(pg, P):
    adj, x = _t(pg["adj_selfloops"]), _t(pg["x"])
    for rank in range(P):
        xin, blocks = OP.oned_partition(rank, P, x, adj, True)
        assert np.array_equal(xin.numpy(), pg[f"p1d_P{P}_r{rank}_inputs"])
        for b, (idx, val, nr, nc) in enumerate(blocks):
            assert np.array_equal(idx.numpy(), pg[f"p1d_P{P}_r{rank}_b{b}_idx"])
            assert np.array_equal(val.numpy(), pg[f"p1d_P{P}_r{rank}_b{b}_val"])          # bit-exact fp32
            assert [nr, nc] == pg[f"p1d_P{P}_r{rank}_b{b}_size"].tolist()


def test_oned_partition_unnormalised(pg):
    edge, x = _t(pg["edge_index"]), _t(pg["x"])
    for rank in range(3):
        _, blocks = OP.oned_partition(rank, 3, x, edge, False)
        for b, (idx, val, _, _) in enumerate(blocks):
            assert np.array_equal(idx.numpy(), pg[f"p1d_nonorm_P3_r{rank}_b{b}_idx"])
            assert np.array_equal(val.numpy(), pg[f"p1d_nonorm_P3_r{rank}_b{b}_val"])


@pytest.mark.parametrize("P,c", [(4, 2), (8, 2)])
def test_15d_partition(pg, P, c):
    adj, x = _t(pg["adj_selfloops"]), _t(pg["x"])
    for rank in range(P):
        xin, blocks = OP.oned_partition(rank, P, x, adj, True, replication=c)
        assert np.array_equal(xin.numpy(), pg[f"p15d_P{P}c{c}_r{rank}_inputs"])
        for b, (idx, val, nr, nc) in enumerate(blocks):
            assert np.array_equal(idx.numpy(), pg[f"p15d_P{P}c{c}_r{rank}_b{b}_idx"])
            assert np.array_equal(val.numpy(), pg[f"p15d_P{P}c{c}_r{rank}_b{b}_val"])
            assert [nr, nc] == pg[f"p15d_P{P}c{c}_r{rank}_b{b}_size"].tolist()


@pytest.mark.parametrize("P", [4, 9])
def test_twod_partition(pg, P):
    adj, x = _t(pg["adj_selfloops51"]), _t(pg["x51"])
    for rank in range(P):
        xin, (idx, val, nr, nc) = OP.twod_partition(rank, P, x, adj, True)
        assert np.array_equal(xin.numpy(), pg[f"p2d_P{P}_r{rank}_inputs"])
        assert np.array_equal(idx.numpy(), pg[f"p2d_P{P}_r{rank}_idx"])
        assert np.array_equal(val.numpy(), pg[f"p2d_P{P}_r{rank}_val"])
        assert [nr, nc] == pg[f"p2d_P{P}_r{rank}_size"].tolist()


def test_threed_partition(pg):
    edge, x = _t(pg["edge_index51"]), _t(pg["x51"])
    for rank in range(8):
        xin, (idx, val, nr, nc) = OP.threed_partition(rank, 8, x, edge)
        assert np.array_equal(xin.numpy(), pg[f"p3d_P8_r{rank}_inputs"])
        assert np.array_equal(idx.numpy(), pg[f"p3d_P8_r{rank}_idx"])
        assert np.array_equal(val.numpy(), pg[f"p3d_P8_r{rank}_val"])
        assert [nr, nc] == pg[f"p3d_P8_r{rank}_size"].tolist()


def test_process_groups(pg):
    for P, c in ((4, 2), (8, 2), (8, 4)):
        rows, cols = OP.proc_groups_15d(P, c)
        assert rows == pg[f"groups15d_P{P}c{c}_rows"].tolist() and cols == pg[f"groups15d_P{P}c{c}_cols"].tolist()
    for P in (4, 9):
        rows, cols = OP.proc_groups_2d(P)
        assert rows == pg[f"groups2d_P{P}_rows"].tolist() and cols == pg[f"groups2d_P{P}_cols"].tolist()
    rows, cols, fibers = OP.proc_groups_3d(8)
    assert rows == pg["groups3d_P8_rows"].tolist()
    assert cols == pg["groups3d_P8_cols"].tolist()
    assert fibers == pg["groups3d_P8_c"].tolist()


def test_coo2csr_and_spmm_definitions():
    g = torch.Generator().manual_seed(5)
    n, m, f = 37, 29, 5
    dense = (torch.rand(n, m, generator=g) < 0.2).float() * torch.randn(n, m, generator=g)
    dense[7] = 0          # an empty row
    sp = dense.to_sparse().coalesce()
    rows, cols, vals = sp.indices()[0], sp.indices()[1], sp.values()
    rowptr = OG.coo2csr(rows.numpy(), n)
    assert rowptr[0] == 0 and rowptr[-1] == vals.numel() and rowptr[7] == rowptr[8]
    assert np.array_equal(np.diff(rowptr), np.bincount(rows.numpy(), minlength=n))
    B = torch.randn(m, f, generator=g)
    C0 = torch.randn(n, f, generator=g)
    want = C0 + dense @ B
    got = OG.spmm_acc(rows, cols, vals, n, m, B, C0.clone())
    assert torch.allclose(got, want, atol=1e-5)
    loop = OG.spmm_rowloop(rowptr, cols.numpy(), vals.numpy(), B, C0, 1.0)
    assert torch.allclose(loop, want, atol=1e-5)


# ------------------------------------------------------------------------------------------ training
def _load_train(golden_dir, name):
    d = np.load(os.path.join(golden_dir, name))
    n, f, mid, classes, epochs, P, c, norm, act = d["cfg"].tolist()
    return d, dict(n=n, f=f, mid=mid, classes=classes, epochs=epochs, P=P, c=c, norm=bool(norm), act=bool(act))


def _check_epochs(d, cfg, records, out_slices, tol=2e-5):
    for ep, r in enumerate(records):
        for rank, (rs, cs) in enumerate(out_slices):
            want = d[f"r{rank}_ep{ep}_out"]
            got = r["out"][rs, cs].numpy()
            assert got.shape == want.shape
            np.testing.assert_allclose(got, want, rtol=1e-4, atol=tol, err_msg=f"out ep{ep} rank{rank}")
        np.testing.assert_allclose(r["gW1"].numpy(), d[f"r0_ep{ep}_gw1"], rtol=1e-4, atol=tol, err_msg=f"gW1 ep{ep}")
        np.testing.assert_allclose(r["gW2"].numpy(), d[f"r0_ep{ep}_gw2"], rtol=1e-4, atol=tol, err_msg=f"gW2 ep{ep}")
        np.testing.assert_allclose(r["W1"].numpy(), d[f"r0_ep{ep}_w1"], rtol=1e-4, atol=tol)
        np.testing.assert_allclose(r["W2"].numpy(), d[f"r0_ep{ep}_w2"], rtol=1e-4, atol=tol)


@pytest.mark.parametrize("name", ["train_1d_P1.npz", "train_1d_P3.npz", "train_1d_P1_plain.npz",
                                  "train_15d_P4.npz", "train_15d_P8.npz"])
def test_train_1d_15d(golden_dir, name):
    d, cfg = _load_train(golden_dir, name)
    edge, x, y, mask = (_t(d[k]) for k in ("edge_index", "x", "y", "mask"))
    n = cfg["n"]
    adj = OP.add_self_loops(edge, n) if cfg["norm"] else edge
    M = OG.matrix_1d(adj, x, cfg["P"], cfg["norm"], cfg["c"])
    n_per = math.ceil(n / (cfg["P"] / cfg["c"]))
    rule = lambda y_, m_: (lambda out: OG.grad_local_mean(out, y_, m_, n_per))
    rec = OG.train(M, x, y, mask, cfg["mid"], cfg["classes"], cfg["epochs"], rule, cfg["act"])
    slices = []
    for rank in range(cfg["P"]):
        rc = rank // cfg["c"]
        slices.append((slice(rc * n_per, min(n, (rc + 1) * n_per)), slice(None)))
    _check_epochs(d, cfg, rec, slices)


def test_train_2d(golden_dir):
    d, cfg = _load_train(golden_dir, "train_2d_P4.npz")
    edge, x, y, mask = (_t(d[k]) for k in ("edge_index", "x", "y", "mask"))
    n, P = cfg["n"], cfg["P"]
    adj = OP.add_self_loops(edge, n)
    M = OG.matrix_2d(adj, x, P, True)
    chunks, ranges = OG.row_chunks_2d(n, P), OG.class_ranges_2d(cfg["classes"], P)
    rule = lambda y_, m_: (lambda out: OG.grad_global_mean(out, y_, m_, chunks, ranges))
    rec = OG.train(M, x, y, mask, cfg["mid"], cfg["classes"], cfg["epochs"], rule, True)
    q = OP.grid_side_2d(P)
    vtx = OP.boundaries(n, n // q, keep=q)
    cs = np.cumsum([0] + OP.chunk_sizes(cfg["classes"], q)).tolist()
    slices = [(slice(vtx[r // q], vtx[r // q + 1]), slice(cs[r % q], cs[r % q + 1])) for r in range(P)]
    _check_epochs(d, cfg, rec, slices)


def test_train_3d(golden_dir):
    d, cfg = _load_train(golden_dir, "train_3d_P8.npz")
    edge, x, y, mask = (_t(d[k]) for k in ("edge_index", "x", "y", "mask"))
    n, P = cfg["n"], cfg["P"]
    q = OP.grid_side_3d(P)
    M = torch.sparse_coo_tensor(edge, torch.ones(edge.size(1)), (n, n)).coalesce()   # unnormalised, no self loops
    chunks, ranges = OG.row_chunks_3d(n, P), OG.class_ranges_3d(cfg["classes"], P)
    rule = lambda y_, m_: (lambda out: OG.grad_global_mean(out, y_, m_, chunks, ranges))
    rec = OG.train(M, x, y, mask, cfg["mid"], cfg["classes"], cfg["epochs"], rule, activations=False)
    cs = np.cumsum([0] + OP.chunk_sizes(cfg["classes"], q)).tolist()
    slices = []
    for rank in range(P):
        i, j, k = OP.coords_3d(rank, q)
        row0, length, _ = chunks[i * q + k]
        slices.append((slice(row0, row0 + length), slice(cs[j], cs[j + 1])))
    _check_epochs(d, cfg, rec, slices, tol=2e-3)
