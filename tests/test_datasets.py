"""The two on-disk formats `--graphname` can read (the reference's Amazon / subgraph3 `.pt` edge lists,
gcn_distr.py:747, 771, and the raw Reddit pair of reddit.py:49-66), on small files written by the test."""
import numpy as np
import pytest
import scipy.sparse as sp
import torch

from cagnet_b200 import datasets, graphs


def _edges(n, e, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, n, (2, e), generator=g)


def test_edge_list_file(tmp_path):
    n, f, classes = 300, 7, 5
    edge_index = _edges(n, 2000, 3)
    path = tmp_path / "data.pt"
    torch.save(edge_index, str(path))
    spec = "file:path=%s,n=%d,f=%d,c=%d" % (path, n, f, classes)
    assert datasets.parse_spec(spec) == ("file", {"path": str(path), "n": n, "f": f, "c": classes})
    x, edge, data, f2, c2, info = datasets.load(spec, seed=4)
    assert torch.equal(edge, edge_index) and (f2, c2) == (f, classes)
    assert x.shape == (n, f) and x.dtype == torch.float32 and 0.0 <= float(x.min()) and float(x.max()) < 1.0
    assert data.y.dtype == torch.int64 and int(data.y.min()) >= 0 and int(data.y.max()) < classes - 1
    assert data.train_mask.dtype == torch.bool and bool(data.train_mask.all())
    assert info["edges"] == 2000 and info["n"] == n
    assert info["nnz_with_self_loops"] == graphs.add_self_loops(edge, n).size(1)
    # same seed, same features and labels; another seed, other features
    x2, _, data2, _, _, _ = datasets.load(spec, seed=4)
    x3, _, _, _, _, _ = datasets.load(spec, seed=5)
    assert torch.equal(x, x2) and torch.equal(data.y, data2.y) and not torch.equal(x, x3)


def test_edge_list_file_shapes_and_errors(tmp_path):
    edge_index = _edges(50, 400, 1)
    # E x 2 in a .npy file, n from the largest id
    np.save(str(tmp_path / "edges.npy"), edge_index.t().contiguous().numpy().astype(np.int32))
    edge, n = datasets.read_edge_list(str(tmp_path / "edges.npy"))
    assert torch.equal(edge, edge_index) and n == int(edge_index.max()) + 1 and edge.dtype == torch.int64
    with pytest.raises(ValueError, match="outside"):
        datasets.read_edge_list(str(tmp_path / "edges.npy"), n=10)
    torch.save(torch.rand(2, 5), str(tmp_path / "floats.pt"))
    with pytest.raises(ValueError, match="integer edge list"):
        datasets.read_edge_list(str(tmp_path / "floats.pt"))
    torch.save(torch.zeros(3, 5, dtype=torch.int64), str(tmp_path / "three.pt"))
    with pytest.raises(ValueError, match="integer edge list"):
        datasets.read_edge_list(str(tmp_path / "three.pt"))
    with pytest.raises(FileNotFoundError):
        datasets.read_edge_list(str(tmp_path / "absent.pt"))
    with pytest.raises(ValueError, match="lacks path="):
        datasets.parse_spec("file:n=5,f=2,c=2")


def test_raw_reddit_pair(tmp_path):
    n, f, classes = 120, 6, 4
    rng = np.random.default_rng(7)
    feature = rng.standard_normal((n, f))                       # float64 on disk, fp32 once loaded
    label = rng.integers(0, classes, n)
    node_types = rng.integers(1, 4, n)
    np.savez(str(tmp_path / "reddit_data.npz"), feature=feature, label=label, node_types=node_types)
    row = rng.integers(0, n, 900)
    col = rng.integers(0, n, 900)
    row, col = np.concatenate([row, row[:50]]), np.concatenate([col, col[:50]])      # 50 duplicates
    adj = sp.coo_matrix((np.ones(row.size), (row, col)), shape=(n, n))
    sp.save_npz(str(tmp_path / "reddit_graph.npz"), adj)

    x, edge, data, f2, c2, info = datasets.load("npz:dir=%s" % tmp_path)
    assert (f2, c2) == (f, int(label.max()) + 1) and x.dtype == torch.float32
    assert torch.allclose(x, torch.from_numpy(feature).float())
    assert torch.equal(data.y, torch.from_numpy(label).long())
    for name, kind in (("train_mask", 1), ("val_mask", 2), ("test_mask", 3)):
        assert torch.equal(getattr(data, name), torch.from_numpy(node_types == kind))
    # coalesced: the distinct (row, col) pairs in row-major order
    pairs = sorted(set(zip(row.tolist(), col.tolist())))
    assert edge.t().tolist() == [list(p) for p in pairs]
    assert info["edges"] == len(pairs) and info["n"] == n
    assert info["nnz_with_self_loops"] == graphs.add_self_loops(edge, n).size(1)

    # a graph whose side differs from the feature rows is refused
    sp.save_npz(str(tmp_path / "reddit_graph.npz"), sp.coo_matrix((n + 1, n + 1)))
    with pytest.raises(ValueError, match="features have"):
        datasets.load("npz:dir=%s" % tmp_path)


def test_loaded_graph_feeds_the_partitioner(tmp_path):
    """What a file yields goes through the same normalisation and 1D partition as a synthetic graph."""
    from cagnet_b200 import partition
    n = 64
    edge_index = _edges(n, 500, 9)
    torch.save(edge_index, str(tmp_path / "data.pt"))
    x, edge, data, f, classes, _ = datasets.load("file:path=%s,f=3,c=3" % (tmp_path / "data.pt"))
    n = x.size(0)
    adj = graphs.add_self_loops(edge, n)
    deg = partition.inv_sqrt_degree(adj, n)
    assert deg.shape == (n,) and bool(torch.isfinite(deg).all())


def _accuracy_worker(rank, world, directory):
    """The 1D driver on the raw Reddit pair, `--accuracy=True` (gcn_distr.py:654-661): returns what it printed and
    this rank's output rows."""
    from cagnet_b200 import datasets, dist1d, graphs
    from oracle.cpu_backend import CpuBackend
    x, edge, data, f, classes, _ = datasets.load("npz:dir=%s" % directory)
    adj = graphs.add_self_loops(edge, x.size(0))
    rt = dist1d.Runtime(CpuBackend(), True, True)
    lines = []
    model = dist1d.run(rank, world, x, adj, data, f, classes, rt, epochs=3, mid_layer=5, run_count=1, accuracy=True,
                       printer=lambda *a: lines.append(" ".join(str(v) for v in a)))
    return lines, model.outputs.detach().numpy().copy()


def test_accuracy_line_from_loaded_splits(tmp_path):
    """Train / validation / test accuracy of the driver's last line, computed from the splits the loader read,
    equals the accuracy of the assembled per-rank outputs over the same splits."""
    from tests.mp_util import run_ranks
    n, f, classes, world = 90, 5, 3, 3
    rng = np.random.default_rng(3)
    label = rng.integers(0, classes, n)
    node_types = rng.integers(1, 4, n)
    np.savez(str(tmp_path / "reddit_data.npz"), feature=rng.standard_normal((n, f)), label=label, node_types=node_types)
    row, col = rng.integers(0, n, 600), rng.integers(0, n, 600)
    both = sp.coo_matrix((np.ones(1200), (np.concatenate([row, col]), np.concatenate([col, row]))), shape=(n, n))
    sp.save_npz(str(tmp_path / "reddit_graph.npz"), both)

    results = run_ranks(world, _accuracy_worker, str(tmp_path))
    outputs = np.concatenate([results[r][1] for r in range(world)], axis=0)
    assert outputs.shape == (n, classes)
    pred = outputs.argmax(axis=1)
    want = [float((pred[node_types == k] == label[node_types == k]).mean()) for k in (1, 2, 3)]
    for lines, _ in results:
        last = [ln for ln in lines if ln.startswith("Epoch: 900")]
        assert len(last) == 1
        got = [float(part.split(":")[1]) for part in last[0].split(",")[1:]]
        assert got == pytest.approx(want, abs=1e-4)
