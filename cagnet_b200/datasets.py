"""`--graphname` resolution.  The reference loads Cora / Reddit through PyG and Amazon / Protein (subgraph3)
from `.pt` edge lists on disk (gcn_distr.py:717-785).  No dataset ships with this package, so every
name resolves to a SEEDED SYNTHETIC graph with the shape the reference hard-codes for it:

    Cora       2,708 vertices, 1,433 features, 7 classes    (Erdos-Renyi, avg degree 4)
    Reddit     232,965 vertices, 602 features, 41 classes   (R-MAT, ~114.6 M nonzeros, 66 % train mask)
    Amazon     14,249,639 vertices, 300 features, 24 classes (R-MAT, ~230.8 M nonzeros)
    subgraph3  8,745,542 vertices, 128 features, 256 classes (R-MAT, ~1.31 B nonzeros)
    subgraph5  2,186,385 vertices, 128 features, 256 classes (R-MAT, edge factor 16)

plus explicit specs, comma separated `key=value` after a kind:

    er:n=16384,deg=16,f=128,c=8
    rmat:n=232965,nnz=114600000,f=602,c=41,train=0.66
    rmat:scale=20,ef=16,f=64,c=16

and two kinds that read the reference's ON-DISK formats when the user has the files:

    file:path=/data/Amazon/processed/data.pt,n=14249639,f=300,c=24
        a torch-saved (or .npy) 2 x E integer edge list, as the Amazon and subgraph3 branches read it
        (gcn_distr.py:747, 771); features, labels and the all-ones train mask are random as they are there
        (gcn_distr.py:752-756), but seeded.  `n` defaults to the largest vertex id + 1.
    npz:dir=/data/Reddit/raw
        the two raw files the reference's Reddit class processes (reddit.py:33-34, 49-66): `reddit_data.npz`
        with `feature`, `label`, `node_types` (1 / 2 / 3 = train / validation / test) and `reddit_graph.npz`,
        a scipy sparse matrix; the edge list is coalesced (sorted, duplicates dropped) as it is there.

No item of any public dataset is reproduced.
"""
import os

import torch

from . import graphs
from .dist1d import Data

NAMED = {
    "Cora": "er:n=2708,deg=4,f=1433,c=7,train=0.3",
    "Reddit": "rmat:n=232965,nnz=114600000,f=602,c=41,train=0.66",
    "Amazon": "rmat:n=14249639,nnz=230800000,f=300,c=24",
    "subgraph3": "rmat:n=8745542,nnz=1310000000,f=128,c=256",
    "subgraph5": "rmat:n=2186385,ef=16,f=128,c=256",
}


def parse_spec(graphname):
    spec = NAMED.get(graphname, graphname)
    if ":" not in spec:
        raise ValueError("unknown graph name %r (known: %s, or er:/rmat: specs)" % (graphname, ", ".join(NAMED)))
    kind, _, rest = spec.partition(":")
    opts = {}
    for item in filter(None, rest.split(",")):
        k, _, v = item.partition("=")
        opts[k.strip()] = _value(k.strip(), v)
    if kind not in ("er", "rmat", "file", "npz"):
        raise ValueError("graph kind must be er, rmat, file or npz, got %r" % kind)
    if "scale" in opts:
        opts["n"] = 1 << int(opts["scale"])
    required = {"er": ("n", "f", "c"), "rmat": ("n", "f", "c"), "file": ("path", "f", "c"), "npz": ("dir",)}[kind]
    for key in required:
        if key not in opts:
            raise ValueError("graph spec %r lacks %s=" % (spec, key))
    return kind, opts


def _value(key, text):
    if key in ("path", "dir"):
        return text
    try:
        return int(text)
    except ValueError:
        return float(text)


def read_edge_list(path, n=None):
    """A 2 x E (or E x 2) integer edge list saved by `torch.save` or `numpy.save` -> (2 x E int64, n).  Vertex
    ids outside [0, n) are an error here rather than an out-of-range gather on the device later."""
    if not os.path.isfile(path):
        raise FileNotFoundError("edge list %r not found" % path)
    if path.endswith(".npy"):
        import numpy as np
        edge_index = torch.from_numpy(np.load(path))
    else:
        edge_index = torch.load(path, map_location="cpu", weights_only=True)
    if not torch.is_tensor(edge_index) or edge_index.dim() != 2 or 2 not in edge_index.shape \
            or edge_index.is_floating_point():
        raise ValueError("%r does not hold a 2 x E integer edge list" % path)
    if edge_index.size(0) != 2:
        edge_index = edge_index.t()
    edge_index = edge_index.to(torch.int64).contiguous()
    top = int(edge_index.max()) + 1 if edge_index.numel() else 0
    if n is None:
        n = top
    if top > n or (edge_index.numel() and int(edge_index.min()) < 0):
        raise ValueError("%r names vertices outside [0, %d)" % (path, n))
    return edge_index, n


def read_reddit_npz(directory):
    """-> (x fp32, edge_index 2 x E int64 sorted by (row, col) without duplicates, y int64, train / val / test
    bool masks) from `reddit_data.npz` and `reddit_graph.npz` (reddit.py:49-66)."""
    import numpy as np
    import scipy.sparse as sp
    nodes = np.load(os.path.join(directory, "reddit_data.npz"))
    x = torch.from_numpy(np.asarray(nodes["feature"])).to(torch.float32)
    y = torch.from_numpy(np.asarray(nodes["label"])).to(torch.int64)
    split = torch.from_numpy(np.asarray(nodes["node_types"]))
    n = x.size(0)
    adj = sp.load_npz(os.path.join(directory, "reddit_graph.npz")).tocoo()
    if adj.shape[0] != n or adj.shape[1] != n:
        raise ValueError("reddit_graph.npz is %s, the features have %d rows" % (adj.shape, n))
    keys = torch.from_numpy(adj.row.astype(np.int64)) * n + torch.from_numpy(adj.col.astype(np.int64))
    keys = torch.unique(keys)                      # sorted: row-major order, one entry per (row, col)
    edge_index = torch.stack([keys // n, keys % n])
    return x, edge_index, y, split == 1, split == 2, split == 3


def load(graphname, device="cpu", seed=1):
    """-> (inputs n x f fp32, edge_index 2 x E int64 without self loops, Data(y, train_mask), f, classes, info)."""
    kind, o = parse_spec(graphname)
    if kind == "npz":
        x, edge_index, y, train, val, test = read_reddit_npz(o["dir"])
        n, f = x.shape
        classes = int(o.get("c", int(y.max()) + 1))
        info = dict(kind=kind, n=n, features=f, classes=classes, edges=int(edge_index.size(1)),
                    nnz_with_self_loops=int((edge_index[0] != edge_index[1]).sum()) + n,
                    train_fraction=float(train.float().mean()), seed=None)
        data = Data(y=y, train_mask=train, val_mask=val, test_mask=test).to(device)
        return x.to(device), edge_index.to(device), data, f, classes, info
    if kind == "file":
        edge_index, n = read_edge_list(o["path"], o.get("n"))
        f, classes = int(o["f"]), int(o["c"])
        g = torch.Generator().manual_seed(seed + 1)
        x = torch.rand(n, f, generator=g)
        y = torch.randint(0, max(classes - 1, 1), (n,), generator=g)      # uniform_(0, c - 1).long(): never c - 1
        info = dict(kind=kind, n=n, features=f, classes=classes, edges=int(edge_index.size(1)),
                    nnz_with_self_loops=int((edge_index[0] != edge_index[1]).sum()) + n, train_fraction=1.0, seed=seed)
        data = Data(y=y, train_mask=torch.ones(n, dtype=torch.bool)).to(device)
        return x.to(device), edge_index.to(device), data, f, classes, info
    n, f, classes = int(o["n"]), int(o["f"]), int(o["c"])
    if kind == "er":
        edge_index = graphs.er_graph(n, int(o.get("deg", 16)), seed=seed, device=device)
    elif "nnz" in o:
        edge_index = graphs.rmat_graph(n, target_nnz=int(o["nnz"]), seed=seed, device=device)
    else:
        edge_index = graphs.rmat_graph(n, edge_factor=o.get("ef", 16), seed=seed, device=device)
    x, y, mask = graphs.node_data(n, f, classes, float(o.get("train", 1.0)), seed + 1, seed + 2, device=device)
    info = dict(kind=kind, n=n, features=f, classes=classes, edges=int(edge_index.size(1)),
                nnz_with_self_loops=int(edge_index.size(1)) + n, train_fraction=float(o.get("train", 1.0)), seed=seed)
    return x, edge_index, Data(y=y, train_mask=mask), f, classes, info
