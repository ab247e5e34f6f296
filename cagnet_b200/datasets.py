"""`--graphname` resolution.  The reference loads Cora / Reddit through PyG and Amazon / Protein (subgraph3)
from `.pt` edge lists on disk (gcn_distr.py:717-785); none of that data is available offline, so every
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

No item of any public dataset is reproduced.
"""
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
        opts[k.strip()] = float(v) if "." in v else int(v)
    if kind not in ("er", "rmat"):
        raise ValueError("graph kind must be er or rmat, got %r" % kind)
    if "scale" in opts:
        opts["n"] = 1 << int(opts["scale"])
    for key in ("n", "f", "c"):
        if key not in opts:
            raise ValueError("graph spec %r lacks %s=" % (spec, key))
    return kind, opts


def load(graphname, device="cpu", seed=1):
    """-> (inputs n x f fp32, edge_index 2 x E int64 without self loops, Data(y, train_mask), f, classes, info)."""
    kind, o = parse_spec(graphname)
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
