"""Seeded synthetic graphs and node data standing in for the datasets the reference loads from disk
(Reddit / Amazon / Protein are read at gcn_distr.py:729-785; none of their items is reproduced here).

Everything is plain torch and runs on whichever device is asked for, so the 115M-edge benchmark graph
is generated on the GPU in seconds while tests use the CPU.  A given (seed, device type) always yields
the same tensors; every consumer of one run shares the same tensors.
"""
import math

import torch

RMAT_ABCD = (0.57, 0.19, 0.19, 0.05)


def _gen(seed, device):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def _pairs_to_edge_index(keys, n):
    lo, hi = keys // n, keys % n
    return torch.stack([torch.cat([lo, hi]), torch.cat([hi, lo])])


def er_graph(n, avg_degree, seed=1, device="cpu"):
    """Erdos-Renyi-style undirected graph: n * avg_degree / 2 vertex pairs drawn uniformly, self pairs
    dropped, duplicates merged, both directions listed.  Returns a 2 x E int64 edge list (no self loops)."""
    g = _gen(seed, device)
    m = n * avg_degree // 2
    u = torch.randint(0, n, (m,), generator=g, device=device)
    v = torch.randint(0, n, (m,), generator=g, device=device)
    keep = u != v
    u, v = u[keep], v[keep]
    keys = torch.unique(torch.minimum(u, v) * n + torch.maximum(u, v))
    return _pairs_to_edge_index(keys, n)


def _rmat_sample(count, scale, n, g, device, abcd):
    a, b, c, _ = abcd
    rows = torch.zeros(count, dtype=torch.int64, device=device)
    cols = torch.zeros(count, dtype=torch.int64, device=device)
    for _level in range(scale):
        r = torch.rand(count, generator=g, device=device)
        row_bit = r >= (a + b)
        col_bit = ((r >= a) & (r < a + b)) | (r >= a + b + c)
        rows = rows * 2 + row_bit
        cols = cols * 2 + col_bit
    keep = (rows < n) & (cols < n) & (rows != cols)
    rows, cols = rows[keep], cols[keep]
    return torch.minimum(rows, cols) * n + torch.maximum(rows, cols)


def rmat_graph(n, target_nnz=None, edge_factor=None, seed=1, device="cpu", abcd=RMAT_ABCD, chunk=1 << 24,
               permute=True):
    """R-MAT graph on n vertices (scale = ceil(log2 n); endpoints >= n rejected), symmetrised, duplicates
    merged, self loops dropped.  Either `edge_factor` (sample edge_factor * n directed edges once, the
    Graph500 convention) or `target_nnz`: sampling is topped up until the matrix the GCN uses
    (2 * pairs + n self loops) has target_nnz nonzeros to within 0.5 % from below.
    With `permute` the vertex labels are shuffled by a seeded random permutation, as Graph500 generators do:
    raw R-MAT puts every hub at a low index, which no real dataset does and which would make contiguous
    block rows wildly unequal.  Returns a 2 x E int64 edge list (both directions, no self loops)."""
    g = _gen(seed, device)
    scale = max(1, math.ceil(math.log2(n)))
    perm = torch.randperm(n, generator=g, device=device) if permute else None

    def relabel(keys):
        if perm is None:
            return keys
        a, b = perm[keys // n], perm[keys % n]
        return torch.unique(torch.minimum(a, b) * n + torch.maximum(a, b))

    def sample(count):
        parts = []
        while count > 0:
            take = min(count, chunk)
            parts.append(_rmat_sample(take, scale, n, g, device, abcd))
            count -= take
        return torch.cat(parts) if len(parts) > 1 else parts[0]

    if target_nnz is None:
        keys = torch.unique(sample(int(edge_factor * n)))
        return _pairs_to_edge_index(relabel(keys), n)
    want = (target_nnz - n) // 2
    keys = torch.empty(0, dtype=torch.int64, device=device)
    yield_est = 1.0
    for _round in range(64):
        need = want - keys.numel()
        if need <= 0.005 * want:
            break
        batch = int(need / max(yield_est, 0.02)) + 1
        before = keys.numel()
        keys = torch.unique(torch.cat([keys, sample(batch)]))
        # pairs gained per sample drawn; it only falls as the graph fills up, so this never overshoots by much
        yield_est = max((keys.numel() - before) / batch, 1e-3) * 0.9
    return _pairs_to_edge_index(relabel(keys), n)


def node_data(n, features, classes, train_fraction=1.0, seed_features=2, seed_labels=3, device="cpu"):
    """fp32 N(0,1) features, uniform int64 labels, bool train mask (Bernoulli(train_fraction), or all true)."""
    x = torch.randn(n, features, generator=_gen(seed_features, device), device=device)
    g = _gen(seed_labels, device)
    y = torch.randint(0, classes, (n,), generator=g, device=device)
    if train_fraction >= 1.0:
        mask = torch.ones(n, dtype=torch.bool, device=device)
    else:
        mask = torch.rand(n, generator=g, device=device) < train_fraction
    return x, y, mask


def add_self_loops(edge_index, n):
    """What `--normalization=True` does to the edge list before partitioning (gcn_distr.py:790-791):
    existing self loops dropped, one (i, i) per vertex appended."""
    keep = edge_index[0] != edge_index[1]
    loops = torch.arange(n, dtype=edge_index.dtype, device=edge_index.device).unsqueeze(0).repeat(2, 1)
    return torch.cat([edge_index[:, keep], loops], dim=1)
