"""Oracle restatement of the reference's native op and of one training epoch of each algorithm.

Single process, whole graph, explicit forward/backward formulas (no autograd through the layers), fp32
with an optional fp64 mode to bound reordered-summation error.  Test infrastructure only.
"""
import math

import numpy as np
import torch

from . import partition as P


# ------------------------------------------------------------------------------------------ native op
def coo2csr(rows, n):
    """cusparseXcoo2csr semantics (sparse_coo_tensor.cu:137-142): rowptr[i] = #{e : rows[e] < i}."""
    rows = np.asarray(rows)
    return np.searchsorted(rows, np.arange(n + 1), side="left").astype(np.int32)


def spmm_acc(rows, cols, vals, n, m, B, C):
    """`spmm_gpu` value semantics (sparse_coo_tensor.cu:149-150, 215-226): C += A.B in place, alpha = beta = 1.
    COO through torch.sparse.mm, the reference-faithful CPU form."""
    A = torch.sparse_coo_tensor(torch.stack([rows.long(), cols.long()]), vals.to(B.dtype), (n, m))
    C.add_(torch.sparse.mm(A, B))
    return C


def spmm_rowloop(rowptr, col, val, B, C, beta):
    """Pure-Python row loop (small cases only): the definition, independent of torch.sparse."""
    out = C.clone() if beta else torch.zeros_like(C)
    for r in range(len(rowptr) - 1):
        for e in range(int(rowptr[r]), int(rowptr[r + 1])):
            out[r] += float(val[e]) * B[int(col[e])]
    return out


# ------------------------------------------------------------------------------------------ assembling M
def assemble(blocks_per_rank, row_starts, col_starts, n, dtype=torch.float32):
    """Global matrix from per-rank block lists: M[row_starts[r] + i, col_starts[b] + j] = blocks[r][b][i, j]."""
    idx, val = [], []
    for r, blocks in enumerate(blocks_per_rank):
        for b, (bi, bv, _nr, _nc) in enumerate(blocks):
            idx.append(torch.stack([bi[0] + row_starts[r], bi[1] + col_starts[b]]))
            val.append(bv)
    return torch.sparse_coo_tensor(torch.cat(idx, 1), torch.cat(val).to(dtype), (n, n)).coalesce()


def matrix_1d(adj, inputs, size, normalization=True, replication=1, dtype=torch.float32):
    """The matrix the 1D / 1.5D loop multiplies by, assembled from the stored (transposed) blocks:
    Z_r = sum_i blocks_r[i] . X_i (gcn_distr.py:221-240)."""
    n = inputs.size(0)
    rows_of = size // replication
    n_per = math.ceil(float(n) / (size / replication))
    starts = list(range(0, n, n_per))
    per_rank = [P.oned_partition(rc * replication, size, inputs, adj, normalization, replication)[1]
                for rc in range(rows_of)]
    return assemble(per_rank, starts, starts, n, dtype)


def matrix_2d(adj, inputs, size, normalization=True, dtype=torch.float32):
    n = inputs.size(0)
    q = P.grid_side_2d(size)
    starts = P.boundaries(n, n // q, keep=q)[:-1]
    per_row = []
    for i in range(q):
        per_row.append([P.twod_partition(i * q + j, size, inputs, adj, normalization)[1] for j in range(q)])
    return assemble(per_row, starts, starts, n, dtype)


# ------------------------------------------------------------------------------------------ loss rules
def grad_local_mean(out, y, mask, n_per_proc):
    """1D / 1.5D (gcn_distr.py:347-362): every block row takes the mean NLL over ITS OWN train rows and
    the weight gradients of the block rows are summed, so dL/d out[i, y_i] = -1/count(block of i)."""
    n = out.size(0)
    G = torch.zeros_like(out)
    loss = out.new_zeros(())
    for lo in range(0, n, n_per_proc):
        hi = min(n, lo + n_per_proc)
        m = mask[lo:hi]
        cnt = int(m.sum())
        if cnt == 0:
            continue
        rows = torch.nonzero(m).squeeze(1) + lo
        G[rows, y[rows]] = -1.0 / cnt
        loss = loss + (-out[rows, y[rows]].sum() / cnt)
    return G, loss


def grad_global_mean(out, y, mask, row_chunks, class_ranges):
    """2D (gcn_distr_2d.py:942-989) and 3D (gcn_distr_3d.py:1080-1122): sum of out[., label] over train rows
    divided by the GLOBAL train count.  Reference quirks reproduced (all vanish for an all-true mask and
    equal chunk sizes):
      * labels and mask of a row chunk with L local rows and chunk index ci are taken as
        split(., L)[ci], i.e. vertices [ci L, ci L + L) -- shifted when L differs between chunks;
      * the labels are first compressed to the train rows (`datay_rank[rank_train_mask]`) and the
        position p in that compressed list is then used as the OUTPUT row (`outputs.index_select(0,
        indices)`, gcn_distr_2d.py:962-973), so with a partial mask label p is paired with local row p;
      * a class range only contributes labels inside it (2D drops the remainder classes of the last
        process column, gcn_distr_2d.py:949-952)."""
    n = out.size(0)
    count = float(mask.sum())
    G = torch.zeros_like(out)
    for (row0, length, ci) in row_chunks:
        lab0 = ci * length
        lab1 = min(n, lab0 + length)
        if lab0 >= n:
            continue
        m = mask[lab0:lab1]
        if int(m.sum()) == 0:
            continue
        compressed = y[lab0:lab1][m]
        for p, label in enumerate(compressed.tolist()):
            if any(lo <= label < hi for lo, hi in class_ranges):
                G[row0 + p, label] += -1.0 / count
    return G


def row_chunks_2d(n, size):
    q = P.grid_side_2d(size)
    vtx = P.boundaries(n, n // q, keep=q)
    return [(vtx[r], vtx[r + 1] - vtx[r], r) for r in range(q)]


def class_ranges_2d(classes, size):
    q = P.grid_side_2d(size)
    per = classes // q
    return [(j * per, min((j + 1) * per, classes)) for j in range(q)]     # sic: no remainder on the last


def row_chunks_3d(n, size):
    q = P.grid_side_3d(size)
    vtx = P.boundaries(n, n // q, keep=q)
    chunks = []
    for i in range(q):
        sizes = P.chunk_sizes(vtx[i + 1] - vtx[i], q)
        start = vtx[i]
        for k in range(q):
            chunks.append((start, sizes[k], i * q + k))
            start += sizes[k]
    return chunks


def class_ranges_3d(classes, size):
    q = P.grid_side_3d(size)
    per = classes // q
    return [(j * per, classes if j == q - 1 else (j + 1) * per) for j in range(q)]


# ------------------------------------------------------------------------------------------ epoch
def _act(z, kind):
    if kind == "relu":
        return torch.relu(z)
    if kind == "log_softmax":
        return torch.log_softmax(z, dim=1)
    return z


def _act_bwd(z, out, g, kind):
    if kind == "relu":
        return g * (z > 0).to(g.dtype)
    if kind == "log_softmax":
        return g - torch.exp(out) * g.sum(dim=1, keepdim=True)
    return g


def epoch(M, X, W1, W2, grad_rule, activations=True):
    """One epoch of the 2-layer GCN exactly as GCNFunc composes it (gcn_distr.py:250-339):
         T = M.H ; Z = T.W ; H' = act(Z)
         dZ = act'(Z) * G ; AG = M.dZ ; grad_H = AG.W^T ; grad_W = H^T.AG
    (backward multiplies by the same stored blocks as forward, gcn_distr.py:326).
    grad_rule(out2) -> (G, loss) or G.  Returns dict(out, gW1, gW2, loss)."""
    a1, a2 = ("relu", "log_softmax") if activations else (None, None)
    T1 = torch.sparse.mm(M, X)
    Z1 = T1 @ W1
    H1 = _act(Z1, a1)
    T2 = torch.sparse.mm(M, H1)
    Z2 = T2 @ W2
    out = _act(Z2, a2)
    res = grad_rule(out)
    G, loss = res if isinstance(res, tuple) else (res, None)
    dZ2 = _act_bwd(Z2, out, G, a2)
    AG2 = torch.sparse.mm(M, dZ2)
    gH1 = AG2 @ W2.t()
    gW2 = H1.t() @ AG2
    dZ1 = _act_bwd(Z1, H1, gH1, a1)
    AG1 = torch.sparse.mm(M, dZ1)
    gW1 = X.t() @ AG1
    return dict(out=out, gW1=gW1, gW2=gW2, loss=loss, H1=H1)


def init_weights(features, mid, classes, dtype=torch.float32):
    """gcn_distr.py:550-555: torch.manual_seed(0); rand(features, mid); rand(mid, classes) on the CPU."""
    torch.manual_seed(0)
    w1 = torch.rand(features, mid)
    w2 = torch.rand(mid, classes)
    return w1.to(dtype), w2.to(dtype)


def train(M, X, y, mask, mid, classes, epochs, grad_rule_factory, activations=True, dtype=torch.float32):
    """Epoch loop with Adam(lr = 0.01) (gcn_distr.py:562, 364).  Returns the per-epoch records."""
    X = X.to(dtype)
    M = M.to(dtype)
    w1, w2 = init_weights(X.size(1), mid, classes, dtype)
    w1 = torch.nn.Parameter(w1)
    w2 = torch.nn.Parameter(w2)
    opt = torch.optim.Adam([w1, w2], lr=0.01)
    records = []
    for _ in range(epochs):
        with torch.no_grad():
            r = epoch(M, X, w1.data, w2.data, grad_rule_factory(y, mask), activations)
        opt.zero_grad()
        w1.grad, w2.grad = r["gW1"].clone(), r["gW2"].clone()
        opt.step()
        r["W1"], r["W2"] = w1.detach().clone(), w2.detach().clone()
        records.append(r)
    return records
