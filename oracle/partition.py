"""Oracle restatement of the reference's CPU partitioners, normalisation and communicator layouts.

Written for clarity, not speed: boolean scans over the whole edge list, exactly the quantities the
reference computes, in the same order.  Test infrastructure only.
"""
import math

import torch


# ------------------------------------------------------------------------------------------ helpers
def add_self_loops(edge_index, n):
    """PyG 1.3.2 `add_remaining_self_loops` as the reference calls it (gcn_distr.py:790-791): existing
    self loops are dropped, the other edges keep their order, one (i, i) per vertex is appended."""
    keep = edge_index[0] != edge_index[1]
    loops = torch.arange(n, dtype=edge_index.dtype).unsqueeze(0).repeat(2, 1)
    return torch.cat([edge_index[:, keep], loops], dim=1)


def boundaries(node_count, n_per_proc, keep=None):
    """`vtx_indices` of split_coo: 0, n_per_proc, 2 n_per_proc, ... (< node_count), then node_count.
    1D/1.5D keep every start (gcn_distr.py:399-400); 2D keeps the first proc_row starts
    (gcn_distr_2d.py:1036-1038), 3D the first proc_c (gcn_distr_3d.py:1168-1170)."""
    starts = list(range(0, node_count, n_per_proc))
    if keep is not None:
        starts = starts[:keep]
    return starts + [node_count]


def split_coo(adj, node_count, n_per_proc, dim, keep=None):
    """gcn_distr.py:398-409: for each boundary pair select the entries whose `dim` index lies in
    [lo, hi), preserving order, and rebase that index by lo.  `adj` is a 2 x E int64 tensor."""
    vtx = boundaries(node_count, n_per_proc, keep)
    parts = []
    for lo, hi in zip(vtx[:-1], vtx[1:]):
        sel = adj[:, adj[dim] >= lo]
        sel = sel[:, sel[dim] < hi].clone()
        sel[dim] -= lo
        parts.append(sel)
    return parts, vtx


def inv_sqrt_degree(adj_full, node_count):
    """gcn_distr.py:440-441: deg = histc(rows as double, bins = n) ** -0.5 (fp64)."""
    deg = torch.histc(adj_full[0].double(), bins=node_count)
    return deg.pow(-0.5)


def scale_block(adj_full, indices, n_rows, n_cols, node_count, row_vtx, col_vtx, normalization=True):
    """gcn_distr.py:412-470.  The block has unit values; the two diagonal products give every entry
    exactly fl32( fl32(d[r]) * fl32(d[c]) ) with d = deg^-1/2 taken in fp64.  Returns the coalesced
    block as (indices 2 x nnz int64 sorted by row then column, values fp32)."""
    blk = torch.sparse_coo_tensor(indices, torch.ones(indices.size(1)), size=(n_rows, n_cols)).coalesce()
    idx, val = blk.indices(), blk.values()
    if not normalization:
        return idx, val
    d = inv_sqrt_degree(adj_full, node_count)
    d_left = d[row_vtx:row_vtx + n_rows].float()
    d_right = d[col_vtx:col_vtx + n_cols].float()
    right = val * d_right[idx[1]]          # (A . D_right): one fp32 product per entry
    return idx, d_left[idx[0]] * right     # (D_left . that): one more


def transpose_coalesce(idx, val, n_rows, n_cols):
    """`am_pbyp[i].t().coalesce()` (gcn_distr.py:546): swap the index rows and re-sort."""
    t = torch.sparse_coo_tensor(torch.stack([idx[1], idx[0]]), val, size=(n_cols, n_rows)).coalesce()
    return t.indices(), t.values()


# ------------------------------------------------------------------------------------------ 1D / 1.5D
def oned_partition(rank, size, inputs, adj, normalization=True, replication=1):
    """gcn_distr.py:472-522 (replication = 1) and gcn_distr_15d.py:497-549.

    Returns (inputs_loc, blocks) where blocks[i] = (idx, val, n_rows, n_cols) is the block the
    training loop multiplies by H_i: the TRANSPOSED, coalesced am_pbyp[i]."""
    n = inputs.size(0)
    rows_of = size // replication
    n_per_proc = math.ceil(float(n) / (size / replication))
    rank_c = rank // replication
    col_parts, vtx = split_coo(adj, n, n_per_proc, 1)
    proc_node_count = vtx[rank_c + 1] - vtx[rank_c]
    row_parts, _ = split_coo(col_parts[rank_c], n, n_per_proc, 0)
    blocks = []
    for i, part in enumerate(row_parts):
        n_rows = vtx[i + 1] - vtx[i] if i == rows_of - 1 else n_per_proc
        idx, val = scale_block(adj, part, n_rows, proc_node_count, n, vtx[i], vtx[rank_c], normalization)
        tidx, tval = transpose_coalesce(idx, val, n_rows, proc_node_count)
        blocks.append((tidx, tval, proc_node_count, n_rows))
    inputs_loc = torch.split(inputs, n_per_proc, dim=0)[rank_c]
    return inputs_loc, blocks


def proc_groups_15d(size, replication):
    """gcn_distr_15d.py:398-419: row groups [i, i + c), column groups range(i, P, c)."""
    rows = [list(range(i, i + replication)) for i in range(0, size, replication)]
    cols = [list(range(i, size, replication)) for i in range(replication)]
    return rows, cols


def stages_15d(rank, size, replication):
    """gcn_distr_15d.py:194-208: the (source rank q, block id) pairs rank `rank` walks through."""
    rank_col = rank % replication
    per = size // (replication ** 2)
    stages = per
    if rank_col == replication - 1:
        stages = (size // replication) - (replication - 1) * per
    out = []
    for i in range(stages):
        q = (rank_col * per + i) * replication + rank_col
        out.append((q, rank_col * per + i))
    return out


# ------------------------------------------------------------------------------------------ 2D
def grid_side_2d(size):
    return math.floor(math.sqrt(size))          # gcn_distr_2d.py:1087-1091


def chunk_sizes(total, parts):
    """floor split with the remainder on the last part (gcn_distr_2d.py:1136-1149 and everywhere else)."""
    per = total // parts
    return [per] * (parts - 1) + [total - per * (parts - 1)]


def twod_partition(rank, size, inputs, adj, normalization=True, q=None):
    """gcn_distr_2d.py:1093-1164 (and gcn_distr_3d.py:1272-1339 with q = cbrt(P) and no scaling):
    block (rank_row, rank_col) of A, coalesced, NOT transposed; H block (rank_row, rank_col)."""
    n = inputs.size(0)
    q = grid_side_2d(size) if q is None else q
    n_per_proc = n // q
    rank_row, rank_col = rank // q, rank % q
    col_parts, vtx = split_coo(adj, n, n_per_proc, 1, keep=q)
    proc_node_count = vtx[rank_col + 1] - vtx[rank_col]
    row_parts, _ = split_coo(col_parts[rank_col], n, n_per_proc, 0, keep=q)
    n_rows = vtx[rank_row + 1] - vtx[rank_row] if rank_row == q - 1 else n_per_proc
    idx, val = scale_block(adj, row_parts[rank_row], n_rows, proc_node_count, n, vtx[rank_row], vtx[rank_col],
                           normalization)
    row_chunks = torch.split(inputs, chunk_sizes(n, q), dim=0)
    inputs_loc = torch.split(row_chunks[rank_row], chunk_sizes(inputs.size(1), q), dim=1)[rank_col]
    return inputs_loc, (idx, val, n_rows, proc_node_count)


def proc_groups_2d(size):
    """gcn_distr_2d.py:516-535."""
    q = grid_side_2d(size)
    rows = [list(range(i * q, i * q + q)) for i in range(q)]
    cols = [list(range(i, size, q)) for i in range(q)]
    return rows, cols


# ------------------------------------------------------------------------------------------ 3D
def grid_side_3d(size):
    c = int(size ** (1.0 / 3.0))                # gcn_distr_3d.py:1245-1270
    if c ** 3 == size:
        return c
    if (c + 1) ** 3 == size:
        return c + 1
    raise ValueError("3D needs a cubic process count")


def coords_3d(rank, q):
    """gcn_distr_3d.py:754-756: rank = i (q c) + j c + k."""
    return (rank // q) // q, (rank // q) % q, rank % q


def threed_partition(rank, size, inputs, adj):
    """gcn_distr_3d.py:1533-1542: the 2D block of the (i, j) pair, then its columns cut into c slabs and
    the H block's rows into c chunks (threed_partition_loc, gcn_distr_3d.py:1341-1382).  The script's
    `normalization` global is a constant False (gcn_distr_3d.py:66), so values stay 1."""
    q = grid_side_3d(size)
    i, j, k = coords_3d(rank, q)
    inputs_2d, (idx, val, n_rows, n_cols) = twod_partition(i * q + j, q * q, inputs, adj, normalization=False, q=q)
    per = n_cols // q
    slabs, vtx = split_coo(idx, n_cols, per, 1, keep=q)
    width = vtx[k + 1] - vtx[k] if k == q - 1 else per
    blk = torch.sparse_coo_tensor(slabs[k], torch.ones(slabs[k].size(1)), size=(n_rows, width)).coalesce()
    inputs_loc = torch.split(inputs_2d, chunk_sizes(inputs_2d.size(0), q), dim=0)[k]
    return inputs_loc, (blk.indices(), blk.values(), n_rows, width)


def proc_groups_3d(size):
    """gcn_distr_3d.py:629-672: row_groups[i][k], col_groups[j][k], c_groups[rank // c]."""
    q = grid_side_3d(size)
    rows = [[list(range(i * q * q + k, (i + 1) * q * q + k, q)) for k in range(q)] for i in range(q)]
    cols = [[list(range(j * q + k, q * q * q + j * q + k, q * q)) for k in range(q)] for j in range(q)]
    fibers = [list(range(i, i + q)) for i in range(0, size, q)]
    return rows, cols, fibers
