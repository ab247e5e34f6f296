"""Block partitioners, normalisation and communicator layouts of the four algorithms.

Same results as the reference's CPU partitioners (`split_coo`, `scale_elements`, `oned_partition`,
`twod_partition`, `threed_partition_loc`; gcn_distr.py:398-522, gcn_distr_2d.py:1032-1164,
gcn_distr_3d.py:1163-1382) -- indices bit-exact, values bit-exact fp32 -- but computed with one range
filter and one key sort per block instead of O(P) boolean scans of the whole edge list, in plain torch
on whichever device holds the edge list (the GPU for the large graphs).
"""
import math
from typing import NamedTuple, Optional

import torch
import torch.distributed as dist



class Block(NamedTuple):
    """Coalesced COO block, entries sorted by row then column.

    A normalised block also carries the two diagonal factors it was scaled with: vals[e] =
    row_scale[rows[e]] * (multiplicity[e] * col_scale[cols[e]]) exactly as computed here (one fp32 rounding per
    product).  The multiply can use that factorisation: the dense hub-by-hub core of such a block is an integer
    matrix between two diagonals (see ops.CsrBlock.extract_core)."""
    rows: torch.Tensor   # int64 [nnz]
    cols: torch.Tensor   # int64 [nnz]
    vals: torch.Tensor   # float32 [nnz]
    n_rows: int
    n_cols: int
    row_scale: Optional[torch.Tensor] = None   # float32 [n_rows]
    col_scale: Optional[torch.Tensor] = None   # float32 [n_cols]


# ------------------------------------------------------------------------------------------ pieces
def chunk_sizes(total, parts):
    """Floor split, remainder on the last part (gcn_distr_2d.py:1136-1149)."""
    per = total // parts
    return [per] * (parts - 1) + [total - per * (parts - 1)]


def boundaries(node_count, n_per_proc, keep=None):
    """Block starts 0, n_per_proc, ... then node_count; 2D/3D keep only the first `keep` starts
    (gcn_distr.py:399-400, gcn_distr_2d.py:1036-1038, gcn_distr_3d.py:1168-1170)."""
    starts = list(range(0, node_count, n_per_proc))
    if keep is not None:
        starts = starts[:keep]
    return starts + [node_count]


def inv_sqrt_degree(adj, node_count, group=None):
    """deg^-1/2 in fp64 then rounded to fp32, deg = occurrences as a row index in the whole edge list.
    The reference takes `histc(rows, bins=n)` (gcn_distr.py:440), which equals this count whenever
    vertices 0 and n-1 occur -- always the case once self loops are added.

    With `group` (a process group whose members all hold the same edge list in the same order and all make this
    call) every member counts its own 1/P slice of the list and one all-reduce of the int64 counts gives the
    degrees: the same integers as the reference's count over the whole list on every rank, at 1/P of the scan."""
    rows = adj[0]
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1 and \
            rows.is_cuda == (dist.get_backend(group) == "nccl"):      # NCCL reduces device tensors only, Gloo host ones
        size, rank = dist.get_world_size(group), dist.get_rank(group)
        per = -(-rows.numel() // size)
        deg = torch.bincount(rows[rank * per:(rank + 1) * per], minlength=node_count)
        dist.all_reduce(deg, group=group)
    else:
        deg = torch.bincount(rows, minlength=node_count)
    return deg.double().pow(-0.5).float()


def coalesce_block(r, c, n_rows, n_cols, d_row=None, d_col=None, row_first=False):
    """Entries (r, c) -> Block; duplicate entries add up (value = multiplicity) as `.coalesce()` does, then
    val = d_row[r] * (val * d_col[c]): the two diagonal products of scale_elements (gcn_distr.py:458-464),
    one fp32 rounding each.  `row_first` applies the row factor first, d_col[c] * (val * d_row[r]): the
    transposed block of a directed graph then holds bit for bit the values of the block it transposes."""
    key, counts = torch.unique(r * n_cols + c, return_counts=True)
    rows = torch.div(key, n_cols, rounding_mode="floor")
    cols = key - rows * n_cols
    vals = counts.to(torch.float32)
    if d_row is not None:
        vals = d_col[cols] * (vals * d_row[rows]) if row_first else d_row[rows] * (vals * d_col[cols])
        return Block(rows, cols, vals, int(n_rows), int(n_cols), d_row.contiguous(), d_col.contiguous())
    return Block(rows, cols, vals, int(n_rows), int(n_cols))


def fuse_columns(blocks):
    """[B0 | B1 | ...]: blocks with the same row count side by side as one coalesced block."""
    if len(blocks) == 1:
        return blocks[0]
    n_rows = blocks[0].n_rows
    offs = [0]
    for b in blocks:
        if b.n_rows != n_rows:
            raise ValueError("fuse_columns: blocks differ in row count")
        offs.append(offs[-1] + b.n_cols)
    rows = torch.cat([b.rows for b in blocks])
    cols = torch.cat([b.cols + o for b, o in zip(blocks, offs)])
    vals = torch.cat([b.vals for b in blocks])
    order = torch.argsort(rows * offs[-1] + cols)
    row_scale = col_scale = None
    if all(b.row_scale is not None and b.col_scale is not None for b in blocks) and \
            all(b.row_scale is blocks[0].row_scale or torch.equal(b.row_scale, blocks[0].row_scale) for b in blocks):
        row_scale, col_scale = blocks[0].row_scale, torch.cat([b.col_scale for b in blocks])
    return Block(rows[order], cols[order], vals[order], n_rows, offs[-1], row_scale, col_scale)


def _in_range(x, lo, hi):
    return (x >= lo) & (x < hi)


# ------------------------------------------------------------------------------------------ 1D / 1.5D
def oned_partition(rank, size, inputs, adj, normalization=True, replication=1, degree_group=None, transposed=False):
    """Blocks and feature rows of one rank for the 1D (replication = 1, gcn_distr.py:472-522) and 1.5D
    (gcn_distr_15d.py:497-549) algorithms.  blocks[i] is what the layer multiplies by H_i: the
    transpose of A[rows_i, cols_rank], coalesced (gcn_distr.py:546), n_rank x n_i.

    `transposed` (not in the reference, which multiplies by the same blocks in the backward pass and is exact
    for undirected graphs only) gives the blocks of the TRANSPOSED operator, A[rows_rank, cols_i] itself, with
    the same degree factors: what the backward pass of a directed graph has to multiply by."""
    n = inputs.size(0)
    n_per_proc = math.ceil(float(n) / (size / replication))
    rank_c = rank // replication
    vtx = boundaries(n, n_per_proc)
    lo, hi = vtx[rank_c], vtx[rank_c + 1]
    d = inv_sqrt_degree(adj, n, degree_group) if normalization else None
    a0, a1 = (adj[1], adj[0]) if transposed else (adj[0], adj[1])
    if lo == 0 and hi == n:
        u, v = a0, a1                         # one block row: nothing to filter (and no 2 x E copy at 1.3 G edges)
    else:
        sel = _in_range(a1, lo, hi)
        u, v = a0[sel], a1[sel] - lo
    blocks = []
    for i in range(len(vtx) - 1):
        s = slice(None) if len(vtx) == 2 else _in_range(u, vtx[i], vtx[i + 1])
        n_i = vtx[i + 1] - vtx[i]
        # stored orientation: row = column vertex of A (local to this rank), column = row vertex (local to block i)
        if normalization:
            blocks.append(coalesce_block(v[s], u[s] - vtx[i], hi - lo, n_i, d[lo:hi], d[vtx[i]:vtx[i + 1]],
                                         row_first=transposed))
        else:
            blocks.append(coalesce_block(v[s], u[s] - vtx[i], hi - lo, n_i))
    inputs_loc = inputs[lo:hi]
    return inputs_loc, blocks


def proc_groups_15d(size, replication):
    """Row groups [i, i + c), column groups range(i, P, c) (gcn_distr_15d.py:398-419)."""
    rows = [list(range(i, i + replication)) for i in range(0, size, replication)]
    cols = [list(range(i, size, replication)) for i in range(replication)]
    return rows, cols


def stages_15d(rank, size, replication):
    """(source rank, block id) per stage for `rank` (gcn_distr_15d.py:194-208): replica column j walks blocks
    j*(P/c^2) ..., the last replica also takes the remainder; with c = 1 this is the 1D loop."""
    rank_col = rank % replication
    per = size // (replication ** 2)
    stages = per
    if rank_col == replication - 1:
        stages = (size // replication) - (replication - 1) * per
    return [((rank_col * per + i) * replication + rank_col, rank_col * per + i) for i in range(stages)]


# ------------------------------------------------------------------------------------------ 2D
def grid_side_2d(size):
    return math.floor(math.sqrt(size))


def twod_partition(rank, size, inputs, adj, normalization=True, q=None, degree_group=None, transposed=False):
    """Block (rank_row, rank_col) of A -- not transposed -- and of H (rows and feature columns floor-split,
    remainder last): gcn_distr_2d.py:1093-1164.  `transposed` (not in the reference): the same block of A^T, the
    operator of a directed graph's backward pass, with the degree factors of A."""
    n = inputs.size(0)
    q = grid_side_2d(size) if q is None else q
    rank_row, rank_col = rank // q, rank % q
    vtx = boundaries(n, n // q, keep=q)
    r0, r1, c0, c1 = vtx[rank_row], vtx[rank_row + 1], vtx[rank_col], vtx[rank_col + 1]
    a0, a1 = (adj[1], adj[0]) if transposed else (adj[0], adj[1])
    sel = _in_range(a0, r0, r1) & _in_range(a1, c0, c1)
    u, v = a0[sel] - r0, a1[sel] - c0
    if normalization:
        d = inv_sqrt_degree(adj, n, degree_group)
        block = coalesce_block(u, v, r1 - r0, c1 - c0, d[r0:r1], d[c0:c1], row_first=transposed)
    else:
        block = coalesce_block(u, v, r1 - r0, c1 - c0)
    fs = [0]
    for w in chunk_sizes(inputs.size(1), q):
        fs.append(fs[-1] + w)
    inputs_loc = inputs[r0:r1, fs[rank_col]:fs[rank_col + 1]]
    return inputs_loc, block


def proc_groups_2d(size):
    """gcn_distr_2d.py:516-535."""
    q = grid_side_2d(size)
    return [list(range(i * q, i * q + q)) for i in range(q)], [list(range(i, size, q)) for i in range(q)]


# ------------------------------------------------------------------------------------------ 3D
def grid_side_3d(size):
    c = int(round(size ** (1.0 / 3.0)))
    if c ** 3 != size:
        raise ValueError("the 3D algorithm needs a cubic number of processes, got %d" % size)
    return c


def coords_3d(rank, q):
    """rank = i*(q*c) + j*c + k with q = c (gcn_distr_3d.py:754-756)."""
    return (rank // q) // q, (rank // q) % q, rank % q


def threed_partition(rank, size, inputs, adj, normalization=False, degree_group=None, transposed=False):
    """2D block (i, j), then its columns cut into c slabs and the H block's rows into c chunks; this rank keeps
    slab / chunk k (gcn_distr_3d.py:1533-1542, 1341-1382).  The reference never normalises here
    (gcn_distr_3d.py:66); `normalization=True` is this package's extension and scales exactly as 2D does."""
    q = grid_side_3d(size)
    i, j, k = coords_3d(rank, q)
    inputs_2d, blk = twod_partition(i * q + j, q * q, inputs, adj, normalization, q=q, degree_group=degree_group,
                                    transposed=transposed)
    vtx = boundaries(blk.n_cols, blk.n_cols // q, keep=q)
    s = _in_range(blk.cols, vtx[k], vtx[k + 1])
    # the reference rebuilds the slab from the coalesced indices with unit values (gcn_distr_3d.py:1357-1364)
    vals = blk.vals[s] if normalization else torch.ones_like(blk.vals[s])
    scales = (blk.row_scale, blk.col_scale[vtx[k]:vtx[k + 1]].contiguous()) if (normalization and blk.row_scale is not None) \
        else (None, None)
    slab = Block(blk.rows[s], blk.cols[s] - vtx[k], vals, blk.n_rows, vtx[k + 1] - vtx[k], *scales)
    rs = [0]
    for w in chunk_sizes(inputs_2d.size(0), q):
        rs.append(rs[-1] + w)
    return inputs_2d[rs[k]:rs[k + 1]], slab


def proc_groups_3d(size):
    """row_groups[i][k], col_groups[j][k], fiber groups [rank // c] (gcn_distr_3d.py:629-672)."""
    q = grid_side_3d(size)
    rows = [[list(range(i * q * q + k, (i + 1) * q * q + k, q)) for k in range(q)] for i in range(q)]
    cols = [[list(range(j * q + k, q * q * q + j * q + k, q * q)) for k in range(q)] for j in range(q)]
    fibers = [list(range(i, i + q)) for i in range(0, size, q)]
    return rows, cols, fibers
