"""Choosing and cutting out the dense core of a power-law CSR block (device-agnostic torch index work).

In a scale-free graph the highest-degree rows meet the highest-degree columns in a rectangle that is far from
sparse.  `choose_core` ranks rows and columns by degree and picks, among the rectangles (top r rows) x (top c
columns) with r and c multiples of `step`, the one that maximises

    nonzeros inside  -  bar * r * c

(`bar` = the density above which a dense cell is cheaper than a gathered nonzero).  `split_core` turns that
choice into a dense r x c matrix plus the CSR arrays of everything else.  The reference has no counterpart: its
SpMM hands the whole block to cuSPARSE (sparse-extension/sparse_coo_tensor.cu:198-226).
"""
import torch


def top_by_degree(deg, limit):
    """The `limit` highest-degree indices (ties by index, so the choice is reproducible) and, for every index, its
    position in that list (`limit` for the ones left out)."""
    order = torch.argsort(deg, descending=True, stable=True)[:limit]
    rank = torch.full((deg.numel(),), limit, dtype=torch.int64, device=deg.device)
    rank[order] = torch.arange(order.numel(), device=deg.device)
    return order, rank


class CoreChoice:
    """r x c rectangle: `rows[i]` / `cols[j]` are the block's row / column of core row i / column j; `er`, `ec`
    give, per nonzero, its position in those lists (>= the list length for rows / columns outside)."""

    def __init__(self, r, c, rows, cols, er, ec, row_of, deg_r, inside, gain):
        self.r, self.c, self.rows, self.cols = r, c, rows, cols
        self.er, self.ec, self.row_of, self.deg_r = er, ec, row_of, deg_r
        self.inside, self.gain = inside, gain        # nonzeros in the rectangle; inside - bar * r * c


def choose_core(rowptr, col, n, m, bar, step=1024, max_side=16384, max_bytes=2 << 30, min_share=0.03,
                bytes_per_cell=4):
    """The best rectangle of a CSR block (rowptr: n + 1 offsets, col: column per nonzero), or None when no
    rectangle saves at least `min_share` of the block's nonzeros' worth of gathers."""
    nnz = int(col.numel())
    step = int(step)
    if nnz == 0 or step <= 0:
        return None
    gr, gc = min(int(max_side), n) // step, min(int(max_side), m) // step
    if gr == 0 or gc == 0:
        return None
    dev = col.device
    rowptr = rowptr.long()
    deg_r = rowptr[1:] - rowptr[:-1]
    col = col.long()
    deg_c = torch.bincount(col, minlength=m)
    order_r, rank_r = top_by_degree(deg_r, gr * step)
    order_c, rank_c = top_by_degree(deg_c, gc * step)
    row_of = torch.repeat_interleave(torch.arange(n, device=dev), deg_r)
    er, ec = rank_r[row_of], rank_c[col]
    near = (er < gr * step) & (ec < gc * step)
    hist = torch.bincount((er[near] // step) * gc + ec[near] // step, minlength=gr * gc).view(gr, gc)
    inside = hist.cumsum(0).cumsum(1).double()          # nonzeros in the top (i+1)*step x (j+1)*step rectangle
    side_r = torch.arange(1, gr + 1, device=dev, dtype=torch.float64) * step
    side_c = torch.arange(1, gc + 1, device=dev, dtype=torch.float64) * step
    cells = side_r[:, None] * side_c[None, :]
    gain = inside - float(bar) * cells
    gain[cells * float(bytes_per_cell) > float(max_bytes)] = float("-inf")
    best = int(torch.argmax(gain))
    i, j = divmod(best, gc)
    if not float(gain[i, j]) >= float(min_share) * nnz:
        return None
    r, c = (i + 1) * step, (j + 1) * step
    return CoreChoice(r, c, order_r[:r], order_c[:c], er, ec, row_of, deg_r, int(inside[i, j]), float(gain[i, j]))


def split_core(col, val, n, choice):
    """(dense r x c fp32 matrix, rest_rowptr int32[n + 1], rest_col, rest_val): the block's entries inside the
    rectangle, densely, and all others in CSR order."""
    in_core = (choice.er < choice.r) & (choice.ec < choice.c)
    dense = torch.zeros(choice.r, choice.c, dtype=torch.float32, device=val.device)
    dense.index_put_((choice.er[in_core], choice.ec[in_core]), val[in_core], accumulate=True)
    keep = ~in_core
    kept = choice.deg_r - torch.bincount(choice.row_of[in_core], minlength=n)
    rest_rowptr = torch.zeros(n + 1, dtype=torch.int32, device=val.device)
    rest_rowptr[1:] = torch.cumsum(kept, 0).int()
    return dense, rest_rowptr, col[keep].contiguous(), val[keep].contiguous()


def integer_core(dense, row_scale, col_scale, limit=256):
    """The multiplicity matrix of a dense core whose block was scaled by two diagonals, or None.

    `dense[i, j]` must equal fl32(row_scale[i] * fl32(cnt * col_scale[j])) -- or, every cell, the other order
    fl32(col_scale[j] * fl32(cnt * row_scale[i])) -- bit for bit with cnt a non-negative
    integer <= `limit` (the two ways partition.coalesce_block computes a normalised entry); then dense =
    diag(row_scale) . cnt . diag(col_scale) and cnt is returned as an fp32 matrix.  Any cell that does not fit --
    scales that do not belong to this block, weighted edges -- makes the answer None and the caller keeps the
    fp32 values."""
    outer = row_scale[:, None] * col_scale[None, :]
    nz = dense != 0
    cnt = torch.where(nz & (outer != 0), torch.round(dense / outer), torch.zeros_like(dense))
    del outer
    if float(cnt.max()) > limit or float(cnt.min()) < 0:
        return None
    back = row_scale[:, None] * (cnt * col_scale[None, :])
    if not bool(torch.equal(back, dense)):
        # the block of a transposed operator is scaled row factor first (coalesce_block(..., row_first=True))
        del back
        back = col_scale[None, :] * (cnt * row_scale[:, None])
        if not bool(torch.equal(back, dense)):
            return None
    return cnt
