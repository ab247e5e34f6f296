"""Dense-core selection and split (host logic, CPU): the chosen rectangle is the best one by brute force, and the
dense part plus the remaining CSR block are exactly the original block."""
import numpy as np
import torch

from cagnet_b200 import core_select, graphs, partition as PP
from oracle import gcn as OG


def _block(n=512, per_vertex=40, seed=3):
    edge = graphs.rmat_graph(n, target_nnz=n * per_vertex, seed=seed)
    adj = graphs.add_self_loops(edge, n)
    _, blocks = PP.oned_partition(0, 1, torch.zeros(n, 1), adj, True)
    b = blocks[0]
    rowptr = torch.from_numpy(OG.coo2csr(b.rows.int().numpy(), n))
    return b, rowptr


def test_choice_is_the_best_rectangle():
    n, step, bar = 512, 16, 0.25
    b, rowptr = _block(n)
    ch = core_select.choose_core(rowptr, b.cols, n, n, bar, step=step, max_side=256, min_share=0.0)
    assert ch is not None
    dense = torch.sparse_coo_tensor(torch.stack([b.rows, b.cols]), torch.ones(b.vals.numel()), (n, n)).to_dense()
    deg_r, deg_c = dense.sum(1), dense.sum(0)
    order_r = torch.argsort(deg_r, descending=True, stable=True)
    order_c = torch.argsort(deg_c, descending=True, stable=True)
    best, arg = -1e30, None
    for r in range(step, 257, step):
        for c in range(step, 257, step):
            inside = float(dense[order_r[:r]][:, order_c[:c]].sum())
            gain = inside - bar * r * c
            if gain > best:
                best, arg = gain, (r, c, inside)
    assert (ch.r, ch.c) == arg[:2] and ch.inside == int(arg[2]) and abs(ch.gain - best) < 1e-6
    assert torch.equal(ch.rows, order_r[:ch.r]) and torch.equal(ch.cols, order_c[:ch.c])


def test_split_keeps_every_entry_once():
    n, step = 512, 16
    b, rowptr = _block(n, seed=4)
    ch = core_select.choose_core(rowptr, b.cols, n, n, 0.2, step=step, max_side=256, min_share=0.0)
    dense, rest_rowptr, rest_col, rest_val = core_select.split_core(b.cols, b.vals, n, ch)
    assert dense.shape == (ch.r, ch.c) and int((dense != 0).sum()) == ch.inside
    assert int(rest_rowptr[-1]) == rest_col.numel() == b.vals.numel() - ch.inside
    assert bool((rest_rowptr[1:] >= rest_rowptr[:-1]).all())
    full = torch.zeros(n, n)
    rest_rows = torch.repeat_interleave(torch.arange(n), (rest_rowptr[1:] - rest_rowptr[:-1]).long())
    full[rest_rows, rest_col.long()] = rest_val
    assert float(full[ch.rows][:, ch.cols].abs().sum()) == 0.0       # nothing of the rectangle is left in the rest
    full[ch.rows[:, None], ch.cols[None, :]] += dense
    want = torch.sparse_coo_tensor(torch.stack([b.rows, b.cols]), b.vals, (n, n)).to_dense()
    assert torch.equal(full, want)


def test_no_rectangle_in_a_uniform_block_and_limits():
    g = torch.Generator().manual_seed(0)
    n = 600
    r = torch.randint(0, n, (n * 8,), generator=g)
    c = torch.randint(0, n, (n * 8,), generator=g)
    blk = PP.coalesce_block(r, c, n, n)
    rowptr = torch.from_numpy(OG.coo2csr(blk.rows.int().numpy(), n))
    assert core_select.choose_core(rowptr, blk.cols, n, n, 0.2, step=32, max_side=256) is None
    assert core_select.choose_core(rowptr, blk.cols, n, n, 0.2, step=1024) is None        # block smaller than a step
    b, rowptr = _block(512)
    big = core_select.choose_core(rowptr, b.cols, 512, 512, 0.01, step=16, max_side=256, min_share=0.0)
    small = core_select.choose_core(rowptr, b.cols, 512, 512, 0.01, step=16, max_side=256, min_share=0.0,
                                    max_bytes=4 * 64 * 64)
    assert big.r * big.c > 64 * 64 >= small.r * small.c
    empty = torch.zeros(0, dtype=torch.int64)
    assert core_select.choose_core(torch.zeros(11, dtype=torch.int32), empty, 10, 10, 0.2, step=2) is None


def test_rectangular_block_of_a_block_row():
    """A rank's block row (fewer rows than columns): rows and columns are ranked separately."""
    n = 512
    b, _ = _block(n, seed=6)
    lo, hi = 128, 384                                  # rows [128, 384) of the graph, all columns
    sel = (b.rows >= lo) & (b.rows < hi)
    rows, cols, vals = b.rows[sel] - lo, b.cols[sel], b.vals[sel]
    rowptr = torch.from_numpy(OG.coo2csr(rows.int().numpy(), hi - lo))
    ch = core_select.choose_core(rowptr, cols, hi - lo, n, 0.15, step=16, max_side=256, min_share=0.0)
    assert ch is not None and ch.r <= hi - lo and ch.c <= 256
    assert int(ch.rows.max()) < hi - lo and int(ch.cols.max()) < n
    dense, rest_rowptr, rest_col, rest_val = core_select.split_core(cols, vals, hi - lo, ch)
    full = torch.zeros(hi - lo, n)
    rest_rows = torch.repeat_interleave(torch.arange(hi - lo), (rest_rowptr[1:] - rest_rowptr[:-1]).long())
    full[rest_rows, rest_col.long()] = rest_val
    full[ch.rows[:, None], ch.cols[None, :]] += dense
    want = torch.sparse_coo_tensor(torch.stack([rows, cols]), vals, (hi - lo, n)).to_dense()
    assert torch.equal(full, want)


def test_integer_core_recovers_multiplicities_exactly():
    """dense = fl32(rs * fl32(cnt * cs)) factors back into the integer matrix; anything else is refused."""
    g = torch.Generator().manual_seed(11)
    r, c = 96, 160
    cnt = (torch.rand(r, c, generator=g) < 0.3).float()
    cnt[3, 5], cnt[7, 7] = 2.0, 3.0
    rs = torch.rand(r, generator=g).double().pow(-0.5).float()
    cs = torch.rand(c, generator=g).double().pow(-0.5).float()
    cs[9] = 0.0                                                     # a padding column: no entry refers to it
    cnt[:, 9] = 0.0
    dense = rs[:, None] * (cnt * cs[None, :])
    got = core_select.integer_core(dense, rs, cs)
    assert got is not None and torch.equal(got, cnt)
    assert torch.equal(got.bfloat16().float(), cnt)                 # small integers are exact in bf16
    assert core_select.integer_core(dense, rs * 1.0001, cs) is None
    weighted = dense.clone()
    weighted[0, 0] = 0.123
    assert core_select.integer_core(weighted, rs, cs) is None
    big = rs[:, None] * (cnt * 300 * cs[None, :])
    assert core_select.integer_core(big, rs, cs) is None            # multiplicity beyond what bf16 holds exactly
    # the block of a transposed operator is scaled in the other order; it differs in some last bits and is accepted
    other = cs[None, :] * (cnt * rs[:, None])
    assert not torch.equal(other, dense)
    got = core_select.integer_core(other, rs, cs)
    assert got is not None and torch.equal(got, cnt)
