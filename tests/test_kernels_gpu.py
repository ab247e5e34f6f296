"""Parity of every kernel, called through the C ABI, against the CPU oracle on the same seeded inputs.

Integer work (CSR offsets) must be bit-exact.  Floating point is fp32 with reordered summation: the
tolerance is 1e-4 relative to the largest reference magnitude, checked against an fp64 evaluation.
"""
import numpy as np
import pytest
import torch

from cagnet_b200 import _native, graphs, ops, partition as PP
from oracle import gcn as OG

pytestmark = pytest.mark.gpu
REL = 1e-4


def _close(got, want64, rel=REL):
    want64 = want64.double()
    scale = max(float(want64.abs().max()), 1e-30)
    err = float((got.double().cpu() - want64).abs().max())
    assert err <= rel * scale, f"max abs err {err:.3e} vs scale {scale:.3e}"


def _random_block(n, m, avg, seed, hubs=0):
    g = torch.Generator().manual_seed(seed)
    nnz = n * avg
    r = torch.randint(0, n, (nnz,), generator=g)
    c = torch.randint(0, m, (nnz,), generator=g)
    for h in range(hubs):                      # a few very long rows
        extra = torch.randint(0, m, (min(m, 3000),), generator=g)
        r = torch.cat([r, torch.full_like(extra, (7 * h + 3) % n)])
        c = torch.cat([c, extra])
    if n > 5:
        keep = r != 5                          # row 5 stays empty
        r, c = r[keep], c[keep]
    blk = PP.coalesce_block(r, c, n, m)
    vals = torch.randn(blk.vals.numel(), generator=g)
    return PP.Block(blk.rows, blk.cols, vals, n, m)


def _dense64(blk):
    return torch.sparse_coo_tensor(torch.stack([blk.rows, blk.cols]), blk.vals.double(), (blk.n_rows, blk.n_cols))


@pytest.mark.parametrize("n,avg", [(1, 1), (100, 3), (5000, 40), (70000, 2), (300, 0)])
def test_coo2csr_bit_exact(n, avg):
    g = torch.Generator().manual_seed(n)
    rows = torch.sort(torch.randint(0, n, (n * avg,), generator=g))[0].int()
    got = ops.coo2csr(rows.cuda(), n).cpu().numpy()
    assert np.array_equal(got, OG.coo2csr(rows.numpy(), n))


@pytest.mark.parametrize("f", [1, 2, 3, 4, 7, 16, 24, 41, 64, 100, 128, 300, 602, 700])
@pytest.mark.parametrize("beta", [0.0, 1.0])
def test_spmm_widths(f, beta):
    blk = _random_block(997, 1203, 9, seed=f)
    A = ops.CsrBlock.from_coo(blk.rows, blk.cols, blk.vals, blk.n_rows, blk.n_cols)
    g = torch.Generator().manual_seed(1000 + f)
    B = torch.randn(blk.n_cols, f, generator=g)
    C0 = torch.randn(blk.n_rows, f, generator=g)
    want = torch.sparse.mm(_dense64(blk), B.double()) + (C0.double() if beta else 0)
    for padded in (True, False):
        Bd = ops.to_padded(B.cuda()) if padded else B.cuda()
        Cd = ops.to_padded(C0.cuda()) if padded else C0.cuda().clone()
        ops.spmm(A, Bd, Cd, beta)
        _close(Cd, want)


@pytest.mark.parametrize("f", [16, 41, 602])
@pytest.mark.parametrize("tile", [0, 8, 16, 32, 64, 128])
def test_spmm_hub_rows_and_tilings(f, tile):
    """Rows beyond the plan threshold go through the block-per-row kernel; tile forces feature tiling."""
    old_long, old_tile = _native.get_param("spmm_long"), _native.get_param("spmm_tile")
    try:
        _native.set_param("spmm_long", 256)
        _native.set_param("spmm_tile", tile)
        blk = _random_block(600, 4000, 20, seed=3, hubs=5)
        A = ops.CsrBlock.from_coo(blk.rows, blk.cols, blk.vals, blk.n_rows, blk.n_cols)
        assert A.long_rows() >= 5
        g = torch.Generator().manual_seed(77)
        B = torch.randn(blk.n_cols, f, generator=g)
        C0 = torch.randn(blk.n_rows, f, generator=g)
        want = torch.sparse.mm(_dense64(blk), B.double()) + C0.double()
        Cd = ops.to_padded(C0.cuda())
        ops.spmm(A, ops.to_padded(B.cuda()), Cd, 1.0)
        _close(Cd, want)
        # without a plan every row takes the warp-per-row path: same numbers within tolerance
        A2 = ops.CsrBlock.from_coo(blk.rows, blk.cols, blk.vals, blk.n_rows, blk.n_cols, plan=False)
        Cd2 = ops.to_padded(C0.cuda())
        ops.spmm(A2, ops.to_padded(B.cuda()), Cd2, 1.0)
        _close(Cd2, want)
    finally:
        _native.set_param("spmm_long", old_long)
        _native.set_param("spmm_tile", old_tile)


def _skewed_block(n, m, seed, hubs=2):
    """Short rows of very different lengths (1 .. ~200 nonzeros, most of them a handful), a few empty ones and
    `hubs` rows beyond the hub threshold: what an R-MAT block with edge factor 16 looks like to the kernels."""
    g = torch.Generator().manual_seed(seed)
    lens = (torch.rand(n, generator=g).pow(6) * 200).long() + (torch.rand(n, generator=g) < 0.9).long()
    r = torch.repeat_interleave(torch.arange(n), lens)
    c = torch.randint(0, m, (r.numel(),), generator=g)
    for h in range(hubs):
        extra = torch.randperm(m, generator=g)[: min(m, 3000)]
        r = torch.cat([r, torch.full_like(extra, (13 * h + 1) % n)])
        c = torch.cat([c, extra])
    blk = PP.coalesce_block(r, c, n, m)
    return PP.Block(blk.rows, blk.cols, torch.randn(blk.vals.numel(), generator=g), n, m)


@pytest.mark.parametrize("f", [1, 3, 8, 16, 24, 41, 64, 100])
@pytest.mark.parametrize("pool,group_max", [(0, 64), (4, 0), (8, 7), (16, 64), (32, 64), (32, 4096)])
def test_spmm_lane_group_kernel(f, pool, group_max):
    """Blocks with few nonzeros per row take the lane-group kernel below 128 columns: every pool size, rows routed
    to a lane group or to the whole warp by length, hub rows left to the block-per-row kernel; beta 0 and 1; NaN in
    the pad columns of B and C must not reach a result, and columns of C beyond f must keep their contents."""
    names = ("spmm_group_pool", "spmm_group_max", "spmm_long")
    old = {k: _native.get_param(k) for k in names}
    try:
        _native.set_param("spmm_group_pool", pool)
        _native.set_param("spmm_group_max", group_max)
        _native.set_param("spmm_long", 512)
        blk = _skewed_block(2311, 3001, seed=f + pool)
        assert blk.vals.numel() <= _native.get_param("spmm_group_avg") * blk.n_rows
        A = ops.CsrBlock.from_coo(blk.rows, blk.cols, blk.vals, blk.n_rows, blk.n_cols)
        assert A.long_rows() >= 2
        g = torch.Generator().manual_seed(5 + f)
        B = torch.randn(blk.n_cols, f, generator=g)
        C0 = torch.randn(blk.n_rows, f, generator=g)
        prod = torch.sparse.mm(_dense64(blk), B.double())
        Bd = _poison_pads(ops.to_padded(B.cuda()))
        for beta in (0.0, 1.0):
            Cd = _poison_pads(ops.to_padded(C0.cuda()))
            ops.spmm(A, Bd, Cd, beta)
            _close(Cd, prod + (C0.double() if beta else 0))
            ld = Cd.stride(0)
            if ld > f:
                assert bool(torch.isnan(ops.base_buffer(Cd).view(-1, ld)[:, f:]).all()), "pad columns of C were written"
        Cd2 = ops.zeros_padded(blk.n_rows, f, "cuda")
        ops.spmm(A, Bd, Cd2, 0.0)
        Cd3 = ops.zeros_padded(blk.n_rows, f, "cuda")
        ops.spmm(A, Bd, Cd3, 0.0)
        assert torch.equal(Cd2, Cd3)                              # bit-reproducible whatever the claim order was
    finally:
        for k, v in old.items():
            _native.set_param(k, v)


@pytest.mark.parametrize("f", [3, 41, 130, 602])
def test_spmm_writes_only_n_by_f(f):
    """C may be a column slice of a wider matrix (same row stride): the columns next to it belong to the caller."""
    for blk in (_random_block(500, 700, 8, seed=f), _random_block(300, 4000, 150, seed=f + 1, hubs=3)):
        A = ops.CsrBlock.from_coo(blk.rows, blk.cols, blk.vals, blk.n_rows, blk.n_cols)
        g = torch.Generator().manual_seed(f)
        B = torch.randn(blk.n_cols, f, generator=g)
        wide = ops.pad_ld(f) + 4
        Z0 = torch.randn(blk.n_rows, wide, generator=g)
        Z = Z0.cuda().clone()
        C = Z[:, :f]
        want = Z0[:, :f].double() + torch.sparse.mm(_dense64(blk), B.double())
        ops.spmm(A, ops.to_padded(B.cuda()), C, 1.0)
        _close(Z[:, :f], want)
        assert torch.equal(Z[:, f:].cpu(), Z0[:, f:]), "columns beyond f were modified"
        Z = Z0.cuda().clone()
        ops.spmm_gpu(blk.rows.int().cuda(), blk.cols.int().cuda(), blk.vals.cuda(), blk.n_rows, blk.n_cols, B.cuda(),
                     Z[:, :f])
        _close(Z[:, :f], want)
        assert torch.equal(Z[:, f:].cpu(), Z0[:, f:])


def test_spmm_is_bit_reproducible():
    blk = _random_block(3000, 3000, 30, seed=8, hubs=3)
    A = ops.CsrBlock.from_coo(blk.rows, blk.cols, blk.vals, blk.n_rows, blk.n_cols)
    B = ops.to_padded(torch.randn(3000, 41, generator=torch.Generator().manual_seed(2)).cuda())
    outs = []
    for _ in range(3):
        C = ops.zeros_padded(3000, 41, "cuda")
        ops.spmm(A, B, C, 0.0)
        outs.append(C.clone())
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_spmm_edge_cases():
    # empty matrix, nnz = 0, single row / column, f = 0
    A = ops.CsrBlock.from_coo(torch.zeros(0, dtype=torch.int64), torch.zeros(0, dtype=torch.int64), torch.zeros(0), 4, 6)
    C = torch.ones(4, 3, device="cuda")
    ops.spmm(A, torch.ones(6, 3, device="cuda"), C, 1.0)
    assert torch.equal(C.cpu(), torch.ones(4, 3))
    ops.spmm(A, torch.ones(6, 3, device="cuda"), C, 0.0)
    assert torch.equal(C.cpu(), torch.zeros(4, 3))
    A1 = ops.CsrBlock.from_coo(torch.tensor([0]), torch.tensor([0]), torch.tensor([2.5]), 1, 1)
    C1 = torch.zeros(1, 1, device="cuda")
    ops.spmm(A1, torch.tensor([[4.0]], device="cuda"), C1, 0.0)
    assert C1.item() == 10.0
    # a non-finite value in B must only reach the rows that reference it
    blk = _random_block(64, 64, 2, seed=1)
    B = torch.randn(64, 8)
    unused = sorted(set(range(64)) - set(blk.cols.tolist()))
    if unused:
        B[unused[0]] = float("inf")
        Ad = ops.CsrBlock.from_coo(blk.rows, blk.cols, blk.vals, 64, 64)
        Cd = torch.zeros(64, 8, device="cuda")
        ops.spmm(Ad, B.cuda(), Cd, 0.0)
        assert torch.isfinite(Cd).all()


def test_malformed_blocks_are_rejected():
    with pytest.raises(RuntimeError, match="malformed"):
        ops.CsrBlock.from_coo(torch.tensor([0, 1]), torch.tensor([0, 9]), torch.ones(2), 2, 4)   # column out of range
    with pytest.raises(RuntimeError, match="malformed"):
        ops.CsrBlock.from_coo(torch.tensor([1, 0]), torch.tensor([0, 1]), torch.ones(2), 2, 4)   # rows not sorted
    with pytest.raises(RuntimeError, match="shape mismatch"):
        A = ops.CsrBlock.from_coo(torch.tensor([0]), torch.tensor([0]), torch.ones(1), 2, 4)
        ops.spmm(A, torch.zeros(5, 3, device="cuda"), torch.zeros(2, 3, device="cuda"))


def test_dropin_spmm_gpu_accumulates_in_place_and_keeps_strides():
    blk = _random_block(200, 150, 6, seed=12)
    B = torch.randn(150, 10)
    C0 = torch.randn(200, 10)
    want = C0.double() + torch.sparse.mm(_dense64(blk), B.double())
    Bd, Cd = B.cuda(), C0.cuda().clone()
    ops.spmm_gpu(blk.rows.int().cuda(), blk.cols.int().cuda(), blk.vals.cuda(), 200, 150, Bd, Cd)
    _close(Cd, want)
    assert Bd.stride() == (10, 1) and Cd.stride() == (10, 1) and torch.equal(Bd.cpu(), B)
    # the column-major-strided views the reference's op leaves behind are accepted too
    Bt = B.t().contiguous().t().cuda()
    Ct = C0.t().contiguous().t().cuda()
    assert Ct.stride() == (1, 200)
    ops.spmm_gpu(blk.rows.int().cuda(), blk.cols.int().cuda(), blk.vals.cuda(), 200, 150, Bt, Ct)
    _close(Ct, want)
    assert Ct.stride() == (1, 200)
    sp = ops.sparse_coo_tensor_gpu(torch.stack([blk.rows, blk.cols]).cuda(), blk.vals.cuda(), (200, 150))
    assert sp.is_sparse and sp.shape == (200, 150) and sp._nnz() == blk.vals.numel()


@pytest.mark.parametrize("n,K,N", [(1000, 602, 16), (777, 16, 41), (300, 41, 16), (513, 128, 64), (129, 7, 3),
                                   (2000, 64, 130), (70001, 602, 10), (100, 1000, 16), (50, 1100, 16)])
@pytest.mark.parametrize("trans", [False, True])
def test_gemm_nn_and_epilogues(n, K, N, trans):
    g = torch.Generator().manual_seed(n + K)
    X = torch.randn(n, K, generator=g)
    W = torch.randn(N, K, generator=g) if trans else torch.randn(K, N, generator=g)
    Z64 = X.double() @ (W.double().t() if trans else W.double())
    Xd, Wd = _poison_pads(ops.to_padded(X.cuda())), W.cuda()
    _close(ops.gemm_nn(Xd, Wd, trans), Z64)
    _close(ops.gemm_nn(X.cuda(), Wd, trans), Z64)                      # unpadded X (scalar loads)
    _close(ops.gemm_nn(Xd, Wd, trans, ops.EPI_RELU), torch.relu(Z64))
    aux = torch.randn(n, N, generator=g)
    _close(ops.gemm_nn(Xd, Wd, trans, ops.EPI_RELU_MASK, aux=ops.to_padded(aux.cuda())), Z64 * (aux > 0))
    if N <= 64:
        _close(ops.gemm_nn(Xd, Wd, trans, ops.EPI_LOG_SOFTMAX), torch.log_softmax(Z64, dim=1))
    else:
        with pytest.raises(RuntimeError, match="log-softmax"):
            ops.gemm_nn(Xd, Wd, trans, ops.EPI_LOG_SOFTMAX)


def _poison_pads(t):
    """NaN in the pad columns [f, ld) of a padded matrix: no kernel may let them reach a result."""
    ld, f = t.stride(0), t.size(1)
    if ld > f and t.size(0) > 0:
        ops.base_buffer(t).view(-1, ld)[:, f:] = float("nan")
    return t


@pytest.mark.parametrize("n,K,N", [(5000, 602, 16), (3000, 16, 41), (10, 5, 3), (4097, 130, 70), (1, 4, 4),
                                   (70001, 602, 10), (257, 66, 16), (64, 64, 1), (20000, 41, 13)])
def test_gemm_tn(n, K, N):
    g = torch.Generator().manual_seed(n)
    H, G = torch.randn(n, K, generator=g), torch.randn(n, N, generator=g)
    want = H.double().t() @ G.double()
    out1 = ops.gemm_tn(_poison_pads(ops.to_padded(H.cuda())), _poison_pads(ops.to_padded(G.cuda())))
    assert not bool(torch.isnan(out1).any())
    _close(out1, want)
    out2 = ops.gemm_tn(ops.to_padded(H.cuda()), ops.to_padded(G.cuda()))
    assert torch.equal(out1, out2)                                      # deterministic split-row reduction
    _close(ops.gemm_tn(H.cuda(), G.cuda()), want)


@pytest.mark.parametrize("n,N", [(1000, 41), (33, 5), (257, 256), (64, 1)])
def test_rowwise_ops(n, N):
    g = torch.Generator().manual_seed(N)
    z, gr = 3 * torch.randn(n, N, generator=g), torch.randn(n, N, generator=g)
    zd, gd = ops.to_padded(z.cuda()), ops.to_padded(gr.cuda())
    _close(ops.relu(zd), torch.relu(z))
    _close(ops.relu_bwd(ops.relu(zd), gd), gr * (z > 0))
    logp = ops.log_softmax(zd)
    _close(logp, torch.log_softmax(z.double(), dim=1))
    z64 = z.double().requires_grad_(True)
    torch.log_softmax(z64, dim=1).backward(gr.double())
    _close(ops.log_softmax_bwd(logp, gd), z64.grad)


def test_nll_masked():
    g = torch.Generator().manual_seed(4)
    n, N = 5000, 41
    logp = torch.log_softmax(torch.randn(n, N, generator=g), dim=1)
    y = torch.randint(0, N, (n,), generator=g)
    mask = torch.rand(n, generator=g) < 0.66
    cnt = int(mask.sum())
    l64 = logp.double().requires_grad_(True)
    want = torch.nn.functional.nll_loss(l64[mask], y[mask])
    want.backward()
    loss, grad = ops.nll_masked(ops.to_padded(logp.cuda()), y.cuda(), mask.cuda(), cnt)
    assert abs(loss.item() - want.item()) <= REL * abs(want.item())
    _close(grad, l64.grad)
    # class-range form used by the 2D / 3D loss: only labels in [lo, hi) count, rebased by lo
    lo, hi = 20, 40
    sub = logp[:, lo:hi].contiguous()
    sel = mask & (y >= lo) & (y < hi)
    want2 = -(sub.double()[sel, (y[sel] - lo)]).sum() / cnt
    loss2, grad2 = ops.nll_masked(ops.to_padded(sub.cuda()), y.cuda(), mask.cuda(), cnt, cls_lo=lo, cls_hi=hi)
    assert abs(loss2.item() - want2.item()) <= REL * abs(want2.item())
    want_g = torch.zeros(n, hi - lo, dtype=torch.float64)
    want_g[sel, y[sel] - lo] = -1.0 / cnt
    _close(grad2, want_g)


def test_spmm_on_rmat_graph_with_normalised_values():
    """The benchmark's own kind of input at a size the CPU checks in seconds: power-law rows, fp32
    D^-1/2 (A + I) D^-1/2 values, width 602 -> 16 -> 41."""
    n = 20000
    edge = graphs.rmat_graph(n, target_nnz=2_000_000, seed=1)
    adj = graphs.add_self_loops(edge, n)
    _, blocks = PP.oned_partition(0, 1, torch.zeros(n, 1), adj, True)
    blk = blocks[0]
    A = ops.CsrBlock.from_coo(blk.rows, blk.cols, blk.vals, n, n)
    M64 = _dense64(blk)
    for f in (602, 16, 41):
        B = torch.randn(n, f, generator=torch.Generator().manual_seed(f))
        C = ops.zeros_padded(n, f, "cuda")
        ops.spmm(A, ops.to_padded(B.cuda()), C, 0.0)
        _close(C, torch.sparse.mm(M64, B.double()))


@pytest.mark.parametrize("n,N", [(500, 21), (33, 128), (7, 1)])
def test_split_log_softmax_pieces(n, N):
    """The row-wise pieces a process row combines with collectives: here the 'collective' is a sum over two
    column halves held by one process, checked against the whole-row log-softmax and its gradient."""
    g = torch.Generator().manual_seed(n)
    z, gr = 2 * torch.randn(n, N, generator=g), torch.randn(n, N, generator=g)
    h = max(1, N // 2)
    parts = [(z[:, :h], gr[:, :h]), (z[:, h:], gr[:, h:])] if N > 1 else [(z, gr)]
    dev = [(ops.to_padded(a.contiguous().cuda()), ops.to_padded(b.contiguous().cuda())) for a, b in parts]
    m = torch.stack([ops.row_reduce(a, ops.ROW_MAX) for a, _ in dev]).max(0)[0]
    s = torch.stack([ops.row_reduce(a, ops.ROW_SUMEXP, m) for a, _ in dev]).sum(0)
    rs = torch.stack([ops.row_reduce(b, ops.ROW_SUM) for _, b in dev]).sum(0)
    want = torch.log_softmax(z.double(), dim=1)
    z64 = z.double().requires_grad_(True)
    torch.log_softmax(z64, dim=1).backward(gr.double())
    col = 0
    for a, b in dev:
        w = a.size(1)
        logp = ops.log_softmax_apply(a, m, s)
        _close(logp, want[:, col:col + w])
        _close(ops.log_softmax_bwd_apply(logp, b, rs), z64.grad[:, col:col + w])
        col += w


def test_accumulating_products():
    g = torch.Generator().manual_seed(9)
    X, W, Z0 = torch.randn(700, 37, generator=g), torch.randn(37, 21, generator=g), torch.randn(700, 21, generator=g)
    Zd = ops.to_padded(Z0.cuda())
    ops.gemm_nn(ops.to_padded(X.cuda()), W.cuda(), False, ops.EPI_ACCUMULATE, out=Zd)
    _close(Zd, Z0.double() + X.double() @ W.double())
    Wt = torch.randn(21, 37, generator=g)
    Zd = ops.to_padded(Z0.cuda())
    ops.gemm_nn(ops.to_padded(X.cuda()), Wt.cuda(), True, ops.EPI_ACCUMULATE, out=Zd)
    _close(Zd, Z0.double() + X.double() @ Wt.double().t())
    # a strided slice of a larger weight, as the SUMMA stages pass it
    big = torch.randn(50, 40, generator=g).cuda()
    part = big[5:42, 11:32]
    _close(ops.gemm_nn(ops.to_padded(X.cuda()), part), X.double() @ part.double().cpu())
    H, G, O0 = torch.randn(900, 13, generator=g), torch.randn(900, 9, generator=g), torch.randn(13, 9, generator=g)
    Od = O0.cuda().clone()
    ops.gemm_tn(H.cuda(), G.cuda(), out=Od, accumulate=True)
    _close(Od, O0.double() + H.double().t() @ G.double())


# ------------------------------------------------------------------------------------------ dense core
@pytest.mark.parametrize("R,K,f", [(128, 128, 128), (200, 77, 602), (1, 5, 130), (300, 1000, 41), (257, 33, 7),
                                   (130, 4865, 602), (64, 2049, 100)])
def test_core_gemm_indexed_rows(R, K, f):
    """C[rows[i]] += sum_j core[i, j] * B[cols[j]] against fp64, ragged sizes and padded rows included."""
    g = torch.Generator().manual_seed(R * 7 + K)
    n, m = R + 50, K + 70
    core = torch.randn(R, K, generator=g)
    core[torch.rand(R, K, generator=g) < 0.5] = 0.0
    rows = torch.randperm(n, generator=g)[:R]
    cols = torch.randperm(m, generator=g)[:K]
    B, C0 = torch.randn(m, f, generator=g), torch.randn(n, f, generator=g)
    want = C0.double()
    want[rows] += core.double() @ B.double()[cols]
    Bd, Cd, cored = ops.to_padded(B.cuda()), ops.to_padded(C0.cuda()), core.cuda()
    rd, cd = rows.int().cuda(), cols.int().cuda()
    ws = torch.empty(max(_native.lib().cagnet_core_gemm_workspace_bytes(R, K, f), 16), dtype=torch.uint8, device="cuda")
    _native.check(_native.lib().cagnet_core_gemm_f32(cored.data_ptr(), cored.stride(0), rd.data_ptr(), R, cd.data_ptr(),
                                                     K, Bd.data_ptr(), Bd.stride(0), Cd.data_ptr(), Cd.stride(0), f,
                                                     ws.data_ptr(), ws.numel(), None), "core_gemm")
    torch.cuda.synchronize()
    _close(Cd, want)


@pytest.mark.parametrize("R,K,f", [(128, 128, 128), (200, 76, 602), (1, 8, 130), (300, 1000, 41), (130, 4864, 602)])
def test_core_gemm_on_tensor_cores(R, K, f):
    """split -> gather + split rows -> tcgen05 3xTF32 multiply in k chunks -> add into listed rows, against fp64."""
    L = _native.lib()
    if L.cagnet_core_gemm_tc_available() != 1:
        pytest.skip("library built without the CUTLASS header tree")
    g = torch.Generator().manual_seed(R * 11 + K)
    n, m = R + 50, K + 70
    core = torch.randn(R, K, generator=g)
    core[torch.rand(R, K, generator=g) < 0.5] = 0.0
    rows = torch.randperm(n, generator=g)[:R]
    cols = torch.randperm(m, generator=g)[:K]
    B, C0 = torch.randn(m, f, generator=g), torch.randn(n, f, generator=g)
    want = C0.double()
    want[rows] += core.double() @ B.double()[cols]
    Bd, Cd, cored = ops.to_padded(B.cuda()), ops.to_padded(C0.cuda()), core.cuda()
    rd, cd = rows.int().cuda(), cols.int().cuda()
    hi, lo = torch.empty_like(cored), torch.empty_like(cored)
    _native.check(L.cagnet_split_tf32_f32(cored.data_ptr(), cored.numel(), hi.data_ptr(), lo.data_ptr(), None), "split")
    assert torch.equal(hi + lo, cored) and int((hi.view(torch.int32) & 0x1fff).abs().max()) == 0
    half = (f + 3) // 4 * 4
    Bs = torch.full((K, 2 * half), float("nan"), device="cuda")
    D = torch.empty(R, 3 * half, device="cuda")
    _native.check(L.cagnet_gather_split_rows_f32(Bd.data_ptr(), Bd.stride(0), cd.data_ptr(), K, f, Bs.data_ptr(), half,
                                                 None), "gather_split")
    assert torch.equal((Bs[:, :f] + Bs[:, half:half + f]).cpu(), B[cols])
    assert not bool(torch.isnan(Bs).any())                  # pad columns of both halves are zeroed
    ws = torch.empty(max(L.cagnet_core_gemm_tc_workspace_bytes(R, K, f), 16), dtype=torch.uint8, device="cuda")
    _native.check(L.cagnet_core_gemm_tc_f32(hi.data_ptr(), lo.data_ptr(), hi.stride(0), R, K, Bs.data_ptr(), half,
                                            D.data_ptr(), f, ws.data_ptr(), ws.numel(), None), "tc")
    _native.check(L.cagnet_add_rows3_f32(D.data_ptr(), half, rd.data_ptr(), R, f, Cd.data_ptr(), Cd.stride(0), None),
                  "add3")
    torch.cuda.synchronize()
    _close(Cd, want, rel=2e-5)       # measured about 2e-6; a single TF32 pass would be 3e-4


def test_core_gemm_rejects_unaligned_rows():
    z = torch.zeros(8, 7, device="cuda")
    idx = torch.arange(4, dtype=torch.int32, device="cuda")
    core = torch.zeros(4, 4, device="cuda")
    rc = _native.lib().cagnet_core_gemm_f32(core.data_ptr(), 4, idx.data_ptr(), 4, idx.data_ptr(), 4, z.data_ptr(), 7,
                                            z.data_ptr(), 7, 7, None, 0, None)
    assert rc == 2 and b"16-byte" in _native.lib().cagnet_last_error_string()


@pytest.mark.parametrize("tensor", [True, False])
@pytest.mark.parametrize("f,beta", [(602, 0.0), (130, 1.0), (128, 0.0)])
def test_spmm_with_dense_core_matches_oracle(f, beta, tensor):
    """A power-law block whose hub rows x hub columns rectangle is cut out and multiplied densely: same product."""
    n = 4096
    edge = graphs.rmat_graph(n, target_nnz=n * 96, seed=5)
    adj = graphs.add_self_loops(edge, n)
    _, blocks = PP.oned_partition(0, 1, torch.zeros(n, 1), adj, True)
    blk = blocks[0]
    old = ops.configure_core(enabled=True, step=64, max_side=1024, min_share=0.0, density=0.1, density_tc=0.1,
                             min_width=128, rounds=3, tensor_cores=tensor)
    try:
        _spmm_with_core(blk, n, f, beta)
    finally:
        ops.configure_core(**old)


def _spmm_with_core(blk, n, f, beta):
    A = ops.CsrBlock.from_coo(blk.rows, blk.cols, blk.vals, n, n)
    assert A.core is not None, "this graph has a dense core at a 10 % density bar"
    src, in_cores, rounds = A, 0, 0
    while src.core is not None:                   # one rectangle per round, each cut out of the previous rest
        dense, core_rows, core_cols = src.core
        assert int((dense != 0).sum()) + src.rest.nnz == src.nnz
        assert len(set(core_rows.tolist())) == dense.size(0) and len(set(core_cols.tolist())) == dense.size(1)
        in_cores += int((dense != 0).sum())
        src, rounds = src.rest, rounds + 1
    assert in_cores + src.nnz == A.nnz and 1 <= rounds <= 3
    g = torch.Generator().manual_seed(f)
    B, C0 = torch.randn(n, f, generator=g), torch.randn(n, f, generator=g)
    want = beta * C0.double() + torch.sparse.mm(_dense64(blk), B.double())
    C = ops.to_padded(C0.cuda())
    ops.spmm(A, ops.to_padded(B.cuda()), C, beta)
    _close(C, want)
    # narrow products keep using the whole CSR block
    Bn = torch.randn(n, 16, generator=g)
    Cn = ops.zeros_padded(n, 16, "cuda")
    before = ops.launch_count()
    ops.spmm(A, ops.to_padded(Bn.cuda()), Cn, 0.0)
    assert ops.launch_count() - before <= 2
    _close(Cn, torch.sparse.mm(_dense64(blk), Bn.double()))


@pytest.mark.parametrize("f,beta", [(602, 0.0), (130, 1.0), (128, 0.0), (41, 1.0), (16, 0.0)])
def test_spmm_with_integer_core_matches_oracle(f, beta):
    """A normalised block that carries its diagonal factors keeps its core as bf16 edge multiplicities and multiplies
    it with three bf16 tensor-core products: same product as the fp64 oracle, to the same tolerance."""
    if not ops.integer_core_available():
        pytest.skip("library built without the tensor-core kernels")
    n = 4096
    edge = graphs.rmat_graph(n, target_nnz=n * 96, seed=5)
    adj = graphs.add_self_loops(edge, n)
    _, blocks = PP.oned_partition(0, 1, torch.zeros(n, 1), adj, True)
    blk = blocks[0]
    assert blk.row_scale is not None and blk.col_scale is not None
    old = ops.configure_core(enabled=True, step=64, max_side_int=2048, min_share=0.0, density_int=0.05, min_width_int=16)
    try:
        A = ops.CsrBlock.from_coo(blk.rows, blk.cols, blk.vals, n, n, row_scale=blk.row_scale, col_scale=blk.col_scale)
        assert A.core_kind() == "bf16-integer"
        cnt = A.core_int[0]
        assert int((cnt != 0).sum()) + A.rest.nnz == A.nnz and float(cnt.float().max()) == 1.0
        g = torch.Generator().manual_seed(f)
        B, C0 = torch.randn(n, f, generator=g), torch.randn(n, f, generator=g)
        want = beta * C0.double() + torch.sparse.mm(_dense64(blk), B.double())
        C = _poison_pads(ops.to_padded(C0.cuda()))
        before = ops.launch_count()
        ops.spmm(A, _poison_pads(ops.to_padded(B.cuda())), C, beta)
        assert ops.launch_count() - before > 2                      # the core kernels ran
        _close(C, want)
        # scales that do not belong to the block: the values do not factor, the fp32 core is kept
        wrong = ops.CsrBlock.from_coo(blk.rows, blk.cols, blk.vals, n, n, row_scale=blk.row_scale * 1.5,
                                      col_scale=blk.col_scale)
        assert wrong.core_int is None
        # an edge listed twice has multiplicity 2: still an exact small integer
        dup = torch.cat([adj, adj[:, :5000]], dim=1)
        _, blocks2 = PP.oned_partition(0, 1, torch.zeros(n, 1), dup, True)
        b2 = blocks2[0]
        A2 = ops.CsrBlock.from_coo(b2.rows, b2.cols, b2.vals, n, n, row_scale=b2.row_scale, col_scale=b2.col_scale)
        if A2.core_int is not None:
            C2 = ops.zeros_padded(n, f, "cuda")
            ops.spmm(A2, ops.to_padded(B.cuda()), C2, 0.0)
            _close(C2, torch.sparse.mm(_dense64(b2), B.double()))
    finally:
        ops.configure_core(**old)


def test_transposed_block_keeps_its_integer_core():
    """The block of the transposed operator (backward pass of a directed graph) is scaled row factor first; it still
    factors into diag . multiplicities . diag, keeps the bf16 core, and multiplies as the fp64 transpose does."""
    if not ops.integer_core_available():
        pytest.skip("library built without the tensor-core kernels")
    n, f = 4096, 130
    edge = graphs.rmat_graph(n, target_nnz=n * 160, seed=5)
    g = torch.Generator().manual_seed(2)
    edge = edge[:, torch.rand(edge.size(1), generator=g) < 0.6]      # drop 40 % of the arcs: no longer symmetric
    adj = graphs.add_self_loops(edge, n)
    fwd = PP.oned_partition(0, 1, torch.zeros(n, 1), adj, True)[1][0]
    bwd = PP.oned_partition(0, 1, torch.zeros(n, 1), adj, True, transposed=True)[1][0]
    D = _dense64(fwd).to_dense()
    assert not torch.equal(D, D.t()) and bwd.vals.numel() >= 80 * n    # above the rows-per-nonzero bar of the core
    assert torch.equal(_dense64(bwd).to_dense(), D.t())
    old = ops.configure_core(enabled=True, step=64, max_side_int=2048, min_share=0.0, density_int=0.05, min_width_int=16)
    try:
        A = ops.CsrBlock.from_coo(bwd.rows, bwd.cols, bwd.vals, n, n, row_scale=bwd.row_scale, col_scale=bwd.col_scale)
        assert A.core_kind() == "bf16-integer"
        B = torch.randn(n, f, generator=g)
        C = _poison_pads(ops.zeros_padded(n, f, "cuda"))
        ops.spmm(A, _poison_pads(ops.to_padded(B.cuda())), C, 0.0)
        _close(C, D.t() @ B.double())
    finally:
        ops.configure_core(**old)


def test_integer_core_kernels_through_the_c_abi():
    """gather + scale + three-term bf16 split, the chunked bf16 multiply and the scaled row add, one by one."""
    if _native.lib().cagnet_core_gemm_int_available() != 1:
        pytest.skip("library built without the tensor-core kernels")
    L = _native.lib()
    g = torch.Generator().manual_seed(3)
    m, f, K, R = 900, 130, 384, 256
    B = ops.to_padded(torch.randn(m, f, generator=g).cuda())
    idx = torch.randperm(m, generator=g)[:K].int().cuda()
    cs = torch.rand(K, generator=g).cuda() + 0.1
    half = (f + 7) // 8 * 8
    Ys = torch.full((K, 3 * half), float("nan"), dtype=torch.bfloat16, device="cuda")
    _native.check(L.cagnet_gather_scale_split3_bf16(B.data_ptr(), B.stride(0), idx.data_ptr(), cs.data_ptr(), K, f,
                                                    Ys.data_ptr(), half, None), "gather_scale_split3")
    y = cs[:, None] * B[idx.long()]
    parts = Ys.view(K, 3, half).float()
    assert torch.equal(parts[:, 0, :f], y.bfloat16().float())
    total = parts[:, 0, :f].double() + parts[:, 1, :f].double() + parts[:, 2, :f].double()
    assert float((total - y.double()).abs().max()) <= 2.0 ** -23 * float(y.abs().max())
    assert float(parts[:, :, f:].abs().max()) == 0.0                       # pad columns are zeros, not NaN
    cnt = (torch.rand(R, K, generator=g) < 0.2).to(torch.bfloat16).cuda()
    cnt[0, :7] = 2.0
    D = torch.empty(R, 3 * half, device="cuda")
    ws = torch.empty(max(L.cagnet_core_gemm_int_workspace_bytes(R, K, f), 16), dtype=torch.uint8, device="cuda")
    old_chunk = _native.get_param("core_chunk_int")
    try:
        _native.set_param("core_chunk_int", 256)                           # two k chunks
        _native.check(L.cagnet_core_gemm_int_bf16(cnt.data_ptr(), K, R, K, Ys.data_ptr(), half, D.data_ptr(), f,
                                                  ws.data_ptr(), ws.numel(), None), "core_gemm_int")
    finally:
        _native.set_param("core_chunk_int", old_chunk)
    _close(D, cnt.double().cpu() @ Ys.double().cpu(), rel=1e-5)
    rows = torch.randperm(700, generator=g)[:R].int().cuda()
    rs = torch.rand(R, generator=g).cuda() + 0.1
    C0 = torch.randn(700, f, generator=g)
    C = _poison_pads(ops.to_padded(C0.cuda()))
    _native.check(L.cagnet_add_rows_scaled3_f32(D.data_ptr(), half, rows.data_ptr(), rs.data_ptr(), R, f, C.data_ptr(),
                                                C.stride(0), None), "add_rows_scaled3")
    want = C0.double()
    want[rows.long().cpu()] += (rs.double()[:, None] * (cnt.double() @ y.double())).cpu()
    _close(C, want)


def test_no_core_for_uniform_graphs():
    blk = _random_block(5000, 5000, 20, seed=3)
    old = ops.configure_core(step=256, max_side=2048)
    try:
        A = ops.CsrBlock.from_coo(blk.rows, blk.cols, blk.vals, blk.n_rows, blk.n_cols)
    finally:
        ops.configure_core(**old)
    assert A.core is None and A.rest is None
