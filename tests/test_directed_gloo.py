"""`directed=True`: the backward pass multiplies by the blocks of the TRANSPOSED operator instead of reusing the
forward blocks (which the reference does, exact for undirected graphs only: gcn_distr.py:326,
gcn_distr_2d.py:683).  Every schedule runs as Gloo ranks on CPU with the checker backend on a graph whose edge
list is NOT symmetric, against fp64 autograd through the dense model."""
import math

import numpy as np
import pytest
import torch

from tests.mp_util import run_ranks

N, F_IN, MID, CLASSES, EPOCHS, EDGES = 64, 8, 6, 4, 3, 420


def _problem():
    g = torch.Generator().manual_seed(11)
    edge = torch.randint(0, N, (2, EDGES), generator=g)             # (u, v) drawn independently: directed
    x = torch.randn(N, F_IN, generator=g)
    y = torch.randint(0, CLASSES, (N,), generator=g)
    mask = torch.rand(N, generator=g) < 0.7
    return edge, x, y, mask


def _dense_operator(adj, normalization, unit_values=False):
    """n x n matrix of the edge list (duplicates add up), optionally D^-1/2 . D^-1/2 with D the row counts."""
    a = torch.zeros(N, N, dtype=torch.float64)
    a.index_put_((adj[0], adj[1]), torch.ones(adj.size(1), dtype=torch.float64), accumulate=True)
    if unit_values:
        a = (a > 0).double()
    if normalization:
        d = torch.bincount(adj[0], minlength=N).double().pow(-0.5)
        a = d[:, None] * a * d[None, :]
    return a


def _expect(m, x, y, mask, row_sets, activations=True):
    """fp64 epochs of out = log_softmax(M relu(M X W1) W2) with loss = sum over `row_sets` of the mean NLL over the
    set's train rows, Adam(lr 0.01); the weights start as the package seeds them."""
    torch.manual_seed(0)
    w1 = torch.rand(F_IN, MID).double().requires_grad_()
    w2 = torch.rand(MID, CLASSES).double().requires_grad_()
    opt = torch.optim.Adam([w1, w2], lr=0.01)
    xs, out = x.double(), {}
    for ep in range(EPOCHS):
        h = m @ xs @ w1
        h = torch.relu(h) if activations else h
        z = m @ h @ w2
        o = torch.log_softmax(z, dim=1) if activations else z
        loss = 0.0
        for rows in row_sets:
            sel = rows[mask[rows]]
            if sel.numel():
                loss = loss - o[sel, y[sel]].mean()
        opt.zero_grad()
        loss.backward()
        out[f"ep{ep}_out"], out[f"ep{ep}_gw1"], out[f"ep{ep}_gw2"] = o.detach().numpy(), w1.grad.numpy().copy(), \
            w2.grad.numpy().copy()
        opt.step()
        out[f"ep{ep}_w1"], out[f"ep{ep}_w2"] = w1.detach().numpy().copy(), w2.detach().numpy().copy()
    return out


def _record(model):
    out = {}
    for ep in range(EPOCHS):
        o = model.train()
        out[f"ep{ep}_out"] = o.detach().numpy().copy()
        out[f"ep{ep}_gw1"] = model.weight1.grad.numpy().copy()
        out[f"ep{ep}_gw2"] = model.weight2.grad.numpy().copy()
        out[f"ep{ep}_w1"] = model.weight1.detach().numpy().copy()
        out[f"ep{ep}_w2"] = model.weight2.detach().numpy().copy()
    return out


def _check(results, want, place, what="directed"):
    for rank, res in enumerate(results):
        if res is None:
            continue
        rows, cols = place(rank)
        for ep in range(EPOCHS):
            np.testing.assert_allclose(res[f"ep{ep}_out"], want[f"ep{ep}_out"][rows][:, cols], rtol=1e-4, atol=2e-5,
                                       err_msg=f"{what} rank {rank} epoch {ep} out")
            for key in ("gw1", "gw2", "w1", "w2"):
                np.testing.assert_allclose(res[f"ep{ep}_{key}"], want[f"ep{ep}_{key}"], rtol=1e-4, atol=2e-5,
                                           err_msg=f"{what} rank {rank} epoch {ep} {key}")


# ------------------------------------------------------------------------------------------ 1D / 1.5D
def _worker_1d(rank, world, replication, collective, groups, order, directed):
    from cagnet_b200 import dist1d, graphs
    from oracle.cpu_backend import CpuBackend
    edge, x, y, mask = _problem()
    adj = graphs.add_self_loops(edge, N)
    rt = dist1d.Runtime(CpuBackend(), True, True, replication, order=order, stage_groups=groups,
                        collective=collective, directed=directed)
    group, row_groups, col_groups = dist1d.make_groups(rank, world, replication)
    model = dist1d.Model(rt, rank, world, x, adj, dist1d.Data(y=y, train_mask=mask), F_IN, CLASSES, group,
                         row_groups, col_groups)
    model.init_weights(MID)
    return _record(model)


@pytest.mark.parametrize("world,replication,collective,groups,order", [
    (3, 1, "all_gather", 2, "reference"), (3, 1, "broadcast", 0, "reference"), (3, 1, "all_gather", 1, "min_width"),
    (4, 2, "all_gather", -1, "reference"), (1, 1, "all_gather", 1, "reference")])
def test_1d_directed_graph(world, replication, collective, groups, order):
    from cagnet_b200 import graphs
    edge, x, y, mask = _problem()
    adj = graphs.add_self_loops(edge, N)
    m = _dense_operator(adj, True).t()                   # the 1D blocks hold the transpose (gcn_distr.py:546)
    per = math.ceil(N / (world // replication))
    row_sets = [torch.arange(r * per, min(N, (r + 1) * per)) for r in range(world // replication)]
    # one local mean per block row: with replication the weight gradient is summed inside a replica column, which
    # holds every block row once
    want = _expect(m, x, y, mask, row_sets)
    results = run_ranks(world, _worker_1d, replication, collective, groups, order, True)
    _check(results, want, lambda rank: (slice((rank // replication) * per, min(N, (rank // replication + 1) * per)),
                                        slice(None)))


def test_1d_without_the_flag_differs_on_a_directed_graph():
    """The reference's backward (forward blocks reused) is NOT the gradient on this graph: the flag matters."""
    from cagnet_b200 import graphs
    edge, x, y, mask = _problem()
    adj = graphs.add_self_loops(edge, N)
    m = _dense_operator(adj, True).t()
    per = math.ceil(N / 3)
    want = _expect(m, x, y, mask, [torch.arange(r * per, min(N, (r + 1) * per)) for r in range(3)])
    plain = run_ranks(3, _worker_1d, 1, "all_gather", 1, "reference", False)
    np.testing.assert_allclose(plain[0]["ep0_out"], want["ep0_out"][:per], rtol=1e-4, atol=2e-5)   # same forward
    assert np.abs(plain[0]["ep0_gw1"] - want["ep0_gw1"]).max() > 1e-3 * np.abs(want["ep0_gw1"]).max()


# ------------------------------------------------------------------------------------------ 2D
def _worker_2d(rank, world, directed):
    from cagnet_b200 import dist2d, graphs
    from oracle.cpu_backend import CpuBackend
    edge, x, y, mask = _problem()
    adj = graphs.add_self_loops(edge, N)
    rt = dist2d.Runtime(CpuBackend(), True, True, reference_label_alignment=False, directed=directed)
    model = dist2d.Model(rt, rank, world, x, adj, dist2d.Data(y=y, train_mask=mask), F_IN, CLASSES)
    model.init_weights(MID)
    return _record(model)


def test_2d_directed_graph():
    from cagnet_b200 import graphs
    edge, x, y, mask = _problem()
    adj = graphs.add_self_loops(edge, N)
    want = _expect(_dense_operator(adj, True), x, y, mask, [torch.arange(N)])
    results = run_ranks(4, _worker_2d, True)
    half, ch = N // 2, CLASSES // 2
    _check(results, want, lambda rank: (slice((rank // 2) * half, (rank // 2 + 1) * half),
                                        slice((rank % 2) * ch, (rank % 2 + 1) * ch)))
    plain = run_ranks(4, _worker_2d, False)
    assert np.abs(plain[0]["ep0_gw1"] - want["ep0_gw1"]).max() > 1e-3 * np.abs(want["ep0_gw1"]).max()


# ------------------------------------------------------------------------------------------ 3D
def _worker_3d(rank, world, normalization, directed):
    from cagnet_b200 import dist3d, graphs
    from oracle.cpu_backend import CpuBackend
    edge, x, y, mask = _problem()
    adj = graphs.add_self_loops(edge, N) if normalization else edge
    rt = dist3d.Runtime(CpuBackend(), activations=True, normalization=normalization,
                        reference_label_alignment=False, directed=directed)
    model = dist3d.Model(rt, rank, world, x, adj, dist3d.Data(y=y, train_mask=mask), F_IN, CLASSES)
    model.init_weights(MID)
    return _record(model)


@pytest.mark.parametrize("normalization", [True, False])
def test_3d_directed_graph(normalization):
    from cagnet_b200 import graphs
    edge, x, y, mask = _problem()
    adj = graphs.add_self_loops(edge, N) if normalization else edge
    # without normalisation the 3D slabs carry unit values (gcn_distr_3d.py:1357-1364)
    want = _expect(_dense_operator(adj, normalization, unit_values=not normalization), x, y, mask, [torch.arange(N)])
    results = run_ranks(8, _worker_3d, normalization, True)
    half, quarter, ch = N // 2, N // 4, CLASSES // 2

    def place(rank):
        i, j, k = rank // 4, (rank // 2) % 2, rank % 2
        r0 = i * half + k * quarter
        return slice(r0, r0 + quarter), slice(j * ch, (j + 1) * ch)

    _check(results, want, place)
