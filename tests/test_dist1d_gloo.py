"""The 1D / 1.5D schedules of the package, run as Gloo ranks on CPU with the checker backend, against the
fixtures the reference's own scripts produced (same seeded inputs) and against the single-process oracle."""
import math
import os

import numpy as np
import pytest
import torch

from tests.mp_util import run_ranks


def _worker(rank, world, case_path, replication, activations, normalization, overlap, order="reference",
            stage_groups=2, collective="all_gather", prefetch=False):
    import numpy as np
    import torch
    from cagnet_b200 import dist1d, graphs
    from oracle.cpu_backend import CpuBackend

    d = np.load(case_path)
    n, f, mid, classes, epochs = d["cfg"][:5].tolist()
    edge, x, y, mask = (torch.from_numpy(d[k]) for k in ("edge_index", "x", "y", "mask"))
    adj = graphs.add_self_loops(edge, n) if normalization else edge
    rt = dist1d.Runtime(CpuBackend(), activations, normalization, replication, timing=False, overlap=overlap,
                        order=order, stage_groups=stage_groups, collective=collective, prefetch_features=prefetch)
    group, row_groups, col_groups = dist1d.make_groups(rank, world, replication)
    model = dist1d.Model(rt, rank, world, x, adj, dist1d.Data(y=y, train_mask=mask), f, classes, group, row_groups,
                         col_groups)
    model.init_weights(mid)
    out = {}
    for ep in range(epochs):
        o = model.train()
        out[f"ep{ep}_out"] = o.detach().numpy().copy()
        out[f"ep{ep}_gw1"] = model.weight1.grad.numpy().copy()
        out[f"ep{ep}_gw2"] = model.weight2.grad.numpy().copy()
        out[f"ep{ep}_w1"] = model.weight1.detach().numpy().copy()
        out[f"ep{ep}_w2"] = model.weight2.detach().numpy().copy()
    out["links"] = {k: list(v) for k, v in rt.timers.links.items()}
    return out


@pytest.mark.parametrize("groups", [1, 2])
def test_feature_prefetch_gives_the_same_epochs(golden_dir, groups):
    """The layer-1 all-gather of epoch k+1 posted during epoch k (own communicator, second buffer set) changes no
    number, and the same bytes are booked per epoch as without it (one gather more: the last one is never read)."""
    path = os.path.join(golden_dir, "train_1d_P3.npz")
    d = np.load(path)
    n, f, mid, classes, epochs, P, c, norm, act = d["cfg"].tolist()
    plain = run_ranks(P, _worker, path, c, True, True, True, "reference", groups, "all_gather", False)
    pre = run_ranks(P, _worker, path, c, True, True, True, "reference", groups, "all_gather", True)
    for rank in range(P):
        for ep in range(epochs):
            for key in ("out", "gw1", "gw2", "w1", "w2"):
                np.testing.assert_array_equal(pre[rank][f"ep{ep}_{key}"], plain[rank][f"ep{ep}_{key}"])
                np.testing.assert_allclose(pre[rank][f"ep{ep}_{key}"], d[f"r{rank}_ep{ep}_{key}"], rtol=1e-4, atol=2e-5)
        a, b = plain[rank]["links"]["h_all_gather"], pre[rank]["links"]["h_all_gather"]
        assert b[0] == a[0] + groups and b[1] > a[1]
        assert plain[rank]["links"]["grad_w_all_reduce"][0] == 2 * epochs


@pytest.mark.parametrize("name,overlap,groups,collective", [
    ("train_1d_P1.npz", True, 2, "all_gather"), ("train_1d_P3.npz", True, 0, "broadcast"),
    ("train_1d_P3.npz", False, 2, "broadcast"), ("train_1d_P3.npz", True, 1, "broadcast"),
    ("train_1d_P3.npz", True, 2, "all_gather"), ("train_1d_P3.npz", False, 1, "all_gather"),
    ("train_1d_P3.npz", True, 5, "all_gather"), ("train_1d_P3.npz", True, -1, "all_gather"),
    ("train_15d_P4.npz", True, -1, "all_gather"),
    ("train_1d_P1_plain.npz", True, 2, "all_gather"), ("train_15d_P4.npz", True, 2, "all_gather"),
    ("train_15d_P8.npz", True, 0, "broadcast"), ("train_15d_P8.npz", True, 2, "broadcast")])
def test_schedule_matches_reference_fixture(golden_dir, name, overlap, groups, collective):
    """broadcast with groups = 0: one broadcast + one multiply per stage (the reference's granularity); 1: all
    stages in one launch; 2: two launch groups; -1: the automatic rule.  all_gather: the 1D blocks travel in one collective per launch
    group (the fixture's last block is shorter than the others, so the padding path is exercised)."""
    path = os.path.join(golden_dir, name)
    d = np.load(path)
    n, f, mid, classes, epochs, P, c, norm, act = d["cfg"].tolist()
    results = run_ranks(P, _worker, path, c, bool(act), bool(norm), overlap, "reference", groups, collective)
    for rank, res in enumerate(results):
        for ep in range(epochs):
            for key in ("out", "gw1", "gw2", "w1", "w2"):
                np.testing.assert_allclose(res[f"ep{ep}_{key}"], d[f"r{rank}_ep{ep}_{key}"], rtol=1e-4, atol=2e-5,
                                           err_msg=f"{name} rank {rank} epoch {ep} {key}")


def test_15d_with_c1_is_the_1d_schedule(golden_dir):
    """Replication 1 through the 1.5D code path reproduces the 1D fixture (same stages, same sources)."""
    from cagnet_b200 import partition
    assert partition.stages_15d(2, 3, 1) == [(0, 0), (1, 1), (2, 2)]
    path = os.path.join(golden_dir, "train_1d_P3.npz")
    d = np.load(path)
    results = run_ranks(3, _worker, path, 1, True, True, True)
    np.testing.assert_allclose(results[1]["ep2_w1"], d["r1_ep2_w1"], rtol=1e-4, atol=2e-5)


@pytest.mark.parametrize("name", ["train_1d_P3.npz", "train_15d_P4.npz", "train_1d_P1_plain.npz"])
def test_min_width_order_gives_the_reference_results(golden_dir, name):
    """A.(H.W) when the layer narrows, (A.H)^T.dZ and A.(dZ.W^T) when it widens: same numbers as the reference
    order up to fp32 summation order (the fixture graphs are symmetric, as the reference's backward assumes)."""
    path = os.path.join(golden_dir, name)
    d = np.load(path)
    n, f, mid, classes, epochs, P, c, norm, act = d["cfg"].tolist()
    results = run_ranks(P, _worker, path, c, bool(act), bool(norm), True, "min_width")
    for rank, res in enumerate(results):
        for ep in range(epochs):
            for key in ("out", "gw1", "gw2", "w1", "w2"):
                want = d[f"r{rank}_ep{ep}_{key}"]
                np.testing.assert_allclose(res[f"ep{ep}_{key}"], want, rtol=1e-4, atol=2e-5 * max(1.0, np.abs(want).max()),
                                           err_msg=f"{name} rank {rank} epoch {ep} {key}")
