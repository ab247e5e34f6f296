"""The distributed schedules on real GPUs over NCCL (one process per GPU), against the reference-generated
fixtures where the fixture's process count fits the box, else against the single-process oracle.
Skipped when fewer GPUs are visible than a case needs."""
import math
import os

import numpy as np
import pytest
import torch

from tests.mp_util import run_ranks

pytestmark = pytest.mark.gpu


def _gpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _worker(rank, world, algo, case_path, replication, activations, normalization):
    import numpy as np
    import torch
    from cagnet_b200 import dist1d, dist2d, dist3d, graphs
    from cagnet_b200.backend import CudaBackend

    d = np.load(case_path)
    n, f, mid, classes, epochs = d["cfg"][:5].tolist()
    edge, x, y, mask = (torch.from_numpy(d[k]) for k in ("edge_index", "x", "y", "mask"))
    adj = graphs.add_self_loops(edge, n) if normalization else edge
    be = CudaBackend()
    data = dist1d.Data(y=y, train_mask=mask)
    if algo in ("1d", "15d"):
        rt = dist1d.Runtime(be, activations, normalization, replication)
        group, row_groups, col_groups = dist1d.make_groups(rank, world, replication)
        model = dist1d.Model(rt, rank, world, x, adj, data, f, classes, group, row_groups, col_groups)
    elif algo == "2d":
        model = dist2d.Model(dist2d.Runtime(be, activations, normalization), rank, world, x, adj, data, f, classes)
    else:
        model = dist3d.Model(dist3d.Runtime(be, activations, normalization), rank, world, x, adj, data, f, classes)
    model.init_weights(mid)
    out = {}
    for ep in range(epochs):
        o = model.train()
        out[f"ep{ep}_out"] = o.detach().cpu().numpy().copy()
        out[f"ep{ep}_gw1"] = model.weight1.grad.cpu().numpy().copy()
        out[f"ep{ep}_gw2"] = model.weight2.grad.cpu().numpy().copy()
        out[f"ep{ep}_w1"] = model.weight1.detach().cpu().numpy().copy()
    return out


def _check_fixture(golden_dir, name, algo):
    path = os.path.join(golden_dir, name)
    d = np.load(path)
    n, f, mid, classes, epochs, P, c, norm, act = d["cfg"].tolist()
    if _gpus() < P:
        pytest.skip(f"needs {P} GPUs")
    if algo == "3d":
        act = norm = 0          # the reference's 3D script is linear and unnormalised whatever the flags say
    results = run_ranks(P, _worker, algo, path, c, bool(act), bool(norm), backend="nccl", timeout=600)
    for rank, res in enumerate(results):
        for ep in range(epochs):
            for key in ("out", "gw1", "gw2", "w1"):
                want = d[f"r{rank}_ep{ep}_{key}"]
                np.testing.assert_allclose(res[f"ep{ep}_{key}"], want, rtol=1e-4, atol=2e-5 * max(1.0, np.abs(want).max()),
                                           err_msg=f"{name} rank {rank} epoch {ep} {key}")


def test_1d_three_gpus_fixture(golden_dir):
    _check_fixture(golden_dir, "train_1d_P3.npz", "1d")


def test_15d_four_gpus_fixture(golden_dir):
    _check_fixture(golden_dir, "train_15d_P4.npz", "15d")


def test_15d_eight_gpus_fixture(golden_dir):
    _check_fixture(golden_dir, "train_15d_P8.npz", "15d")


def test_2d_four_gpus_fixture(golden_dir):
    _check_fixture(golden_dir, "train_2d_P4.npz", "2d")


def test_3d_eight_gpus_fixture(golden_dir):
    _check_fixture(golden_dir, "train_3d_P8.npz", "3d")


def test_1d_two_gpus_against_oracle(golden_dir):
    """No fixture was generated for P = 2: the expectation comes from the oracle (itself pinned to the fixtures)."""
    if _gpus() < 2:
        pytest.skip("needs 2 GPUs")
    from oracle import gcn as OG
    from oracle import partition as OP
    path = os.path.join(golden_dir, "train_1d_P1.npz")
    d = np.load(path)
    n, f, mid, classes, epochs = d["cfg"][:5].tolist()
    edge, x, y, mask = (torch.from_numpy(d[k]) for k in ("edge_index", "x", "y", "mask"))
    adj = OP.add_self_loops(edge, n)
    n_per = math.ceil(n / 2)
    M = OG.matrix_1d(adj, x, 2, True)
    rule = lambda y_, m_: (lambda out: OG.grad_local_mean(out, y_, m_, n_per))
    rec = OG.train(M, x, y, mask, mid, classes, epochs, rule, True)
    results = run_ranks(2, _worker, "1d", path, 1, True, True, backend="nccl", timeout=600)
    for rank, res in enumerate(results):
        rows = slice(rank * n_per, min(n, (rank + 1) * n_per))
        for ep in range(epochs):
            np.testing.assert_allclose(res[f"ep{ep}_out"], rec[ep]["out"][rows].numpy(), rtol=1e-4, atol=2e-5)
            np.testing.assert_allclose(res[f"ep{ep}_gw1"], rec[ep]["gW1"].numpy(), rtol=1e-4, atol=2e-5)
            np.testing.assert_allclose(res[f"ep{ep}_w1"], rec[ep]["W1"].numpy(), rtol=1e-4, atol=2e-5)


def _oracle_worker(rank, world, algo, replication):
    """One epoch of the benchmark's parity graph through the CUDA kernels and NCCL; rank 0 returns the errors
    against the fp64 oracle at the same rank count (what `bench.py` prints as "parity")."""
    import argparse
    import torch
    import bench
    args = argparse.Namespace(replication=replication, order="reference", stage_groups=-1, collective="all_gather",
                              prefetch=1, cache_blocks=1)
    ctx = bench.Context(rank, world, torch.device("cuda", rank))
    result, ok = bench.parity_leg(ctx, algo, args)
    return result


@pytest.mark.parametrize("algo,world,c", [("1d", 2, 1), ("1d", 4, 1), ("15d", 4, 2), ("2d", 4, 1), ("1d", 8, 1),
                                          ("15d", 8, 2), ("3d", 8, 1)])
def test_epoch_against_oracle_at_the_same_rank_count(algo, world, c):
    """Every schedule at P = 2, 4 or 8 on a 4,099-vertex R-MAT graph (normalised, activated, partial train mask, rows
    not divisible by P): rank-local outputs, loss and weight gradients against the oracle evaluated for that P."""
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    res = run_ranks(world, _oracle_worker, algo, c, backend="nccl", timeout=600)[0]
    assert res["ok"], res
    assert res["out"] <= 1e-4 and res["loss"] <= 1e-4 and res["gW1"] <= 1e-3 and res["gW2"] <= 1e-3
