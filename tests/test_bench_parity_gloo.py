"""The benchmark's parity leg on CPU: the four schedules as Gloo ranks with the checker backend, compared by
`bench.parity_errors` with the fp64 oracle evaluated for the same rank count -- including the 3D algorithm in its
normalised, activated mode (the one the 1.31 B-edge configuration runs), which no reference fixture covers because
the reference's 3D script is linear and unnormalised."""
import pytest

from tests.mp_util import run_ranks

SPEC = "rmat:n=1031,nnz=40000,f=26,c=10,train=0.66"


def _worker(rank, world, algo, replication):
    import torch
    import bench
    from cagnet_b200 import dist1d, dist2d, dist3d
    from oracle.cpu_backend import CpuBackend

    x, adj, data, f, classes, _ = bench.load_problem(SPEC, "cpu")
    be = CpuBackend()
    if algo in ("1d", "15d"):
        c = 1 if algo == "1d" else replication
        rt = dist1d.Runtime(be, True, True, c, prefetch_features=(algo == "1d"))
        group, rows, cols = dist1d.make_groups(rank, world, c)
        model = dist1d.Model(rt, rank, world, x, adj, data, f, classes, group, rows, cols)
    elif algo == "2d":
        model = dist2d.Model(dist2d.Runtime(be, True, True), rank, world, x, adj, data, f, classes)
    else:
        model = dist3d.Model(dist3d.Runtime(be, True, True), rank, world, x, adj, data, f, classes)
    model.init_weights(bench.HIDDEN)
    out = model.train()
    return bench.parity_errors(algo, world, replication, model, out, x, adj, data, classes, rank)


@pytest.mark.parametrize("algo,world,c", [("1d", 2, 1), ("1d", 4, 1), ("15d", 8, 2), ("2d", 4, 1), ("3d", 8, 1)])
def test_parity_leg_over_gloo(algo, world, c):
    errs = run_ranks(world, _worker, algo, c)[0]
    assert errs["out"] <= 1e-4 and errs["loss"] <= 1e-4 and errs["gW1"] <= 1e-3 and errs["gW2"] <= 1e-3, errs
