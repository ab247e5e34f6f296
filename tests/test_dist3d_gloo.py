"""The 3D (split-3D-SpMM) schedule as 8 Gloo ranks on CPU with the checker backend, against the fixture produced
by the reference's own gcn_distr_3d.py (linear, unnormalised model) on the same seeded inputs."""
import os

import numpy as np
import pytest

from tests.mp_util import run_ranks


def _worker(rank, world, case_path, cache_blocks, overlap, padded=False):
    import numpy as np
    import torch
    from cagnet_b200 import dist3d
    from oracle.cpu_backend import CpuBackend, PaddedCpuBackend
    Backend = PaddedCpuBackend if padded else CpuBackend

    d = np.load(case_path)
    n, f, mid, classes, epochs = d["cfg"][:5].tolist()
    edge, x, y, mask = (torch.from_numpy(d[k]) for k in ("edge_index", "x", "y", "mask"))
    rt = dist3d.Runtime(Backend(), activations=False, normalization=False, overlap=overlap, cache_blocks=cache_blocks)
    model = dist3d.Model(rt, rank, world, x, edge, dist3d.Data(y=y, train_mask=mask), f, classes)
    model.init_weights(mid)
    out = {}
    for ep in range(epochs):
        o = model.train()
        out[f"ep{ep}_out"] = o.detach().numpy().copy()
        out[f"ep{ep}_gw1"] = model.weight1.grad.numpy().copy()
        out[f"ep{ep}_gw2"] = model.weight2.grad.numpy().copy()
        out[f"ep{ep}_w1"] = model.weight1.detach().numpy().copy()
        out[f"ep{ep}_w2"] = model.weight2.detach().numpy().copy()
    return out


@pytest.mark.parametrize("cache_blocks,overlap,padded", [(True, True, False), (False, False, False), (True, True, True)])
def test_3d_matches_reference_fixture(golden_dir, cache_blocks, overlap, padded):
    path = os.path.join(golden_dir, "train_3d_P8.npz")
    d = np.load(path)
    epochs, P = int(d["cfg"][4]), int(d["cfg"][5])
    results = run_ranks(P, _worker, path, cache_blocks, overlap, padded)
    for rank, res in enumerate(results):
        for ep in range(epochs):
            for key in ("out", "gw1", "gw2", "w1", "w2"):
                want = d[f"r{rank}_ep{ep}_{key}"]
                # the model is linear and unnormalised: activations reach 1e3, so the absolute floor scales with them
                np.testing.assert_allclose(res[f"ep{ep}_{key}"], want, rtol=1e-4, atol=1e-5 * max(1.0, np.abs(want).max()),
                                           err_msg=f"rank {rank} epoch {ep} {key}")
