"""The four entry scripts end to end on one GPU: flags -> synthetic graph -> partition -> timed runs -> report."""
import importlib
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

COMMON = ["--accperrank=1", "--epochs=3", "--graphname=er:n=3000,deg=8,f=20,c=6,train=0.7", "--timing=True",
          "--midlayer=8"]


@pytest.mark.parametrize("script,extra,width", [
    ("gcn_distr", ["--runcount=2", "--normalization=True", "--activations=True", "--accuracy=True"], 6),
    ("gcn_distr_15d", ["--runcount=1", "--normalization=True", "--activations=True", "--replication=1"], 6),
    ("gcn_distr_2d", ["--runcount=1", "--normalization=True", "--activations=True", "--accuracy=True"], 6),
    ("gcn_distr_3d", [], 6),
    # backward over the transposed blocks (this package's flag), every script
    ("gcn_distr", ["--runcount=1", "--normalization=True", "--activations=True", "--directed=True"], 6),
    ("gcn_distr_15d", ["--runcount=1", "--normalization=True", "--activations=True", "--replication=1",
                       "--directed=True"], 6),
    ("gcn_distr_2d", ["--runcount=1", "--normalization=True", "--activations=True", "--directed=True"], 6),
    ("gcn_distr_3d", ["--directed=True"], 6),
])
def test_script_runs_and_reports(script, extra, width, capsys, monkeypatch):
    for var in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(var, raising=False)
    mod = importlib.import_module(script)
    out = mod.main(COMMON + extra)
    torch.cuda.synchronize()
    assert out is not None and tuple(out.shape) == (3000, width)
    assert torch.isfinite(out).all()
    text = capsys.readouterr().out
    assert "rank: 0 comm_time:" in text and "rank: 0 comp_time:" in text and "Epoch: 002" in text
    if "--accuracy=True" in extra:
        assert "Train:" in text
