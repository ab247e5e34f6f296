"""Flag surface of the entry scripts: the reference's flags, its string booleans and its required-argument rule."""
import os

import pytest

from cagnet_b200 import datasets, launch


def test_reference_flags_parse():
    a = launch.parse_args("1d", ["--accperrank=6", "--epochs=100", "--graphname=Reddit", "--timing=False",
                                 "--midlayer=16", "--runcount=1", "--normalization=True", "--activations=True"])
    assert (a.accperrank, a.epochs, a.graphname, a.midlayer, a.runcount) == (6, 100, "Reddit", 16, 1)
    assert a.timing is False and a.normalization is True and a.activations is True and a.accuracy is False
    b = launch.parse_args("15d", ["--epochs=2", "--graphname=Amazon", "--timing=True", "--midlayer=16", "--runcount=1",
                                  "--replication=2", "--local_rank=3"])
    assert b.replication == 2 and b.timing is True and b.normalization is False       # booleans default to off
    c = launch.parse_args("3d", ["--accperrank=8", "--epochs=5", "--graphname=subgraph3", "--timing=False",
                                 "--midlayer=16"])
    assert c.runcount == 1 and c.normalization is False and c.activations is False    # the reference's 3D model
    assert a.directed is False and c.directed is False               # the reference's backward unless asked
    d = launch.parse_args("2d", ["--epochs=2", "--graphname=Cora", "--timing=False", "--midlayer=16", "--runcount=1",
                                 "--directed=True"])
    assert d.directed is True


def test_missing_required_argument_exits():
    with pytest.raises(SystemExit):
        launch.parse_args("1d", ["--epochs=3", "--graphname=Cora"])


def test_graph_names_resolve_to_the_reference_shapes():
    assert datasets.parse_spec("Reddit") == ("rmat", {"n": 232965, "nnz": 114600000, "f": 602, "c": 41, "train": 0.66})
    assert datasets.parse_spec("Amazon")[1]["n"] == 14249639 and datasets.parse_spec("Amazon")[1]["f"] == 300
    assert datasets.parse_spec("subgraph3")[1]["c"] == 256
    assert datasets.parse_spec("rmat:scale=10,ef=8,f=4,c=3")[1]["n"] == 1024
    with pytest.raises(ValueError):
        datasets.parse_spec("NoSuchGraph")
    x, edge, data, f, classes, info = datasets.load("er:n=200,deg=6,f=5,c=3", device="cpu")
    assert x.shape == (200, 5) and data.y.max() < 3 and data.train_mask.all() and info["edges"] == edge.size(1)


def test_bench_arms_on_a_machine_without_a_gpu():
    """The reference arm of bench.py is the CPU restatement and runs anywhere; the product arm refuses to run without
    a CUDA device instead of falling back to anything."""
    import json
    import subprocess
    import sys
    import torch
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--workload", "tiny", "--steps", "1",
                          "--warmup", "0"], cwd=root, capture_output=True, text=True, timeout=300)
    assert ref.returncode == 0, ref.stderr[-500:]
    line = json.loads(ref.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "gcn_epoch_ms" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["e2e"]["h2d_bytes_per_step"] == 0
    if not torch.cuda.is_available():
        ours = subprocess.run([sys.executable, "bench.py", "--workload", "tiny"], cwd=root, capture_output=True,
                              text=True, timeout=300)
        assert ours.returncode != 0 and "no CPU fallback" in (ours.stderr + ours.stdout)
