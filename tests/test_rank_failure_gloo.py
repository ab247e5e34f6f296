"""Failure detection on the host, no GPU involved: a rank that leaves between two epochs (no collective of its
own in flight) must surface on the surviving rank as an exception from its next collective, within the
process-group timeout, instead of a hang.  Two Gloo ranks on CPU with the checker backend and a 5 s timeout."""
import datetime
import os
import sys
import time
import traceback

import torch.multiprocessing as mp

from tests.mp_util import ROOT, _free_port


def _leave(queue):
    queue.close()
    queue.join_thread()        # the message must be on the pipe before the process goes away
    os._exit(0)


def _rank(rank, world, port, case_path, queue):
    try:
        if ROOT not in sys.path:
            sys.path.insert(0, ROOT)
        import numpy as np
        import torch
        import torch.distributed as dist
        from cagnet_b200 import dist1d, graphs
        from oracle.cpu_backend import CpuBackend

        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        torch.set_num_threads(1)
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
        d = np.load(case_path)
        n, f, mid, classes = d["cfg"][:4].tolist()
        edge, x, y, mask = (torch.from_numpy(d[k]) for k in ("edge_index", "x", "y", "mask"))
        rt = dist1d.Runtime(CpuBackend(), True, True, 1)
        group, rows, cols = dist1d.make_groups(rank, world, 1)
        model = dist1d.Model(rt, rank, world, x, graphs.add_self_loops(edge, n), dist1d.Data(y=y, train_mask=mask), f,
                             classes, group, rows, cols)
        model.init_weights(mid)
        model.train()                                  # epoch 1: both ranks
        dist.barrier()
        if rank == 1:
            queue.put((rank, "left", 0.0))
            _leave(queue)                              # leaves between steps, nothing of its own in flight
        time.sleep(1.0)
        t0 = time.time()
        try:
            model.train()                              # epoch 2: the peer is gone
            queue.put((rank, "no error", time.time() - t0))
        except Exception as exc:                       # noqa: BLE001  (any error type will do: it must not hang)
            queue.put((rank, "raised " + type(exc).__name__, time.time() - t0))
        _leave(queue)
    except Exception:
        queue.put((rank, "setup failed: " + traceback.format_exc(), 0.0))


def test_departed_rank_raises_within_the_timeout(golden_dir):
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    path = os.path.join(golden_dir, "train_1d_P1.npz")
    procs = [ctx.Process(target=_rank, args=(r, 2, port, path, queue)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    try:
        for _ in range(2):
            rank, status, seconds = queue.get(timeout=120)
            got[rank] = (status, seconds)
    finally:
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.kill()
    assert got[1][0] == "left", got
    assert got[0][0].startswith("raised"), got
    assert got[0][1] < 60.0, got
