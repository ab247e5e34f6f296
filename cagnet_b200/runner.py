"""The epoch / timing loop shared by the 2D and 3D entry scripts: `run_count` runs, each reseeding the weights,
report of the median run by rank-0 wall time with the per-category breakdown (gcn_distr_2d.py:1212-1345,
gcn_distr_3d.py:1516-1647)."""
import statistics
import time

import torch
import torch.distributed as dist


def run_training(model, epochs, mid_layer, run_count, untimed_first_epoch, printer=print):
    rt, rank = model.rt, model.rank
    timers = rt.timers
    comm = model.grid.comm
    outputs = None

    def sync():
        if hasattr(rt.backend, "synchronize"):
            rt.backend.synchronize()

    for i in range(run_count):
        timers.start_run(i)
        model.init_weights(mid_layer)
        first = 0
        if untimed_first_epoch:                      # 3D: gcn_distr_3d.py:1548-1557; 2D times every epoch
            with timers.paused():
                outputs = model.train()
            first = 1
        if comm:
            dist.barrier(model.grid.group)
        sync()
        tstart = time.time()
        printer(f"Starting training... rank {rank} run {i}")
        for epoch in range(first, epochs):
            outputs = model.train()
            printer("Epoch: {:03d}".format(epoch))
        sync()
        timers.runs[i]["total_time"] = time.time() - tstart
    if comm:
        dist.barrier(model.grid.group)
    totals = [timers.runs[i]["total_time"] for i in range(run_count)]
    median_idx = totals.index(statistics.median_low(totals))
    if rank == 0:
        printer(f"total_times_r0: {totals}")
    printer(f"rank: {rank} median_idx: {median_idx}")
    timers.report(rank, median_idx, total_label="Time", printer=printer)
    printer(f"rank: {rank} {outputs}")
    model.outputs = outputs
    return model


def gather_outputs_2d(model, outputs):
    """All-gather the final activations along the process row (class columns) then the process column (vertex
    rows): gcn_distr_2d.py:1348-1379."""
    g = model.grid
    dense = outputs.detach().contiguous()
    if not g.comm:
        return dense
    from . import partition
    q = g.q
    c_sizes = partition.chunk_sizes(model.classes, q)
    pad = torch.zeros(dense.size(0), max(c_sizes), device=dense.device)
    pad[:, :dense.size(1)] = dense
    parts = [torch.empty_like(pad) for _ in range(q)]
    dist.all_gather(parts, pad, group=g.row_group)
    row_block = torch.cat([parts[j][:, :c_sizes[j]] for j in range(q)], dim=1)
    pad = torch.zeros(max(model.row_sizes), model.classes, device=dense.device)
    pad[:row_block.size(0)] = row_block
    parts = [torch.empty_like(pad) for _ in range(q)]
    dist.all_gather(parts, pad, group=g.col_group)
    return torch.cat([parts[i][:model.row_sizes[i]] for i in range(q)], dim=0)
