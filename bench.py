"""Benchmark of the GCN hot path: one step = one full-batch training epoch (2 layers forward, masked NLL,
backward, Adam) of the 1D algorithm on the 232,965-vertex / ~114.6 M-nonzero synthetic R-MAT graph with
602 input features, 16 hidden units and 41 classes, over N GPUs of one node (strong scaling: the graph is
fixed, P = N block rows).

    python bench.py [--gpus N] [--steps K] [--warmup W]          one JSON line on stdout (rank 0)
    python bench.py --impl reference ...                         the CPU restatement of the reference, same line

For N > 1 launch through `python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N`.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOAD = "rmat:n=232965,nnz=114600000,f=602,c=41,train=0.66"
WORKLOAD_NAME = ("1D 2-layer GCN epoch, R-MAT(.57,.19,.19,.05) 232965 vertices ~114.6M nonzeros sym-normalised fp32, "
                 "features 602 N(0,1), hidden 16, 41 classes, 66% train mask, Adam lr 0.01")
HIDDEN = 16
METRIC, UNIT = "gcn_epoch_ms", "ms"


# ------------------------------------------------------------------------------------------ helpers
def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def dense_core_info(model):
    """What rank 0's first adjacency block was split into (rows x columns of the dense core, its nonzeros, and
    whether it is multiplied on the tensor cores), or None when the block is all-sparse."""
    try:
        blk = model.am_pbyp.groups[0].block
        if blk.core is None:
            return None
        dense = blk.core[0]
        return {"rows": int(dense.size(0)), "cols": int(dense.size(1)), "nnz": int(blk.nnz - blk.rest.nnz),
                "tensor_cores": blk.core_split is not None}
    except (AttributeError, IndexError):      # an informational field must not cost the line
        return None


def spmm_traffic_bytes():
    """DRAM bytes per launch of the dominant SpMM from the committed ncu summary, or None."""
    try:
        with open(os.path.join(ROOT, "profiles", "spmm_f602_traffic.json")) as fh:
            return json.load(fh).get("dram_bytes_per_launch")
    except Exception:
        return None


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed regions run."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.idx, self.proc, self.path = device_index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.QUERY,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if not sm:
            return None
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "samples": len(sm), "reasons": sorted(reasons)}


def build_cpu_problem(model, data_y, data_mask):
    """Host copies of exactly the tensors the GPU run uses: the normalised matrix (CSR), features, labels, mask."""
    blk = model.am_pbyp.groups[0].block
    n = blk.n
    M = torch.sparse_csr_tensor(blk.rowptr.cpu().long(), blk.col.cpu().long(), blk.val.cpu(), size=(n, blk.m))
    X = model.inputs_loc.cpu().contiguous()
    return M, X, data_y.cpu(), data_mask.cpu()


def cpu_epoch_timer(M, X, y, mask, classes, threads):
    """One epoch of the CPU restatement (oracle) on `threads` host threads; returns a closure timing one epoch."""
    from oracle import gcn as OG                     # the checker, used here only as the timed CPU baseline
    torch.set_num_threads(threads)
    w1, w2 = OG.init_weights(X.size(1), HIDDEN, classes)
    w1, w2 = torch.nn.Parameter(w1), torch.nn.Parameter(w2)
    opt = torch.optim.Adam([w1, w2], lr=0.01)
    n = X.size(0)

    def one_epoch():
        t0 = time.perf_counter()
        with torch.no_grad():
            r = OG.epoch(M, X, w1.data, w2.data, lambda out: OG.grad_local_mean(out, y, mask, n), True)
        opt.zero_grad()
        w1.grad, w2.grad = r["gW1"], r["gW2"]
        opt.step()
        return (time.perf_counter() - t0) * 1e3, float(r["loss"])

    return one_epoch


# ------------------------------------------------------------------------------------------ arms
def setup_distributed(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29512")
    return rank, world, local


def load_problem(device):
    from cagnet_b200 import datasets, graphs
    x, edge, data, f, classes, info = datasets.load(WORKLOAD, device=device)
    adj = graphs.add_self_loops(edge, x.size(0))
    return x, adj, data, f, classes, info


def run_ours(args):
    rank, world, local = setup_distributed(args)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback "
                         "(use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    from cagnet_b200 import dist1d, ops
    from cagnet_b200.backend import CudaBackend

    x, adj, data, f, classes, info = load_problem(device)
    be = CudaBackend(device)
    rt = dist1d.Runtime(be, activations=True, normalization=True, replication=1, timing=False, overlap=True,
                        order=args.order, stage_groups=args.stage_groups, collective=args.collective)
    group, row_groups, col_groups = dist1d.make_groups(rank, world, 1)
    model = dist1d.Model(rt, rank, world, x, adj, data, f, classes, group, row_groups, col_groups)
    nnz_total = int(adj.size(1))
    y_all, mask_all = data.y, data.train_mask
    del x, adj
    torch.cuda.empty_cache()
    model.init_weights(HIDDEN)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    for _ in range(max(args.warmup, 3)):
        model.train()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()

    # ---- device-resident timed region
    barrier()
    be.start_spmm_timing()
    launches0 = ops.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()          # a profiler attached with "profile from start off" sees only this region
    e0.record()
    for _ in range(args.steps):
        model.train()
    e1.record()
    barrier()
    torch.cuda.profiler.stop()
    launches = ops.launch_count() - launches0
    spmm_times = be.stop_spmm_timing()
    t = torch.tensor([e0.elapsed_time(e1)], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    loss_resident = float(model.last_loss.item())

    # ---- end to end: every step's features, labels and mask come from pinned host memory, the loss goes back.
    # Two device slots: the copy for step k+1 runs on a copy stream while step k computes (what a data loader
    # does); every step still consumes a copy made inside the timed region.
    from cagnet_b200 import ops as _ops
    hx = _ops.base_buffer(model.inputs_loc).cpu().pin_memory()          # padded rows: one contiguous DMA
    hy = model.datay_rank.cpu().pin_memory()
    hm = model.rank_train_mask.cpu().pin_memory()
    h2d = hx.numel() * 4 + hy.numel() * 8 + hm.numel()
    slots = [(model.inputs_loc, model.datay_rank, model.rank_train_mask),
             (_ops.empty_padded(model.inputs_loc.size(0), model.inputs_loc.size(1), device),
              torch.empty_like(model.datay_rank), torch.empty_like(model.rank_train_mask))]
    copy_stream = torch.cuda.Stream(device)
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]
    for ev in consumed:
        ev.record()

    def prefetch(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])
            x, y, m = slots[slot]
            _ops.base_buffer(x).copy_(hx, non_blocking=True)
            y.copy_(hy, non_blocking=True)
            m.copy_(hm, non_blocking=True)
            ready[slot].record(copy_stream)

    def e2e_steps(count):
        loss = 0.0
        prefetch(0)
        for k in range(count):
            slot = k % 2
            torch.cuda.current_stream().wait_event(ready[slot])
            model.inputs_loc, model.datay_rank, model.rank_train_mask = slots[slot]
            if k + 1 < count:
                prefetch(1 - slot)
            model.train()
            consumed[slot].record()
            loss = float(model.last_loss.item())          # device -> host read of the step's result
        return loss

    e2e_steps(2)
    barrier()
    e0.record()
    loss_host = e2e_steps(args.steps)
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / args.steps
    clocks = sampler.stop() if rank == 0 else None

    # ---- the same epoch with the sparse products at the narrower width (reported beside, never as `value`)
    alt = None
    if args.order == "reference":
        rt.order = "min_width"
        for _ in range(3):
            model.train()
        barrier()
        e0.record()
        for _ in range(args.steps):
            model.train()
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        alt = {"order": "min_width: A.(H.W) in the narrowing layer, (A.H)^T.dZ and A.(dZ.W^T) in the widening one",
               "value": float(t.item()) / args.steps, "unit": UNIT, "loss": float(model.last_loss.item())}
        rt.order = "reference"

    if rank == 0:
        # dominant kernel: the SpMM against the 602-wide feature matrix (forward of layer 1)
        wide = [(n_, m_, nnz_, f_, beta, ms) for (n_, m_, nnz_, f_, beta, ms) in spmm_times if f_ == f]
        alg = sum(4 * (n_ + 1) + 8 * nnz_ + 4 * m_ * f_ + 4 * n_ * f_ * (1 + int(beta != 0)) for (n_, m_, nnz_, f_, beta, _) in wide)
        wide_ms = sum(ms for *_, ms in wide)
        all_alg = sum(4 * (n_ + 1) + 8 * nnz_ + 4 * m_ * f_ + 4 * n_ * f_ * (1 + int(beta != 0))
                      for (n_, m_, nnz_, f_, beta, _) in spmm_times)
        all_ms = sum(ms for *_, ms in spmm_times)
        peak, peak_kind = measured_peak_gbs()
        achieved = alg / wide_ms / 1e6 if wide_ms > 0 else 0.0
        line = {
            "metric": METRIC, "value": ms_per_step, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD_NAME, "algorithm": "1d", "ranks": world, "nnz": nnz_total,
                       "vertices": info["n"], "l2": "inputs larger than L2 (CSR 0.92 GB + features 0.56 GB per epoch)"},
            "spmm_gbs": all_alg / all_ms / 1e6 if all_ms > 0 else None,
            "spmm_ms_per_epoch": all_ms / args.steps,
            "roofline": {"bound": "hbm", "kernel": "spmm f=602 (hub-row and warp-per-row launches on the sparse part; gather+split, tcgen05 3xTF32 multiplies in k chunks and row-add launches on the dense core)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_kind, "launch_ms": wide_ms / max(len(wide), 1),
                         "traffic": spmm_traffic_bytes()},
            "e2e": {"value": e2e_ms, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": launches, "clocks": clocks, "loss": loss_resident, "loss_e2e": loss_host,
            "multiplication_order": args.order, "stage_groups": args.stage_groups, "collective": args.collective,
            "alt_order": alt,
            "dense_core": dense_core_info(model),
        }
        if world == 1:
            M, X, y, mask = build_cpu_problem(model, y_all, mask_all)
            threads = os.cpu_count() or 1
            epoch_fn = cpu_epoch_timer(M, X, y, mask, classes, threads)
            cpu_ms, _ = epoch_fn()
            line["cpu_baseline"] = {"value": cpu_ms, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": "1 full epoch of the same workload, torch.sparse CSR fp32"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args):
    """The reference's CPU math (oracle restatement, torch.sparse CSR) on all host threads, same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    device = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    from cagnet_b200 import partition
    x, adj, data, f, classes, info = load_problem(device)
    _, blocks = partition.oned_partition(0, 1, x, adj, True)
    blk = blocks[0]
    n = x.size(0)
    rowptr = torch.searchsorted(blk.rows.contiguous(), torch.arange(n + 1, device=blk.rows.device))
    M = torch.sparse_csr_tensor(rowptr.cpu(), blk.cols.cpu(), blk.vals.cpu(), size=(n, n))
    X, y, mask = x.cpu(), data.y.cpu(), data.train_mask.cpu()
    nnz_total = int(blk.vals.numel())
    del x, adj, blocks, blk
    threads = os.cpu_count() or 1
    epoch_fn = cpu_epoch_timer(M, X, y, mask, classes, threads)
    budget_s = 240.0
    t_start = time.perf_counter()
    times = []
    warm = max(args.warmup, 0)
    first, _ = epoch_fn()                                   # always one untimed epoch (thread pools, page faults)
    est = first / 1e3
    steps = args.steps
    done_warm = 1
    while done_warm < warm and (time.perf_counter() - t_start) + est * (steps + 1) < budget_s:
        epoch_fn()
        done_warm += 1
    for _ in range(steps):
        if times and (time.perf_counter() - t_start) + est > budget_s:
            break
        ms, _ = epoch_fn()
        times.append(ms)
    value = sum(times) / len(times)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": len(times), "warmup": done_warm, "ms_per_step": value, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD_NAME, "algorithm": "single process (the 1D math with P = 1)", "nnz": nnz_total,
                   "vertices": info["n"]},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "%d full epochs of the same workload (time-capped), torch.sparse CSR fp32" % len(times)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--order", default="reference", choices=["reference", "min_width"],
                    help="reference: (A.H).W as the reference computes it; min_width: sparse products at the narrower width")
    ap.add_argument("--collective", default="all_gather", choices=["all_gather", "broadcast"],
                    help="how H blocks travel in a 1D sparse product: one all-gather per launch group, or one "
                         "broadcast per source rank as the reference issues them")
    ap.add_argument("--stage-groups", type=int, default=-1,
                    help="launch groups per distributed sparse product (0 = one per stage, as the reference; -1 = automatic)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
