"""Benchmark of the GCN hot path: one step = one full-batch training epoch (2 layers forward, masked NLL,
backward, Adam) over N GPUs of one node (strong scaling: the graph is fixed, the ranks split it).

    python bench.py [--gpus N] [--steps K] [--warmup W]          one JSON line on stdout (rank 0)
    python bench.py --impl reference ...                         the CPU restatement of the reference, same line
    python bench.py --workload cfg3 --algorithm 15d --gpus 8     the other BASELINE configurations at full size
    python bench.py --workload cfg4 --algorithm 3d,1d --gpus 8   several algorithms on one generated graph (one line each)

Default: the 1D algorithm on the 232,965-vertex / ~114.6 M-nonzero synthetic R-MAT graph with 602 input features,
16 hidden units and 41 classes (BASELINE configuration 2, the one the metric is quoted on).
For N > 1 launch through `python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N`.

Before anything is timed, every run trains ONE epoch of a small seeded graph with the same algorithm on the same
N ranks through the CUDA + NCCL path and compares outputs, loss and weight gradients with the CPU oracle evaluated
for the same rank count (`"parity"` in the line); a mismatch beyond 1e-4 (1e-3 for the weight gradients, which are
sums of thousands of signed terms) ends the run with a non-zero exit code.
"""
import argparse
import json
import math
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

HIDDEN = 16
METRIC, UNIT = "gcn_epoch_ms", "ms"
RMAT = "R-MAT(.57,.19,.19,.05)"
WORKLOADS = {
    "cfg2": {"spec": "rmat:n=232965,nnz=114600000,f=602,c=41,train=0.66", "algorithm": "1d",
             "name": "2-layer GCN epoch, " + RMAT + " 232965 vertices ~114.6M nonzeros sym-normalised fp32, "
                     "features 602 N(0,1), hidden 16, 41 classes, 66% train mask, Adam lr 0.01"},
    "cfg3": {"spec": "rmat:n=14249639,nnz=230800000,f=300,c=24", "algorithm": "15d",
             "name": "2-layer GCN epoch, " + RMAT + " 14249639 vertices ~230.8M nonzeros sym-normalised fp32, "
                     "features 300 N(0,1), hidden 16, 24 classes, Adam lr 0.01"},
    "cfg4": {"spec": "rmat:n=8745542,nnz=1310000000,f=128,c=256", "algorithm": "2d",
             "name": "2-layer GCN epoch, " + RMAT + " 8745542 vertices ~1.31B nonzeros sym-normalised fp32, "
                     "features 128 N(0,1), hidden 16, 256 classes, Adam lr 0.01"},
    # a few seconds end to end: for trying the harness itself
    "tiny": {"spec": "rmat:n=30011,nnz=900000,f=130,c=12,train=0.66", "algorithm": "1d",
             "name": "2-layer GCN epoch, " + RMAT + " 30011 vertices ~0.9M nonzeros (harness check)"},
}
PARITY_SPEC = "rmat:n=4099,nnz=600000,f=160,c=10,train=0.66"
NVLINK_MEASURED_GBS, NVLINK_NOMINAL_GBS = 770.0, 900.0      # peer copy per direction measured on this pool; nominal
TRAFFIC_FILE = os.path.join("profiles", "spmm_f602_traffic.json")


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
        blk = model.am_pbyp.groups[0].block if hasattr(model, "am_pbyp") else model.adj_block
        if blk.core is None:
            return None
        rows, cols = blk.core_shape()
        return {"rows": rows, "cols": cols, "nnz": int(blk.nnz - blk.rest.nnz), "kind": blk.core_kind(),
                "tensor_cores": blk.core_kind() in ("bf16-integer", "3xtf32")}
    except (AttributeError, IndexError):      # an informational field must not cost the line
        return None


def spmm_traffic_bytes():
    """DRAM bytes per launch of the dominant SpMM of the default workload on ONE GPU, from the committed ncu
    summary (not measured in this run), or None."""
    try:
        with open(os.path.join(ROOT, TRAFFIC_FILE)) as fh:
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


# ------------------------------------------------------------------------------------------ models
def setup_distributed(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29512")
    return rank, world, local


def load_problem(spec, device):
    from cagnet_b200 import datasets, graphs
    x, edge, data, f, classes, info = datasets.load(spec, device=device)
    adj = graphs.add_self_loops(edge, x.size(0))
    return x, adj, data, f, classes, info


def check_ranks(algo, world, replication):
    if algo == "15d" and (world % replication or (world // replication) % replication):
        raise SystemExit("bench.py: the 1.5D algorithm needs P divisible by c^2 (P = %d, c = %d)" % (world, replication))
    if algo == "2d" and int(math.isqrt(world)) ** 2 != world:
        raise SystemExit("bench.py: the 2D algorithm needs a square number of ranks, got %d" % world)
    if algo == "3d" and round(world ** (1.0 / 3.0)) ** 3 != world:
        raise SystemExit("bench.py: the 3D algorithm needs a cubic number of ranks, got %d" % world)


class Context:
    """Process groups are created once per process and shared by the parity model and the timed model."""

    def __init__(self, rank, world, device):
        self.rank, self.world, self.device = rank, world, device
        self.groups1d = {}
        self.grid2d = self.grid3d = None
        self.prefetch_group = None


def make_model(ctx, algo, args, x, adj, data, f, classes):
    """-> (model, rt): the package's own Model of the algorithm, built from the whole graph on this rank's GPU."""
    from cagnet_b200 import dist1d, dist2d, dist3d
    from cagnet_b200.backend import CudaBackend
    rank, world = ctx.rank, ctx.world
    be = CudaBackend(ctx.device)
    if algo in ("1d", "15d"):
        c = 1 if algo == "1d" else args.replication
        rt = dist1d.Runtime(be, activations=True, normalization=True, replication=c, timing=False, overlap=True,
                            order=args.order, stage_groups=args.stage_groups, collective=args.collective,
                            prefetch_features=bool(args.prefetch) and algo == "1d" and world > 1)
        if c not in ctx.groups1d:
            ctx.groups1d[c] = dist1d.make_groups(rank, world, c)
        group, row_groups, col_groups = ctx.groups1d[c]
        rt.prefetch_group = ctx.prefetch_group
        model = dist1d.Model(rt, rank, world, x, adj, data, f, classes, group, row_groups, col_groups)
        ctx.prefetch_group = rt.prefetch_group
        return model, rt
    if algo == "2d":
        rt = dist2d.Runtime(be, activations=True, normalization=True, timing=False, overlap=True,
                            cache_blocks=bool(args.cache_blocks))
        if ctx.grid2d is None:
            ctx.grid2d = dist2d.Grid(rank, world)
        return dist2d.Model(rt, rank, world, x, adj, data, f, classes, grid=ctx.grid2d), rt
    rt = dist3d.Runtime(be, activations=True, normalization=True, timing=False, overlap=True,
                        cache_blocks=bool(args.cache_blocks))
    if ctx.grid3d is None:
        ctx.grid3d = dist3d.Grid(rank, world)
    return dist3d.Model(rt, rank, world, x, adj, data, f, classes, grid=ctx.grid3d), rt


def step_tensors(algo):
    """Names of the model attributes a step reads from the data loader: features, labels, mask."""
    return ("inputs_loc", "datay_rank", "rank_train_mask") if algo in ("1d", "15d") else ("inputs_loc", "y_eff", "mask_eff")


# ------------------------------------------------------------------------------------------ parity leg
def _gather_to_all(t, world):
    """Every rank's 2-D fp32 block on every rank: padded to the largest block, one all-gather."""
    if world == 1:
        return [t.detach().cpu()]
    t = t.contiguous()
    shape = torch.tensor([t.size(0), t.size(1)], device=t.device)
    shapes = [torch.empty_like(shape) for _ in range(world)]
    dist.all_gather(shapes, shape)
    rows, cols = max(int(s[0]) for s in shapes), max(int(s[1]) for s in shapes)
    pad = torch.zeros(rows, cols, device=t.device)
    pad[:t.size(0), :t.size(1)] = t
    out = torch.empty(world * rows, cols, device=t.device)
    dist.all_gather_into_tensor(out, pad)
    out = out.cpu()
    return [out[r * rows:r * rows + int(shapes[r][0]), :int(shapes[r][1])] for r in range(world)]


def oracle_expectation(algo, world, replication, x, adj, y, mask, classes):
    """fp64 CPU oracle of one epoch at P = world: (record, [(row slice, column slice) per rank], loss)."""
    from oracle import gcn as OG                     # the checker: never inside a timed region
    from oracle import partition as OP
    n, f = x.size(0), x.size(1)
    w1, w2 = OG.init_weights(f, HIDDEN, classes, torch.float64)
    if algo in ("1d", "15d"):
        c = 1 if algo == "1d" else replication
        n_per = math.ceil(n / (world / c))
        M = OG.matrix_1d(adj, x, world, True, c, dtype=torch.float64)
        rec = OG.epoch(M, x.double(), w1, w2, lambda o: OG.grad_local_mean(o, y, mask, n_per))
        slices = [(slice((r // c) * n_per, min(n, (r // c + 1) * n_per)), slice(None)) for r in range(world)]
        return rec, slices, float(rec["loss"])
    if algo == "2d":
        q = OP.grid_side_2d(world)
        M = OG.matrix_2d(adj, x, world, True, dtype=torch.float64)
        chunks, ranges = OG.row_chunks_2d(n, world), OG.class_ranges_2d(classes, world)
        vtx = OP.boundaries(n, n // q, keep=q)
        cs = [0]
        for w in OP.chunk_sizes(classes, q):
            cs.append(cs[-1] + w)
        slices = [(slice(vtx[r // q], vtx[r // q + 1]), slice(cs[r % q], cs[r % q + 1])) for r in range(world)]
    else:
        q = OP.grid_side_3d(world)
        M = OG.matrix_2d(adj, x, q * q, True, dtype=torch.float64)      # the 3D blocks are the q x q grid's, cut into slabs
        chunks, ranges = OG.row_chunks_3d(n, world), OG.class_ranges_3d(classes, world)
        cs = [0]
        for w in OP.chunk_sizes(classes, q):
            cs.append(cs[-1] + w)
        slices = []
        for r in range(world):
            i, j, k = OP.coords_3d(r, q)
            row0, length, _ = chunks[i * q + k]
            slices.append((slice(row0, row0 + length), slice(cs[j], cs[j + 1])))
    G = {}

    def rule(out):
        G["g"] = OG.grad_global_mean(out, y, mask, chunks, ranges)
        return G["g"]

    rec = OG.epoch(M, x.double(), w1, w2, rule)
    return rec, slices, float((rec["out"] * G["g"]).sum())


def parity_errors(algo, world, replication, model, out, x, adj, data, classes, rank):
    """One finished epoch of `model` against the oracle at the same P: {"out", "loss", "gW1", "gW2"} as
    max |err| / max |expected| on rank 0 (None elsewhere).  Collective: every rank calls it."""
    pieces = _gather_to_all(out.detach().float(), world)
    loss = model.last_loss.detach().clone().reshape(1).float()
    if world > 1:
        dist.all_reduce(loss)
    dup = replication if algo == "15d" else 1                                 # replicas hold the same rows
    loss = float(loss.item()) / dup
    gw1, gw2 = model.weight1.grad.detach().cpu(), model.weight2.grad.detach().cpu()
    if rank != 0:
        return None
    rec, slices, want_loss = oracle_expectation(algo, world, replication, x, adj, data.y, data.train_mask, classes)

    def rel(a, b):
        return float((a.double() - b).abs().max() / b.abs().max().clamp_min(1e-30))

    return {"out": max(rel(pieces[r], rec["out"][slices[r][0], slices[r][1]]) for r in range(world)),
            "loss": abs(loss - want_loss) / max(abs(want_loss), 1e-30),
            "gW1": rel(gw1, rec["gW1"]), "gW2": rel(gw2, rec["gW2"])}


def parity_leg(ctx, algo, args):
    """One epoch of PARITY_SPEC with `algo` on all ranks (CUDA kernels, NCCL) against the oracle at the same P."""
    rank, world, device = ctx.rank, ctx.world, ctx.device
    x, adj, data, f, classes, info = load_problem(PARITY_SPEC, "cpu")        # same tensors on every rank and for the oracle
    model, rt = make_model(ctx, algo, args, x.to(device), adj.to(device), data, f, classes)
    model.init_weights(HIDDEN)
    out = model.train()
    torch.cuda.synchronize(device)
    errs = parity_errors(algo, world, args.replication, model, out, x, adj, data, classes, rank)
    result = None
    if rank == 0:
        ok = errs["out"] <= 1e-4 and errs["loss"] <= 1e-4 and errs["gW1"] <= 1e-3 and errs["gW2"] <= 1e-3
        result = dict(errs, ok=ok, graph=PARITY_SPEC, nnz=info["nnz_with_self_loops"], algorithm=algo, P=world,
                      against="fp64 CPU oracle of the reference's epoch at the same P; max |err| / max |expected|; "
                              "bounds 1e-4 (out, loss), 1e-3 (weight gradients)")
    del model
    torch.cuda.empty_cache()
    flag = torch.tensor([1 if (result is None or result["ok"]) else 0], device=device)
    if world > 1:
        dist.broadcast(flag, src=0)
    return result, bool(flag.item())


# ------------------------------------------------------------------------------------------ collectives leg
def collectives_leg(model, rt, world, device, epochs=3):
    """Per collective of an epoch: calls, bytes a rank moves over NVLink, milliseconds (CUDA events around the
    blocking form of each call on the launching stream), bandwidth and its fraction of the link rate.  `ms` is the
    smallest figure over the ranks (the last rank to arrive sees the transfer alone), `ms_max` the largest (it
    includes waiting for the slowest rank)."""
    if world == 1:
        return None
    timers = rt.timers
    timers.links = {}
    timers.use_events(lambda: torch.cuda.Event(enable_timing=True))
    for _ in range(epochs):
        model.train()
    torch.cuda.synchronize(device)
    timers.flush_events()
    timers.enabled = timers.event_mode = False
    mine = {k: [v[0] / epochs, v[1] / epochs, v[2] / epochs] for k, v in timers.links.items()}
    everyone = [None] * world
    dist.all_gather_object(everyone, mine)
    names = []
    for rec in everyone:
        for k in rec:
            if k not in names:
                names.append(k)
    out = []
    for name in names:
        recs = [r[name] for r in everyone if name in r and r[name][0] > 0]
        nbytes = max(r[1] for r in recs)
        timed = [r[2] for r in recs if r[2] > 0]
        ms, ms_max = (min(timed), max(timed)) if timed else (None, None)
        gbs = nbytes / ms / 1e6 if ms else None
        out.append({"name": name, "calls_per_epoch": max(r[0] for r in recs), "bytes_per_rank": int(nbytes),
                    "ms": ms, "ms_max": ms_max, "gbs": gbs,
                    "frac_of_770": gbs / NVLINK_MEASURED_GBS if gbs else None,
                    "frac_of_900": gbs / NVLINK_NOMINAL_GBS if gbs else None})
    return out


# ------------------------------------------------------------------------------------------ library leg
def library_leg(model, widths, device):
    """cuSPARSE's SpMM (through torch.sparse.mm on a CUDA CSR tensor, the call the reference's op wraps:
    sparse_coo_tensor.cu:215-226) on the same block and widths, next to this library's kernels.  A baseline only:
    nothing in the package calls it."""
    from cagnet_b200 import ops
    blk = model.am_pbyp.groups[0].block
    A = torch.sparse_csr_tensor(blk.rowptr, blk.col, blk.val, size=(blk.n, blk.m))
    g = torch.Generator(device=device).manual_seed(5)
    res = {}
    for f in widths:
        B = torch.randn(blk.m, f, device=device, generator=g)
        Bp, Cp = ops.to_padded(B), ops.empty_padded(blk.n, f, device)

        def timed(fn):
            for _ in range(2):
                fn()
            ts = []
            for _ in range(5):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize(device)
                ts.append(e0.elapsed_time(e1))
            return statistics.median(ts)

        try:
            lib_ms = timed(lambda: torch.sparse.mm(A, B))
        except Exception as exc:                                   # an informational field must not cost the line
            res[str(f)] = {"error": str(exc)[:120]}
            continue
        ours_ms = timed(lambda: ops.spmm(blk, Bp, Cp, 0.0))
        res[str(f)] = {"cusparse_ms": lib_ms, "ours_ms": ours_ms, "speedup": lib_ms / ours_ms}
        del B, Bp, Cp
    return {"kind": "cuSPARSE SpMM via torch.sparse.mm (CUDA CSR int32, fp32), median of 5 launches, C = A.B",
            "block": [blk.n, blk.m, blk.nnz], "widths": res}


# ------------------------------------------------------------------------------------------ one algorithm
def run_algorithm(ctx, algo, args, workload, problem, data, f, classes, info, last):
    """`problem` = {"x": features, "adj": edge list}: emptied once the last algorithm's model is built, so that the
    21 GB edge list of the 1.31 B-edge graph is not held through the timed part."""
    rank, world, device = ctx.rank, ctx.world, ctx.device
    x, adj = problem["x"], problem["adj"]
    from cagnet_b200 import _native, ops

    parity, parity_ok = (None, True)
    if not args.no_parity:
        parity, parity_ok = parity_leg(ctx, algo, args)

    t_build = time.perf_counter()
    model, rt = make_model(ctx, algo, args, x, adj, data, f, classes)
    be = rt.backend
    nnz_total = int(adj.size(1))
    y_all, mask_all = data.y, data.train_mask
    del x, adj
    if last:
        problem.clear()
        torch.cuda.empty_cache()
    torch.cuda.synchronize(device)
    build_s = time.perf_counter() - t_build
    model.init_weights(HIDDEN)
    names = step_tensors(algo)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def reduce_max(ms):
        t = torch.tensor([ms], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        model.train()
    sampler = ClockSampler(device.index)
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
    ms_per_step = reduce_max(e0.elapsed_time(e1)) / args.steps
    loss_resident = float(model.last_loss.item())
    peak_mem = torch.cuda.max_memory_allocated(device)

    # ---- end to end: every step's features, labels and mask come from pinned host memory, the loss goes back.
    # Two device slots: the copy for step k+1 runs on a copy stream while step k computes (what a data loader
    # does); every step still consumes a copy made inside the timed region.
    cur = tuple(getattr(model, nm) for nm in names)
    hx = ops.base_buffer(cur[0]).cpu().pin_memory()          # padded rows: one contiguous DMA
    hy = cur[1].cpu().pin_memory()
    hm = cur[2].cpu().pin_memory()
    h2d = hx.numel() * 4 + hy.numel() * 8 + hm.numel()
    slots = [cur, (ops.empty_padded(cur[0].size(0), cur[0].size(1), device), torch.empty_like(cur[1]),
                   torch.empty_like(cur[2]))]
    copy_stream = torch.cuda.Stream(device)
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]
    for ev in consumed:
        ev.record()

    def prefetch(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])
            xs, ys, ms = slots[slot]
            ops.base_buffer(xs).copy_(hx, non_blocking=True)
            ys.copy_(hy, non_blocking=True)
            ms.copy_(hm, non_blocking=True)
            ready[slot].record(copy_stream)

    def drop_feature_prefetch():
        plan = getattr(model, "am_pbyp", None)
        if hasattr(plan, "prefetched"):
            plan.prefetched.clear()          # the next epoch gathers its own copy of the features

    def e2e_steps(count):
        loss = 0.0
        drop_feature_prefetch()
        prefetch(0)
        for k in range(count):
            slot = k % 2
            torch.cuda.current_stream().wait_event(ready[slot])
            for nm, t in zip(names, slots[slot]):
                setattr(model, nm, t)
            if k + 1 < count:
                prefetch(1 - slot)
                if getattr(rt, "prefetch_features", False):
                    rt.next_features = (slots[1 - slot][0], ready[1 - slot])   # the gather of step k+1 reads that copy
            elif getattr(rt, "prefetch_features", False):
                rt.next_features = None
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
    e2e_ms = reduce_max(e0.elapsed_time(e1)) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    for nm, t in zip(names, slots[0]):
        setattr(model, nm, t)
    if getattr(rt, "prefetch_features", False):
        rt.next_features = None

    # ---- the same epoch with the sparse products at the narrower width (reported beside, never as `value`)
    alt = None
    if algo in ("1d", "15d") and args.order == "reference" and not args.no_alt:
        rt.order = "min_width"
        for _ in range(3):
            model.train()
        barrier()
        e0.record()
        for _ in range(args.steps):
            model.train()
        e1.record()
        barrier()
        alt = {"order": "min_width: A.(H.W) in the narrowing layer, (A.H)^T.dZ and A.(dZ.W^T) in the widening one",
               "value": reduce_max(e0.elapsed_time(e1)) / args.steps, "unit": UNIT, "loss": float(model.last_loss.item())}
        rt.order = "reference"

    drop_feature_prefetch()
    collectives = collectives_leg(model, rt, world, device)

    if rank == 0:
        def alg_bytes(n_, m_, nnz_, f_, beta):
            return 4 * (n_ + 1) + 8 * nnz_ + 4 * m_ * f_ + 4 * n_ * f_ * (1 + int(beta != 0))

        # dominant kernel: the SpMM of layer 1's forward (the widest sparse product of the epoch)
        f_wide = max(f_ for (_, _, _, f_, _, _) in spmm_times)
        wide = [r for r in spmm_times if r[3] == f_wide]
        alg = sum(alg_bytes(*r[:5]) for r in wide)
        wide_ms = sum(r[5] for r in wide)
        all_alg = sum(alg_bytes(*r[:5]) for r in spmm_times)
        all_ms = sum(r[5] for r in spmm_times)
        per_width = {}
        for r in spmm_times:
            per_width.setdefault(r[3], []).append(r[5])
        peak, peak_kind = measured_peak_gbs()
        achieved = alg / wide_ms / 1e6 if wide_ms > 0 else 0.0
        calls = max(len(wide) // max(args.steps, 1), 1)
        launch_ms = wide_ms / max(len(wide), 1)
        sm_mhz = (clocks or {}).get("sm_mhz") or 1965.0
        fma_peak = 148 * 128 * 2 * sm_mhz * 1e6 / 1e12                       # TFLOP/s of fp32 FMA at the sampled clock
        flops = sum(2.0 * r[2] * r[3] for r in wide) / max(len(wide), 1)
        core_kernel = None
        if dense_core_info(model) is not None:
            core_kernel = {"bf16-integer": "tcgen05 kind::f16 (bf16 multiplicities x 3 bf16 terms)",
                           "3xtf32": "tcgen05 kind::tf32 (3xTF32)", "fp32-fma": "sgemm"}[dense_core_info(model)["kind"]]
        line = {
            "metric": METRIC, "value": ms_per_step, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload["name"], "algorithm": algo, "ranks": world, "nnz": nnz_total,
                       "vertices": info["n"], "l2": "inputs larger than L2 (CSR + features re-read every epoch)"},
            "spmm_gbs": all_alg / all_ms / 1e6 if all_ms > 0 else None,
            "spmm_ms_per_epoch": all_ms / args.steps,
            "spmm_ms_by_width": {str(k): sum(v) / args.steps for k, v in sorted(per_width.items())},
            "roofline": {"bound": "hbm",
                         "kernel": "spmm f=%d on rank 0 (hub-row and warp-per-row / lane-group launches on the sparse part; "
                                   "gather+split, tcgen05 multiplies in k chunks and row-add launches on a dense core)" % f_wide,
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak if peak else None,
                         "peak_source": peak_kind, "launch_ms": launch_ms, "calls_per_epoch": calls,
                         "traffic": spmm_traffic_bytes() if (world == 1 and args.workload == "cfg2" and algo == "1d") else None,
                         "traffic_source": ("ncu capture of this multiply on 1 GPU, committed as %s; not measured in this run"
                                            % TRAFFIC_FILE) if (world == 1 and args.workload == "cfg2" and algo == "1d") else None,
                         "fma_floor_ms": flops / (fma_peak * 1e12) * 1e3, "fma_peak_tflops": fma_peak,
                         "fma_peak_source": "148 SMs x 128 fp32 lanes x 2 flop x the SM clock sampled in this run",
                         "hbm_floor_ms": (alg / max(len(wide), 1)) / (peak * 1e9) * 1e3,
                         "binds": "neither floor: the gathers of B rows (4 nnz f bytes per multiply) run at the L2-to-SM "
                                  "rate on graphs this dense, at the DRAM rate on the sparse ones"},
            "e2e": {"value": e2e_ms, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": launches, "clocks": clocks, "loss": loss_resident, "loss_e2e": loss_host,
            "multiplication_order": args.order, "stage_groups": getattr(model, "launch_groups", args.stage_groups),
            "collective": args.collective,
            "feature_prefetch": bool(getattr(rt, "prefetch_features", False)),
            "alt_order": alt, "dense_core": dense_core_info(model), "core_kernel": core_kernel,
            "core_kernel_built": "tcgen05" if _native.lib().cagnet_core_gemm_tc_available() == 1 else "sgemm",
            "parity": parity, "collectives": collectives,
            "setup_s": build_s, "peak_device_bytes": int(peak_mem),
        }
        if world == 1 and algo == "1d" and args.workload in ("cfg2", "tiny"):
            M, X, y, mask = build_cpu_problem(model, y_all, mask_all)
            threads = os.cpu_count() or 1
            epoch_fn = cpu_epoch_timer(M, X, y, mask, classes, threads)
            cpu_ms, _ = epoch_fn()
            line["cpu_baseline"] = {"value": cpu_ms, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": "1 full epoch of the same workload, torch.sparse CSR fp32"}
            if not args.no_library:
                line["library_baseline"] = library_leg(model, sorted(per_width), device)
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    del model
    torch.cuda.empty_cache()
    return parity_ok


def run_ours(args):
    rank, world, local = setup_distributed(args)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback "
                         "(use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    workload = WORKLOADS[args.workload]
    algos = [a for a in (args.algorithm or workload["algorithm"]).split(",") if a]
    for a in algos:
        if a not in ("1d", "15d", "2d", "3d"):
            raise SystemExit("bench.py: unknown algorithm %r" % a)
        check_ranks(a, world, args.replication)
    ctx = Context(rank, world, device)
    x, adj, data, f, classes, info = load_problem(args.spec or workload["spec"], device)
    ok = True
    problem = {"x": x, "adj": adj}
    del x, adj
    for i, a in enumerate(algos):
        ok = run_algorithm(ctx, a, args, workload, problem, data, f, classes, info, i == len(algos) - 1) and ok
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not ok:
        raise SystemExit("bench.py: parity check against the oracle FAILED (see the \"parity\" field)")


def run_reference(args):
    """The reference's CPU math (oracle restatement, torch.sparse CSR) on all host threads, same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    device = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    from cagnet_b200 import partition
    workload = WORKLOADS[args.workload]
    x, adj, data, f, classes, info = load_problem(args.spec or workload["spec"], device)
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
        "config": {"workload": workload["name"], "algorithm": "single process (the 1D math with P = 1)", "nnz": nnz_total,
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
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS),
                    help="cfg2: 233K vertices / 115M nonzeros / 602 features (the metric's configuration); cfg3: 14.25M / "
                         "231M / 300; cfg4: 8.75M / 1.31B / 128")
    ap.add_argument("--algorithm", default=None,
                    help="1d, 15d, 2d or 3d, or a comma-separated list run one after the other on the same graph "
                         "(default: the workload's own: cfg2 1d, cfg3 15d, cfg4 2d)")
    ap.add_argument("--replication", type=int, default=2, help="replication factor c of the 1.5D algorithm")
    ap.add_argument("--spec", default=None, help="graph spec overriding the workload's (see cagnet_b200.datasets)")
    ap.add_argument("--order", default="reference", choices=["reference", "min_width"],
                    help="reference: (A.H).W as the reference computes it; min_width: sparse products at the narrower width")
    ap.add_argument("--collective", default="all_gather", choices=["all_gather", "broadcast"],
                    help="how H blocks travel in a 1D sparse product: one all-gather per launch group, or one "
                         "broadcast per source rank as the reference issues them")
    ap.add_argument("--stage-groups", type=int, default=-1,
                    help="launch groups per distributed sparse product (0 = one per stage, as the reference; -1 = automatic)")
    ap.add_argument("--prefetch", type=int, default=1,
                    help="1D all-gather schedule: post the next epoch's layer-1 feature gather under the current epoch (1) or not (0)")
    ap.add_argument("--cache-blocks", type=int, default=1,
                    help="2D / 3D: receivers keep the adjacency blocks after the first epoch (1) or they are re-broadcast "
                         "every epoch as the reference does (0)")
    ap.add_argument("--no-parity", action="store_true", help="skip the small-graph parity epoch")
    ap.add_argument("--no-alt", action="store_true", help="skip the min_width side measurement")
    ap.add_argument("--no-library", action="store_true", help="skip the cuSPARSE side measurement")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
