"""Command line and process bootstrap shared by the four entry scripts (gcn_distr.py, gcn_distr_15d.py,
gcn_distr_2d.py, gcn_distr_3d.py): the reference's flags with its string-boolean convention
(gcn_distr.py:802-838), its OpenMPI / SLURM environment mapping and NCCL initialisation
(gcn_distr.py:689-712), then the algorithm's `run`."""
import argparse
import os
import socket

import torch
import torch.distributed as dist


def parse_args(algorithm, argv=None):
    p = argparse.ArgumentParser(description="full-batch GCN training, %s algorithm" % algorithm)
    p.add_argument("--local_rank", type=int)
    p.add_argument("--accperrank", type=int)
    p.add_argument("--epochs", type=int)
    p.add_argument("--graphname", type=str)
    p.add_argument("--timing", type=str)
    p.add_argument("--midlayer", type=int)
    if algorithm != "3d":
        p.add_argument("--runcount", type=int)
        p.add_argument("--normalization", type=str)
        p.add_argument("--activations", type=str)
        p.add_argument("--accuracy", type=str)
        p.add_argument("--download", type=bool)
    else:
        # not in the reference's 3D script (linear, unnormalised model); the defaults reproduce it
        p.add_argument("--runcount", type=int, default=1)
        p.add_argument("--normalization", type=str, default="False")
        p.add_argument("--activations", type=str, default="False")
        p.add_argument("--accuracy", type=str, default="False")
    if algorithm == "15d":
        p.add_argument("--replication", type=int)
    # additions of this package
    p.add_argument("--seed", type=int, default=1, help="seed of the synthetic graph")
    p.add_argument("--overlap", type=str, default="True", help="overlap the broadcast of block k+1 with the SpMM of block k")
    p.add_argument("--backend", type=str, default="nccl", help="torch.distributed backend (nccl)")
    p.add_argument("--order", type=str, default="reference", choices=["reference", "min_width"],
                   help="min_width: run every sparse product at the narrower of a layer's two widths")
    p.add_argument("--collective", type=str, default="all_gather", choices=["all_gather", "broadcast"],
                   help="1D: move H blocks with one all-gather per launch group, or one broadcast per source rank")
    p.add_argument("--prefetch", type=str, default="True",
                   help="1D all-gather schedule: post the next epoch's layer-1 feature gather under the current epoch")
    p.add_argument("--directed", type=str, default="False",
                   help="backward pass over the transposed adjacency blocks (a second copy of the graph): the true "
                        "gradients for an edge list that is not symmetric; the reference reuses the forward blocks")
    p.add_argument("--stagegroups", type=int, default=-1,
                   help="launch groups per sparse product (0 = one per stage, -1 = automatic)")
    args = p.parse_args(argv)
    print(args)
    missing = [k for k in ("epochs", "graphname", "timing", "midlayer", "runcount") if getattr(args, k) is None]
    if missing and not getattr(args, "download", False):
        print(f"Error: missing argument {args.epochs} {args.graphname} {args.timing} {args.midlayer} {args.runcount}")
        raise SystemExit(1)
    args.timing = args.timing == "True"
    args.normalization = args.normalization == "True"
    args.activations = args.activations == "True"
    args.accuracy = args.accuracy == "True"
    args.overlap = args.overlap == "True"
    args.prefetch = args.prefetch == "True"
    args.directed = args.directed == "True"
    if algorithm == "15d" and not args.replication:
        args.replication = 1
    if not args.accperrank:
        args.accperrank = max(torch.cuda.device_count(), 1)
    return args


def init_distributed(args):
    """RANK / WORLD_SIZE from OpenMPI or SLURM when present, MASTER_ADDR default 127.0.0.1, MASTER_PORT default
    1234 (the reference hard-codes it; a launcher's value is kept), device = rank % accperrank."""
    print(socket.gethostname())
    env = os.environ
    if "OMPI_COMM_WORLD_RANK" in env:
        env["RANK"] = env["OMPI_COMM_WORLD_RANK"]
    if "OMPI_COMM_WORLD_SIZE" in env and "WORLD_SIZE" not in env:
        env["WORLD_SIZE"] = env["OMPI_COMM_WORLD_SIZE"]
    if "SLURM_PROCID" in env:
        env["RANK"] = env["SLURM_PROCID"]
    if "SLURM_NTASKS" in env:
        env["WORLD_SIZE"] = env["SLURM_NTASKS"]
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    env.setdefault("MASTER_PORT", "1234")
    env.setdefault("RANK", "0")
    env.setdefault("WORLD_SIZE", "1")
    rank, size = int(env["RANK"]), int(env["WORLD_SIZE"])
    if not torch.cuda.is_available():
        raise SystemExit("cagnet_b200: no CUDA device visible; there is no CPU execution path")
    devid = rank % args.accperrank
    device = torch.device("cuda:{}".format(devid))
    torch.cuda.set_device(device)
    if size > 1:
        dist.init_process_group(backend=args.backend, device_id=device)
    print("Processes: " + str(size))
    print(f"device: {device}")
    return rank, size, device


def load_inputs(args, device):
    from . import datasets, graphs
    inputs, edge_index, data, features, classes, info = datasets.load(args.graphname, device=device, seed=args.seed)
    print(f"graph: {info}", flush=True)
    adj_matrix = graphs.add_self_loops(edge_index, inputs.size(0)) if args.normalization else edge_index
    return inputs, adj_matrix, data, features, classes
