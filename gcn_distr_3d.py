"""3D (split-3D-SpMM) full-batch GCN training on a cubic grid of B200 GPUs -- drop-in for the reference script of
the same name (which takes only --accperrank --epochs --graphname --timing --midlayer and trains a linear,
unnormalised model; --normalization / --activations are additions and default to that behaviour).

    torchrun --nproc-per-node 8 gcn_distr_3d.py --accperrank=8 --epochs=50 --graphname=subgraph3 --timing=False \
        --midlayer=16
"""
from cagnet_b200 import dist3d, launch, runner
from cagnet_b200.backend import CudaBackend


def main(argv=None):
    args = launch.parse_args("3d", argv)
    rank, size, device = launch.init_distributed(args)
    inputs, adj_matrix, data, features, classes = launch.load_inputs(args, device)
    print("Processes: " + str(size), flush=True)
    rt = dist3d.Runtime(CudaBackend(device), args.activations, args.normalization, args.timing, args.overlap,
                        directed=args.directed)
    grid = dist3d.Grid(rank, size)
    print("Before partitioning...", flush=True)
    model = dist3d.Model(rt, rank, size, inputs, adj_matrix, data, features, classes, grid)
    print("After partitioning...", flush=True)
    runner.run_training(model, args.epochs, args.midlayer, args.runcount, untimed_first_epoch=True,
                        printer=lambda *a: print(*a, flush=True))
    return model.outputs


if __name__ == "__main__":
    print(main())
