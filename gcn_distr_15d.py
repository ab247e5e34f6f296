"""1.5D full-batch GCN training (block rows over P/c processes, replication factor c) on B200 GPUs -- drop-in
for the reference script of the same name.

    torchrun --nproc-per-node 8 gcn_distr_15d.py --accperrank=8 --epochs=100 --graphname=Amazon --timing=False \
        --midlayer=16 --runcount=1 --replication=2 --normalization=True --activations=True
"""
from cagnet_b200 import dist1d, launch
from cagnet_b200.backend import CudaBackend


def main(argv=None):
    args = launch.parse_args("15d", argv)
    print(f"Arguments: epochs: {args.epochs} graph: {args.graphname} timing: {args.timing} mid: {args.midlayer} "
          f"norm: {args.normalization} act: {args.activations} acc: {args.accuracy} runs: {args.runcount} "
          f"rep: {args.replication}")
    rank, size, device = launch.init_distributed(args)
    if size % (args.replication ** 2) != 0 and size % args.replication != 0:
        raise SystemExit("the process count must be a multiple of the replication factor")
    inputs, adj_matrix, data, features, classes = launch.load_inputs(args, device)
    rt = dist1d.Runtime(CudaBackend(device), args.activations, args.normalization, args.replication, args.timing,
                        args.overlap, order=args.order, stage_groups=args.stagegroups, collective=args.collective,
                        directed=args.directed)
    model = dist1d.run(rank, size, inputs, adj_matrix, data, features, classes, rt, args.epochs, args.midlayer,
                       args.runcount, args.accuracy, printer=lambda *a: print(*a, flush=True))
    return None if model is None else model.outputs


if __name__ == "__main__":
    print(main())
