"""1D (block-row) full-batch GCN training on B200 GPUs -- drop-in for the reference script of the same name.

    torchrun --nproc-per-node 8 gcn_distr.py --accperrank=8 --epochs=100 --graphname=Reddit --timing=False \
        --midlayer=16 --runcount=1 --normalization=True --activations=True

Same flags as the reference (README.md:59-71).  Graph names resolve to seeded synthetic graphs of the shapes the
reference hard-codes (see cagnet_b200/datasets.py); explicit `er:` / `rmat:` specs are accepted too.
"""
from cagnet_b200 import dist1d, launch
from cagnet_b200.backend import CudaBackend


def main(argv=None):
    args = launch.parse_args("1d", argv)
    print(f"Arguments: epochs: {args.epochs} graph: {args.graphname} timing: {args.timing} mid: {args.midlayer} "
          f"norm: {args.normalization} act: {args.activations} acc: {args.accuracy} runs: {args.runcount}")
    rank, size, device = launch.init_distributed(args)
    inputs, adj_matrix, data, features, classes = launch.load_inputs(args, device)
    rt = dist1d.Runtime(CudaBackend(device), args.activations, args.normalization, 1, args.timing, args.overlap,
                        order=args.order, stage_groups=args.stagegroups, collective=args.collective,
                        prefetch_features=args.prefetch and not args.timing, directed=args.directed)
    model = dist1d.run(rank, size, inputs, adj_matrix, data, features, classes, rt, args.epochs, args.midlayer,
                       args.runcount, args.accuracy, printer=lambda *a: print(*a, flush=True))
    return None if model is None else model.outputs


if __name__ == "__main__":
    print(main())
