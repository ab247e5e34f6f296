"""2D (SUMMA) full-batch GCN training on a floor(sqrt(P)) x floor(sqrt(P)) grid of B200 GPUs -- drop-in for the
reference script of the same name.

    torchrun --nproc-per-node 4 gcn_distr_2d.py --accperrank=4 --epochs=50 --graphname=subgraph3 --timing=False \
        --midlayer=16 --runcount=1 --normalization=True --activations=True
"""
from cagnet_b200 import dist1d, dist2d, launch, runner
from cagnet_b200.backend import CudaBackend


def main(argv=None):
    args = launch.parse_args("2d", argv)
    print(f"Arguments: epochs: {args.epochs} graph: {args.graphname} timing: {args.timing} mid: {args.midlayer} "
          f"norm: {args.normalization} act: {args.activations} acc: {args.accuracy} runs: {args.runcount}")
    rank, size, device = launch.init_distributed(args)
    inputs, adj_matrix, data, features, classes = launch.load_inputs(args, device)
    print("Processes: " + str(size), flush=True)
    rt = dist2d.Runtime(CudaBackend(device), args.activations, args.normalization, args.timing, args.overlap,
                        directed=args.directed)
    grid = dist2d.Grid(rank, size)
    if not grid.active:                               # surplus ranks beyond the square grid do nothing
        return None
    model = dist2d.Model(rt, rank, size, inputs, adj_matrix, data, features, classes, grid)
    print(f"rank: {rank} adj_matrix_loc.nnz: {model.nnz_of[rank]}", flush=True)
    runner.run_training(model, args.epochs, args.midlayer, args.runcount, untimed_first_epoch=False,
                        printer=lambda *a: print(*a, flush=True))
    if args.accuracy:
        accs = dist1d.test(runner.gather_outputs_2d(model, model.outputs), data)
        print("Epoch: {:03d}, Train: {:.4f}, Val: {:.4f}, Test: {:.4f}".format(200, accs[0], accs[1], accs[2]))
    return model.outputs


if __name__ == "__main__":
    print(main())
