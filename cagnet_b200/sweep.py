"""Standalone SpMM sweep on one GPU: `python -m cagnet_b200.sweep [--scales 20 22 24] [--widths 16 64 128 256 602]`.

R-MAT graphs with 2^scale vertices and edge factor 16 (symmetrised, self loops added, sym-normalised fp32 CSR)
times dense fp32 N(0,1) matrices of the given widths, C = A.B.  For every point: milliseconds (median of 5
launches by CUDA events on the launching stream, after 2 warm-up launches), algorithmic GB/s
(4(n+1) + 8 nnz + 4 m f + 4 n f bytes per launch) and its fraction of the HBM peak, and the no-reuse gather rate
(8 nnz + 4 nnz f bytes).  With --cpu the same product is timed through torch.sparse (CSR, all host threads) where
it fits the --cpu-seconds budget.  One JSON line per point on stdout.
"""
import argparse
import json
import os
import time

import torch

from . import graphs, ops, partition


def _median_ms(fn, iters=5, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]


def _peak_gbs():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--scales", type=int, nargs="+", default=[20, 22, 24])
    ap.add_argument("--widths", type=int, nargs="+", default=[16, 64, 128, 256, 602])
    ap.add_argument("--edge-factor", type=int, default=16)
    ap.add_argument("--cpu", action="store_true", help="also time torch.sparse CSR on the host")
    ap.add_argument("--cpu-seconds", type=float, default=20.0, help="skip CPU points estimated to take longer")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("cagnet_b200.sweep: no CUDA device (there is no CPU execution path)")
    dev = torch.device("cuda", torch.cuda.current_device())
    peak, peak_kind = _peak_gbs()
    for scale in args.scales:
        n = 1 << scale
        edge = graphs.rmat_graph(n, edge_factor=args.edge_factor, seed=1, device=dev)
        adj = graphs.add_self_loops(edge, n)
        del edge
        _, blocks = partition.oned_partition(0, 1, torch.zeros(n, 1, device=dev), adj, True)
        del adj
        blk = blocks[0]
        A = ops.CsrBlock.from_coo(blk.rows, blk.cols, blk.vals, n, n, row_scale=blk.row_scale, col_scale=blk.col_scale)
        del blocks, blk
        torch.cuda.empty_cache()
        cpu_mat, cpu_rate = None, None
        if args.cpu:
            cpu_mat = torch.sparse_csr_tensor(A.rowptr.cpu().long(), A.col.cpu().long(), A.val.cpu(), size=(n, n))
        for f in args.widths:
            B = ops.to_padded(torch.randn(n, f, device=dev, generator=torch.Generator(device=dev).manual_seed(2)))
            C = ops.empty_padded(n, f, dev)
            ms = _median_ms(lambda: ops.spmm(A, B, C, 0.0))
            alg = A.bytes_alg(f, 0.0)
            rec = {"scale": scale, "vertices": n, "nnz": A.nnz, "f": f, "ms": ms, "alg_gbs": alg / ms / 1e6,
                   "frac_of_hbm_peak": alg / ms / 1e6 / peak, "peak_gbs": peak, "peak_source": peak_kind,
                   "gather_gbs": (8 * A.nnz + 4 * A.nnz * f) / ms / 1e6, "hub_rows": A.long_rows(),
                   "dense_core": None if A.core is None else list(A.core_shape()) + [A.nnz - A.rest.nnz, A.core_kind()],
                   "dense_core_used": A.core is not None and f >= (ops.CORE["min_width_int"] if A.core_int is not None
                                                                    else ops.CORE["min_width"]), "cpu_ms": None,
                   "cpu_threads": None}
            if cpu_mat is not None:
                flops = 2.0 * A.nnz * f
                est = flops / cpu_rate if cpu_rate else 0.0
                if est <= args.cpu_seconds:
                    Bc = B.cpu().contiguous()
                    t0 = time.perf_counter()
                    torch.sparse.mm(cpu_mat, Bc)
                    dt = time.perf_counter() - t0
                    cpu_rate = flops / dt
                    rec["cpu_ms"], rec["cpu_threads"] = dt * 1e3, torch.get_num_threads()
                    del Bc
            print(json.dumps(rec), flush=True)
            del B, C
        del A, cpu_mat
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
