"""Generate the committed golden fixtures by running the reference's OWN Python code on CPU.

Usage (in a container that has the reference checkout; never at test time):

    python tests/golden/make_golden.py --reference /path/to/CAGNET --out tests/golden

What runs is the unmodified reference source (`gcn_distr.py`, `gcn_distr_15d.py`,
`gcn_distr_2d.py`, `gcn_distr_3d.py`), imported as modules.  Only what cannot exist on a
CPU-only box without network is replaced, at import time, by stand-ins defined in this file:

* `sparse_coo_tensor_cpp.spmm_gpu` (cuSPARSE in the reference, sparse_coo_tensor.cu:113-240):
  a CPU `C += A.B` through `torch.sparse.mm`, value semantics only.
* `sparse_coo_tensor_cpp.sparse_coo_tensor_gpu` (sparse_coo_tensor.cu:43-54):
  `torch.sparse_coo_tensor`.
* `torch_sparse.spspmm` (PyPI torch-sparse 0.4.3, un-vendored): a scipy CSR x CSR product in
  fp32 returning coalesced COO.  The reference only calls it with a diagonal operand
  (gcn_distr.py:458-464) so every output entry is exactly one fp32 product.
* `torch_geometric.utils.add_remaining_self_loops` (PyG 1.3.2): drop existing self loops, keep the
  other edges in order, append one (i, i) per vertex.
* `torch_geometric.data.Data`: attribute bag.  Other PyG / torch_scatter imports: empty stubs.
* `torch.cuda.FloatTensor` / `torch.cuda.LongTensor`: CPU constructors that ignore `device=`.
* NCCL -> Gloo process groups (one OS process per rank, 127.0.0.1 rendezvous).

The glue below that replaces the reference's `run()`/`main()` (weight seeding, Adam, calling
`train` once per epoch) follows gcn_distr.py:548-609, gcn_distr_15d.py:582-637,
gcn_distr_2d.py:1212-1302 and gcn_distr_3d.py:1516-1570.

Outputs: small `.npz` files (inputs AND reference outputs) that the tests read; the tests never
import the reference.
"""
import argparse
import importlib.util
import os
import socket
import sys
import types

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


# --------------------------------------------------------------------------- stand-ins
class _Data:
    def __init__(self, **kw):
        self.__dict__.update(kw)

    def to(self, *_a, **_k):
        return self

    def __call__(self, *keys):
        for k in keys:
            if k in self.__dict__:
                yield k, self.__dict__[k]


def _add_remaining_self_loops(edge_index, edge_weight=None, fill_value=1, num_nodes=None):
    n = int(edge_index.max()) + 1 if num_nodes is None else num_nodes
    keep = edge_index[0] != edge_index[1]
    loops = torch.arange(n, dtype=edge_index.dtype).unsqueeze(0).repeat(2, 1)
    return torch.cat([edge_index[:, keep], loops], dim=1), None


def _spspmm(index_a, value_a, index_b, value_b, m, k, n):
    import scipy.sparse as sp

    a = sp.csr_matrix((value_a.numpy().astype(np.float32),
                       (index_a[0].numpy(), index_a[1].numpy())), shape=(m, k))
    b = sp.csr_matrix((value_b.numpy().astype(np.float32),
                       (index_b[0].numpy(), index_b[1].numpy())), shape=(k, n))
    c = (a @ b).tocoo()
    order = np.lexsort((c.col, c.row))
    idx = torch.from_numpy(np.stack([c.row[order], c.col[order]]).astype(np.int64))
    return idx, torch.from_numpy(c.data[order].astype(np.float32))


def _spmm_gpu(rows, cols, vals, n, m, b, c):
    a = torch.sparse_coo_tensor(torch.stack([rows.long(), cols.long()]), vals, (n, m))
    c.add_(torch.sparse.mm(a, b))


def _sparse_coo_tensor_gpu(indices, values, size):
    return torch.sparse_coo_tensor(indices, values, size)


def _cpu_ctor(base):
    def ctor(*args, device=None):
        return base(*args)
    return ctor


def install_stubs(reference_dir):
    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    dummy = type("Dummy", (), {})
    mod("torch_geometric")
    mod("torch_geometric.data", Data=_Data, Dataset=dummy)
    mod("torch_geometric.datasets", Planetoid=dummy, PPI=dummy)
    mod("torch_geometric.nn", GCNConv=dummy, ChebConv=dummy)
    mod("torch_geometric.utils", add_remaining_self_loops=_add_remaining_self_loops,
        to_dense_adj=None, dense_to_sparse=None, to_scipy_sparse_matrix=None)
    mod("torch_geometric.transforms")
    mod("reddit", Reddit=dummy)
    mod("torch_scatter", scatter_add=None)
    mod("torch_sparse", spspmm=_spspmm)
    mod("sparse_coo_tensor_cpp", spmm_gpu=_spmm_gpu, sparse_coo_tensor_gpu=_sparse_coo_tensor_gpu)
    torch.cuda.FloatTensor = _cpu_ctor(torch.FloatTensor)
    torch.cuda.LongTensor = _cpu_ctor(torch.LongTensor)
    sys.path.insert(0, reference_dir)


def load_reference(reference_dir, fname):
    spec = importlib.util.spec_from_file_location("ref_" + fname[:-3], os.path.join(reference_dir, fname))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


# --------------------------------------------------------------------------- inputs
def make_case(n, avg_deg, f, classes, seed, train_frac=0.7):
    """Small seeded undirected graph (no self loops, both directions listed), features, labels, mask."""
    g = torch.Generator().manual_seed(seed)
    m = n * avg_deg // 2
    u = torch.randint(0, n, (m,), generator=g)
    v = torch.randint(0, n, (m,), generator=g)
    keep = u != v
    u, v = u[keep], v[keep]
    key = torch.unique(torch.minimum(u, v) * n + torch.maximum(u, v))
    lo, hi = key // n, key % n
    edge_index = torch.stack([torch.cat([lo, hi]), torch.cat([hi, lo])])
    # every vertex must occur (torch.histc bins span [min, max] of the row list)
    x = torch.randn(n, f, generator=g)
    y = torch.randint(0, classes, (n,), generator=g)
    mask = torch.rand(n, generator=g) < train_frac
    return edge_index, x, y, mask


def coo_np(t):
    t = t.coalesce()
    return t.indices().numpy().astype(np.int64), t.values().numpy().astype(np.float32), np.array(t.size(), dtype=np.int64)


# --------------------------------------------------------------------------- partition goldens
def partition_goldens(refdir, out):
    install_stubs(refdir)
    res = {}
    edge_index, x, y, mask = make_case(50, 6, 6, 5, seed=11)
    adj, _ = _add_remaining_self_loops(edge_index, num_nodes=50)
    res["edge_index"] = edge_index.numpy()
    res["adj_selfloops"] = adj.numpy()
    res["x"] = x.numpy()

    # ---- 1D: split_coo, scale_elements, oned_partition (gcn_distr.py:398-522)
    r1 = load_reference(refdir, "gcn_distr.py")
    r1.normalization = True
    for dim in (0, 1):
        parts, vtx = r1.split_coo(adj.clone(), 50, 13, dim)
        res[f"split1d_dim{dim}_vtx"] = np.array(vtx, dtype=np.int64)
        for i, p in enumerate(parts):
            res[f"split1d_dim{dim}_part{i}"] = p.numpy()
    for P in (1, 3, 4):
        for rank in range(P):
            xin, aloc, pbyp = r1.oned_partition(rank, P, x.clone(), adj.clone(), None, 6, 5, torch.device("cpu"))
            res[f"p1d_P{P}_r{rank}_inputs"] = xin.numpy()
            i, v, s = coo_np(aloc)
            res[f"p1d_P{P}_r{rank}_aloc_idx"], res[f"p1d_P{P}_r{rank}_aloc_val"], res[f"p1d_P{P}_r{rank}_aloc_size"] = i, v, s
            for b, blk in enumerate(pbyp):
                i, v, s = coo_np(blk.t())          # run() stores the transposed, coalesced block: gcn_distr.py:546
                res[f"p1d_P{P}_r{rank}_b{b}_idx"], res[f"p1d_P{P}_r{rank}_b{b}_val"], res[f"p1d_P{P}_r{rank}_b{b}_size"] = i, v, s
    # un-normalised variant for one P
    r1.normalization = False
    for rank in range(3):
        _, _, pbyp = r1.oned_partition(rank, 3, x.clone(), edge_index.clone(), None, 6, 5, torch.device("cpu"))
        for b, blk in enumerate(pbyp):
            i, v, s = coo_np(blk.t())
            res[f"p1d_nonorm_P3_r{rank}_b{b}_idx"], res[f"p1d_nonorm_P3_r{rank}_b{b}_val"] = i, v

    # ---- 1.5D (gcn_distr_15d.py:497-549)
    r15 = load_reference(refdir, "gcn_distr_15d.py")
    r15.normalization = True
    for P, c in ((4, 2), (8, 2)):
        r15.replication = c
        for rank in range(P):
            xin, aloc, pbyp = r15.oned_partition(rank, P, x.clone(), adj.clone(), None, 6, 5, torch.device("cpu"))
            res[f"p15d_P{P}c{c}_r{rank}_inputs"] = xin.numpy()
            for b, blk in enumerate(pbyp):
                i, v, s = coo_np(blk.t())
                res[f"p15d_P{P}c{c}_r{rank}_b{b}_idx"], res[f"p15d_P{P}c{c}_r{rank}_b{b}_val"], res[f"p15d_P{P}c{c}_r{rank}_b{b}_size"] = i, v, s

    # ---- 2D (gcn_distr_2d.py:1032-1164): n = 51 so that floor(51/2) leaves a remainder
    edge51, x51, _, _ = make_case(51, 6, 7, 5, seed=12)
    adj51, _ = _add_remaining_self_loops(edge51, num_nodes=51)
    res["edge_index51"], res["adj_selfloops51"], res["x51"] = edge51.numpy(), adj51.numpy(), x51.numpy()
    r2 = load_reference(refdir, "gcn_distr_2d.py")
    r2.normalization = True
    for P in (4, 9):
        for rank in range(P):
            xin, aloc, _ = r2.twod_partition(rank, P, x51.clone(), adj51.clone(), None, 7, 5, torch.device("cpu"))
            i, v, s = coo_np(aloc)
            res[f"p2d_P{P}_r{rank}_inputs"] = xin.numpy()
            res[f"p2d_P{P}_r{rank}_idx"], res[f"p2d_P{P}_r{rank}_val"], res[f"p2d_P{P}_r{rank}_size"] = i, v, s

    # ---- 3D (gcn_distr_3d.py:1272-1382); the script's normalization global is a hard-coded False
    r3 = load_reference(refdir, "gcn_distr_3d.py")
    for rank in range(8):
        xin, aloc, _ = r3.twod_partition(rank, 8, x51.clone(), edge51.clone(), None, 7, 5, torch.device("cpu"))
        aloc = aloc.coalesce()
        xin3, aloc3 = r3.threed_partition_loc(rank, 8, xin, aloc.indices(), aloc.size(0), aloc.size(1),
                                              None, 7, 5, torch.device("cpu"))
        i, v, s = coo_np(aloc3)
        res[f"p3d_P8_r{rank}_inputs"] = xin3.numpy()
        res[f"p3d_P8_r{rank}_idx"], res[f"p3d_P8_r{rank}_val"], res[f"p3d_P8_r{rank}_size"] = i, v, s

    # ---- communicator membership (dist.new_group replaced by "return the rank list")
    real_new_group = dist.new_group
    dist.new_group = lambda ranks=None, **_k: list(ranks)
    try:
        for P, c in ((4, 2), (8, 2), (8, 4)):
            r15.replication = c
            rows, cols = r15.get_proc_groups(0, P)
            res[f"groups15d_P{P}c{c}_rows"], res[f"groups15d_P{P}c{c}_cols"] = np.array(rows), np.array(cols)
        for P in (4, 9):
            rows, cols = r2.get_proc_groups(0, P, None)
            res[f"groups2d_P{P}_rows"], res[f"groups2d_P{P}_cols"] = np.array(rows), np.array(cols)
        rows, cols, cs = r3.get_proc_groups(0, 8, None)
        res["groups3d_P8_rows"], res["groups3d_P8_cols"], res["groups3d_P8_c"] = np.array(rows), np.array(cols), np.array(cs)
    finally:
        dist.new_group = real_new_group

    np.savez_compressed(os.path.join(out, "partition_golden.npz"), **res)
    print("wrote partition_golden.npz with", len(res), "arrays")


# --------------------------------------------------------------------------- training goldens
def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _train_worker(rank, size, port, refdir, algo, cfg, case, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(size))
    torch.set_num_threads(1)
    install_stubs(refdir)
    dist.init_process_group("gloo", rank=rank, world_size=size)
    edge_index, x, y, mask = (torch.from_numpy(a) for a in case)
    n, f = x.shape
    classes, mid, epochs = cfg["classes"], cfg["mid"], cfg["epochs"]
    cpu = torch.device("cpu")
    fname = {"1d": "gcn_distr.py", "15d": "gcn_distr_15d.py", "2d": "gcn_distr_2d.py", "3d": "gcn_distr_3d.py"}[algo]
    ref = load_reference(refdir, fname)
    ref.timing = False
    ref.device = cpu
    ref.acc_per_rank = 1
    ref.run = 0
    if algo != "3d":
        ref.normalization = cfg["normalization"]
        ref.activations = cfg["activations"]
    normalization = cfg["normalization"] and algo != "3d"
    # per-run timing accumulators are module-level dicts keyed [run][rank] (gcn_distr.py:42-51)
    for name, val in list(vars(ref).items()):
        if isinstance(val, dict) and not name.startswith("__") and (name.endswith("_time") or name.endswith("_words")
                                                                     or name.startswith("summa")):
            val[0] = {rank: 0.0}
    adj = _add_remaining_self_loops(edge_index, num_nodes=n)[0] if normalization else edge_index
    data = _Data(y=y, train_mask=mask)
    inputs = x.clone().requires_grad_(True)

    group = dist.new_group(list(range(size)))
    if algo == "1d":
        inputs_loc, adj_loc, pbyp = ref.oned_partition(rank, size, inputs, adj, data, f, classes, cpu)
        pbyp = [b.t().coalesce() for b in pbyp]
        step = lambda w1, w2, opt: ref.train(inputs_loc, w1, w2, adj_loc, pbyp, opt, data, rank, size, group)
    elif algo == "15d":
        ref.replication = cfg["replication"]
        row_groups, col_groups = ref.get_proc_groups(rank, size)
        inputs_loc, adj_loc, pbyp = ref.oned_partition(rank, size, inputs, adj, data, f, classes, cpu)
        pbyp = [b.t().coalesce() for b in pbyp]
        step = lambda w1, w2, opt: ref.train(inputs_loc, w1, w2, adj_loc, pbyp, opt, data, rank, size, group,
                                             row_groups, col_groups)
    elif algo == "2d":
        row_groups, col_groups = ref.get_proc_groups(rank, size, group)
        q_ = ref.proc_row_size(size)
        rr, rc = rank // q_, rank % q_
        tgroups = [[dist.new_group([i * q_ + j, j * q_ + i]) if i * q_ + j < j * q_ + i else None
                    for j in range(q_)] for i in range(q_)]
        tgroup = tgroups[rr][rc] if rank < rc * q_ + rr else tgroups[rc][rr]
        inputs_loc, adj_loc, _ = ref.twod_partition(rank, size, inputs, adj, data, f, classes, cpu)
        adj_loc = adj_loc.coalesce()
        step = lambda w1, w2, opt: ref.train(inputs_loc, w1, w2, n, adj_loc, None, opt, data, rank, size, 1, group,
                                             row_groups, col_groups, tgroup)
    else:
        row_groups, col_groups, c_groups = ref.get_proc_groups(rank, size, group)
        q_ = ref.proc_row_size(size)
        rr, rc, rk = (rank // q_) // q_, (rank // q_) % q_, rank % q_
        tg = {}
        for i in range(q_):
            for j in range(q_):
                for k in range(q_):
                    a, b = i * q_ * q_ + j * q_ + k, j * q_ * q_ + i * q_ + k
                    if a < b:
                        tg[(a, b)] = dist.new_group([a, b])
        rank_t = rc * q_ * q_ + rr * q_ + rk
        tgroup = tg.get((min(rank, rank_t), max(rank, rank_t)))
        inputs_loc, adj_loc, _ = ref.twod_partition(rank, size, inputs, adj, data, f, classes, cpu)
        adj_loc = adj_loc.coalesce()
        inputs_loc, adj_loc = ref.threed_partition_loc(rank, size, inputs_loc, adj_loc.indices(), adj_loc.size(0),
                                                       adj_loc.size(1), data, f, classes, cpu)
        adj_loc = adj_loc.coalesce()
        step = lambda w1, w2, opt: ref.train(inputs_loc, w1, w2, n, adj_loc, None, opt, data, rank, size, 1, group,
                                             row_groups, col_groups, tgroup, c_groups)

    torch.manual_seed(0)
    w1 = torch.nn.Parameter(torch.rand(f, mid, requires_grad=True))
    w2 = torch.nn.Parameter(torch.rand(mid, classes, requires_grad=True))
    opt = torch.optim.Adam([w1, w2], lr=0.01)
    out = {}
    for ep in range(epochs):
        o = step(w1, w2, opt)
        out[f"ep{ep}_out"] = o.detach().numpy().copy()
        out[f"ep{ep}_gw1"] = w1.grad.detach().numpy().copy()
        out[f"ep{ep}_gw2"] = w2.grad.detach().numpy().copy()
        out[f"ep{ep}_w1"] = w1.detach().numpy().copy()
        out[f"ep{ep}_w2"] = w2.detach().numpy().copy()
    q.put((rank, out))
    dist.barrier()
    dist.destroy_process_group()


def training_goldens(refdir, out):
    runs = [
        ("1d", 1, dict(n=50, f=6, mid=4, classes=5)),
        ("1d", 3, dict(n=50, f=6, mid=4, classes=5)),
        ("1d", 1, dict(n=50, f=6, mid=4, classes=5, activations=False, normalization=False, tag="plain")),
        ("15d", 4, dict(n=50, f=6, mid=4, classes=5, replication=2)),
        ("15d", 8, dict(n=50, f=6, mid=4, classes=5, replication=2)),
        ("2d", 4, dict(n=51, f=7, mid=4, classes=5)),
        ("3d", 8, dict(n=51, f=8, mid=4, classes=6)),
    ]
    for algo, P, cfg in runs:
        cfg = dict(dict(epochs=3, normalization=True, activations=True, replication=1, tag=""), **cfg)
        edge_index, x, y, mask = make_case(cfg["n"], 6, cfg["f"], cfg["classes"], seed=21)
        case = tuple(a.numpy() for a in (edge_index, x, y, mask))
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=_train_worker, args=(r, P, port, refdir, algo, cfg, case, q)) for r in range(P)]
        for p in procs:
            p.start()
        res = dict(edge_index=case[0], x=case[1], y=case[2], mask=case[3],
                   cfg=np.array([cfg["n"], cfg["f"], cfg["mid"], cfg["classes"], cfg["epochs"], P, cfg["replication"],
                                 int(cfg["normalization"]), int(cfg["activations"])], dtype=np.int64))
        for _ in range(P):
            while True:
                try:
                    rank, o = q.get(timeout=5)
                    break
                except Exception:
                    if any(p.exitcode not in (None, 0) for p in procs):
                        for p in procs:
                            p.kill()
                        raise RuntimeError(f"a rank of {algo} P={P} died")
            for k, v in o.items():
                res[f"r{rank}_{k}"] = v
        for p in procs:
            p.join()
            assert p.exitcode == 0, (algo, P, p.exitcode)
        name = f"train_{algo}_P{P}{('_' + cfg['tag']) if cfg['tag'] else ''}.npz"
        np.savez_compressed(os.path.join(out, name), **res)
        print("wrote", name)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=os.path.dirname(os.path.abspath(__file__)))
    ap.add_argument("--only", default="all", choices=["all", "partition", "training"])
    a = ap.parse_args()
    if a.only in ("all", "partition"):
        partition_goldens(a.reference, a.out)
    if a.only in ("all", "training"):
        training_goldens(a.reference, a.out)
