"""Per-category wall-clock accumulators with the reference's category names and report format
(gcn_distr.py:42-94, 613-637; gcn_distr_15d.py:67-99, 662-672; gcn_distr_2d.py:109-131, 1324-1344).

With `--timing=True` every bracketed region is fenced by a device synchronisation, as the 1.5D/2D/3D
reference scripts do, which serialises communication and compute; with timing off the brackets cost
nothing and the schedules overlap.
"""
import time
from contextlib import contextmanager

CATEGORIES_1D = ("comm_time", "comp_time", "scomp_time", "dcomp_time", "bcast_comm_time", "barrier_time",
                 "barrier_subset_time", "op1_comm_time", "op2_comm_time")
CATEGORIES_15D = ("comm_time", "comp_time", "scomp_time", "dcomp_time", "bcast_comm_time", "bcast_words",
                  "reduce_comm_time", "op_comm_time", "barrier_time")
CATEGORIES_2D = ("comm_time", "comp_time", "summa_sparse_comp", "summa_sparse_bcast1", "summa_sparse_bcast1_words",
                 "summa_sparse_bcast2", "summa_sparse_bcast2_fwd", "summa_sparse_bcast2_bwd",
                 "summa_sparse_bcast2_words", "summa_comp", "summa_bcast1", "summa_bcast2", "summa_loc_bcast",
                 "transpose_time", "grad_weight_time", "loss_calc_time", "summa_sparse_time", "summa_time",
                 "summa_loc_time")
CATEGORIES_3D = ("comm_time", "comp_time", "summa_sparse_comp", "summa_sparse_bcast1", "summa_sparse_bcast1_words",
                 "summa_sparse_bcast2", "summa_sparse_reduce", "summa_sparse_bcast2_words", "summa_comp",
                 "summa_bcast1", "summa_bcast2", "summa_reduce", "summa_loc_bcast", "transpose_time",
                 "loss_calc_time")


class Timers:
    def __init__(self, categories, enabled=False, sync=None):
        self.categories = tuple(categories)
        self.enabled = bool(enabled)
        self.sync = sync if sync is not None else (lambda: None)
        self.runs = {}
        self.run = 0
        self.start_run(0)

    def start_run(self, run):
        self.run = run
        self.runs[run] = {c: 0.0 for c in self.categories}
        self.runs[run]["total_time"] = 0.0

    def add(self, category, value):
        if category in self.runs[self.run]:
            self.runs[self.run][category] += value

    def count(self, category, value):
        """Counters (e.g. words broadcast) accumulate whether or not timing is on."""
        self.add(category, value)

    @contextmanager
    def region(self, *categories):
        if not self.enabled:
            yield
            return
        self.sync()
        t0 = time.time()
        try:
            yield
        finally:
            self.sync()
            dt = time.time() - t0
            for c in categories:
                self.add(c, dt)

    @contextmanager
    def paused(self):
        was, self.enabled = self.enabled, False
        try:
            yield
        finally:
            self.enabled = was

    def report(self, rank, run, total_label="total_time", printer=print):
        rec = self.runs[run]
        printer(f"rank: {rank} {total_label}: {rec['total_time']}")
        for c in self.categories:
            printer(f"rank: {rank} {c}: {rec[c]}")
