"""Host-side mirror of the reference's GPU tier for the expert-FFN path: which experts are resident
on a device, and the job-list calls the scheduler's GPU lane makes against them
(crates/peregrine-model/src/gpu.rs:623-661, 1359-1383, 1896-2090).

The contract that matters to the caller: ``compute(layer, jobs, hidden)`` takes jobs
``[(expert, gathered rows [nr * hidden])]`` and returns one output per job **in job order**, whatever
grouping by residency format happened underneath; ``compute_reduced`` returns the gate-weighted
``[s_n, hidden]`` partial instead.  Residency differs from the reference in one deliberate way: a
checkpoint whose experts are grouped int4 (``gs`` = 32 ... 256, multiples of 32) stays packed on the
device through ``coli_cuda_tensor_upload_grouped`` instead of being expanded to fp32.
"""
from __future__ import annotations

import numpy as np

from . import cuda
from .container import QtFmt, QtWeight, SafeTensors, expert_names


def partition_by_format(fmt):
    """Job indices grouped by residency format (True = int4), int4 class first, order inside a class
    kept, no empty class (crates/peregrine-model/src/gpu.rs:623-634)."""
    int4 = [i for i, f in enumerate(fmt) if f]
    f32s = [i for i, f in enumerate(fmt) if not f]
    return [c for c in (int4, f32s) if c]


def scatter_by_index(total: int, classes, results):
    """Inverse of ``partition_by_format``: ``results[c][i]`` goes back to position ``classes[c][i]``.
    ``None`` when the shapes disagree, an index is out of range or repeated, or a position stays
    empty (crates/peregrine-model/src/gpu.rs:643-661)."""
    if len(classes) != len(results):
        return None
    slots = [None] * total
    filled = [False] * total
    for idxs, vals in zip(classes, results):
        if len(idxs) != len(vals):
            return None
        for i, v in zip(idxs, vals):
            if i < 0 or i >= total or filled[i]:
                return None
            slots[i] = v
            filled[i] = True
    if not all(filled):
        return None
    return slots


class GpuTier:
    """Experts of one device, keyed ``(layer, expert)``, with the format each was uploaded in."""

    def __init__(self, device: int, hidden: int, inter: int, int4: bool = True):
        self.device, self.hidden, self.inter, self.int4 = device, hidden, inter, int4
        self.experts = {}    # (layer, e) -> cuda.GpuExpert
        self.precision = {}  # (layer, e) -> True when int4-resident

    # ---- residency ----
    def upload_expert(self, st: SafeTensors, layer: int, e: int, int4: bool | None = None) -> bool:
        """Loads one expert from the checkpoint and makes it resident; returns whether it stayed int4.
        Per-row int4 uploads raw (as the reference, gpu.rs:1359-1383); grouped int4 with a group size
        the tile stream holds (32, 64, 128, 256) uploads raw too; anything else is dequantised to fp32."""
        want_int4 = self.int4 if int4 is None else int4
        h, it = self.hidden, self.inter
        gn, un, dn = expert_names(layer, e)
        gate = QtWeight.load(st, gn, it, h)
        up = QtWeight.load(st, un, it, h)
        down = QtWeight.load(st, dn, h, it)
        ws = (gate, up, down)

        def packable(w):
            return w.fmt == QtFmt.Int4 or (w.fmt == QtFmt.Int4Grouped and w.gs in (32, 64, 128, 256))

        # gate and up share one launch, so they must share a format; down may differ (a grouped
        # checkpoint whose down matrix is no wider than one group is detected as per-row: one scale
        # per row either way, and the two forms multiply the same numbers)
        if want_int4 and all(packable(w) for w in ws) and (gate.fmt, gate.gs) == (up.fmt, up.gs):
            def put(w):
                if w.fmt == QtFmt.Int4:
                    return cuda.Tensor.upload(self.device, w.q, w.scale, 2, w.i, w.o)
                return cuda.Tensor.upload_grouped(self.device, w.q, w.scale, w.i, w.o, w.gs)

            ex = cuda.GpuExpert(put(gate), put(up), put(down))
            kept = True
        else:
            ex = cuda.GpuExpert.upload(self.device, gate.dequant(), up.dequant(), down.dequant(), h, it)
            kept = False
        self.insert(layer, e, ex, kept)
        return kept

    def insert(self, layer: int, e: int, expert: cuda.GpuExpert, int4: bool) -> None:
        old = self.experts.pop((layer, e), None)
        if old is not None:
            old.free()
        self.experts[(layer, e)] = expert
        self.precision[(layer, e)] = bool(int4)

    def has(self, layer: int, e: int) -> bool:
        return (layer, e) in self.experts

    # ---- the GPU lane's calls ----
    def _validate(self, layer, jobs, hidden, what):
        for e, xg in jobs:
            if (layer, e) not in self.experts:
                raise cuda.CudaError(f"gpu expert ({layer},{e}) not resident")
            if hidden == 0 or np.asarray(xg).size % hidden:
                raise cuda.CudaError(f"gpu {what}: ragged gathered rows")

    def compute(self, layer: int, jobs, hidden: int):
        """One ``expert_group`` call per residency format; outputs back in job order
        (crates/peregrine-model/src/gpu.rs:1896-1950)."""
        if not jobs:
            return []
        self._validate(layer, jobs, hidden, "compute")
        fmt = [self.precision.get((layer, e), self.int4) for e, _ in jobs]
        classes = partition_by_format(fmt)
        per_class = []
        for idxs in classes:
            refs = [self.experts[(layer, jobs[i][0])] for i in idxs]
            rows = [np.asarray(jobs[i][1]).size // hidden for i in idxs]
            x = np.concatenate([np.asarray(jobs[i][1], np.float32).reshape(-1) for i in idxs])
            y = cuda.expert_group(refs, rows, x, hidden).reshape(-1)
            outs, off = [], 0
            for r in rows:
                n = r * hidden
                if off + n > y.size:
                    raise cuda.CudaError("gpu compute: expert_group returned a short buffer")
                outs.append(y[off:off + n].copy())
                off += n
            per_class.append(outs)
        out = scatter_by_index(len(jobs), classes, per_class)
        if out is None:
            raise cuda.CudaError("gpu compute: format partition is not a bijection")
        return out

    def compute_reduced(self, layer: int, jobs, hidden: int, dst, weights, s_n: int) -> np.ndarray:
        """``compute`` with the gate-weighted accumulation on the device: one ``[s_n, hidden]`` partial.
        ``dst[k]`` / ``weights[k]`` describe the rows in the flattened job order; class partials are
        added in class order (crates/peregrine-model/src/gpu.rs:2022-2090)."""
        acc = np.zeros((s_n, hidden), np.float32)
        if not jobs:
            return acc
        if hidden == 0 or s_n == 0:
            raise cuda.CudaError("gpu compute_reduced: empty hidden or batch")
        total = sum(np.asarray(xg).size // max(hidden, 1) for _, xg in jobs)
        dst = np.asarray(dst, np.int64)
        weights = np.asarray(weights, np.float32)
        if dst.size != total or weights.size != total:
            raise cuda.CudaError("gpu compute_reduced: dst/weights length != total rows")
        self._validate(layer, jobs, hidden, "compute_reduced")
        job_at = np.concatenate([[0], np.cumsum([np.asarray(xg).size // hidden for _, xg in jobs])]).astype(int)
        fmt = [self.precision.get((layer, e), self.int4) for e, _ in jobs]
        for idxs in partition_by_format(fmt):
            refs = [self.experts[(layer, jobs[i][0])] for i in idxs]
            rows = [np.asarray(jobs[i][1]).size // hidden for i in idxs]
            x = np.concatenate([np.asarray(jobs[i][1], np.float32).reshape(-1) for i in idxs])
            cdst = np.concatenate([dst[job_at[i]:job_at[i + 1]] for i in idxs])
            crw = np.concatenate([weights[job_at[i]:job_at[i + 1]] for i in idxs])
            layout = cuda.ReduceLayout.build(cdst, s_n)
            if layout is None:
                raise cuda.CudaError("gpu compute_reduced: row destination out of range")
            part = cuda.expert_group_reduce(refs, rows, x, hidden, layout, crw, s_n)
            if part.shape != acc.shape:
                raise cuda.CudaError("gpu compute_reduced: short partial")
            acc = (acc + part).astype(np.float32)
        return acc

    def free(self):
        for ex in self.experts.values():
            ex.free()
        self.experts.clear()
        self.precision.clear()
