"""Expert parallelism over the GPUs of one node: one process per GPU, the routed
experts block-partitioned over the ranks, ``torch.distributed`` (NCCL over
NVLink) for the two exchanges of a layer.

Protocol per MoE layer and decode step (all ranks hold the router and the shared
expert; rank r holds routed experts ``[r*E/G, (r+1)*E/G)``):

1. dispatch  — all-gather of the home tokens: every rank gets ``x_all[M, D]``.
   With top-8 over 8 ranks a token is needed on ~2/3 of the ranks, so the
   all-gather moves about 1.5x what a token-by-token all-to-all would.
2. every rank routes the whole batch (same kernel, same inputs: identical ids,
   weights and batch-union order everywhere) and runs its own experts; pair rows it
   does not own stay zero.
3. combine   — sum-reduction of the pair-row buffers over the ranks.  Each row has
   exactly one non-zero contributor, so the sum is exact whatever order the
   collective uses; the order-sensitive part, the routing-weighted sum in
   batch-union order, happens afterwards on the home rank
   (crates/peregrine-model/src/concurrent.rs:1866-1929; docs/scale-out-design.md:62-67
   asks for exactly this: never sum partials in arrival order).
"""
from __future__ import annotations

import numpy as np

from . import cuda
from .resident import upload_expert
from .synth import SynthLayer


def owned_range(n_experts: int, rank: int, world: int) -> range:
    per = -(-n_experts // world)
    return range(min(rank * per, n_experts), min((rank + 1) * per, n_experts))


def home_range(m: int, rank: int, world: int) -> range:
    per = -(-m // world)
    return range(min(rank * per, m), min((rank + 1) * per, m))


def upload_ep_layer(device: int, layer: SynthLayer, rank: int, world: int) -> cuda.MoeLayer:
    """Uploads router, shared expert and only the routed experts this rank owns."""
    ml = cuda.MoeLayer(device, layer.hidden, layer.inter, layer.n_experts, layer.k, layer.norm_topk,
                       layer.routed_scale, layer.router_w, layer.router_bias)
    ml.set_ep(rank, world)
    for e in owned_range(layer.n_experts, rank, world):
        ml.set_expert(e, upload_expert(device, layer.experts[e], layer.hidden, layer.inter))
    if layer.shared is not None:
        ml.set_shared(upload_expert(device, layer.shared, layer.hidden, layer.inter))
    return ml


class EpLayerRunner:
    """Runs one expert-parallel layer step for this rank on torch tensors.

    ``forward(x_local)`` takes the rank's home tokens ``[M/G, D]`` (fp32, on this
    rank's GPU) and returns their outputs.  ``group=None`` with world 1 skips the
    collectives (used by the single-GPU emulation in the tests)."""

    def __init__(self, ml: cuda.MoeLayer, device: int, rank: int, world: int, m_total: int, group=None):
        import torch

        if m_total % world:
            raise ValueError("the decode batch must be a multiple of the number of ranks")
        self.ml, self.device, self.rank, self.world, self.m_total, self.group = ml, device, rank, world, m_total, group
        self.m_local = m_total // world
        self.stream = torch.cuda.ExternalStream(cuda.lib().coli_cuda_stream(device), device=device)
        with torch.cuda.stream(self.stream):
            self.x_all = torch.empty((m_total, ml.hidden), dtype=torch.float32, device=device)
            self.y_pairs = torch.empty((m_total * (ml.k + 1), ml.hidden), dtype=torch.float32, device=device)
            self.out = torch.empty((self.m_local, ml.hidden), dtype=torch.float32, device=device)
        self.stream.synchronize()

    def forward(self, x_local):
        import torch
        import torch.distributed as dist

        with torch.cuda.stream(self.stream):
            if self.world > 1:
                dist.all_gather_into_tensor(self.x_all, x_local.contiguous(), group=self.group)
            else:
                self.x_all.copy_(x_local)
            self.ml.ep_partial_dev(self.y_pairs.data_ptr(), self.x_all.data_ptr(), self.m_total)
            if self.world > 1:
                dist.all_reduce(self.y_pairs, op=dist.ReduceOp.SUM, group=self.group)
            self.ml.ep_combine_dev(self.out.data_ptr(), self.y_pairs.data_ptr(), self.m_total,
                                   self.rank * self.m_local, self.m_local)
        return self.out


def ep_reference_step(layer, x_all: np.ndarray, rank: int, world: int, pair_rows_of, union, idx, keff):
    """Host restatement of what one rank contributes (used by the CPU protocol test):
    returns the pair-row buffer with only this rank's rows filled.  ``pair_rows_of(e, tokens)``
    computes the un-weighted expert output rows for expert e (``e == n_experts``: shared)."""
    m, k = x_all.shape[0], layer.k
    rows = np.zeros((m * (k + 1), layer.hidden), np.float32)
    own = owned_range(layer.n_experts, rank, world)
    home = home_range(m, rank, world)
    p = 0
    for e in union:
        toks = [s for s in range(m) if e in idx[s, : keff[s]]]
        if e in own and toks:
            rows[p:p + len(toks)] = pair_rows_of(int(e), toks)
        p += len(toks)
    if layer.shared is not None and len(home):
        toks = list(home)
        rows[p + home.start:p + home.start + len(toks)] = pair_rows_of(layer.n_experts, toks)
    return rows
