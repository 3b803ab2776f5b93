"""Expert parallelism over the GPUs of one node: one process per GPU, the routed experts
block-partitioned over the ranks, tokens data-parallel, and a token-by-token exchange (all-to-all)
done by the backend's own kernels through peer memory over NVLink.  ``torch.distributed`` is used
once, at set-up, to hand every rank the memory handles of the others.

Protocol per MoE layer and decode step (all ranks hold the router and the shared expert; rank r holds
routed experts ``[r*E/G, (r+1)*E/G)`` and the home tokens ``[r*M/G, (r+1)*M/G)``):

1. route     — every rank routes its home tokens only and stores their picks (expert ids, kept
   counts: 4 bytes per pick) into every rank's copy of the batch-wide pick table;
2. dispatch  — with all picks present every rank derives the same batch-union order and pair layout;
   each (home token, picked expert) pair's int8 row + scale + block sums (6.5 KB at hidden 6144, a
   quarter of the fp32 row; exact, quantisation is deterministic) goes to the expert's owner;
3. experts   — the owner runs gate/up + SwiGLU and down on the rows it received and stores each
   un-weighted, un-reduced output row into the token's home rank;
4. combine   — the home rank sums its tokens' rows with the gate weights in batch-union order, the
   shared expert (computed locally) last: partial results are never added in arrival order
   (crates/peregrine-model/src/concurrent.rs:1866-1929; docs/scale-out-design.md:62-67).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import cuda
from .resident import upload_expert
from .synth import SynthLayer


def owned_range(n_experts: int, rank: int, world: int) -> range:
    per = -(-n_experts // world)
    return range(min(rank * per, n_experts), min((rank + 1) * per, n_experts))


def owner_of(e: int, n_experts: int, world: int) -> int:
    return int(e) // (-(-n_experts // world))


def home_range(m: int, rank: int, world: int) -> range:
    per = -(-m // world)
    return range(min(rank * per, m), min((rank + 1) * per, m))


def batch_plan(idx: np.ndarray, keff: np.ndarray, n_experts: int):
    """Host mirror of the batch-wide plan every rank derives from the gathered picks: the batch-union
    order (first seen, tokens ascending then picks ascending, crates/peregrine-model/src/router.rs:420-430),
    pair rows expert by expert in that order with tokens ascending inside an expert
    (mlp.rs:83-95), the shared expert's rows last.  Returns ``(union, pair_of, shared0)`` with
    ``pair_of[(token, expert)]`` the pair row."""
    m = idx.shape[0]
    union, seen = [], set()
    for s in range(m):
        for kk in range(int(keff[s])):
            e = int(idx[s, kk])
            if e not in seen:
                seen.add(e)
                union.append(e)
    pair_of, p = {}, 0
    for e in union:
        for s in range(m):
            if e in [int(v) for v in idx[s, : int(keff[s])]]:
                pair_of[(s, e)] = p
                p += 1
    return union, pair_of, p


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


class EpWorkspace:
    """A rank's exchange block (peer-visible device memory) for batches of ``m`` tokens; one block
    serves every layer of the same width and top-k."""

    def __init__(self, device: int, rank: int, world: int, m: int, hidden: int, k: int):
        self.device, self.rank, self.world, self.m, self.hidden, self.k = device, rank, world, m, hidden, k
        self.handle = C.c_void_p()
        if cuda.lib().coli_cuda_ep_create(C.byref(self.handle), device, rank, world, m, hidden, k) != 1:
            raise cuda.CudaError("cuda ep_create failed")

    @property
    def base(self) -> int:
        return int(cuda.lib().coli_cuda_ep_local_base(self.handle))

    @property
    def nbytes(self) -> int:
        return int(cuda.lib().coli_cuda_ep_block_bytes(self.handle))

    def export(self) -> bytes:
        buf = (C.c_ubyte * 64)()
        if cuda.lib().coli_cuda_ep_export(self.handle, buf) != 1:
            raise cuda.CudaError("cuda ep_export failed")
        return bytes(buf)

    def attach(self, peer: int, handle: bytes) -> None:
        buf = (C.c_ubyte * 64).from_buffer_copy(handle)
        if cuda.lib().coli_cuda_ep_attach(self.handle, peer, buf) != 1:
            raise cuda.CudaError(f"cuda ep_attach({peer}) failed")

    def attach_ptr(self, peer: int, base: int) -> None:
        if cuda.lib().coli_cuda_ep_attach_ptr(self.handle, peer, C.c_void_p(base)) != 1:
            raise cuda.CudaError(f"cuda ep_attach_ptr({peer}) failed")

    def connect(self, group=None) -> None:
        """One process per GPU: every rank publishes its block's handle and maps the others'."""
        import torch.distributed as dist

        handles = [None] * self.world
        dist.all_gather_object(handles, self.export(), group=group)
        for r, h in enumerate(handles):
            if r != self.rank:
                self.attach(r, h)
        dist.barrier(group=group)

    def free(self) -> None:
        if self.handle:
            cuda.lib().coli_cuda_ep_free(self.handle)
            self.handle = C.c_void_p()


def connect_emulated(workspaces) -> None:
    """Ranks emulated inside one process on one device: every block is directly addressable."""
    for a in workspaces:
        for b in workspaces:
            if a.rank != b.rank:
                a.attach_ptr(b.rank, b.base)


class EpLayerRunner:
    """One rank's expert-parallel layer step on torch tensors: ``forward(x_local)`` takes the rank's
    home tokens ``[M/G, D]`` (fp32, on this rank's GPU) and returns their outputs.  The four phases
    are also exposed one by one (``route`` / ``dispatch`` / ``experts`` / ``finish``) so that several
    ranks emulated on one device can be stepped phase by phase: a phase only waits for data that an
    earlier phase of another rank has sent."""

    def __init__(self, ml: cuda.MoeLayer, ws: EpWorkspace):
        import torch

        self.ml, self.ws = ml, ws
        self.m_local = ws.m // ws.world
        self.stream = torch.cuda.ExternalStream(cuda.lib().coli_cuda_stream(ws.device), device=ws.device)
        with torch.cuda.stream(self.stream):
            self.out = torch.empty((self.m_local, ml.hidden), dtype=torch.float32, device=ws.device)
        self.stream.synchronize()

    def _ok(self, rc, what):
        if rc != 1:
            raise cuda.CudaError(f"expert parallel: {what} failed")

    def route(self, x_local):
        self._ok(cuda.lib().coli_cuda_moe_layer_ep_route_dev(self.ml.handle, self.ws.handle,
                                                             C.c_void_p(x_local.data_ptr())), "route")

    def dispatch(self):
        self._ok(cuda.lib().coli_cuda_moe_layer_ep_dispatch_dev(self.ml.handle, self.ws.handle), "dispatch")

    def experts(self):
        self._ok(cuda.lib().coli_cuda_moe_layer_ep_experts_dev(self.ml.handle, self.ws.handle), "experts")

    def finish(self):
        self._ok(cuda.lib().coli_cuda_moe_layer_ep_finish_dev(self.ml.handle, self.ws.handle,
                                                              C.c_void_p(self.out.data_ptr())), "combine")
        return self.out

    def forward(self, x_local):
        self._ok(cuda.lib().coli_cuda_moe_layer_ep_forward_dev(self.ml.handle, self.ws.handle,
                                                               C.c_void_p(self.out.data_ptr()),
                                                               C.c_void_p(x_local.data_ptr())), "layer step")
        return self.out
