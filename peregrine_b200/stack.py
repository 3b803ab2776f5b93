"""Synthetic FFN-only decode stack (the shape family of the benchmark's full-stack config) on one device.

    embed -> [ rmsnorm -> (dense SwiGLU | MoE layer) -> residual add ] x L -> rmsnorm -> lm_head -> argmax

This is the loop shape of the reference's batched decode step with attention left out
(crates/peregrine-model/src/model.rs:1971-2006 per layer, :4260-4261 final norm + lm_head,
sample.rs:21-43 greedy pick).  Everything stays on the device between steps: token ids feed
the next step's embedding gather without a host round trip.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field

import numpy as np

from . import cuda
from .resident import upload_expert, upload_layer
from .synth import SynthExpert, SynthLayer, SynthMatrix, synth_expert, synth_layer, synth_matrix


@dataclass
class SynthStack:
    hidden: int
    vocab: int
    eps: float
    embed: np.ndarray                  # fp32 [vocab, hidden]
    norms: list                        # per layer fp32 [hidden]
    final_norm: np.ndarray
    lm_head: SynthMatrix               # int4 [vocab, hidden]
    layers: list = field(default_factory=list)   # SynthExpert (dense) or SynthLayer (MoE)


def synth_stack(seed: int, hidden: int, inter: int, dense_inter: int, n_experts: int, k: int, n_layers: int,
                first_dense: int, vocab: int, gs: int = 32, distinct_experts: int | None = None,
                scale_std: float = 0.02) -> SynthStack:
    """``scale_std``: standard deviation of the weight scales.  At hidden sizes in the thousands the
    default 0.02 makes every FFN output dwarf the residual stream and greedy decoding collapses onto
    one token whatever the input; wide stacks pass a smaller value so that the ids keep depending on
    the tokens (the arithmetic under test is the same)."""
    rng = np.random.default_rng(seed)
    embed = rng.standard_normal((vocab, hidden)).astype(np.float32)
    norms = [(1.0 + 0.1 * rng.standard_normal(hidden)).astype(np.float32) for _ in range(n_layers)]
    final_norm = (1.0 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)
    lm_head = synth_matrix(rng, vocab, hidden, gs)
    layers = []
    for li in range(n_layers):
        if li < first_dense:
            layers.append(synth_expert(rng, hidden, dense_inter, gs, scale_std))
        else:
            layers.append(synth_layer(seed * 1000 + li, hidden, inter, n_experts, k, gs, shared=True,
                                      distinct_experts=distinct_experts, scale_std=scale_std))
    return SynthStack(hidden, vocab, 1e-5, embed, norms, final_norm, lm_head, layers)


class _DevBuf:
    def __init__(self, device: int, host: np.ndarray | None = None, nbytes: int | None = None):
        self.device = device
        self.nbytes = host.nbytes if host is not None else nbytes
        self.ptr = cuda.lib().coli_cuda_pipe_alloc(device, self.nbytes)
        if not self.ptr:
            raise cuda.CudaError("device allocation failed")
        if host is not None:
            host = np.ascontiguousarray(host)
            if cuda.lib().coli_cuda_pipe_upload(device, self.ptr, host.ctypes.data, host.nbytes) != 1:
                raise cuda.CudaError("device upload failed")

    def download(self, shape, dtype):
        out = np.empty(shape, dtype)
        if cuda.lib().coli_cuda_pipe_download(self.device, self.ptr, out.ctypes.data, out.nbytes) != 1:
            raise cuda.CudaError("device download failed")
        return out

    def free(self):
        if self.ptr:
            cuda.lib().coli_cuda_pipe_free(self.device, self.ptr)
            self.ptr = None


class DeviceStack:
    """The stack resident on one device; ``decode`` runs greedy steps without host round trips.

    Expert parallel (``ep`` = an ``EpWorkspace`` connected to the other ranks): this rank holds the
    routed experts it owns of every MoE layer and decodes ``batch`` = its home tokens; everything
    outside the MoE layers is per token, so only those layers exchange."""

    def __init__(self, device: int, st: SynthStack, batch: int, max_steps: int, ep=None, repeats: str = "upload"):
        L = cuda.lib()
        self.device, self.st, self.batch, self.max_steps, self.ep = device, st, batch, max_steps, ep
        self.embed = _DevBuf(device, st.embed)
        self.norms = [_DevBuf(device, w) for w in st.norms]
        self.final_norm = _DevBuf(device, st.final_norm)
        self.lm_head = cuda.Tensor.upload_grouped(device, st.lm_head.q, st.lm_head.scale, st.hidden, st.vocab,
                                                  st.lm_head.gs)
        self.layers = []
        for layer in st.layers:
            if isinstance(layer, SynthLayer):
                if ep is not None:
                    from .ep import owned_range

                    self.layers.append(upload_layer(device, layer, owned_range(layer.n_experts, ep.rank, ep.world),
                                                    ep.rank, ep.world, repeats))
                else:
                    self.layers.append(upload_layer(device, layer, repeats=repeats))
            else:
                self.layers.append(upload_expert(device, layer, st.hidden, layer.gate.o_n))
        d, b = st.hidden, batch
        widest = max([l.gate.o_n for l in st.layers if isinstance(l, SynthExpert)] + [1])
        self.x = _DevBuf(device, nbytes=b * d * 4)
        self.nrm = _DevBuf(device, nbytes=b * d * 4)
        self.ffn = _DevBuf(device, nbytes=b * d * 4)
        self.g = _DevBuf(device, nbytes=b * widest * 4)
        self.u = _DevBuf(device, nbytes=b * widest * 4)
        self.logits = _DevBuf(device, nbytes=b * st.vocab * 4)
        self.ids = _DevBuf(device, nbytes=(max_steps + 1) * b * 4)
        self.graphs = None  # step graphs: None = not tried yet, [] = not available
        self.ping = self.pong = None
        self._L = L

    def _ok(self, rc, what):
        if rc != 1:
            raise cuda.CudaError(f"stack: {what} failed")

    def step(self, t: int):
        """ids[t] -> ids[t+1], all on the device's stream, one call per operation."""
        b = self.batch
        self._step_ops(self.ids.ptr + t * b * 4, self.ids.ptr + (t + 1) * b * 4)

    def _step_ops(self, ids_in_ptr: int, ids_out_ptr: int):
        L, dev, st, b, d = self._L, self.device, self.st, self.batch, self.st.hidden
        vp = C.c_void_p
        ids_in = vp(ids_in_ptr)
        ids_out = vp(ids_out_ptr)
        self._ok(L.coli_cuda_pipe_embed(dev, vp(self.x.ptr), vp(self.embed.ptr), ids_in, b, d, st.vocab), "embed")
        for li, layer in enumerate(self.layers):
            self._ok(L.coli_cuda_pipe_rmsnorm(dev, vp(self.nrm.ptr), vp(self.x.ptr), vp(self.norms[li].ptr), b, d,
                                              C.c_float(st.eps)), "rmsnorm")
            if isinstance(layer, cuda.MoeLayer):
                if self.ep is not None:
                    self._ok(L.coli_cuda_moe_layer_ep_forward_dev(layer.handle, self.ep.handle, vp(self.ffn.ptr),
                                                                  vp(self.nrm.ptr)), "expert-parallel layer")
                else:
                    layer.forward_dev(self.ffn.ptr, self.nrm.ptr, b)
            else:
                inter = layer.gate.o_n
                self._ok(L.coli_cuda_pipe_gemm(layer.gate.handle, vp(self.g.ptr), vp(self.nrm.ptr), b), "gate")
                self._ok(L.coli_cuda_pipe_gemm(layer.up.handle, vp(self.u.ptr), vp(self.nrm.ptr), b), "up")
                self._ok(L.coli_cuda_pipe_silu_mul(dev, vp(self.g.ptr), vp(self.u.ptr), b * inter), "silu_mul")
                self._ok(L.coli_cuda_pipe_gemm(layer.down.handle, vp(self.ffn.ptr), vp(self.g.ptr), b), "down")
            self._ok(L.coli_cuda_pipe_add(dev, vp(self.x.ptr), vp(self.ffn.ptr), b * d), "residual")
        self._ok(L.coli_cuda_pipe_rmsnorm(dev, vp(self.nrm.ptr), vp(self.x.ptr), vp(self.final_norm.ptr), b, d,
                                          C.c_float(st.eps)), "final rmsnorm")
        self._ok(L.coli_cuda_pipe_gemm(self.lm_head.handle, vp(self.logits.ptr), vp(self.nrm.ptr), b), "lm_head")
        self._ok(L.coli_cuda_pipe_argmax(dev, ids_out, vp(self.logits.ptr), b, st.vocab), "argmax")

    def start(self, ids0: np.ndarray):
        ids0 = np.ascontiguousarray(ids0, np.int32)
        self._ok(self._L.coli_cuda_pipe_upload(self.device, C.c_void_p(self.ids.ptr), ids0.ctypes.data, ids0.nbytes),
                 "ids upload")

    def result(self, steps: int) -> np.ndarray:
        return self.ids.download((steps + 1, self.batch), np.int32)[1:]

    def _record_step_graphs(self) -> bool:
        """Records one decode step twice as a replayable graph (ids: ping -> pong and pong -> ping), in
        the manner of the reference's COLI_CUDA_GRAPH pipe capture (cuda/backend_cuda.h:178-184): a step
        is ~90 launches whose arguments never change, and enqueueing them one by one from the host takes
        longer than the device needs to run them.  Needs one step already run (buffers sized, expert
        tables uploaded).  Expert-parallel stacks keep the call-by-call path: their exchange numbers
        its steps on the host."""
        if self.ep is not None or os.environ.get("PEREGRINE_B200_STACK_GRAPH") == "0":
            return False
        L, dev, b = self._L, self.device, self.batch
        self.ping = _DevBuf(dev, nbytes=b * 4)
        self.pong = _DevBuf(dev, nbytes=b * 4)
        graphs = []
        for src, dst in ((self.ping, self.pong), (self.pong, self.ping)):
            if L.coli_cuda_graph_begin(dev) != 1:
                return False
            try:
                self._step_ops(src.ptr, dst.ptr)
                ok = True
            except cuda.CudaError:
                ok = False
            g = C.c_void_p()
            if L.coli_cuda_graph_end(dev, C.byref(g)) != 1 or not ok:
                for h in graphs:
                    L.coli_cuda_graph_free(h)
                return False
            graphs.append(g)
        self.graphs = graphs
        return True

    def run(self, steps: int):
        """Enqueues `steps` greedy steps from ids[0] (see ``start``): ids[t + 1] = step(ids[t])."""
        if steps > self.max_steps:
            raise ValueError("more steps than the id buffer holds")
        if steps < 1:
            return
        L, dev, b = self._L, self.device, self.batch
        vp = C.c_void_p
        if self.graphs is None:
            self.step(0)  # call by call: sizes every buffer, uploads the expert tables
            self.graphs = [] if not self._record_step_graphs() else self.graphs
            first = 1
        else:
            first = 0
        if not self.graphs:
            for t in range(first, steps):
                self.step(t)
            return
        row = lambda t: vp(self.ids.ptr + t * b * 4)
        self._ok(L.coli_cuda_pipe_copy2d(dev, vp(self.ping.ptr), b, row(first), b, b, 1), "ids to the step graph")
        bufs = (self.ping, self.pong)
        for t in range(first, steps):
            k = (t - first) & 1
            self._ok(L.coli_cuda_graph_launch_async(self.graphs[k]), "step graph launch")
            self._ok(L.coli_cuda_pipe_copy2d(dev, row(t + 1), b, vp(bufs[1 - k].ptr), b, b, 1), "ids of the step")

    def decode(self, ids0: np.ndarray, steps: int) -> np.ndarray:
        """Greedy decode: returns int32 ids [steps, batch] (the tokens picked at each step)."""
        self.start(ids0)
        self.run(steps)
        return self.result(steps)

    def free(self):
        for g in self.graphs or []:
            self._L.coli_cuda_graph_free(g)
        self.graphs = []
        for buf in (self.ping, self.pong):
            if buf is not None:
                buf.free()
        for l in self.layers:
            l.free()
        self.lm_head.free()
        for b in [self.embed, self.final_norm, self.x, self.nrm, self.ffn, self.g, self.u, self.logits, self.ids] + \
                self.norms:
            b.free()
