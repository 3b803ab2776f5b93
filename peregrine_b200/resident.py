"""Uploads a synthetic layer (``synth.SynthLayer``) into a ``cuda.MoeLayer``."""
from __future__ import annotations

from . import cuda
from .synth import SynthExpert, SynthLayer


def upload_expert(device: int, ex: SynthExpert, hidden: int, inter: int) -> cuda.GpuExpert:
    g, u, d = ex.gate, ex.up, ex.down
    if g.gs:
        return cuda.GpuExpert.upload_int4_grouped(device, (g.q, g.scale), (u.q, u.scale), (d.q, d.scale), hidden,
                                                  inter, g.gs)
    return cuda.GpuExpert.upload_int4(device, (g.q, g.scale), (u.q, u.scale), (d.q, d.scale), hidden, inter)


def upload_layer(device: int, layer: SynthLayer) -> cuda.MoeLayer:
    ml = cuda.MoeLayer(device, layer.hidden, layer.inter, layer.n_experts, layer.k, layer.norm_topk,
                       layer.routed_scale, layer.router_w, layer.router_bias)
    for e, ex in enumerate(layer.experts):
        ml.set_expert(e, upload_expert(device, ex, layer.hidden, layer.inter))
    if layer.shared is not None:
        # width moe_inter * n_shared (crates/peregrine-model/src/model.rs:1838): read from the matrices
        ml.set_shared(upload_expert(device, layer.shared, layer.hidden, layer.shared.gate.o_n))
    return ml
