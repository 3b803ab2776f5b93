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


def upload_layer(device: int, layer: SynthLayer, owned=None, rank: int = 0, world: int = 1,
                 repeats: str = "upload") -> cuda.MoeLayer:
    """Makes a synthetic layer resident.  ``owned``: the routed experts to attach (default all; an
    expert-parallel rank passes its own range together with rank / world).  A layer built with
    ``distinct_experts`` names the same host blob for several experts; ``repeats`` says what the
    device gets for the repeats: "upload" repacks and uploads every expert separately, "clone" uploads
    each blob once and copies it on the device (distinct memory, no host work), "share" attaches the
    same resident tensors again (parity runs that do not care about memory footprint)."""
    ml = cuda.MoeLayer(device, layer.hidden, layer.inter, layer.n_experts, layer.k, layer.norm_topk,
                       layer.routed_scale, layer.router_w, layer.router_bias)
    if world > 1:
        ml.set_ep(rank, world)
    first = {}
    for e in (range(layer.n_experts) if owned is None else owned):
        ex = layer.experts[e]
        if repeats == "upload" or id(ex) not in first:
            ge = upload_expert(device, ex, layer.hidden, layer.inter)
            first.setdefault(id(ex), ge)
        else:
            ge = first[id(ex)].clone() if repeats == "clone" else first[id(ex)]
        ml.set_expert(e, ge)
    if layer.shared is not None:
        # width moe_inter * n_shared (crates/peregrine-model/src/model.rs:1838): read from the matrices
        ml.set_shared(upload_expert(device, layer.shared, layer.hidden, layer.shared.gate.o_n))
    return ml
