"""Oracle-side view of a synthetic layer (test helper)."""
import numpy as np

import oracle as po


def o_weight(m):
    return po.Weight(m.q, m.scale, 4 if m.gs else 2, m.gs, m.i_n, m.o_n)


def o_expert(ex):
    return (o_weight(ex.gate), o_weight(ex.up), o_weight(ex.down))


def oracle_layer_forward(layer, x, threads=1, want_routing=False):
    experts = [o_expert(e) for e in layer.experts]
    shared = o_expert(layer.shared) if layer.shared is not None else None
    x = np.ascontiguousarray(x, np.float32)
    return po.moe_forward(x, layer.router_w, layer.router_bias, experts, shared, x.shape[0], layer.hidden, layer.k,
                          layer.norm_topk, layer.routed_scale, threads=threads, want_routing=want_routing)


def rel_err(a, b):
    """max |a-b| / max(|b|, eps) per element, the tolerance form used by the parity gates."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b) / np.maximum(np.abs(b), 1e-6)))
