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


def oracle_stack_decode(st, ids0, steps, threads=4):
    """CPU restatement of peregrine_b200.stack.DeviceStack.decode with the oracle's functions:
    embed -> [rmsnorm -> (dense swiglu | moe_forward) -> residual] x L -> rmsnorm -> lm_head -> argmax
    (crates/peregrine-model/src/model.rs:1971-2006, 4260-4261; sample.rs:21-43)."""
    from peregrine_b200.synth import SynthLayer

    ids = np.array(ids0, np.int32)
    out = []
    lm = o_weight(st.lm_head)
    for _ in range(steps):
        x = st.embed[ids].astype(np.float32).copy()
        b = x.shape[0]
        for li, layer in enumerate(st.layers):
            nrm = np.stack([po.rmsnorm(x[s], st.norms[li], st.eps) for s in range(b)])
            if isinstance(layer, SynthLayer):
                ffn = oracle_layer_forward(layer, nrm, threads=threads)
            else:
                g, u, d = o_expert(layer)
                ffn = po.swiglu(g, u, d, nrm, b)
            x = (x + ffn).astype(np.float32)
        nrm = np.stack([po.rmsnorm(x[s], st.final_norm, st.eps) for s in range(b)])
        logits = lm.apply(nrm, b)
        ids = np.array([po.argmax(logits[s]) for s in range(b)], np.int32)
        out.append(ids.copy())
    return np.stack(out)
