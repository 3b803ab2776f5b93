"""Seeded synthetic MoE layers in the reference's container format.

Weights are int4 nibbles uniform on [-8, 7] stored +8, two per byte with the
even element in the low nibble (crates/peregrine-core/src/pack.rs:505-511);
scales are |N(0, 0.02)| per group of ``gs`` along K (or per row); router weights
are N(0, 0.02); activations N(0, 1).  No dataset stands behind these: they only
reproduce the shapes and value distributions of the benchmark configurations.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass
class SynthMatrix:
    q: np.ndarray       # uint8 [O * ceil(K/2)]
    scale: np.ndarray   # float32 [O] or [O * ng]
    i_n: int
    o_n: int
    gs: int             # 0 = per-row scale


@dataclass
class SynthExpert:
    gate: SynthMatrix
    up: SynthMatrix
    down: SynthMatrix


@dataclass
class SynthLayer:
    hidden: int
    inter: int
    n_experts: int
    k: int
    gs: int
    norm_topk: bool
    routed_scale: float
    router_w: np.ndarray
    router_bias: np.ndarray
    experts: list = field(default_factory=list)
    shared: SynthExpert | None = None


def synth_matrix(rng: np.random.Generator, o_n: int, i_n: int, gs: int, scale_std: float = 0.02) -> SynthMatrix:
    rb = (i_n + 1) // 2
    q = rng.integers(0, 256, size=o_n * rb, dtype=np.uint8)
    if i_n % 2:
        q.reshape(o_n, rb)[:, -1] &= 0x0F
    ng = -(-i_n // gs) if gs else 1
    scale = np.abs(rng.standard_normal(o_n * ng).astype(np.float32) * np.float32(scale_std))
    scale = np.maximum(scale, np.float32(scale_std * 5e-5)).astype(np.float32)
    return SynthMatrix(q, scale, i_n, o_n, gs)


def synth_expert(rng, hidden: int, inter: int, gs: int, scale_std: float = 0.02) -> SynthExpert:
    return SynthExpert(synth_matrix(rng, inter, hidden, gs, scale_std), synth_matrix(rng, inter, hidden, gs, scale_std),
                       synth_matrix(rng, hidden, inter, gs, scale_std))


def zipf_bias(rng, n_experts: int, s: float = 1.1, strength: float = 0.35) -> np.ndarray:
    """Selection bias that skews expert popularity towards Zipf(s) over a fixed
    random permutation of the experts.  The bias only affects which experts are
    chosen, never their weights (crates/peregrine-model/src/router.rs:86-110)."""
    ranks = rng.permutation(n_experts) + 1
    p = ranks.astype(np.float64) ** (-s)
    p /= p.sum()
    b = strength * (np.log(p) - np.log(p).max())
    return b.astype(np.float32)


def synth_layer(seed: int, hidden: int, inter: int, n_experts: int, k: int, gs: int = 32, shared: bool = True,
                norm_topk: bool = True, routed_scale: float = 2.5, zipf: bool = False,
                distinct_experts: int | None = None, scale_std: float = 0.02) -> SynthLayer:
    """``distinct_experts`` < n_experts reuses weight blobs cyclically (host RAM
    saver for CPU-side tests only; a device upload still makes n_experts copies)."""
    rng = np.random.default_rng(seed)
    router_w = (rng.standard_normal((n_experts, hidden)).astype(np.float32) * np.float32(0.02))
    bias = zipf_bias(rng, n_experts) if zipf else np.zeros(n_experts, np.float32)
    layer = SynthLayer(hidden, inter, n_experts, k, gs, norm_topk, routed_scale, router_w, bias)
    nd = n_experts if distinct_experts is None else min(distinct_experts, n_experts)
    blobs = [synth_expert(rng, hidden, inter, gs, scale_std) for _ in range(nd)]
    layer.experts = [blobs[e % nd] for e in range(n_experts)]
    if shared:
        layer.shared = synth_expert(rng, hidden, inter, gs, scale_std)
    return layer


def synth_tokens(seed: int, m: int, hidden: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((m, hidden)).astype(np.float32)


def expert_bytes(hidden: int, inter: int, gs: int) -> int:
    """Algorithmic bytes of one expert: 3*D*I nibbles + their scales."""
    nib = 3 * hidden * inter // 2
    if gs:
        return nib + 3 * hidden * inter // gs * 4
    return nib + (2 * inter + hidden) * 4
