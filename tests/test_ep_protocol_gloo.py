"""The expert-parallel protocol with real processes on CPU (gloo, world size 2), the oracle standing
in for the device kernels: every rank routes ITS home tokens only, the picks are all-gathered, every
rank derives the batch plan, each (token, expert) pair's int8 row + scale goes to the expert's owner
(token by token: an all-to-all), the owner returns the un-weighted output row to the token's home
rank, and the home rank combines in batch-union order.  The gathered result must equal the
single-process oracle layer bit for bit — in particular re-computing an expert from the int8 row
that crossed the wire gives the same bits as computing it from the fp32 token."""
import os
import socket

import numpy as np
import pytest

import oracle as po
from peregrine_b200.ep import batch_plan, home_range, owned_range, owner_of
from peregrine_b200.synth import synth_layer, synth_tokens
from tests.refmodel import o_expert, oracle_layer_forward

HID, INTER, NE, K = 128, 64, 8, 3


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _expert_rows_from_int8(ex, xq, sx, n):
    """down(silu(gate x) * up x) for rows that arrive already quantised (what the owner receives)."""
    g, u, d = ex.gate, ex.up, ex.down
    mm = (lambda w, q, s, i, o: po.matmul_i4g_idot(q, s, w.q, w.scale, n, i, o, w.gs)) if g.gs else \
        (lambda w, q, s, i, o: po.matmul_i4_idot(q, s, w.q, w.scale, n, i, o))
    gate = mm(g, xq, sx, HID, INTER)
    up = mm(u, xq, sx, HID, INTER)
    h = po.silu_mul(gate, up)
    hq = np.empty((n, INTER), np.int8)
    sh = np.empty(n, np.float32)
    for r in range(n):
        hq[r], sh[r] = po.qrow_i8(h[r])
    return mm(d, hq, sh, INTER, HID)


def _worker(rank, world, port, m, out_dir):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    layer = synth_layer(11, hidden=HID, inter=INTER, n_experts=NE, k=K, gs=32)
    x_full = synth_tokens(3, m, HID)
    home = home_range(m, rank, world)
    x_local = x_full[home.start:home.stop].copy()
    ml = len(home)
    # 1. route the home tokens only; all-gather the picks
    idx_l, w_l, keff_l = po.route(x_local, layer.router_w, layer.router_bias, ml, HID, NE, K, layer.norm_topk,
                                  layer.routed_scale)
    picks = [None] * world
    dist.all_gather_object(picks, (idx_l, keff_l))
    idx = np.concatenate([p[0] for p in picks], 0)
    keff = np.concatenate([p[1] for p in picks], 0)
    # 2. batch plan (identical on every rank) and dispatch of int8 rows to the owners
    union, pair_of, shared0 = batch_plan(idx, keff, NE)
    outbox = {r: [] for r in range(world)}
    for i, s in enumerate(home):
        xq, sx = po.qrow_i8(x_local[i])
        for kk in range(int(keff[s])):
            e = int(idx[s, kk])
            outbox[owner_of(e, NE, world)].append((pair_of[(s, e)], e, s, xq, sx))
    boxes = [None] * world
    dist.all_gather_object(boxes, outbox)          # stands in for the all-to-all: rank r reads box[.][r]
    inbox = [item for b in boxes for item in b[rank]]
    assert all(e in owned_range(NE, rank, world) for _, e, _, _, _ in inbox)
    # 3. the owner computes its experts on the received rows and returns un-weighted rows to the home ranks
    back = {r: [] for r in range(world)}
    for e in sorted({it[1] for it in inbox}):
        rows = sorted([it for it in inbox if it[1] == e], key=lambda it: it[2])  # tokens ascending
        xq = np.stack([it[3] for it in rows])
        sx = np.array([it[4] for it in rows], np.float32)
        y = _expert_rows_from_int8(layer.experts[e], xq, sx, len(rows))
        for it, yr in zip(rows, y):
            back[it[2] // (m // world)].append((it[0], yr))
    backs = [None] * world
    dist.all_gather_object(backs, back)
    y_rows = {p: yr for b in backs for p, yr in b[rank]}
    # 4. ordered combine of the home tokens: batch-union order, shared expert (local) last
    g, u, d = o_expert(layer.shared)
    shared = po.swiglu(g, u, d, x_local, ml)
    out = np.zeros((ml, HID), np.float32)
    for i, s in enumerate(home):
        acc = np.zeros(HID, np.float32)
        for e in union:
            if (s, e) in pair_of:
                kk = [int(v) for v in idx[s, : int(keff[s])]].index(e)
                acc = acc + (w_l[i, kk] * y_rows[pair_of[(s, e)]]).astype(np.float32)
        out[i] = acc + shared[i]
    np.save(os.path.join(out_dir, f"out{rank}.npy"), out)
    dist.destroy_process_group()


@pytest.mark.parametrize("m", [2, 6])
def test_ep_protocol_two_ranks_gloo(tmp_path, m):
    import torch.multiprocessing as mp

    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, m, str(tmp_path)), nprocs=world, join=True)
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)], 0)
    layer = synth_layer(11, hidden=HID, inter=INTER, n_experts=NE, k=K, gs=32)
    want = oracle_layer_forward(layer, synth_tokens(3, m, HID))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_batch_plan_matches_oracle_union():
    layer = synth_layer(5, hidden=HID, inter=INTER, n_experts=NE, k=K, gs=32)
    x = synth_tokens(9, 7, HID)
    idx, w, keff = po.route(x, layer.router_w, layer.router_bias, 7, HID, NE, K, True, 2.5)
    union, pair_of, shared0 = batch_plan(idx, keff, NE)
    assert list(union) == list(po.batch_union(idx, keff, 7, K, NE))
    assert sorted(pair_of.values()) == list(range(shared0)) and shared0 == int(keff.sum())
