"""The expert-parallel protocol with real collectives on CPU (gloo, world size 2): all-gather of the
home tokens, every rank fills the pair rows of the experts it owns (the oracle stands in for the
device), sum-reduction of the disjoint buffers, ordered combine of the home tokens.  The gathered
result must equal the single-process oracle layer bit for bit."""
import os
import socket

import numpy as np
import pytest

import oracle as po
from peregrine_b200.ep import ep_reference_step, home_range, owned_range
from peregrine_b200.synth import synth_layer, synth_tokens
from tests.refmodel import o_expert, oracle_layer_forward


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, m, out_dir):
    import torch
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    layer = synth_layer(11, hidden=128, inter=64, n_experts=8, k=3, gs=32)
    x_full = synth_tokens(3, m, 128)
    home = home_range(m, rank, world)
    x_local = torch.from_numpy(x_full[home.start:home.stop].copy())
    # 1. dispatch: all-gather of the home tokens
    gathered = [torch.empty_like(x_local) for _ in range(world)]
    dist.all_gather(gathered, x_local)
    x_all = torch.cat(gathered, 0).numpy()
    # 2. every rank routes the whole batch identically
    idx, w, keff = po.route(x_all, layer.router_w, layer.router_bias, m, 128, 8, 3, layer.norm_topk,
                            layer.routed_scale)
    union = po.batch_union(idx, keff, m, 3, 8)

    def pair_rows_of(e, toks):
        ex = layer.shared if e == layer.n_experts else layer.experts[e]
        g, u, d = o_expert(ex)
        return po.swiglu(g, u, d, x_all[toks], len(toks))

    rows = torch.from_numpy(ep_reference_step(layer, x_all, rank, world, pair_rows_of, union, idx, keff))
    # 3. combine exchange: sum of disjoint buffers
    dist.all_reduce(rows, op=dist.ReduceOp.SUM)
    rows = rows.numpy()
    # ordered combine of the home tokens (batch-union order, shared expert last)
    pair_of = {}
    p = 0
    for e in union:
        for s in range(m):
            if e in idx[s, : keff[s]]:
                pair_of[(s, int(e))] = p
                p += 1
    shared0 = p
    out = np.zeros((len(home), 128), np.float32)
    for i, s in enumerate(home):
        acc = np.zeros(128, np.float32)
        for e in union:
            if (s, int(e)) in pair_of:
                kk = list(idx[s, : keff[s]]).index(e)
                acc = acc + (w[s, kk] * rows[pair_of[(s, int(e))]]).astype(np.float32)
        out[i] = acc + rows[shared0 + s]
    np.save(os.path.join(out_dir, f"out{rank}.npy"), out)
    assert list(owned_range(8, rank, world)) == list(range(rank * 4, rank * 4 + 4))
    dist.destroy_process_group()


@pytest.mark.parametrize("m", [2, 6])
def test_ep_protocol_two_ranks_gloo(tmp_path, m):
    import torch.multiprocessing as mp

    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, m, str(tmp_path)), nprocs=world, join=True)
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)], 0)
    layer = synth_layer(11, hidden=128, inter=64, n_experts=8, k=3, gs=32)
    want = oracle_layer_forward(layer, synth_tokens(3, m, 128))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
