"""Expert parallelism with the ranks emulated on one GPU: `world` layer objects, each holding only the
experts its rank owns, each with its own exchange block; the blocks are cross-attached by address and
the four phases are stepped rank by rank (a phase only waits for what an earlier phase of another
rank has already sent, so nothing ever spins on a kernel that has not run).  The gathered outputs of
the home tokens must equal the oracle's single-process layer bit for bit, for every world size, and
over several steps in a row (the exchange blocks alternate between two sets)."""
import numpy as np
import pytest

from peregrine_b200 import cuda
from peregrine_b200.ep import EpLayerRunner, EpWorkspace, connect_emulated, upload_ep_layer
from peregrine_b200.synth import synth_layer, synth_tokens
from tests.gpu_common import bits
from tests.refmodel import oracle_layer_forward

pytestmark = pytest.mark.gpu


def run_emulated(dev, layer, xs, world):
    """xs: list of batches [m, D]; returns the list of gathered outputs."""
    import torch

    m, d = xs[0].shape
    mls = [upload_ep_layer(dev, layer, r, world) for r in range(world)]
    wss = [EpWorkspace(dev, r, world, m, d, layer.k) for r in range(world)]
    connect_emulated(wss)
    runs = [EpLayerRunner(ml, ws) for ml, ws in zip(mls, wss)]
    stream, m_loc = runs[0].stream, m // world
    outs = []
    with torch.cuda.stream(stream):
        for x in xs:
            xd = torch.from_numpy(x).cuda(dev)
            for r, run in enumerate(runs):
                run.route(xd[r * m_loc:(r + 1) * m_loc])
            for run in runs:
                run.dispatch()
            for run in runs:
                run.experts()
            outs.append(torch.cat([run.finish().clone() for run in runs], 0))
    stream.synchronize()
    assert cuda.last_device_error(dev) == 0
    # the batch-wide routing every rank derived is the single-device routing
    routing = [ml.last_routing(m) for ml in mls]
    for ws in wss:
        ws.free()
    for ml in mls:
        ml.free()
    return [o.cpu().numpy() for o in outs], routing


@pytest.mark.parametrize("world,m", [(2, 2), (2, 8), (4, 8), (8, 8), (8, 32)])
def test_emulated_ranks_equal_the_single_device_layer(dev, world, m):
    layer = synth_layer(40 + world + m, hidden=256, inter=96, n_experts=16, k=4, gs=32)
    xs = [synth_tokens(world * 100 + m + i, m, 256) for i in range(3)]
    got, routing = run_emulated(dev, layer, xs, world)
    for x, g in zip(xs, got):
        assert np.array_equal(bits(g), bits(oracle_layer_forward(layer, x, threads=4)))
    want, idx, w, keff, uni = oracle_layer_forward(layer, xs[-1], threads=4, want_routing=True)
    for r, (gidx, gw, gkeff, guni) in enumerate(routing):
        assert np.array_equal(gidx, idx) and np.array_equal(gkeff, keff) and list(guni) == list(uni)
        lo, hi = r * (m // world), (r + 1) * (m // world)
        assert np.array_equal(bits(gw[lo:hi]), bits(w[lo:hi]))  # gate weights: the home tokens' only


def test_emulated_ranks_per_row_format_and_no_shared_expert(dev):
    layer = synth_layer(91, hidden=128, inter=64, n_experts=8, k=2, gs=0, shared=False)
    xs = [synth_tokens(7, 4, 128)]
    got, _ = run_emulated(dev, layer, xs, 4)
    assert np.array_equal(bits(got[0]), bits(oracle_layer_forward(layer, xs[0])))


def test_single_rank_ep_equals_plain_forward(dev):
    import torch

    layer = synth_layer(77, hidden=256, inter=64, n_experts=8, k=2, gs=32)
    x = synth_tokens(5, 4, 256)
    ml = upload_ep_layer(dev, layer, 0, 1)
    ws = EpWorkspace(dev, 0, 1, 4, 256, 2)
    run = EpLayerRunner(ml, ws)
    with torch.cuda.stream(run.stream):
        out = run.forward(torch.from_numpy(x).cuda(dev)).clone()
    run.stream.synchronize()
    assert np.array_equal(bits(out.cpu().numpy()), bits(oracle_layer_forward(layer, x)))
    ws.free()
    ml.free()
