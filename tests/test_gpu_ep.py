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


def test_two_layers_share_the_exchange_blocks(dev):
    """A stack's MoE layers share one exchange block per rank: two layers stepped alternately for a few
    decode steps (every layer step takes the next of the two buffer sets) give the oracle's bits."""
    import torch

    world, m, d = 2, 4, 256
    layers = [synth_layer(300 + i, hidden=d, inter=64, n_experts=8, k=2, gs=32) for i in range(2)]
    wss = [EpWorkspace(dev, r, world, m, d, 2) for r in range(world)]
    connect_emulated(wss)
    runs = [[EpLayerRunner(upload_ep_layer(dev, layer, r, world), wss[r]) for r in range(world)] for layer in layers]
    stream = runs[0][0].stream
    x = synth_tokens(12, m, d)
    want = x.copy()
    with torch.cuda.stream(stream):
        cur = torch.from_numpy(x).cuda(dev)
        for step in range(3):
            for li in range(2):
                for r, run in enumerate(runs[li]):
                    run.route(cur[r * 2:(r + 1) * 2])
                for run in runs[li]:
                    run.dispatch()
                for run in runs[li]:
                    run.experts()
                cur = torch.cat([run.finish().clone() for run in runs[li]], 0) * 0.01
    stream.synchronize()
    for step in range(3):
        for li in range(2):
            want = (oracle_layer_forward(layers[li], want) * np.float32(0.01)).astype(np.float32)
    assert np.array_equal(bits(cur.cpu().numpy()), bits(want))
    assert cuda.last_device_error(dev) == 0
    for ws in wss:
        ws.free()


def test_a_silent_peer_runs_the_wait_out_and_is_reported(dev):
    """Failure detection without a fault: rank 0 plans a step for which rank 1 never published its
    picks.  The bounded wait gives up after about a second, the error word says so, the rank's later
    waits give up at once (the queued launches drain in microseconds), and after a reset the pair of
    ranks computes correctly again."""
    import time

    import torch

    world, m, d = 2, 2, 128
    layer = synth_layer(55, hidden=d, inter=64, n_experts=4, k=2, gs=32)
    wss = [EpWorkspace(dev, r, world, m, d, 2) for r in range(world)]
    connect_emulated(wss)
    runs = [EpLayerRunner(upload_ep_layer(dev, layer, r, world), wss[r]) for r in range(world)]
    stream = runs[0].stream
    x = synth_tokens(3, m, d)
    with torch.cuda.stream(stream):
        xd = torch.from_numpy(x).cuda(dev)
        runs[0].route(xd[0:1])
        runs[0].dispatch()          # waits for rank 1's picks, which never come
        stream.synchronize()
        t0 = time.perf_counter()
        runs[0].experts()
        runs[0].finish()
        stream.synchronize()
        drained = time.perf_counter() - t0
    assert cuda.last_device_error(dev) == 1   # kErrBarrierTimeout, cleared by the read
    assert drained < 0.5                      # nothing waited a second time
    # the ranks meet again (here: the test itself), clear the state and realign their step counters
    for ws in wss:
        assert cuda.lib().coli_cuda_ep_reset(ws.handle) == 1
    with torch.cuda.stream(stream):
        runs[1].route(xd[1:2])      # rank 1 catches up with the step rank 0 already counted
        runs[1].dispatch()
        runs[1].experts()
        runs[1].finish()
        stream.synchronize()
        cuda.last_device_error(dev)  # rank 1's own view of that broken step does not matter
        for ws in wss:
            assert cuda.lib().coli_cuda_ep_reset(ws.handle) == 1
        for r, run in enumerate(runs):
            run.route(xd[r:r + 1])
        for run in runs:
            run.dispatch()
        for run in runs:
            run.experts()
        got = torch.cat([run.finish().clone() for run in runs], 0)
    stream.synchronize()
    assert cuda.last_device_error(dev) == 0
    assert np.array_equal(bits(got.cpu().numpy()), bits(oracle_layer_forward(layer, x)))
    for ws in wss:
        ws.free()
