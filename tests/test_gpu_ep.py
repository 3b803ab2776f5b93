"""Expert-parallel decomposition on one GPU: `world` layer objects, each holding only the experts
its rank owns, run the partial forward on the same batch; the pair-row buffers are summed (standing
in for the collective) and every rank combines its home tokens.  The result must equal the oracle's
single-process layer bit for bit, for every world size."""
import numpy as np
import pytest

from peregrine_b200 import cuda
from peregrine_b200.ep import EpLayerRunner, upload_ep_layer
from peregrine_b200.synth import synth_layer, synth_tokens
from tests.gpu_common import bits
from tests.refmodel import oracle_layer_forward

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,m", [(2, 2), (2, 8), (4, 8), (8, 32)])
def test_ep_partials_sum_to_the_single_device_layer(dev, world, m):
    import torch

    layer = synth_layer(40 + world + m, hidden=256, inter=96, n_experts=16, k=4, gs=32)
    x = synth_tokens(world * 100 + m, m, 256)
    want = oracle_layer_forward(layer, x, threads=4)
    runners = []
    for r in range(world):
        ml = upload_ep_layer(dev, layer, r, world)
        runners.append(EpLayerRunner(ml, dev, r, 1, m))  # collectives are emulated below
        runners[-1].rank, runners[-1].world_emulated = r, world
    stream = runners[0].stream
    m_local = m // world
    with torch.cuda.stream(stream):
        x_all = torch.from_numpy(x).cuda(dev)
        total = None
        for r, run in enumerate(runners):
            run.ml.ep_partial_dev(run.y_pairs.data_ptr(), x_all.data_ptr(), m)
            total = run.y_pairs.clone() if total is None else total + run.y_pairs
        outs = []
        for r, run in enumerate(runners):
            out = torch.empty((m_local, 256), dtype=torch.float32, device=dev)
            run.ml.ep_combine_dev(out.data_ptr(), total.data_ptr(), m, r * m_local, m_local)
            outs.append(out)
        got = torch.cat(outs, 0)
    stream.synchronize()
    got = got.cpu().numpy()
    assert np.array_equal(bits(got), bits(want))
    # every pair row has exactly one owner: the partial buffers never overlap
    with torch.cuda.stream(stream):
        nz = sum((run.y_pairs != 0).any(dim=1).to(torch.int32) for run in runners)
    stream.synchronize()
    assert int(nz.max().item()) <= 1
    assert cuda.last_device_error(dev) == 0
    for run in runners:
        run.ml.free()


def test_single_rank_ep_equals_plain_forward(dev):
    import torch

    layer = synth_layer(77, hidden=256, inter=64, n_experts=8, k=2, gs=32)
    x = synth_tokens(5, 4, 256)
    ml = upload_ep_layer(dev, layer, 0, 1)
    run = EpLayerRunner(ml, dev, 0, 1, 4)
    with torch.cuda.stream(run.stream):
        out = run.forward(torch.from_numpy(x).cuda(dev)).clone()
    run.stream.synchronize()
    want = oracle_layer_forward(layer, x)
    assert np.array_equal(bits(out.cpu().numpy()), bits(want))
    ml.free()
