"""KAD-CNet-S on the B200 engine against the reference-made fixture and the CPU oracle."""
import json

import numpy as np
import pytest
import torch

from helpers import rel_err, round_to
from oracle import kad_oracle as ko
from oracle import seeding

pytestmark = pytest.mark.gpu


def _sd(golden_dir, dtype=None):
    g = np.load(golden_dir / 'detector_s.npz')
    shapes = json.loads(bytes(g['shapes_json']).decode())
    sd = seeding.seeded_state_dict(shapes, seed=int(g['seed']))
    return g, sd


def test_engine_fp32_matches_fixture(golden_dir):
    import kadcnet
    from kadcnet.postprocess import non_max_suppression
    g, sd = _sd(golden_dir)
    fast = kadcnet.load_model(None, 'optimized', 'cuda:0', state_dict=sd, dtype=torch.float32)
    img = seeding.seeded_input((1, 3, 160, 192), seed=int(g['seed']), kind='image')
    y, raw = fast(img.cuda().float() / 255)
    ref = torch.from_numpy(g['y'])
    assert y.shape == ref.shape
    assert rel_err(y.cpu(), ref) <= 1e-5
    assert (raw[0].cpu().float() - torch.from_numpy(g['raw0'])).abs().max().item() <= 1e-3
    det = non_max_suppression(y, 0.001, 0.65, max_det=300)[0].cpu()
    gd = torch.from_numpy(g['det'])
    assert det.shape == gd.shape
    assert torch.equal(det[:, 5], gd[:, 5])
    assert (det[:, :4] - gd[:, :4]).abs().max().item() <= 1e-2


@pytest.mark.parametrize('backend', ['optimized', 'graph'])
def test_engine_fp16_relative(golden_dir, backend):
    """fp16 engine vs the fp32 oracle on fp16-rounded weights and input: relative 1e-2."""
    import kadcnet
    from kadconv import ops
    g, sd = _sd(golden_dir)
    sd16 = {k: round_to(v, torch.float16) for k, v in sd.items()}
    img = seeding.seeded_input((2, 3, 160, 192), seed=5, kind='image')
    x = round_to(img.float() / 255, torch.float16)
    ref, _ = ko.detector(sd16, x)
    fast = kadcnet.load_model(None, backend, 'cuda:0', state_dict=sd16, dtype=torch.float16)
    y, raw = fast(x.cuda().half())
    y2, _ = fast(x.cuda().half())
    torch.cuda.synchronize()
    ops.check_status(torch.device('cuda', 0))
    assert torch.equal(y, y2)
    # boxes in pixels and scores in [0,1] have different scales: check them separately
    assert rel_err(y[:, :4].float().cpu(), ref[:, :4]) <= 1e-2
    assert rel_err(y[:, 4:].float().cpu(), ref[:, 4:]) <= 1e-2
