"""KAD-CNet-S on the B200 engine against the reference-made fixture and the CPU oracle."""
import json

import numpy as np
import pytest
import torch

from helpers import rel_err, round_to
from oracle import kad_oracle as ko
from oracle import seeding

pytestmark = pytest.mark.gpu


def match_fraction(det, ref, tol=0.05):
    """Fraction of reference detections that have a detection of the same class within `tol` pixels."""
    if ref.shape[0] == 0:
        return 1.0
    hit = 0
    for r in ref:
        same = det[det[:, 5] == r[5]]
        if same.shape[0] and (same[:, :4] - r[:4]).abs().amax(1).min().item() <= tol:
            hit += 1
    return hit / ref.shape[0]


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
    # NMS of the reference's own y, run on the GPU, reproduces the fixture's detections (the CPU and CUDA
    # library NMS may order exact score ties differently, hence a match fraction and not bit equality) ...
    gd = torch.from_numpy(g['det'])
    det_ref = non_max_suppression(ref.cuda(), 0.001, 0.65, max_det=300)[0].cpu()
    assert match_fraction(det_ref, gd) >= 0.97 and abs(det_ref.shape[0] - gd.shape[0]) <= 2
    # ... and so does NMS of the engine's y, except where a 1e-6 difference flips a borderline IoU comparison
    det = non_max_suppression(y, 0.001, 0.65, max_det=300)[0].cpu()
    assert match_fraction(det, gd) >= 0.95 and abs(det.shape[0] - gd.shape[0]) <= 3


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
