"""Host-side logic that needs no GPU: error reporting, cache invalidation, checkpoint loading, the NMS explanation helper."""
import json

import numpy as np
import pytest
import torch

import nms_explain as ne
from helpers import kadconv_shapes
from oracle import kad_oracle as ko
from oracle import seeding


def test_status_word_raises_once_and_clears():
    from kadconv import ops
    cleared = []
    ops.raise_if_aborted([0, 0, 0, 0], lambda: cleared.append(1))          # nothing recorded: no exception, nothing cleared
    assert not cleared
    with pytest.raises(RuntimeError, match='role 3, detail 7, block 11'):
        ops.raise_if_aborted([3, 7, 11, 0], lambda: cleared.append(1))
    assert cleared == [1]


def test_parameter_fingerprint_follows_weight_changes():
    """The folded / packed copies of a layer's parameters are rebuilt when this fingerprint changes: it must change on
    load_state_dict (in-place copy), on an in-place edit, and on a cast that replaces the storage; and stay put otherwise."""
    import kadconv
    from kadconv.fast import parameter_fingerprint
    layer = kadconv.KADConv(24).eval()
    f0 = parameter_fingerprint(layer)
    assert parameter_fingerprint(layer) == f0
    layer.load_state_dict(seeding.seeded_state_dict(kadconv_shapes(24), seed=1))
    f1 = parameter_fingerprint(layer)
    assert f1 != f0
    with torch.no_grad():
        layer.weight[1][0].weight.mul_(2.0)
    f2 = parameter_fingerprint(layer)
    assert f2 != f1
    layer.double()
    assert parameter_fingerprint(layer) != f2


def test_pickled_checkpoints_load(tmp_path, golden_dir):
    """load_model on checkpoint files of the three kinds the reference's loader accepts (KAD-CNet/inference/runtime.py:44-60):
    {'model': module, 'ema': None}, {'model': ..., 'ema': module} (the EMA weights win under 'auto'), and a bare state_dict;
    half-precision checkpoints are loaded as float32."""
    import kadcnet
    from kadcnet.model import DetectionModel
    g = np.load(golden_dir / 'detector_s.npz')
    shapes = json.loads(bytes(g['shapes_json']).decode())
    sd_a = seeding.seeded_state_dict(shapes, seed=5)
    sd_b = seeding.seeded_state_dict(shapes, seed=6)
    ma, mb = DetectionModel(), DetectionModel()
    ma.load_state_dict(sd_a); mb.load_state_dict(sd_b)
    p1, p2, p3 = tmp_path / 'model_only.pt', tmp_path / 'with_ema.pt', tmp_path / 'state_dict.pt'
    torch.save({'model': ma.half(), 'ema': None, 'epoch': 3}, p1)
    torch.save({'model': ma, 'ema': mb}, p2)
    torch.save(sd_b, p3)

    def first_weights(model):
        return {k: v for k, v in model.state_dict().items() if k.startswith('model.1.')}

    m1 = kadcnet.load_model(str(p1), 'raw', 'cpu', fuse=False)
    assert all(v.dtype == torch.float32 for v in m1.state_dict().values() if v.is_floating_point())
    for k, v in first_weights(m1).items():
        if v.is_floating_point():
            assert torch.equal(v, sd_a[k].half().float())
    m2 = kadcnet.load_model(str(p2), 'raw', 'cpu', fuse=False)
    assert all(torch.equal(v, sd_b[k]) for k, v in first_weights(m2).items())
    m2m = kadcnet.load_model(str(p2), 'raw', 'cpu', fuse=False, checkpoint_key='model')
    assert all(torch.equal(v, sd_a[k].half().float() if v.is_floating_point() else sd_a[k]) for k, v in first_weights(m2m).items())
    m3 = kadcnet.load_model(str(p3), 'raw', 'cpu', fuse=False)
    assert all(torch.equal(v, sd_b[k]) for k, v in first_weights(m3).items())
    with pytest.raises(ValueError):
        kadcnet.load_model(str(p1), 'raw', 'cpu', checkpoint_key='ema')
    # a loaded checkpoint runs: fused forward on a small image
    m = kadcnet.load_model(str(p3), 'raw', 'cpu')
    with torch.no_grad():
        y, raw = m(torch.rand(1, 3, 128, 128))
    assert y.shape == (1, 24, 16 * 16 + 8 * 8 + 4 * 4) and len(raw) == 3


def test_nms_differences_are_explained_or_flagged(golden_dir):
    """The helper the detector acceptance tests rest on: (a) its exact greedy NMS equals the oracle's and the reference-made
    detections; (b) rounding-size perturbations of the prediction change the kept set only through decisions inside the
    tolerance, and every differing box gets a reason; (c) a real localisation error (a box moved by 40 pixels) is flagged."""
    g = np.load(golden_dir / 'detector_s.npz')
    y = torch.from_numpy(g['y'])[0]
    cb = ne.candidates(y, 0.001)
    kb = ne.greedy_keep(cb, 0.65)
    rows = torch.cat((cb['box'][kb], cb['conf'][kb, None], cb['cls'][kb, None].float()), 1)
    assert torch.equal(rows, torch.from_numpy(g['det']))
    assert torch.equal(rows, ko.non_max_suppression(y[None], 0.001, 0.65, max_det=300)[0])
    gen = torch.Generator().manual_seed(1)
    for rel in (1e-6, 1e-5, 1e-4):
        ya = y * (1 + rel * torch.randn(y.shape, generator=gen))
        ca = ne.candidates(ya, 0.001)
        ka = ne.greedy_keep(ca, 0.65)
        rep = ne.check_explained(ka, ca, cb, 0.001, 0.65, eps_iou=20 * rel, eps_score=4 * rel)
        assert rep['ok'], rep
        reasons = ne.trace_differences(ka, kb, ca, cb, 0.65, 20 * rel, 4 * rel, 0.001)
        assert set(reasons) == set(ka) ^ set(kb)
        assert all(r[0] in ('iou', 'order', 'cascade', 'threshold', 'class') for r in reasons.values()), reasons
    # identical predictions: identical result, nothing to explain
    assert ne.check_explained(kb, cb, cb, 0.001, 0.65, 0.0, 0.0)['ok'] and not ne.trace_differences(kb, kb, cb, cb, 0.65, 0.0, 0.0, 0.001)
    # a localisation error is not a threshold effect: move the best box of the result by 40 pixels
    yb = y.clone()
    yb[0, kb[0]] += 40.0
    cbad = ne.candidates(yb, 0.001)
    kbad = ne.greedy_keep(cbad, 0.65)
    assert set(kbad) != set(kb)
    assert not ne.check_explained(kbad, cbad, cb, 0.001, 0.65, eps_iou=1e-3, eps_score=1e-4)['ok']
