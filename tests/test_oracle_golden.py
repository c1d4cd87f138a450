"""The CPU oracle must reproduce what the reference's own modules produced (tests/golden/*.npz)."""
import json

import numpy as np
import torch

from oracle import kad_oracle as ko
from oracle import seeding


def _kadconv_shapes(dim, se_min_hidden=32):
    widths = [dim - (dim // 3) * 2, dim // 3, dim // 3]
    s = {}
    for i, c in enumerate(widths):
        h = max(se_min_hidden, c)
        s[f'convs.{i}.0.weight'] = (c, dim, 1, 1); s[f'convs.{i}.0.bias'] = (c,)
        d = f'convs.{i}.1'
        s[d + '.weight'] = (c, c, 3, 3); s[d + '.bias'] = (c,)
        s[d + '.conv_offset.weight'] = (18, c, 3, 3); s[d + '.conv_offset.bias'] = (18,)
        e = d + '.RCA_mask.excite'
        s[e + '.0.weight'] = (c, 1, 1, 11); s[e + '.0.bias'] = (c,)
        for leaf in ('weight', 'bias', 'running_mean', 'running_var'):
            s[f'{e}.1.{leaf}'] = (c,)
        s[e + '.1.num_batches_tracked'] = ()
        s[e + '.3.weight'] = (c, 1, 11, 1); s[e + '.3.bias'] = (c,)
        s[e + '.4.weight'] = (9, c, 1, 1); s[e + '.4.bias'] = (9,)
        for leaf in ('weight', 'bias', 'running_mean', 'running_var'):
            s[f'convs.{i}.2.{leaf}'] = (c,)
        s[f'convs.{i}.2.num_batches_tracked'] = ()
        s[f'fc.{i}.0.weight'] = (h, c); s[f'fc.{i}.0.bias'] = (h,)
        s[f'fc.{i}.2.weight'] = (c, h); s[f'fc.{i}.2.bias'] = (c,)
        s[f'weight.{i}.0.weight'] = (1, c, 1, 1)
    return s


def test_deform_conv_matches_torchvision_fixture(golden_dir):
    g = np.load(golden_dir / 'dcn_op.npz')
    t = {k: torch.from_numpy(g[k]) for k in g.files}
    y = ko.deform_conv2d(t['x'], t['offset'], t['weight'], t['bias'], t['mask'])
    assert (y - t['y']).abs().max().item() <= 2e-5
    y64 = ko.deform_conv2d(t['x'].double(), t['offset'].double(), t['weight'].double(), t['bias'].double(),
                           t['mask'].double())
    assert (y64.float() - t['y']).abs().max().item() <= 2e-5


def test_kadconv_matches_reference_fixture(golden_dir):
    for name in ('kadconv_c24', 'kadconv_c64'):
        g = np.load(golden_dir / f'{name}.npz')
        dim, seed, shape = int(g['dim']), int(g['seed']), tuple(int(v) for v in g['shape'])
        sd = seeding.seeded_state_dict(_kadconv_shapes(dim), seed=seed)
        x = seeding.seeded_input(shape, seed=seed)
        y = ko.kadconv(sd, '', x)
        assert y.shape == x.shape
        assert (y - torch.from_numpy(g['y'])).abs().max().item() <= 1e-5
        # branch internals: offsets, sigmoid mask and DSC output of every branch
        for i in range(3):
            xi = torch.nn.functional.avg_pool2d(x, 2 ** i) if i else x
            t = torch.nn.functional.conv2d(xi, sd[f'convs.{i}.0.weight'], sd[f'convs.{i}.0.bias'])
            d, off, msk = ko.dsc(sd, f'convs.{i}.1', t, return_parts=True)
            assert (off - torch.from_numpy(g[f'offset{i}'])).abs().max().item() <= 1e-5
            assert (msk - torch.from_numpy(g[f'mask{i}'])).abs().max().item() <= 1e-5
            assert (d - torch.from_numpy(g[f'dsc{i}'])).abs().max().item() <= 1e-5
        assert float(np.std(g['offset0'])) > 0.1   # the fixture really exercises deformation


def test_detector_matches_reference_fixture(golden_dir):
    g = np.load(golden_dir / 'detector_s.npz')
    shapes = json.loads(bytes(g['shapes_json']).decode())
    sd = seeding.seeded_state_dict(shapes, seed=int(g['seed']))
    img = seeding.seeded_input((1, 3, 160, 192), seed=int(g['seed']), kind='image')
    y, raw = ko.detector(sd, img.float() / 255, strides=tuple(float(s) for s in g['stride']))
    ref = torch.from_numpy(g['y'])
    assert y.shape == ref.shape
    assert ((y - ref).abs().max() / ref.abs().max()).item() <= 1e-5
    assert (raw[0] - torch.from_numpy(g['raw0'])).abs().max().item() <= 1e-3
    det = ko.non_max_suppression(ref, 0.001, 0.65, max_det=300)[0]
    gd = torch.from_numpy(g['det'])
    assert det.shape == gd.shape and gd.shape[0] > 10
    assert torch.equal(det, gd)     # same boxes, same order, bit for bit


def test_c_restatement_matches_fixture(golden_dir):
    """The plain-C deformable convolution (oracle/dsc_oracle.c) against the torchvision-made fixture."""
    import ctypes
    import subprocess
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    subprocess.run(['make', '-s', '-C', str(root / 'oracle')], check=True)
    lib = ctypes.CDLL(str(root / 'oracle' / '_build' / 'libkad_oracle.so'))
    g = np.load(golden_dir / 'dcn_op.npz')
    a = {k: np.ascontiguousarray(g[k], dtype=np.float32) for k in g.files}
    B, Cin, H, W = a['x'].shape
    Cout = a['weight'].shape[0]
    y = np.zeros((B, Cout, H, W), dtype=np.float32)
    P = ctypes.POINTER(ctypes.c_float)
    ptr = lambda t: t.ctypes.data_as(P)
    lib.kad_oracle_deform_conv3x3(ptr(a['x']), ptr(a['offset']), ptr(a['mask']), ptr(a['weight']), ptr(a['bias']), ptr(y),
                                  B, Cin, Cout, H, W)
    assert np.abs(y - a['y']).max() <= 2e-5
