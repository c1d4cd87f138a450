"""Generate the golden fixtures in this directory by running the REFERENCE modules on CPU.

Run where the reference checkout is available: set KAD_REFERENCE_ROOT to its path (default: `reference`
beside this repository). The tests never need it: they only read the committed .npz files.

    python tests/golden/make_golden.py

Fixtures (all float32, weights are NOT stored: they are regenerated from oracle/seeding.py):
  kadconv_c24.npz   KADConv(24) on [2,24,13,11]: output, plus per-branch offset / mask / DSC output
  kadconv_c64.npz   KADConv(64) on [1,64,25,25] (odd size: 25 -> 12 -> 6 pyramid): output
  dcn_op.npz        torchvision.ops.deform_conv2d on [2,16,9,12] -> 24 channels, offsets N(0,2)
  detector_s.npz    KAD-CNet-S (dior_s_base graph) on [1,3,160,192]: y[1,24,A], NMS detections and the
                    model's state_dict key -> shape table (so the weights can be regenerated)
  preprocess.npz    letterbox() (cv2) + BGR->RGB + CHW on eight small images, and scale_boxes(...).round() of seeded boxes
"""
import json
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch
import torchvision

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
REF = Path(os.environ.get('KAD_REFERENCE_ROOT', str(ROOT.parent / 'reference')))
sys.path.insert(0, str(ROOT))
from oracle import seeding  # noqa: E402


def _stub(name, **attrs):
    m = types.ModuleType(name)
    m.__dict__.update(attrs)
    sys.modules[name] = m
    return m


def import_reference_detector():
    """The detector imports plotting packages that are absent here and unused at inference."""
    ip = _stub('IPython'); ipd = _stub('IPython.display', display=lambda *a, **k: None); ip.display = ipd
    mpl = _stub('matplotlib', use=lambda *a, **k: None, rc=lambda *a, **k: None)
    mpl.pyplot = _stub('matplotlib.pyplot')
    _stub('seaborn')
    sys.path.insert(0, str(REF / 'KAD-CNet'))
    import models.yolo as yolo
    from utils.general import non_max_suppression
    return yolo, non_max_suppression


def golden_kadconv():
    sys.path.insert(0, str(REF / 'KAD-Conv'))
    from kadconv import KADConv
    for name, dim, shape, seed in (('kadconv_c24', 24, (2, 24, 13, 11), 3), ('kadconv_c64', 64, (1, 64, 25, 25), 4)):
        layer = KADConv(dim).eval()
        sd = seeding.seeded_state_dict(seeding.shapes_of(layer), seed=seed)
        layer.load_state_dict(sd)
        x = seeding.seeded_input(shape, seed=seed)
        parts = {}
        with torch.no_grad():
            y = layer(x)
            for i, conv in enumerate(layer.convs):
                xi = torch.nn.functional.avg_pool2d(x, 2 ** i) if i else x
                t = conv[0](xi)
                d = conv[1]
                parts[f'offset{i}'] = d.conv_offset(t).numpy()
                parts[f'mask{i}'] = torch.sigmoid(d.RCA_mask(t)).numpy()
                parts[f'dsc{i}'] = d(t).numpy()
        np.savez_compressed(HERE / f'{name}.npz', y=y.numpy(), seed=seed, dim=dim, shape=np.array(shape), **parts)
        print(name, 'offset std', float(np.std(parts['offset0'])), 'y absmax', float(y.abs().max()))


def golden_dcn():
    g = np.random.default_rng(7)
    x = torch.from_numpy(g.standard_normal((2, 16, 9, 12)).astype(np.float32))
    off = torch.from_numpy((2.0 * g.standard_normal((2, 18, 9, 12))).astype(np.float32))
    msk = torch.sigmoid(torch.from_numpy(g.standard_normal((2, 9, 9, 12)).astype(np.float32)))
    w = torch.from_numpy(g.uniform(-1 / 12, 1 / 12, (24, 16, 3, 3)).astype(np.float32))
    b = torch.from_numpy(g.standard_normal(24).astype(np.float32))
    y = torchvision.ops.deform_conv2d(x, off, w, b, stride=1, padding=1, mask=msk)
    np.savez_compressed(HERE / 'dcn_op.npz', x=x.numpy(), offset=off.numpy(), mask=msk.numpy(), weight=w.numpy(),
                        bias=b.numpy(), y=y.numpy())
    print('dcn_op', tuple(y.shape))


def golden_detector():
    yolo, nms = import_reference_detector()
    torch.manual_seed(0)
    model = yolo.DetectionModel(str(REF / 'KAD-CNet/configs/dior_s_base.yaml')).eval()
    shapes = seeding.shapes_of(model)
    sd = seeding.seeded_state_dict(shapes, seed=11)
    model.load_state_dict(sd)
    model = model.float().fuse().eval()
    img = seeding.seeded_input((1, 3, 160, 192), seed=11, kind='image')
    x = img.float() / 255
    with torch.no_grad():
        y, raw = model(x)
        det = nms(y, 0.001, 0.65, max_det=300)[0]
    np.savez_compressed(HERE / 'detector_s.npz', y=y.numpy(), det=det.numpy(), seed=11,
                        stride=model.stride.numpy(), raw0=raw[0].numpy(),
                        shapes_json=np.frombuffer(json.dumps(shapes).encode(), dtype=np.uint8))
    print('detector', tuple(y.shape), 'detections', tuple(det.shape), 'max score', float(y[:, 4:].max()))


def golden_preprocess():
    """letterbox() of the reference (on the real cv2) + the BGR->RGB / CHW step of its inference script, and scale_boxes(...).round(),
    on small seeded images: up- and down-scaling, an exact 2x shrink (OpenCV's area path), no resize at all, odd sizes."""
    import_reference_detector()
    from utils.augmentations import letterbox
    from utils.general import scale_boxes
    cases = [((60, 80), 64), ((96, 72), 64), ((48, 64), 96), ((128, 128), 64), ((64, 64), 64), ((37, 91), 96), ((75, 50), 64), ((33, 200), 128)]
    out = {'n': len(cases)}
    for i, (shape, size) in enumerate(cases):
        g = np.random.default_rng([77, i])
        img = g.integers(0, 256, shape + (3,), dtype=np.uint8)
        proc, ratio, pad = letterbox(img, new_shape=(size, size), auto=False, stride=32)
        x = np.ascontiguousarray(proc[:, :, ::-1].transpose(2, 0, 1))
        boxes = g.uniform(-4, size + 4, (40, 4)).astype(np.float32)
        boxes[:, 2:] = boxes[:, :2] + np.abs(boxes[:, 2:] - boxes[:, :2])
        scaled = scale_boxes(x.shape[1:], torch.from_numpy(boxes.copy()), img.shape).round().numpy()
        out.update({f'img{i}': img, f'x{i}': x, f'size{i}': size, f'ratio{i}': np.array(ratio), f'pad{i}': np.array(pad), f'boxes{i}': boxes, f'scaled{i}': scaled})
    np.savez_compressed(HERE / 'preprocess.npz', **out)
    print('preprocess', len(cases), 'cases')


if __name__ == '__main__':
    golden_kadconv()
    golden_dcn()
    golden_detector()
    golden_preprocess()
