"""KAD-CNet-S module definitions: state_dict compatibility with the reference and fixture parity on CPU."""
import json

import numpy as np
import torch

from oracle import kad_oracle as ko
from oracle import seeding


def _fixture(golden_dir):
    g = np.load(golden_dir / 'detector_s.npz')
    shapes = json.loads(bytes(g['shapes_json']).decode())
    return g, shapes


def test_state_dict_keys_match_reference(golden_dir):
    from kadcnet.model import DetectionModel
    g, shapes = _fixture(golden_dir)
    m = DetectionModel()
    mine = seeding.shapes_of(m)
    assert sorted(mine) == sorted(shapes)
    assert all(tuple(mine[k]) == tuple(shapes[k]) for k in shapes)
    assert [float(s) for s in m.stride] == [8.0, 16.0, 32.0]


def test_plain_model_and_nms_match_fixture(golden_dir):
    import kadcnet
    from kadcnet.postprocess import non_max_suppression
    g, shapes = _fixture(golden_dir)
    sd = seeding.seeded_state_dict(shapes, seed=int(g['seed']))
    model = kadcnet.load_model(None, 'raw', 'cpu', state_dict=sd)
    img = seeding.seeded_input((1, 3, 160, 192), seed=int(g['seed']), kind='image')
    with torch.no_grad():
        y, raw = model(img.float() / 255)
    ref = torch.from_numpy(g['y'])
    assert ((y - ref).abs().max() / ref.abs().max()).item() <= 1e-5
    det = non_max_suppression(ref, 0.001, 0.65, max_det=300)[0]
    assert torch.equal(det, torch.from_numpy(g['det']))
    # oracle NMS (no torchvision) agrees with the package's
    assert torch.equal(ko.non_max_suppression(ref, 0.001, 0.65, max_det=300)[0], det)


def test_optimized_backend_refuses_cpu():
    import pytest
    import kadcnet
    with pytest.raises(ValueError):
        kadcnet.load_model(None, 'optimized', 'cpu')


def test_conv3x3_weight_packing_host_logic():
    """pack_conv3x3_weight is host-side layout work: [Cout, Cin/g, 3, 3] -> [Cout, 9, Cin] tap-major; a grouped
    convolution becomes the dense one with zeros outside each group's block (checked through torch's conv2d on CPU)."""
    import torch.nn.functional as F
    from kadconv import ops
    g = torch.Generator().manual_seed(0)
    x = torch.randn((1, 16, 7, 9), generator=g)
    w = torch.randn((8, 4, 3, 3), generator=g)
    packed = ops.pack_conv3x3_weight(w, torch.float32, groups=4)
    assert tuple(packed.shape) == (8, 9, 16)
    dense = packed.reshape(8, 3, 3, 16).permute(0, 3, 1, 2).contiguous()        # back to [Cout, Cin, 3, 3]
    assert torch.allclose(F.conv2d(x, dense, None, 1, 1), F.conv2d(x, w, None, 1, 1, 1, 4), atol=1e-6)
    plain = ops.pack_conv3x3_weight(w, torch.float16)
    assert plain.dtype == torch.float16 and tuple(plain.shape) == (8, 9, 4)
    assert torch.equal(plain[3, 5].float(), w[3, :, 1, 2].half().float())        # tap 5 = (ky 1, kx 2)
