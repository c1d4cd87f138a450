"""Letterbox preprocessing and box rescaling: the CPU oracle against the reference-made fixture (cv2 + the reference's
letterbox / scale_boxes), the host-side geometry and coefficient tables, and the CUDA kernels against the same fixture."""
import numpy as np
import pytest
import torch

from oracle import preprocess_oracle as po


def _cases(golden_dir):
    g = np.load(golden_dir / 'preprocess.npz')
    for i in range(int(g['n'])):
        yield i, g[f'img{i}'], g[f'x{i}'], int(g[f'size{i}']), g[f'ratio{i}'], g[f'pad{i}'], g[f'boxes{i}'], g[f'scaled{i}']


def test_oracle_reproduces_reference_letterbox_and_scale_boxes(golden_dir):
    n = 0
    for i, img, x, size, ratio, pad, boxes, scaled in _cases(golden_dir):
        proc, r, p = po.letterbox(img, (size, size))
        assert np.array_equal(po.to_network_input(proc)[0], x), f'case {i}: letterbox differs from the reference'
        assert np.allclose(r, ratio, rtol=0, atol=0) and np.allclose(p, pad, rtol=0, atol=0)
        assert np.array_equal(po.scale_boxes(x.shape[1:], boxes, img.shape), scaled), f'case {i}: scale_boxes differs'
        n += 1
    assert n == 8


def test_host_geometry_and_tables_follow_the_reference(golden_dir):
    from kadcnet import preprocess as pp
    for i, img, x, size, ratio, pad, boxes, scaled in _cases(golden_dir):
        g = pp.letterbox_geometry(img.shape[:2], (size, size))
        assert g['out_shape'] == tuple(x.shape[1:]) and tuple(g['ratio']) == tuple(ratio) and tuple(g['pad']) == tuple(pad)
        new_w, new_h = g['new_unpad']
        # the tables drive the same integer passes as the oracle's resize: rebuild the resized image from them on the host
        if (new_h, new_w) != img.shape[:2] and not (img.shape[0] == 2 * new_h and img.shape[1] == 2 * new_w):
            xo, xa = pp.resize_tables(img.shape[1], new_w, True)
            yo, yb = pp.resize_tables(img.shape[0], new_h, False)
            v = img.astype(np.int32)
            rows = v[:, xo] * xa[None, :, 0, None].astype(np.int32) + v[:, np.minimum(xo + 1, img.shape[1] - 1)] * xa[None, :, 1, None].astype(np.int32)
            y0, y1 = np.clip(yo, 0, img.shape[0] - 1), np.clip(yo + 1, 0, img.shape[0] - 1)
            out = (((yb[:, 0, None, None].astype(np.int32) * (rows[y0] >> 4)) >> 16) + ((yb[:, 1, None, None].astype(np.int32) * (rows[y1] >> 4)) >> 16) + 2) >> 2
            assert np.array_equal(out.astype(np.uint8), po.resize_linear_u8(img, new_w, new_h))
    # auto / scaleup options, against the oracle's letterbox (which restates the reference's expressions)
    geo = pp.letterbox_geometry((300, 500), 640, auto=True, stride=32)
    ref = po.letterbox(np.zeros((300, 500, 3), np.uint8), 640, auto=True)[0]
    assert geo['out_shape'] == ref.shape[:2]
    assert pp.letterbox_geometry((100, 80), 640, scaleup=False)['new_unpad'] == (80, 100)
    assert pp.scale_boxes_geometry((64, 64), (60, 80, 3))[0] == min(64 / 60, 64 / 80)


@pytest.mark.gpu
def test_letterbox_and_scale_boxes_kernels_match_the_reference(golden_dir):
    """kad_letterbox_u8 and kad_scale_boxes through kadcnet.preprocess against the reference-made fixture: bit-equal pixels (resize
    up, down, exact 2x shrink, no resize, odd sizes, padding on either axis) and bit-equal rounded boxes."""
    from kadcnet import preprocess as pp
    for i, img, x, size, ratio, pad, boxes, scaled in _cases(golden_dir):
        out, r, p = pp.letterbox_device(torch.from_numpy(img).cuda(), (size, size))
        assert out.shape == (1,) + x.shape and out.dtype == torch.uint8
        assert np.array_equal(out[0].cpu().numpy(), x), f'case {i}'
        assert tuple(r) == tuple(ratio) and tuple(p) == tuple(pad)
        # two images in one call, different counts; rows past the count stay untouched
        n = boxes.shape[0]
        dets = torch.zeros((2, n + 3, 6), dtype=torch.float32)
        dets[0, :n, :4] = torch.from_numpy(boxes); dets[1, :n - 5, :4] = torch.from_numpy(boxes[:n - 5])
        dets[..., 4] = 0.5; dets[0, n:, :4] = -7.0
        counts = torch.tensor([n, n - 5], dtype=torch.int32)
        res = pp.scale_boxes_device(dets.cuda(), counts.cuda(), x.shape[1:], [img.shape, img.shape]).cpu()
        assert np.array_equal(res[0, :n, :4].numpy(), scaled) and np.array_equal(res[1, :n - 5, :4].numpy(), scaled[:n - 5])
        assert torch.equal(res[0, n:, :4], torch.full((3, 4), -7.0)) and torch.equal(res[..., 4], dets[..., 4])
    # a full-size image: 1080 x 1920 BGR -> 800 x 800 letterbox, against the oracle
    g = np.random.default_rng(5)
    big = g.integers(0, 256, (1080, 1920, 3), dtype=np.uint8)
    out, _, _ = pp.letterbox_device(torch.from_numpy(big).cuda(), (800, 800))
    assert np.array_equal(out[0].cpu().numpy(), po.to_network_input(po.letterbox(big, (800, 800))[0])[0])


@pytest.mark.gpu
def test_letterboxed_uint8_feeds_the_engine(golden_dir):
    """The whole device path of the inference script: BGR image -> letterbox kernel -> engine (uint8 entry) -> batched NMS ->
    scale_boxes kernel, against the same steps on the host (oracle letterbox, reference-order scale_boxes) around the same engine."""
    import json
    import kadcnet
    from kadcnet import preprocess as pp
    from kadcnet.postprocess import non_max_suppression_device
    from kadconv import ops
    from oracle import seeding
    g = np.load(golden_dir / 'detector_s.npz')
    sd = seeding.seeded_state_dict(json.loads(bytes(g['shapes_json']).decode()), seed=int(g['seed']))
    fast = kadcnet.load_model(None, 'optimized', 'cuda:0', state_dict=sd, dtype=torch.float16)
    img = np.random.default_rng(9).integers(0, 256, (150, 260, 3), dtype=np.uint8)
    x, _, _ = pp.letterbox_device(torch.from_numpy(img).cuda(), (160, 192))
    assert np.array_equal(x.cpu().numpy(), po.to_network_input(po.letterbox(img, (160, 192))[0]))
    y = fast(x)[0]
    dets, counts = ops.nms_batched(y.contiguous(), 0.25, 0.65, 300)
    ref = [d.cpu().numpy().copy() for d in non_max_suppression_device(y, 0.25, 0.65, max_det=300)]
    pp.scale_boxes_device(dets, counts, x.shape[2:], [img.shape])
    n = int(counts[0])
    assert n == ref[0].shape[0] and n > 0
    assert np.array_equal(dets[0, :n, :4].cpu().numpy(), po.scale_boxes(tuple(x.shape[2:]), ref[0][:, :4], img.shape))
    assert np.array_equal(dets[0, :n, 4:].cpu().numpy(), ref[0][:, 4:])
