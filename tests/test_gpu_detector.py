"""KAD-CNet-S on the B200 engine against the reference-made fixture and the CPU oracle."""
import json

import numpy as np
import pytest
import torch

from helpers import rel_err, round_to
from oracle import kad_oracle as ko
from oracle import seeding

import nms_explain as ne

pytestmark = pytest.mark.gpu

# Half-precision tolerances of the configs[3] acceptance test. Measured on a B200 (two image seeds): against the fp32 modules the
# engine's scores differ by at most 2.3e-3 and its box coordinates by at most 0.26 px (the modules' own fp16 path: 5.1e-3 and
# 0.75 px), and every NMS difference is explained once IoU comparisons get 0.02 and score comparisons 2e-3 of slack. The
# constants leave a 1.5x margin over that.
C3_EPS_SCORE = 3e-3
C3_EPS_IOU = 0.03


@pytest.fixture(autouse=True)
def library_convolutions_by_heuristics(monkeypatch):
    """load_model() turns on cuDNN's autotuning like the reference's loader does; the algorithm it picks for a 3x3 convolution
    then depends on timing noise, and with it the half-precision rounding of the library convolutions on BOTH sides of the
    comparisons below. For tests that assert measured tolerances the library picks by heuristics instead: the same
    computation on every run."""
    import kadcnet.runtime as rt
    tuned = rt.numerical_protocol

    def protocol():
        tuned()
        torch.backends.cudnn.benchmark = False
    monkeypatch.setattr(rt, 'numerical_protocol', protocol)
    yield
    torch.backends.cudnn.benchmark = False


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


def _sd_alive(golden_dir):
    """Weights under which the detector is a non-trivial function of the image: with the initialisers' own gain the signal fades
    over the 60 layers and every anchor gets nearly the same scores (the fixture above: thousands of exact score ties); a gain of
    2.6 keeps activations at unit scale, scores spread over (0.02, 0.7) and nearly all distinct."""
    g = np.load(golden_dir / 'detector_s.npz')
    shapes = json.loads(bytes(g['shapes_json']).decode())
    return seeding.seeded_state_dict(shapes, seed=int(g['seed']), weight_gain=2.6, cls_gain=30.0, cls_bias=-6.0)


def test_engine_fp32_matches_fixture(golden_dir):
    import kadcnet
    from kadcnet.postprocess import non_max_suppression_device
    g, sd = _sd(golden_dir)
    fast = kadcnet.load_model(None, 'optimized', 'cuda:0', state_dict=sd, dtype=torch.float32)
    img = seeding.seeded_input((1, 3, 160, 192), seed=int(g['seed']), kind='image')
    y, raw = fast(img.cuda().float() / 255)
    ref = torch.from_numpy(g['y'])
    assert y.shape == ref.shape
    assert rel_err(y.cpu(), ref) <= 1e-5
    assert (raw[0].cpu().float() - torch.from_numpy(g['raw0'])).abs().max().item() <= 1e-3
    # absolute per-box bound, each scale on its own (a wrong anchor order or offset on one scale cannot hide behind a global maximum)
    for lo, hi in ((0, 480), (480, 600), (600, 630)):
        assert (y[:, :4, lo:hi].cpu() - ref[:, :4, lo:hi]).abs().max().item() <= 1e-3          # pixels
        assert (y[:, 4:, lo:hi].cpu() - ref[:, 4:, lo:hi]).abs().max().item() <= 1e-5          # scores
    # Detections. The batched NMS kernel on the reference's own y reproduces the reference-made detections bit for bit ...
    gd = torch.from_numpy(g['det'])
    assert torch.equal(non_max_suppression_device(ref.cuda(), 0.001, 0.65, max_det=300)[0].cpu(), gd)
    # ... and on the engine's y it equals exact greedy NMS of that y; where that result differs from the reference-made one,
    # every difference is a decision that sits on a threshold: the kept set is a valid NMS solution of the REFERENCE's boxes and
    # scores once IoU comparisons get 1e-3 and score comparisons 1e-5 of slack, and each differing box is traced to an IoU within
    # that slack of 0.65, to a score tie (this random-init model emits exact ties), or to a box that differs for such a reason.
    det = non_max_suppression_device(y, 0.001, 0.65, max_det=300)[0].cpu()
    ca, cb = ne.candidates(y[0].cpu(), 0.001), ne.candidates(ref[0], 0.001)
    ka, kb = ne.greedy_keep(ca, 0.65), ne.greedy_keep(cb, 0.65)
    assert torch.equal(det, torch.cat((ca['box'][ka], ca['conf'][ka, None], ca['cls'][ka, None].float()), 1)[:300])
    rep = ne.check_explained(ka, ca, cb, 0.001, 0.65, eps_iou=1e-3, eps_score=1e-5)
    assert rep['ok'], rep
    reasons = ne.trace_differences(ka, kb, ca, cb, 0.65, 1e-3, 1e-5, 0.001)
    assert all(r[0] is not None for r in reasons.values()), reasons
    print(f'fp32 fixture: {len(kb)} reference detections, {len(set(ka) ^ set(kb))} differing boxes, reasons '
          f'{sorted((r[0] for r in reasons.values()))}')


def test_c3_config_detections_against_same_dtype_reference(golden_dir):
    """BASELINE configs[3] as written: fp16, one uint8 3x800x800 image, conf 0.001, IoU 0.65, max_det 300, through
    load_model(..., 'optimized') + the batched NMS kernel, against the plain modules run in fp16 on the same GPU (the
    reference's own half-precision path: library kernels, decode in half) + the reference-order NMS.
    Bit-identical detections cannot be expected between two half-precision evaluation orders (this engine decodes in fp32 and
    rounds once, the modules decode in half; the class scores carry up to 1e-2 of relative error on both sides), so the
    criterion is the one that can be stated exactly: the engine's kept set must be a valid greedy-NMS solution of the
    REFERENCE's boxes and scores within the half-precision tolerances below, and every differing box must trace to a decision
    inside them. The kernel itself is exact on its own input."""
    import kadcnet
    from kadcnet.postprocess import non_max_suppression, non_max_suppression_device
    from kadconv import ops
    sd = _sd_alive(golden_dir)
    img = seeding.seeded_input((1, 3, 800, 800), seed=3, kind='image').cuda()
    raw16 = kadcnet.load_model(None, 'raw', 'cuda:0', state_dict=sd).half()
    with torch.no_grad():
        yb = raw16(img.half() / 255)[0]
    fast = kadcnet.load_model(None, 'optimized', 'cuda:0', state_dict=sd, dtype=torch.float16)
    ya = fast(img)[0]
    torch.cuda.synchronize(); ops.check_status(img.device)
    assert ya.dtype == yb.dtype == torch.float16 and ya.shape == yb.shape == (1, 24, 13125)
    det = non_max_suppression_device(ya, 0.001, 0.65, max_det=300)[0].cpu()
    det_ref = non_max_suppression(yb, 0.001, 0.65, max_det=300)[0].cpu().float()
    ca, cb = ne.candidates(ya[0].cpu(), 0.001), ne.candidates(yb[0].cpu(), 0.001)
    ka, kb = ne.greedy_keep(ca, 0.65), ne.greedy_keep(cb, 0.65)
    rows = lambda c, k: torch.cat((c['box'][k], c['conf'][k, None], c['cls'][k, None].float()), 1)[:300]
    assert torch.equal(det, rows(ca, ka))                       # the kernel is exact greedy NMS of its input
    assert det_ref.shape[0] == min(300, len(kb))
    rep = ne.check_explained(ka, ca, cb, 0.001, 0.65, eps_iou=C3_EPS_IOU, eps_score=C3_EPS_SCORE)
    assert rep['ok'], {k: (v[:5] if isinstance(v, list) else v) for k, v in rep.items()}
    reasons = ne.trace_differences(ka, kb, ca, cb, 0.65, C3_EPS_IOU, C3_EPS_SCORE, 0.001)
    assert all(r[0] is not None for r in reasons.values())
    from collections import Counter
    print(f'c3 fp16 vs the fp16 modules: candidates {int(ca["cand"].sum())} / {int(cb["cand"].sum())}, kept {len(ka)} / {len(kb)}, differing '
          f'{len(set(ka) ^ set(kb))} (top 300: {len(set(ka[:300]) ^ set(kb[:300]))}), reasons {dict(Counter(r[0] for r in reasons.values()))}')
    # the same against the fp32 modules, and how the two half-precision paths compare with fp32: the engine (fp32 accumulation
    # and decode, one rounding per stored tensor) must be at least as close to the fp32 result as the modules' own fp16 path is
    raw32 = kadcnet.load_model(None, 'raw', 'cuda:0', state_dict=sd)
    with torch.no_grad():
        y32 = raw32(img.float() / 255)[0]
    c32 = ne.candidates(y32[0].cpu(), 0.001)
    k32 = ne.greedy_keep(c32, 0.65)
    rep32 = ne.check_explained(ka, ca, c32, 0.001, 0.65, eps_iou=C3_EPS_IOU, eps_score=C3_EPS_SCORE)
    assert rep32['ok'], {k: (v[:5] if isinstance(v, list) else v) for k, v in rep32.items()}
    assert all(r[0] is not None for r in ne.trace_differences(ka, k32, ca, c32, 0.65, C3_EPS_IOU, C3_EPS_SCORE, 0.001).values())
    e_box, e_cls = rel_err(ya[:, :4].float(), y32[:, :4]), rel_err(ya[:, 4:].float(), y32[:, 4:])
    r_box, r_cls = rel_err(yb[:, :4].float(), y32[:, :4]), rel_err(yb[:, 4:].float(), y32[:, 4:])
    print(f'c3 vs the fp32 modules: engine box {e_box:.2e} cls {e_cls:.2e}; fp16 modules box {r_box:.2e} cls {r_cls:.2e}; '
          f'differing boxes engine {len(set(ka) ^ set(k32))}, fp16 modules {len(set(kb) ^ set(k32))}')
    assert e_box <= 1e-2 and e_cls <= 1e-2                      # the stated fp16 bar (relative 1e-2), boxes and scores separately
    assert e_box <= r_box and e_cls <= r_cls
    for lo, hi in ((0, 10000), (10000, 12500), (12500, 13125)):  # per scale: <= 1 px and <= 1e-2 in score, absolutely
        assert (ya[:, :4, lo:hi].float() - y32[:, :4, lo:hi]).abs().max().item() <= 1.0
        assert (ya[:, 4:, lo:hi].float() - y32[:, 4:, lo:hi]).abs().max().item() <= 1e-2


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


def test_engine_fp16_with_own_conv3x3(golden_dir):
    """Every 3x3 convolution (stride 1 and 2, grouped head convolutions, ELAN slices) on the package's tcgen05
    implicit GEMM instead of the library: same relative-1e-2 bar against the fp32 oracle, bit-equal reruns."""
    import kadcnet
    from kadconv import ops
    g, sd = _sd(golden_dir)
    sd16 = {k: round_to(v, torch.float16) for k, v in sd.items()}
    img = seeding.seeded_input((2, 3, 160, 192), seed=5, kind='image')
    x = round_to(img.float() / 255, torch.float16)
    ref, _ = ko.detector(sd16, x)
    fast = kadcnet.load_model(None, 'optimized', 'cuda:0', state_dict=sd16, dtype=torch.float16, conv3x3='tcgen05')
    y, _ = fast(x.cuda().half())
    y2, _ = fast(x.cuda().half())
    torch.cuda.synchronize()
    ops.check_status(torch.device('cuda', 0))
    assert torch.equal(y, y2)
    assert rel_err(y[:, :4].float().cpu(), ref[:, :4]) <= 1e-2
    assert rel_err(y[:, 4:].float().cpu(), ref[:, 4:]) <= 1e-2


@pytest.mark.parametrize('dtype', [torch.float32, torch.float16])
def test_batched_nms_kernel_matches_oracle(golden_dir, dtype):
    """kad_nms_batched against the oracle's greedy NMS on the same prediction tensor (bit-equal boxes and order)."""
    from kadcnet.postprocess import non_max_suppression_device
    g = np.load(golden_dir / 'detector_s.npz')
    y = torch.from_numpy(g['y'])
    rng = np.random.default_rng(0)
    # a batch of three: the fixture, a jittered copy, and one with few candidates
    y2 = y.clone(); y2[:, :4] += torch.from_numpy(rng.normal(0, 3.0, y[:, :4].shape).astype(np.float32))
    y3 = y.clone(); y3[:, 4:] *= 0.0015
    pred = torch.cat((y, y2, y3), 0).to(dtype)
    ref = ko.non_max_suppression(pred.float() if dtype == torch.float32 else pred, 0.001, 0.65, max_det=300)
    out = non_max_suppression_device(pred.cuda(), 0.001, 0.65, max_det=300)
    for r, o in zip(ref, out):
        assert o.shape[0] == r.shape[0]
        assert torch.equal(o.cpu(), r.float())
    assert out[2].shape[0] < out[0].shape[0]
    # max_det cap and the fixture's own detections
    capped = non_max_suppression_device(pred.cuda(), 0.001, 0.65, max_det=7)
    assert all(c.shape[0] == min(7, r.shape[0]) and torch.equal(c.cpu(), r[:7].float()) for c, r in zip(capped, ref))
    if dtype == torch.float32:
        assert torch.equal(out[0].cpu(), torch.from_numpy(g['det']))


def test_engine_uint8_input_equals_float_input(golden_dir):
    """The uint8 entry (first layer on the raw image in one kernel: /255, 3x3 stride-2 convolution, bias, SiLU, NHWC) agrees
    with feeding the normalised float image through the library convolution, and with the float32 reference model."""
    import kadcnet
    g, sd = _sd(golden_dir)
    fast = kadcnet.load_model(None, 'optimized', 'cuda:0', state_dict=sd, dtype=torch.float16)
    assert fast.stem is not None
    img = seeding.seeded_input((2, 3, 160, 192), seed=9, kind='image').cuda()
    y8, _ = fast(img)
    yf, _ = fast((img.float() / 255).half())
    assert y8.shape == yf.shape
    assert rel_err(y8.float(), yf.float()) <= 1e-2
    raw = kadcnet.load_model(None, 'raw', 'cuda:0', state_dict=sd)
    with torch.no_grad():
        yr = raw(img.float() / 255)[0]
    assert rel_err(y8.float(), yr.float()) <= 1e-2 and rel_err(yf.float(), yr.float()) <= 1e-2


def test_engine_at_the_full_benchmark_size(golden_dir):
    """800x800 (the size bench.py runs, too large for the CPU oracle in a test): the fp16 engine on raw uint8 images
    against the plain fp32 modules executed on the GPU (library kernels only), and the batched NMS kernel against the
    reference-order NMS on the same predictions. The graph backend replays the same result."""
    import kadcnet
    from kadcnet.postprocess import non_max_suppression, non_max_suppression_device
    from kadconv import ops
    sd = _sd_alive(golden_dir)
    img = seeding.seeded_input((2, 3, 800, 800), seed=21, kind='image').cuda()
    raw = kadcnet.load_model(None, 'raw', 'cuda:0', state_dict=sd)
    with torch.no_grad():
        ref = raw(img.float() / 255)[0].float()
    fast = kadcnet.load_model(None, 'optimized', 'cuda:0', state_dict=sd, dtype=torch.float16)
    y, _ = fast(img)
    torch.cuda.synchronize(); ops.check_status(img.device)
    assert y.shape == ref.shape == (2, 24, 13125)
    assert rel_err(y[:, :4].float(), ref[:, :4]) <= 1e-2          # boxes (pixels)
    assert rel_err(y[:, 4:].float(), ref[:, 4:]) <= 1e-2          # class scores
    for lo, hi in ((0, 10000), (10000, 12500), (12500, 13125)):   # each scale on its own, absolutely: <= 1 px (2 half-precision steps at 800)
        assert (y[:, :4, lo:hi].float() - ref[:, :4, lo:hi]).abs().max().item() <= 1.0
    graph = kadcnet.load_model(None, 'graph', 'cuda:0', state_dict=sd, dtype=torch.float16)
    yg, _ = graph(img)
    yg2, _ = graph(img)
    assert torch.equal(yg, yg2) and rel_err(yg.float(), y.float()) <= 1e-3
    # the batched NMS kernel at the configuration's thresholds: exactly the boxes, scores, classes and order of the reference-order NMS
    dets = non_max_suppression_device(y, 0.001, 0.65, max_det=300)
    dets_ref = non_max_suppression(y, 0.001, 0.65, max_det=300)
    for d, r in zip(dets, dets_ref):
        assert d.shape == r.shape and torch.equal(d.cpu(), r.cpu().float())


def test_own_conv3x3_at_the_full_benchmark_size(golden_dir):
    """800x800: the engine with every 3x3 convolution on the package's tcgen05 kernel (maps 400x400 ... 25x25, odd
    199 / 99 / 49 inputs of the stride-2 layers) against the plain fp32 modules on the GPU, same bars as the default engine."""
    import kadcnet
    from kadconv import ops
    sd = _sd_alive(golden_dir)
    img = seeding.seeded_input((2, 3, 800, 800), seed=21, kind='image').cuda()
    raw = kadcnet.load_model(None, 'raw', 'cuda:0', state_dict=sd)
    with torch.no_grad():
        ref = raw(img.float() / 255)[0].float()
    fast = kadcnet.load_model(None, 'optimized', 'cuda:0', state_dict=sd, dtype=torch.float16, conv3x3='tcgen05')
    y, _ = fast(img)
    y2, _ = fast(img)
    torch.cuda.synchronize(); ops.check_status(img.device)
    assert torch.equal(y, y2)
    assert rel_err(y[:, :4].float(), ref[:, :4]) <= 1e-2
    assert rel_err(y[:, 4:].float(), ref[:, 4:]) <= 1e-2


def test_streaming_pipeline_matches_direct_calls(golden_dir):
    """DetectionPipeline (copies overlapped with the forward graph, padded detections + counts) returns, batch by batch and
    in order, what the direct call + non_max_suppression_device returns."""
    import kadcnet
    from kadcnet.postprocess import non_max_suppression_device
    g, sd = _sd(golden_dir)
    fast = kadcnet.load_model(None, 'optimized', 'cuda:0', state_dict=sd, dtype=torch.float16)
    batches = [seeding.seeded_input((2, 3, 160, 192), seed=30 + i, kind='image').pin_memory() for i in range(5)]
    pipe = kadcnet.DetectionPipeline(fast, (2, 3, 160, 192), 0.25, 0.65, 300)
    got = list(pipe.run(batches))
    assert len(got) == 5
    for b, dets in zip(batches, got):
        ref = non_max_suppression_device(fast(b.cuda())[0], 0.25, 0.65, max_det=300)
        assert len(dets) == 2
        for d, r in zip(dets, ref):
            assert not d.is_cuda and d.shape == r.shape and torch.equal(d, r.cpu())
    assert list(pipe.run([])) == []
    again = list(pipe.run(batches[:1]))
    assert all(torch.equal(a, b) for a, b in zip(again[0], got[0]))


def test_streaming_pipeline_with_two_graphs_side_by_side(golden_dir):
    """splits=2: the halves of every batch go through two CUDA graphs replayed on two streams at once; the detections equal
    those of the direct call on each half (same kernels on the same half-batch shape), batch by batch."""
    import kadcnet
    from kadcnet.postprocess import non_max_suppression_device
    g, sd = _sd(golden_dir)
    fast = kadcnet.load_model(None, 'optimized', 'cuda:0', state_dict=sd, dtype=torch.float16)
    batches = [seeding.seeded_input((4, 3, 160, 192), seed=40 + i, kind='image').pin_memory() for i in range(4)]
    pipe = kadcnet.DetectionPipeline(fast, (4, 3, 160, 192), 0.25, 0.65, 300, splits=2)
    got = list(pipe.run(batches))
    assert len(got) == 4
    for b, dets in zip(batches, got):
        y = torch.cat([fast(b[:2].cuda())[0], fast(b[2:].cuda())[0]], 0)
        ref = non_max_suppression_device(y, 0.25, 0.65, max_det=300)
        assert len(dets) == 4
        for d, r in zip(dets, ref):
            assert torch.equal(d, r.cpu())
    with pytest.raises(ValueError):
        kadcnet.DetectionPipeline(fast, (3, 3, 160, 192), splits=2)
