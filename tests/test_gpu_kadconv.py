"""The KADConv module on the B200 pipeline against the CPU oracle and the reference-made fixtures."""
import numpy as np
import pytest
import torch

from helpers import kadconv_shapes, rel_err, round_to
from oracle import kad_oracle as ko
from oracle import seeding

pytestmark = pytest.mark.gpu


def _layer(dim, seed, dtype=torch.float32, scale_mode='uniform', se_min_hidden=32):
    import kadconv
    layer = kadconv.KADConv(dim, se_min_hidden=se_min_hidden).eval()
    sd = seeding.seeded_state_dict(kadconv_shapes(dim, se_min_hidden), seed=seed, scale_mode=scale_mode)
    if dtype != torch.float32:
        sd = {k: round_to(v, dtype) for k, v in sd.items()}
    layer.load_state_dict(sd)
    return layer, sd


@pytest.mark.parametrize('name', ['kadconv_c24', 'kadconv_c64'])
def test_fixture_fp32(golden_dir, name):
    import kadconv
    g = np.load(golden_dir / f'{name}.npz')
    dim, seed, shape = int(g['dim']), int(g['seed']), tuple(int(v) for v in g['shape'])
    layer, _ = _layer(dim, seed)
    x = seeding.seeded_input(shape, seed=seed)
    kadconv.enable_fast_inference(layer.cuda())
    with torch.no_grad():
        y = layer(x.cuda()).cpu()
    assert y.shape == x.shape
    assert (y - torch.from_numpy(g['y'])).abs().max().item() <= 1e-4


def test_c0_config_fp32():
    """configs[0]: KADConv(64), [2,64,80,80] fp32, max-abs 1e-4."""
    import kadconv
    layer, sd = _layer(64, 0)
    x = seeding.seeded_input((2, 64, 80, 80), seed=0)
    ref = ko.kadconv(sd, '', x)
    kadconv.enable_fast_inference(layer.cuda())
    with torch.no_grad():
        y = layer(x.cuda()).cpu()
        y_cl = layer(x.cuda().contiguous(memory_format=torch.channels_last)).cpu()
    assert (y - ref).abs().max().item() <= 1e-4
    assert (y_cl - ref).abs().max().item() <= 1e-4


@pytest.mark.parametrize('dim,shape', [(32, (1, 32, 25, 25)), (48, (2, 48, 12, 50)), (30, (1, 30, 9, 14)), (66, (1, 66, 6, 5))])
def test_odd_sizes_fp32(dim, shape):
    """Odd sizes (25 -> 12 -> 6 pyramid), H != W, widths that are no multiple of anything."""
    import kadconv
    layer, sd = _layer(dim, sum(shape))
    x = seeding.seeded_input(shape, seed=sum(shape))
    ref = ko.kadconv(sd, '', x)
    kadconv.enable_fast_inference(layer.cuda())
    with torch.no_grad():
        y = layer(x.cuda()).cpu()
    assert (y - ref).abs().max().item() <= 1e-4


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_16bit_relative(dtype):
    import kadconv
    layer, sd = _layer(48, 21, dtype=dtype)
    x = round_to(seeding.seeded_input((2, 48, 20, 28), seed=21), dtype)
    ref = ko.kadconv(sd, '', x)
    kadconv.enable_fast_inference(layer.cuda())
    with torch.no_grad():
        y = layer(x.cuda().to(dtype)).float().cpu()
    assert rel_err(y, ref) <= 1e-2


def test_16bit_many_images_column_strip_mask():
    """A batch large enough that the LCSA mask of the full-resolution branch runs as column strips (4 rows per
    thread, shared 11x1 window terms); H != W, the last strip of a column is ragged (52 = 6 * 8 + 4)."""
    import kadconv
    dtype = torch.float16
    layer, sd = _layer(32, 23, dtype=dtype)
    x = round_to(seeding.seeded_input((48, 32, 52, 50), seed=23), dtype)
    ref = ko.kadconv(sd, '', x)
    kadconv.enable_fast_inference(layer.cuda())
    with torch.no_grad():
        y = layer(x.cuda().to(dtype)).float().cpu()
    assert rel_err(y, ref) <= 1e-2


def test_wide_layer_uses_tensor_path_fp16():
    """KADConv(96): all three branches are 32 channels wide -> the DSCs run on tcgen05."""
    import kadconv
    from kadconv import ops
    dtype = torch.float16
    layer, sd = _layer(96, 5, dtype=dtype, se_min_hidden=64)
    x = round_to(seeding.seeded_input((2, 96, 24, 20), seed=5), dtype)
    ref = ko.kadconv(sd, '', x)
    kadconv.enable_fast_inference(layer.cuda())
    with torch.no_grad():
        y = layer(x.cuda().to(dtype)).float().cpu()
    ops.check_status(torch.device('cuda', 0))
    assert rel_err(y, ref) <= 1e-2


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
def test_c2_width_layer_16bit(dtype):
    """KADConv(128), the layer of configs[2] (bf16 there), with N(0,1) branch scales: branch widths 44 / 42 / 42, i.e. the
    warp-MMA deformable convolution with six 8-column accumulator tiles per warp and the pyramid kernel at the same width
    (the kernels the c2 benchmark times), against the fp32 oracle on values rounded to the storage type. H != W."""
    import kadconv
    from kadconv import ops
    layer, sd = _layer(128, 41, dtype=dtype, scale_mode='normal')
    x = round_to(seeding.seeded_input((2, 128, 40, 36), seed=41), dtype)
    ref = ko.kadconv(sd, '', x)
    kadconv.enable_fast_inference(layer.cuda())
    with torch.no_grad():
        y = layer(x.cuda().to(dtype))
        y2 = layer(x.cuda().to(dtype))
    ops.check_status(torch.device('cuda', 0))
    assert ops.dsc_mma_supported(44, 44, dtype, 40, 36) and ops.pyramid_project_supported(128, [44, 42, 42], dtype, 40, 36)
    assert torch.equal(y, y2)
    assert rel_err(y.float().cpu(), ref) <= 1e-2


def test_fast_mode_refuses_cpu_and_training():
    import kadconv
    layer, _ = _layer(24, 1)
    kadconv.enable_fast_inference(layer.cuda())
    with pytest.raises(RuntimeError):
        layer(torch.zeros(1, 24, 8, 8))
    layer.train()
    with pytest.raises(RuntimeError):
        layer(torch.zeros(1, 24, 8, 8, device='cuda'))
    layer.eval()
    kadconv.disable_fast_inference(layer)
    assert 'forward' not in vars(layer)


@pytest.mark.parametrize('dtype', [torch.float32, torch.float16])
def test_layer_call_matches_stepwise_kernels(dtype):
    """kad_kadconv_forward (one call, three streams, one workspace) is bit-identical to issuing the same kernels one
    by one on a single stream, also when called twice in a row and inside a CUDA graph."""
    import kadconv
    from kadconv import fast, ops
    layer, _ = _layer(48, 31, dtype=dtype)
    kadconv.enable_fast_inference(layer.cuda())
    x = round_to(seeding.seeded_input((3, 27, 22, 48), seed=31), dtype).cuda().to(dtype)     # NHWC
    ref = fast.kadconv_forward_nhwc_stepwise(layer, x)
    a = fast.kadconv_forward_nhwc(layer, x)
    b = fast.kadconv_forward_nhwc(layer, x)
    torch.cuda.synchronize()
    assert torch.equal(a, ref) and torch.equal(b, ref)
    # the ways the layer call can produce the LCSA masks (separate kernels; first stage finished in the pyramid kernel's tail; masks
    # evaluated inside the deformable convolutions; one launch for the three branches) give the same bits
    try:
        for scheme in (1, 2, 3, 4):
            fast.LAYER_SCHEME = scheme
            assert torch.equal(fast.kadconv_forward_nhwc(layer, x), ref), scheme
            assert torch.equal(fast.kadconv_forward_nhwc(layer, x), ref), scheme
    finally:
        fast.LAYER_SCHEME = 0
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fast.kadconv_forward_nhwc(layer, x)
    torch.cuda.current_stream().wait_stream(s)
    with torch.cuda.graph(g, stream=s):
        out = fast.kadconv_forward_nhwc(layer, x)
        out2 = fast.kadconv_forward_nhwc(layer, out)      # a second fork/join inside the same capture
    g.replay(); g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, ref)
    assert torch.equal(out2, fast.kadconv_forward_nhwc_stepwise(layer, ref))
    ops.check_status(x.device)


@pytest.mark.parametrize('dtype,dim', [(torch.float16, 32), (torch.bfloat16, 48)])
def test_first_call_equals_later_calls(dtype, dim):
    """The kernels of the layer are launched programmatically and read their parameters before they wait for the work in front of
    them. The very first call of a layer derives those parameters (folding, packing, conversions) on the same stream just before
    it launches: its result must be the one every later call gives, bit for bit, also when parameters change in between."""
    import kadconv
    for trial in range(3):
        layer, _ = _layer(dim, 50 + trial, dtype)
        layer = layer.cuda().to(dtype)
        kadconv.enable_fast_inference(layer)
        x = round_to(seeding.seeded_input((4, dim, 36, 44), seed=60 + trial), dtype).cuda().to(dtype)
        with torch.no_grad():
            first = layer(x).clone()
            again = layer(x).clone()
            assert torch.equal(first, again)
            for p in layer.parameters():                    # new parameters: the cached copies are rebuilt inside the next call
                p.mul_(1.01)
            changed = layer(x).clone()
            assert torch.equal(changed, layer(x)) and not torch.equal(changed, first)
