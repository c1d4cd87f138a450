"""Deformable convolution kernels (SIMT and tcgen05) against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from helpers import dcn_inputs, nhwc, rel_err, round_to
from oracle import kad_oracle as ko

pytestmark = pytest.mark.gpu


def _run(x, off, msk, w, b, dtype, path, act=0, scale=None, post=None, want_gap=False, off_dtype=torch.float32):
    from kadconv import ops
    dev = 'cuda'
    xg = nhwc(x).to(dev, dtype)
    og = None if off is None else nhwc(off).to(dev, off_dtype)
    mg = None if msk is None else nhwc(msk).to(dev, off_dtype)
    Cout, Cin = w.shape[:2]
    if path in (ops.PATH_TC, ops.PATH_TC_PAIR):
        wp = ops.pack_dsc_weight_tc(w.to(dev), dtype)
    else:
        wp = ops.pack_dsc_weight_simt(w.to(dev))
    shift = None if b is None else (b if scale is None else b * scale).to(dev)
    out = ops.dsc_forward(xg, wp, og, mg, scale=None if scale is None else scale.to(dev), shift=shift,
                          post=None if post is None else post.to(dev), act=act, path=path, want_gap=want_gap, cout=Cout)
    torch.cuda.synchronize()
    ops.check_status(xg.device)
    return out


@pytest.mark.parametrize('shape', [(2, 16, 24, 9, 12), (1, 22, 22, 25, 25), (2, 10, 10, 7, 5), (1, 44, 42, 13, 17),
                                   (1, 130, 140, 6, 9)])
def test_simt_fp32_matches_oracle(shape):
    B, Cin, Cout, H, W = shape
    x, off, msk, w, b = dcn_inputs(B, Cin, Cout, H, W, seed=sum(shape))
    ref = ko.deform_conv2d(x, off, w, b, msk)
    y = _run(x, off, msk, w, b, torch.float32, 0).cpu().permute(0, 3, 1, 2)
    assert (y - ref).abs().max().item() <= 1e-4


def test_simt_matches_torchvision_golden(golden_dir):
    g = np.load(golden_dir / 'dcn_op.npz')
    t = {k: torch.from_numpy(g[k]) for k in g.files}
    y = _run(t['x'], t['offset'], t['mask'], t['weight'], t['bias'], torch.float32, 0).cpu().permute(0, 3, 1, 2)
    assert (y - t['y']).abs().max().item() <= 1e-4


def test_simt_plain_conv_mode_and_epilogue():
    """offset = mask = NULL is an ordinary 3x3 convolution; scale/shift/ReLU/post are applied in order."""
    x, _, _, w, b = dcn_inputs(2, 12, 18, 11, 8, seed=5)
    g = np.random.default_rng(1)
    scale = torch.from_numpy(g.uniform(0.5, 1.5, 18).astype(np.float32))
    post = torch.from_numpy(g.standard_normal(18).astype(np.float32))
    ref = torch.nn.functional.conv2d(x, w, b, padding=1)
    y = _run(x, None, None, w, b, torch.float32, 0).cpu().permute(0, 3, 1, 2)
    assert (y - ref).abs().max().item() <= 1e-4
    ref2 = torch.relu(ref * scale.view(1, -1, 1, 1)) * post.view(1, -1, 1, 1)
    y2, gap = _run(x, None, None, w, b, torch.float32, 0, act=2, scale=scale, post=post, want_gap=True)
    assert (y2.cpu().permute(0, 3, 1, 2) - ref2).abs().max().item() <= 1e-4
    assert (gap.sum(1).cpu() - ref2.sum((2, 3))).abs().max().item() <= 1e-3


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_simt_16bit_matches_oracle(dtype):
    x, off, msk, w, b = dcn_inputs(2, 21, 21, 12, 10, seed=9)
    x, w = round_to(x, dtype), w
    ref = ko.deform_conv2d(x, off, w, b, msk)
    y = _run(x, off, msk, w, b, dtype, 0).float().cpu().permute(0, 3, 1, 2)
    assert rel_err(y, ref) <= 1e-2


@pytest.mark.parametrize('shape,dtype', [((2, 64, 64, 20, 25), torch.float16), ((1, 32, 48, 9, 7), torch.float16),
                                         ((2, 96, 256, 13, 30), torch.float16), ((1, 256, 256, 25, 50), torch.float16),
                                         ((1, 64, 32, 16, 16), torch.bfloat16), ((3, 128, 144, 10, 11), torch.bfloat16)])
def test_tc_matches_oracle(shape, dtype):
    """tcgen05 implicit GEMM: offsets N(0,2) px, so many samples leave the image and some leave the
    staged window (the slow path)."""
    B, Cin, Cout, H, W = shape
    x, off, msk, w, b = dcn_inputs(B, Cin, Cout, H, W, seed=sum(shape))
    x, w = round_to(x, dtype), round_to(w, dtype)
    ref = ko.deform_conv2d(x, off, w, b, msk)
    y = _run(x, off, msk, w, b, dtype, 1).float().cpu().permute(0, 3, 1, 2)
    assert rel_err(y, ref) <= 1e-2


def test_tc_large_offsets_and_epilogue():
    """Offsets N(0,6): most samples take the out-of-window path; fused scale/shift/ReLU/post and SE sums."""
    B, Cin, Cout, H, W = 2, 64, 64, 18, 21
    x, off, msk, w, b = dcn_inputs(B, Cin, Cout, H, W, seed=77, offset_std=6.0)
    dtype = torch.float16
    x, w = round_to(x, dtype), round_to(w, dtype)
    g = np.random.default_rng(2)
    scale = torch.from_numpy(g.uniform(0.5, 1.5, Cout).astype(np.float32))
    post = torch.from_numpy(g.uniform(0.5, 1.5, Cout).astype(np.float32))
    ref = torch.relu(ko.deform_conv2d(x, off, w, None, msk) * scale.view(1, -1, 1, 1) + (b * scale).view(1, -1, 1, 1)) * post.view(1, -1, 1, 1)
    y, gap = _run(x, off, msk, w, b, dtype, 1, act=2, scale=scale, post=post, want_gap=True)
    y = y.float().cpu().permute(0, 3, 1, 2)
    assert rel_err(y, ref) <= 1e-2
    assert rel_err(gap.sum(1).cpu(), y.sum((2, 3))) <= 1e-3      # sums of what was stored
    # 16-bit offsets and mask are accepted too
    y16 = _run(x, round_to(off, dtype), round_to(msk, dtype), w, b, dtype, 1, off_dtype=dtype).float().cpu().permute(0, 3, 1, 2)
    ref16 = ko.deform_conv2d(x, round_to(off, dtype), w, b, round_to(msk, dtype))
    assert rel_err(y16, ref16) <= 1e-2


def test_tc_is_deterministic():
    x, off, msk, w, b = dcn_inputs(2, 64, 64, 20, 25, seed=3)
    a = _run(x, off, msk, w, b, torch.float16, 1)
    c = _run(x, off, msk, w, b, torch.float16, 1)
    assert torch.equal(a, c)


def test_linearity_at_full_c1_size():
    """C1 size [16,256,100,100] fp16: too big for the CPU oracle in a test, so check a size-independent
    property (the operator is linear in the weights: y(W1+W2) = y(W1) + y(W2)) plus an oracle check of one
    image row block."""
    from kadconv import ops
    g = torch.Generator(device='cuda').manual_seed(0)
    B, C, H, W = 16, 256, 100, 100
    x = torch.randn((B, H, W, C), device='cuda', generator=g).half()
    off = 2.0 * torch.randn((B, H, W, 18), device='cuda', generator=g)
    msk = torch.sigmoid(torch.randn((B, H, W, 9), device='cuda', generator=g))
    w1 = ((torch.rand((C, C, 3, 3), device='cuda', generator=g) * 2 - 1) / 48).half().float()
    w2 = ((torch.rand((C, C, 3, 3), device='cuda', generator=g) * 2 - 1) / 48).half().float()
    w12 = (w1 + w2).half().float()
    ys = []
    for w in (w1, w2, w12):
        ys.append(ops.dsc_forward(x, ops.pack_dsc_weight_tc(w, torch.float16), off.half(), msk.half(), path=1, cout=C).float())
    torch.cuda.synchronize()
    ops.check_status(x.device)
    err = ((ys[0] + ys[1]) - ys[2]).abs().max() / ys[2].abs().max()
    assert err.item() <= 1e-2
    # oracle on image 3 (full image so that the sampling sees the true borders)
    xi = x[3:4].permute(0, 3, 1, 2).float().cpu()
    ref = ko.deform_conv2d(xi, off[3:4].half().float().permute(0, 3, 1, 2).cpu(), w1.cpu(), None,
                           msk[3:4].half().float().permute(0, 3, 1, 2).cpu())
    assert rel_err(ys[0][3:4].cpu().permute(0, 3, 1, 2), ref) <= 1e-2


@pytest.mark.parametrize('shape', [(2, 64, 64, 20, 25), (1, 96, 256, 13, 30), (3, 128, 96, 10, 11), (1, 32, 32, 19, 17)])
def test_tc_pair_kernel_matches_single(shape):
    """The CTA-pair variant (tcgen05 cta_group::2) gives bit-identical results to the one-CTA kernel,
    including an odd tile count (one CTA of the last pair has no tile)."""
    B, Cin, Cout, H, W = shape
    x, off, msk, w, b = dcn_inputs(B, Cin, Cout, H, W, seed=sum(shape) + 1)
    x, w = round_to(x, torch.float16), round_to(w, torch.float16)
    g = np.random.default_rng(4)
    scale = torch.from_numpy(g.uniform(0.5, 1.5, Cout).astype(np.float32))
    y1, g1 = _run(x, off, msk, w, b, torch.float16, 1, act=2, scale=scale, want_gap=True)
    y2, g2 = _run(x, off, msk, w, b, torch.float16, 2, act=2, scale=scale, want_gap=True)
    assert torch.equal(y1, y2) and torch.equal(g1, g2)
    ref = torch.relu(ko.deform_conv2d(x, off, w, None, msk) * scale.view(1, -1, 1, 1) + (b * scale).view(1, -1, 1, 1))
    assert rel_err(y2.float().cpu().permute(0, 3, 1, 2), ref) <= 1e-2


# ---- path 3: warp-level tensor-core kernel for small channel counts --------------------------------------------

@pytest.mark.parametrize('shape,dtype', [((2, 12, 12, 20, 25), torch.float16), ((1, 10, 10, 9, 7), torch.float16),
                                         ((2, 21, 21, 13, 30), torch.float16), ((1, 22, 22, 50, 50), torch.float16),
                                         ((1, 44, 43, 16, 16), torch.float16), ((2, 64, 64, 10, 11), torch.float16),
                                         ((1, 7, 5, 33, 9), torch.float16), ((2, 21, 21, 12, 10), torch.bfloat16),
                                         ((1, 32, 18, 17, 19), torch.bfloat16)])
def test_mma_matches_oracle(shape, dtype):
    """Odd channel counts (2-byte aligned pixels), partial 16-channel chunks, pixel counts that do not fill a warp."""
    from kadconv import ops
    B, Cin, Cout, H, W = shape
    x, off, msk, w, b = dcn_inputs(B, Cin, Cout, H, W, seed=sum(shape) + 3)
    x, w = round_to(x, dtype), round_to(w, dtype)
    ref = ko.deform_conv2d(x, off, w, b, msk)
    y = _run(x, off, msk, w, b, dtype, ops.PATH_MMA).float().cpu().permute(0, 3, 1, 2)
    assert rel_err(y, ref) <= 1e-2


def test_mma_plain_conv_mode_epilogue_and_large_offsets():
    from kadconv import ops
    dtype = torch.float16
    x, off, msk, w, b = dcn_inputs(2, 12, 18, 11, 8, seed=5, offset_std=6.0)
    x, w = round_to(x, dtype), round_to(w, dtype)
    g = np.random.default_rng(1)
    scale = torch.from_numpy(g.uniform(0.5, 1.5, 18).astype(np.float32))
    post = torch.from_numpy(g.uniform(0.5, 1.5, 18).astype(np.float32))
    # offset = mask = NULL: ordinary convolution, float32 output (the offset convolution's configuration)
    ref = torch.nn.functional.conv2d(x, w, b, padding=1)
    from kadconv import ops as _ops
    xg = nhwc(x).cuda().half()
    y = _ops.dsc_forward(xg, _ops.pack_dsc_weight_simt(w.cuda()), shift=b.cuda(), path=ops.PATH_MMA, y_f32=True)
    assert y.dtype == torch.float32
    assert rel_err(y.cpu().permute(0, 3, 1, 2), ref) <= 2e-3
    # deformable with offsets N(0,6) (most samples partly or fully outside), fused scale/shift/ReLU/post, SE sums
    ref2 = torch.relu(ko.deform_conv2d(x, off, w, None, msk) * scale.view(1, -1, 1, 1) + (b * scale).view(1, -1, 1, 1)) * post.view(1, -1, 1, 1)
    y2, gap = _run(x, off, msk, w, b, dtype, ops.PATH_MMA, act=2, scale=scale, post=post, want_gap=True)
    y2 = y2.float().cpu().permute(0, 3, 1, 2)
    assert rel_err(y2, ref2) <= 1e-2
    assert rel_err(gap.sum(1).cpu(), y2.sum((2, 3))) <= 1e-3
    a = _run(x, off, msk, w, b, dtype, ops.PATH_MMA)
    c = _run(x, off, msk, w, b, dtype, ops.PATH_MMA)
    assert torch.equal(a, c)


@pytest.mark.parametrize('shape,dtype', [((2, 12, 12, 20, 25), torch.float16), ((1, 21, 21, 31, 18), torch.float16),
                                         ((1, 44, 44, 12, 12), torch.float16), ((2, 10, 10, 9, 14), torch.bfloat16)])
def test_mma_fused_offset_convolution(shape, dtype):
    """With offset_weight the kernel computes offsets = conv3x3(x) + bias itself (DSC.forward, kad_conv.py:64-67)."""
    from kadconv import ops
    B, Cin, Cout, H, W = shape
    x, _, msk, w, b = dcn_inputs(B, Cin, Cout, H, W, seed=sum(shape) + 11)
    g = np.random.default_rng(sum(shape))
    w_off = round_to(torch.from_numpy((g.standard_normal((18, Cin, 3, 3)) * (1.5 / np.sqrt(9 * Cin))).astype(np.float32)), dtype)
    b_off = torch.from_numpy(g.standard_normal(18).astype(np.float32) * 0.5)
    x, w = round_to(x, dtype), round_to(w, dtype)
    off = torch.nn.functional.conv2d(x, w_off, b_off, padding=1)
    ref = ko.deform_conv2d(x, off, w, b, msk)
    xg = nhwc(x).cuda().to(dtype)
    mg = nhwc(msk).cuda()
    y, gap = ops.dsc_forward(xg, ops.pack_dsc_weight_simt(w.cuda()), None, mg, shift=b.cuda(), path=ops.PATH_MMA, want_gap=True,
                             offset_weight=ops.pack_dsc_weight_simt(w_off.cuda()), offset_bias=b_off.cuda())
    y = y.float().cpu().permute(0, 3, 1, 2)
    assert rel_err(y, ref) <= 1e-2
    assert rel_err(gap.sum(1).cpu(), y.sum((2, 3))) <= 1e-3
    # and it agrees with the two-kernel sequence on the same path
    offg = ops.dsc_forward(xg, ops.pack_dsc_weight_simt(w_off.cuda()), shift=b_off.cuda(), path=ops.PATH_MMA, y_f32=True)
    y2 = ops.dsc_forward(xg, ops.pack_dsc_weight_simt(w.cuda()), offg, mg, shift=b.cuda(), path=ops.PATH_MMA)
    assert rel_err(y2.float().cpu().permute(0, 3, 1, 2), y) <= 2e-3


@pytest.mark.parametrize('shape,dtype', [((1, 12, 12, 70, 20), torch.float16), ((2, 21, 22, 90, 33), torch.float16),
                                         ((1, 10, 10, 64, 50), torch.bfloat16)])
def test_mma_samples_outside_the_staged_rows(shape, dtype):
    """Tall images with offsets N(0, 8): many samples leave the rows staged in shared memory and are read from global
    memory (the per-tap slow variant), many leave the image."""
    from kadconv import ops
    B, Cin, Cout, H, W = shape
    x, off, msk, w, b = dcn_inputs(B, Cin, Cout, H, W, seed=sum(shape) + 5, offset_std=8.0)
    x, w = round_to(x, dtype), round_to(w, dtype)
    ref = ko.deform_conv2d(x, off, w, b, msk)
    y = _run(x, off, msk, w, b, dtype, ops.PATH_MMA).float().cpu().permute(0, 3, 1, 2)
    assert rel_err(y, ref) <= 1e-2


def test_mma_rejects_what_it_cannot_run():
    from kadconv import ops
    x = torch.zeros((1, 8, 8, 80), device='cuda', dtype=torch.float16)
    with pytest.raises(RuntimeError, match='warp-MMA'):
        ops.dsc_forward(x, torch.zeros((9, 80, 8), device='cuda'), path=ops.PATH_MMA)
    with pytest.raises(RuntimeError, match='warp-MMA'):
        ops.dsc_forward(x[..., :8].contiguous().float(), torch.zeros((9, 8, 8), device='cuda'), path=ops.PATH_MMA)
    # rows too long for shared memory
    assert not ops.dsc_mma_supported(64, 64, torch.float16, 8, 4000)
    assert ops.dsc_mma_supported(44, 44, torch.bfloat16, 200, 200)
    with pytest.raises(RuntimeError, match='warp-MMA'):
        ops.dsc_forward(torch.zeros((1, 4, 4000, 64), device='cuda', dtype=torch.float16), torch.zeros((9, 64, 64), device='cuda'), path=ops.PATH_MMA)
