"""Smaller kernels against torch CPU references: layout, pooled projection, LCSA mask, SE, merge, 1x1 GEMM."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from helpers import nhwc, rel_err, round_to

pytestmark = pytest.mark.gpu


def _rand(shape, seed, scale=1.0):
    return torch.from_numpy((scale * np.random.default_rng(seed).standard_normal(shape)).astype(np.float32))


@pytest.mark.parametrize('dtype', [torch.float32, torch.float16])
def test_layout_round_trip(dtype):
    from kadconv import ops
    x = _rand((3, 37, 9, 21), 0).to(dtype).cuda()
    n = ops.to_nhwc(x)
    assert torch.equal(n, x.permute(0, 2, 3, 1).contiguous())
    assert torch.equal(ops.to_nchw(n), x)


@pytest.mark.parametrize('pool', [1, 2, 4])
def test_pool_project(pool):
    from kadconv import ops
    x = _rand((2, 45, 13, 18), 1)
    w = _rand((22, 45), 2, 0.2); b = _rand((22,), 3, 0.1)
    ref = F.conv2d(F.avg_pool2d(x, pool) if pool > 1 else x, w.view(22, 45, 1, 1), b)
    y = ops.pool_project(nhwc(x).cuda(), w.cuda(), b.cuda(), pool=pool).cpu().permute(0, 3, 1, 2)
    assert (y - ref).abs().max().item() <= 1e-5
    ys = ops.pool_project(nhwc(x).cuda(), w.cuda(), b.cuda(), pool=pool, act=ops.ACT_SILU).cpu().permute(0, 3, 1, 2)
    assert (ys - F.silu(ref)).abs().max().item() <= 1e-5


def test_pool_project_wide_and_sliced():
    from kadconv import ops
    x = _rand((1, 300, 5, 7), 4)
    w = _rand((150, 200), 5, 0.1)
    ref = F.conv2d(x[:, :200], w.view(150, 200, 1, 1))
    out = torch.zeros((1, 5, 7, 160), device='cuda')
    ops.pool_project(nhwc(x).cuda(), w.cuda(), None, cin=200, out=out, out_coff=8)
    assert (out[..., 8:158].cpu().permute(0, 3, 1, 2) - ref).abs().max().item() <= 1e-4
    assert out[..., :8].abs().max().item() == 0 and out[..., 158:].abs().max().item() == 0


def test_lcsa_mask_matches_module():
    import kadconv
    from kadconv import ops
    from kadconv.fast import _bn_fold
    torch.manual_seed(0)
    m = kadconv.LCSA(21, 9).eval()
    bn = m.excite[1]
    bn.running_mean.normal_(0, 0.2); bn.running_var.uniform_(0.5, 1.5); bn.weight.data.uniform_(0.5, 1.5); bn.bias.data.normal_(0, 0.1)
    x = _rand((2, 21, 14, 9), 6)
    with torch.no_grad():
        ref = torch.sigmoid(m(x))
    ex = m.excite
    bm, ba = _bn_fold(bn)
    f = lambda t: t.detach().float().contiguous().cuda()
    prm = dict(w1=f(ex[0].weight.view(21, 11)), b1=f(ex[0].bias), bn_m=f(bm), bn_a=f(ba), w2=f(ex[3].weight.view(21, 11)),
               b2=f(ex[3].bias), w3=f(ex[4].weight.view(9, 21)), b3=f(ex[4].bias))
    y = ops.lcsa_mask(nhwc(x).cuda(), prm).cpu().permute(0, 3, 1, 2)
    assert (y - ref).abs().max().item() <= 1e-5


def test_se_squeeze_excite_rescale():
    from kadconv import ops
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        x = round_to(_rand((2, 64, 21, 17), 7), dtype)
        w1 = _rand((16, 64), 8, 0.2); b1 = _rand((16,), 9, 0.1); w2 = _rand((64, 16), 10, 0.2); b2 = _rand((64,), 11, 0.1)
        a = torch.sigmoid(F.linear(F.relu(F.linear(x.mean((2, 3)), w1, b1)), w2, b2))
        ref = x * a.view(2, 64, 1, 1)
        xg = nhwc(x).cuda().to(dtype)
        gap = ops.se_squeeze(xg)
        att = ops.se_excite(gap, 21 * 17, w1.cuda(), b1.cuda(), w2.cuda(), b2.cuda())
        y = ops.se_rescale(xg, att).float().cpu().permute(0, 3, 1, 2)
        assert (att.cpu() - a).abs().max().item() <= 1e-5
        assert rel_err(y, ref) <= tol


def test_merge_upsample_residual():
    from kadconv import ops
    B, H, W = 2, 25, 18
    cs = (22, 21, 21)
    x = _rand((B, 64, H, W), 12)
    ys = [_rand((B, c, H // (2 ** i), W // (2 ** i)), 13 + i) for i, c in enumerate(cs)]
    atts = [torch.sigmoid(_rand((B, c), 20 + i)) for i, c in enumerate(cs)]
    feats = []
    for i in range(3):
        t = ys[i] * atts[i].view(B, -1, 1, 1)
        if i:
            t = F.interpolate(t, size=(H, W), mode='bilinear', align_corners=False)
        feats.append(t)
    ref = torch.cat(feats, 1) + x
    out = ops.merge_upsample_residual(nhwc(x).cuda(), [nhwc(t).cuda() for t in ys], [a.cuda() for a in atts])
    assert (out.cpu().permute(0, 3, 1, 2) - ref).abs().max().item() <= 1e-5


@pytest.mark.parametrize('dim,dtype', [(32, torch.float16), (64, torch.float16), (16, torch.bfloat16), (128, torch.bfloat16)])
def test_merge_vectorised_with_attention_inside(dim, dtype):
    """16-bit, C % 8 == 0: the kernel that owns 8-channel vectors. The squeeze-excite MLP evaluated inside the kernel
    gives bit-identical results to kad_se_excite + a merge with given attentions; out may be a channel slice."""
    from kadconv import ops
    B, H, W = 3, 26, 19
    cs = (dim - 2 * (dim // 3), dim // 3, dim // 3)
    x = round_to(_rand((B, dim, H, W), 12), dtype)
    ys = [round_to(_rand((B, c, H >> i, W >> i), 13 + i), dtype) for i, c in enumerate(cs)]
    tiles = (5, 3, 2)
    gaps = [_rand((B, tiles[i], c), 40 + i, 30.0) for i, c in enumerate(cs)]
    hid = [max(c // 4, 2) for c in cs]
    fcs = [(_rand((hid[i], c), 50 + i, 0.3), _rand((hid[i],), 54 + i, 0.1), _rand((c, hid[i]), 58 + i, 0.3), _rand((c,), 62 + i, 0.1)) for i, c in enumerate(cs)]
    atts, feats = [], []
    for i in range(3):
        mean = gaps[i].sum(1) / ((H >> i) * (W >> i))
        a = torch.sigmoid(F.linear(F.relu(F.linear(mean, fcs[i][0], fcs[i][1])), fcs[i][2], fcs[i][3]))
        atts.append(a)
        t = ys[i] * a.view(B, -1, 1, 1)
        if i:
            t = F.interpolate(t, size=(H, W), mode='bilinear', align_corners=False)
        feats.append(t)
    ref = torch.cat(feats, 1) + x
    xg = nhwc(x).cuda().to(dtype)
    yg = [nhwc(t).cuda().to(dtype) for t in ys]
    se = [(gaps[i].cuda(),) + tuple(t.cuda() for t in fcs[i]) for i in range(3)]
    out = ops.merge_upsample_residual(xg, yg, se=se)
    assert rel_err(out.float().cpu().permute(0, 3, 1, 2), ref) <= 1e-2
    att_dev = [ops.se_excite(se[i][0], (H >> i) * (W >> i), *se[i][1:]) for i in range(3)]
    for i in range(3):
        assert (att_dev[i].cpu() - atts[i]).abs().max().item() <= 1e-5
    out2 = ops.merge_upsample_residual(xg, yg, att_dev)
    assert torch.equal(out, out2)
    wide = torch.full((B, H, W, 2 * dim + 8), 7.0, dtype=dtype, device='cuda')
    ops.merge_upsample_residual(xg, yg, se=se, out=wide, out_coff=8)
    assert torch.equal(wide[..., 8:8 + dim], out) and bool((wide[..., :8] == 7).all()) and bool((wide[..., 8 + dim:] == 7).all())


def test_merge_general_shapes_with_attention_arguments():
    """float32 / C % 8 != 0 take the general kernel; the attention arguments then run kad_se_excite into att[]."""
    from kadconv import ops
    B, H, W, dim = 2, 13, 9, 20
    cs = (8, 6, 6)
    x = _rand((B, dim, H, W), 12)
    ys = [_rand((B, c, H >> i, W >> i), 13 + i) for i, c in enumerate(cs)]
    gaps = [_rand((B, 2, c), 40 + i, 10.0) for i, c in enumerate(cs)]
    fcs = [(_rand((3, c), 50 + i, 0.3), _rand((3,), 54 + i, 0.1), _rand((c, 3), 58 + i, 0.3), _rand((c,), 62 + i, 0.1)) for i, c in enumerate(cs)]
    feats = []
    for i in range(3):
        a = torch.sigmoid(F.linear(F.relu(F.linear(gaps[i].sum(1) / ((H >> i) * (W >> i)), fcs[i][0], fcs[i][1])), fcs[i][2], fcs[i][3]))
        t = ys[i] * a.view(B, -1, 1, 1)
        feats.append(F.interpolate(t, size=(H, W), mode='bilinear', align_corners=False) if i else t)
    ref = torch.cat(feats, 1) + x
    se = [(gaps[i].cuda(),) + tuple(t.cuda() for t in fcs[i]) for i in range(3)]
    out = ops.merge_upsample_residual(nhwc(x).cuda(), [nhwc(t).cuda() for t in ys], se=se)
    assert (out.cpu().permute(0, 3, 1, 2) - ref).abs().max().item() <= 1e-5


@pytest.mark.parametrize('M,K,N,dtype', [(1000, 128, 256, torch.bfloat16), (333, 72, 64, torch.float16), (5000, 360, 128, torch.float16),
                                         (777, 512, 288, torch.float16), (129, 64, 32, torch.bfloat16), (4096, 96, 48, torch.float16)])
def test_gemm1x1_bias_silu(M, K, N, dtype):
    """Fused 1x1 GEMM + bias + SiLU on tcgen05 (detector shapes incl. K, N that are no multiple of 64)."""
    from kadconv import ops
    x = round_to(_rand((M, K), 30), dtype); w = round_to(_rand((N, K), 31, 1.0 / np.sqrt(K)), dtype); b = _rand((N,), 32, 0.1)
    ref = F.silu(x @ w.t() + b)
    y = ops.gemm1x1_bias_act(x.cuda().to(dtype).view(1, M, 1, K), w.cuda().to(dtype), b.cuda(), act=ops.ACT_SILU)
    torch.cuda.synchronize()
    ops.check_status(torch.device('cuda', 0))
    assert rel_err(y.float().cpu().view(M, N), ref) <= 1e-2


def test_gemm1x1_slices_in_place():
    """Reads a channel slice of a wider tensor and writes into a channel slice of the output (concat-free)."""
    from kadconv import ops
    dtype = torch.float16
    x = round_to(_rand((600, 160), 33), dtype); w = round_to(_rand((40, 64), 34, 0.125), dtype)
    ref = x[:, :64] @ w.t()
    out = torch.zeros((600, 96), dtype=dtype, device='cuda')
    ops.gemm1x1_bias_act(x.cuda().to(dtype), w.cuda().to(dtype), None, act=ops.ACT_NONE, k=64, out=out, out_coff=16)
    torch.cuda.synchronize()
    ops.check_status(torch.device('cuda', 0))
    assert rel_err(out[:, 16:56].float().cpu(), ref) <= 1e-2
    assert out[:, :16].abs().max().item() == 0 and out[:, 56:].abs().max().item() == 0


@pytest.mark.parametrize('B,Cin,Cout,H,W,stride,dtype', [
    (2, 64, 64, 25, 25, 1, torch.float16),        # one full-K chunk, 5x25 tiles
    (3, 144, 144, 20, 30, 1, torch.float16),      # three chunks per tap, the last one 16 wide; H != W
    (2, 40, 72, 26, 22, 2, torch.float16),        # stride 2, channel counts that are no multiple of 16
    (2, 72, 144, 19, 23, 2, torch.bfloat16),      # stride 2 on odd sizes (AConv after its 2x2 stride-1 pool)
    (1, 216, 288, 13, 9, 2, torch.float16),       # two output-channel tiles
    (2, 32, 32, 7, 131, 1, torch.bfloat16),       # a row wider than a tile
    (1, 8, 8, 1, 1, 1, torch.float16),            # smallest legal problem
])
def test_conv3x3_bias_silu(B, Cin, Cout, H, W, stride, dtype):
    """3x3 convolution + bias + SiLU on tcgen05 against torch's fp32 conv2d on pre-rounded values (relative 1e-2)."""
    from kadconv import ops
    x = round_to(_rand((B, Cin, H, W), 60), dtype); w = round_to(_rand((Cout, Cin, 3, 3), 61, 1.0 / np.sqrt(9 * Cin)), dtype)
    b = _rand((Cout,), 62, 0.1)
    ref = F.silu(F.conv2d(x, w, b, stride, 1))
    y = ops.conv3x3_bias_act(nhwc(x).cuda().to(dtype), ops.pack_conv3x3_weight(w, dtype).cuda(), b.cuda(), act=ops.ACT_SILU, stride=stride)
    torch.cuda.synchronize()
    ops.check_status(torch.device('cuda', 0))
    assert tuple(y.shape) == (B, ref.shape[2], ref.shape[3], Cout)
    assert rel_err(y.float().cpu().permute(0, 3, 1, 2), ref) <= 1e-2


def test_conv3x3_slices_and_groups():
    """Reads a channel slice, writes a channel slice (concat-free), and runs a grouped convolution as a dense one."""
    from kadconv import ops
    dtype = torch.float16
    x = round_to(_rand((2, 96, 11, 14), 63), dtype); w = round_to(_rand((64, 16, 3, 3), 64, 0.1), dtype)
    ref = F.conv2d(x[:, 32:96], w, None, 1, 1, 1, 4)
    out = torch.zeros((2, 11, 14, 80), dtype=dtype, device='cuda')
    ops.conv3x3_bias_act(nhwc(x).cuda().to(dtype), ops.pack_conv3x3_weight(w, dtype, groups=4).cuda(), None, act=ops.ACT_NONE,
                         in_coff=32, cin=64, out=out, out_coff=8)
    torch.cuda.synchronize()
    ops.check_status(torch.device('cuda', 0))
    assert rel_err(out[..., 8:72].float().cpu().permute(0, 3, 1, 2), ref) <= 1e-2
    assert out[..., :8].abs().max().item() == 0 and out[..., 72:].abs().max().item() == 0


def test_conv3x3_rejects_bad_arguments():
    from kadconv import ops
    x = torch.zeros((1, 4, 4, 12), dtype=torch.float16, device='cuda')
    with pytest.raises(RuntimeError):
        ops.conv3x3_bias_act(x, torch.zeros((8, 9, 12), dtype=torch.float16, device='cuda'))      # Cin % 8 != 0
    with pytest.raises(RuntimeError):
        ops.conv3x3_bias_act(x.float(), torch.zeros((8, 9, 12), dtype=torch.float32, device='cuda'))   # fp32 has no tensor path


@pytest.mark.parametrize('dtype,tol', [(torch.float32, 1e-5), (torch.float16, 2e-3)])
def test_head_decode(dtype, tol):
    """DFL expectation + dist2bbox + sigmoid in one kernel per scale against the reference's op sequence in fp32
    (KAD-CNet/models/yolo.py:112-127): three scales, non-square maps, anchors in (scale, y, x) order."""
    from kadconv import ops
    reg_max, nc, B = 16, 20, 3
    sizes, strides = [(20, 24), (10, 12), (5, 6)], [8.0, 16.0, 32.0]
    raws = [round_to(_rand((B, h, w, 4 * reg_max + nc), 70 + i, 2.0), dtype) for i, (h, w) in enumerate(sizes)]
    # reference sequence on [B, no, A]
    allr = torch.cat([r.reshape(B, -1, 4 * reg_max + nc) for r in raws], 1).transpose(1, 2)
    bx, cl = allr.split((4 * reg_max, nc), 1)
    A = bx.shape[2]
    d = (bx.reshape(B, 4, reg_max, A).softmax(2) * torch.arange(reg_max, dtype=torch.float32).view(1, 1, reg_max, 1)).sum(2)
    pts, st = [], []
    for (h, w), s in zip(sizes, strides):
        sy, sx = torch.meshgrid(torch.arange(h) + 0.5, torch.arange(w) + 0.5, indexing='ij')
        pts.append(torch.stack((sx, sy), -1).view(-1, 2)); st.append(torch.full((h * w, 1), s))
    anc, stv = torch.cat(pts).t().unsqueeze(0), torch.cat(st).t()
    lt, rb = d.split(2, 1)
    x1y1, x2y2 = anc - lt, anc + rb
    ref = torch.cat((torch.cat(((x1y1 + x2y2) / 2, x2y2 - x1y1), 1) * stv, cl.sigmoid()), 1)
    y = ops.head_decode([r.cuda().to(dtype) for r in raws], strides, reg_max, nc)
    assert tuple(y.shape) == (B, 4 + nc, A)
    assert rel_err(y[:, :4].float().cpu(), ref[:, :4]) <= tol
    assert rel_err(y[:, 4:].float().cpu(), ref[:, 4:]) <= tol


def test_avg_pool():
    from kadconv import ops
    for dtype in (torch.float32, torch.bfloat16):
        x = round_to(_rand((2, 24, 13, 18), 40), dtype)
        for pool in (2, 4):
            ref = F.avg_pool2d(x, pool)
            y = ops.avg_pool(nhwc(x).cuda().to(dtype), pool).float().cpu().permute(0, 3, 1, 2)
            assert rel_err(y, ref) <= (1e-6 if dtype == torch.float32 else 1e-2)


def test_detector_glue_kernels():
    from kadconv import ops
    for dtype in (torch.float32, torch.float16):
        x = round_to(_rand((2, 24, 9, 14), 50), dtype)
        ref = F.avg_pool2d(x, 2, 1, 0, False, True)
        y = ops.avg_pool2x2s1(nhwc(x).cuda().to(dtype)).float().cpu().permute(0, 3, 1, 2)
        assert rel_err(y, ref) <= (1e-6 if dtype == torch.float32 else 2e-3)
        t = round_to(_rand((5, 7, 16), 51), dtype); b = _rand((16,), 52, 0.3)
        out = ops.bias_act_(t.cuda().to(dtype).clone(), b.cuda(), ops.ACT_SILU).float().cpu()
        assert rel_err(out, F.silu(t + b)) <= (1e-5 if dtype == torch.float32 else 2e-3)
    img = torch.from_numpy(np.random.default_rng(3).integers(0, 256, (2, 3, 11, 13), dtype=np.uint8))
    y = ops.image_to_nhwc(img.cuda(), torch.float16, cpad=8).cpu()
    ref = (img.float() / 255).half().permute(0, 2, 3, 1)
    assert torch.equal(y[..., :3], ref) and y[..., 3:].abs().max().item() == 0


@pytest.mark.parametrize('shape,dtype', [((2, 3, 50, 70, 40), torch.float16), ((1, 3, 33, 47, 32), torch.bfloat16), ((2, 1, 16, 16, 8), torch.float16),
                                         ((1, 4, 21, 130, 64), torch.float16), ((70, 3, 150, 136, 40), torch.float16), ((3, 3, 37, 68, 16), torch.bfloat16)])
def test_stem_conv_on_uint8_images(shape, dtype):
    """uint8 planes -> /255 -> 3x3 stride-2 convolution + bias + SiLU -> NHWC, against torch in float32 (odd sizes, image
    borders, widths that do not fill the 32-pixel tiles; widths that are multiples of four take the word-staged path, and the
    batch of 70 gives every block several row tiles, the last of them partial)."""
    from kadconv import ops
    B, Cin, H, W, Cout = shape
    g = np.random.default_rng(sum(shape))
    img = torch.from_numpy(g.integers(0, 256, (B, Cin, H, W), dtype=np.uint8))
    w = round_to(_rand((Cout, Cin, 3, 3), 70, 1.0 / np.sqrt(9 * Cin)), dtype)
    b = _rand((Cout,), 71, 0.2)
    ref = F.silu(F.conv2d(img.float() / 255.0, w, b, stride=2, padding=1))
    y = ops.stem_conv_u8(img.cuda(), w.cuda(), b.cuda(), dtype)
    assert tuple(y.shape) == (B, ref.shape[2], ref.shape[3], Cout)
    assert rel_err(y.float().cpu().permute(0, 3, 1, 2), ref) <= (4e-3 if dtype == torch.float16 else 1e-2)
    y0 = ops.stem_conv_u8(img.cuda(), w.cuda(), None, dtype, act=ops.ACT_NONE, scale=1.0)
    ref0 = F.conv2d(img.float(), w, None, stride=2, padding=1)
    assert rel_err(y0.float().cpu().permute(0, 3, 1, 2), ref0) <= (2e-3 if dtype == torch.float16 else 1e-2)


@pytest.mark.parametrize('dtype,C1,C2', [(torch.float16, 16, 24), (torch.bfloat16, 216, 288), (torch.float32, 5, 3), (torch.float16, 7, 8)])
def test_upsample2x_concat(dtype, C1, C2):
    from kadconv import ops
    B, h, w = 2, 7, 5
    low = round_to(_rand((B, C1, h, w), 80), dtype); skip = round_to(_rand((B, C2, 2 * h, 2 * w), 81), dtype)
    ref = torch.cat((F.interpolate(low, scale_factor=2, mode='nearest'), skip), 1)
    out = ops.upsample2x_concat(nhwc(low).cuda().to(dtype), nhwc(skip).cuda().to(dtype))
    assert torch.equal(out.float().cpu().permute(0, 3, 1, 2), ref)


@pytest.mark.parametrize('dtype,C,act', [(torch.float16, 40, 1), (torch.bfloat16, 72, 2), (torch.float32, 9, 1), (torch.float16, 12, 0)])
def test_bias_act_into_a_channel_slice(dtype, C, act):
    from kadconv import ops
    y = round_to(_rand((3, 11, 13, C), 90, 2.0), dtype); b = _rand((C,), 91, 0.5)
    z = y + b
    ref = F.silu(z) if act == 1 else (F.relu(z) if act == 2 else z)
    wide = torch.full((3, 11, 13, C + 24), 3.0, dtype=dtype, device='cuda')
    ops.bias_act_to(y.cuda().to(dtype), b.cuda(), wide, 16, act)
    tol = 1e-5 if dtype == torch.float32 else (4e-3 if dtype == torch.float16 else 1e-2)
    assert rel_err(wide[..., 16:16 + C].float().cpu(), ref) <= tol
    assert bool((wide[..., :16] == 3).all()) and bool((wide[..., 16 + C:] == 3).all())
    inplace = ops.bias_act_(y.cuda().to(dtype).clone(), b.cuda(), act)
    assert torch.equal(inplace, wide[..., 16:16 + C])


@pytest.mark.parametrize('shape,dtype', [((2, 32, 26, 19), torch.float16), ((1, 64, 50, 50), torch.float16), ((2, 128, 12, 70), torch.bfloat16),
                                         ((1, 24, 9, 7), torch.float16), ((1, 72, 21, 33), torch.bfloat16), ((2, 16, 13, 203), torch.float16),
                                         ((1, 40, 6, 131), torch.bfloat16)])
def test_pyramid_projection(shape, dtype):
    """One kernel for the three pooled 1x1 projections of a KAD-Conv layer: odd sizes (floor-mode pooling drops the
    last rows / columns), widths with partial 16-channel chunks, several column tiles."""
    from kadconv import ops
    B, dim, H, W = shape
    cs = (dim - 2 * (dim // 3), dim // 3, dim // 3)
    x = round_to(_rand((B, dim, H, W), 100), dtype)
    ws = [round_to(_rand((c, dim), 101 + i, 1.0 / np.sqrt(dim)), dtype) for i, c in enumerate(cs)]
    bs = [_rand((c,), 105 + i, 0.1) for i, c in enumerate(cs)]
    assert ops.pyramid_project_supported(dim, cs, dtype, H, W)
    ts = ops.pyramid_project(nhwc(x).cuda().to(dtype), [w.cuda() for w in ws], [b.cuda() for b in bs])
    for i in range(3):
        pooled = round_to(F.avg_pool2d(x, 2 ** i), dtype) if i else x
        ref = F.conv2d(pooled, ws[i].view(cs[i], dim, 1, 1), bs[i])
        assert tuple(ts[i].shape) == (B, H >> i, W >> i, cs[i])
        assert rel_err(ts[i].float().cpu().permute(0, 3, 1, 2), ref) <= (2e-3 if dtype == torch.float16 else 1e-2)
    # agrees with the three single projections
    for i in range(3):
        single = ops.pool_project(nhwc(x).cuda().to(dtype), ws[i].cuda(), bs[i].cuda(), pool=2 ** i)
        assert rel_err(ts[i].float(), single.float()) <= (2e-3 if dtype == torch.float16 else 1e-2)


@pytest.mark.parametrize('shape,dtype', [((2, 32, 26, 19), torch.float16), ((1, 64, 50, 50), torch.float16), ((2, 128, 12, 70), torch.bfloat16),
                                         ((3, 64, 7, 5), torch.float16), ((2, 16, 13, 203), torch.float16), ((1, 40, 22, 131), torch.bfloat16)])
def test_lcsa_mask_from_pyramid_partial_sums(shape, dtype):
    """The row / column sums the pyramid kernel emits as by-products give the same LCSA mask as summing the branch
    tensors in a second pass (kad_lcsa_sums + kad_lcsa_mask), also on maps narrower than a block."""
    from kadconv import ops
    B, dim, H, W = shape
    cs = (dim - 2 * (dim // 3), dim // 3, dim // 3)
    x = round_to(_rand((B, dim, H, W), 110), dtype)
    ws = [_rand((c, dim), 111 + i, 1.0 / np.sqrt(dim)) for i, c in enumerate(cs)]
    bs = [_rand((c,), 115 + i, 0.1) for i, c in enumerate(cs)]
    ts, parts = ops.pyramid_project(nhwc(x).cuda().to(dtype), [w.cuda() for w in ws], [b.cuda() for b in bs], want_partials=True)
    for i, c in enumerate(cs):
        t = ts[i]
        assert rel_err(parts[i][0].sum(2).cpu(), t.float().sum(2).cpu()) <= 1e-5
        assert rel_err(parts[i][1].sum(1).cpu(), t.float().sum(1).cpu()) <= 1e-5
        f = lambda a: a.cuda()
        prm = dict(w1=f(_rand((c, 11), 120 + i, 0.3)), b1=f(_rand((c,), 123 + i, 0.1)), bn_m=f(1.0 + _rand((c,), 126 + i, 0.1)), bn_a=f(_rand((c,), 129 + i, 0.1)),
                   w2=f(_rand((c, 11), 132 + i, 0.3)), b2=f(_rand((c,), 135 + i, 0.1)), w3=f(_rand((9, c), 138 + i, 0.3)), b3=f(_rand((9,), 141 + i, 0.1)))
        assert ops.lcsa_mask_from_partials_supported(t.shape[1], t.shape[2], c)
        m1 = ops.lcsa_mask_from_partials(parts[i][0], parts[i][1], prm, dtype, mask_f32=True)
        m0 = ops.lcsa_mask(t, prm, mask_f32=True)
        assert (m1 - m0).abs().max().item() <= 2e-5


@pytest.mark.parametrize('shape,dtype', [((2, 32, 26, 19), torch.float16), ((3, 64, 50, 50), torch.float16), ((2, 128, 14, 28), torch.bfloat16),
                                         ((5, 48, 9, 30), torch.float16)])
def test_inline_lcsa_mask_equals_mask_tensor(shape, dtype):
    """The five-launch form of a KAD-Conv branch (LCSA first stage finished in the pyramid kernel's tail by the last block of each
    image, mask evaluated inside the deformable convolution by the lane that owns the pixel) against the step-by-step form
    (partial sums -> preparation kernel -> mask kernel -> mask tensor -> deformable convolution): same arithmetic in the same
    order, so outputs and channel sums are bit-identical; also on the second call (the block counters reset themselves),
    on image borders (rows nearer than 5 to the edge) and on maps where a group of 256 pixels spans many rows."""
    from kadconv import ops
    B, dim, H, W = shape
    cs = (dim - 2 * (dim // 3), dim // 3, dim // 3)
    f = lambda a: a.cuda()
    x = nhwc(round_to(_rand((B, dim, H, W), 210), dtype)).cuda().to(dtype)
    ws = [f(_rand((c, dim), 211 + i, 1.0 / np.sqrt(dim))) for i, c in enumerate(cs)]
    bs = [f(_rand((c,), 215 + i, 0.1)) for i, c in enumerate(cs)]
    prms = [dict(w1=f(_rand((c, 11), 220 + i, 0.3)), b1=f(_rand((c,), 223 + i, 0.1)), bn_m=f(1.0 + _rand((c,), 226 + i, 0.1)), bn_a=f(_rand((c,), 229 + i, 0.1)),
                 w2=f(_rand((c, 11), 232 + i, 0.3)), b2=f(_rand((c,), 235 + i, 0.1)), w3=f(_rand((9, c), 238 + i, 0.3)), b3=f(_rand((9,), 241 + i, 0.1)))
            for i, c in enumerate(cs)]
    assert ops.pyramid_lcsa_supported(dim, cs, dtype, H, W)
    # (declined where the staged kernel behind the tail variant would tile the columns differently from kad_pyramid_project)
    assert not ops.pyramid_lcsa_supported(128, (44, 42, 42), torch.bfloat16, 12, 70)
    ts0, parts = ops.pyramid_project(x, ws, bs, want_partials=True)
    for rep in range(2):
        ts1, lops = ops.pyramid_project_lcsa(x, ws, bs, prms)
        for i, c in enumerate(cs):
            h, w = H >> i, W >> i
            assert torch.equal(ts1[i], ts0[i])
            assert rel_err(lops[i]['rowmean'].cpu(), ts0[i].float().mean(2).cpu()) <= 1e-5
            if not ops.dsc_mma_inline_mask_supported(c, c, dtype, h, w):
                continue
            wd = ops.pack_dsc_weight_simt(f(_rand((c, c, 3, 3), 250 + i, 1.0 / np.sqrt(9 * c))))
            wo = ops.pack_dsc_weight_simt(f(_rand((18, c, 3, 3), 260 + i, 0.6 / np.sqrt(9 * c))))
            bo = f(_rand((18,), 270 + i, 0.2))
            mask = ops.lcsa_mask_from_partials(parts[i][0], parts[i][1], prms[i], dtype, mask_f32=True)
            y0, g0 = ops.dsc_forward(ts0[i], wd, None, mask, act=ops.ACT_RELU, path=ops.PATH_MMA, want_gap=True, offset_weight=wo, offset_bias=bo)
            inl = dict(lops[i], w2=prms[i]['w2'], b2=prms[i]['b2'], w3=prms[i]['w3'], b3=prms[i]['b3'])
            y1, g1 = ops.dsc_forward(ts1[i], wd, None, None, act=ops.ACT_RELU, path=ops.PATH_MMA, want_gap=True, offset_weight=wo, offset_bias=bo,
                                     lcsa_inline=inl)
            torch.cuda.synchronize()
            assert torch.equal(y1, y0) and torch.equal(g1, g0)
    assert int(ops.layer_counters(x.device).abs().sum()) == 0


@pytest.mark.parametrize('shape,dtype', [((3, 25, 25, 144), torch.float16), ((2, 7, 5, 16), torch.bfloat16), ((1, 50, 40, 8), torch.float16), ((2, 3, 9, 24), torch.float16)])
def test_spp_pooling_chain_in_place(shape, dtype):
    """kad_spp_pool3: the three chained 5x5 max-pools of SPPELAN written into the channel quarters of the concatenation, against
    torch's max_pool2d + cat (exact: a maximum has no rounding), on maps smaller than the window too."""
    import torch.nn.functional as F
    from kadconv import ops
    B, H, W, C = shape
    y1 = _rand((B, C, H, W), 300).to(dtype)
    ys = [y1]
    for _ in range(3):
        ys.append(F.max_pool2d(ys[-1].float(), 5, 1, 2).to(dtype))
    ref = torch.cat([nhwc(t) for t in ys], -1)
    assert ops.spp_pool3_supported(H, W, C, dtype)
    cat = torch.full((B, H, W, 4 * C), float('nan'), dtype=dtype).cuda()
    cat[..., :C] = nhwc(y1).cuda()
    out = ops.spp_pool3_(cat, C)
    assert torch.equal(out.cpu(), ref)
    assert not ops.spp_pool3_supported(100, 100, 144, dtype) and not ops.spp_pool3_supported(25, 25, 12, dtype)


@pytest.mark.parametrize('shape,dtype', [((2, 32, 26, 19), torch.float16), ((3, 64, 50, 50), torch.float16), ((2, 48, 100, 100), torch.float16),
                                         ((5, 48, 9, 30), torch.bfloat16), ((2, 64, 25, 25), torch.float16)])
def test_three_lcsa_masks_in_one_launch(shape, dtype):
    """kad_lcsa_masks3_from_partials (first stage recomputed per block in shared memory, column strips) gives the bits of the
    per-branch preparation + mask kernels, on maps where those run as strips and where they run one pixel per thread."""
    from kadconv import ops
    B, dim, H, W = shape
    cs = (dim - 2 * (dim // 3), dim // 3, dim // 3)
    f = lambda a: a.cuda()
    x = nhwc(round_to(_rand((B, dim, H, W), 410), dtype)).cuda().to(dtype)
    ws = [f(_rand((c, dim), 411 + i, 1.0 / np.sqrt(dim))) for i, c in enumerate(cs)]
    bs = [f(_rand((c,), 415 + i, 0.1)) for i, c in enumerate(cs)]
    prms = [dict(w1=f(_rand((c, 11), 420 + i, 0.3)), b1=f(_rand((c,), 423 + i, 0.1)), bn_m=f(1.0 + _rand((c,), 426 + i, 0.1)), bn_a=f(_rand((c,), 429 + i, 0.1)),
                 w2=f(_rand((c, 11), 432 + i, 0.3)), b2=f(_rand((c,), 435 + i, 0.1)), w3=f(_rand((9, c), 438 + i, 0.3)), b3=f(_rand((9,), 441 + i, 0.1)))
            for i, c in enumerate(cs)]
    ts, parts = ops.pyramid_project(x, ws, bs, want_partials=True)
    assert ops.lcsa_masks3_supported(H, W, cs)
    masks = ops.lcsa_masks3_from_partials(parts, prms, dtype, H, W)
    for i in range(3):
        ref = ops.lcsa_mask_from_partials(parts[i][0], parts[i][1], prms[i], dtype, mask_f32=True)
        assert torch.equal(masks[i], ref), i
    assert not ops.lcsa_masks3_supported(200, 200, (44, 42, 42))


@pytest.mark.parametrize('dtype', [torch.float16, torch.float32])
@pytest.mark.parametrize('case', [(32, 16, 16, 16, 48, 32), (30, 7, 5, 22, 40, 11), (24, 8, 12, 12, 12, 0), (9, 3, 3, 9, 10, 1)])
def test_copy_channels_moves_exactly_the_slice(dtype, case):
    """kad_copy_channels against tensor slicing, with every vector width (16, 8, 4, 2 bytes) and an untouched remainder."""
    from kadconv import ops
    cs, soff, C, _, cd, doff = case
    g = torch.Generator().manual_seed(5)
    src = torch.randn((3, 17, 13, cs), generator=g).to(dtype).cuda()
    dst = torch.randn((3, 17, 13, cd), generator=g).to(dtype).cuda()
    want = dst.clone(); want[..., doff:doff + C] = src[..., soff:soff + C]
    got = ops.copy_channels(src, soff, C, dst, doff)
    assert got is dst and torch.equal(dst, want)
    dense = ops.copy_channels(src, soff, C)
    assert dense.is_contiguous() and torch.equal(dense, src[..., soff:soff + C])
    with pytest.raises(ValueError):
        ops.copy_channels(src, cs - C + 1, C)


@pytest.mark.parametrize('dtype,cin,cout,shape', [(torch.float16, 12, 12, (3, 30, 41)), (torch.bfloat16, 21, 21, (2, 9, 7)), (torch.float16, 16, 16, (2, 50, 50)),
                                                   (torch.float16, 44, 44, (1, 20, 24))])
def test_packed_mma_fragments_equal_in_kernel_staging(dtype, cin, cout, shape):
    """kad_dsc_mma_pack_frags writes, once, the weight fragments every block of the warp-MMA kernel would derive from the two
    float32 weights; a launch that copies them gives the same bits as one that derives them."""
    from kadconv import ops
    B, H, W = shape
    f = lambda a: a.cuda()
    x = nhwc(round_to(_rand((B, cin, H, W), 400), dtype)).cuda().to(dtype)
    wd = ops.pack_dsc_weight_simt(f(_rand((cout, cin, 3, 3), 401, 1.0 / np.sqrt(9 * cin))))
    wo = ops.pack_dsc_weight_simt(f(_rand((18, cin, 3, 3), 402, 0.6 / np.sqrt(9 * cin))))
    bo = f(_rand((18,), 403, 0.2))
    mask = torch.sigmoid(f(_rand((B, H, W, 9), 404)))
    assert ops.dsc_mma_supported(cin, cout, dtype, H, W)
    frags = ops.pack_dsc_mma_frags(wd, wo, dtype)
    y0, g0 = ops.dsc_forward(x, wd, None, mask, act=ops.ACT_RELU, path=ops.PATH_MMA, want_gap=True, offset_weight=wo, offset_bias=bo)
    y1, g1 = ops.dsc_forward(x, wd, None, mask, act=ops.ACT_RELU, path=ops.PATH_MMA, want_gap=True, offset_weight=wo, offset_bias=bo, mma_frags=frags)
    torch.cuda.synchronize()
    assert torch.equal(y1, y0) and torch.equal(g1, g0)
    with pytest.raises(ValueError):
        ops.dsc_forward(x, wd, None, mask, path=ops.PATH_MMA, offset_weight=wo, offset_bias=bo, mma_frags=frags[:-16])
