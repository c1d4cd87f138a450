"""Operator-level wrappers: torch tensors in, C-ABI calls on the current CUDA stream, torch tensors out.

Activations are NHWC here: a tensor of shape [B, H, W, C] that is contiguous. PyTorch only provides
device memory, the stream and the caching allocator (so the calls stay CUDA-graph capturable).
"""
import ctypes

import torch

from . import _abi
from ._abi import ACT_NONE, ACT_RELU, ACT_SILU, KAD_BF16, KAD_F16, KAD_F32, PATH_MMA, PATH_SIMT, PATH_TC, PATH_TC_PAIR

_DT = {torch.float32: KAD_F32, torch.float16: KAD_F16, torch.bfloat16: KAD_BF16}


def dtype_code(t):
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f'kadconv supports float32, float16 and bfloat16 activations, got {t.dtype}') from None


def _cuda(t, name):
    if not t.is_cuda:
        raise RuntimeError(f'kadconv: {name} must be a CUDA tensor (there is no CPU path)')
    if not t.is_contiguous():
        raise RuntimeError(f'kadconv: {name} must be contiguous')
    return t


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _f32(t, name):
    if t is None:
        return None
    if t.dtype != torch.float32:
        raise TypeError(f'kadconv: {name} must be float32')
    return _cuda(t, name)


def to_nhwc(x):
    """[B,C,H,W] logical tensor -> contiguous [B,H,W,C]; free when x is already channels_last."""
    if x.dim() != 4:
        raise ValueError('expected a 4-D tensor')
    v = x.permute(0, 2, 3, 1)
    if v.is_contiguous():
        return v
    x = _cuda(x.contiguous(), 'x')
    B, C, H, W = x.shape
    out = torch.empty((B, H, W, C), dtype=x.dtype, device=x.device)
    _abi.check(_abi.load().kad_nchw_to_nhwc(_ptr(x), _ptr(out), B, C, H, W, dtype_code(x), _stream()), 'kad_nchw_to_nhwc')
    return out


def to_nchw(y):
    """Contiguous [B,H,W,C] -> contiguous [B,C,H,W]."""
    y = _cuda(y, 'y')
    B, H, W, C = y.shape
    out = torch.empty((B, C, H, W), dtype=y.dtype, device=y.device)
    _abi.check(_abi.load().kad_nhwc_to_nchw(_ptr(y), _ptr(out), B, C, H, W, dtype_code(y), _stream()), 'kad_nhwc_to_nchw')
    return out


def pack_dsc_weight_simt(w):
    """[Cout,Cin,3,3] -> float32 [9,Cin,Cout] on the weight's device."""
    w = _cuda(w.detach().float().contiguous(), 'weight')
    Cout, Cin = w.shape[:2]
    out = torch.empty((9, Cin, Cout), dtype=torch.float32, device=w.device)
    _abi.check(_abi.load().kad_dsc_pack_weight_simt(_ptr(w), _ptr(out), Cin, Cout, _stream()), 'kad_dsc_pack_weight_simt')
    return out


def dsc_tc_supported(Cin, Cout, dtype):
    return bool(_abi.load().kad_dsc_tc_supported(Cin, Cout, _DT[dtype]))


def dsc_mma_supported(Cin, Cout, dtype, H, W):
    return dtype in _DT and bool(_abi.load().kad_dsc_mma_supported(Cin, Cout, _DT[dtype], H, W))


def pack_dsc_weight_tc(w, dtype):
    """[Cout,Cin,3,3] -> the tensor path's packed K-major operand in `dtype`."""
    w = _cuda(w.detach().float().contiguous(), 'weight')
    Cout, Cin = w.shape[:2]
    lib = _abi.load()
    nbytes = lib.kad_dsc_packed_weight_bytes(Cin, Cout, _DT[dtype])
    if nbytes == 0:
        raise RuntimeError(f'the tensor path does not support Cin={Cin} Cout={Cout} {dtype}')
    out = torch.empty(nbytes // 2, dtype=dtype, device=w.device)
    _abi.check(lib.kad_dsc_pack_weight_tc(_ptr(w), _ptr(out), Cin, Cout, _DT[dtype], _stream()), 'kad_dsc_pack_weight_tc')
    return out


_status = {}


def status_word(device):
    """Per-device int32[4] the tensor-core kernels report a timed-out wait in (checked by check_status)."""
    key = (device.type, device.index)
    if key not in _status:
        _status[key] = torch.zeros(4, dtype=torch.int32, device=device)
    return _status[key]


def raise_if_aborted(words, clear=None):
    """`words`: the four status integers as host values. Raises RuntimeError when a kernel recorded a wait that gave up
    (its results are then not valid); `clear()` is called first so that one failure is reported once."""
    if int(words[0]) != 0:
        if clear is not None:
            clear()
        raise RuntimeError(f'kadconv tensor-core kernel aborted: role {int(words[0])}, detail {int(words[1])}, block {int(words[2])}')


def check_status(device):
    """Synchronises and raises if a tensor-core kernel gave up on a wait since the last check."""
    raise_if_aborted(status_word(device).cpu().tolist(), status_word(device).zero_)


_monitor = {}


def status_poll(device):
    """Non-blocking: raises if a status snapshot taken by an earlier status_snapshot() has arrived on the host and shows an
    aborted kernel. The public entry points (FastDetector.forward, StaticGraph.__call__, the fast KADConv forward) call this on
    entry and status_snapshot() on exit, so a kernel that gave up surfaces as an exception on the next call at the latest,
    without a host synchronisation on the inference path; callers that synchronise anyway use check_status()."""
    m = _monitor.get((device.type, device.index))
    if m is not None and m['pending'] and m['event'].query():
        m['pending'] = False
        raise_if_aborted(m['host'].tolist(), status_word(device).zero_)


def status_snapshot(device):
    """Enqueues an asynchronous copy of the device status word into pinned host memory (skipped while a stream capture is
    in progress, and while the previous snapshot is still in flight)."""
    if torch.cuda.is_current_stream_capturing():
        return
    key = (device.type, device.index)
    m = _monitor.get(key)
    if m is None:
        m = _monitor[key] = {'host': torch.zeros(4, dtype=torch.int32).pin_memory(), 'event': torch.cuda.Event(), 'pending': False}
    if m['pending'] and not m['event'].query():
        return
    m['host'].copy_(status_word(device), non_blocking=True)
    m['event'].record(torch.cuda.current_stream(device))
    m['pending'] = True


def dsc_forward(x, weight, offset=None, mask=None, scale=None, shift=None, post=None, act=ACT_NONE,
                path=PATH_SIMT, y_f32=False, want_gap=False, cout=None, offset_weight=None, offset_bias=None, lcsa_inline=None, mma_frags=None):
    """Deformable 3x3 convolution with fused epilogue on NHWC tensors.

    x [B,H,W,Cin]; offset [B,H,W,18] (float32 or x.dtype) or None; mask [B,H,W,9] or None;
    weight: pack_dsc_weight_simt(...) for PATH_SIMT / PATH_MMA or pack_dsc_weight_tc(...) for PATH_TC.
    PATH_MMA only: offset_weight (pack_dsc_weight_simt of the offset convolution's weight, [9,Cin,18]) and
    offset_bias ([18]) make the kernel compute the offsets itself instead of reading `offset`; with them, lcsa_inline =
    dict(rowmean [B,H,Cin], A [B,W,Cp], Sm [W,Cp] from pyramid_project_lcsa, and the LCSA's w2 [Cin,11], b2, w3 [9,Cin], b3) makes
    the kernel evaluate the modulation mask itself instead of reading `mask`.
    Returns y [B,H,W,Cout] (and the per-tile channel sums [B,tiles,Cout] when want_gap).
    """
    lib = _abi.load()
    x = _cuda(x, 'x')
    B, H, W, Cin = x.shape
    if path in (PATH_SIMT, PATH_MMA):
        if weight.dim() != 3 or weight.shape[0] != 9 or weight.shape[1] != Cin or weight.dtype != torch.float32:
            raise ValueError('SIMT path expects weight packed as float32 [9,Cin,Cout]')
        Cout = weight.shape[2]
    else:
        if cout is None:
            raise ValueError('tensor path needs cout')
        Cout = cout
    a = _abi.KadDscArgs()
    a.x = x.data_ptr(); a.weight = _cuda(weight, 'weight').data_ptr()
    if offset is not None:
        _cuda(offset, 'offset')
        if tuple(offset.shape) != (B, H, W, 18):
            raise ValueError(f'offset must be [B,H,W,18], got {tuple(offset.shape)}')
        a.offset = offset.data_ptr(); a.offset_f32 = int(offset.dtype == torch.float32)
        if not a.offset_f32 and offset.dtype != x.dtype:
            raise TypeError('offset must be float32 or the activation dtype')
    if mask is not None:
        _cuda(mask, 'mask')
        if tuple(mask.shape) != (B, H, W, 9):
            raise ValueError(f'mask must be [B,H,W,9], got {tuple(mask.shape)}')
        a.mask = mask.data_ptr(); a.mask_f32 = int(mask.dtype == torch.float32)
        if not a.mask_f32 and mask.dtype != x.dtype:
            raise TypeError('mask must be float32 or the activation dtype')
    if offset_weight is not None:
        if path != PATH_MMA:
            raise ValueError('offset_weight is an option of PATH_MMA')
        if tuple(_f32(offset_weight, 'offset_weight').shape) != (9, Cin, 18):
            raise ValueError('offset_weight must be float32 [9,Cin,18]')
        a.offset_weight = offset_weight.data_ptr()
        if offset_bias is not None:
            if _f32(offset_bias, 'offset_bias').numel() != 18:
                raise ValueError('offset_bias must have 18 elements')
            a.offset_bias = offset_bias.data_ptr()
    if mma_frags is not None:        # pack_dsc_mma_frags(weight, offset_weight, ...): every block copies the fragments instead of deriving them
        if offset_weight is None or lcsa_inline is not None:
            raise ValueError('mma_frags goes with offset_weight and a mask tensor (PATH_MMA)')
        if mma_frags.dtype != torch.uint8 or mma_frags.numel() != _abi.load().kad_dsc_mma_frag_bytes(Cin, Cout, dtype_code(x)):
            raise ValueError('mma_frags must be the uint8 tensor pack_dsc_mma_frags made for these channel counts and this dtype')
        a.mma_frags = _cuda(mma_frags, 'mma_frags').data_ptr()
    if lcsa_inline is not None:
        if offset_weight is None:
            raise ValueError('lcsa_inline goes with offset_weight (PATH_MMA)')
        Cp = (Cin + 3) & ~3
        want = {'rowmean': (B, H, Cin), 'A': (B, W, Cp), 'Sm': (W, Cp), 'w2': (Cin, 11), 'b2': (Cin,), 'w3': (9, Cin), 'b3': (9,)}
        for name, shape in want.items():
            t = _f32(lcsa_inline[name], 'lcsa_inline.' + name)
            if tuple(t.shape) != shape:
                raise ValueError(f'lcsa_inline[{name!r}] must be {shape}, got {tuple(t.shape)}')
            setattr(a, 'lcsa_' + name, t.data_ptr())
    for name, t in (('scale', scale), ('shift', shift), ('post', post)):
        if t is not None:
            if _f32(t, name).numel() != Cout:
                raise ValueError(f'{name} must have {Cout} elements')
            setattr(a, name, t.data_ptr())
    y = torch.empty((B, H, W, Cout), dtype=torch.float32 if y_f32 else x.dtype, device=x.device)
    gap = None
    if want_gap:
        tiles = lib.kad_dsc_gap_tiles(H, W, Cin, Cout, path)
        gap = torch.empty((B, tiles, Cout), dtype=torch.float32, device=x.device)
        a.gap_partial = gap.data_ptr()
    a.y = y.data_ptr()
    a.B, a.H, a.W, a.Cin, a.Cout = B, H, W, Cin, Cout
    a.dtype = dtype_code(x); a.y_f32 = int(y_f32); a.act = act; a.path = path
    a.status = status_word(x.device).data_ptr()
    _abi.check(lib.kad_dsc_forward(ctypes.byref(a), _stream()), 'kad_dsc_forward')
    return (y, gap) if want_gap else y


def pool_project(x, w, bias=None, pool=1, act=ACT_NONE, cin=None, out=None, out_coff=0):
    """avg-pool (pool x pool, floor) + 1x1 conv + bias + activation. x [B,H,W,Cx] NHWC; only the first
    `cin` channels (default all) are read. With `out` ([B,Ho,Wo,Cy]) the result is written into its channels
    [out_coff, out_coff + Cout) in place; otherwise a new tensor is returned."""
    x = _cuda(x, 'x'); w = _f32(w, 'w'); bias = _f32(bias, 'bias')
    B, H, W, Cx = x.shape
    Cin = Cx if cin is None else cin
    Cout = w.shape[0]
    if w.shape[1] != Cin:
        raise ValueError(f'weight is {tuple(w.shape)} but Cin = {Cin}')
    Ho, Wo = H // pool, W // pool
    if out is None:
        out = torch.empty((B, Ho, Wo, Cout), dtype=x.dtype, device=x.device)
        dst, ycs = out, Cout
    else:
        _cuda(out, 'out')
        ycs = out.shape[3]
        dst = out.view(-1)[out_coff:]
    _abi.check(_abi.load().kad_pool_project(_ptr(x), _ptr(w), _ptr(bias), ctypes.c_void_p(dst.data_ptr()), B, H, W, Cin, Cout, pool, act,
                                            Cx, ycs, dtype_code(x), _stream()), 'kad_pool_project')
    return out


def lcsa_mask(x, prm, mask_f32=True):
    """sigmoid(LCSA(x)) for NHWC x -> [B,H,W,9]. `prm`: dict of float32 tensors w1[C,11], b1, bn_m, bn_a,
    w2[C,11], b2, w3[9,C], b3 (BatchNorm already folded into bn_m / bn_a)."""
    lib = _abi.load()
    x = _cuda(x, 'x')
    B, H, W, C = x.shape
    dev = x.device
    rows = torch.empty((B, H, C), dtype=torch.float32, device=dev)
    cols = torch.empty((B, W, C), dtype=torch.float32, device=dev)
    _abi.check(lib.kad_lcsa_sums(_ptr(x), _ptr(rows), _ptr(cols), B, H, W, C, dtype_code(x), _stream()), 'kad_lcsa_sums')
    scratch = torch.empty(B * W * C + W * C, dtype=torch.float32, device=dev)
    mask = torch.empty((B, H, W, 9), dtype=torch.float32 if mask_f32 else x.dtype, device=dev)
    _abi.check(lib.kad_lcsa_mask(_ptr(rows), _ptr(cols), _ptr(prm['w1']), _ptr(prm['b1']), _ptr(prm['bn_m']), _ptr(prm['bn_a']),
                                 _ptr(prm['w2']), _ptr(prm['b2']), _ptr(prm['w3']), _ptr(prm['b3']), _ptr(scratch), _ptr(mask),
                                 B, H, W, C, int(mask_f32), dtype_code(x), _stream()), 'kad_lcsa_mask')
    return mask


def se_excite(gap, count, w1, b1, w2, b2):
    """gap [B,tiles,C] per-tile sums over `count` pixels -> attention [B,C] float32."""
    B, tiles, C = gap.shape
    Hd = w1.shape[0]
    att = torch.empty((B, C), dtype=torch.float32, device=gap.device)
    _abi.check(_abi.load().kad_se_excite(_ptr(gap), tiles, ctypes.c_float(1.0 / count), _ptr(_f32(w1, 'w1')), _ptr(_f32(b1, 'b1')),
                                         _ptr(_f32(w2, 'w2')), _ptr(_f32(b2, 'b2')), _ptr(att), B, C, Hd, _stream()), 'kad_se_excite')
    return att


def se_squeeze(x):
    x = _cuda(x, 'x')
    B, H, W, C = x.shape
    lib = _abi.load()
    tiles = lib.kad_se_squeeze_tiles(H, W)
    gap = torch.empty((B, tiles, C), dtype=torch.float32, device=x.device)
    _abi.check(lib.kad_se_squeeze(_ptr(x), _ptr(gap), B, H, W, C, dtype_code(x), _stream()), 'kad_se_squeeze')
    return gap


def se_rescale(x, att):
    x = _cuda(x, 'x')
    B, H, W, C = x.shape
    y = torch.empty_like(x)
    _abi.check(_abi.load().kad_se_rescale(_ptr(x), _ptr(_f32(att, 'att')), _ptr(y), B, H, W, C, dtype_code(x), _stream()), 'kad_se_rescale')
    return y


def merge_upsample_residual(x, ys, atts=None, se=None, out=None, out_coff=0):
    """out = cat_i(upsample(ys[i] * att_i)) + x, all NHWC. The attentions are either given (atts[i] float32 [B,c_i]) or
    computed inside the kernel from se[i] = (gap [B,tiles,c_i], fc_w1, fc_b1, fc_w2, fc_b2), the channel sums of
    dsc_forward(want_gap=True) and the weights of the branch's fc. With `out` ([B,H,W,Cy]) the result is written into
    its channels [out_coff, out_coff + C) in place."""
    x = _cuda(x, 'x')
    B, H, W, C = x.shape
    a = _abi.KadMergeArgs()
    if out is None:
        out = torch.empty_like(x)
        a.out = out.data_ptr()
    else:
        if out.shape[:3] != x.shape[:3] or out.dtype != x.dtype or not out.is_contiguous() or out_coff + C > out.shape[3]:
            raise ValueError('out must be a contiguous [B,H,W,Cy] tensor of the same dtype with room for C channels at out_coff')
        a.out = out.data_ptr() + out_coff * out.element_size(); a.out_cstride = out.shape[3]
    a.x = x.data_ptr()
    keep = []
    for i in range(3):
        yi = _cuda(ys[i], f'y{i}')
        a.y[i] = yi.data_ptr()
        a.c[i], a.h[i], a.w[i] = yi.shape[3], yi.shape[1], yi.shape[2]
        if se is not None:
            gap, w1, b1, w2, b2 = se[i]
            if tuple(gap.shape) != (B, gap.shape[1], yi.shape[3]):
                raise ValueError(f'gap{i} must be [B,tiles,{yi.shape[3]}]')
            a.gap[i] = _f32(gap, 'gap').data_ptr(); a.gap_tiles[i] = gap.shape[1]; a.hidden[i] = w1.shape[0]
            a.fc_w1[i] = _f32(w1, 'fc_w1').data_ptr(); a.fc_b1[i] = _f32(b1, 'fc_b1').data_ptr()
            a.fc_w2[i] = _f32(w2, 'fc_w2').data_ptr(); a.fc_b2[i] = _f32(b2, 'fc_b2').data_ptr()
            att = torch.empty((B, yi.shape[3]), dtype=torch.float32, device=x.device)
            keep.append(att)
        else:
            att = _f32(atts[i], f'att{i}')
        a.att[i] = att.data_ptr()
    a.B, a.H, a.W, a.C, a.dtype = B, H, W, C, dtype_code(x)
    _abi.check(_abi.load().kad_merge_upsample_residual(ctypes.byref(a), _stream()), 'kad_merge_upsample_residual')
    return out


def gemm1x1_supported(K, N, dtype):
    return dtype in (torch.float16, torch.bfloat16) and bool(_abi.load().kad_gemm1x1_tc_supported(K, N, _DT[dtype]))


def gemm1x1_bias_act(x, w, bias=None, act=ACT_SILU, k=None, out=None, out_coff=0):
    """1x1 convolution on tensor cores. x [..., Cx] NHWC (first k channels used), w [N, Kp] in x.dtype
    (Kp = k rounded up to 8), bias float32 [N]. Writes into out[..., out_coff:out_coff+N] when given."""
    x = _cuda(x, 'x'); w = _cuda(w, 'w')
    Cx = x.shape[-1]
    K = Cx if k is None else k
    N = w.shape[0]
    M = x.numel() // Cx
    if out is None:
        out = torch.empty(tuple(x.shape[:-1]) + (N,), dtype=x.dtype, device=x.device)
        dst, ldy = out, N
    else:
        ldy = out.shape[-1]
        dst = out.view(-1)[out_coff:]
    _abi.check(_abi.load().kad_gemm1x1_bias_act(_ptr(x), _ptr(w), _ptr(_f32(bias, 'bias')), ctypes.c_void_p(dst.data_ptr()), M, K, N, Cx, ldy, act,
                                                dtype_code(x), _ptr(status_word(x.device)), _stream()), 'kad_gemm1x1_bias_act')
    return out


def gemm1x1_bias_act_raw(src, shape, w, bias, act, k, out=None, out_coff=0):
    """Like gemm1x1_bias_act, for an input that is a channel slice of a wider NHWC tensor: `src` is a
    flat view starting at the slice's first element, `shape` the [B,H,W,Cx] shape of the full tensor."""
    Cx = shape[-1]
    M = 1
    for d in shape[:-1]:
        M *= d
    N = w.shape[0]
    if out is None:
        out = torch.empty(tuple(shape[:-1]) + (N,), dtype=w.dtype, device=w.device)
        dst, ldy = out, N
    else:
        ldy = out.shape[-1]
        dst = out.view(-1)[out_coff:]
    _abi.check(_abi.load().kad_gemm1x1_bias_act(ctypes.c_void_p(src.data_ptr()), _ptr(w), _ptr(_f32(bias, 'bias')),
                                                ctypes.c_void_p(dst.data_ptr()), M, k, N, Cx, ldy, act, _DT[w.dtype],
                                                _ptr(status_word(w.device)), _stream()), 'kad_gemm1x1_bias_act')
    return out


def conv3x3_supported(cin, cout, stride, dtype):
    return dtype in (torch.float16, torch.bfloat16) and bool(_abi.load().kad_conv3x3_tc_supported(cin, cout, stride, _DT[dtype]))


def pack_conv3x3_weight(weight, dtype, groups=1):
    """Conv2d weight [Cout, Cin/groups, 3, 3] -> [Cout, 9, Cin] in `dtype` (tap-major, channels innermost). A grouped
    convolution becomes the equivalent dense one (zeros outside each group's block)."""
    cout, cg = weight.shape[:2]
    w = weight.detach().float().permute(0, 2, 3, 1).reshape(cout, 9, cg)
    if groups > 1:
        dense = w.new_zeros((cout, 9, cg * groups))
        og = cout // groups
        for g in range(groups):
            dense[g * og:(g + 1) * og, :, g * cg:(g + 1) * cg] = w[g * og:(g + 1) * og]
        w = dense
    return w.to(dtype).contiguous()


def conv3x3_bias_act(x, w, bias=None, act=ACT_SILU, stride=1, in_coff=0, cin=None, out=None, out_coff=0):
    """3x3 convolution, padding 1, on tensor cores. x [B,H,W,Cx] NHWC (channels [in_coff, in_coff+cin) are read),
    w [Cout,9,cin] in x.dtype (pack_conv3x3_weight), bias float32 [Cout]. Writes out[..., out_coff:out_coff+Cout] when
    `out` [B,Ho,Wo,Cy] is given."""
    x = _cuda(x, 'x'); w = _cuda(w, 'w')
    B, H, W, Cx = x.shape
    N, _, K = w.shape
    if cin is not None and cin != K:
        raise ValueError(f'conv3x3_bias_act: weight has {K} input channels, cin = {cin}')
    Ho, Wo = (H - 1) // stride + 1, (W - 1) // stride + 1
    if out is None:
        out = torch.empty((B, Ho, Wo, N), dtype=x.dtype, device=x.device)
        dst, ldy = out, N
    else:
        if tuple(out.shape[:3]) != (B, Ho, Wo):
            raise ValueError(f'conv3x3_bias_act: out has shape {tuple(out.shape)}, expected [{B},{Ho},{Wo},*]')
        ldy = out.shape[-1]
        dst = out.view(-1)[out_coff:]
    src = x.view(-1)[in_coff:] if in_coff else x
    bptr = _ptr(_f32(bias, 'bias')) if bias is not None else None
    _abi.check(_abi.load().kad_conv3x3_bias_act(ctypes.c_void_p(src.data_ptr()), _ptr(w), bptr, ctypes.c_void_p(dst.data_ptr()),
                                                B, H, W, K, N, stride, Cx, ldy, act, dtype_code(x), _ptr(status_word(x.device)), _stream()),
               'kad_conv3x3_bias_act')
    return out


def nms_batched(pred, conf_thres, iou_thres, max_det=300, max_wh=7680.0, out=None):
    """pred [B,4+nc,A] (DDetect's y) -> (dets [B,max_det,6] float32, counts [B] int32), all on the device, one launch.
    `out` = (dets, counts) reuses existing buffers (they are cleared first)."""
    pred = _cuda(pred, 'pred')
    B, no, A = pred.shape
    if out is None:
        dets = torch.zeros((B, max_det, 6), dtype=torch.float32, device=pred.device)
        counts = torch.zeros(B, dtype=torch.int32, device=pred.device)
    else:
        dets, counts = out
        if tuple(dets.shape) != (B, max_det, 6) or dets.dtype != torch.float32 or tuple(counts.shape) != (B,) or counts.dtype != torch.int32:
            raise ValueError('out must be (float32 [B,max_det,6], int32 [B])')
        _cuda(dets, 'dets').zero_(); _cuda(counts, 'counts').zero_()
    _abi.check(_abi.load().kad_nms_batched(_ptr(pred), B, no - 4, A, ctypes.c_float(conf_thres), ctypes.c_float(iou_thres), max_det,
                                           ctypes.c_float(max_wh), _ptr(dets), _ptr(counts), dtype_code(pred), _stream()), 'kad_nms_batched')
    return dets, counts


def head_decode(raws, strides, reg_max, nc):
    """DDetect's inference decode on the device: raws = per-scale [B,H,W,4*reg_max+nc] NHWC tensors, strides = their
    pixel strides. Returns pred [B, 4+nc, A] (xywh in pixels + sigmoid scores), anchors in (scale, y, x) order."""
    B = raws[0].shape[0]
    A = sum(r.shape[1] * r.shape[2] for r in raws)
    pred = torch.empty((B, 4 + nc, A), dtype=raws[0].dtype, device=raws[0].device)
    off = 0
    for r, s in zip(raws, strides):
        r = _cuda(r, 'raw')
        _, H, W, no = r.shape
        if no != 4 * reg_max + nc:
            raise ValueError(f'head_decode: {no} channels, expected {4 * reg_max + nc}')
        _abi.check(_abi.load().kad_head_decode(_ptr(r), _ptr(pred), B, H, W, reg_max, nc, ctypes.c_float(float(s)), off, A, dtype_code(r), _stream()),
                   'kad_head_decode')
        off += H * W
    return pred


def avg_pool(x, pool):
    """NHWC average pool, kernel = stride = pool, floor mode."""
    x = _cuda(x, 'x')
    B, H, W, C = x.shape
    y = torch.empty((B, H // pool, W // pool, C), dtype=x.dtype, device=x.device)
    _abi.check(_abi.load().kad_avg_pool(_ptr(x), _ptr(y), B, H, W, C, pool, dtype_code(x), _stream()), 'kad_avg_pool')
    return y


def avg_pool2x2s1(x):
    """NHWC 2x2 average pool with stride 1 (no padding)."""
    x = _cuda(x, 'x')
    B, H, W, C = x.shape
    y = torch.empty((B, H - 1, W - 1, C), dtype=x.dtype, device=x.device)
    _abi.check(_abi.load().kad_avg_pool2x2s1(_ptr(x), _ptr(y), B, H, W, C, dtype_code(x), _stream()), 'kad_avg_pool2x2s1')
    return y


def bias_act_(y, bias, act=ACT_SILU):
    """In place y = act(y + bias) over the last dimension of a contiguous tensor."""
    y = _cuda(y, 'y')
    C = y.shape[-1]
    _abi.check(_abi.load().kad_bias_act_inplace(_ptr(y), _ptr(_f32(bias, 'bias')), y.numel() // C, C, act, dtype_code(y), _stream()),
               'kad_bias_act_inplace')
    return y


def bias_act_to(y, bias, out, out_coff=0, act=ACT_SILU):
    """out[..., out_coff:out_coff+C] = act(y + bias) for contiguous y [..., C] and contiguous out [..., Cy] (same leading shape)."""
    y = _cuda(y, 'y'); out = _cuda(out, 'out')
    C = y.shape[-1]
    if out.shape[:-1] != y.shape[:-1] or out.dtype != y.dtype or out_coff + C > out.shape[-1]:
        raise ValueError('out must have the leading shape and dtype of y and room for C channels at out_coff')
    _abi.check(_abi.load().kad_bias_act_to(_ptr(y), _ptr(_f32(bias, 'bias')), ctypes.c_void_p(out.data_ptr() + out_coff * out.element_size()),
                                           y.numel() // C, C, out.shape[-1], act, dtype_code(y), _stream()), 'kad_bias_act_to')
    return out


def parameters_fence(device):
    """One ordinary, tiny piece of work on the current stream. Most kernels of this package are launched with programmatic stream
    serialization and read their PARAMETERS (weights, bias, folded BatchNorm vectors) before they wait for the kernel in front of
    them; parameters that the stream has only just produced (folding, packing, a dtype conversion) must therefore not come from the
    kernel IMMEDIATELY before such a launch. Whatever runs between the two (this call) restores the ordinary stream order for them.
    Called wherever this package derives parameters; a caller of the C ABI that computes weights on the stream right before a call
    does the same, or synchronises once."""
    _FENCE.setdefault(str(device), torch.zeros(1, dtype=torch.int32, device=device)).zero_()


_FENCE = {}


def pack_dsc_mma_frags(weight_simt, offset_weight_simt, dtype):
    """Weight fragments of the warp-MMA deformable convolution with fused offsets (both convolutions), packed once for `dtype`:
    pass the result as dsc_forward(..., mma_frags=...) together with the two weights it was made from."""
    w = _f32(weight_simt, 'weight_simt'); wo = _f32(offset_weight_simt, 'offset_weight_simt')
    cin, cout = w.shape[1], w.shape[2]
    if tuple(wo.shape) != (9, cin, 18):
        raise ValueError('offset_weight_simt must be float32 [9,Cin,18]')
    n = _abi.load().kad_dsc_mma_frag_bytes(cin, cout, _DT[dtype])
    if n == 0:
        raise ValueError('no warp-MMA path for these channel counts / this dtype')
    out = torch.empty(n, dtype=torch.uint8, device=w.device)
    _abi.check(_abi.load().kad_dsc_mma_pack_frags(_ptr(w), _ptr(wo), _ptr(out), cin, cout, _DT[dtype], _stream()), 'kad_dsc_mma_pack_frags')
    return out


def copy_channels(src, src_coff, C, dst=None, dst_coff=0):
    """dst[..., dst_coff:dst_coff+C] = src[..., src_coff:src_coff+C] for contiguous tensors with the same leading shape; with
    dst=None a new dense [..., C] tensor is returned (what `src[..., a:b].contiguous()` gives, in one vectorised kernel)."""
    src = _cuda(src, 'src')
    if dst is None:
        dst = torch.empty(src.shape[:-1] + (C,), dtype=src.dtype, device=src.device)
    dst = _cuda(dst, 'dst')
    if dst.shape[:-1] != src.shape[:-1] or dst.dtype != src.dtype:
        raise ValueError('dst must have the leading shape and dtype of src')
    if src_coff < 0 or dst_coff < 0 or src_coff + C > src.shape[-1] or dst_coff + C > dst.shape[-1]:
        raise ValueError('channel slice outside the tensor')
    _abi.check(_abi.load().kad_copy_channels(_ptr(src), src.shape[-1], src_coff, _ptr(dst), dst.shape[-1], dst_coff,
                                             src.numel() // src.shape[-1], C, dtype_code(src), _stream()), 'kad_copy_channels')
    return dst


def upsample2x_concat(low, skip):
    """cat((nearest-2x-upsample(low), skip), channels): low [B,h,w,C1], skip [B,2h,2w,C2] -> [B,2h,2w,C1+C2], NHWC."""
    low = _cuda(low, 'low'); skip = _cuda(skip, 'skip')
    B, h, w, C1 = low.shape
    if skip.shape[:3] != (B, 2 * h, 2 * w) or skip.dtype != low.dtype:
        raise ValueError(f'skip must be [B,{2 * h},{2 * w},C2] of the same dtype, got {tuple(skip.shape)}')
    out = torch.empty((B, 2 * h, 2 * w, C1 + skip.shape[3]), dtype=low.dtype, device=low.device)
    _abi.check(_abi.load().kad_upsample2x_concat(_ptr(low), _ptr(skip), _ptr(out), B, h, w, C1, skip.shape[3], dtype_code(low), _stream()),
               'kad_upsample2x_concat')
    return out


def image_to_nhwc(img_u8, dtype, cpad=8, scale=1.0 / 255.0):
    """uint8 [B,C,H,W] -> dtype [B,H,W,cpad], scaled, extra channels zero."""
    img_u8 = _cuda(img_u8, 'img')
    if img_u8.dtype != torch.uint8:
        raise TypeError('image_to_nhwc expects a uint8 tensor')
    B, C, H, W = img_u8.shape
    y = torch.empty((B, H, W, cpad), dtype=dtype, device=img_u8.device)
    _abi.check(_abi.load().kad_image_to_nhwc(_ptr(img_u8), _ptr(y), B, C, H, W, cpad, ctypes.c_float(scale), _DT[dtype], _stream()),
               'kad_image_to_nhwc')
    return y


def stem_conv_supported(cin, cout, dtype):
    return dtype in _DT and bool(_abi.load().kad_stem_conv_supported(cin, cout, _DT[dtype]))


def stem_conv_u8(img_u8, w, bias, dtype, act=ACT_SILU, scale=1.0 / 255.0):
    """uint8 [B,Cin,H,W] -> act(conv3x3 stride 2 pad 1 (img * scale) + bias) as dtype [B,OH,OW,Cout] (NHWC).
    w float32 [Cout,Cin,3,3], bias float32 [Cout] or None."""
    img_u8 = _cuda(img_u8, 'img')
    if img_u8.dtype != torch.uint8:
        raise TypeError('stem_conv_u8 expects a uint8 tensor')
    w = _f32(w, 'w')
    B, C, H, W = img_u8.shape
    if tuple(w.shape[1:]) != (C, 3, 3):
        raise ValueError(f'w must be [Cout,{C},3,3]')
    y = torch.empty((B, (H - 1) // 2 + 1, (W - 1) // 2 + 1, w.shape[0]), dtype=dtype, device=img_u8.device)
    _abi.check(_abi.load().kad_stem_conv_u8(_ptr(img_u8), _ptr(w), _ptr(_f32(bias, 'bias')), _ptr(y), B, C, H, W, w.shape[0],
                                            ctypes.c_float(scale), act, _DT[dtype], _stream()), 'kad_stem_conv_u8')
    return y


def pyramid_project_supported(dim, cs, dtype, H, W):
    return dtype in _DT and bool(_abi.load().kad_pyramid_project_supported(dim, cs[0], cs[1], cs[2], _DT[dtype], H, W))


_counters = {}


def layer_counters(device):
    """Per-device int32[65536] of zeros for the kernels that count finished blocks per image (every such kernel leaves
    them zero again). Created on first use; create it outside any stream capture."""
    key = (device.type, device.index)
    if key not in _counters:
        _counters[key] = torch.zeros(65536, dtype=torch.int32, device=device)
    return _counters[key]


def pyramid_lcsa_supported(dim, cs, dtype, H, W):
    return dtype in _DT and bool(_abi.load().kad_pyramid_lcsa_supported(dim, cs[0], cs[1], cs[2], _DT[dtype], H, W))


def dsc_mma_inline_mask_supported(Cin, Cout, dtype, H, W):
    return dtype in _DT and bool(_abi.load().kad_dsc_mma_inline_mask_supported(Cin, Cout, _DT[dtype], H, W))


def pyramid_project_lcsa(x, ws, bs, lcsas):
    """pyramid_project that also finishes the first stage of the three LCSAs in the kernel's tail. lcsas[i]: dict with
    w1 [c_i,11], b1, bn_m, bn_a (folded BatchNorm). Returns (ts, ops) where ops[i] = dict(rowmean [B,h_i,c_i], A [B,w_i,Cp_i],
    Sm [w_i,Cp_i]) is what dsc_forward(..., lcsa_inline=...) consumes."""
    x = _cuda(x, 'x')
    B, H, W, dim = x.shape
    cs = [int(w.shape[0]) for w in ws]
    lib = _abi.load()
    nct, nrg = ctypes.c_int(0), ctypes.c_int(0)
    _abi.check(lib.kad_pyramid_partial_dims(B, H, W, dim, cs[0], cs[1], cs[2], dtype_code(x), ctypes.byref(nct), ctypes.byref(nrg)), 'kad_pyramid_partial_dims', 0)
    a = _abi.KadPyramidArgs()
    a.x = x.data_ptr(); a.B, a.H, a.W, a.dim, a.dtype = B, H, W, dim, dtype_code(x)
    a.counters = layer_counters(x.device).data_ptr()
    ts, outs, keep = [], [], []
    for i in range(3):
        h, w, c = H >> i, W >> i, cs[i]
        Cp = (c + 3) & ~3
        t = torch.empty((B, h, w, c), dtype=x.dtype, device=x.device)
        rp = torch.empty((B, h, nct.value, c), dtype=torch.float32, device=x.device)
        cp = torch.empty((B, nrg.value, w, c), dtype=torch.float32, device=x.device)
        o = {'rowmean': torch.empty((B, h, c), dtype=torch.float32, device=x.device),
             'A': torch.empty((B, w, Cp), dtype=torch.float32, device=x.device), 'Sm': torch.empty((w, Cp), dtype=torch.float32, device=x.device)}
        a.w[i] = _f32(ws[i], 'w').data_ptr(); a.bias[i] = _f32(bs[i], 'bias').data_ptr() if bs[i] is not None else None
        a.t[i] = t.data_ptr(); a.c[i] = c; a.rowpart[i] = rp.data_ptr(); a.colpart[i] = cp.data_ptr()
        l = lcsas[i]
        a.lcsa_w1[i] = _f32(l['w1'], 'w1').data_ptr(); a.lcsa_b1[i] = _f32(l['b1'], 'b1').data_ptr()
        a.lcsa_bn_scale[i] = _f32(l['bn_m'], 'bn_m').data_ptr(); a.lcsa_bn_shift[i] = _f32(l['bn_a'], 'bn_a').data_ptr()
        a.lcsa_rowmean[i] = o['rowmean'].data_ptr(); a.lcsa_A[i] = o['A'].data_ptr(); a.lcsa_Sm[i] = o['Sm'].data_ptr()
        ts.append(t); outs.append(o); keep += [rp, cp]
    _abi.check(lib.kad_pyramid_project_lcsa(ctypes.byref(a), _stream()), 'kad_pyramid_project_lcsa')
    return ts, outs


def pyramid_project(x, ws, bs, want_partials=False):
    """t[i] = conv1x1(avg_pool2d(x, 2**i), ws[i]) + bs[i] for i = 0, 1, 2 in one kernel. x [B,H,W,dim] NHWC (f16/bf16),
    ws[i] float32 [c_i, dim], bs[i] float32 [c_i] or None. Returns the three NHWC tensors, and with want_partials also the
    partial sums for lcsa_mask_from_partials: a list of (rowpart [B,h_i,n_col_tiles,c_i], colpart [B,n_row_groups,w_i,c_i])."""
    x = _cuda(x, 'x')
    B, H, W, dim = x.shape
    cs = [int(w.shape[0]) for w in ws]
    lib = _abi.load()
    ts = [torch.empty((B, H >> i, W >> i, cs[i]), dtype=x.dtype, device=x.device) for i in range(3)]
    P3 = ctypes.c_void_p * 3
    wp = P3(*[_f32(w, 'w').data_ptr() for w in ws])
    bp = P3(*[(_f32(b, 'b').data_ptr() if b is not None else None) for b in bs])
    tp = P3(*[t.data_ptr() for t in ts])
    cp = (ctypes.c_int * 3)(*cs)
    parts, rp, cpp = None, None, None
    if want_partials:
        nct, nrg = ctypes.c_int(0), ctypes.c_int(0)
        _abi.check(lib.kad_pyramid_partial_dims(B, H, W, dim, cs[0], cs[1], cs[2], dtype_code(x), ctypes.byref(nct), ctypes.byref(nrg)),
                   'kad_pyramid_partial_dims', 0)
        parts = [(torch.empty((B, H >> i, nct.value, cs[i]), dtype=torch.float32, device=x.device),
                  torch.empty((B, nrg.value, W >> i, cs[i]), dtype=torch.float32, device=x.device)) for i in range(3)]
        rp = P3(*[p[0].data_ptr() for p in parts]); cpp = P3(*[p[1].data_ptr() for p in parts])
    _abi.check(lib.kad_pyramid_project(_ptr(x), wp, bp, tp, B, H, W, dim, cp, dtype_code(x), rp, cpp, _stream()), 'kad_pyramid_project')
    return (ts, parts) if want_partials else ts


def lcsa_mask_from_partials_supported(H, W, C):
    return bool(_abi.load().kad_lcsa_mask_from_partials_supported(H, W, C))


def lcsa_mask_from_partials(rowpart, colpart, prm, dtype, mask_f32=False):
    """LCSA mask [B,H,W,9] from the partial sums of pyramid_project (rowpart [B,H,nct,C], colpart [B,nrg,W,C]);
    prm as for lcsa_mask. The mask is float32 if mask_f32 else `dtype` (the dtype of the branch tensor)."""
    rowpart = _f32(rowpart, 'rowpart'); colpart = _f32(colpart, 'colpart')
    B, H, nct, C = rowpart.shape
    nrg, W = colpart.shape[1], colpart.shape[2]
    dev = rowpart.device
    scratch = torch.empty((B + 1) * W * ((C + 3) // 4 * 4), dtype=torch.float32, device=dev)
    rowsum = torch.empty((B, H, C), dtype=torch.float32, device=dev)
    mask = torch.empty((B, H, W, 9), dtype=torch.float32 if mask_f32 else dtype, device=dev)
    _abi.check(_abi.load().kad_lcsa_mask_from_partials(
        _ptr(rowpart), nct, _ptr(colpart), nrg, _ptr(prm['w1']), _ptr(prm['b1']), _ptr(prm['bn_m']), _ptr(prm['bn_a']),
        _ptr(prm['w2']), _ptr(prm['b2']), _ptr(prm['w3']), _ptr(prm['b3']), _ptr(scratch), _ptr(rowsum), _ptr(mask),
        B, H, W, C, int(mask_f32), _DT[dtype], _stream()), 'kad_lcsa_mask_from_partials', 2)
    return mask


def spp_pool3_supported(H, W, C, dtype):
    return dtype in _DT and bool(_abi.load().kad_spp_pool3_supported(H, W, C, _DT[dtype]))


def spp_pool3_(cat, C):
    """cat [B,H,W,4*C] NHWC with y1 in channels [0, C): fills the other three quarters with the chained 5x5 max-pools
    (stride 1, padding 2) of SPPELAN, in place. Returns cat."""
    cat = _cuda(cat, 'cat')
    B, H, W, C4 = cat.shape
    if C4 != 4 * C:
        raise ValueError('cat must have 4*C channels')
    _abi.check(_abi.load().kad_spp_pool3(_ptr(cat), B, H, W, C, dtype_code(cat), _stream()), 'kad_spp_pool3')
    return cat


def lcsa_masks3_supported(H, W, cs):
    return bool(_abi.load().kad_lcsa_masks3_supported(H, W, cs[0], cs[1], cs[2]))


def lcsa_masks3_from_partials(parts, prms, dtype, H, W, mask_f32=True):
    """The LCSA masks of the three branches in one launch. parts[i] = (rowpart [B,h_i,nct,c_i], colpart [B,nrg,w_i,c_i]) from
    pyramid_project(..., want_partials=True); prms[i] as for lcsa_mask. Returns three masks [B,h_i,w_i,9]."""
    B, _, nct, _ = parts[0][0].shape
    nrg = parts[0][1].shape[1]
    dev = parts[0][0].device
    cs = [int(p[0].shape[3]) for p in parts]
    masks = [torch.empty((B, H >> i, W >> i, 9), dtype=torch.float32 if mask_f32 else dtype, device=dev) for i in range(3)]
    arr = lambda ts: (ctypes.c_void_p * 3)(*[t.data_ptr() for t in ts])
    f = lambda key: arr([_f32(p[key], key) for p in prms])
    c3 = (ctypes.c_int * 3)(*cs)
    _abi.check(_abi.load().kad_lcsa_masks3_from_partials(
        arr([_f32(p[0], 'rowpart') for p in parts]), arr([_f32(p[1], 'colpart') for p in parts]), nct, nrg,
        f('w1'), f('b1'), f('bn_m'), f('bn_a'), f('w2'), f('b2'), f('w3'), f('b3'), arr(masks), B, H, W, c3, int(mask_f32), _DT[dtype], _stream()),
        'kad_lcsa_masks3_from_partials')
    return masks
