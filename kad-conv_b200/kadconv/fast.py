"""enable_fast_inference / disable_fast_inference: the B200 pipeline behind the reference's switch.

Same call as KAD-Conv/kadconv/fast.py:68-118 of the reference project: layers are found by class NAME
('KADConv', 'KADC4', 'KADC4_m'), their ``forward`` is replaced per instance, ``disable_fast_inference``
restores the plain forward. Differences, all on purpose:
  * batch >= 1, H != W, float32 / float16 / bfloat16, NCHW-contiguous or channels_last inputs
    (the reference's fast path takes float32 (1,C,H,H) contiguous only, fast.py:38-40);
  * no silent fallback: an input the CUDA path cannot take (CPU tensor, training mode) raises.

Per layer and call the pipeline is, in NHWC:
  pool+project (x3) -> per branch: LCSA sums, LCSA mask, offset conv, DSC(+BN+ReLU+scale+SE partial sums),
  SE excite -> merge (attention, bilinear upsample, concat, residual).
Folded parameters are computed once per (layer, device) and cached on the module.
"""
import types

import torch

from . import ops

_LAYER_TYPES = {'KADConv', 'KADC4', 'KADC4_m'}
_FAST_ATTR = '_kad_b200'
# How kad_kadconv_forward produces the LCSA masks (KadLayerArgs.scheme): 0 = the library's choice, 1 = separate kernels,
# 2 = first stage in the pyramid kernel's tail + one mask kernel per branch, 3 = masks inside the deformable convolutions,
# 4 = one launch for the three branches.
# All forms are bit-identical; tests and benchmarks switch this to compare them.
LAYER_SCHEME = 0


def _bn_fold(bn):
    eps = bn.eps
    m = bn.weight.detach().float() / torch.sqrt(bn.running_var.detach().float() + eps)
    a = bn.bias.detach().float() - bn.running_mean.detach().float() * m
    return m, a


class _BranchParams:
    """Float32, contiguous, device-resident parameters of one KAD-Conv branch."""

    def __init__(self, conv_seq, fc, scale_seq, device):
        proj, dsc, bn = conv_seq[0], conv_seq[1], conv_seq[2]
        f = lambda t: t.detach().float().contiguous().to(device)
        c = dsc.weight.shape[0]
        self.c = c
        self.w_proj = f(proj.weight.view(proj.weight.shape[0], -1))
        self.b_proj = f(proj.bias)
        ex = dsc.RCA_mask.excite
        m1, a1 = _bn_fold(ex[1])
        self.lcsa = dict(w1=f(ex[0].weight.view(c, 11)), b1=f(ex[0].bias), bn_m=f(m1), bn_a=f(a1),
                         w2=f(ex[3].weight.view(c, 11)), b2=f(ex[3].bias),
                         w3=f(ex[4].weight.view(9, c)), b3=f(ex[4].bias))
        self.w_off = ops.pack_dsc_weight_simt(dsc.conv_offset.weight.to(device))
        self.b_off = f(dsc.conv_offset.bias)
        self.dsc_weight_raw = f(dsc.weight)
        self.w_dsc_simt = ops.pack_dsc_weight_simt(self.dsc_weight_raw)
        self.w_dsc_tc = {}
        self.w_dsc_mma = {}
        m, a = _bn_fold(bn)
        self.ep_scale = f(m)
        self.ep_shift = f(a + dsc.bias.detach().float() * m)     # conv bias passes through the BN affine
        self.ep_post = f(scale_seq[0].weight.view(-1))
        self.fc_w1, self.fc_b1 = f(fc[0].weight), f(fc[0].bias)
        self.fc_w2, self.fc_b2 = f(fc[2].weight), f(fc[2].bias)

    def dsc_weight(self, dtype, h, w):
        """(path, packed weight) for activations of `dtype` on an h x w map."""
        if dtype != torch.float32 and ops.dsc_tc_supported(self.c, self.c, dtype):
            if dtype not in self.w_dsc_tc:
                self.w_dsc_tc[dtype] = ops.pack_dsc_weight_tc(self.dsc_weight_raw, dtype)
            return ops.PATH_TC, self.w_dsc_tc[dtype]
        if ops.dsc_mma_supported(self.c, self.c, dtype, h, w):
            if dtype not in self.w_dsc_mma:      # fragments of both convolutions, packed once: the kernel's blocks copy them
                self.w_dsc_mma[dtype] = ops.pack_dsc_mma_frags(self.w_dsc_simt, self.w_off, dtype)
            return ops.PATH_MMA, self.w_dsc_simt
        return ops.PATH_SIMT, self.w_dsc_simt


def parameter_fingerprint(layer):
    """Changes whenever a parameter or buffer of the layer is replaced (load_state_dict on a meta/cast module, .half(),
    .to()) or updated in place (optimizer step, load_state_dict's copy_, manual edits): storage address and version
    counter of every tensor of the layer."""
    return tuple((t.data_ptr(), t._version) for t in list(layer.parameters()) + list(layer.buffers()))


def _prepare(layer, device):
    """Folded / packed parameters of the layer on `device`, rebuilt when the layer's tensors have changed since they
    were derived (the plain forward reads live parameters, so the fast one must not run on stale copies)."""
    st = getattr(layer, _FAST_ATTR, None)
    fp = parameter_fingerprint(layer)
    if st is None or st['device'] != device or st['fingerprint'] != fp:
        st = {'device': device, 'fingerprint': fp,
              'branches': [_BranchParams(layer.convs[i], layer.fc[i], layer.weight[i], device) for i in range(layer.n)]}
        object.__setattr__(layer, _FAST_ATTR, st)
        ops.parameters_fence(device)         # the kernels read these before they wait for the work in front of them
    return st


def _layer_args(layer, st, dtype, H, W):
    """ctypes argument block of kad_kadconv_forward for this layer, activation dtype and map size (built once, then reused)."""
    import ctypes
    from . import _abi
    key = ('args', dtype, H, W)
    if key not in st:
        a = _abi.KadLayerArgs()
        tc_mask = 0
        keep = []
        for i, br in enumerate(st['branches']):
            p = a.br[i]
            path, w = br.dsc_weight(dtype, H >> i, W >> i)
            fields = dict(w_proj=br.w_proj, b_proj=br.b_proj, lcsa_w1=br.lcsa['w1'], lcsa_b1=br.lcsa['b1'], lcsa_bn_scale=br.lcsa['bn_m'],
                          lcsa_bn_shift=br.lcsa['bn_a'], lcsa_w2=br.lcsa['w2'], lcsa_b2=br.lcsa['b2'], lcsa_w3=br.lcsa['w3'], lcsa_b3=br.lcsa['b3'],
                          w_off=br.w_off, b_off=br.b_off, w_dsc_simt=br.w_dsc_simt, ep_scale=br.ep_scale, ep_shift=br.ep_shift,
                          ep_post=br.ep_post, fc_w1=br.fc_w1, fc_b1=br.fc_b1, fc_w2=br.fc_w2, fc_b2=br.fc_b2)
            for name, t in fields.items():
                setattr(p, name, t.data_ptr())
            if path == ops.PATH_TC:
                p.w_dsc_tc = w.data_ptr(); keep.append(w); tc_mask |= 1 << i
            if path == ops.PATH_MMA:
                p.w_dsc_mma = br.w_dsc_mma[dtype].data_ptr()
            p.c, p.hidden = br.c, br.fc_w1.shape[0]
        a.dtype = ops._DT[dtype]
        # per branch: project, 2 LCSA sums, 2 LCSA mask, offset conv (unless fused), DSC, SE (unless inside the merge); + merge
        dim = sum(br.c for br in st['branches'])
        launches = 25 - sum(1 for i, br in enumerate(st['branches']) if br.dsc_weight(dtype, H >> i, W >> i)[0] == ops.PATH_MMA)
        if dtype != torch.float32 and dim % 8 == 0:
            launches -= 3
        if ops.pyramid_project_supported(dim, [br.c for br in st['branches']], dtype, H, W):
            launches -= 2
            if all(ops.lcsa_mask_from_partials_supported(H >> i, W >> i, br.c) for i, br in enumerate(st['branches'])):
                launches -= 6      # row/column sums come out of the pyramid kernel
        st[key] = (a, tc_mask, keep, launches)
        ops.parameters_fence(st['device'])   # packed deformable-convolution weights may have just been produced
        a.counters = ops.layer_counters(st['device']).data_ptr()
    return st[key]


def kadconv_forward_nhwc(layer, x, out=None, out_coff=0):
    """The accelerated KADConv forward on a contiguous NHWC tensor; returns NHWC. One C-ABI call per layer
    (kad_kadconv_forward): the three branches run on three streams and all intermediates live in one workspace.
    With `out` ([B,H,W,Cy], contiguous) the result is written into its channels [out_coff, out_coff + C) in place."""
    import ctypes
    from . import _abi
    if layer.n != 3:
        raise RuntimeError('the B200 pipeline implements the 3-branch KAD-Conv (n=3)')
    x = ops._cuda(x, 'x')
    B, H, W, C = x.shape
    if H < 4 or W < 4:
        raise RuntimeError(f'KAD-Conv needs H, W >= 4 for its 1/4-resolution branch, got {H}x{W}')
    st = _prepare(layer, x.device)
    a, tc_mask, _, launches = _layer_args(layer, st, x.dtype, H, W)
    lib = _abi.load()
    nbytes = lib.kad_kadconv_workspace_bytes(B, H, W, C, a.dtype, tc_mask)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    if out is None:
        out = torch.empty_like(x)
        out_ptr, a.out_cstride = out.data_ptr(), 0
    else:
        if out.shape[:3] != x.shape[:3] or out.dtype != x.dtype or not out.is_contiguous() or out_coff + C > out.shape[3]:
            raise ValueError('out must be a contiguous [B,H,W,Cy] tensor of the same dtype with room for C channels at out_coff')
        out_ptr, a.out_cstride = out.data_ptr() + out_coff * out.element_size(), out.shape[3]
    a.x, a.out, a.workspace, a.workspace_bytes = x.data_ptr(), out_ptr, ws.data_ptr(), nbytes
    a.status = ops.status_word(x.device).data_ptr()
    a.B, a.H, a.W, a.dim = B, H, W, C
    a.scheme = LAYER_SCHEME
    launches = lib.kad_kadconv_launch_count(B, H, W, C, a.dtype, tc_mask, 1, a.scheme)
    _abi.check(lib.kad_kadconv_forward(ctypes.byref(a), ops._stream()), 'kad_kadconv_forward', launches)
    return out


def kadconv_forward_nhwc_stepwise(layer, x):
    """The same computation issued kernel by kernel from Python on the current stream (kept for tests that
    look at intermediate tensors)."""
    B, H, W, C = x.shape
    st = _prepare(layer, x.device)
    ys, atts = [], []
    brs = st['branches']
    pyramid = ops.pyramid_project_supported(C, [br.c for br in brs], x.dtype, H, W)
    partials = pyramid and all(ops.lcsa_mask_from_partials_supported(H >> i, W >> i, br.c) for i, br in enumerate(brs))
    ts, parts = None, None
    if pyramid:
        ts = ops.pyramid_project(x, [br.w_proj for br in brs], [br.b_proj for br in brs], want_partials=partials)
        if partials:
            ts, parts = ts
    for i, br in enumerate(brs):
        t = ts[i] if pyramid else ops.pool_project(x, br.w_proj, br.b_proj, pool=2 ** i)
        if partials:
            mask = ops.lcsa_mask_from_partials(parts[i][0], parts[i][1], br.lcsa, t.dtype, mask_f32=True)
        else:
            mask = ops.lcsa_mask(t, br.lcsa, mask_f32=True)
        path, w = br.dsc_weight(t.dtype, t.shape[1], t.shape[2])
        if path == ops.PATH_MMA:      # the offset convolution runs inside the DSC kernel
            y, gap = ops.dsc_forward(t, w, None, mask, scale=br.ep_scale, shift=br.ep_shift, post=br.ep_post, act=ops.ACT_RELU,
                                     path=path, want_gap=True, offset_weight=br.w_off, offset_bias=br.b_off)
        else:
            off_path = ops.PATH_MMA if ops.dsc_mma_supported(br.c, 18, t.dtype, t.shape[1], t.shape[2]) else ops.PATH_SIMT
            offset = ops.dsc_forward(t, br.w_off, shift=br.b_off, y_f32=True, path=off_path)
            y, gap = ops.dsc_forward(t, w, offset, mask, scale=br.ep_scale, shift=br.ep_shift, post=br.ep_post,
                                     act=ops.ACT_RELU, path=path, want_gap=True, cout=br.c)
        atts.append(ops.se_excite(gap, t.shape[1] * t.shape[2], br.fc_w1, br.fc_b1, br.fc_w2, br.fc_b2))
        ys.append(y)
    return ops.merge_upsample_residual(x, ys, atts)


def _fast_forward(layer, x):
    if layer.training:
        raise RuntimeError('kadconv fast inference is enabled: call model.eval() (or disable_fast_inference for training)')
    if not x.is_cuda:
        raise RuntimeError('kadconv fast inference has no CPU path: move the input to the GPU')
    if x.dim() != 4:
        raise ValueError('KADConv expects a [B,C,H,W] tensor')
    channels_last = x.permute(0, 2, 3, 1).is_contiguous()
    capturing = torch.cuda.is_current_stream_capturing()
    if not capturing:
        ops.status_poll(x.device)        # a tensor-core kernel of an earlier call that gave up on a wait raises here
    out = kadconv_forward_nhwc(layer, ops.to_nhwc(x))
    if not capturing:
        ops.status_snapshot(x.device)
    if channels_last:
        return out.permute(0, 3, 1, 2)      # same logical shape, channels_last memory like the input
    return ops.to_nchw(out)


def enable_fast_inference(model, build_dir=None, allow_untested_gpu=False):
    """Switch every KAD-Conv layer in ``model`` to the B200 CUDA pipeline (in place); returns ``model``.

    ``build_dir`` and ``allow_untested_gpu`` are accepted for call compatibility with the reference; the
    library is prebuilt in-tree and targets sm_100a only.
    """
    from . import _abi
    _abi.load()
    if model.training:
        raise ValueError('call model.eval() before enable_fast_inference()')
    device = next(model.parameters()).device
    if device.type != 'cuda':
        raise ValueError('move the model to a CUDA device first')
    if torch.cuda.get_device_capability(device)[0] != 10:
        raise ValueError('the kadconv_b200 kernels are built for sm_100a (B200) only')
    layers = [m for m in model.modules() if type(m).__name__ in _LAYER_TYPES]
    if not layers:
        raise ValueError('no KAD-Conv layer found in the model')
    for layer in layers:
        _prepare(layer, device)
        layer.forward = types.MethodType(_fast_forward, layer)
    return model


def disable_fast_inference(model):
    """Go back to the plain PyTorch forward."""
    for m in model.modules():
        if type(m).__name__ in _LAYER_TYPES:
            if 'forward' in vars(m):
                del m.forward
            if _FAST_ATTR in vars(m):
                object.__delattr__(m, _FAST_ATTR)
    return model
