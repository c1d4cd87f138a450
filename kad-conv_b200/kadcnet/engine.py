"""B200 execution of KAD-CNet-S: NHWC, fp16/bf16, KAD-Conv layers and 1x1 convolutions on the
kadconv_b200 CUDA kernels.

The engine walks the same graph as kadcnet.model.DetectionModel (which mirrors the reference's
DetectionModel._forward_once, KAD-CNet/models/yolo.py:538-559) but keeps every activation as a
contiguous [B,H,W,C] tensor:
  * every KAD-Conv layer (42 in KAD-CNet-S)  -> kadconv.fast.kadconv_forward_nhwc (CUDA pipeline)
  * every Conv with k = 1 (+ folded BN + SiLU) -> tcgen05 GEMM + bias + SiLU, reading channel slices in
    place (the ELAN / CSP `chunk` never copies)
  * 3x3 convolutions, pools, nearest upsampling -> library kernels on channels_last views (outside the
    KAD-Conv hot path; they are the next item to be replaced)
  * head decode -> one kernel per scale (softmax expectation, box, sigmoid) in fp32 with one rounding at the store.
There is no CPU path: the engine raises on a non-CUDA input.

Error reporting: the tcgen05 kernels bound every wait; one that gives up records that in a device status word and its
results are not valid. FastDetector.forward and StaticGraph.__call__ look at that word without synchronising (a snapshot
taken after each call is examined at the next one), non_max_suppression_device and DetectionPipeline read it together with
their results, and kadconv.ops.check_status(device) checks it at once (it synchronises).
"""
import torch
import torch.nn.functional as F

from kadconv import ops
from kadconv.fast import kadconv_forward_nhwc

from . import model as M


def _nchw_view(t):
    """[B,H,W,C] contiguous -> logical [B,C,H,W] view (channels_last strides), no copy."""
    return t.permute(0, 3, 1, 2)


def _nhwc(t):
    """logical [B,C,H,W] tensor in channels_last memory -> [B,H,W,C] contiguous view (copy only if needed)."""
    v = t.permute(0, 2, 3, 1)
    return v if v.is_contiguous() else v.contiguous()


class _Conv1x1:
    def __init__(self, conv_mod, dtype, device):
        conv = conv_mod.conv
        assert conv.kernel_size == (1, 1) and conv.groups == 1 and conv.bias is not None, 'fuse() the model first'
        self.n, self.k = conv.out_channels, conv.in_channels
        self.act = ops.ACT_SILU if isinstance(conv_mod.act, torch.nn.SiLU) else ops.ACT_NONE
        w = conv.weight.detach().float().view(self.n, self.k)
        self.bias = conv.bias.detach().float().contiguous().to(device)
        self.tc = ops.gemm1x1_supported(self.k, self.n, dtype)
        self.w = (w.to(dtype) if self.tc else w).contiguous().to(device)

    def __call__(self, x, in_coff=0, cx=None, out=None, out_coff=0):
        """x [B,H,W,Cx]; reads channels [in_coff, in_coff+k)."""
        if self.tc and (in_coff * x.element_size()) % 16 == 0:
            src = x if in_coff == 0 else x.view(-1)[in_coff:]
            return ops.gemm1x1_bias_act_raw(src, x.shape, self.w, self.bias, self.act, self.k, out, out_coff)
        xs = x[..., in_coff:in_coff + self.k].contiguous() if (in_coff or x.shape[-1] != self.k) else x
        return ops.pool_project(xs, self.w.float(), self.bias, pool=1, act=self.act, out=out, out_coff=out_coff)


class _ConvKxK:
    """3x3 convolution + bias + SiLU. Default: the library convolution on a channels_last view without bias, then one
    kadconv kernel for bias + SiLU (it lands the result in a channel slice of a concatenation). With `own=True`
    (FastDetector(conv3x3='tcgen05')) and padding 1, stride 1 or 2, channel counts that are multiples of 8: this
    package's tcgen05 implicit GEMM (grouped convolutions as the equivalent dense one), which reads and writes channel
    slices in place; it is bit-for-bit deterministic and parity-tested, but at the detector's narrow widths (32-288
    channels) it is still slower than the library's kernels, so it is not the default. `cin_pad` zero-pads the input
    channels of the weight (a float image is padded from 3 to 8 channels)."""

    def __init__(self, conv_mod, dtype, device, cin_pad=None, own=False):
        conv = conv_mod.conv if hasattr(conv_mod, 'conv') else conv_mod
        w = conv.weight.detach().to(device, dtype)
        if cin_pad is not None and cin_pad > w.shape[1]:
            w = F.pad(w, (0, 0, 0, 0, 0, cin_pad - w.shape[1]))
        self.b = conv.bias.detach().float().contiguous().to(device)
        self.stride, self.padding, self.groups = conv.stride, conv.padding, conv.groups
        self.act = ops.ACT_SILU if (hasattr(conv_mod, 'act') and isinstance(conv_mod.act, torch.nn.SiLU)) else ops.ACT_NONE
        cin = w.shape[1] * conv.groups
        self.own = (own and conv.kernel_size == (3, 3) and conv.padding == (1, 1) and conv.dilation == (1, 1) and conv.stride in ((1, 1), (2, 2))
                    and conv.groups <= 8 and ops.conv3x3_supported(cin, conv.out_channels, conv.stride[0], dtype))
        if self.own:
            self.w = ops.pack_conv3x3_weight(w, dtype, groups=conv.groups).to(device)
            self.cin = cin
        else:
            self.w = w.contiguous(memory_format=torch.channels_last)

    def __call__(self, x, out=None, out_coff=0, in_coff=0):
        if self.own:
            if out is not None and (out.shape[-1] % 8 or out_coff % 8):       # the kernel stores 16-byte vectors: rows must stay aligned
                y = ops.conv3x3_bias_act(x, self.w, self.b, act=self.act, stride=self.stride[0], in_coff=in_coff, cin=self.cin)
                out[..., out_coff:out_coff + y.shape[-1]].copy_(y)
                return out
            return ops.conv3x3_bias_act(x, self.w, self.b, act=self.act, stride=self.stride[0], in_coff=in_coff, cin=self.cin,
                                        out=out, out_coff=out_coff)
        if in_coff or x.shape[-1] != self.w.shape[1] * self.groups:
            x = ops.copy_channels(x, in_coff, self.w.shape[1] * self.groups)
        y = _nhwc(F.conv2d(_nchw_view(x), self.w, None, self.stride, self.padding, 1, self.groups))
        if out is None:
            return ops.bias_act_(y, self.b, self.act)
        return ops.bias_act_to(y, self.b, out, out_coff, self.act)    # lands in its slice of a concatenation


def _conv(conv_mod, dtype, device, own3x3=False):
    k = conv_mod.conv.kernel_size
    if k == (1, 1) and conv_mod.conv.groups == 1:
        return _Conv1x1(conv_mod, dtype, device)
    return _ConvKxK(conv_mod, dtype, device, own=own3x3)


class FastDetector(torch.nn.Module):
    """Callable with the model's signature: forward(x[B,3,H,W]) -> (y[B,4+nc,A], [raw P3,P4,P5] as NCHW views)."""

    def __init__(self, model, dtype=torch.float16, conv3x3='library'):
        """conv3x3: 'library' (cuDNN through torch, the faster choice at this model's widths) or 'tcgen05' (this
        package's implicit-GEMM kernel for every 3x3 convolution with padding 1 and stride 1 or 2)."""
        super().__init__()
        if conv3x3 not in ('library', 'tcgen05'):
            raise ValueError("conv3x3 must be 'library' or 'tcgen05'")
        self.own3x3 = conv3x3 == 'tcgen05'
        if any(hasattr(m, 'bn') for m in model.modules() if isinstance(m, M.Conv)):
            raise ValueError('call model.fuse() first: the engine runs the Conv+BN-folded model')
        if model.training:
            raise ValueError('call model.eval() first')
        device = next(model.parameters()).device
        if device.type != 'cuda':
            raise ValueError('move the model to a CUDA device first (there is no CPU path)')
        self.model, self.dtype, self.device = model, dtype, device
        self.stride = model.stride
        self._fused_up = set()
        self.plan = [self._compile(m) for m in model.model]
        ops.parameters_fence(device)         # converted weights and biases: see kadconv.ops.parameters_fence
        # raw uint8 images: the first layer (3x3, stride 2) runs as one kernel that also normalises and changes layout
        self.stem = None
        first = model.model[0]
        if isinstance(first, M.Conv):
            cv = first.conv
            if (cv.kernel_size == (3, 3) and cv.stride == (2, 2) and cv.padding == (1, 1) and cv.groups == 1 and cv.dilation == (1, 1)
                    and ops.stem_conv_supported(cv.in_channels, cv.out_channels, dtype)):
                act = ops.ACT_SILU if isinstance(first.act, torch.nn.SiLU) else (ops.ACT_NONE if isinstance(first.act, torch.nn.Identity) else None)
                if act is not None:
                    self.stem = (cv.weight.detach().float().contiguous().to(device), cv.bias.detach().float().contiguous().to(device), act)

    # ---- per-module closures -------------------------------------------------------------------
    def _compile(self, m):
        dt, dev = self.dtype, self.device
        if isinstance(m, M.Conv):
            c = _ConvKxK(m, dt, dev, cin_pad=8) if (m.i == 0 and m.conv.in_channels < 8 and m.conv.kernel_size != (1, 1)) else _conv(m, dt, dev, self.own3x3)
            return lambda x: c(x)
        if isinstance(m, M.AConv):
            c = _ConvKxK(m.cv1, dt, dev, own=self.own3x3)
            return lambda x: c(ops.avg_pool2x2s1(x))
        if isinstance(m, M.ELAN1):
            cv1, cv2, cv3, cv4 = (_conv(t, dt, dev, self.own3x3) for t in (m.cv1, m.cv2, m.cv3, m.cv4))
            half = m.c

            widths = (m.cv1.conv.out_channels, m.cv2.conv.out_channels, m.cv3.conv.out_channels)

            def elan(x):
                cat = torch.empty(x.shape[:3] + (sum(widths),), dtype=x.dtype, device=x.device)
                cv1(x, out=cat, out_coff=0)
                if isinstance(cv2, _ConvKxK) and isinstance(cv3, _ConvKxK) and cv2.own and cv3.own:
                    # the 3x3 convolutions read their input slice of the concatenation and write their own slice
                    cv2(cat, in_coff=half, out=cat, out_coff=widths[0])
                    cv3(cat, in_coff=widths[0], out=cat, out_coff=widths[0] + widths[1])
                else:
                    # the library convolution wants a dense input: one vectorised slice copy each way
                    y2 = cv2(ops.copy_channels(cat, half, widths[0] - half))
                    ops.copy_channels(y2, 0, widths[1], cat, widths[0])
                    cv3(y2, out=cat, out_coff=widths[0] + widths[1])
                return cv4(cat)
            return elan
        if isinstance(m, M.RepNCSPELAN4_KADC):
            cv1, cv4 = _conv(m.cv1, dt, dev, self.own3x3), _conv(m.cv4, dt, dev, self.own3x3)
            b2, c2 = self._csp(m.cv2[0]), _conv(m.cv2[1], dt, dev, self.own3x3)
            b3, c3 = self._csp(m.cv3[0]), _conv(m.cv3[1], dt, dev, self.own3x3)
            half = m.c

            wt, w2, w3 = m.cv1.conv.out_channels, m.cv2[1].conv.out_channels, m.cv3[1].conv.out_channels

            def gelan(x):
                # every producer writes its slice of the concatenation; the CSP blocks read their input as a slice of it
                cat = torch.empty(x.shape[:3] + (wt + w2 + w3,), dtype=x.dtype, device=x.device)
                cv1(x, out=cat, out_coff=0)
                c2(b2(cat, half, wt - half), out=cat, out_coff=wt)
                c3(b3(cat, wt, w2), out=cat, out_coff=wt + w2)
                return cv4(cat)
            return gelan
        if isinstance(m, M.SPPELAN):
            cv1, cv5 = _conv(m.cv1, dt, dev, self.own3x3), _conv(m.cv5, dt, dev, self.own3x3)

            c3 = m.cv1.conv.out_channels
            five = all(getattr(sp.m, 'kernel_size', None) == 5 and sp.m.stride == 1 and sp.m.padding == 2 for sp in (m.cv2, m.cv3, m.cv4))

            def spp(x):
                B, H, W, _ = x.shape
                if five and ops.spp_pool3_supported(H, W, c3, x.dtype):
                    # cv1 lands in the first quarter of the concatenation, one kernel fills the other three with the pooling chain
                    cat = torch.empty((B, H, W, 4 * c3), dtype=x.dtype, device=x.device)
                    cv1(x, out=cat, out_coff=0)
                    return cv5(ops.spp_pool3_(cat, c3))
                ys = [cv1(x)]
                for sp in (m.cv2, m.cv3, m.cv4):
                    ys.append(_nhwc(sp.m(_nchw_view(ys[-1]))))
                return cv5(torch.cat(ys, -1))
            return spp
        if isinstance(m, torch.nn.Upsample):
            nxt = self.model.model[m.i + 1] if m.i + 1 < len(self.model.model) else None
            if (isinstance(nxt, M.Concat) and isinstance(nxt.f, (list, tuple)) and len(nxt.f) == 2 and nxt.f[0] == -1
                    and m.i not in self.model.save and float(m.scale_factor) == 2.0 and m.mode == 'nearest'):
                self._fused_up.add(m.i + 1)
                return lambda x: x           # the Concat that follows upsamples and concatenates in one kernel

            def up(x):
                B, H, W, C = x.shape
                return x.view(B, H, 1, W, 1, C).expand(B, H, 2, W, 2, C).reshape(B, 2 * H, 2 * W, C)
            return up
        if isinstance(m, M.Concat):
            if m.i in self._fused_up:
                return lambda xs: ops.upsample2x_concat(xs[0], xs[1])
            return lambda xs: torch.cat(xs, -1)
        if isinstance(m, M.DDetect):
            return self._head(m)
        raise TypeError(f'no B200 execution for {type(m).__name__}')

    def _csp(self, m):
        """RepNCSP_KADC: cv3(cat(KADConv x n (cv1(x)), cv2(x))); x is read as a channel slice in place."""
        dt, dev = self.dtype, self.device
        cv1, cv2, cv3 = _conv(m.cv1, dt, dev, self.own3x3), _conv(m.cv2, dt, dev, self.own3x3), _conv(m.cv3, dt, dev, self.own3x3)
        layers = list(m.m)

        def csp(x, in_coff, cin):
            """x [B,H,W,Cx]: reads channels [in_coff, in_coff + cin)."""
            assert cin == cv1.k
            a = cv1(x, in_coff=in_coff)
            c = a.shape[-1]
            cat = torch.empty(a.shape[:-1] + (2 * c,), dtype=a.dtype, device=a.device)
            for j, layer in enumerate(layers):      # the last KAD-Conv layer writes straight into the concatenation
                a = kadconv_forward_nhwc(layer, a, out=cat if j == len(layers) - 1 else None)
            if not layers:
                cat[..., :c].copy_(a)
            cv2(x, in_coff=in_coff, out=cat, out_coff=c)
            return cv3(cat)
        return csp

    def _head(self, m):
        dt, dev = self.dtype, self.device
        box = [[_ConvKxK(s[0], dt, dev, own=self.own3x3), _ConvKxK(s[1], dt, dev, own=self.own3x3), _ConvKxK(s[2], dt, dev, own=self.own3x3)] for s in m.cv2]
        cls = [[_ConvKxK(s[0], dt, dev, own=self.own3x3), _ConvKxK(s[1], dt, dev, own=self.own3x3), _ConvKxK(s[2], dt, dev, own=self.own3x3)] for s in m.cv3]
        strides = [float(v) for v in m.stride]

        def head(feats):
            raw = []
            nb = 4 * m.reg_max
            for i, f in enumerate(feats):
                # the last convolution of each branch writes its slice of the raw map [B,H,W,no]: no concatenation pass
                r = torch.empty(f.shape[:3] + (nb + m.nc,), dtype=f.dtype, device=f.device)
                box[i][2](box[i][1](box[i][0](f)), out=r, out_coff=0)
                cls[i][2](cls[i][1](cls[i][0](f)), out=r, out_coff=nb)
                raw.append(r)
            # DFL expectation, dist2bbox and the class sigmoid of the reference's sequence (KAD-CNet/models/yolo.py:112-127)
            # in one kernel per scale, anchors in (scale, y, x) order
            y = ops.head_decode(raw, strides, m.reg_max, m.nc)
            return y, [_nchw_view(r) for r in raw]
        return head

    # ---- forward -------------------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, x):
        """x: float [B,3,H,W] in [0,1] (any float dtype), or a uint8 image batch [B,3,H,W] in [0,255], which is
        normalised by 1/255 on the way in (the `/255` of the reference's inference scripts)."""
        if not x.is_cuda:
            raise RuntimeError('FastDetector has no CPU path: move the input to the GPU')
        capturing = torch.cuda.is_current_stream_capturing()
        if not capturing:
            ops.status_poll(x.device)
        first = self.model.model[0]
        pad8 = isinstance(first, M.Conv) and first.conv.in_channels < 8 and first.conv.kernel_size != (1, 1)
        skip_first = False
        if x.dtype == torch.uint8 and self.stem is not None:
            x = ops.stem_conv_u8(x.contiguous(), self.stem[0], self.stem[1], self.dtype, act=self.stem[2])
            skip_first = True
        elif x.dtype == torch.uint8:
            x = ops.image_to_nhwc(x.contiguous(), self.dtype, cpad=8 if pad8 else x.shape[1])
        else:
            x = ops.to_nhwc(x.to(self.dtype))
            if pad8:
                x = F.pad(x, (0, 8 - x.shape[-1]))
        ys = []
        save = self.model.save
        for m, fn in zip(self.model.model, self.plan):
            if m.f != -1:
                x = ys[m.f] if isinstance(m.f, int) else [x if j == -1 else ys[j] for j in m.f]
            if not (skip_first and m.i == 0):
                x = fn(x)
            ys.append(x if m.i in save else None)
        if not capturing:
            ops.status_snapshot(self.device)
        return x
