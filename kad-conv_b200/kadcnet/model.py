"""KAD-CNet-S as plain PyTorch modules with the reference's attribute names and state_dict keys.

Mirrors, for the inference path only, the classes of the reference project:
  Conv / AConv / ELAN1 / SPPELAN / SP / Concat / DFL   KAD-CNet/models/common.py:43-67, :187-193, :232-243, :535-598
  KADC4 / KADC4_m / RepNCSP_KADC / RepNCSPELAN4_KADC   KAD-CNet/models/module/KADC/module.py:14-111
  DDetect                                              KAD-CNet/models/yolo.py:78-136
  DetectionModel (graph of configs/dior_s_base.yaml / dior_s_mgl.yaml, fuse())   KAD-CNet/models/yolo.py:574-664, :744-813
A checkpoint's state_dict from the reference loads into DetectionModel here (keys 'model.{i}....').
This file is the module definition; the B200 execution of it lives in kadcnet.engine.
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from kadconv.kad_conv import KADConv

BN_EPS, BN_MOMENTUM = 1e-3, 0.03      # set on every BatchNorm2d by the reference's initialize_weights


def make_divisible(x, divisor):
    return math.ceil(x / divisor) * divisor


def _bn(c):
    return nn.BatchNorm2d(c, eps=BN_EPS, momentum=BN_MOMENTUM)


class Conv(nn.Module):
    """conv (no bias) + BatchNorm + SiLU; after fuse() the BN is folded and ``bn`` is removed."""

    def __init__(self, c1, c2, k=1, s=1, p=None, g=1, act=True):
        super().__init__()
        self.conv = nn.Conv2d(c1, c2, k, s, k // 2 if p is None else p, groups=g, bias=False)
        self.bn = _bn(c2)
        self.act = nn.SiLU() if act is True else nn.Identity()

    def forward(self, x):
        y = self.conv(x)
        if hasattr(self, 'bn'):
            y = self.bn(y)
        return self.act(y)

    def fuse(self):
        if not hasattr(self, 'bn'):
            return self
        bn, conv = self.bn, self.conv
        fused = nn.Conv2d(conv.in_channels, conv.out_channels, conv.kernel_size, conv.stride, conv.padding,
                          groups=conv.groups, bias=True).requires_grad_(False).to(conv.weight.device)
        with torch.no_grad():
            m = bn.weight / torch.sqrt(bn.running_var + bn.eps)
            fused.weight.copy_(conv.weight * m.view(-1, 1, 1, 1))
            fused.bias.copy_(bn.bias - bn.running_mean * m)
        self.conv = fused
        del self.bn
        return self


class AConv(nn.Module):
    def __init__(self, c1, c2):
        super().__init__()
        self.cv1 = Conv(c1, c2, 3, 2, 1)

    def forward(self, x):
        return self.cv1(F.avg_pool2d(x, 2, 1, 0, False, True))


class ELAN1(nn.Module):
    def __init__(self, c1, c2, c3, c4):
        super().__init__()
        self.c = c3 // 2
        self.cv1 = Conv(c1, c3, 1, 1)
        self.cv2 = Conv(c3 // 2, c4, 3, 1)
        self.cv3 = Conv(c4, c4, 3, 1)
        self.cv4 = Conv(c3 + 2 * c4, c2, 1, 1)

    def forward(self, x):
        y = list(self.cv1(x).chunk(2, 1))
        y.extend(m(y[-1]) for m in (self.cv2, self.cv3))
        return self.cv4(torch.cat(y, 1))


class SP(nn.Module):
    def __init__(self, k=3, s=1):
        super().__init__()
        self.m = nn.MaxPool2d(kernel_size=k, stride=s, padding=k // 2)

    def forward(self, x):
        return self.m(x)


class SPPELAN(nn.Module):
    def __init__(self, c1, c2, c3):
        super().__init__()
        self.c = c3
        self.cv1 = Conv(c1, c3, 1, 1)
        self.cv2, self.cv3, self.cv4 = SP(5), SP(5), SP(5)
        self.cv5 = Conv(4 * c3, c2, 1, 1)

    def forward(self, x):
        y = [self.cv1(x)]
        y.extend(m(y[-1]) for m in (self.cv2, self.cv3, self.cv4))
        return self.cv5(torch.cat(y, 1))


class KADC4(KADConv):
    """KAD-Conv inside the detector (SE hidden width at least 32)."""
    se_min_hidden = 32

    def __init__(self, dim, n=3):
        super().__init__(dim, n=n, se_min_hidden=type(self).se_min_hidden)


class KADC4_m(KADC4):
    """Variant used by the MGL-trained checkpoint (SE hidden width at least 64)."""
    se_min_hidden = 64


KAD_CONV_VARIANTS = {'KADC4': KADC4, 'KADC4_m': KADC4_m}


class RepNCSP_KADC(nn.Module):
    def __init__(self, c1, c2, n=1, e=0.5, kadc_variant=None):
        super().__init__()
        c_ = int(c2 * e)
        self.cv1 = Conv(c1, c_, 1, 1)
        self.cv2 = Conv(c1, c_, 1, 1)
        self.cv3 = Conv(2 * c_, c2, 1)
        block = KAD_CONV_VARIANTS[kadc_variant] if isinstance(kadc_variant, str) else (kadc_variant or KADC4)
        self.m = nn.Sequential(*(block(c_) for _ in range(n)))

    def forward(self, x):
        return self.cv3(torch.cat((self.m(self.cv1(x)), self.cv2(x)), 1))


class RepNCSPELAN4_KADC(nn.Module):
    def __init__(self, c1, c2, c3, c4, c5=1, kadc_variant=None):
        super().__init__()
        self.c = c3 // 2
        self.cv1 = Conv(c1, c3, 1, 1)
        self.cv2 = nn.Sequential(RepNCSP_KADC(c3 // 2, c4, c5, kadc_variant=kadc_variant), Conv(c4, c4, 3, 1))
        self.cv3 = nn.Sequential(RepNCSP_KADC(c4, c4, c5, kadc_variant=kadc_variant), Conv(c4, c4, 3, 1))
        self.cv4 = Conv(c3 + 2 * c4, c2, 1, 1)

    def forward(self, x):
        y = list(self.cv1(x).chunk(2, 1))
        y.extend(m(y[-1]) for m in (self.cv2, self.cv3))
        return self.cv4(torch.cat(y, 1))


class Concat(nn.Module):
    def __init__(self, dimension=1):
        super().__init__()
        self.d = dimension

    def forward(self, x):
        return torch.cat(x, self.d)


class DFL(nn.Module):
    def __init__(self, c1=16):
        super().__init__()
        self.conv = nn.Conv2d(c1, 1, 1, bias=False).requires_grad_(False)
        self.conv.weight.data[:] = torch.arange(c1, dtype=torch.float).view(1, c1, 1, 1)
        self.c1 = c1

    def forward(self, x):
        b, _, a = x.shape
        return self.conv(x.view(b, 4, self.c1, a).transpose(2, 1).softmax(1)).view(b, 4, a)


def make_anchors(feats, strides, offset=0.5):
    pts, st = [], []
    dtype, device = feats[0].dtype, feats[0].device
    for f, s in zip(feats, strides):
        h, w = f.shape[2:]
        sx = torch.arange(end=w, device=device, dtype=dtype) + offset
        sy = torch.arange(end=h, device=device, dtype=dtype) + offset
        sy, sx = torch.meshgrid(sy, sx, indexing='ij')
        pts.append(torch.stack((sx, sy), -1).view(-1, 2))
        st.append(torch.full((h * w, 1), float(s), dtype=dtype, device=device))
    return torch.cat(pts), torch.cat(st)


class DDetect(nn.Module):
    def __init__(self, nc=80, ch=()):
        super().__init__()
        self.nc, self.nl, self.reg_max = nc, len(ch), 16
        self.no = nc + 4 * self.reg_max
        self.stride = torch.zeros(self.nl)
        c2 = make_divisible(max(ch[0] // 4, self.reg_max * 4, 16), 4)
        c3 = max(ch[0], min(nc * 2, 128))
        self.cv2 = nn.ModuleList(nn.Sequential(Conv(x, c2, 3), Conv(c2, c2, 3, g=4), nn.Conv2d(c2, 4 * self.reg_max, 1, groups=4)) for x in ch)
        self.cv3 = nn.ModuleList(nn.Sequential(Conv(x, c3, 3), Conv(c3, c3, 3), nn.Conv2d(c3, nc, 1)) for x in ch)
        self.dfl = DFL(self.reg_max)
        self.shape, self.anchors, self.strides = None, torch.empty(0), torch.empty(0)

    def forward(self, x):
        x = list(x)
        shape = x[0].shape
        for i in range(self.nl):
            x[i] = torch.cat((self.cv2[i](x[i]), self.cv3[i](x[i])), 1)
        if self.training:
            return x
        if self.shape != shape or self.anchors.device != x[0].device or self.anchors.dtype != x[0].dtype:
            self.anchors, self.strides = (t.transpose(0, 1) for t in make_anchors(x, self.stride, 0.5))
            self.shape = shape
        box, cls = torch.cat([xi.view(shape[0], self.no, -1) for xi in x], 2).split((4 * self.reg_max, self.nc), 1)
        d = self.dfl(box)
        lt, rb = d.split(2, 1)
        a = self.anchors.unsqueeze(0)
        x1y1, x2y2 = a - lt, a + rb
        dbox = torch.cat(((x1y1 + x2y2) / 2, x2y2 - x1y1), 1) * self.strides
        return torch.cat((dbox, cls.sigmoid()), 1), x

    def bias_init(self):
        for a, b, s in zip(self.cv2, self.cv3, self.stride):
            a[-1].bias.data[:] = 1.0
            b[-1].bias.data[:self.nc] = math.log(5 / self.nc / (640 / float(s)) ** 2)


def s_config(variant='KADC4', nc=20, width=1.1):
    """The KAD-CNet-S graph: rows of (from, module name, args), channel counts before the width multiple."""
    k = {'kadc_variant': variant}
    rows = [
        (-1, 'Conv', [32, 3, 2]), (-1, 'Conv', [64, 3, 2]), (-1, 'ELAN1', [64, 64, 32]),
        (-1, 'AConv', [128]), (-1, 'RepNCSPELAN4_KADC', [128, 128, 64, 3]),
        (-1, 'AConv', [192]), (-1, 'RepNCSPELAN4_KADC', [192, 192, 96, 3]),
        (-1, 'AConv', [256]), (-1, 'RepNCSPELAN4_KADC', [256, 256, 128, 3]),
        (-1, 'SPPELAN', [256, 128]),
        (-1, 'nn.Upsample', [None, 2, 'nearest']), ([-1, 6], 'Concat', [1]), (-1, 'RepNCSPELAN4_KADC', [192, 192, 96, 3]),
        (-1, 'nn.Upsample', [None, 2, 'nearest']), ([-1, 4], 'Concat', [1]), (-1, 'RepNCSPELAN4_KADC', [128, 128, 64, 3]),
        (-1, 'AConv', [96]), ([-1, 12], 'Concat', [1]), (-1, 'RepNCSPELAN4_KADC', [192, 192, 96, 3]),
        (-1, 'AConv', [128]), ([-1, 9], 'Concat', [1]), (-1, 'RepNCSPELAN4_KADC', [256, 256, 128, 3]),
        ([15, 18, 21], 'DDetect', ['nc']),
    ]
    return {'nc': nc, 'width_multiple': width, 'depth_multiple': 1.0, 'rows': rows, 'kadc': k}


def load_yaml_config(path):
    """Reads a model YAML of the reference's schema (backbone + head lists of [from, number, module, args])."""
    import yaml
    with open(path, encoding='ascii', errors='ignore') as f:
        d = yaml.safe_load(f)
    rows = []
    for frm, _n, mod, args in d['backbone'] + d['head']:
        args = list(args)
        kw = {}
        if args and isinstance(args[-1], dict):
            kw = args.pop()
        rows.append((frm, mod, args, kw))
    variant = None
    out_rows = []
    for frm, mod, args, kw in rows:
        if 'kadc_variant' in kw:
            variant = kw['kadc_variant']
        if mod == 'RepNCSPELAN4_KADC' and len(args) > 4:
            variant = args[4]
            args = args[:4]
        out_rows.append((frm, mod, args))
    return {'nc': d['nc'], 'width_multiple': d['width_multiple'], 'depth_multiple': d.get('depth_multiple', 1.0),
            'rows': out_rows, 'kadc': {'kadc_variant': variant or 'KADC4'}}


_SCALED = {'Conv', 'AConv', 'ELAN1', 'SPPELAN', 'RepNCSPELAN4_KADC'}


class DetectionModel(nn.Module):
    """KAD-CNet detector built from a graph description; forward(x) -> (y[B,4+nc,A], [raw P3,P4,P5]) in eval mode."""

    def __init__(self, cfg=None, ch=3, nc=None):
        super().__init__()
        if cfg is None:
            cfg = s_config()
        elif isinstance(cfg, str) or hasattr(cfg, '__fspath__'):
            cfg = load_yaml_config(cfg)
        if nc:
            cfg = dict(cfg, nc=nc)
        self.cfg = cfg
        gw = cfg['width_multiple']
        layers, chans, save = [], [], set()
        c_prev = ch
        for i, (frm, mod, args) in enumerate(cfg['rows']):
            args = [cfg['nc'] if a == 'nc' else a for a in args]
            c_in = c_prev if frm == -1 else (chans[frm] if isinstance(frm, int) else None)
            if mod in _SCALED:
                c2 = make_divisible(args[0] * gw, 8)
                rest = args[1:]
                if mod == 'Conv':
                    m = Conv(c_in, c2, *rest)
                elif mod == 'AConv':
                    m = AConv(c_in, c2)
                elif mod == 'ELAN1':
                    m = ELAN1(c_in, c2, *rest)
                elif mod == 'SPPELAN':
                    m = SPPELAN(c_in, c2, *rest)
                else:
                    m = RepNCSPELAN4_KADC(c_in, c2, *rest, **cfg['kadc'])
            elif mod == 'nn.Upsample':
                m, c2 = nn.Upsample(None, args[1], args[2]), c_in
            elif mod == 'Concat':
                m, c2 = Concat(args[0]), sum(c_prev if j == -1 else chans[j] for j in frm)
            elif mod == 'DDetect':
                m, c2 = DDetect(args[0], [chans[j] for j in frm]), None
            else:
                raise ValueError(f'module {mod} is not part of the KAD-CNet-S inference graph')
            m.i, m.f, m.type = i, frm, mod
            save.update(j % i for j in ([frm] if isinstance(frm, int) else frm) if j != -1)
            layers.append(m)
            chans.append(c2)
            c_prev = c2
        self.model = nn.Sequential(*layers)
        self.save = sorted(save)
        self.names = [str(i) for i in range(cfg['nc'])]
        head = self.model[-1]
        # strides are a property of the graph: discover them with a 256x256 dummy forward, as the reference does
        s = 256
        self.eval()
        with torch.no_grad():
            head.training = True
            feats = self._forward_once(torch.zeros(1, ch, s, s))
            head.training = False
        head.stride = torch.tensor([s / f.shape[-2] for f in feats])
        self.stride = head.stride
        head.bias_init()
        self.train()

    def _forward_once(self, x):
        ys = []
        for m in self.model:
            if m.f != -1:
                x = ys[m.f] if isinstance(m.f, int) else [x if j == -1 else ys[j] for j in m.f]
            x = m(x)
            ys.append(x if m.i in self.save else None)
        return x

    def forward(self, x):
        return self._forward_once(x)

    def fuse(self):
        for m in self.modules():
            if isinstance(m, Conv):
                m.fuse()
        return self

    def _apply(self, fn):
        super()._apply(fn)
        head = self.model[-1]
        head.stride = fn(head.stride)
        head.anchors = fn(head.anchors)
        head.strides = fn(head.strides)
        return self
