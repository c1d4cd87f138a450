"""Plain-torch CPU restatement of the KAD-Conv operator and the KAD-CNet-S detector forward.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py). Every function works on a flat ``state_dict``
whose keys are the reference's parameter names, so the same seeded weights can be loaded into the
reference modules (to pin this file) and into the CUDA-backed modules (to check them).

Reference locations restated here (paths relative to the reference project):
  * modulated deformable convolution: the sampling rule of torchvision.ops.deform_conv2d as the
    reference restates it in KAD-CNet/inference/acceleration/kadc_dcn_direct.py:49-107
  * LCSA  KAD-Conv/kadconv/kad_conv.py:24-39   (== KAD-CNet/models/module/ops.py:20-37)
  * DSC   KAD-Conv/kadconv/kad_conv.py:63-67   (== KAD-CNet/models/module/ops.py:68-72)
  * KADConv.forward  KAD-Conv/kadconv/kad_conv.py:112-121 (== KAD-CNet/models/module/KADC/module.py:50-62)
  * Conv/AConv/ELAN1/SPPELAN  KAD-CNet/models/common.py:43-67, :563-598
  * RepNCSP_KADC / RepNCSPELAN4_KADC  KAD-CNet/models/module/KADC/module.py:74-106
  * DDetect.forward  KAD-CNet/models/yolo.py:102-127, DFL common.py:232-243,
    make_anchors / dist2bbox  KAD-CNet/utils/tal/anchor_generator.py:8-32
  * fuse_conv_and_bn  KAD-CNet/utils/torch_utils.py:244-265
  * non_max_suppression  KAD-CNet/utils/general.py:881-990 (greedy NMS restated, no torchvision)
"""
import math

import torch
import torch.nn.functional as F

BN_EPS = 1e-3  # KAD-Conv/kadconv/kad_conv.py:14; KAD-CNet/utils/torch_utils.py:208-217


# ----------------------------------------------------------------------------- operator level

def deform_conv2d(x, offset, weight, bias=None, mask=None, stride=1, padding=1):
    """Modulated deformable convolution (DCNv2), NCHW, one offset group, one weight group.

    out[b,o,y,x] = bias[o] + sum_{i,k} W[o,i,k] * mask[b,k,y,x] * bilinear(x[b,i], py, px)
    with py = y*stride - padding + ky + offset[b,2k,y,x], px likewise with offset[b,2k+1,y,x],
    k = ky*KW + kx. A sample contributes only when -1 < py < H and -1 < px < W; each of its
    four corners contributes only when it lies inside the image (zero padding).
    """
    B, C, H, W = x.shape
    O, Ci, KH, KW = weight.shape
    assert Ci == C
    Ho = (H + 2 * padding - KH) // stride + 1
    Wo = (W + 2 * padding - KW) // stride + 1
    dt = x.dtype
    ys = torch.arange(Ho, dtype=dt).view(1, Ho, 1) * stride - padding
    xs = torch.arange(Wo, dtype=dt).view(1, 1, Wo) * stride - padding
    xf = x.reshape(B, C, H * W)
    out = torch.zeros(B, O, Ho, Wo, dtype=dt)
    for ky in range(KH):
        for kx in range(KW):
            k = ky * KW + kx
            py = ys + ky + offset[:, 2 * k]
            px = xs + kx + offset[:, 2 * k + 1]
            valid = (py > -1) & (py < H) & (px > -1) & (px < W)
            y0 = torch.floor(py)
            x0 = torch.floor(px)
            ly, lx = py - y0, px - x0
            y0, x0 = y0.long(), x0.long()
            sampled = torch.zeros(B, C, Ho, Wo, dtype=dt)
            for dy, dx, wgt in ((0, 0, (1 - ly) * (1 - lx)), (0, 1, (1 - ly) * lx),
                                (1, 0, ly * (1 - lx)), (1, 1, ly * lx)):
                yy, xx = y0 + dy, x0 + dx
                ok = valid & (yy >= 0) & (yy < H) & (xx >= 0) & (xx < W)
                idx = (yy.clamp(0, H - 1) * W + xx.clamp(0, W - 1)).view(B, 1, Ho * Wo).expand(B, C, Ho * Wo)
                v = torch.gather(xf, 2, idx).view(B, C, Ho, Wo)
                sampled = sampled + v * (wgt * ok.to(dt)).unsqueeze(1)
            if mask is not None:
                sampled = sampled * mask[:, k].unsqueeze(1)
            out = out + torch.einsum('oc,bchw->bohw', weight[:, :, ky, kx], sampled)
    if bias is not None:
        out = out + bias.view(1, O, 1, 1)
    return out


def batch_norm(sd, p, x, eps=BN_EPS):
    m = sd[p + '.weight'] / torch.sqrt(sd[p + '.running_var'] + eps)
    a = sd[p + '.bias'] - sd[p + '.running_mean'] * m
    return x * m.view(1, -1, 1, 1) + a.view(1, -1, 1, 1)


def lcsa(sd, p, x):
    """Mask logits [B,9,H,W]; ``p`` is the prefix of the LCSA module (its ``excite`` Sequential)."""
    c = x.shape[1]
    g = x.mean(dim=3, keepdim=True) + x.mean(dim=2, keepdim=True)
    e = p + '.excite'
    g = F.conv2d(g, sd[e + '.0.weight'], sd[e + '.0.bias'], padding=(0, 5), groups=c)
    g = F.relu(batch_norm(sd, e + '.1', g))
    g = F.conv2d(g, sd[e + '.3.weight'], sd[e + '.3.bias'], padding=(5, 0), groups=c)
    return F.conv2d(g, sd[e + '.4.weight'], sd[e + '.4.bias'])


def dsc(sd, p, x, return_parts=False):
    offset = F.conv2d(x, sd[p + '.conv_offset.weight'], sd[p + '.conv_offset.bias'], padding=1)
    mask = torch.sigmoid(lcsa(sd, p + '.RCA_mask', x))
    y = deform_conv2d(x, offset, sd[p + '.weight'], sd[p + '.bias'], mask)
    return (y, offset, mask) if return_parts else y


def kadconv(sd, p, x, n=3):
    """KADConv / KADC4 forward. ``p`` is the module prefix ('' for a bare layer)."""
    p = p + '.' if p and not p.endswith('.') else p
    feats = []
    for i in range(n):
        y = F.avg_pool2d(x, 2 ** i) if i > 0 else x
        y = F.conv2d(y, sd[f'{p}convs.{i}.0.weight'], sd[f'{p}convs.{i}.0.bias'])
        y = dsc(sd, f'{p}convs.{i}.1', y)
        y = F.relu(batch_norm(sd, f'{p}convs.{i}.2', y))
        y = y * sd[f'{p}weight.{i}.0.weight']
        a = y.mean(dim=(2, 3))
        a = F.relu(F.linear(a, sd[f'{p}fc.{i}.0.weight'], sd[f'{p}fc.{i}.0.bias']))
        a = torch.sigmoid(F.linear(a, sd[f'{p}fc.{i}.2.weight'], sd[f'{p}fc.{i}.2.bias']))
        y = y * a.view(x.shape[0], -1, 1, 1)
        if i > 0:
            y = F.interpolate(y, size=x.shape[2:], mode='bilinear', align_corners=False)
        feats.append(y)
    return torch.cat(feats, 1) + x


# ----------------------------------------------------------------------------- detector level

def make_divisible(x, d):
    return math.ceil(x / d) * d


# KAD-CNet-S graph (KAD-CNet/configs/dior_s_base.yaml:1-137): (from, module, args) with the
# width multiple 1.1 applied to the first argument the way parse_model does (models/yolo.py:767-771).
def detector_layers(width=1.1):
    w = lambda c: make_divisible(c * width, 8)
    return [
        (-1, 'Conv', (w(32), 3, 2)), (-1, 'Conv', (w(64), 3, 2)), (-1, 'ELAN1', (w(64), 64, 32)),
        (-1, 'AConv', (w(128),)), (-1, 'KADC', (w(128), 128, 64, 3)),
        (-1, 'AConv', (w(192),)), (-1, 'KADC', (w(192), 192, 96, 3)),
        (-1, 'AConv', (w(256),)), (-1, 'KADC', (w(256), 256, 128, 3)),
        (-1, 'SPPELAN', (w(256), 128)),
        (-1, 'Up', ()), ((-1, 6), 'Cat', ()), (-1, 'KADC', (w(192), 192, 96, 3)),
        (-1, 'Up', ()), ((-1, 4), 'Cat', ()), (-1, 'KADC', (w(128), 128, 64, 3)),
        (-1, 'AConv', (w(96),)), ((-1, 12), 'Cat', ()), (-1, 'KADC', (w(192), 192, 96, 3)),
        (-1, 'AConv', (w(128),)), ((-1, 9), 'Cat', ()), (-1, 'KADC', (w(256), 256, 128, 3)),
        ((15, 18, 21), 'DDetect', (20,)),
    ]


def conv_silu(sd, p, x, stride=1, groups=1, act=True):
    """``Conv`` block in its fused form: BN folded into the convolution, then SiLU."""
    w = sd[p + '.conv.weight']
    m = sd[p + '.bn.weight'] / torch.sqrt(sd[p + '.bn.running_var'] + BN_EPS)
    wf = w * m.view(-1, 1, 1, 1)
    bf = sd[p + '.bn.bias'] - sd[p + '.bn.running_mean'] * m
    y = F.conv2d(x, wf, bf, stride=stride, padding=w.shape[-1] // 2, groups=groups)
    return F.silu(y) if act else y


def _elan1(sd, p, x):
    y = list(conv_silu(sd, p + '.cv1', x).chunk(2, 1))
    y.append(conv_silu(sd, p + '.cv2', y[-1]))
    y.append(conv_silu(sd, p + '.cv3', y[-1]))
    return conv_silu(sd, p + '.cv4', torch.cat(y, 1))


def _aconv(sd, p, x):
    return conv_silu(sd, p + '.cv1', F.avg_pool2d(x, 2, 1, 0, False, True), stride=2)


def _repncsp_kadc(sd, p, x, n):
    y = conv_silu(sd, p + '.cv1', x)
    for j in range(n):
        y = kadconv(sd, f'{p}.m.{j}', y)
    return conv_silu(sd, p + '.cv3', torch.cat((y, conv_silu(sd, p + '.cv2', x)), 1))


def _kadc_elan(sd, p, x, n):
    y = list(conv_silu(sd, p + '.cv1', x).chunk(2, 1))
    for cv in ('.cv2', '.cv3'):
        t = _repncsp_kadc(sd, p + cv + '.0', y[-1], n)
        y.append(conv_silu(sd, p + cv + '.1', t))
    return conv_silu(sd, p + '.cv4', torch.cat(y, 1))


def _sppelan(sd, p, x):
    y = [conv_silu(sd, p + '.cv1', x)]
    for _ in range(3):
        y.append(F.max_pool2d(y[-1], 5, 1, 2))
    return conv_silu(sd, p + '.cv5', torch.cat(y, 1))


def make_anchors(shapes, strides, dtype=torch.float32):
    pts, st = [], []
    for (h, w), s in zip(shapes, strides):
        sx = torch.arange(w, dtype=dtype) + 0.5
        sy = torch.arange(h, dtype=dtype) + 0.5
        sy, sx = torch.meshgrid(sy, sx, indexing='ij')
        pts.append(torch.stack((sx, sy), -1).view(-1, 2))
        st.append(torch.full((h * w, 1), s, dtype=dtype))
    return torch.cat(pts).t(), torch.cat(st).t()


def ddetect(sd, p, feats, strides, nc=20, reg_max=16):
    raw = []
    for i, f in enumerate(feats):
        b = conv_silu(sd, f'{p}.cv2.{i}.0', f)
        b = conv_silu(sd, f'{p}.cv2.{i}.1', b, groups=4)
        b = F.conv2d(b, sd[f'{p}.cv2.{i}.2.weight'], sd[f'{p}.cv2.{i}.2.bias'], groups=4)
        c = conv_silu(sd, f'{p}.cv3.{i}.0', f)
        c = conv_silu(sd, f'{p}.cv3.{i}.1', c)
        c = F.conv2d(c, sd[f'{p}.cv3.{i}.2.weight'], sd[f'{p}.cv3.{i}.2.bias'])
        raw.append(torch.cat((b, c), 1))
    B = feats[0].shape[0]
    no = nc + 4 * reg_max
    anchors, st = make_anchors([r.shape[2:] for r in raw], strides, feats[0].dtype)
    box, cls = torch.cat([r.view(B, no, -1) for r in raw], 2).split((4 * reg_max, nc), 1)
    A = box.shape[2]
    prob = box.view(B, 4, reg_max, A).softmax(2)
    dist = (prob * torch.arange(reg_max, dtype=prob.dtype).view(1, 1, reg_max, 1)).sum(2)
    lt, rb = dist[:, :2], dist[:, 2:]
    x1y1 = anchors.unsqueeze(0) - lt
    x2y2 = anchors.unsqueeze(0) + rb
    dbox = torch.cat(((x1y1 + x2y2) / 2, x2y2 - x1y1), 1) * st
    return torch.cat((dbox, cls.sigmoid()), 1), raw


def detector(sd, x, strides=(8.0, 16.0, 32.0), width=1.1):
    """KAD-CNet-S forward on a fused-equivalent model; returns (y[B,4+nc,A], [raw P3,P4,P5])."""
    ys = []
    for i, (frm, kind, args) in enumerate(detector_layers(width)):
        if isinstance(frm, tuple):
            inp = [x if j == -1 else ys[j] for j in frm]
        else:
            inp = x if frm == -1 else ys[frm]
        p = f'model.{i}'
        if kind == 'Conv':
            x = conv_silu(sd, p, inp, stride=args[2])
        elif kind == 'ELAN1':
            x = _elan1(sd, p, inp)
        elif kind == 'AConv':
            x = _aconv(sd, p, inp)
        elif kind == 'KADC':
            x = _kadc_elan(sd, p, inp, args[3])
        elif kind == 'SPPELAN':
            x = _sppelan(sd, p, inp)
        elif kind == 'Up':
            x = F.interpolate(inp, scale_factor=2, mode='nearest')
        elif kind == 'Cat':
            x = torch.cat(inp, 1)
        elif kind == 'DDetect':
            return ddetect(sd, p, inp, strides, nc=args[0])
        ys.append(x)
    raise AssertionError('no head')


# ----------------------------------------------------------------------------- post-processing

def box_iou_one_to_many(b, bs):
    ix1 = torch.maximum(b[0], bs[:, 0]); iy1 = torch.maximum(b[1], bs[:, 1])
    ix2 = torch.minimum(b[2], bs[:, 2]); iy2 = torch.minimum(b[3], bs[:, 3])
    inter = (ix2 - ix1).clamp(min=0) * (iy2 - iy1).clamp(min=0)
    a = (b[2] - b[0]) * (b[3] - b[1])
    as_ = (bs[:, 2] - bs[:, 0]) * (bs[:, 3] - bs[:, 1])
    return inter / (a + as_ - inter)


def greedy_nms(boxes, scores, iou_thres):
    """Indices kept by greedy NMS in decreasing score order (stable for ties), boxes are xyxy.
    A box is suppressed when its IoU with an already kept box is strictly greater than the
    threshold (the rule of torchvision.ops.nms, which the reference calls at general.py:972)."""
    order = torch.argsort(scores, descending=True, stable=True)
    alive = torch.ones(len(order), dtype=torch.bool)
    keep = []
    for pos in range(len(order)):
        if not alive[pos]:
            continue
        i = order[pos]
        keep.append(int(i))
        rest = order[pos + 1:]
        iou = box_iou_one_to_many(boxes[i], boxes[rest])
        alive[pos + 1:] &= ~(iou > iou_thres)
    return torch.tensor(keep, dtype=torch.long)


def non_max_suppression(pred, conf_thres=0.001, iou_thres=0.65, max_det=300, max_wh=7680, max_nms=30000):
    """Best-class NMS on y[B,4+nc,A] -> list of [n,6] (xyxy, conf, cls), multi_label off."""
    out = []
    for x in pred:
        x = x.t()
        x = x[x[:, 4:].amax(1) > conf_thres]
        if not x.shape[0]:
            out.append(torch.zeros(0, 6, dtype=pred.dtype)); continue
        box = torch.stack((x[:, 0] - x[:, 2] / 2, x[:, 1] - x[:, 3] / 2,
                           x[:, 0] + x[:, 2] / 2, x[:, 1] + x[:, 3] / 2), 1)
        conf, j = x[:, 4:].max(1, keepdim=True)
        x = torch.cat((box, conf, j.float()), 1)[conf.view(-1) > conf_thres]     # float32 from here on, as in the reference
        if not x.shape[0]:
            out.append(torch.zeros(0, 6, dtype=pred.dtype)); continue
        x = x[x[:, 4].argsort(descending=True, stable=True)[:max_nms]]   # equal scores: lower anchor index first
        keep = greedy_nms(x[:, :4] + x[:, 5:6] * max_wh, x[:, 4], iou_thres)[:max_det]
        out.append(x[keep])
    return out
