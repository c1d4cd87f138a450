"""Image preprocessing and box post-scaling of the reference's inference script, on the device.

Mirrors KAD-CNet/inference/infer_dior.py:36-57 of the reference project: `letterbox` (utils/augmentations.py:106-136:
cv2.resize to the unpadded size, constant border 114), BGR -> RGB, HWC -> CHW, and after NMS `scale_boxes(...).round()`
(utils/general.py:824-868) back to the original image. `letterbox_geometry` and `resize_tables` are host arithmetic (they
reproduce the reference's and OpenCV's rounding rules); the pixels and the boxes are processed by CUDA kernels
(kad_letterbox_u8, kad_scale_boxes). The `/255` of the script is applied by the detector's first layer, which takes uint8.
"""
import ctypes

import numpy as np
import torch


def letterbox_geometry(shape, new_shape=(640, 640), auto=False, scale_fill=False, scaleup=True, stride=32):
    """(h0, w0) -> dict(new_unpad=(w, h), top, bottom, left, right, ratio=(rw, rh), pad=(dw, dh), out_shape=(H, W)), the numbers
    letterbox() derives before it touches a pixel (same expressions, Python float arithmetic, round() and int())."""
    if isinstance(new_shape, int):
        new_shape = (new_shape, new_shape)
    h0, w0 = int(shape[0]), int(shape[1])
    r = min(new_shape[0] / h0, new_shape[1] / w0)
    if not scaleup:
        r = min(r, 1.0)
    ratio = (r, r)
    new_unpad = (int(round(w0 * r)), int(round(h0 * r)))
    dw, dh = new_shape[1] - new_unpad[0], new_shape[0] - new_unpad[1]
    if auto:
        dw, dh = dw % stride, dh % stride
    elif scale_fill:
        dw, dh = 0.0, 0.0
        new_unpad = (new_shape[1], new_shape[0])
        ratio = (new_shape[1] / w0, new_shape[0] / h0)
    dw /= 2
    dh /= 2
    top, bottom = int(round(dh - 0.1)), int(round(dh + 0.1))
    left, right = int(round(dw - 0.1)), int(round(dw + 0.1))
    return {'new_unpad': new_unpad, 'top': top, 'bottom': bottom, 'left': left, 'right': right, 'ratio': ratio, 'pad': (dw, dh),
            'out_shape': (new_unpad[1] + top + bottom, new_unpad[0] + left + right)}


def resize_tables(src, dst, clamp_fraction):
    """Source offsets (int32 [dst]) and 11-bit fixed-point coefficient pairs (int16 [dst, 2]) of OpenCV's bilinear resize of an
    8-bit image along one axis from `src` to `dst` samples: position (d + 0.5) * (src / dst) - 0.5 evaluated in double and cast
    to float, floor, fraction in float, coefficients rounded half-to-even from (1 - f) * 2048 and f * 2048. Along x
    (clamp_fraction=True) positions left of the first or at / right of the last sample snap to that sample with f = 0; along y
    the offsets are only clipped when the rows are fetched (the kernel does that)."""
    scale = 1.0 / (dst / src)
    f = ((np.arange(dst, dtype=np.float64) + 0.5) * scale - 0.5).astype(np.float32)
    s = np.floor(f).astype(np.int32)
    f = (f - s.astype(np.float32)).astype(np.float32)
    if clamp_fraction:
        lo, hi = s < 0, s >= src - 1
        f[lo] = 0; s[lo] = 0
        f[hi] = 0; s[hi] = src - 1
    coef = np.stack((np.rint((np.float32(1.0) - f) * np.float32(2048)), np.rint(f * np.float32(2048))), 1)
    return s, np.clip(coef, -32768, 32767).astype(np.int16)


_table_cache = {}


def _device_tables(h0, w0, new_h, new_w, device):
    key = (h0, w0, new_h, new_w, str(device))
    if key not in _table_cache:
        xo, xa = resize_tables(w0, new_w, True)
        yo, yb = resize_tables(h0, new_h, False)
        _table_cache[key] = tuple(torch.from_numpy(np.ascontiguousarray(t)).to(device) for t in (xo, xa, yo, yb))
    return _table_cache[key]


def letterbox_device(image_bgr, new_shape=(640, 640), color=114, auto=False, scale_fill=False, scaleup=True, stride=32, out=None):
    """image_bgr: uint8 CUDA tensor [H0, W0, 3] in BGR order (cv2.imread layout). Returns (x, ratio, (dw, dh)) where x is the
    letterboxed image as uint8 [1, 3, H, W] RGB planes on the same device (feed it to the B200 engine as is) and ratio / pad are
    what letterbox() returns. `out` may supply the destination ([1,3,H,W] or [3,H,W] uint8, e.g. a slice of a batch)."""
    from kadconv import _abi, ops
    if not image_bgr.is_cuda or image_bgr.dtype != torch.uint8 or image_bgr.dim() != 3 or image_bgr.shape[2] != 3:
        raise ValueError('letterbox_device expects a uint8 CUDA tensor [H, W, 3] (there is no CPU path)')
    image_bgr = image_bgr.contiguous()
    h0, w0 = int(image_bgr.shape[0]), int(image_bgr.shape[1])
    g = letterbox_geometry((h0, w0), new_shape, auto, scale_fill, scaleup, stride)
    new_w, new_h = g['new_unpad']
    H, W = g['out_shape']
    if out is None:
        out = torch.empty((1, 3, H, W), dtype=torch.uint8, device=image_bgr.device)
    if out.dtype != torch.uint8 or not out.is_contiguous() or tuple(out.shape[-3:]) != (3, H, W) or out.numel() != 3 * H * W:
        raise ValueError(f'out must be a contiguous uint8 tensor [1,3,{H},{W}]')
    area = (h0 == 2 * new_h and w0 == 2 * new_w)
    if area:
        xo = xa = yo = yb = None
    else:
        xo, xa, yo, yb = _device_tables(h0, w0, new_h, new_w, image_bgr.device)
    p = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    _abi.check(_abi.load().kad_letterbox_u8(p(image_bgr), p(out), h0, w0, H, W, new_h, new_w, g['top'], g['left'], int(area),
                                            p(xo), p(xa), p(yo), p(yb), int(color), ops._stream()), 'kad_letterbox_u8')
    return out.view(1, 3, H, W), g['ratio'], g['pad']


def scale_boxes_geometry(img1_shape, img0_shape):
    """(gain, pad_x, pad_y, width0, height0) of scale_boxes() for a network input of img1_shape = (H, W) and an original image of
    img0_shape = (h0, w0[, c]): the reference's Python float arithmetic."""
    gain = min(img1_shape[0] / img0_shape[0], img1_shape[1] / img0_shape[1])
    pad = (img1_shape[1] - img0_shape[1] * gain) / 2, (img1_shape[0] - img0_shape[0] * gain) / 2
    return gain, pad[0], pad[1], float(img0_shape[1]), float(img0_shape[0])


def scale_boxes_device(dets, counts, img1_shape, img0_shapes, round_boxes=True):
    """dets float32 [B, max_det, 6] and counts int32 [B] as kadconv.ops.nms_batched returns them; img0_shapes: one (h0, w0) per
    image. Rescales the boxes to the original images in place (scale_boxes + clip_boxes, then .round() as the inference script
    does) and returns dets."""
    from kadconv import _abi, ops
    B, max_det = dets.shape[0], dets.shape[1]
    if len(img0_shapes) != B:
        raise ValueError('one original shape per image')
    geom = torch.tensor([scale_boxes_geometry(img1_shape, s) for s in img0_shapes], dtype=torch.float32).to(dets.device)
    if not dets.is_cuda or dets.dtype != torch.float32 or not dets.is_contiguous() or counts.dtype != torch.int32:
        raise ValueError('dets must be a contiguous float32 CUDA tensor [B,max_det,6] and counts int32 [B]')
    _abi.check(_abi.load().kad_scale_boxes(ctypes.c_void_p(dets.data_ptr()), ctypes.c_void_p(counts.data_ptr()), ctypes.c_void_p(geom.data_ptr()),
                                           B, max_det, int(round_boxes), ops._stream()), 'kad_scale_boxes')
    return dets
