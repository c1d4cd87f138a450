"""CPU restatement of the inference script's preprocessing and box rescaling. TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Follows the reference project's KAD-CNet/utils/augmentations.py:106-136 (letterbox), KAD-CNet/inference/infer_dior.py:39-46
(BGR -> RGB, HWC -> CHW) and KAD-CNet/utils/general.py:824-868 (scale_boxes, clip_boxes) + infer_dior.py:56 (.round()).
letterbox calls cv2.resize(INTER_LINEAR), a third-party routine (opencv-python; the container has 4.13.0): its published
algorithm for 8-bit images is restated in `resize_linear_u8` (11-bit fixed-point coefficients, integer horizontal and vertical
passes, rounded 2x2 mean for an exact 2x shrink). Pinned by tests/golden/preprocess.npz, which was produced by the
reference's letterbox() running on the real cv2 (tests/golden/make_golden.py).
"""
import numpy as np


def _tables(src, dst):
    scale = 1.0 / (dst / src)
    f = ((np.arange(dst, dtype=np.float64) + 0.5) * scale - 0.5).astype(np.float32)
    s = np.floor(f).astype(np.int64)
    return s, (f - s.astype(np.float32)).astype(np.float32)


def resize_linear_u8(img, new_w, new_h):
    """cv2.resize(img, (new_w, new_h), interpolation=cv2.INTER_LINEAR) for a uint8 HxWx3 image."""
    H, W = img.shape[:2]
    if (W, H) == (new_w, new_h):
        return img.copy()
    v = img.astype(np.int32)
    if W == 2 * new_w and H == 2 * new_h:
        return ((v[0::2, 0::2] + v[0::2, 1::2] + v[1::2, 0::2] + v[1::2, 1::2] + 2) >> 2).astype(np.uint8)
    sx, fx = _tables(W, new_w)
    lo, hi = sx < 0, sx >= W - 1
    fx[lo] = 0; sx[lo] = 0
    fx[hi] = 0; sx[hi] = W - 1
    one = np.float32(2048)
    a0 = np.rint((np.float32(1) - fx) * one).astype(np.int32); a1 = np.rint(fx * one).astype(np.int32)
    sy, fy = _tables(H, new_h)
    b0 = np.rint((np.float32(1) - fy) * one).astype(np.int32); b1 = np.rint(fy * one).astype(np.int32)
    y0, y1 = np.clip(sy, 0, H - 1), np.clip(sy + 1, 0, H - 1)
    rows = v[:, sx] * a0[None, :, None] + v[:, np.minimum(sx + 1, W - 1)] * a1[None, :, None]
    out = (((b0[:, None, None] * (rows[y0] >> 4)) >> 16) + ((b1[:, None, None] * (rows[y1] >> 4)) >> 16) + 2) >> 2
    return out.astype(np.uint8)


def letterbox(im, new_shape=(640, 640), color=(114, 114, 114), auto=False, scaleup=True, stride=32):
    """Returns (image, ratio, (dw, dh)) like the reference's letterbox (scaleFill left out: the inference script never sets it)."""
    shape = im.shape[:2]
    if isinstance(new_shape, int):
        new_shape = (new_shape, new_shape)
    r = min(new_shape[0] / shape[0], new_shape[1] / shape[1])
    if not scaleup:
        r = min(r, 1.0)
    new_unpad = int(round(shape[1] * r)), int(round(shape[0] * r))
    dw, dh = new_shape[1] - new_unpad[0], new_shape[0] - new_unpad[1]
    if auto:
        dw, dh = np.mod(dw, stride), np.mod(dh, stride)
    dw /= 2
    dh /= 2
    if shape[::-1] != new_unpad:
        im = resize_linear_u8(im, new_unpad[0], new_unpad[1])
    top, bottom = int(round(dh - 0.1)), int(round(dh + 0.1))
    left, right = int(round(dw - 0.1)), int(round(dw + 0.1))
    out = np.empty((im.shape[0] + top + bottom, im.shape[1] + left + right, 3), dtype=np.uint8)
    out[...] = np.asarray(color, dtype=np.uint8)
    out[top:top + im.shape[0], left:left + im.shape[1]] = im
    return out, (r, r), (dw, dh)


def to_network_input(processed_bgr):
    """processed[:, :, ::-1].transpose(2, 0, 1), uint8 [1,3,H,W] (the `/255` is the model's business)."""
    return np.ascontiguousarray(processed_bgr[:, :, ::-1].transpose(2, 0, 1))[None]


def scale_boxes(img1_shape, boxes, img0_shape, do_round=True):
    """float32 [n,4] xyxy boxes from the network input's frame to the original image's; float32 arithmetic with the Python-float
    gain and padding cast to float32, as torch's in-place tensor-scalar ops compute it."""
    gain = min(img1_shape[0] / img0_shape[0], img1_shape[1] / img0_shape[1])
    pad = (img1_shape[1] - img0_shape[1] * gain) / 2, (img1_shape[0] - img0_shape[0] * gain) / 2
    b = boxes.astype(np.float32).copy()
    b[:, [0, 2]] -= np.float32(pad[0])
    b[:, [1, 3]] -= np.float32(pad[1])
    b /= np.float32(gain)
    b[:, [0, 2]] = b[:, [0, 2]].clip(0, img0_shape[1])
    b[:, [1, 3]] = b[:, [1, 3]].clip(0, img0_shape[0])
    return np.rint(b) if do_round else b
