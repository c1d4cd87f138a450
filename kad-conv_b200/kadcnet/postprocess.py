"""Detection post-processing with the reference's semantics.

Mirrors non_max_suppression of the reference project (KAD-CNet/utils/general.py:881-990) for the
inference configuration the detector scripts use (best class per box, class-offset batched NMS,
max_det cap): same operation order, so the same candidates in the same order reach NMS.
"""
import torch


def xywh2xyxy(x):
    y = x.clone()
    y[..., 0] = x[..., 0] - x[..., 2] / 2
    y[..., 1] = x[..., 1] - x[..., 3] / 2
    y[..., 2] = x[..., 0] + x[..., 2] / 2
    y[..., 3] = x[..., 1] + x[..., 3] / 2
    return y


def _nms(boxes, scores, iou_thres):
    import torchvision
    return torchvision.ops.nms(boxes, scores, iou_thres)


def non_max_suppression(prediction, conf_thres=0.25, iou_thres=0.45, classes=None, agnostic=False, max_det=300):
    """prediction: y[B,4+nc,A] (or the (y, raw) tuple). Returns a list of [n,6] tensors (xyxy, conf, cls)."""
    if isinstance(prediction, (list, tuple)):
        prediction = prediction[0]
    if not 0 <= conf_thres <= 1 or not 0 <= iou_thres <= 1:
        raise ValueError('thresholds must lie in [0, 1]')
    bs = prediction.shape[0]
    nc = prediction.shape[1] - 4
    max_wh, max_nms = 7680, 30000
    xc = prediction[:, 4:4 + nc].amax(1) > conf_thres
    output = [torch.zeros((0, 6), device=prediction.device)] * bs
    for xi, x in enumerate(prediction):
        x = x.T[xc[xi]]
        if not x.shape[0]:
            continue
        box, cls = x.split((4, nc), 1)
        box = xywh2xyxy(box)
        conf, j = cls.max(1, keepdim=True)
        x = torch.cat((box, conf, j.float()), 1)[conf.view(-1) > conf_thres]
        if classes is not None:
            x = x[(x[:, 5:6] == torch.tensor(classes, device=x.device)).any(1)]
        n = x.shape[0]
        if not n:
            continue
        x = x[x[:, 4].argsort(descending=True)[:max_nms]]
        c = x[:, 5:6] * (0 if agnostic else max_wh)
        i = _nms(x[:, :4] + c, x[:, 4], iou_thres)
        output[xi] = x[i[:max_det]]
    return output


def non_max_suppression_device(prediction, conf_thres=0.25, iou_thres=0.45, max_det=300):
    """Same result structure as non_max_suppression, computed by one batched CUDA kernel (kad_nms_batched):
    no per-image Python loop and no host synchronisation before the final read of the counts."""
    from kadconv import ops
    if isinstance(prediction, (list, tuple)):
        prediction = prediction[0]
    dets, counts = ops.nms_batched(prediction.contiguous(), conf_thres, iou_thres, max_det)
    # one device-to-host read for the counts and the kernels' status word: a forward whose tensor-core kernel gave up on a
    # wait must not hand out detections
    host = torch.cat((counts, ops.status_word(prediction.device))).tolist()
    ops.raise_if_aborted(host[-4:], ops.status_word(prediction.device).zero_)
    return [dets[i, :n] for i, n in enumerate(host[:-4])]
