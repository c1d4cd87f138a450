"""Explaining every difference between two NMS results (test infrastructure).

Two prediction tensors that agree to rounding error can still give different detections: greedy NMS takes hard
decisions (confidence > threshold, IoU > threshold, score order) and one flipped decision changes which later boxes
survive. "Identical boxes after NMS" can therefore only be shown up to those decisions. This module makes that exact.

Greedy best-class NMS (non_max_suppression of the reference, KAD-CNet/utils/general.py:881-990) keeps the unique
set S of candidates such that
    (1) no candidate in S overlaps a higher-scored member of S of its class by more than the IoU threshold, and
    (2) every candidate outside S overlaps a higher-scored member of S of its class by more than the threshold.
`check_explained` verifies that the kept set computed from prediction A satisfies (1) and (2) on prediction B's
boxes and scores when every comparison gets a tolerance: IoU within eps_iou of the threshold, scores within
eps_score of each other or of the confidence threshold, best-class margins within eps_score. With zero tolerance
the conditions have exactly one solution (B's own result), so any difference between the two results then lies in
decisions that sit inside the tolerance, and `trace_differences` names for each differing box the near-threshold
decision (or the chain of differing boxes leading to one) that accounts for it.
"""
import torch


def candidates(y_img, conf_thres):
    """y_img [4+nc, A] -> dict of per-anchor tensors: xyxy box, confidence, class, best-class margin, candidate flag."""
    cx, cy, w, h = y_img[0], y_img[1], y_img[2], y_img[3]        # corners in the prediction's own dtype, as xywh2xyxy computes them
    box = torch.stack((cx - w / 2, cy - h / 2, cx + w / 2, cy + h / 2), 1).float()
    cls = y_img[4:].t().float()
    top2 = cls.topk(min(2, cls.shape[1]), 1)
    conf, j = top2.values[:, 0], top2.indices[:, 0]
    margin = top2.values[:, 0] - top2.values[:, 1] if cls.shape[1] > 1 else torch.full_like(conf, float('inf'))
    return {'box': box, 'conf': conf, 'cls': j, 'margin': margin, 'cand': conf > conf_thres}


def pair_iou(b1, b2):
    """IoU matrix [n, m] of xyxy boxes."""
    lt = torch.maximum(b1[:, None, :2], b2[None, :, :2])
    rb = torch.minimum(b1[:, None, 2:], b2[None, :, 2:])
    inter = (rb - lt).clamp(min=0).prod(2)
    a1 = (b1[:, 2] - b1[:, 0]) * (b1[:, 3] - b1[:, 1])
    a2 = (b2[:, 2] - b2[:, 0]) * (b2[:, 3] - b2[:, 1])
    return inter / (a1[:, None] + a2[None, :] - inter)


def greedy_keep(c, iou_thres):
    """Anchor indices kept by exact greedy best-class NMS of one image's candidates, in decreasing score (ties: lower anchor first)."""
    idx = torch.nonzero(c['cand']).view(-1)
    order = idx[torch.argsort(c['conf'][idx], descending=True, stable=True)]
    box, cls = c['box'][order], c['cls'][order]
    n = order.shape[0]
    alive = torch.ones(n, dtype=torch.bool)
    keep = []
    for p in range(n):
        if not alive[p]:
            continue
        keep.append(int(order[p]))
        if p + 1 < n:
            iou = pair_iou(box[p:p + 1], box[p + 1:])[0]
            alive[p + 1:] &= ~((iou > iou_thres) & (cls[p + 1:] == cls[p]))
    return keep


def check_explained(keep_a, ca, cb, conf_thres, iou_thres, eps_iou, eps_score):
    """Is A's kept set (anchor indices, before any max_det cap) a greedy-NMS solution of B's data up to the tolerances?
    Returns a dict with the lists of violations (all empty = every difference is explained) and the counts of decisions
    that needed the tolerance."""
    kept = torch.tensor(sorted(keep_a), dtype=torch.long)
    box, conf, cls = cb['box'], cb['conf'], cb['cls']
    out = {'membership': [], 'class': [], 'kept_overlap': [], 'unsuppressed': []}
    # candidate membership and best class
    flip = torch.nonzero(ca['cand'] != cb['cand']).view(-1)
    out['membership'] = [int(i) for i in flip if abs(float(conf[i]) - conf_thres) > eps_score]
    both = ca['cand'] & cb['cand']
    dcls = torch.nonzero(both & (ca['cls'] != cb['cls'])).view(-1)
    out['class'] = [int(i) for i in dcls if float(cb['margin'][i]) > eps_score]
    # anchors whose class differs between A and B are near-ties by the check above: judge them under A's class
    cls = torch.where(both & (ca['cls'] != cb['cls']), ca['cls'], cls)
    cand = torch.nonzero(ca['cand'] | cb['cand']).view(-1)
    is_kept = torch.zeros(conf.shape[0], dtype=torch.bool)
    is_kept[kept] = True
    near = 0
    if kept.numel():
        iou = pair_iou(box[cand], box[kept])                                   # [n_cand, n_kept]
        same = cls[cand][:, None] == cls[kept][None, :]
        not_self = cand[:, None] != kept[None, :]
        higher_clear = conf[kept][None, :] > conf[cand][:, None] + eps_score     # certainly ahead in B's order
        higher_maybe = conf[kept][None, :] >= conf[cand][:, None] - eps_score    # possibly ahead
        ck = is_kept[cand]
        # (1) a kept box must not be clearly suppressed by a clearly higher-scored kept box
        bad1 = ck[:, None] & same & not_self & higher_clear & (iou > iou_thres + eps_iou)
        out['kept_overlap'] = [(int(cand[i]), int(kept[k])) for i, k in torch.nonzero(bad1)]
        # (2) a dropped candidate needs a plausible suppressor; candidates that only exist near the confidence threshold are exempt
        plausible = same & not_self & higher_maybe & (iou >= iou_thres - eps_iou)
        drop = ~ck & (conf[cand] > conf_thres + eps_score)
        out['unsuppressed'] = [int(cand[i]) for i in torch.nonzero(drop & ~plausible.any(1)).view(-1)]
        band = same & not_self & ((iou - iou_thres).abs() <= eps_iou)
        near = int(band.any(1).sum())
    else:
        out['unsuppressed'] = [int(i) for i in cand if float(conf[i]) > conf_thres + eps_score]
    out['near_threshold_candidates'] = near
    out['ok'] = not (out['membership'] or out['class'] or out['kept_overlap'] or out['unsuppressed'])
    return out


def trace_differences(keep_a, keep_b, ca, cb, iou_thres, eps_iou, eps_score, conf_thres):
    """For every anchor kept by exactly one of the two runs, the reason, judged on B's data:
    'threshold'  its confidence is within eps_score of the confidence threshold;
    'class'      its best class (or that of the box that suppresses it) differs between A and B: a tie of the two best class
                 scores within eps_score (check_explained verifies the margin);
    'iou'        its IoU with a kept box of the other run lies within eps_iou of the IoU threshold (a direct flip);
    'order'      it overlaps a kept box of the other run whose score is within eps_score of its own (order flip);
    'cascade'    the box that suppresses it in the other run is itself a differing box (second entry: that box);
    None         unexplained."""
    sa, sb = set(keep_a), set(keep_b)
    box, conf, cls = cb['box'], cb['conf'], cb['cls']
    flip = ca['cls'] != cb['cls']
    res = {}
    for d, other, own in [(d, sb, sa) for d in sa - sb] + [(d, sa, sb) for d in sb - sa]:
        # d is kept in `own` and dropped in `other`: look at the kept boxes of `other` that could have suppressed it there
        if abs(float(conf[d]) - conf_thres) <= eps_score:
            res[d] = ('threshold', None); continue
        if bool(flip[d]):
            res[d] = ('class', None); continue
        ks = torch.tensor(sorted(other), dtype=torch.long)
        if ks.numel() == 0:
            res[d] = (None, None); continue
        iou = pair_iou(box[d:d + 1], box[ks])[0]
        near = iou >= iou_thres - eps_iou
        close = near & (cls[ks] == cls[d])
        reason = None
        for k, v in zip(ks[close].tolist(), iou[close].tolist()):
            if abs(v - iou_thres) <= eps_iou:
                reason = ('iou', k); break
            if abs(float(conf[k]) - float(conf[d])) <= eps_score:
                reason = ('order', k); break
        if reason is None:
            # clearly overlapping suppressors in `other` must be absent from `own` (else d could not be kept there): cascade
            for k in ks[close].tolist():
                if k not in own:
                    reason = ('cascade', k); break
        if reason is None:
            # an overlapping box whose class differs between the two predictions suppresses d in one of them only
            for k in ks[near & flip[ks]].tolist():
                reason = ('class', k); break
        res[d] = reason if reason is not None else (None, None)
    return res
