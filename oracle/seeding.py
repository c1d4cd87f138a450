"""Seeded, reproducible weights for the parity harness.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

The reference zero-initialises the DSC offset convolution (KAD-Conv/kadconv/kad_conv.py:60-61,
KAD-CNet/models/module/ops.py:65-66), leaves BatchNorm identity-like, and biases the detector's
class logits so low that no score clears the 0.001 threshold (KAD-CNet/models/yolo.py:134-136).
A parity check on such a model never exercises the deformable sampling, the BN fold or NMS, so
every tensor is redrawn here from a per-key generator that depends only on (seed, key name):
the same call gives the same weights for the reference modules and for the CUDA-backed ones,
on any machine, without shipping the tensors.
"""
import math
import zlib

import numpy as np
import torch


def _rng(seed, key):
    return np.random.default_rng([int(seed), zlib.crc32(key.encode())])


def seeded_state_dict(shapes, seed=0, offset_std=0.5, scale_mode='uniform', cls_bias=-3.0, weight_gain=1.0, cls_gain=60.0):
    """``shapes``: mapping key -> shape (e.g. from ``module.state_dict()``). Returns float32 tensors.

    offset_std: target standard deviation, in pixels, of the DSC offsets for unit-variance input.
    scale_mode: 'uniform' draws branch scales from U(0.5,1.5); 'normal' from N(0,1).
    cls_bias: mean of the detector's class-logit biases (stock init is about -10, which leaves NMS no candidates).
    weight_gain: factor on every convolution / linear weight except the offset convolutions, the LCSA, the DFL and the class
        logits. With 1.0 (the bound 1/sqrt(fan_in) of the reference's initialisers) the signal fades from layer to layer and a
        60-layer detector computes nearly the same scores for every image and position; about 2.6 keeps it alive, so that
        scores and boxes vary over the image (the acceptance test of the detector uses that).
    cls_gain: factor on the class-logit weights of the detector head.
    """
    bn = {k[:-len('.running_mean')] for k in shapes if k.endswith('.running_mean')}
    out = {}
    for key, shape in shapes.items():
        shape = tuple(shape)
        g = _rng(seed, key)
        prefix, _, leaf = key.rpartition('.')
        if leaf == 'num_batches_tracked':
            v = np.zeros(shape, dtype=np.int64)
            out[key] = torch.from_numpy(v)
            continue
        if prefix in bn:
            if leaf == 'running_var':
                v = g.uniform(0.5, 1.5, shape)
            elif leaf == 'weight':
                v = g.uniform(0.5, 1.5, shape)
            else:  # bias, running_mean
                v = g.normal(0.0, 0.1, shape)
        elif 'dfl.conv' in key:
            v = np.arange(int(np.prod(shape)), dtype=np.float64).reshape(shape)
        elif 'conv_offset' in key:
            if leaf == 'weight':
                fan_in = int(np.prod(shape[1:]))
                v = g.normal(0.0, offset_std / math.sqrt(fan_in), shape)
            else:
                v = g.normal(0.0, 0.1 * offset_std, shape)
        elif len(shape) == 4 and shape[0] == 1 and shape[2:] == (1, 1) and '.weight.' in '.' + key:
            # branch-selection scale [1,c,1,1] (keys 'weight.{i}.0.weight')
            v = g.normal(0.0, 1.0, shape) if scale_mode == 'normal' else g.uniform(0.5, 1.5, shape)
        elif leaf == 'weight':
            fan_in = int(np.prod(shape[1:])) if len(shape) > 1 else shape[0]
            bound = 1.0 / math.sqrt(max(fan_in, 1))
            if '.cv3.' in key and key.endswith('.2.weight'):
                bound *= cls_gain   # detector class logits: spread the scores so that NMS is not a field of ties
            elif 'RCA_mask' not in key:
                bound *= weight_gain
            v = g.uniform(-bound, bound, shape)
        else:  # plain conv / linear bias
            v = g.normal(0.0, 0.1, shape)
            if '.cv3.' in key and key.endswith('.2.bias'):
                v = v + cls_bias   # detector class logits
        out[key] = torch.from_numpy(np.asarray(v, dtype=np.float32).reshape(shape))
    return out


def shapes_of(module_or_sd):
    sd = module_or_sd.state_dict() if hasattr(module_or_sd, 'state_dict') else module_or_sd
    return {k: tuple(v.shape) for k, v in sd.items()}


def seeded_input(shape, seed=0, kind='normal'):
    g = np.random.default_rng([int(seed), 0x1234])
    if kind == 'normal':
        return torch.from_numpy(g.standard_normal(shape).astype(np.float32))
    if kind == 'image':  # uint8 RGB uniform in [0,255]
        return torch.from_numpy(g.integers(0, 256, shape, dtype=np.uint8))
    raise ValueError(kind)
