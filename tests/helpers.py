"""Shared helpers for the parity tests."""
import numpy as np
import torch

from oracle import seeding


def kadconv_shapes(dim, se_min_hidden=32):
    """state_dict key -> shape of a KADConv(dim) layer (reference key names)."""
    widths = [dim - (dim // 3) * 2, dim // 3, dim // 3]
    s = {}
    for i, c in enumerate(widths):
        h = max(se_min_hidden, c)
        s[f'convs.{i}.0.weight'] = (c, dim, 1, 1); s[f'convs.{i}.0.bias'] = (c,)
        d = f'convs.{i}.1'
        s[d + '.weight'] = (c, c, 3, 3); s[d + '.bias'] = (c,)
        s[d + '.conv_offset.weight'] = (18, c, 3, 3); s[d + '.conv_offset.bias'] = (18,)
        e = d + '.RCA_mask.excite'
        s[e + '.0.weight'] = (c, 1, 1, 11); s[e + '.0.bias'] = (c,)
        for leaf in ('weight', 'bias', 'running_mean', 'running_var'):
            s[f'{e}.1.{leaf}'] = (c,)
        s[e + '.1.num_batches_tracked'] = ()
        s[e + '.3.weight'] = (c, 1, 11, 1); s[e + '.3.bias'] = (c,)
        s[e + '.4.weight'] = (9, c, 1, 1); s[e + '.4.bias'] = (9,)
        for leaf in ('weight', 'bias', 'running_mean', 'running_var'):
            s[f'convs.{i}.2.{leaf}'] = (c,)
        s[f'convs.{i}.2.num_batches_tracked'] = ()
        s[f'fc.{i}.0.weight'] = (h, c); s[f'fc.{i}.0.bias'] = (h,)
        s[f'fc.{i}.2.weight'] = (c, h); s[f'fc.{i}.2.bias'] = (c,)
        s[f'weight.{i}.0.weight'] = (1, c, 1, 1)
    return s


def round_to(t, dtype):
    """Values representable in `dtype`, held in float32 (so a float32 oracle sees what the GPU sees)."""
    return t.to(dtype).float() if t.is_floating_point() else t


def rel_err(a, ref):
    """max|a - ref| / max|ref| -- the 'global relative' error the reference's own checks use
    (KAD-CNet/inference/check_equivalence.py:15-17)."""
    return ((a.float() - ref.float()).abs().max() / ref.float().abs().max().clamp_min(1e-12)).item()


def dcn_inputs(B, Cin, Cout, H, W, seed, offset_std=2.0):
    g = np.random.default_rng(seed)
    x = torch.from_numpy(g.standard_normal((B, Cin, H, W)).astype(np.float32))
    off = torch.from_numpy((offset_std * g.standard_normal((B, 18, H, W))).astype(np.float32))
    msk = torch.sigmoid(torch.from_numpy(g.standard_normal((B, 9, H, W)).astype(np.float32)))
    bound = 1.0 / np.sqrt(9 * Cin)
    w = torch.from_numpy(g.uniform(-bound, bound, (Cout, Cin, 3, 3)).astype(np.float32))
    b = torch.from_numpy((0.1 * g.standard_normal(Cout)).astype(np.float32))
    return x, off, msk, w, b


def nhwc(t):
    return t.permute(0, 2, 3, 1).contiguous()
