"""Operator-level public API: a stand-in for ``torchvision.ops.deform_conv2d`` as DSC.forward calls it
(KAD-Conv/kadconv/kad_conv.py:66-67 of the reference project): 3x3 kernel, stride 1, padding 1,
dilation 1, one offset group, NCHW logical tensors in and out. CUDA only."""
import torch

from . import ops


class PackedDeformWeight:
    """A [Cout,Cin,3,3] weight packed once for the kernels (tensor-core layout when the shape allows)."""

    def __init__(self, weight, dtype):
        w = weight.detach().float()
        self.cout, self.cin = w.shape[:2]
        self.dtype = dtype
        if dtype != torch.float32 and ops.dsc_tc_supported(self.cin, self.cout, dtype):
            self.path, self.packed = ops.PATH_TC, ops.pack_dsc_weight_tc(w, dtype)
        else:
            self.path, self.packed = ops.PATH_SIMT, ops.pack_dsc_weight_simt(w)


def _pair(v):
    return tuple(v) if isinstance(v, (tuple, list)) else (v, v)


def deform_conv2d(input, offset, weight, bias=None, stride=(1, 1), padding=(1, 1), dilation=(1, 1), mask=None):
    if not input.is_cuda:
        raise RuntimeError('kadconv.functional.deform_conv2d has no CPU path')
    if _pair(stride) != (1, 1) or _pair(padding) != (1, 1) or _pair(dilation) != (1, 1):
        raise NotImplementedError('only stride 1, padding 1, dilation 1 (the DSC configuration) is implemented')
    if not isinstance(weight, PackedDeformWeight):
        if tuple(weight.shape[2:]) != (3, 3):
            raise NotImplementedError('only 3x3 kernels are implemented')
        weight = PackedDeformWeight(weight, input.dtype)
    if offset.shape[1] != 18 or (mask is not None and mask.shape[1] != 9):
        raise NotImplementedError('one offset group of a 3x3 kernel is implemented (18 offset / 9 mask channels)')
    channels_last = input.permute(0, 2, 3, 1).is_contiguous()
    x = ops.to_nhwc(input)
    off = ops.to_nhwc(offset)
    msk = None if mask is None else ops.to_nhwc(mask)
    shift = None if bias is None else bias.detach().float().contiguous()
    y = ops.dsc_forward(x, weight.packed, off, msk, shift=shift, path=weight.path, cout=weight.cout)
    return y.permute(0, 3, 1, 2) if channels_last else ops.to_nchw(y)
