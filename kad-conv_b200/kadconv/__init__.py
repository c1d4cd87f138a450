"""kadconv for B200: the reference's module API (KADConv, DSC, LCSA, enable_/disable_fast_inference)
backed by hand-written sm_100a CUDA kernels behind a C ABI (libkadconv_b200.so)."""
from .kad_conv import DSC, KADConv, LCSA
from .fast import disable_fast_inference, enable_fast_inference

__all__ = ['KADConv', 'DSC', 'LCSA', 'enable_fast_inference', 'disable_fast_inference']
