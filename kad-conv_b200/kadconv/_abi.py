"""ctypes binding of libkadconv_b200.so (the C ABI declared in include/kadconv_b200.h).

The library is the only compute back end of this package: there is no CPU path and no other
GPU back end. If it has not been built, importing this module raises with the build command.
"""
import ctypes
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_longlong, c_size_t, c_void_p
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / '_lib' / 'libkadconv_b200.so'

KAD_F32, KAD_F16, KAD_BF16 = 0, 1, 2
ACT_NONE, ACT_SILU, ACT_RELU = 0, 1, 2
PATH_SIMT, PATH_TC, PATH_TC_PAIR, PATH_MMA = 0, 1, 2, 3


class KadDscArgs(Structure):
    _fields_ = [('x', c_void_p), ('offset', c_void_p), ('mask', c_void_p), ('weight', c_void_p),
                ('scale', c_void_p), ('shift', c_void_p), ('post', c_void_p),
                ('y', c_void_p), ('gap_partial', c_void_p),
                ('B', c_int), ('H', c_int), ('W', c_int), ('Cin', c_int), ('Cout', c_int),
                ('dtype', c_int), ('offset_f32', c_int), ('mask_f32', c_int), ('y_f32', c_int), ('act', c_int),
                ('path', c_int), ('status', c_void_p),
                ('offset_weight', c_void_p), ('offset_bias', c_void_p),
                ('lcsa_rowmean', c_void_p), ('lcsa_A', c_void_p), ('lcsa_Sm', c_void_p),
                ('lcsa_w2', c_void_p), ('lcsa_b2', c_void_p), ('lcsa_w3', c_void_p), ('lcsa_b3', c_void_p),
                ('mma_frags', c_void_p)]


class KadPyramidArgs(Structure):
    _fields_ = [('x', c_void_p), ('w', c_void_p * 3), ('bias', c_void_p * 3), ('t', c_void_p * 3),
                ('B', c_int), ('H', c_int), ('W', c_int), ('dim', c_int), ('c', c_int * 3), ('dtype', c_int),
                ('rowpart', c_void_p * 3), ('colpart', c_void_p * 3), ('counters', c_void_p),
                ('lcsa_w1', c_void_p * 3), ('lcsa_b1', c_void_p * 3), ('lcsa_bn_scale', c_void_p * 3), ('lcsa_bn_shift', c_void_p * 3),
                ('lcsa_rowmean', c_void_p * 3), ('lcsa_A', c_void_p * 3), ('lcsa_Sm', c_void_p * 3)]


class KadMergeArgs(Structure):
    _fields_ = [('x', c_void_p), ('out', c_void_p), ('y', c_void_p * 3), ('att', c_void_p * 3),
                ('c', c_int * 3), ('h', c_int * 3), ('w', c_int * 3),
                ('B', c_int), ('H', c_int), ('W', c_int), ('C', c_int), ('dtype', c_int),
                ('gap', c_void_p * 3), ('fc_w1', c_void_p * 3), ('fc_b1', c_void_p * 3), ('fc_w2', c_void_p * 3), ('fc_b2', c_void_p * 3),
                ('gap_tiles', c_int * 3), ('hidden', c_int * 3), ('out_cstride', c_int)]


class KadBranchParams(Structure):
    _fields_ = [(n, c_void_p) for n in ('w_proj', 'b_proj', 'lcsa_w1', 'lcsa_b1', 'lcsa_bn_scale', 'lcsa_bn_shift', 'lcsa_w2', 'lcsa_b2',
                                        'lcsa_w3', 'lcsa_b3', 'w_off', 'b_off', 'w_dsc_simt', 'w_dsc_tc', 'w_dsc_mma', 'ep_scale', 'ep_shift', 'ep_post',
                                        'fc_w1', 'fc_b1', 'fc_w2', 'fc_b2')] + [('c', c_int), ('hidden', c_int)]


class KadLayerArgs(Structure):
    _fields_ = [('x', c_void_p), ('out', c_void_p), ('workspace', c_void_p), ('workspace_bytes', c_size_t), ('status', c_void_p),
                ('B', c_int), ('H', c_int), ('W', c_int), ('dim', c_int), ('dtype', c_int), ('br', KadBranchParams * 3),
                ('out_cstride', c_int), ('counters', c_void_p), ('scheme', c_int)]


# name -> (restype, argtypes); every symbol declared in include/kadconv_b200.h
SIGNATURES = {
    'kad_version': (c_int, []),
    'kad_struct_size': (c_int, [c_int]),
    'kad_last_error_string': (c_char_p, []),
    'kad_nchw_to_nhwc': (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'kad_nhwc_to_nchw': (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'kad_dsc_forward': (c_int, [POINTER(KadDscArgs), c_void_p]),
    'kad_dsc_gap_tiles': (c_int, [c_int, c_int, c_int, c_int, c_int]),
    'kad_dsc_tc_supported': (c_int, [c_int, c_int, c_int]),
    'kad_pyramid_project_supported': (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    'kad_pyramid_project': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    'kad_pyramid_lcsa_supported': (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    'kad_pyramid_project_lcsa': (c_int, [POINTER(KadPyramidArgs), c_void_p]),
    'kad_dsc_mma_inline_mask_supported': (c_int, [c_int, c_int, c_int, c_int, c_int]),
    'kad_dsc_mma_frag_bytes': (c_size_t, [c_int, c_int, c_int]),
    'kad_dsc_mma_pack_frags': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    'kad_kadconv_launch_count': (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    'kad_pyramid_partial_dims': (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, POINTER(c_int), POINTER(c_int)]),
    'kad_lcsa_mask_from_partials_supported': (c_int, [c_int, c_int, c_int]),
    'kad_lcsa_mask_from_partials': (c_int, [c_void_p, c_int, c_void_p, c_int] + [c_void_p] * 8 + [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'kad_lcsa_masks3_supported': (c_int, [c_int, c_int, c_int, c_int, c_int]),
    'kad_lcsa_masks3_from_partials': (c_int, [c_void_p, c_void_p, c_int, c_int] + [c_void_p] * 9 + [c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p]),
    'kad_stem_conv_supported': (c_int, [c_int, c_int, c_int]),
    'kad_stem_conv_u8': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]),
    'kad_dsc_mma_supported': (c_int, [c_int, c_int, c_int, c_int, c_int]),
    'kad_dsc_pack_weight_tc': (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    'kad_dsc_packed_weight_bytes': (c_size_t, [c_int, c_int, c_int]),
    'kad_dsc_pack_weight_simt': (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    'kad_pool_project': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_int, c_int, c_int, c_void_p]),
    'kad_avg_pool': (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'kad_avg_pool2x2s1': (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'kad_bias_act_inplace': (c_int, [c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p]),
    'kad_bias_act_to': (c_int, [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p]),
    'kad_copy_channels': (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_longlong, c_int, c_int, c_void_p]),
    'kad_upsample2x_concat': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'kad_image_to_nhwc': (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]),
    'kad_lcsa_sums': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'kad_lcsa_mask': (c_int, [c_void_p] * 12 + [c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'kad_lcsa_mask_noalloc_max_floats': (c_size_t, []),
    'kad_lcsa_mask_noalloc': (c_int, [c_void_p] * 11 + [c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'kad_se_excite': (c_int, [c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                              c_void_p]),
    'kad_se_squeeze_tiles': (c_int, [c_int, c_int]),
    'kad_se_squeeze': (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'kad_se_rescale': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'kad_merge_upsample_residual': (c_int, [POINTER(KadMergeArgs), c_void_p]),
    'kad_kadconv_workspace_bytes': (c_size_t, [c_int, c_int, c_int, c_int, c_int, c_int]),
    'kad_kadconv_forward': (c_int, [POINTER(KadLayerArgs), c_void_p]),
    'kad_nms_max_anchors': (c_int, []),
    'kad_nms_batched': (c_int, [c_void_p, c_int, c_int, c_int, c_float, c_float, c_int, c_float, c_void_p, c_void_p, c_int, c_void_p]),
    'kad_head_decode': (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p]),
    'kad_gemm1x1_tc_supported': (c_int, [c_int, c_int, c_int]),
    'kad_gemm1x1_bias_act': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int,
                                     c_int, c_void_p, c_void_p]),
    'kad_spp_pool3_supported': (c_int, [c_int, c_int, c_int, c_int]),
    'kad_spp_pool3': (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'kad_letterbox_u8': (c_int, [c_void_p, c_void_p] + [c_int] * 9 + [c_void_p] * 4 + [c_int, c_void_p]),
    'kad_scale_boxes': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    'kad_conv3x3_tc_supported': (c_int, [c_int, c_int, c_int, c_int]),
    'kad_conv3x3_bias_act': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                     c_int, c_int, c_void_p, c_void_p]),
}

_lib = None


def library_path():
    return _LIB_PATH


def load():
    """Load the shared library once; raise if it is missing (no fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise RuntimeError(
            f'{_LIB_PATH} is missing: build the CUDA library first with '
            f'`python {_LIB_PATH.parents[2] / "build.py"}` (needs nvcc with sm_100a support). '
            'kadconv has no CPU or PyTorch fallback for its accelerated path.')
    lib = ctypes.CDLL(str(_LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)     # AttributeError if the library does not export a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


# Number of kernels launched through this binding so far (a plain counter the benchmark reads).
KERNELS_LAUNCHED = [0]
_KERNELS_PER_CALL = {'kad_lcsa_sums': 2, 'kad_lcsa_mask': 2, 'kad_kadconv_forward': 25}


def check(code, what, launches=None):
    KERNELS_LAUNCHED[0] += _KERNELS_PER_CALL.get(what, 1) if launches is None else launches
    if code != 0:
        msg = load().kad_last_error_string().decode(errors='replace')
        raise RuntimeError(f'{what} failed ({code}): {msg}')
