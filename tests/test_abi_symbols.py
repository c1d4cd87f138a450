"""The C-ABI library builds for sm_100a, loads, and exports every symbol the header declares."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _declared():
    text = (ROOT / 'include' / 'kadconv_b200.h').read_text()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(kad_[a-z0-9_]+)\s*\(', text)))


def test_header_symbols_exported():
    import __graft_entry__ as ge
    lib_path = ge.build_library()
    lib = ctypes.CDLL(str(lib_path))
    names = _declared()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f'{n} declared in the header but not exported'


def test_python_binding_covers_header():
    from kadconv import _abi
    assert sorted(_abi.SIGNATURES) == _declared()
    lib = _abi.load()
    assert lib.kad_version() >= 100
    assert lib.kad_last_error_string() is not None


def test_argument_errors_do_not_need_a_gpu():
    from kadconv import _abi
    lib = _abi.load()
    # null pointers are rejected before any CUDA call
    assert lib.kad_dsc_forward(None, None) == -1
    assert b'null' in lib.kad_last_error_string()
    assert lib.kad_dsc_tc_supported(256, 256, _abi.KAD_F16) == 1
    assert lib.kad_dsc_tc_supported(22, 22, _abi.KAD_F16) == 0
    assert lib.kad_dsc_tc_supported(256, 256, _abi.KAD_F32) == 0
    assert lib.kad_dsc_packed_weight_bytes(256, 256, _abi.KAD_F16) == 36 * 256 * 64 * 2
    assert lib.kad_gemm1x1_tc_supported(128, 256, _abi.KAD_BF16) == 1
    assert lib.kad_gemm1x1_tc_supported(130, 256, _abi.KAD_BF16) == 0


def test_ctypes_structs_have_the_size_the_library_was_compiled_with():
    """The library reads every field of an argument struct: a declaration that is too short (a field added to the header and
    not to the binding) would be read past its end. kad_struct_size gives sizeof as compiled."""
    from kadconv import _abi
    lib = _abi.load()
    for which, cls in enumerate((_abi.KadDscArgs, _abi.KadPyramidArgs, _abi.KadMergeArgs, _abi.KadBranchParams, _abi.KadLayerArgs)):
        assert lib.kad_struct_size(which) == ctypes.sizeof(cls), cls.__name__
    assert lib.kad_struct_size(99) == -1
