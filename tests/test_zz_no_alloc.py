"""The allocation-free LCSA mask entry point against the regular one (collected last on purpose).

Who needs it: a host that cannot create device memory at the point where it calls the library, e.g. a server whose
own pool owns all of HBM, or a frame loop that must not pay cudaMalloc's device-wide synchronisation. The variant
takes no scratch argument (the scratch is a fixed array inside the library image), so the test only hands it
inputs and an output, twice in a row with different sizes, and expects the regular entry point's result.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _params(C, seed):
    g = np.random.default_rng(seed)
    f = lambda *shape, s=0.3: torch.from_numpy((s * g.standard_normal(shape)).astype(np.float32)).cuda()
    return dict(w1=f(C, 11), b1=f(C, s=0.1), bn_m=torch.from_numpy(g.uniform(0.5, 1.5, C).astype(np.float32)).cuda(), bn_a=f(C, s=0.1),
                w2=f(C, 11), b2=f(C, s=0.1), w3=f(9, C), b3=f(9, s=0.1))


def _both(B, H, W, C, seed):
    from kadconv import _abi
    lib = _abi.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = np.random.default_rng(seed)
    x = torch.from_numpy(g.standard_normal((B, H, W, C)).astype(np.float32)).cuda()
    prm = _params(C, seed + 1)
    rows = torch.empty((B, H, C), device='cuda'); cols = torch.empty((B, W, C), device='cuda')
    _abi.check(lib.kad_lcsa_sums(_p(x), _p(rows), _p(cols), B, H, W, C, _abi.KAD_F32, stream), 'kad_lcsa_sums')
    args = [_p(rows), _p(cols)] + [_p(prm[k]) for k in ('w1', 'b1', 'bn_m', 'bn_a', 'w2', 'b2', 'w3', 'b3')]
    scratch = torch.empty(B * W * C + W * C, device='cuda')
    ref = torch.empty((B, H, W, 9), device='cuda'); out = torch.full((B, H, W, 9), -1.0, device='cuda')
    _abi.check(lib.kad_lcsa_mask(*args, _p(scratch), _p(ref), B, H, W, C, 1, _abi.KAD_F32, stream), 'kad_lcsa_mask')
    _abi.check(lib.kad_lcsa_mask_noalloc(*args, _p(out), B, H, W, C, 1, _abi.KAD_F32, stream), 'kad_lcsa_mask_noalloc')
    torch.cuda.synchronize()
    return ref, out, x, prm


def _oracle_mask(x_nhwc, prm):
    """sigmoid(LCSA(x)) by the CPU oracle (oracle/kad_oracle.py:lcsa), from the folded parameters the entry points take: the
    folded BatchNorm (scale m, shift a) is handed to the oracle as weight = m, bias = a with zero mean and unit variance."""
    from oracle import kad_oracle as ko
    C = x_nhwc.shape[3]
    c = lambda t: t.detach().cpu()
    e = 'l.excite'
    sd = {e + '.0.weight': c(prm['w1']).view(C, 1, 1, 11), e + '.0.bias': c(prm['b1']),
          e + '.1.weight': c(prm['bn_m']) * (1.0 + ko.BN_EPS) ** 0.5, e + '.1.bias': c(prm['bn_a']),
          e + '.1.running_mean': torch.zeros(C), e + '.1.running_var': torch.ones(C),
          e + '.3.weight': c(prm['w2']).view(C, 1, 11, 1), e + '.3.bias': c(prm['b2']),
          e + '.4.weight': c(prm['w3']).view(9, C, 1, 1), e + '.4.bias': c(prm['b3'])}
    return torch.sigmoid(ko.lcsa(sd, 'l', c(x_nhwc).permute(0, 3, 1, 2))).permute(0, 2, 3, 1)


def test_noalloc_matches_regular_entry_point_twice():
    # second call is smaller than the first: whatever the first left in the shared array must not matter
    for (B, H, W, C), seed in (((3, 20, 31, 44), 1), ((2, 9, 14, 21), 2)):
        ref, out, x, prm = _both(B, H, W, C, seed)
        assert (out - ref).abs().max().item() <= 1e-5
        assert 0.0 < float(out.min()) and float(out.max()) < 1.0
        # ... and both agree with the CPU oracle's LCSA on the same input (the entry point itself, not only its sibling)
        assert (out.cpu() - _oracle_mask(x, prm)).abs().max().item() <= 1e-5


def test_noalloc_rejects_oversize():
    from kadconv import _abi
    lib = _abi.load()
    limit = lib.kad_lcsa_mask_noalloc_max_floats()
    assert limit == 1 << 20
    B, W, C = 64, 200, 256          # (B+1)*W*C floats > limit
    assert (B + 1) * W * C > limit
    dummy = torch.zeros(16, device='cuda')
    rc = lib.kad_lcsa_mask_noalloc(*[_p(dummy)] * 11, B, 200, W, C, 1, _abi.KAD_F32, None)
    assert rc == -3
    assert b'exceeds' in lib.kad_last_error_string()
