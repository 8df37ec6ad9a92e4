"""The allocation-free attention reverse entry point against the allocating one.

femto_attention_bwd_static exists for hosts that may not call cudaMalloc while the step runs (an
allocator that owns the whole device, a no-allocation phase).  It must give exactly what
femto_attention_bwd gives, on back-to-back calls that share the built-in scratch array, and must
refuse shapes larger than that array.  Collected last so a failure here cannot hide other tests.
"""
import pytest
import torch

from femtochat_b200 import _lib

pytestmark = pytest.mark.gpu


def _case(dtype, B, T, H, Hkv, hd, left, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    td = torch.bfloat16 if dtype == _lib.BF16 else torch.float32
    mk = lambda *s: torch.randn(*s, generator=g, device="cuda").to(td)
    Q, K, V, dO = mk(B, T, H, hd), mk(B, T, Hkv, hd), mk(B, T, Hkv, hd), mk(B, T, H, hd)
    O = torch.zeros_like(Q)
    lse = torch.zeros(B, H, T, device="cuda")
    L = _lib.lib()
    _lib.check(L.femto_attention_fwd(dtype, _lib.ptr(O), None, None, _lib.ptr(lse), _lib.ptr(Q), _lib.ptr(K), _lib.ptr(V),
                                     B, T, H, Hkv, hd, left, None, None))
    return Q, K, V, dO, O, lse


def _bwd(fn, dtype, Q, K, V, dO, O, lse, left):
    B, T, H, hd = Q.shape
    Hkv = K.shape[2]
    dQ, dK, dV = torch.full_like(Q, 7.0), torch.full_like(K, 7.0), torch.full_like(V, 7.0)
    L = _lib.lib()
    if fn == "static":
        _lib.check(L.femto_attention_bwd_static(dtype, _lib.ptr(dQ), _lib.ptr(dK), _lib.ptr(dV), _lib.ptr(dO), _lib.ptr(Q),
                                                _lib.ptr(K), _lib.ptr(V), _lib.ptr(O), _lib.ptr(lse), B, T, H, Hkv, hd, left,
                                                None, None))
    else:    # the allocating entry point: lse form of the statistics, accumulate = 0
        _lib.check(L.femto_attention_bwd(dtype, _lib.ptr(dQ), _lib.ptr(dK), _lib.ptr(dV), _lib.ptr(dO), _lib.ptr(Q), _lib.ptr(K),
                                         _lib.ptr(V), _lib.ptr(O), _lib.ptr(lse), None, None, B, T, H, Hkv, hd, left, None, 0,
                                         None))
    torch.cuda.synchronize()
    return dQ, dK, dV


@pytest.mark.parametrize("dtype,shape", [(_lib.BF16, (2, 256, 4, 2, 128, 100)), (_lib.F32, (2, 40, 4, 2, 16, 40))])
def test_static_scratch_matches_allocating_entry_point_twice(dtype, shape):
    L = _lib.lib()
    B, T, H, Hkv, hd, left = shape
    first = _case(dtype, B, T, H, Hkv, hd, left, seed=1)
    second = _case(dtype, B, T, H, Hkv, hd, left, seed=2)   # different data: stale scratch would show
    for data in (first, second):
        ref = _bwd("allocating", dtype, *data, left)
        got = _bwd("static", dtype, *data, left)
        for r, g in zip(ref, got):
            assert torch.isfinite(g.float()).all()
            assert torch.equal(r, g)     # same kernels, same order of summation: bit-identical


def test_static_scratch_rejects_oversized_shapes():
    L = _lib.lib()
    t = torch.zeros(8, device="cuda")
    rc = L.femto_attention_bwd_static(_lib.F32, _lib.ptr(t), _lib.ptr(t), _lib.ptr(t), _lib.ptr(t), _lib.ptr(t), _lib.ptr(t),
                                      _lib.ptr(t), _lib.ptr(t), _lib.ptr(t), 64, 4096, 16, 16, 64, 4096, None, None)
    assert rc == -2
    assert b"exceeds the built-in scratch" in L.femto_last_error(None)
