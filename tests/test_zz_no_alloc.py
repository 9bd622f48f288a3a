"""The allocation-free BatchNorm-backward entry point of libkb200.so, called through its exported C symbol.

Collected last (file name) so that it also runs after every other GPU test has used the library.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from keras_b200.kernels import build

    build.build()
    lib = ctypes.CDLL(build.LIB_PATH)
    lib.kb200_last_error.restype = ctypes.c_char_p
    for name in ("kb200_bn_bwd_static", "kb200_bn_bwd_static_setup", "kb200_bn_bwd_static_max_channels", "kb200_bn_bwd_reduce", "kb200_bn_bwd_apply"):
        getattr(lib, name).restype = ctypes.c_int
    return lib


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _case(M, C, dtype, relu, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(M, C, device="cuda", generator=g).to(dtype)
    dy = torch.randn(M, C, device="cuda", generator=g).to(dtype)
    y = torch.randn(M, C, device="cuda", generator=g).to(dtype) if relu else None
    xf = x.float()
    mean = xf.mean(0).contiguous()
    invstd = torch.rsqrt(xf.var(0, unbiased=False) + 1e-3).contiguous()
    gamma = (torch.rand(C, device="cuda", generator=g) + 0.5).contiguous()
    return x, dy, y, mean, invstd, gamma


def _existing(lib, x, dy, y, mean, invstd, gamma, stream):
    M, C = x.shape
    dt = 1 if x.dtype == torch.bfloat16 else 0
    sums = torch.empty(2 * C, dtype=torch.float32, device="cuda")
    coef = torch.empty(3 * C, dtype=torch.float32, device="cuda")
    dx, dres = torch.empty_like(x), torch.empty_like(x)
    assert lib.kb200_bn_bwd_reduce(_p(dy), _p(x), _p(y), _p(mean), _p(invstd), ctypes.c_longlong(M), ctypes.c_int(C), ctypes.c_int(dt), _p(sums), stream) == 0
    assert lib.kb200_bn_bwd_apply(_p(dy), _p(x), _p(y), _p(mean), _p(invstd), _p(gamma), _p(sums), _p(coef), _p(dx), _p(dres), ctypes.c_longlong(M), ctypes.c_int(C), ctypes.c_int(dt), stream) == 0
    return dx, dres, sums[C:].clone(), sums[:C].clone()


def _static(lib, x, dy, y, mean, invstd, gamma, stream):
    M, C = x.shape
    dt = 1 if x.dtype == torch.bfloat16 else 0
    dx, dres = torch.empty_like(x), torch.empty_like(x)
    dgamma = torch.empty(C, dtype=torch.float32, device="cuda")
    dbeta = torch.empty(C, dtype=torch.float32, device="cuda")
    rc = lib.kb200_bn_bwd_static(_p(dy), _p(x), _p(y), _p(mean), _p(invstd), _p(gamma), _p(dx), _p(dres), _p(dgamma), _p(dbeta), ctypes.c_longlong(M), ctypes.c_int(C), ctypes.c_int(dt), stream)
    assert rc == 0, lib.kb200_last_error()
    return dx, dres, dgamma, dbeta


def _reference(x, dy, y, mean, invstd, gamma):
    xf, d = x.float(), dy.float()
    if y is not None:
        d = d * (y.float() > 0)
    xhat = (xf - mean) * invstd
    dbeta, dgamma = d.sum(0), (d * xhat).sum(0)
    M = x.shape[0]
    dx = gamma * invstd * (d - dbeta / M - xhat * dgamma / M)
    return dx, d, dgamma, dbeta


def test_bn_bwd_static_matches_existing_entry_point_twice():
    lib = _lib()
    torch.cuda.set_device(0)
    assert lib.kb200_bn_bwd_static_setup() == 0, lib.kb200_last_error()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # two calls in a row sharing the static scratch: a wide bf16 case, then a narrower fp32 one
    for (M, C, dtype, relu, seed) in [(4100, 512, torch.bfloat16, True, 1), (1537, 64, torch.float32, False, 2)]:
        args = _case(M, C, dtype, relu, seed)
        got = _static(lib, *args, stream)
        want = _existing(lib, *args, stream)
        ref = _reference(*args)
        torch.cuda.synchronize()
        lo = dtype == torch.bfloat16
        for g, w, r in zip(got, want, ref):
            torch.testing.assert_close(g.float(), w.float(), rtol=2e-2 if lo else 1e-4, atol=2e-2 if lo else 1e-3)
            torch.testing.assert_close(g.float(), r, rtol=3e-2 if lo else 1e-3, atol=6e-2 if lo else 5e-3)


def test_bn_bwd_static_rejects_oversize_channels():
    lib = _lib()
    torch.cuda.set_device(0)
    cap = lib.kb200_bn_bwd_static_max_channels()
    assert cap == 4096
    t = torch.zeros(8, device="cuda")
    rc = lib.kb200_bn_bwd_static(_p(t), _p(t), _p(None), _p(t), _p(t), _p(None), _p(t), _p(None), _p(None), _p(t), ctypes.c_longlong(1), ctypes.c_int(cap + 8), ctypes.c_int(0), ctypes.c_void_p(0))
    assert rc != 0
    assert b"KB200_BN_STATIC_MAX_C" in lib.kb200_last_error()
    torch.cuda.synchronize()
