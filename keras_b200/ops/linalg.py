"""Linear-algebra ops (``keras.ops.linalg``); library calls (cuSOLVER/LAPACK via torch).

Semantics follow keras/src/ops/linalg.py and keras/src/backend/torch/linalg.py.
"""

import torch

from keras_b200.core.dtypes import result_type, to_torch_dtype
from keras_b200.ops._dispatch import op
from keras_b200.ops.numpy import _floatize, _t


def _square_check(x, name):
    if x.ndim < 2:
        raise ValueError(f"Input must have rank >= 2. Received: input.shape = {tuple(x.shape)} with rank = {x.ndim}")
    if x.shape[-1] != x.shape[-2]:
        raise ValueError(f"Input must be a square matrix. Received: input.shape = {tuple(x.shape)}")


@op("linalg")
def cholesky(x, upper=False):
    x = _floatize(x)
    _square_check(x, "cholesky")
    return torch.linalg.cholesky(x, upper=upper)


@op("linalg")
def cholesky_inverse(x, upper=False):
    x = _floatize(x)
    return torch.cholesky_inverse(x, upper=upper)


@op("linalg")
def det(x):
    x = _floatize(x)
    _square_check(x, "det")
    return torch.det(x)


@op("linalg")
def eig(x):
    x = _floatize(x)
    _square_check(x, "eig")
    return torch.linalg.eig(x)


@op("linalg")
def eigh(x):
    x = _floatize(x)
    _square_check(x, "eigh")
    return torch.linalg.eigh(x)


@op("linalg")
def inv(x):
    x = _floatize(x)
    _square_check(x, "inv")
    return torch.linalg.inv(x)


@op("linalg")
def lu_factor(x):
    x = _floatize(x)
    LU, pivots = torch.linalg.lu_factor(x)
    return LU, (pivots - 1).to(torch.int32)


@op("linalg")
def norm(x, ord=None, axis=None, keepdims=False):
    x = _floatize(x)
    if isinstance(axis, list):
        axis = tuple(axis)
    if isinstance(axis, tuple) and len(axis) == 2 or (axis is None and x.ndim == 2 and ord is not None):
        if ord is None:
            ord = "fro"
        return torch.linalg.matrix_norm(x, ord=ord, dim=axis if axis is not None else (-2, -1), keepdim=keepdims)
    if axis is None and ord is None:
        r = torch.linalg.vector_norm(x.reshape(-1), ord=2)
        return r.reshape((1,) * x.ndim) if keepdims else r
    if ord is None:
        ord = 2
    if isinstance(ord, str):
        raise ValueError(f"Invalid `ord` argument for vector norm. Received: ord={ord}")
    return torch.linalg.vector_norm(x, ord=ord, dim=axis, keepdim=keepdims)


@op("linalg")
def qr(x, mode="reduced"):
    if mode not in {"reduced", "complete"}:
        raise ValueError(f"`mode` argument value not supported. Expected one of {{'reduced', 'complete'}}. Received: mode={mode}")
    return torch.linalg.qr(_floatize(x), mode=mode)


@op("linalg")
def solve(a, b):
    a, b = _floatize(a), _floatize(b)
    d = to_torch_dtype(result_type(a.dtype, b.dtype))
    return torch.linalg.solve(a.to(d), b.to(d))


@op("linalg")
def solve_triangular(a, b, lower=False):
    a, b = _floatize(a), _floatize(b)
    d = to_torch_dtype(result_type(a.dtype, b.dtype))
    a, b = a.to(d), b.to(d)
    if b.ndim == a.ndim - 1:
        return torch.linalg.solve_triangular(a, b.unsqueeze(-1), upper=not lower).squeeze(-1)
    return torch.linalg.solve_triangular(a, b, upper=not lower)


@op("linalg")
def svd(x, full_matrices=True, compute_uv=True):
    x = _floatize(x)
    if not compute_uv:
        return torch.linalg.svdvals(x)
    return torch.linalg.svd(x, full_matrices=full_matrices)


@op("linalg")
def lstsq(a, b, rcond=None):
    a, b = _floatize(a), _floatize(b)
    d = to_torch_dtype(result_type(a.dtype, b.dtype))
    a, b = a.to(d), b.to(d)
    squeeze = b.ndim == 1
    if squeeze:
        b = b.unsqueeze(-1)
    sol = torch.linalg.pinv(a, rtol=rcond) @ b if rcond is not None else torch.linalg.lstsq(a, b).solution
    return sol.squeeze(-1) if squeeze else sol


@op("linalg")
def pinv(x, rcond=None, hermitian=False):
    return torch.linalg.pinv(_floatize(x), rtol=rcond, hermitian=hermitian)


@op("linalg")
def matrix_power(x, n):
    x = _t(x)
    _square_check(x, "matrix_power")
    if n < 0:
        x = _floatize(x)
    return torch.linalg.matrix_power(x, n)


@op("linalg")
def matrix_rank(x, tol=None):
    return torch.linalg.matrix_rank(_floatize(x), atol=tol).to(torch.int32)


def jvp(fun, primals, tangents, has_aux=False):
    from torch.func import jvp as _jvp

    primals = tuple(_t(p) for p in primals)
    tangents = tuple(_t(t) for t in tangents)
    return _jvp(fun, primals, tangents, has_aux=has_aux)


from keras_b200.core.export_registry import keras_export as _ke

_ke(["keras.ops.jvp", "keras.ops.linalg.jvp"])(jvp)
