"""Access to the reference implementation as a numerics oracle.

The reference (Keras 3 on its torch backend, CPU) is imported into the same process as ``keras_b200``; tests feed
both the same inputs and compare values and dtypes.  The reference tree is looked for beside this repository
(directory ``reference``) or where ``KERAS_B200_REFERENCE`` points; tests skip when it is absent.
"""

import os
import sys
import tempfile

import numpy as np
import pytest

_REF = None


def reference_path():
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    return os.environ.get("KERAS_B200_REFERENCE", os.path.join(os.path.dirname(here), "reference"))


def ref():
    """The reference ``keras`` module (imported once), or skip the calling test."""
    global _REF
    if _REF is not None:
        return _REF
    path = reference_path()
    if not os.path.isdir(os.path.join(path, "keras", "src")):
        pytest.skip("reference tree not found")
    os.environ.setdefault("KERAS_BACKEND", "torch")
    os.environ.setdefault("KERAS_HOME", tempfile.mkdtemp(prefix="keras_ref_home_"))
    os.environ.setdefault("KERAS_TORCH_DEVICE", "cpu")
    if path not in sys.path:
        sys.path.append(path)
    try:
        import keras
    except Exception as e:  # pragma: no cover
        pytest.skip(f"reference does not import: {e}")
    _REF = keras
    return keras


def to_np(x):
    import torch

    if isinstance(x, torch.Tensor):
        x = x.detach().cpu()
        if x.dtype == torch.bfloat16:
            x = x.float()
        return x.numpy()
    if hasattr(x, "numpy") and not isinstance(x, np.ndarray):
        try:
            return to_np(x.numpy())
        except Exception:
            pass
    return np.asarray(x)


def dtype_name(x):
    import torch

    if isinstance(x, torch.Tensor):
        return str(x.dtype).replace("torch.", "")
    return str(np.asarray(x).dtype)


def assert_same(ours, theirs, what, rtol=1e-5, atol=1e-5, check_dtype=True):
    """Compare two results that may be tensors or (nested) sequences of tensors."""
    if isinstance(theirs, (list, tuple)):
        assert isinstance(ours, (list, tuple)) and len(ours) == len(theirs), f"{what}: structure differs"
        for i, (a, b) in enumerate(zip(ours, theirs)):
            assert_same(a, b, f"{what}[{i}]", rtol, atol, check_dtype)
        return
    a, b = to_np(ours), to_np(theirs)
    assert a.shape == b.shape, f"{what}: shape {a.shape} vs reference {b.shape}"
    if check_dtype:
        assert dtype_name(ours) == dtype_name(theirs), f"{what}: dtype {dtype_name(ours)} vs reference {dtype_name(theirs)}"
    if b.dtype.kind in "fc":
        np.testing.assert_allclose(a, b, rtol=rtol, atol=atol, err_msg=what, equal_nan=True)
    else:
        np.testing.assert_array_equal(a, b, err_msg=what)
