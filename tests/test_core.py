import json
import os

import numpy as np
import pytest
import torch

import keras_b200 as keras
from keras_b200 import tree
from keras_b200.core import dtypes

HERE = os.path.dirname(__file__)


def test_result_type_matches_reference_table():
    # table generated once by running the reference's `keras.backend.result_type`
    golden = json.load(open(os.path.join(HERE, "golden_result_type.json")))
    conv = lambda s: int if s == "pyint" else float if s == "pyfloat" else s
    for key, expected in golden.items():
        parts = [conv(p) for p in key.split(",")]
        try:
            got = dtypes.result_type(*parts)
        except ValueError:
            got = "ERR"
        assert got == expected, (key, got, expected)


def test_float8_has_no_implicit_promotion():
    with pytest.raises(ValueError):
        dtypes.result_type("float8_e4m3fn", "float32")


def test_variable_basics():
    v = keras.Variable(np.ones((2, 3), "float32"), name="w")
    assert v.shape == (2, 3) and v.dtype == "float32" and v.path == "w"
    v.assign(np.full((2, 3), 2.0, "float32"))
    v.assign_add(np.ones((2, 3), "float32"))
    np.testing.assert_allclose(v.numpy(), 3.0)
    with pytest.raises(ValueError):
        v.assign(np.ones((3, 2), "float32"))
    assert (v + 1).shape == (2, 3)
    with keras.name_scope("outer"):
        w = keras.Variable(0.0, name="b")
    assert w.path == "outer/b"


def test_stateless_scope_defers_and_overrides():
    v = keras.Variable(np.zeros((2,), "float32"))
    with keras.StatelessScope(state_mapping=[(v, np.ones((2,), "float32"))]) as scope:
        np.testing.assert_allclose(v.value.numpy(), 1.0)
        v.assign(v.value + 1)
    np.testing.assert_allclose(scope.get_current_value(v).numpy(), 2.0)
    np.testing.assert_allclose(v.numpy(), 0.0)


def test_tree_roundtrip():
    s = {"b": [1, (2, 3)], "a": 4}
    flat = tree.flatten(s)
    assert flat == [4, 1, 2, 3]
    assert tree.pack_sequence_as(s, flat) == s
    assert tree.map_structure(lambda x: x * 2, s) == {"b": [2, (4, 6)], "a": 8}
    assert [p for p, _ in tree.flatten_with_path(s)] == [("a",), ("b", 0), ("b", 1, 0), ("b", 1, 1)]
    with pytest.raises(ValueError):
        tree.assert_same_structure(s, {"a": 1})


def test_autocast_scope():
    from keras_b200.core.variables import AutocastScope

    v = keras.Variable(np.ones((2,), "float32"))
    with AutocastScope("bfloat16"):
        assert v.value.dtype == torch.bfloat16
    assert v.value.dtype == torch.float32


def test_kernel_front_ends_import_without_gpu():
    import importlib

    for name in ("gemm", "ops", "dispatch", "conv", "attention", "microbench", "build", "loader"):
        importlib.import_module(f"keras_b200.kernels.{name}")


def test_convolution_tiling_choices_without_a_gpu():
    """The host-side planning of the tcgen05 convolution (which pixel tile, whether vertical taps share one TMA box) is plain
    C++ and can be asked without a device: the ResNet-50 3x3 layers with 64 and 128 channels share rows, the others do not."""
    import ctypes
    import os

    import keras_b200

    path = os.path.join(os.path.dirname(keras_b200.__file__), "kernels", "libkb200.so")
    if not os.path.exists(path):
        pytest.skip("kernel library not built")
    lib = ctypes.CDLL(path)
    shares = lib.kb200_conv_igemm_shares_rows
    assert shares(256, 56, 56, 64, 64, 3, 3, 1) == 1 and shares(256, 56, 56, 64, 64, 3, 3, -1) == 1
    assert shares(256, 28, 28, 128, 128, 3, 3, 1) == 1
    assert shares(256, 14, 14, 256, 256, 3, 3, 1) == 0      # would need a quarter more tiles
    assert shares(256, 7, 7, 512, 512, 3, 3, 1) == 0
    assert shares(256, 56, 56, 64, 256, 1, 1, 0) == 0       # nothing to share in a 1x1 filter
    assert shares(2, 20, 20, 64, 64, 3, 3, 2) == 0          # dilated rows are not adjacent
    plan = (ctypes.c_int * 3)()
    assert lib.kb200_conv_igemm_plan(256, 56, 56, 64, 64, 3, 3, 1, plan) == 0
    grid, n_tiles, bn = plan[0], plan[1], plan[2]
    assert bn == 64 and n_tiles == 1 and 0 < grid <= 148
    assert lib.kb200_conv_igemm_plan(256, 14, 14, 256, 1024, 1, 1, 0, plan) == 0
    assert plan[2] == 256 and plan[1] == 4 and plan[0] % 4 == 0
