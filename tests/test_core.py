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
