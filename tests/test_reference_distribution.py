"""``keras.distribution`` bookkeeping (mesh, layouts, layout map lookups) against the reference, on one process."""

import numpy as np
import pytest

import keras_b200 as keras
from tests import oracle


def _mesh(k, shape=(2, 4), names=("data", "model")):
    return k.distribution.DeviceMesh(shape, list(names), devices=[f"gpu:{i}" for i in range(int(np.prod(shape)))])


def test_layout_map_lookup_rules_match_reference():
    rk = oracle.ref()
    outcomes = []
    for k in (rk, keras):
        lm = k.distribution.LayoutMap(_mesh(k))
        lm["dense.*kernel"] = (None, "model")
        lm["dense.*bias"] = k.distribution.TensorLayout(("model",))
        lm["conv"] = ("model", None, None, None)
        seen = []
        for path in ["dense/kernel", "dense_1/kernel", "my_dense/kernel", "dense/kernel/extra", "conv", "conv2d", "dense/bias", "nothing"]:
            layout = lm[path]
            seen.append((path, None if layout is None else tuple(layout.axes)))
        lm["dense/k.*"] = (None, None)
        try:
            lm["dense/kernel"]
            seen.append("no error")
        except ValueError:
            seen.append("multiple")
        with pytest.raises(ValueError):
            lm["conv"] = (None,)
        with pytest.raises(ValueError):
            lm["bad"] = ("not_an_axis",)
        outcomes.append((seen, len(lm), list(lm)))
    assert outcomes[1] == outcomes[0]


def test_mesh_and_strategy_facts_match_reference():
    rk = oracle.ref()
    facts = []
    for k in (rk, keras):
        mesh = _mesh(k)
        with pytest.raises(ValueError):
            k.distribution.DeviceMesh((2, 2), ["a"], devices=["gpu:0"] * 4)
        with pytest.raises(ValueError):
            k.distribution.DeviceMesh((3,), ["a"], devices=["gpu:0", "gpu:1"])
        lm = k.distribution.LayoutMap(mesh)
        lm["w"] = ("model", None)
        mp = k.distribution.ModelParallel(layout_map=lm, batch_dim_name="data")
        dp = k.distribution.DataParallel(devices=[f"gpu:{i}" for i in range(4)])
        var = k.Variable(np.zeros((4, 4), "float32"), name="w")
        other = k.Variable(np.zeros((3,), "float32"), name="other")
        facts.append((mesh.shape, list(mesh.axis_names), mp.batch_dim_name, mp.num_model_replicas, dp.batch_dim_name, dp.num_model_replicas,
                      tuple(mp.get_variable_layout(var).axes), tuple(mp.get_variable_layout(other).axes), tuple(mp.get_data_layout((8, 5, 5)).axes),
                      tuple(dp.get_data_layout((8, 3)).axes), tuple(dp.get_variable_layout(var).axes), mp.get_tensor_layout("nope") is None))
        with mp.scope():
            assert k.distribution.distribution() is mp
        assert k.distribution.distribution() is None
    assert facts[1] == facts[0]
