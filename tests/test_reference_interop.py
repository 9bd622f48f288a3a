"""Checkpoint and config interchange with the reference.

* ``.keras`` archives written here are loaded by the reference in a child process (its ``h5py`` import is served by this
  package's HDF5 reader, because neither h5py nor libhdf5 is installed) and must give the same predictions and optimizer
  step; the bytes of the HDF5 writer are therefore checked against this package's own reader only.
* configs serialized by the reference are deserialized here, weights transferred, predictions compared.
* a config that names a module outside the allow-list must not get that module imported.
"""

import json
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

import keras_b200 as keras
from tests import oracle

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent(
    """
    import os, sys, types, json
    import numpy as np
    sys.path.insert(0, {repo!r})
    from keras_b200.saving import h5py_compat
    h5py_compat.install()
    sys.path.append({ref!r})
    import keras
    assert keras.__file__.startswith({ref!r}), keras.__file__
    model = keras.saving.load_model({path!r})
    x = np.load({x!r})
    got = model.predict(x, verbose=0)
    want = np.load({y!r})
    out = {{"max_err": float(np.abs(got - want).max()), "iterations": int(model.optimizer.iterations.numpy()) if model.optimizer is not None else -1,
           "class": type(model).__name__, "weights": len(model.weights)}}
    print("RESULT " + json.dumps(out))
    """
)


def _sequential(k):
    return k.Sequential([k.Input((6, 6, 2)), k.layers.Conv2D(3, 3, padding="same"), k.layers.BatchNormalization(), k.layers.ReLU(),
                         k.layers.GlobalAveragePooling2D(), k.layers.Dense(4, activation="softmax")])


def _functional(k):
    inp = k.Input((5, 8))
    shared = k.layers.Dense(8, activation="relu", name="shared")
    h = shared(inp)
    h = k.layers.MultiHeadAttention(2, 4, name="mha")(h, h, use_causal_mask=True)
    h = k.layers.LayerNormalization()(k.layers.Add()([h, shared(h)]))
    h = k.layers.BatchNormalization()(h)
    out = k.layers.Dense(3, name="head")(k.layers.GlobalAveragePooling1D()(h))
    return k.Model(inp, out, name="tiny_functional")


@pytest.mark.parametrize("kind", ["sequential", "functional"])
def test_reference_loads_archives_written_here(kind, tmp_path):
    oracle.ref()  # skips when the reference is absent
    rng = np.random.default_rng(0)
    if kind == "sequential":
        model, x, y = _sequential(keras), rng.normal(size=(8, 6, 6, 2)).astype("float32"), rng.integers(0, 4, (8,))
        model.compile(optimizer=keras.optimizers.Adam(1e-2), loss="sparse_categorical_crossentropy")
    else:
        model, x, y = _functional(keras), rng.normal(size=(8, 5, 8)).astype("float32"), rng.normal(size=(8, 3)).astype("float32")
        model.compile(optimizer=keras.optimizers.SGD(1e-2, momentum=0.9), loss="mse")
    model.fit(x, y, batch_size=4, epochs=1, verbose=0)
    path = str(tmp_path / f"{kind}.keras")
    model.save(path)
    np.save(tmp_path / "x.npy", x)
    np.save(tmp_path / "y.npy", model.predict(x, verbose=0))
    script = CHILD.format(repo=REPO, ref=oracle.reference_path(), path=path, x=str(tmp_path / "x.npy"), y=str(tmp_path / "y.npy"))
    env = dict(os.environ, KERAS_BACKEND="torch", KERAS_HOME=str(tmp_path / "home"), KERAS_TORCH_DEVICE="cpu", PYTHONPATH="")
    proc = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=env, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    line = [l for l in proc.stdout.splitlines() if l.startswith("RESULT ")][-1]
    result = json.loads(line[len("RESULT "):])
    assert result["max_err"] < 1e-5, result
    assert result["iterations"] == 2, result
    assert result["weights"] == len(model.weights)
    assert result["class"] == ("Sequential" if kind == "sequential" else "Functional")


@pytest.mark.parametrize("kind", ["sequential", "functional"])
def test_configs_serialized_by_the_reference_load_here(kind):
    rk = oracle.ref()
    theirs = _sequential(rk) if kind == "sequential" else _functional(rk)
    theirs.compile(optimizer=rk.optimizers.Adam(3e-3), loss="mse")
    config = json.loads(json.dumps(rk.saving.serialize_keras_object(theirs)))
    if kind == "functional":
        assert config["module"] == "keras.src.models.functional"
    ours = keras.saving.deserialize_keras_object(config)
    assert type(ours).__name__ == type(theirs).__name__
    ours.set_weights(theirs.get_weights())
    shape = (4, 6, 6, 2) if kind == "sequential" else (4, 5, 8)
    x = np.random.default_rng(1).normal(size=shape).astype("float32")
    np.testing.assert_allclose(ours.predict(x, verbose=0), theirs.predict(x, verbose=0), rtol=1e-4, atol=1e-5)
    assert type(ours.optimizer).__name__ == "Adam" and abs(float(ours.optimizer.learning_rate) - 3e-3) < 1e-9
    # and our own config names the same classes the reference would
    mine = keras.saving.serialize_keras_object(ours)
    assert (mine["module"], mine["class_name"], mine["registered_name"]) == (config["module"], config["class_name"], config["registered_name"])


def test_unknown_modules_are_never_imported(tmp_path):
    trap = tmp_path / "kb200_trap_module.py"
    trap.write_text("import os\nopen(os.path.join(os.path.dirname(__file__), 'imported.flag'), 'w').write('x')\n"
                    "class Thing:\n    @classmethod\n    def from_config(cls, config):\n        return cls()\n")
    sys.path.insert(0, str(tmp_path))
    try:
        for safe_mode in (True, False):
            with pytest.raises(TypeError):
                keras.saving.deserialize_keras_object({"module": "kb200_trap_module", "class_name": "Thing", "config": {}, "registered_name": "Thing"},
                                                      safe_mode=safe_mode)
        assert not (tmp_path / "imported.flag").exists()
        assert "kb200_trap_module" not in sys.modules
        # an allow-listed package still only yields savable classes
        with pytest.raises(TypeError):
            keras.saving.deserialize_keras_object({"module": "keras_b200.saving.hdf5", "class_name": "File", "config": {}, "registered_name": "File"})
    finally:
        sys.path.remove(str(tmp_path))


CHILD_SAVE = textwrap.dedent(
    """
    import os, sys, json
    import numpy as np
    sys.path.insert(0, {repo!r})
    from keras_b200.saving import h5py_compat
    h5py_compat.install()
    sys.path.append({ref!r})
    import keras
    assert keras.__file__.startswith({ref!r}), keras.__file__
    keras.utils.set_random_seed(5)
    rng = np.random.default_rng(0)
    if {kind!r} == "sequence":
        i = keras.Input((12, 6)); h = keras.layers.Bidirectional(keras.layers.LSTM(5, return_sequences=True))(i)
        h = keras.layers.MultiHeadAttention(2, 4)(h, h); h = keras.layers.LayerNormalization()(h)
        model = keras.Model(i, keras.layers.Dense(3, activation="softmax")(keras.layers.GlobalAveragePooling1D()(h)))
        x, y = rng.normal(size=(8, 12, 6)).astype("float32"), rng.integers(0, 3, (8,))
        model.compile(optimizer=keras.optimizers.Adam(1e-2), loss="sparse_categorical_crossentropy")
    else:
        i = keras.Input((16, 16, 3)); h = keras.layers.Conv2D(8, 3, padding="same")(i); h = keras.layers.BatchNormalization()(h); h = keras.layers.ReLU()(h)
        h = keras.layers.DepthwiseConv2D(3)(h); h = keras.layers.SeparableConv2D(6, 3)(h); h = keras.layers.GroupNormalization(2)(h)
        h = keras.layers.Conv2DTranspose(4, 3, strides=2, padding="same")(h); h = keras.layers.PReLU()(h)
        model = keras.Model(i, keras.layers.Dense(2)(keras.layers.Flatten()(keras.layers.MaxPooling2D()(h))))
        x, y = rng.normal(size=(8, 16, 16, 3)).astype("float32"), rng.normal(size=(8, 2)).astype("float32")
        model.compile(optimizer=keras.optimizers.SGD(1e-2, momentum=0.9), loss="mse")
    model.fit(x, y, batch_size=4, epochs=1, verbose=0)
    model.save({path!r})
    model.save_weights({wpath!r})
    np.save({x!r}, x)
    np.save({y!r}, model.predict(x, verbose=0))
    print("RESULT " + json.dumps({{"weights": len(model.weights), "iterations": int(model.optimizer.iterations.numpy())}}))
    """
)


@pytest.mark.parametrize("kind", ["sequence", "vision"])
def test_archives_written_by_the_reference_load_here(kind, tmp_path):
    """The reverse direction: the reference's own saver decides the layout of the archive (its ``h5py`` calls are served by this
    package's HDF5 writer, since no h5py is installed); this framework loads the ``.keras`` file and the ``.weights.h5`` file and
    predicts the same."""
    oracle.ref()
    path, wpath = str(tmp_path / f"{kind}.keras"), str(tmp_path / f"{kind}.weights.h5")
    script = CHILD_SAVE.format(repo=REPO, ref=oracle.reference_path(), kind=kind, path=path, wpath=wpath, x=str(tmp_path / "x.npy"), y=str(tmp_path / "y.npy"))
    env = dict(os.environ, KERAS_BACKEND="torch", KERAS_HOME=str(tmp_path / "home"), KERAS_TORCH_DEVICE="cpu", PYTHONPATH="")
    proc = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=env, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    result = json.loads([l for l in proc.stdout.splitlines() if l.startswith("RESULT ")][-1][len("RESULT "):])
    x, want = np.load(tmp_path / "x.npy"), np.load(tmp_path / "y.npy")
    model = keras.saving.load_model(path)
    np.testing.assert_allclose(model.predict(x, verbose=0), want, rtol=1e-4, atol=1e-5)
    assert len(model.weights) == result["weights"]
    assert int(model.optimizer.iterations) == result["iterations"] == 2
    # weights only, into a freshly initialised copy of the architecture
    fresh = keras.Model.from_config(model.get_config())
    assert not np.allclose(fresh.predict(x, verbose=0), want, atol=1e-3)
    fresh.load_weights(wpath)
    np.testing.assert_allclose(fresh.predict(x, verbose=0), want, rtol=1e-4, atol=1e-5)
