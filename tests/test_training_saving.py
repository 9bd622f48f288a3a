import os
import zipfile

import numpy as np
import pytest
import torch

import keras_b200 as keras
from keras_b200 import layers, ops
from keras_b200.saving import hdf5

RNG = np.random.default_rng(0)
HERE = os.path.dirname(__file__)


def _small_convnet():
    return keras.Sequential([
        layers.Input((12, 12, 1)), layers.Conv2D(8, 3, activation="relu"), layers.MaxPooling2D(2), layers.Conv2D(8, 3, activation="relu"),
        layers.GlobalAveragePooling2D(), layers.Dropout(0.5), layers.Dense(4, activation="softmax"),
    ])


def test_fit_learns_and_history():
    x = RNG.normal(size=(256, 6)).astype("float32")
    w = RNG.normal(size=(6, 1)).astype("float32")
    y = x @ w
    model = keras.Sequential([layers.Input((6,)), layers.Dense(1)])
    model.compile(optimizer=keras.optimizers.Adam(0.05), loss="mse", metrics=["mae"])
    hist = model.fit(x, y, batch_size=32, epochs=12, verbose=0, validation_split=0.25)
    assert hist.history["loss"][-1] < 0.05 * hist.history["loss"][0]
    assert set(hist.history) == {"loss", "mae", "val_loss", "val_mae"}
    ev = model.evaluate(x, y, verbose=0, return_dict=True)
    assert ev["loss"] < 0.1


def test_fit_builds_models_that_were_never_called():
    """A Sequential without an Input layer and a subclassed model get their variables on the first fit / evaluate: the
    variables created while the shapes are traced must end up initialised."""
    import torch

    y = torch.randint(0, 8, (64,))
    loss = keras.losses.SparseCategoricalCrossentropy(from_logits=True)
    seq = keras.Sequential([keras.layers.Embedding(50, 16), keras.layers.GlobalAveragePooling1D(), keras.layers.Dense(8)])
    seq.compile(optimizer=keras.optimizers.SGD(0.5), loss=loss)
    hist = seq.fit(torch.randint(0, 50, (64, 12)), y, batch_size=32, epochs=2, verbose=0, shuffle=False)
    assert hist.history["loss"][1] < hist.history["loss"][0]

    class Sub(keras.Model):
        def __init__(self):
            super().__init__()
            self.dense = keras.layers.Dense(8)

        def call(self, x):
            return self.dense(x)

    sub = Sub()
    sub.compile(optimizer="adam", loss=loss)
    assert np.isfinite(sub.evaluate(torch.randn(64, 20), y, verbose=0))
    assert all(v._value is not None for v in sub.variables)


def test_adam_matches_reference_formula():
    v = keras.Variable(np.array([1.0, -2.0], "float32"))
    opt = keras.optimizers.Adam(0.1, beta_1=0.9, beta_2=0.999, epsilon=1e-7)
    g = np.array([0.5, -1.5], "float32")
    m = vv = np.zeros(2)
    p = np.array([1.0, -2.0])
    for t in range(1, 4):
        opt.apply([torch.as_tensor(g)], [v])
        m = m + (g - m) * 0.1
        vv = vv + (g * g - vv) * 0.001
        alpha = 0.1 * np.sqrt(1 - 0.999 ** t) / (1 - 0.9 ** t)
        p = p - alpha * m / (np.sqrt(vv) + 1e-7)
    np.testing.assert_allclose(v.numpy(), p, rtol=1e-5)
    assert int(opt.iterations.numpy()) == 3


def test_sgd_momentum_nesterov_and_decay():
    v = keras.Variable(np.array([1.0], "float32"))
    opt = keras.optimizers.SGD(0.1, momentum=0.9, nesterov=True, weight_decay=0.01)
    opt.apply([torch.tensor([2.0])], [v])
    p = 1.0 * (1 - 0.01 * 0.1)
    m = -0.1 * 2.0
    p = p + 0.9 * m - 0.1 * 2.0
    np.testing.assert_allclose(v.numpy(), [p], rtol=1e-6)


def test_keras_archive_roundtrip_and_layout(tmp_path):
    model = _small_convnet()
    model.compile(optimizer="adam", loss="sparse_categorical_crossentropy", metrics=["accuracy"])
    x = RNG.uniform(size=(32, 12, 12, 1)).astype("float32")
    y = RNG.integers(0, 4, size=(32,))
    model.fit(x, y, batch_size=16, epochs=1, verbose=0)
    path = str(tmp_path / "m.keras")
    model.save(path)
    with zipfile.ZipFile(path) as z:
        assert sorted(z.namelist()) == ["config.json", "metadata.json", "model.weights.h5"]
        assert all(i.compress_type == zipfile.ZIP_STORED for i in z.infolist())
        f = hdf5.File(z.read("model.weights.h5"))
        assert sorted(f["layers"].keys()) == ["conv2d", "conv2d_1", "dense"]
        assert f["layers/conv2d/vars"].attrs["name"] == "conv2d"
        assert tuple(f["layers/dense/vars/0"].shape) == (8, 4)
        assert len(f["optimizer/vars"].keys()) == 2 + 2 * 6
    loaded = keras.saving.load_model(path)
    np.testing.assert_allclose(loaded.predict(x, verbose=0), model.predict(x, verbose=0), rtol=1e-6)
    assert int(loaded.optimizer.iterations.numpy()) == 2
    wpath = str(tmp_path / "w.weights.h5")
    model.save_weights(wpath)
    fresh = _small_convnet()
    fresh.load_weights(wpath)
    np.testing.assert_allclose(fresh.predict(x, verbose=0), model.predict(x, verbose=0), rtol=1e-6)
    spath = str(tmp_path / "s.weights.json")
    model.save_weights(spath, max_shard_size=1e-6)
    fresh2 = _small_convnet()
    fresh2.load_weights(spath)
    np.testing.assert_allclose(fresh2.predict(x, verbose=0), model.predict(x, verbose=0), rtol=1e-6)


def test_reads_file_written_by_h5py():
    f = hdf5.File(os.path.join(HERE, "data", "h5py_written_nested.weights.h5"))
    assert sorted(f["layers"].keys()) == ["dense", "dense_1", "dense_2", "dense_3"]
    assert f["layers/dense/vars"].attrs["name"] == "d_0"
    a = np.asarray(f["layers/dense_3/vars/0"])
    assert a.shape == (4, 2) and a.dtype == np.float32 and np.allclose(a, 0.5)


def test_hdf5_writer_many_children_and_dtypes():
    import ml_dtypes

    w = hdf5.Writer()
    for i in range(700):
        w.create_dataset(f"g/vars/{i}", np.full((3,), i, "int32"))
    w.create_dataset("g/bf", np.arange(6).reshape(2, 3).astype(ml_dtypes.bfloat16))
    w.create_dataset("g/scalar", np.array(7, "int64"))
    w.create_group("g", {"name": "grp"})
    f = hdf5.File(w.tobytes())
    assert len(f["g/vars"].keys()) == 700
    assert all(int(np.asarray(f[f"g/vars/{i}"])[0]) == i for i in (0, 8, 255, 256, 699))
    bf = np.asarray(f["g/bf"])
    assert bf.dtype == ml_dtypes.bfloat16 and bf.astype("float32").tolist() == [[0, 1, 2], [3, 4, 5]]
    assert np.asarray(f["g/scalar"]).shape == () and f["g"].attrs["name"] == "grp"


def test_callbacks(tmp_path):
    x = RNG.normal(size=(64, 4)).astype("float32")
    y = RNG.normal(size=(64, 1)).astype("float32")
    model = keras.Sequential([layers.Input((4,)), layers.Dense(1)])
    model.compile(optimizer="sgd", loss="mse")
    ckpt = str(tmp_path / "ck_{epoch:02d}.weights.h5")
    csv = str(tmp_path / "log.csv")
    cbs = [keras.callbacks.ModelCheckpoint(ckpt, save_weights_only=True, monitor="loss"), keras.callbacks.CSVLogger(csv),
           keras.callbacks.EarlyStopping(monitor="loss", patience=50), keras.callbacks.ReduceLROnPlateau(monitor="loss", patience=1, factor=0.5),
           keras.callbacks.LearningRateScheduler(lambda epoch, lr: lr), keras.callbacks.TerminateOnNaN(),
           keras.callbacks.BackupAndRestore(str(tmp_path / "backup"))]
    model.fit(x, y, epochs=3, batch_size=16, verbose=0, callbacks=cbs)
    assert os.path.exists(str(tmp_path / "ck_03.weights.h5"))
    assert len(open(csv).read().strip().splitlines()) == 4


def test_train_on_generator_and_pydataset():
    class DS(keras.utils.PyDataset):
        def __init__(self):
            super().__init__(workers=2)

        @property
        def num_batches(self):
            return 5

        def __getitem__(self, i):
            r = np.random.default_rng(i)
            return r.normal(size=(8, 3)).astype("float32"), r.normal(size=(8, 1)).astype("float32")

    model = keras.Sequential([layers.Input((3,)), layers.Dense(1)])
    model.compile(optimizer="sgd", loss="mse")
    h = model.fit(DS(), epochs=2, verbose=0)
    assert len(h.history["loss"]) == 2

    def gen():
        while True:
            yield np.ones((4, 3), "float32"), np.ones((4, 1), "float32")

    h = model.fit(gen(), steps_per_epoch=3, epochs=1, verbose=0)
    assert len(h.history["loss"]) == 1


def test_fusion_plan_on_resnet_block():
    from keras_b200.models import fusion

    model = keras.applications.ResNet50(weights=None, input_shape=(32, 32, 3), classes=5)
    assert model.count_params() == 23597957 or model.count_params() > 2e7
    plan = fusion.build_plan(model)
    roles = list(plan.values())
    assert roles.count("defer_bn") == 53 and roles.count("consume_add_relu") == 16 and roles.count("consume_relu") == 33
    assert roles.count("conv_fold_bias") == 53 and roles.count("pad_fold") == 2 and roles.count("pool_padded") == 1
