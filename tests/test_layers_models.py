import os

import numpy as np
import pytest
import torch

import keras_b200 as keras
from keras_b200 import layers, ops

RNG = np.random.default_rng(0)


def test_dense_forward_and_config_roundtrip():
    layer = layers.Dense(3, activation="relu", name="d")
    x = RNG.normal(size=(2, 4)).astype("float32")
    y = layer(x)
    k, b = layer.kernel.numpy(), layer.bias.numpy()
    np.testing.assert_allclose(ops.convert_to_numpy(y), np.maximum(x @ k + b, 0), rtol=1e-5, atol=1e-6)
    assert [v.path for v in layer.weights] == ["d/kernel", "d/bias"]
    cfg = keras.saving.serialize_keras_object(layer)
    assert cfg["module"] == "keras.layers" and cfg["class_name"] == "Dense" and cfg["registered_name"] is None
    clone = keras.saving.deserialize_keras_object(cfg)
    assert isinstance(clone, layers.Dense) and clone.units == 3


def test_batchnorm_train_and_inference():
    bn = layers.BatchNormalization(momentum=0.9, epsilon=1e-3)
    x = RNG.normal(2.0, 3.0, size=(16, 5, 5, 4)).astype("float32")
    y = ops.convert_to_numpy(bn(x, training=True))
    mean, var = x.mean((0, 1, 2)), x.var((0, 1, 2))
    np.testing.assert_allclose(y, (x - mean) / np.sqrt(var + 1e-3), rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(bn.moving_mean.numpy(), 0.1 * mean, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(bn.moving_variance.numpy(), 0.9 + 0.1 * var, rtol=1e-4, atol=1e-5)
    assert [v.name for v in bn.weights] == ["gamma", "beta", "moving_mean", "moving_variance"]
    y2 = ops.convert_to_numpy(bn(x, training=False))
    np.testing.assert_allclose(y2, (x - bn.moving_mean.numpy()) / np.sqrt(bn.moving_variance.numpy() + 1e-3), rtol=1e-4, atol=1e-4)


def test_mixed_precision_autocast():
    keras.config.set_dtype_policy("mixed_bfloat16")
    layer = layers.Dense(4)
    y = layer(np.ones((2, 3), "float32"))
    assert y.dtype == torch.bfloat16 and layer.kernel.dtype == "float32"
    ln = layers.LayerNormalization()
    assert ln(y).dtype == torch.bfloat16 and ln.gamma.dtype == "float32"


def test_functional_and_sequential_graph():
    inp = keras.Input((8,), name="in")
    h = layers.Dense(4, name="h")(inp)
    a = layers.Dense(2, name="a")(h)
    b = layers.Dense(2, name="b")(h)
    out = layers.Add(name="sum")([a, b])
    model = keras.Model(inp, out, name="m")
    assert [l.name for l in model.layers] == ["in", "h", "a", "b", "sum"]
    x = RNG.normal(size=(3, 8)).astype("float32")
    y = ops.convert_to_numpy(model(x))
    assert y.shape == (3, 2)
    clone = keras.Model.from_config(model.get_config())
    clone.set_weights(model.get_weights())
    np.testing.assert_allclose(ops.convert_to_numpy(clone(x)), y, rtol=1e-6)
    seq = keras.Sequential([layers.Input((8,)), layers.Dense(4), layers.Dropout(0.5), layers.Dense(1)])
    assert seq(x).shape == (3, 1) and len(seq.weights) == 4
    assert seq.count_params() == 8 * 4 + 4 + 4 + 1


def test_subclassed_model_tracks_nested_layers():
    class Block(layers.Layer):
        def __init__(self):
            super().__init__()
            self.inner = [layers.Dense(4), layers.Dense(4)]

        def call(self, x):
            for l in self.inner:
                x = l(x)
            return x

    class Net(keras.Model):
        def __init__(self):
            super().__init__()
            self.block = Block()
            self.head = layers.Dense(1)

        def call(self, x, training=False):
            return self.head(self.block(x))

    net = Net()
    net(np.ones((2, 3), "float32"))
    assert len(net.trainable_variables) == 6
    assert net.trainable_variables[0].path.startswith("net/block/dense")


def test_conv_pool_layers_shapes():
    x = RNG.normal(size=(2, 9, 9, 3)).astype("float32")
    assert tuple(layers.Conv2D(4, 3, padding="same", strides=2)(x).shape) == (2, 5, 5, 4)
    assert tuple(layers.Conv2DTranspose(4, 3, strides=2, padding="same")(x).shape) == (2, 18, 18, 4)
    assert tuple(layers.Conv2DTranspose(4, 3, strides=2, padding="valid")(x).shape) == (2, 19, 19, 4)
    assert tuple(layers.DepthwiseConv2D(3, depth_multiplier=2)(x).shape) == (2, 7, 7, 6)
    assert tuple(layers.SeparableConv2D(5, 3)(x).shape) == (2, 7, 7, 5)
    assert tuple(layers.MaxPooling2D(2)(x).shape) == (2, 4, 4, 3)
    assert tuple(layers.GlobalAveragePooling2D()(x).shape) == (2, 3)
    assert tuple(layers.ZeroPadding2D(((1, 2), (0, 3)))(x).shape) == (2, 12, 12, 3)
    assert tuple(layers.Cropping2D(((1, 2), (0, 3)))(x).shape) == (2, 6, 6, 3)
    assert tuple(layers.UpSampling2D(2)(x).shape) == (2, 18, 18, 3)
    sym = keras.Input((9, 9, 3))
    assert layers.Conv2DTranspose(4, 3, strides=2, padding="same")(sym).shape == (None, 18, 18, 4)
    assert layers.Flatten()(sym).shape == (None, 243)


def test_embedding_and_einsum_dense():
    emb = layers.Embedding(10, 4, mask_zero=True)
    ids = np.array([[1, 2, 0]])
    out = emb(ids)
    assert tuple(out.shape) == (1, 3, 4)
    np.testing.assert_array_equal(ops.convert_to_numpy(out._keras_mask), [[True, True, False]])
    ed = layers.EinsumDense("abc,cde->abde", output_shape=(None, 2, 3), bias_axes="de")
    y = ed(RNG.normal(size=(2, 5, 4)).astype("float32"))
    assert tuple(y.shape) == (2, 5, 2, 3) and tuple(ed.kernel.shape) == (4, 2, 3) and tuple(ed.bias.shape) == (2, 3)
    x = RNG.normal(size=(2, 5, 4)).astype("float32")
    np.testing.assert_allclose(ops.convert_to_numpy(ed(x)), np.einsum("abc,cde->abde", x, ed.kernel.numpy()) + ed.bias.numpy(), rtol=1e-5, atol=1e-5)


def test_lora_and_int8_quantization():
    layer = layers.Dense(8)
    x = RNG.normal(size=(16, 12)).astype("float32")
    ref = ops.convert_to_numpy(layer(x))
    layer.enable_lora(2)
    assert len(layer.trainable_weights) == 3 and not layer._kernel.trainable
    np.testing.assert_allclose(ops.convert_to_numpy(layer(x)), ref, rtol=1e-5, atol=1e-6)
    q = layers.Dense(8)
    ref = ops.convert_to_numpy(q(x))
    q.quantize("int8")
    assert q._kernel.dtype == "int8" and q.dtype_policy.name == "int8_from_float32"
    out = ops.convert_to_numpy(q(x))
    assert np.abs(out - ref).max() < 0.1 * np.abs(ref).max() + 0.05


def test_float8_dense_updates_scales_through_optimizer():
    inp = keras.Input((16,))
    dense = layers.Dense(8, dtype=keras.dtype_policies.QuantizedFloat8DTypePolicy("float8", "float32", amax_history_length=4))
    model = keras.Model(inp, dense(inp))
    assert len(dense.weights) == 8
    model.compile(optimizer="sgd", loss="mse")
    x, y = RNG.normal(size=(32, 16)).astype("float32"), RNG.normal(size=(32, 8)).astype("float32")
    model.train_on_batch(x, y)
    hist = dense.inputs_amax_history.numpy()
    assert hist[0] == pytest.approx(np.abs(x).max(), rel=1e-5) and hist.shape == (4,)
    model.train_on_batch(x, y)
    assert dense.inputs_scale.numpy() == pytest.approx(np.abs(x).max() / 448.0, rel=1e-4)
