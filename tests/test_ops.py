import numpy as np
import pytest
import torch

import keras_b200 as keras
from keras_b200 import ops

RNG = np.random.default_rng(0)


def _np(x):
    return ops.convert_to_numpy(x)


@pytest.mark.parametrize("name", ["add", "subtract", "multiply", "maximum", "minimum", "arctan2", "hypot", "logaddexp"])
def test_binary_against_numpy(name):
    a, b = RNG.normal(size=(3, 4)).astype("float32"), RNG.normal(size=(4,)).astype("float32")
    np.testing.assert_allclose(_np(getattr(ops, name)(a, b)), getattr(np, name)(a, b), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("name", ["exp", "log1p", "sin", "cosh", "tanh", "sqrt", "arcsinh", "floor", "ceil", "sign", "square", "negative"])
def test_unary_against_numpy(name):
    a = np.abs(RNG.normal(size=(5, 3)).astype("float32")) + 0.1
    np.testing.assert_allclose(_np(getattr(ops, name)(a)), getattr(np, name)(a), rtol=1e-5, atol=1e-6)


def test_reductions_and_dtypes():
    a = RNG.integers(0, 5, size=(4, 6)).astype("int32")
    assert ops.mean(a).dtype == torch.float32
    np.testing.assert_allclose(_np(ops.mean(a, axis=1)), a.mean(1), rtol=1e-6)
    assert _np(ops.sum(a.astype("int8"))).dtype == np.int32
    np.testing.assert_allclose(_np(ops.var(a.astype("float32"), axis=0)), a.var(0), rtol=1e-5)
    np.testing.assert_array_equal(_np(ops.argmax(a, axis=1)), a.argmax(1))
    assert ops.add(np.ones(2, "int32"), 1.5).dtype == torch.float32
    assert ops.add(np.ones(2, "float16"), np.ones(2, "bfloat16" if False else "float16")).dtype == torch.float16
    assert ops.divide(np.ones(2, "int32"), np.ones(2, "int32")).dtype == torch.float32


def test_shape_ops():
    a = RNG.normal(size=(2, 3, 4)).astype("float32")
    np.testing.assert_allclose(_np(ops.transpose(a, (2, 0, 1))), a.transpose(2, 0, 1))
    np.testing.assert_allclose(_np(ops.concatenate([a, a], axis=1)), np.concatenate([a, a], 1))
    np.testing.assert_allclose(_np(ops.pad(a, [(0, 0), (1, 2), (0, 0)], mode="reflect")), np.pad(a, [(0, 0), (1, 2), (0, 0)], mode="reflect"))
    np.testing.assert_allclose(_np(ops.pad(a, [(0, 0), (1, 2), (0, 0)], mode="symmetric")), np.pad(a, [(0, 0), (1, 2), (0, 0)], mode="symmetric"))
    np.testing.assert_allclose(_np(ops.take(a, [2, 0], axis=2)), np.take(a, [2, 0], axis=2))
    parts = ops.split(a, [1, 3], axis=2)
    assert [tuple(p.shape) for p in parts] == [(2, 3, 1), (2, 3, 2), (2, 3, 1)]
    np.testing.assert_allclose(_np(ops.einsum("abc,cd->abd", a, np.ones((4, 2), "float32"))), np.einsum("abc,cd->abd", a, np.ones((4, 2), "float32")), rtol=1e-5)
    np.testing.assert_allclose(_np(ops.rearrange(a, "b h (w c) -> b (h w) c", c=2)), a.reshape(2, 6, 2))


def test_symbolic_shapes():
    x = keras.KerasTensor((None, 8, 4))
    assert ops.matmul(x, np.ones((4, 5), "float32")).shape == (None, 8, 5)
    assert ops.mean(x, axis=1).shape == (None, 4)
    assert ops.reshape(x, (-1, 32)).shape == (None, 32)
    assert ops.softmax(x).dtype == "float32"
    assert (x + 1.0).shape == (None, 8, 4)
    assert ops.cast(x, "bfloat16").dtype == "bfloat16"


def test_conv_and_pool_match_direct_computation():
    x = RNG.normal(size=(2, 7, 7, 3)).astype("float32")
    k = RNG.normal(size=(3, 3, 3, 4)).astype("float32")
    out = _np(ops.conv(x, k, strides=2, padding="same"))
    assert out.shape == (2, 4, 4, 4)
    # direct computation: TF-style SAME padding (total 2 → 1 before, 1 after for in=7,s=2,k=3)
    xp = np.pad(x, [(0, 0), (1, 1), (1, 1), (0, 0)])
    ref = np.zeros_like(out)
    for i in range(4):
        for j in range(4):
            patch = xp[:, 2 * i:2 * i + 3, 2 * j:2 * j + 3, :]
            ref[:, i, j, :] = np.tensordot(patch, k, axes=([1, 2, 3], [0, 1, 2]))
    np.testing.assert_allclose(out, ref, rtol=1e-4, atol=1e-4)
    p = _np(ops.max_pool(x, 2, 2, padding="valid"))
    np.testing.assert_allclose(p, x[:, :6, :6, :].reshape(2, 3, 2, 3, 2, 3).max(axis=(2, 4)))
    ap = _np(ops.average_pool(x, 3, 2, padding="same"))
    assert ap.shape == (2, 4, 4, 3)
    np.testing.assert_allclose(ap[:, 0, 0, :], x[:, :2, :2, :].mean(axis=(1, 2)), rtol=1e-5)


def test_losses_and_norms():
    logits = RNG.normal(size=(6, 10)).astype("float32")
    labels = RNG.integers(0, 10, size=(6,))
    lse = np.log(np.exp(logits).sum(-1))
    ref = lse - logits[np.arange(6), labels]
    np.testing.assert_allclose(_np(ops.sparse_categorical_crossentropy(labels, logits, from_logits=True)), ref, rtol=1e-5)
    x = RNG.normal(size=(4, 16)).astype("float32")
    g, b = RNG.normal(size=(16,)).astype("float32"), RNG.normal(size=(16,)).astype("float32")
    ln = (x - x.mean(-1, keepdims=True)) / np.sqrt(x.var(-1, keepdims=True) + 1e-3) * g + b
    np.testing.assert_allclose(_np(ops.layer_normalization(x, g, b, epsilon=1e-3)), ln, rtol=1e-4, atol=1e-5)
    rms = x / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-6) * g
    np.testing.assert_allclose(_np(ops.rms_normalization(x, g, epsilon=1e-6)), rms, rtol=1e-4, atol=1e-5)
    m, v = ops.moments(x, axes=[0])
    np.testing.assert_allclose(_np(m), x.mean(0), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(_np(v), x.var(0), rtol=1e-4, atol=1e-6)


def test_attention_matches_explicit_softmax():
    q = RNG.normal(size=(2, 5, 4, 8)).astype("float32")
    k = RNG.normal(size=(2, 5, 2, 8)).astype("float32")
    v = RNG.normal(size=(2, 5, 2, 8)).astype("float32")
    out = _np(ops.dot_product_attention(q, k, v, is_causal=True))
    kk, vv = np.repeat(k, 2, axis=2), np.repeat(v, 2, axis=2)
    logits = np.einsum("btnh,bsnh->bnts", q, kk) / np.sqrt(8)
    mask = np.tril(np.ones((5, 5), bool))
    logits = np.where(mask, logits, -1e30)
    p = np.exp(logits - logits.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    ref = np.einsum("bnts,bsnh->btnh", p, vv)
    np.testing.assert_allclose(out, ref, rtol=1e-4, atol=1e-5)


def test_image_and_math_ops():
    img = RNG.uniform(size=(2, 8, 8, 3)).astype("float32")
    assert tuple(ops.image.resize(img, (4, 6)).shape) == (2, 4, 6, 3)
    hsv = ops.image.rgb_to_hsv(img)
    np.testing.assert_allclose(_np(ops.image.hsv_to_rgb(hsv)), img, atol=1e-5)
    ident = np.array([1, 0, 0, 0, 1, 0, 0, 0], "float32")
    np.testing.assert_allclose(_np(ops.image.affine_transform(img, ident)), img, atol=1e-5)
    data = np.arange(10, dtype="float32")
    np.testing.assert_allclose(_np(ops.segment_sum(data, np.array([0, 0, 1, 1, 1, 2, 2, 2, 2, 3]), 4)), [1, 9, 26, 9])
    vals, idx = ops.top_k(np.array([1.0, 5.0, 3.0], "float32"), 2)
    np.testing.assert_allclose(_np(vals), [5, 3])
    re, im = ops.rfft(data)
    np.testing.assert_allclose(_np(re), np.fft.rfft(data).real, rtol=1e-4, atol=1e-4)
