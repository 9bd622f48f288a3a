"""Layers against the reference: same constructor arguments, the reference's weights transferred with
``get_weights`` / ``set_weights`` (which also pins the weight order), then forward outputs and the gradient of a
scalar with respect to the input are compared (CPU, float32)."""

import numpy as np
import pytest
import torch

import keras_b200 as keras
from tests import oracle


def _x(shape, seed=0, integer=None):
    rng = np.random.default_rng(seed)
    if integer is not None:
        return rng.integers(0, integer, shape).astype("int32")
    return rng.normal(size=shape).astype("float32")


# (layer class, constructor kwargs, input shapes, call kwargs, integer vocabulary or None)
LAYERS = [
    ("Dense", dict(units=5, activation="gelu"), [(3, 7)], {}, None),
    ("EinsumDense", dict(equation="abc,cde->abde", output_shape=(None, 2, 3), bias_axes="de"), [(2, 4, 6)], {}, None),
    ("TernaryDense", dict(units=5, activation="relu"), [(3, 7)], {}, None),
    ("TernaryDense", dict(units=4, threshold=0.2, use_bias=False), [(3, 7)], {}, None),
    ("Embedding", dict(input_dim=11, output_dim=4, mask_zero=True), [(3, 5)], {}, 11),
    ("Conv1D", dict(filters=4, kernel_size=3, padding="causal", dilation_rate=2), [(2, 9, 3)], {}, None),
    ("Conv2D", dict(filters=4, kernel_size=3, strides=2, padding="same", activation="relu"), [(2, 9, 8, 3)], {}, None),
    ("Conv3D", dict(filters=2, kernel_size=2, padding="valid"), [(1, 4, 5, 4, 3)], {}, None),
    ("Conv2D", dict(filters=6, kernel_size=3, groups=3, padding="same"), [(2, 6, 6, 3)], {}, None),
    ("DepthwiseConv2D", dict(kernel_size=3, depth_multiplier=2, padding="same"), [(2, 6, 7, 3)], {}, None),
    ("SeparableConv2D", dict(filters=5, kernel_size=3, strides=2, padding="same"), [(2, 8, 8, 3)], {}, None),
    ("Conv1DTranspose", dict(filters=3, kernel_size=3, strides=2, padding="same"), [(2, 7, 4)], {}, None),
    ("Conv2DTranspose", dict(filters=3, kernel_size=(3, 2), strides=(2, 3), padding="same"), [(2, 5, 4, 4)], {}, None),
    ("Conv2DTranspose", dict(filters=3, kernel_size=3, strides=2, padding="valid", output_padding=1), [(2, 5, 4, 4)], {}, None),
    ("Conv3DTranspose", dict(filters=2, kernel_size=2, strides=2, padding="same"), [(1, 3, 3, 3, 2)], {}, None),
    ("BatchNormalization", dict(momentum=0.9, epsilon=1e-4), [(4, 5, 5, 3)], dict(training=True), None),
    ("BatchNormalization", dict(axis=1), [(4, 3, 6)], dict(training=False), None),
    ("LayerNormalization", dict(axis=(-2, -1)), [(2, 4, 6)], {}, None),
    ("RMSNormalization", dict(), [(2, 4, 6)], {}, None),
    ("GroupNormalization", dict(groups=2), [(2, 5, 5, 4)], {}, None),
    ("UnitNormalization", dict(axis=-1), [(3, 6)], {}, None),
    ("SpectralNormalization", dict(layer=("Dense", dict(units=5))), [(3, 7)], dict(training=False), None),
    ("MultiHeadAttention", dict(num_heads=2, key_dim=3, value_dim=4, output_shape=5), [(2, 5, 6), (2, 7, 6)], dict(use_causal_mask=False), None),
    ("MultiHeadAttention", dict(num_heads=2, key_dim=3), [(2, 6, 6), (2, 6, 6)], dict(use_causal_mask=True), None),
    ("GroupQueryAttention", dict(head_dim=4, num_query_heads=4, num_key_value_heads=2), [(2, 5, 8), (2, 5, 8)], dict(use_causal_mask=True), None),
    ("Attention", dict(use_scale=True, score_mode="dot"), [(2, 4, 6), (2, 5, 6)], {}, None),
    ("AdditiveAttention", dict(), [(2, 4, 6), (2, 5, 6)], {}, None),
    ("LSTM", dict(units=5, return_sequences=True), [(2, 6, 4)], {}, None),
    ("GRU", dict(units=5, reset_after=False, return_state=True), [(2, 6, 4)], {}, None),
    ("SimpleRNN", dict(units=4, go_backwards=True), [(2, 6, 4)], {}, None),
    ("Bidirectional", dict(layer=("LSTM", dict(units=3, return_sequences=True)), merge_mode="sum"), [(2, 5, 4)], {}, None),
    ("TimeDistributed", dict(layer=("Dense", dict(units=3))), [(2, 5, 4)], {}, None),
    ("ConvLSTM2D", dict(filters=2, kernel_size=3, padding="same"), [(1, 3, 5, 5, 2)], {}, None),
    ("PReLU", dict(shared_axes=[1]), [(2, 4, 5)], {}, None),
    ("ELU", dict(alpha=0.7), [(3, 5)], {}, None),
    ("LeakyReLU", dict(negative_slope=0.2), [(3, 5)], {}, None),
    ("Softmax", dict(axis=(1, 2)), [(2, 3, 4)], {}, None),
    ("ReLU", dict(max_value=1.0, negative_slope=0.1, threshold=0.2), [(3, 5)], {}, None),
    ("MaxPooling2D", dict(pool_size=3, strides=2, padding="same"), [(2, 7, 8, 3)], {}, None),
    ("AveragePooling2D", dict(pool_size=2, strides=1, padding="same"), [(2, 5, 6, 3)], {}, None),
    ("AveragePooling1D", dict(pool_size=3, strides=2, padding="valid"), [(2, 9, 3)], {}, None),
    ("MaxPooling3D", dict(pool_size=2), [(1, 4, 4, 4, 2)], {}, None),
    ("GlobalAveragePooling2D", dict(keepdims=True), [(2, 5, 6, 3)], {}, None),
    ("GlobalMaxPooling1D", dict(), [(2, 5, 3)], {}, None),
    ("AdaptiveAveragePooling2D", dict(output_size=(2, 3)), [(2, 7, 8, 3)], {}, None),
    ("AdaptiveMaxPooling1D", dict(output_size=3), [(2, 8, 3)], {}, None),
    ("UpSampling2D", dict(size=(2, 3), interpolation="bilinear"), [(2, 3, 4, 2)], {}, None),
    ("ZeroPadding2D", dict(padding=((1, 2), (0, 3))), [(2, 3, 4, 2)], {}, None),
    ("Cropping2D", dict(cropping=((1, 0), (1, 1))), [(2, 5, 5, 2)], {}, None),
    ("Permute", dict(dims=(2, 1, 3)), [(2, 3, 4, 5)], {}, None),
    ("RepeatVector", dict(n=3), [(2, 5)], {}, None),
    ("Reshape", dict(target_shape=(-1, 2)), [(3, 4, 5)], {}, None),
    ("Flatten", dict(), [(2, 3, 4)], {}, None),
    ("Add", dict(), [(2, 3), (2, 3)], {}, None),
    ("Concatenate", dict(axis=1), [(2, 3), (2, 4)], {}, None),
    ("Dot", dict(axes=1, normalize=True), [(2, 4), (2, 4)], {}, None),
    ("Maximum", dict(), [(2, 3), (2, 3)], {}, None),
    ("Normalization", dict(mean=[1.0, 2.0, 3.0], variance=[1.0, 4.0, 9.0]), [(4, 3)], {}, None),
    ("Rescaling", dict(scale=1 / 127.5, offset=-1), [(2, 3)], {}, None),
    ("CategoryEncoding", dict(num_tokens=6, output_mode="multi_hot"), [(3, 4)], {}, 6),
    ("Discretization", dict(bin_boundaries=[-0.5, 0.0, 0.5]), [(3, 4)], {}, None),
    ("Resizing", dict(height=5, width=7, interpolation="bilinear"), [(2, 8, 6, 3)], {}, None),
    ("CenterCrop", dict(height=4, width=3), [(2, 8, 6, 3)], {}, None),
    ("Masking", dict(mask_value=0.0), [(2, 4, 3)], {}, None),
    ("ActivityRegularization", dict(l1=0.1), [(2, 4)], {}, None),
    ("MelSpectrogram", dict(fft_length=32, sequence_stride=16, num_mel_bins=8, sampling_rate=800), [(2, 128)], {}, None),
    ("AdaptiveAveragePooling1D", dict(output_size=3), [(2, 10, 4)], {}, None),
    ("AdaptiveAveragePooling3D", dict(output_size=(2, 3, 2)), [(2, 6, 7, 5, 3)], {}, None),
    ("AdaptiveMaxPooling2D", dict(output_size=(3, 2)), [(2, 9, 7, 3)], {}, None),
    ("AdaptiveMaxPooling3D", dict(output_size=2), [(2, 6, 7, 5, 3)], {}, None),
    ("AveragePooling3D", dict(pool_size=2, strides=1, padding="same"), [(2, 5, 6, 4, 3)], {}, None),
    ("MaxPooling1D", dict(pool_size=3, strides=2, padding="same"), [(2, 11, 4)], {}, None),
    ("ConvLSTM1D", dict(filters=4, kernel_size=3, padding="same", return_sequences=True), [(2, 5, 8, 3)], {}, None),
    ("ConvLSTM3D", dict(filters=2, kernel_size=2, padding="same"), [(1, 3, 4, 4, 4, 2)], {}, None),
    ("Cropping1D", dict(cropping=(1, 2)), [(2, 8, 3)], {}, None),
    ("Cropping3D", dict(cropping=((1, 0), (0, 1), (1, 1))), [(2, 5, 5, 5, 2)], {}, None),
    ("DepthwiseConv1D", dict(kernel_size=3, depth_multiplier=2, padding="same", strides=2), [(2, 9, 4)], {}, None),
    ("SeparableConv1D", dict(filters=5, kernel_size=3, padding="same", depth_multiplier=2), [(2, 9, 4)], {}, None),
    ("GlobalAveragePooling1D", dict(), [(2, 7, 4)], {}, None),
    ("GlobalAveragePooling3D", dict(keepdims=True), [(2, 3, 4, 5, 6)], {}, None),
    ("GlobalMaxPooling2D", dict(), [(2, 5, 6, 4)], {}, None),
    ("GlobalMaxPooling3D", dict(), [(2, 3, 4, 5, 6)], {}, None),
    ("Identity", dict(), [(2, 3)], {}, None),
    ("UpSampling1D", dict(size=3), [(2, 4, 3)], {}, None),
    ("UpSampling3D", dict(size=(2, 1, 2)), [(2, 3, 3, 3, 2)], {}, None),
    ("ZeroPadding1D", dict(padding=(1, 2)), [(2, 4, 3)], {}, None),
    ("ZeroPadding3D", dict(padding=((1, 0), (2, 1), (0, 1))), [(2, 3, 3, 3, 2)], {}, None),
    ("STFTSpectrogram", dict(mode="log", frame_length=32, frame_step=8, fft_length=64), [(2, 200, 1)], {}, None),
    ("STFTSpectrogram", dict(mode="stft", frame_length=32, frame_step=16, expand_dims=True, padding="same", window="hamming"), [(2, 200, 1)], {}, None),
    ("ReversibleEmbedding", dict(input_dim=20, output_dim=6), [(2, 5)], {}, 20),
    ("Activation", dict(activation="hard_silu"), [(3, 5)], {}, None),
    ("RandomCrop", dict(height=4, width=5), [(2, 8, 8, 3)], dict(training=False), None),
]


def test_equalization_follows_the_reference_per_channel_over_the_batch():
    rk = oracle.ref()
    images = (np.random.default_rng(4).random((2, 16, 16, 3)) * 255).astype("float32")
    for kwargs in (dict(value_range=(0, 255)), dict(value_range=(0, 255), bins=64)):
        expected = rk.layers.Equalization(**kwargs)(torch.tensor(images))
        oracle.assert_same(keras.layers.Equalization(**kwargs)(torch.tensor(images)), expected, "Equalization", rtol=1e-5, atol=1e-4)
    unit = images / 255.0
    expected = rk.layers.Equalization(value_range=(0, 1))(torch.tensor(unit))
    oracle.assert_same(keras.layers.Equalization(value_range=(0, 1))(torch.tensor(unit)), expected, "Equalization 0..1", rtol=1e-5, atol=1e-5)
    same = keras.layers.Equalization()(torch.tensor(images), training=False)
    np.testing.assert_array_equal(same.numpy(), images)


def _make(k, name, kwargs):
    kwargs = dict(kwargs)
    if "layer" in kwargs and isinstance(kwargs["layer"], tuple):
        inner_name, inner_kwargs = kwargs["layer"]
        kwargs["layer"] = getattr(k.layers, inner_name)(**inner_kwargs)
    return getattr(k.layers, name)(**kwargs)


def _ids():
    seen, out = {}, []
    for name, *_ in LAYERS:
        seen[name] = seen.get(name, 0) + 1
        out.append(f"{name}_{seen[name]}")
    return out


@pytest.mark.parametrize("spec", LAYERS, ids=_ids())
def test_layer_matches_reference(spec):
    rk = oracle.ref()
    name, kwargs, shapes, call_kwargs, vocab = spec
    if not hasattr(rk.layers, name):
        pytest.skip("layer absent from this reference version")
    inputs = [_x(s, seed=i, integer=vocab) for i, s in enumerate(shapes)]
    theirs, ours = _make(rk, name, kwargs), _make(keras, name, kwargs)
    merging = name in ("Add", "Concatenate", "Dot", "Maximum", "Attention", "AdditiveAttention")

    def run(layer, tensors):
        if merging:
            return layer(tensors, **call_kwargs)
        return layer(*tensors, **call_kwargs)

    expected = run(theirs, [torch.tensor(a) for a in inputs])
    run(ours, [torch.tensor(a) for a in inputs])  # builds
    weights = theirs.get_weights()
    assert [tuple(w.shape) for w in ours.get_weights()] == [tuple(w.shape) for w in weights], "weight order or shapes differ"
    ours.set_weights(weights)
    mine = [torch.tensor(a, requires_grad=vocab is None) for a in inputs]
    got = run(ours, mine)
    # Discretization: the reference's integer width depends on which of its backends ends up running the layer
    oracle.assert_same(got, expected, name, rtol=2e-4, atol=2e-5, check_dtype=name != "Discretization")
    if vocab is None and isinstance(got, torch.Tensor) and got.requires_grad:
        ref_in = [torch.tensor(a, requires_grad=True) for a in inputs]
        out_ref = run(theirs, ref_in)
        probe = torch.tensor(np.random.default_rng(9).normal(size=tuple(got.shape)).astype("float32"))
        (got * probe).sum().backward()
        (out_ref * probe).sum().backward()
        for g_ours, g_ref in zip(mine, ref_in):
            if g_ref.grad is not None:
                oracle.assert_same(g_ours.grad, g_ref.grad, name + " input gradient", rtol=5e-4, atol=5e-5)


def test_get_weights_order_of_a_model_with_batchnorm():
    rk = oracle.ref()

    def build(k):
        return k.Sequential([k.Input((6, 6, 3)), k.layers.Conv2D(4, 3), k.layers.BatchNormalization(), k.layers.ReLU(), k.layers.Flatten(), k.layers.Dense(2)])

    theirs, ours = build(rk), build(keras)
    assert [w.name for w in ours.weights] == [w.name for w in theirs.weights]
    ours.set_weights(theirs.get_weights())
    x = _x((3, 6, 6, 3))
    oracle.assert_same(ours.predict(x, verbose=0), theirs.predict(x, verbose=0), "predict", rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("make,shape", [
    (lambda k: k.layers.Dense(24), (5, 7, 16)),
    (lambda k: k.layers.EinsumDense("abc,cde->abde", output_shape=(None, 4, 6), bias_axes="de"), (3, 5, 16)),
    (lambda k: k.layers.EinsumDense("abcd,cde->abe", output_shape=(None, 16), bias_axes="e"), (3, 5, 4, 6)),
    (lambda k: k.layers.EinsumDense("abc,cd->abd", output_shape=(None, 12)), (3, 5, 16)),
    (lambda k: k.layers.EinsumDense("abc,dce->abde", output_shape=(None, 4, 6)), (3, 5, 16)),
    (lambda k: k.layers.EinsumDense("abc,bcd->ad", output_shape=7), (3, 5, 16)),
], ids=["dense", "attention_projection", "attention_output", "rank3", "kernel_axes_reordered", "two_contracted_axes"])
def test_int8_quantized_layers_match_reference(make, shape):
    """quantize("int8"): per-channel int8 kernels and activations quantised per row at call time; codes, scales and the
    de-scaled product are the reference's."""
    rk = oracle.ref()
    x = _x(shape, seed=11)
    theirs, ours = make(rk), make(keras)
    theirs(torch.tensor(x))
    ours(torch.tensor(x))
    ours.set_weights(theirs.get_weights())
    theirs.quantize("int8")
    ours.quantize("int8")
    assert [w.path.split("/")[-1] for w in ours.weights] == [w.path.split("/")[-1] for w in theirs.weights]
    for mine, ref_w in zip(ours.get_weights(), theirs.get_weights()):
        oracle.assert_same(mine, ref_w, "quantised weights", rtol=1e-6, atol=1e-7)
    oracle.assert_same(ours(torch.tensor(x)), theirs(torch.tensor(x)), "int8 forward", rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("shape,grid", [((2, 16, 16, 3), (8, 8)), ((1, 30, 45, 2), (4, 4)), ((1, 64, 64, 1), (8, 8))])
def test_clahe_matches_reference(shape, grid):
    rk = oracle.ref()
    images = (np.random.default_rng(5).random(shape) * 255).astype("float32")
    expected = rk.layers.ContrastLimitedAdaptiveHistogramEqualization(tile_grid_size=grid)(torch.tensor(images))
    got = keras.layers.ContrastLimitedAdaptiveHistogramEqualization(tile_grid_size=grid)(torch.tensor(images))
    oracle.assert_same(got, expected, "CLAHE", rtol=1e-5, atol=1e-3)
    unit = images / 255.0
    expected = rk.layers.ContrastLimitedAdaptiveHistogramEqualization(value_range=(0, 1), clip_limit=2.0, tile_grid_size=grid)(torch.tensor(unit))
    got = keras.layers.ContrastLimitedAdaptiveHistogramEqualization(value_range=(0, 1), clip_limit=2.0, tile_grid_size=grid)(torch.tensor(unit))
    oracle.assert_same(got, expected, "CLAHE 0..1", rtol=1e-5, atol=1e-5)


AUGMENTATIONS = [
    ("RandomFlip", dict(seed=1)), ("RandomFlip", dict(mode="vertical", seed=2)),
    ("RandomRotation", dict(factor=0.2, seed=1)), ("RandomRotation", dict(factor=(-0.1, 0.3), fill_mode="constant", interpolation="nearest", seed=3)),
    ("RandomZoom", dict(height_factor=0.3, seed=1)), ("RandomZoom", dict(height_factor=(-0.2, 0.3), width_factor=0.2, fill_mode="nearest", seed=1)),
    ("RandomTranslation", dict(height_factor=0.2, width_factor=0.3, seed=1)),
    ("RandomBrightness", dict(factor=0.3, seed=1)), ("RandomContrast", dict(factor=0.4, seed=1)), ("RandomCrop", dict(height=6, width=5, seed=1)),
    ("RandomHue", dict(factor=0.5, value_range=(0, 255), seed=1)), ("RandomSaturation", dict(factor=0.5, value_range=(0, 255), seed=1)),
    ("RandomGrayscale", dict(factor=0.7, seed=1)), ("RandomSharpness", dict(factor=0.5, value_range=(0, 255), seed=1)),
    ("RandomShear", dict(x_factor=0.3, y_factor=0.2, seed=1)), ("RandomPosterization", dict(factor=3, value_range=(0, 255), seed=1)),
    ("RandomColorDegeneration", dict(factor=0.6, value_range=(0, 255), seed=1)),
    ("RandomGaussianBlur", dict(factor=1.0, kernel_size=3, sigma=1.0, value_range=(0, 255), seed=1)),
    ("RandomInvert", dict(factor=0.7, value_range=(0, 255), seed=1)),  # RandomElasticTransform: the reference's displacement field ignores the seed
    ("Solarization", dict(addition_factor=0.3, threshold_factor=0.4, value_range=(0, 255), seed=1)), ("AutoContrast", dict(value_range=(0, 255))),
    ("MixUp", dict(alpha=0.3, seed=1)), ("CutMix", dict(factor=0.8, seed=1)),
    ("RandomColorJitter", dict(value_range=(0, 255), brightness_factor=0.2, contrast_factor=0.3, saturation_factor=0.4, hue_factor=0.1, seed=1)), ("GaussianNoise", dict(stddev=0.3, seed=1)), ("GaussianDropout", dict(rate=0.3, seed=1)),
    ("AlphaDropout", dict(rate=0.3, seed=1)), ("SpatialDropout2D", dict(rate=0.4, seed=1)), ("Dropout", dict(rate=0.4, noise_shape=(2, 1, 1, 3), seed=1)),
]


@pytest.mark.parametrize("spec", AUGMENTATIONS, ids=[f"{n}_{i}" for i, (n, _) in enumerate(AUGMENTATIONS)])
def test_seeded_augmentation_in_training_matches_reference(spec):
    """Same seed, same picture: the draws come in the reference's order and mean what they mean there."""
    rk = oracle.ref()
    name, kwargs = spec
    if not hasattr(rk.layers, name):
        pytest.skip("layer absent from this reference version")
    images = (np.random.default_rng(0).random((2, 12, 10, 3)) * 255).astype("float32")
    theirs, ours = getattr(rk.layers, name)(**kwargs), getattr(keras.layers, name)(**kwargs)
    for call in range(2):
        expected = theirs(torch.tensor(images), training=True)
        oracle.assert_same(ours(torch.tensor(images), training=True), expected, f"{name}, call {call}", rtol=1e-3, atol=1e-2)
