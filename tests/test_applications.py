"""Application builders: parameter counts equal the published architectures; small-input forward passes run."""

import numpy as np
import pytest

import keras_b200 as keras

COUNTS = {
    "VGG16": 138357544, "ResNet50": 25636712, "ResNet50V2": 25613800, "MobileNet": 4253864, "MobileNetV2": 3538984, "DenseNet121": 8062504,
    "EfficientNetB0": 5330571, "EfficientNetV2B0": 7200312, "ConvNeXtTiny": 28589128, "NASNetMobile": 5326716, "Xception": 22910480,
    "InceptionV3": 23851784,
}


@pytest.mark.parametrize("name", sorted(COUNTS))
def test_parameter_counts(name):
    model = getattr(keras.applications, name)(weights=None)
    assert model.count_params() == COUNTS[name]


@pytest.mark.parametrize("name,size", [("MobileNetV3Small", 64), ("EfficientNetV2B0", 64), ("DenseNet121", 64), ("ConvNeXtTiny", 64)])
def test_small_forward(name, size):
    model = getattr(keras.applications, name)(weights=None, input_shape=(size, size, 3), classes=7)
    out = model.predict(np.random.rand(2, size, size, 3).astype("float32") * 255, verbose=0)
    assert out.shape == (2, 7) and np.allclose(out.sum(-1), 1.0, atol=1e-4)


def test_namespaces_and_preprocessing():
    assert keras.applications.resnet50.ResNet50 is keras.applications.ResNet50
    assert keras.applications.efficientnet_v2.EfficientNetV2S is keras.applications.EfficientNetV2S
    x = np.full((1, 4, 4, 3), 255.0, "float32")
    np.testing.assert_allclose(keras.applications.mobilenet_v2.preprocess_input(x.copy()), 1.0)
    assert keras.applications.mobilenet_v3.preprocess_input(x) is x
    with pytest.raises(ValueError):
        keras.applications.VGG16(weights="imagenet")


@pytest.mark.parametrize("name,size,kwargs", [("MobileNetV2", 64, dict(alpha=0.35)), ("EfficientNetB0", 64, {}), ("ConvNeXtTiny", 64, {}), ("DenseNet121", 64, {}),
                                              ("Xception", 96, {}), ("NASNetMobile", 64, {})])
def test_application_outputs_match_reference_with_transferred_weights(name, size, kwargs):
    """Same constructor, the reference's (perturbed) weights through get_weights / set_weights, same input: the predictions agree,
    which exercises every layer type of the family in place (depthwise convolutions, squeeze-excite, layer scale, ...)."""
    import torch

    from tests import oracle

    rk = oracle.ref()
    rng = np.random.default_rng(0)
    theirs = getattr(rk.applications, name)(weights=None, input_shape=(size, size, 3), classes=10, **kwargs)
    ours = getattr(keras.applications, name)(weights=None, input_shape=(size, size, 3), classes=10, **kwargs)
    weights = [w + rng.normal(size=w.shape).astype(w.dtype) * 0.02 if w.dtype.kind == "f" else w for w in theirs.get_weights()]
    weights = [np.abs(w) + 0.5 if "variance" in v.path else w for w, v in zip(weights, theirs.weights)]
    theirs.set_weights(weights)
    ours.set_weights(weights)
    x = torch.tensor(rng.random((2, size, size, 3)).astype("float32") * 255)
    expected = theirs(x, training=False).detach().numpy()
    got = ours(x, training=False).detach().numpy()
    np.testing.assert_allclose(got, expected, rtol=1e-4, atol=2e-6)
