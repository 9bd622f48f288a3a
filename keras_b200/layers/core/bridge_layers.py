"""Layers that wrap other frameworks' callables: ``JaxLayer``, ``FlaxLayer`` (keras/src/utils/jax_layer.py) and
``TFSMLayer`` (keras/src/export/tfsm_layer.py).  They need JAX / Flax / TensorFlow runtimes, which this framework does not
bundle; constructing one raises an ``ImportError`` that names the missing runtime (the torch equivalent is
``TorchModuleWrapper``)."""

from keras_b200.core.export_registry import keras_export
from keras_b200.layers.layer import Layer


def _bridge(name, runtime, hint):
    def __init__(self, *args, **kwargs):
        raise ImportError(f"`{name}` wraps a {runtime} callable and needs the {runtime} runtime, which is not available in this framework. {hint}")

    cls = type(name, (Layer,), {"__init__": __init__, "__doc__": f"Bridge to {runtime}; unavailable without that runtime."})
    cls.__module__ = __name__
    return keras_export(f"keras.layers.{name}")(cls)


JaxLayer = _bridge("JaxLayer", "JAX", "Wrap torch modules with `keras.layers.TorchModuleWrapper` instead.")
FlaxLayer = _bridge("FlaxLayer", "Flax/JAX", "Wrap torch modules with `keras.layers.TorchModuleWrapper` instead.")
TFSMLayer = _bridge("TFSMLayer", "TensorFlow SavedModel", "Reload artefacts written with `format='torch_export'` through `keras.export.load_exported`.")
