"""``Wrapper``: base class for layers that wrap one inner layer (keras/src/layers/core/wrapper.py)."""

from keras_b200.core.export_registry import keras_export
from keras_b200.layers.layer import Layer


@keras_export("keras.layers.Wrapper")
class Wrapper(Layer):
    def __init__(self, layer, **kwargs):
        try:
            assert isinstance(layer, Layer)
        except Exception:
            raise ValueError(f"Layer {layer} supplied to Wrapper isn't a supported layer type. Please ensure wrapped layer is a valid Keras layer.")
        super().__init__(**kwargs)
        self.layer = layer

    def build(self, input_shape=None):
        if not self.layer.built:
            self.layer.build(input_shape)
            self.layer.built = True
        self.built = True

    def get_config(self):
        from keras_b200.saving import serialization_lib

        return {**super().get_config(), "layer": serialization_lib.serialize_keras_object(self.layer)}

    @classmethod
    def from_config(cls, config, custom_objects=None):
        from keras_b200.saving import serialization_lib

        config = dict(config)
        config["layer"] = serialization_lib.deserialize_keras_object(config.pop("layer"), custom_objects=custom_objects)
        return cls(**config)
