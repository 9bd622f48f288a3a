"""``Sequential``: a linear stack of layers (keras/src/models/sequential.py:20-396).

The stack is compiled lazily into an inner ``Functional`` once the input shape is known; models
whose layers cannot be traced symbolically fall back to a plain loop.
"""

import copy
import inspect

from keras_b200 import tree
from keras_b200.core.dtypes import standardize_dtype
from keras_b200.core.export_registry import keras_export
from keras_b200.core.keras_tensor import KerasTensor
from keras_b200.layers.core.input_layer import InputLayer
from keras_b200.layers.layer import Layer
from keras_b200.models.functional import Functional
from keras_b200.models.model import Model


@keras_export(["keras.Sequential", "keras.models.Sequential"])
class Sequential(Model):
    def __init__(self, layers=None, trainable=True, name=None):
        super().__init__(trainable=trainable, name=name)
        self._functional = None
        self._stack = []
        if layers:
            for layer in layers:
                self.add(layer, rebuild=False)
            self._maybe_rebuild()

    def add(self, layer, rebuild=True):
        if not self._stack:
            if getattr(layer, "_input_shape_arg", None) is not None:
                self.add(InputLayer(shape=layer._input_shape_arg))
        if hasattr(layer, "_keras_history"):
            origin = layer._keras_history[0]
            if isinstance(origin, InputLayer):
                layer = origin
        if not isinstance(layer, Layer):
            raise ValueError(f"Only instances of `keras.Layer` can be added to a Sequential model. Received: {layer} (of type {type(layer)})")
        if not self._is_layer_name_unique(layer):
            raise ValueError(f"All layers added to a Sequential model should have unique names. Name '{layer.name}' is already the name of a layer in this model. Update the `name` argument to pass a unique name.")
        if isinstance(layer, InputLayer) and self._stack and isinstance(self._stack[0], InputLayer):
            raise ValueError(f"Sequential model '{self.name}' has already been configured to use input shape {self._stack[0].batch_shape}. You cannot add a different Input layer to it.")
        self._stack.append(layer)
        if rebuild:
            self._maybe_rebuild()
        else:
            self.built = False
            self._functional = None

    def pop(self, rebuild=True):
        layer = self._stack.pop()
        self.built = False
        self._functional = None
        self._layers[:] = [l for l in self._layers if l is not layer]
        if rebuild:
            self._maybe_rebuild()
        return layer

    def _maybe_rebuild(self):
        self.built = False
        self._functional = None
        if self._stack and isinstance(self._stack[0], InputLayer) and len(self._stack) > 1:
            self.build(self._stack[0].batch_shape)
        elif hasattr(self, "_manual_input_shape"):
            pass

    def _lock_state(self):
        pass

    def _obj_type(self):
        return "Sequential"

    def build(self, input_shape=None):
        try:
            input_shape = tuple(None if d is None else int(d) for d in input_shape)
        except Exception:
            return
        if not self._stack:
            raise ValueError(f"Sequential model {self.name} cannot be built because it has no layers. Call `model.add(layer)`.")
        if isinstance(self._stack[0], InputLayer):
            if tuple(self._stack[0].batch_shape) != tuple(input_shape):
                raise ValueError(f"Sequential model '{self.name}' has already been configured to use input shape {self._stack[0].batch_shape}. You cannot build it with input_shape {input_shape}")
        else:
            dtype = self._stack[0].compute_dtype
            self._stack = [InputLayer(batch_shape=input_shape, dtype=dtype)] + self._stack
        inputs = self._stack[0].output
        x = inputs
        for layer in self._stack[1:]:
            try:
                x = layer(x)
            except NotImplementedError:
                # layer cannot be called symbolically: use the eager loop fallback
                return
            except TypeError as e:
                sig = inspect.signature(layer.call)
                positional = [p for p in sig.parameters.values() if p.default == inspect.Parameter.empty and p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
                if len(positional) != 1:
                    raise ValueError(
                        "Layers added to a Sequential model can only have a single positional argument, the input tensor. "
                        f"Layer {layer.__class__.__name__} has multiple positional arguments: {positional}"
                    )
                raise e
        outputs = x
        self._functional = Functional(inputs=inputs, outputs=outputs)

    def call(self, inputs, training=None, mask=None, **kwargs):
        if self._functional is not None:
            return self._functional.call(inputs, training=training, mask=mask, **kwargs)
        for layer in self.layers:
            kw = {}
            if layer._plan.has_mask:
                kw["mask"] = mask
            if layer._plan.has_training and training is not None:
                kw["training"] = training
            outputs = layer(inputs, **kw)
            inputs = outputs
            mask = tree.map_structure(lambda x: getattr(x, "_keras_mask", None), outputs)
        return outputs

    def __call__(self, inputs, training=None, mask=None, **kwargs):
        if not self.built and self._functional is None and not isinstance(inputs, dict):
            shape = getattr(inputs, "shape", None)
            if shape is not None and not (self._stack and isinstance(self._stack[0], InputLayer)):
                self.build((None,) + tuple(shape[1:]) if not isinstance(inputs, KerasTensor) else tuple(shape))
        return super().__call__(inputs, training=training, mask=mask, **kwargs)

    @property
    def layers(self):
        layers = self._stack
        if layers and isinstance(layers[0], InputLayer):
            return layers[1:]
        return layers[:]

    @layers.setter
    def layers(self, _):
        raise AttributeError("`Sequential.layers` attribute is reserved and should not be used. Use `add()` and `pop()` to change the layers in this model.")

    def _flatten_layers(self, include_self=True, recursive=True):
        # sub-layers are the stack (the inner Functional shares them)
        out = [self] if include_self else []
        seen = {id(self)}
        for layer in self._stack:
            for l in (layer._flatten_layers(include_self=True, recursive=True) if recursive else [layer]):
                if id(l) not in seen:
                    seen.add(id(l))
                    out.append(l)
        return out

    def compute_output_spec(self, inputs, training=None, mask=None, **kwargs):
        if self._functional is not None:
            return self._functional.compute_output_spec(inputs, training=training, mask=mask)
        for layer in self.layers:
            outputs = layer.compute_output_spec(inputs, **({"training": training} if layer._plan.has_training else {}))
            inputs = outputs
        return outputs

    def compute_output_shape(self, input_shape):
        if self._functional is not None:
            return self._functional.compute_output_shape(input_shape)
        for layer in self.layers:
            output_shape = layer.compute_output_shape(input_shape)
            input_shape = output_shape
        return output_shape

    @property
    def input_shape(self):
        if self._functional is not None:
            return self._functional.input_shape
        raise AttributeError(f"Sequential model '{self.name}' has no defined input shape yet.")

    @property
    def output_shape(self):
        if self._functional is not None:
            return self._functional.output_shape
        raise AttributeError(f"Sequential model '{self.name}' has no defined output shape yet.")

    @property
    def inputs(self):
        if self._functional is not None:
            return self._functional.inputs
        raise AttributeError(f"Sequential model '{self.name}' has no defined inputs yet.")

    @property
    def outputs(self):
        if self._functional is not None:
            return self._functional.outputs
        raise AttributeError(f"Sequential model '{self.name}' has no defined outputs yet.")

    @property
    def input_dtype(self):
        layers = self._stack
        if layers and isinstance(layers[0], InputLayer):
            return layers[0].dtype
        return super().input_dtype

    def _is_layer_name_unique(self, layer):
        for ref in self._stack:
            if layer.name == ref.name and ref is not layer:
                return False
        return True

    def get_config(self):
        from keras_b200.saving import serialization_lib

        layer_configs = [serialization_lib.serialize_keras_object(layer) for layer in self._stack]
        config = Model.get_config(self)
        config["name"] = self.name
        config["layers"] = copy.deepcopy(layer_configs)
        if self._functional is not None or (self._stack and isinstance(self._stack[0], InputLayer)):
            config["build_input_shape"] = self._stack[0].batch_shape
        return config

    @classmethod
    def from_config(cls, config, custom_objects=None):
        from keras_b200.saving import serialization_lib

        if "name" in config:
            name = config["name"]
            build_input_shape = config.get("build_input_shape")
            layer_configs = config["layers"]
        else:
            name = None
            build_input_shape = None
            layer_configs = config
        model = cls(name=name)
        for layer_config in layer_configs:
            if "module" not in layer_config:
                from keras_b200.legacy.saving import legacy_serialization

                layer = legacy_serialization.deserialize_layer(layer_config, custom_objects=custom_objects)
            else:
                layer = serialization_lib.deserialize_keras_object(layer_config, custom_objects=custom_objects)
            model.add(layer)
        if not model._functional and build_input_shape and isinstance(build_input_shape, (tuple, list)):
            model.build(build_input_shape)
        return model
