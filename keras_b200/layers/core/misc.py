"""Small core layers: ``Identity``, ``Lambda``, ``Masking`` (keras/src/layers/core/*.py)."""

import inspect
import types

import torch

from keras_b200 import ops, tree
from keras_b200.core.export_registry import keras_export
from keras_b200.core.keras_tensor import KerasTensor
from keras_b200.layers.layer import Layer


@keras_export("keras.layers.Identity")
class Identity(Layer):
    def __init__(self, **kwargs):
        super().__init__(**kwargs)
        self.supports_masking = True
        self.built = True

    def call(self, inputs):
        return inputs

    def compute_output_shape(self, input_shape):
        return input_shape

    def compute_output_spec(self, inputs):
        return tree.map_structure(lambda x: KerasTensor(x.shape, dtype=x.dtype, sparse=x.sparse), inputs)


@keras_export("keras.layers.Masking")
class Masking(Layer):
    def __init__(self, mask_value=0.0, **kwargs):
        super().__init__(**kwargs)
        if isinstance(mask_value, dict) and mask_value.get("config", None):
            from keras_b200.saving import serialization_lib

            mask_value = serialization_lib.deserialize_keras_object(mask_value)
        self.mask_value = mask_value
        self.supports_masking = True
        self.built = True

    def compute_mask(self, inputs, mask=None):
        return ops.any(ops.not_equal(inputs, self.mask_value), axis=-1)

    def call(self, inputs):
        boolean_mask = ops.any(ops.not_equal(inputs, self.mask_value), axis=-1, keepdims=True)
        outputs = inputs * ops.cast(boolean_mask, inputs.dtype)
        try:
            outputs._keras_mask = ops.squeeze(boolean_mask, axis=-1)
        except AttributeError:
            pass
        return outputs

    def compute_output_shape(self, input_shape):
        return input_shape

    def get_config(self):
        from keras_b200.saving import serialization_lib

        return {**super().get_config(), "mask_value": serialization_lib.serialize_keras_object(self.mask_value) if isinstance(self.mask_value, torch.Tensor) else self.mask_value}


@keras_export("keras.layers.Lambda")
class Lambda(Layer):
    def __init__(self, function, output_shape=None, mask=None, arguments=None, **kwargs):
        super().__init__(**kwargs)
        self.arguments = arguments or {}
        self.function = function
        if mask is not None:
            self.supports_masking = True
        self.mask = mask
        self._output_shape = output_shape
        self._already_warned = False
        fn_args = inspect.getfullargspec(function).args if not isinstance(function, type) else []
        self._fn_expects_training_arg = "training" in fn_args
        self._fn_expects_mask_arg = "mask" in fn_args
        self.built = True

    def compute_output_shape(self, input_shape):
        if self._output_shape is None:
            try:
                from keras_b200.core.tensor import compute_output_spec

                spec = compute_output_spec(self.call, tree.map_shape_structure(lambda s: KerasTensor(s, dtype=self.compute_dtype), input_shape))
                return tree.map_structure(lambda x: x.shape, spec)
            except Exception:
                raise NotImplementedError(
                    "We could not automatically infer the shape of the Lambda's output. Please specify the `output_shape` argument for this Lambda layer."
                )
        if callable(self._output_shape):
            return self._output_shape(input_shape)
        batch = tree.flatten(input_shape)[0] if False else (input_shape[0] if not isinstance(input_shape[0], (tuple, list)) else input_shape[0][0])

        def add_batch(s):
            return (batch,) + tuple(s)

        return tree.map_shape_structure(add_batch, self._output_shape) if not isinstance(self._output_shape, (list, tuple)) or isinstance(self._output_shape[0], (list, tuple)) else add_batch(self._output_shape)

    def compute_output_spec(self, inputs, mask=None, training=None):
        if self._output_shape is None:
            from keras_b200.core.tensor import compute_output_spec

            kw = {}
            return compute_output_spec(lambda x: self.call(x, mask=mask, training=training), inputs)
        shapes = self.compute_output_shape(tree.map_structure(lambda x: x.shape, inputs))
        return tree.map_shape_structure(lambda s: KerasTensor(s, dtype=self.compute_dtype), shapes)

    def call(self, inputs, mask=None, training=None):
        kwargs = dict(self.arguments)
        if self._fn_expects_mask_arg:
            kwargs["mask"] = mask
        if self._fn_expects_training_arg:
            kwargs["training"] = training
        return self.function(inputs, **kwargs)

    def compute_mask(self, inputs, mask=None):
        if callable(self.mask):
            return self.mask(inputs, mask)
        return self.mask

    def get_config(self):
        from keras_b200.saving import serialization_lib

        cfg = {"function": self._serialize_function_to_config(self.function)}
        if self._output_shape is not None:
            if callable(self._output_shape):
                cfg["output_shape"] = self._serialize_function_to_config(self._output_shape)
            else:
                cfg["output_shape"] = self._output_shape
        if self.mask is not None:
            if callable(self.mask):
                cfg["mask"] = self._serialize_function_to_config(self.mask)
            else:
                cfg["mask"] = serialization_lib.serialize_keras_object(self.mask)
        cfg["arguments"] = serialization_lib.serialize_keras_object(self.arguments)
        return {**super().get_config(), **cfg}

    def _serialize_function_to_config(self, fn):
        from keras_b200.saving import serialization_lib

        if isinstance(fn, types.LambdaType) and fn.__name__ == "<lambda>":
            code, defaults, closure = serialization_lib.func_dump(fn)
            return {"class_name": "__lambda__", "config": {"code": code, "defaults": defaults, "closure": closure}}
        if callable(fn):
            return serialization_lib.serialize_keras_object(fn)
        raise ValueError(f"Invalid input type for serialization. Received: {fn} of type {type(fn)}.")

    @staticmethod
    def _raise_for_lambda_deserialization(safe_mode):
        if safe_mode:
            raise ValueError(
                "Requested the deserialization of a `Lambda` layer whose `function` is a Python lambda. This carries a "
                "potential risk of arbitrary code execution and thus it is disallowed by default. If you trust the "
                "source of the artifact, you can override this error by passing `safe_mode=False` to the loading "
                "function, or calling `keras.config.enable_unsafe_deserialization()."
            )

    @classmethod
    def from_config(cls, config, custom_objects=None, safe_mode=None):
        from keras_b200.saving import serialization_lib

        safe_mode = safe_mode if safe_mode is not None else serialization_lib.in_safe_mode()
        if safe_mode is None:
            safe_mode = True
        config = dict(config)
        for key in ("function", "output_shape", "mask"):
            v = config.get(key)
            if isinstance(v, dict) and v.get("class_name") == "__lambda__":
                cls._raise_for_lambda_deserialization(safe_mode)
                inner = v["config"]
                config[key] = serialization_lib.func_load(inner["code"], defaults=inner["defaults"], closure=inner["closure"])
            elif isinstance(v, dict):
                config[key] = serialization_lib.deserialize_keras_object(v, custom_objects=custom_objects)
            elif key == "output_shape" and isinstance(v, list):
                config[key] = tuple(v)
        if "arguments" in config:
            config["arguments"] = serialization_lib.deserialize_keras_object(config["arguments"], custom_objects=custom_objects)
        return cls(**config)
