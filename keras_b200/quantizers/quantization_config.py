"""Quantization configs (keras/src/quantizers/quantization_config.py)."""

from keras_b200.core.export_registry import keras_export

_MODES = ("int8", "float8", "int4", "gptq", "awq", "ternary")


@keras_export("keras.quantizers.QuantizationConfig")
class QuantizationConfig:
    def __init__(self, weight_quantizer=None, activation_quantizer=None):
        self.weight_quantizer = weight_quantizer
        self.activation_quantizer = activation_quantizer

    @property
    def mode(self):
        raise NotImplementedError("Subclasses must implement this property. Do not instantiate QuantizationConfig directly.")

    def get_config(self):
        from keras_b200.saving import serialization_lib

        return {
            "weight_quantizer": serialization_lib.serialize_keras_object(self.weight_quantizer),
            "activation_quantizer": serialization_lib.serialize_keras_object(self.activation_quantizer),
        }

    @classmethod
    def from_config(cls, config):
        from keras_b200.saving import serialization_lib

        return cls(
            weight_quantizer=serialization_lib.deserialize_keras_object(config.get("weight_quantizer")),
            activation_quantizer=serialization_lib.deserialize_keras_object(config.get("activation_quantizer")),
        )

    @staticmethod
    def weight_quantizer_or_default(config, default):
        if config is not None and config.weight_quantizer is not None:
            return config.weight_quantizer
        return default

    @staticmethod
    def activation_quantizer_or_default(config, default):
        if config is not None:
            return config.activation_quantizer
        return default


def _simple(name, mode_name, export):
    def mode(self):
        return mode_name

    cls = type(name, (QuantizationConfig,), {"mode": property(mode)})
    cls.__module__ = __name__
    return keras_export(export)(cls)


@keras_export("keras.quantizers.Int8QuantizationConfig")
class Int8QuantizationConfig(QuantizationConfig):
    def __init__(self, weight_quantizer=None, activation_quantizer="default"):
        from keras_b200 import quantizers

        if activation_quantizer == "default":
            activation_quantizer = quantizers.AbsMaxQuantizer(axis=-1)
        super().__init__(weight_quantizer, activation_quantizer)

    mode = property(lambda self: "int8")


@keras_export("keras.quantizers.Int4QuantizationConfig")
class Int4QuantizationConfig(QuantizationConfig):
    def __init__(self, weight_quantizer=None, activation_quantizer="default", block_size=128):
        from keras_b200 import quantizers

        if activation_quantizer == "default":
            activation_quantizer = quantizers.AbsMaxQuantizer(axis=-1)
        super().__init__(weight_quantizer, activation_quantizer)
        self.block_size = block_size

    mode = property(lambda self: "int4")

    def get_config(self):
        return {**super().get_config(), "block_size": self.block_size}


@keras_export("keras.quantizers.Float8QuantizationConfig")
class Float8QuantizationConfig(QuantizationConfig):
    def __init__(self):
        super().__init__(None, None)

    mode = property(lambda self: "float8")

    def get_config(self):
        return {}

    @classmethod
    def from_config(cls, config):
        return cls()


@keras_export("keras.quantizers.TernaryQuantizationConfig")
class TernaryQuantizationConfig(QuantizationConfig):
    def __init__(self):
        super().__init__(None, None)

    mode = property(lambda self: "ternary")

    def get_config(self):
        return {}

    @classmethod
    def from_config(cls, config):
        return cls()


@keras_export("keras.quantizers.GPTQConfig")
class GPTQConfig(QuantizationConfig):
    def __init__(self, dataset=None, tokenizer=None, *, weight_bits=4, num_samples=128, calibration_batch_size=8, per_channel=True,
                 sequence_length=512, hessian_damping=0.01, group_size=128, symmetric=False, activation_order=False,
                 quantization_layer_structure=None):
        super().__init__()
        if weight_bits not in (2, 3, 4, 8):
            raise ValueError(f"Unsupported weight_bits {weight_bits}. Supported values are 2, 3, 4, and 8.")
        if num_samples <= 0:
            raise ValueError("num_samples must be a positive integer.")
        if calibration_batch_size <= 0:
            raise ValueError("calibration_batch_size must be a positive integer.")
        self.calibration_batch_size = calibration_batch_size
        if sequence_length <= 0:
            raise ValueError("sequence_length must be a positive integer.")
        if hessian_damping < 0 or hessian_damping > 1:
            raise ValueError("hessian_damping must be between 0 and 1.")
        if group_size < -1 or group_size == 0:
            raise ValueError("Invalid group_size. Supported values are -1 (whole-tensor) or a positive integer, " f"but got {group_size}.")
        self.dataset, self.tokenizer = dataset, tokenizer
        self.weight_bits, self.num_samples, self.per_channel = weight_bits, num_samples, per_channel
        self.sequence_length, self.hessian_damping, self.group_size = sequence_length, hessian_damping, group_size
        self.symmetric, self.activation_order = symmetric, activation_order
        self.quantization_layer_structure = quantization_layer_structure

    mode = property(lambda self: "gptq")

    def dtype_policy_string(self):
        return f"gptq/{self.weight_bits}/{self.group_size}"

    def get_config(self):
        return {"dataset": None, "tokenizer": None, "weight_bits": self.weight_bits, "num_samples": self.num_samples,
                "calibration_batch_size": self.calibration_batch_size, "per_channel": self.per_channel, "sequence_length": self.sequence_length, "hessian_damping": self.hessian_damping,
                "group_size": self.group_size, "symmetric": self.symmetric, "activation_order": self.activation_order,
                "quantization_layer_structure": None}  # live layer objects: calibration-time only, never saved

    @classmethod
    def from_config(cls, config):
        return cls(**config)


@keras_export("keras.quantizers.AWQConfig")
class AWQConfig(QuantizationConfig):
    def __init__(self, dataset=None, tokenizer=None, *, weight_bits=4, num_samples=128, sequence_length=512, group_size=128,
                 num_grid_points=20, apply_clip=True, quantization_layer_structure=None):
        super().__init__()
        if weight_bits != 4:
            raise ValueError(f"AWQ only supports 4-bit quantization. Received weight_bits={weight_bits}.")
        if num_samples <= 0:
            raise ValueError("num_samples must be a positive integer.")
        if sequence_length <= 0:
            raise ValueError("sequence_length must be a positive integer.")
        self.apply_clip = bool(apply_clip)
        if group_size < -1 or group_size == 0:
            raise ValueError(f"Invalid group_size. Supported values are -1 (per-channel) or a positive integer, but got {group_size}.")
        if num_grid_points <= 0:
            raise ValueError("num_grid_points must be a positive integer.")
        self.dataset, self.tokenizer = dataset, tokenizer
        self.weight_bits, self.num_samples, self.sequence_length = weight_bits, num_samples, sequence_length
        self.group_size, self.num_grid_points = group_size, num_grid_points
        self.quantization_layer_structure = quantization_layer_structure

    mode = property(lambda self: "awq")

    def dtype_policy_string(self):
        return f"awq/{self.weight_bits}/{self.group_size}"

    def get_config(self):
        return {"dataset": None, "tokenizer": None, "weight_bits": self.weight_bits, "num_samples": self.num_samples,
                "sequence_length": self.sequence_length, "group_size": self.group_size, "num_grid_points": self.num_grid_points,
                "apply_clip": self.apply_clip, "quantization_layer_structure": None}  # live layer objects: calibration-time only, never saved

    @classmethod
    def from_config(cls, config):
        return cls(**config)


def validate_and_resolve_config(mode, config):
    """Return a config object for ``mode`` (``mode`` may be None when ``config`` carries it)."""
    if config is not None:
        if not isinstance(config, QuantizationConfig):
            raise ValueError(f"Argument `config` must be an instance of `QuantizationConfig`. Received: config={config} (of type {type(config)})")
        if mode is not None and mode != config.mode:
            raise ValueError(f"Contradictory arguments: mode='{mode}' incompatible with config.mode='{config.mode}'")
        return config
    if mode is None:
        raise ValueError("You must provide either `mode` or `config` to `quantize`.")
    if mode not in _MODES:
        raise ValueError(f"Invalid quantization mode. Expected one of {_MODES}. Received: mode={mode}")
    if mode == "int8":
        return Int8QuantizationConfig()
    if mode == "int4":
        return Int4QuantizationConfig()
    if mode == "float8":
        return Float8QuantizationConfig()
    if mode == "ternary":
        return TernaryQuantizationConfig()
    if mode == "gptq":
        raise ValueError("For GPTQ, you must pass a `GPTQConfig` object in the `config` argument.")
    if mode == "awq":
        raise ValueError("For AWQ, you must pass an `AWQConfig` object in the `config` argument.")
