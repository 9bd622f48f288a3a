"""State and arithmetic of a kernel quantised by a calibrated weight-only method (GPTQ or AWQ), shared by ``Dense`` and
``EinsumDense``.

Storage follows the reference's checkpoints (keras/src/layers/core/dense.py:604-800, einsum_dense.py:653-760): the
codes of the kernel transposed, ``[out, in]``, packed along the output axis (two 4-bit or four 2-bit codes per byte,
whole bytes for 3 and 8 bits) as ``quantized_kernel``; ``kernel_scale`` and ``kernel_zero`` (uint8) of shape ``[out,
n_groups]``; ``g_idx`` (float32) mapping each input feature to its group; for AWQ also ``awq_scales [in]``.  Between
``quantize(...)`` and calibration the layer still owns its float kernel and computes with it; calibration
(``keras_b200.quantizers.calibration``) fills the integer state and drops the float kernel.
"""

import math

import torch

from keras_b200 import quantizers
from keras_b200.quantizers import weight_only


def _policy_of(layer):
    from keras_b200.dtype_policies.dtype_policy_map import DTypePolicyMap

    policy = layer.dtype_policy
    if isinstance(policy, DTypePolicyMap):
        policy = policy[layer.path]
    return policy


def weight_bits_for(layer, config, mode):
    """Bit width from the config handed to ``quantize`` or, for a layer rebuilt from a saved model, from its dtype policy."""
    if config is not None and getattr(config, "mode", None) == mode:
        return config.weight_bits
    policy = _policy_of(layer)
    if getattr(policy, "quantization_mode", None) == mode and hasattr(policy, "weight_bits"):
        return policy.weight_bits
    raise ValueError(f"For {mode.upper()} quantization, the weight_bits must be specified either through a `dtype_policy` of that mode or the "
                     "`config` argument.")


def group_size_for(layer, config, mode):
    if config is not None and getattr(config, "mode", None) == mode:
        return config.group_size
    policy = _policy_of(layer)
    if getattr(policy, "quantization_mode", None) == mode and hasattr(policy, "group_size"):
        return policy.group_size
    raise ValueError(f"For {mode.upper()} quantization, the group_size must be specified either through a `dtype_policy` of that mode or the "
                     "`config` argument.")


def _packed_rows(columns, bits):
    return {4: (columns + 1) // 2, 2: (columns + 3) // 4}.get(bits, columns)


class CalibratedKernel:
    """Mixin.  The host layer provides ``add_weight``, ``_kernel`` (the float kernel) and calls ``_calibrated_build`` from its
    ``quantized_build``."""

    is_gptq_calibrated = False
    is_awq_calibrated = False

    SPEC = {"gptq": ["bias", "quantized_kernel", "kernel_scale", "kernel_zero", "g_idx"],
            "awq": ["bias", "quantized_kernel", "kernel_scale", "kernel_zero", "awq_scales", "g_idx"]}

    def _calibrated_build(self, rows, columns, mode, config):
        """Allocate the integer state for a kernel that acts as ``[rows, columns]`` (input features x output features)."""
        bits = weight_bits_for(self, config, mode)
        group = group_size_for(self, config, mode)
        n_groups = 1 if group == -1 else math.ceil(rows / group)
        self._calibrated_shape = (rows, columns)
        self._calibrated_bits = bits
        # a layer rebuilt from a saved model's dtype policy never had a float kernel: its integer state is what it computes with
        integer_only = getattr(self, "_kernel", None) is None
        self.is_gptq_calibrated = integer_only and mode == "gptq"
        self.is_awq_calibrated = integer_only and mode == "awq"
        self.quantized_kernel = self.add_weight(name="kernel", shape=(_packed_rows(columns, bits), rows), initializer="zeros", dtype="uint8",
                                                trainable=False)
        self.kernel_scale = self.add_weight(name="kernel_scale", shape=(columns, n_groups), initializer="ones", trainable=False)
        self.kernel_zero = self.add_weight(name="kernel_zero", shape=(columns, n_groups), initializer="zeros", dtype="uint8", trainable=False)
        if mode == "awq":
            self.awq_scales = self.add_weight(name="awq_scales", shape=(rows,), initializer="ones", trainable=False)
        self.g_idx = self.add_weight(name="g_idx", shape=(rows,), initializer="zeros", dtype="float32", trainable=False)

    @property
    def _calibrated(self):
        return self.is_gptq_calibrated or self.is_awq_calibrated

    def _calibrated_codes(self):
        """Unsigned codes ``[columns, rows]`` (unpacked)."""
        rows, columns = self._calibrated_shape
        packed = self.quantized_kernel.value
        bits = self._calibrated_bits
        if bits == 4:
            return quantizers.unpack_int4(packed, columns, axis=0, dtype="uint8")
        if bits == 2:
            return quantizers.unpack_int2(packed, columns, axis=0, dtype="uint8")
        return packed

    def _calibrated_matrix(self, dtype=None):
        """The kernel as floats, ``[rows, columns]``."""
        scale = self.kernel_scale.value
        matrix = weight_only.dequantize(self._calibrated_codes(), scale, self.kernel_zero.value, self.g_idx.value.to(torch.int64)).T
        if self.is_awq_calibrated:
            matrix = matrix / self.awq_scales.value.to(matrix.dtype).unsqueeze(-1)
        return matrix if dtype is None else matrix.to(dtype)

    def _store_calibrated(self, mode, codes, scale, zero, g_idx, awq_scales=None):
        """Take the solver's result (codes ``[columns, rows]``), pack it, and let go of the float kernel."""
        bits = self._calibrated_bits
        codes = codes.to(torch.uint8)
        if bits == 4:
            codes, _, _ = quantizers.pack_int4(codes, axis=0, dtype="uint8")
        elif bits == 2:
            codes, _, _ = quantizers.pack_int2(codes, axis=0, dtype="uint8")
        self.quantized_kernel.assign(codes)
        self.kernel_scale.assign(scale)
        self.kernel_zero.assign(zero)
        self.g_idx.assign(g_idx.to(torch.float32))
        if mode == "awq":
            self.awq_scales.assign(awq_scales)
        self._drop_float_kernel()
        self.is_gptq_calibrated = mode == "gptq"
        self.is_awq_calibrated = mode == "awq"

    def _drop_float_kernel(self):
        kernel = getattr(self, "_kernel", None)
        if kernel is None:
            return
        self._tracker_unlock()
        try:
            self._untrack_variable(kernel)
            del self._kernel
        finally:
            self._lock_state()

    def _calibrated_names(self, mode):
        if not self._calibrated:
            raise ValueError(f"A layer quantised with mode '{mode}' can only be saved after calibration: call `model.quantize` with a config that "
                             "carries a dataset.")
        return [n for n in self.SPEC[mode] if not (n == "bias" and self.bias is None)]

    def _calibrated_save(self, store, mode):
        for i, name in enumerate(self._calibrated_names(mode)):
            store[str(i)] = getattr(self, name)

    def _calibrated_load(self, store, mode):
        """A saved layer of these modes is always calibrated: it was rebuilt from its dtype policy with integer state only."""
        self.is_gptq_calibrated, self.is_awq_calibrated = mode == "gptq", mode == "awq"
        names = self._calibrated_names(mode)
        if len(store.keys()) != len(names):
            raise ValueError(f"Layer '{self.name}' expected {len(names)} variables, but received {len(store.keys())} variables during loading. "
                             f"Expected: {names}")
        for i, name in enumerate(names):
            value = store[str(i)]
            target = getattr(self, name)
            if name == "quantized_kernel" and tuple(value.shape) != tuple(target.shape) and self._calibrated_bits == 2:
                # older checkpoints stored 2-bit codes one per byte
                value, _, _ = quantizers.pack_int2(torch.as_tensor(value).to(torch.uint8), axis=0, dtype="uint8")
            target.assign(value)
        self._drop_float_kernel()
