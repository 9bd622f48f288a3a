"""``Embedding`` and ``ReversibleEmbedding``.

Behaviour of keras/src/layers/core/embedding.py:193-197 (``take`` + cast to compute dtype),
``mask_zero``, LoRA, int8; ``ReversibleEmbedding`` adds a tied/untied ``reverse=True`` logits
projection (keras/src/layers/core/reversible_embedding.py).
"""

import torch

from keras_b200 import constraints, initializers, ops, quantizers, regularizers
from keras_b200.core.export_registry import keras_export
from keras_b200.core.keras_tensor import KerasTensor
from keras_b200.layers.layer import Layer


@keras_export("keras.layers.Embedding")
class Embedding(Layer):
    def __init__(self, input_dim, output_dim, embeddings_initializer="uniform", embeddings_regularizer=None, embeddings_constraint=None,
                 mask_zero=False, weights=None, lora_rank=None, lora_alpha=None, quantization_config=None, **kwargs):
        input_length = kwargs.pop("input_length", None)
        super().__init__(**kwargs)
        self.input_dim, self.output_dim = input_dim, output_dim
        self.embeddings_initializer = initializers.get(embeddings_initializer)
        self.embeddings_regularizer = regularizers.get(embeddings_regularizer)
        self.embeddings_constraint = constraints.get(embeddings_constraint)
        self.mask_zero = mask_zero
        self.supports_masking = mask_zero
        self.autocast = False
        self.lora_rank = lora_rank
        self.lora_alpha = lora_alpha if lora_alpha is not None else lora_rank
        self.lora_enabled = False
        self.quantization_config = quantization_config
        self._is_quantized = False
        if weights is not None:
            self.build()
            if not (isinstance(weights, list) and len(weights) == 1):
                weights = [weights]
            self.set_weights(weights)

    def build(self, input_shape=None):
        if self.built:
            return
        shape = (self.input_dim, self.output_dim)
        if self.quantization_mode:
            self.quantized_build(shape, mode=self.quantization_mode)
        if self.quantization_mode != "int8":
            self._embeddings = self.add_weight(shape=shape, initializer=self.embeddings_initializer, name="embeddings",
                                               regularizer=self.embeddings_regularizer, constraint=self.embeddings_constraint, trainable=True)
        self.built = True
        if self.lora_rank:
            self.enable_lora(self.lora_rank, lora_alpha=self.lora_alpha)

    @property
    def embeddings(self):
        if not self.built:
            raise AttributeError("You must build the layer before accessing `embeddings`.")
        if self.lora_enabled:
            return ops.add(self._embeddings.value, (self.lora_alpha / self.lora_rank) * ops.matmul(self.lora_embeddings_a.value, self.lora_embeddings_b.value))
        return self._embeddings

    def call(self, inputs):
        if not isinstance(inputs, KerasTensor) and inputs.dtype not in (torch.int32, torch.int64):
            inputs = inputs.to(torch.int32)
        fused = self._gather_on_device(inputs)
        if fused is not None:
            return fused
        out = ops.take(self.embeddings, inputs, axis=0)
        return ops.cast(out, self.compute_dtype)

    def _gather_on_device(self, inputs):
        """Gather and cast in one kernel; the gradient is scattered straight into the table's fp32 gradient storage."""
        if not isinstance(inputs, torch.Tensor) or not inputs.is_cuda or self.lora_enabled:
            return None
        from keras_b200.core import dtypes
        from keras_b200.kernels import dispatch

        table = self._embeddings.value
        if not isinstance(table, torch.Tensor):
            return None
        ids = torch.where(inputs < 0, inputs + table.shape[0], inputs)
        return dispatch.embedding(self._embeddings, table, ids, dtypes.to_torch_dtype(self.compute_dtype))

    def compute_mask(self, inputs, mask=None):
        if not self.mask_zero:
            return None
        return ops.not_equal(inputs, 0)

    def compute_output_shape(self, input_shape):
        return (*input_shape, self.output_dim)

    def compute_output_spec(self, inputs):
        return KerasTensor(self.compute_output_shape(inputs.shape), dtype=self.compute_dtype)

    def enable_lora(self, rank, lora_alpha=None, a_initializer="he_uniform", b_initializer="zeros"):
        if self.embeddings_constraint:
            raise ValueError("Lora is incompatible with embedding constraints. In order to enable lora on this layer, remove the `embeddings_constraint` argument.")
        if not self.built:
            raise ValueError("Cannot enable lora on a layer that isn't yet built.")
        if self.lora_enabled:
            raise ValueError("lora is already enabled. This can only be done once per layer.")
        self._tracker_unlock()
        self.lora_embeddings_a = self.add_weight(name="lora_embeddings_a", shape=(self.input_dim, rank), initializer=initializers.get(a_initializer), regularizer=self.embeddings_regularizer)
        self.lora_embeddings_b = self.add_weight(name="lora_embeddings_b", shape=(rank, self.output_dim), initializer=initializers.get(b_initializer), regularizer=self.embeddings_regularizer)
        self._embeddings.trainable = False
        self._lock_state()
        self._invalidate()
        self.lora_enabled = True
        self.lora_rank = rank
        self.lora_alpha = lora_alpha if lora_alpha is not None else rank

    def _saved(self):
        out = [("embeddings", self._embeddings)]
        if self._is_quantized and self.quantization_mode == "int8":
            out.append(("embeddings_scale", self.embeddings_scale))
        return out

    def save_own_variables(self, store):
        if not self.built:
            return
        emb, scale = self._embeddings, getattr(self, "embeddings_scale", None)
        if self.lora_enabled:
            delta = (self.lora_alpha / self.lora_rank) * torch.matmul(self.lora_embeddings_a._value, self.lora_embeddings_b._value)
            if self._is_quantized and self.quantization_mode == "int8":
                full = self._embeddings._value.to(torch.float32) / self.embeddings_scale._value[:, None] + delta
                emb, scale = quantizers.abs_max_quantize(full, axis=-1, to_numpy=False)
                scale = scale.squeeze(-1)
            else:
                emb = self._embeddings._value + delta.to(self._embeddings._value.dtype)
        store["0"] = emb
        if self._is_quantized and self.quantization_mode == "int8":
            store["1"] = scale

    def load_own_variables(self, store):
        if not self.built:
            return
        targets = self._saved()
        if len(store.keys()) != len(targets):
            raise ValueError(f"Layer '{self.name}' expected {len(targets)} variables, but received {len(store.keys())} variables during loading. Expected: {[n for n, _ in targets]}")
        for i, (_, v) in enumerate(targets):
            v.assign(store[str(i)])
        if self.lora_enabled:
            self.lora_embeddings_a.assign(torch.zeros_like(self.lora_embeddings_a._value))
            self.lora_embeddings_b.assign(torch.zeros_like(self.lora_embeddings_b._value))

    def get_config(self):
        cfg = {
            "input_dim": self.input_dim, "output_dim": self.output_dim,
            "embeddings_initializer": initializers.serialize(self.embeddings_initializer),
            "embeddings_regularizer": regularizers.serialize(self.embeddings_regularizer),
            "activity_regularizer": regularizers.serialize(self.activity_regularizer),
            "embeddings_constraint": constraints.serialize(self.embeddings_constraint), "mask_zero": self.mask_zero,
        }
        if self.lora_rank:
            cfg["lora_rank"] = self.lora_rank
            cfg["lora_alpha"] = self.lora_alpha
        return {**super().get_config(), **cfg}

    def quantized_build(self, embeddings_shape, mode, config=None):
        if mode != "int8":
            raise self._quantization_mode_error(mode)
        self._embeddings = self.add_weight(name="embeddings", shape=embeddings_shape, initializer="zeros", dtype="int8", trainable=False)
        self.embeddings_scale = self.add_weight(name="embeddings_scale", shape=(self.input_dim,), initializer="ones", trainable=False)
        self._is_quantized = True

    def _int8_call(self, inputs, training=None):
        if inputs.dtype not in (torch.int32, torch.int64):
            inputs = inputs.to(torch.int32)
        rows = ops.take(self._embeddings.value, inputs, axis=0).to(to_compute(self))
        scale = ops.take(self.embeddings_scale.value, inputs, axis=0).to(rows.dtype)
        out = rows / scale.unsqueeze(-1)
        if self.lora_enabled:
            lora = ops.matmul(ops.take(self.lora_embeddings_a.value, inputs, axis=0), self.lora_embeddings_b.value)
            out = out + (self.lora_alpha / self.lora_rank) * lora.to(out.dtype)
        return out

    def quantize(self, mode=None, type_check=True, config=None):
        if type_check and type(self) is not Embedding:
            raise self._not_implemented_error(self.quantize)
        self.quantization_config = config
        shape = (self.input_dim, self.output_dim)
        if mode == "int8":
            q, scale = quantizers.abs_max_quantize(self._embeddings._value, axis=-1, to_numpy=False)
            self._untrack_variable(self._embeddings)
            del self._embeddings
            self.quantized_build(shape, mode)
            self._embeddings.assign(q)
            self.embeddings_scale.assign(scale.squeeze(-1))
        else:
            raise self._quantization_mode_error(mode)
        quantizers.set_quantized_policy(self, mode)


def to_compute(layer):
    from keras_b200.core.dtypes import to_torch_dtype

    return to_torch_dtype(layer.compute_dtype)


@keras_export("keras.layers.ReversibleEmbedding")
class ReversibleEmbedding(Embedding):
    def __init__(self, input_dim, output_dim, tie_weights=True, embeddings_initializer="uniform", embeddings_regularizer=None,
                 embeddings_constraint=None, mask_zero=False, reverse_dtype=None, logit_soft_cap=None, **kwargs):
        super().__init__(input_dim, output_dim, embeddings_initializer=embeddings_initializer, embeddings_regularizer=embeddings_regularizer,
                         embeddings_constraint=embeddings_constraint, mask_zero=mask_zero, **kwargs)
        self.tie_weights = tie_weights
        self.reverse_dtype = reverse_dtype
        self.logit_soft_cap = logit_soft_cap

    def build(self, inputs_shape=None):
        super().build(inputs_shape)
        if not self.tie_weights and self.quantization_mode != "int8" and not hasattr(self, "reverse_embeddings"):
            self._tracker_unlock()
            self.reverse_embeddings = self.add_weight(shape=(self.output_dim, self.input_dim), initializer=self.embeddings_initializer, name="reverse_embeddings", trainable=True)
            self._lock_state()

    def call(self, inputs, reverse=False):
        if not reverse:
            return super().call(inputs)
        kernel = ops.transpose(self.embeddings.value if hasattr(self.embeddings, "value") else self.embeddings) if self.tie_weights else self.reverse_embeddings.value
        if self.reverse_dtype is not None:
            inputs = ops.cast(inputs, self.reverse_dtype)
            kernel = ops.cast(kernel, self.reverse_dtype)
        else:
            kernel = ops.cast(kernel, inputs.dtype)
        logits = ops.matmul(inputs, kernel)
        if self.logit_soft_cap is not None:
            logits = ops.tanh(logits / self.logit_soft_cap) * self.logit_soft_cap
        return logits

    def compute_output_shape(self, input_shape, reverse=False):
        if reverse:
            return tuple(input_shape[:-1]) + (self.input_dim,)
        return super().compute_output_shape(input_shape)

    def compute_output_spec(self, inputs, reverse=False):
        if reverse:
            return KerasTensor(self.compute_output_shape(inputs.shape, reverse=True), dtype=self.reverse_dtype or self.compute_dtype)
        return super().compute_output_spec(inputs)

    def save_own_variables(self, store):
        if not self.built:
            return
        super().save_own_variables(store)
        if not self.tie_weights:
            store[str(len(store.keys()))] = self.reverse_embeddings

    def load_own_variables(self, store):
        if not self.built:
            return
        if self.tie_weights:
            return super().load_own_variables(store)
        n = len(store.keys())
        self._embeddings.assign(store["0"])
        self.reverse_embeddings.assign(store[str(n - 1)])

    def get_config(self):
        return {**super().get_config(), "tie_weights": self.tie_weights, "reverse_dtype": self.reverse_dtype, "logit_soft_cap": self.logit_soft_cap}
