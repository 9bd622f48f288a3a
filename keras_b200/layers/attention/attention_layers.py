"""Attention layers: ``MultiHeadAttention``, ``GroupedQueryAttention``, ``Attention``, ``AdditiveAttention``.

API and numerics follow keras/src/layers/attention/multi_head_attention.py:20-880,
grouped_query_attention.py, attention.py and additive_attention.py.  The 4-D case without dropout or returned
scores goes through ``ops.dot_product_attention`` (flash path on CUDA) directly on ``[B, T, N, H]`` tensors;
every other case builds explicit einsum equations over the attention axes.
"""

import math
import string

from keras_b200 import constraints, initializers, ops, regularizers
from keras_b200.core import config
from keras_b200.core.export_registry import keras_export
from keras_b200.layers.activations.activation_layers import Softmax
from keras_b200.layers.core.einsum_dense import EinsumDense
from keras_b200.layers.layer import Layer
from keras_b200.layers.regularization.regularization_layers import Dropout

_LETTERS = string.ascii_lowercase


def _proj_equation(free_dims, bound_dims, output_dims):
    """Einsum for projecting the last ``bound_dims`` axes of an input onto ``output_dims`` new axes."""
    lhs = _LETTERS[: free_dims + bound_dims]
    bound = lhs[free_dims:]
    new = _LETTERS[free_dims + bound_dims: free_dims + bound_dims + output_dims]
    return f"{lhs},{bound}{new}->{lhs[:free_dims]}{new}", new, free_dims + output_dims


def _attention_equations(rank, attn_axes):
    """(scores equation ``key,query->scores``, combine equation ``scores,value->out``, rank of scores)
    for projected tensors of ``rank`` = [batch, *dims, heads, channels]."""
    target = _LETTERS[:rank]
    batch_dims = tuple(i for i in range(rank) if i not in attn_axes and i != rank - 1)
    next_letter = rank
    source = ""
    for i in range(rank):
        if i in batch_dims or i == rank - 1:
            source += target[i]
        else:
            source += _LETTERS[next_letter]
            next_letter += 1
    product = "".join([target[i] for i in batch_dims] + [target[i] for i in attn_axes] + [source[i] for i in attn_axes])
    dot = f"{source},{target}->{product}"
    combine = f"{product},{source}->{target}"
    return dot, combine, len(product)


def _full_shape(rank, last):
    return [None] * (rank - len(last)) + list(last)


@keras_export("keras.layers.MultiHeadAttention")
class MultiHeadAttention(Layer):
    def __init__(self, num_heads, key_dim, value_dim=None, dropout=0.0, use_bias=True, output_shape=None, attention_axes=None, sliding_window=None,
                 flash_attention=None, kernel_initializer="glorot_uniform", bias_initializer="zeros", kernel_regularizer=None, bias_regularizer=None,
                 activity_regularizer=None, kernel_constraint=None, bias_constraint=None, use_gate=False, seed=None, **kwargs):
        for nm, v in (("num_heads", num_heads), ("key_dim", key_dim)):
            if not isinstance(v, int) or v <= 0:
                raise ValueError(f"Received an invalid value for argument `{nm}`, expected a positive integer. Received: {nm}={v}")
        if value_dim is not None and (not isinstance(value_dim, int) or value_dim <= 0):
            raise ValueError(f"Received an invalid value for argument `value_dim`, expected a positive integer or `None`. Received: value_dim={value_dim}")
        super().__init__(**kwargs)
        self.supports_masking = True
        self._num_heads, self._key_dim = num_heads, key_dim
        self._value_dim = value_dim if value_dim else key_dim
        self._dropout, self._use_bias, self._use_gate = dropout, use_bias, use_gate
        if output_shape:
            if isinstance(output_shape, int):
                output_shape = (output_shape,)
            try:
                output_shape = tuple(output_shape)
            except Exception:
                raise ValueError(f"Invalid `output_shape`: {output_shape}. When specified, the `output_shape` should be of type tuple, list, or int.")
        self._output_shape = output_shape
        self._flash_attention = flash_attention or config.is_flash_attention_enabled()
        self._kernel_initializer = initializers.get(kernel_initializer)
        self._bias_initializer = initializers.get(bias_initializer)
        self._kernel_regularizer = regularizers.get(kernel_regularizer)
        self._bias_regularizer = regularizers.get(bias_regularizer)
        self._activity_regularizer = regularizers.get(activity_regularizer)
        self._kernel_constraint = constraints.get(kernel_constraint)
        self._bias_constraint = constraints.get(bias_constraint)
        if isinstance(attention_axes, int):
            attention_axes = (attention_axes,)
        elif attention_axes and not isinstance(attention_axes, (list, tuple)):
            raise ValueError(f"`attention_axes` must be an int, list, or tuple.Received: attention_axes={attention_axes}")
        self._attention_axes = attention_axes
        if sliding_window is not None and (not isinstance(sliding_window, int) or sliding_window <= 0):
            raise ValueError(f"`sliding_window` must be `None` or a positive integer. Received: sliding_window={sliding_window}")
        self._sliding_window = sliding_window
        self.seed = seed
        self._inverse_sqrt_key_dim = 1.0 / math.sqrt(float(key_dim))
        if self._flash_attention and self._dropout > 0.0:
            raise ValueError("Dropout is not supported when flash attention is enabled. Please set dropout to 0.0 to use flash attention.")

    num_heads = property(lambda self: self._num_heads)
    key_dim = property(lambda self: self._key_dim)
    value_dim = property(lambda self: self._value_dim)
    dropout = property(lambda self: self._dropout)
    use_bias = property(lambda self: self._use_bias)
    output_shape = property(lambda self: self._output_shape)
    attention_axes = property(lambda self: self._attention_axes)
    query_dense = property(lambda self: self._query_dense)
    key_dense = property(lambda self: self._key_dense)
    value_dense = property(lambda self: self._value_dense)
    output_dense = property(lambda self: self._output_dense)

    def get_config(self):
        return {
            **super().get_config(),
            "num_heads": self._num_heads, "key_dim": self._key_dim, "value_dim": self._value_dim, "dropout": self._dropout,
            "use_bias": self._use_bias, "use_gate": self._use_gate, "output_shape": self._output_shape,
            "attention_axes": self._attention_axes, "sliding_window": self._sliding_window,
            "kernel_initializer": initializers.serialize(self._kernel_initializer),
            "bias_initializer": initializers.serialize(self._bias_initializer),
            "kernel_regularizer": regularizers.serialize(self._kernel_regularizer),
            "bias_regularizer": regularizers.serialize(self._bias_regularizer),
            "activity_regularizer": regularizers.serialize(self._activity_regularizer),
            "kernel_constraint": constraints.serialize(self._kernel_constraint),
            "bias_constraint": constraints.serialize(self._bias_constraint),
            "seed": self.seed,
        }

    def _sublayer_kwargs(self):
        kw = dict(kernel_regularizer=self._kernel_regularizer, bias_regularizer=self._bias_regularizer,
                  activity_regularizer=self._activity_regularizer, kernel_constraint=self._kernel_constraint,
                  bias_constraint=self._bias_constraint, dtype=self.dtype_policy)
        # fresh initializer objects per sub-layer so that each draws its own values
        kw["kernel_initializer"] = self._kernel_initializer.__class__.from_config(self._kernel_initializer.get_config())
        kw["bias_initializer"] = self._bias_initializer.__class__.from_config(self._bias_initializer.get_config())
        return kw

    def _projection(self, in_rank, heads_dims, name, activation=None):
        eq, bias_axes, out_rank = _proj_equation(in_rank - 1, bound_dims=1, output_dims=2)
        layer = EinsumDense(eq, output_shape=_full_shape(out_rank - 1, heads_dims), bias_axes=bias_axes if self._use_bias else None,
                            name=name, activation=activation, **self._sublayer_kwargs())
        return layer, out_rank

    def build(self, query_shape, value_shape, key_shape=None):
        key_shape = value_shape if key_shape is None else key_shape
        if tuple(value_shape[1:-1]) != tuple(key_shape[1:-1]):
            raise ValueError(f"All dimensions of `value` and `key`, except the last one, must be equal. Received: value_shape={value_shape} and key_shape={key_shape}")
        self._query_dense, out_rank = self._projection(len(query_shape), [self._num_heads, self._key_dim], "query")
        self._query_dense.build(query_shape)
        self._key_dense, _ = self._projection(len(key_shape), [self._num_heads, self._key_dim], "key")
        self._key_dense.build(key_shape)
        if self._use_gate:
            self._gate_dense, _ = self._projection(len(query_shape), [self._num_heads, self._value_dim], "gate", activation="sigmoid")
            self._gate_dense.build(query_shape)
        self._value_dense, out_rank = self._projection(len(value_shape), [self._num_heads, self._value_dim], "value")
        self._value_dense.build(value_shape)
        self._build_attention(out_rank)
        self._output_dense = self._make_output_dense(query_shape, self._sublayer_kwargs(), "attention_output")
        o_in = list(self._query_dense.compute_output_shape(query_shape))
        o_in[-1] = self._value_dim
        self._output_dense.build(tuple(o_in))

    def _make_output_dense(self, query_shape, common_kwargs, name=None):
        out_shape = self._output_shape if self._output_shape else [query_shape[-1]]
        eq, bias_axes, out_rank = _proj_equation(len(query_shape) - 1, bound_dims=2, output_dims=len(out_shape))
        return EinsumDense(eq, output_shape=_full_shape(out_rank - 1, out_shape), bias_axes=bias_axes if self._use_bias else None, name=name, **common_kwargs)

    def _build_attention(self, rank):
        if self._attention_axes is None:
            self._attention_axes = tuple(range(1, rank - 2))
        else:
            self._attention_axes = tuple(a if a >= 0 else (rank - 1) + a for a in self._attention_axes)
        self._dot_product_equation, self._combine_equation, scores_rank = _attention_equations(rank, self._attention_axes)
        norm_axes = tuple(range(scores_rank - len(self._attention_axes), scores_rank))
        self._softmax = Softmax(axis=norm_axes, dtype=self.dtype_policy)
        self._dropout_layer = Dropout(rate=self._dropout, dtype=self.dtype_policy, seed=self.seed)

    def _masked_softmax(self, attention_scores, attention_mask=None):
        if attention_mask is not None:
            axis = -len(self._attention_axes) * 2 - 1
            for _ in range(len(attention_scores.shape) - len(attention_mask.shape)):
                attention_mask = ops.expand_dims(attention_mask, axis=axis)
        return self._softmax(attention_scores, mask=attention_mask)

    def _compute_attention(self, query, key, value, attention_mask=None, training=None, return_attention_scores=False, use_causal_mask=False):
        fast = (len(query.shape) == 4 and self._dropout == 0.0 and not return_attention_scores and tuple(self._attention_axes) == (1,)
                and self._flash_attention is not False)
        if self._flash_attention and return_attention_scores:
            raise ValueError("Returning attention scores is not supported when flash attention is enabled. Please disable flash attention to access attention scores.")
        if fast:
            if attention_mask is not None:
                axis = -len(self._attention_axes) * 2 - 1
                for _ in range(4 - len(attention_mask.shape)):
                    attention_mask = ops.expand_dims(attention_mask, axis=axis)
                attention_mask = ops.cast(attention_mask, "bool")
            out = ops.dot_product_attention(query, key, value, bias=None, mask=attention_mask, scale=self._inverse_sqrt_key_dim,
                                            is_causal=use_causal_mask, flash_attention=self._flash_attention or None)
            return out, None
        if use_causal_mask:
            causal = self._compute_causal_mask(query, value)
            attention_mask = causal if attention_mask is None else ops.logical_and(ops.cast(attention_mask, "bool"), causal)
        query = ops.multiply(query, ops.cast(self._inverse_sqrt_key_dim, query.dtype))
        scores = ops.einsum(self._dot_product_equation, key, query)
        scores = self._masked_softmax(scores, attention_mask)
        dropped = self._dropout_layer(scores, training=training) if self._dropout > 0.0 else scores
        return ops.einsum(self._combine_equation, dropped, value), scores

    def call(self, query, value, key=None, query_mask=None, value_mask=None, key_mask=None, attention_mask=None, return_attention_scores=False,
             training=None, use_causal_mask=False):
        if key is None:
            key = value
        # The masks are handled here, at the level of the layer: the projections below see plain tensors
        # (keras/src/layers/attention/multi_head_attention.py:626-631).  Unlike there, an explicit ``query_mask`` is
        # honoured and the inputs get their masks back afterwards, so another consumer of the same tensor still sees them.
        carried = [(t, t._keras_mask) for t in {id(t): t for t in (query, value, key)}.values() if getattr(t, "_keras_mask", None) is not None]
        if query_mask is None:
            query_mask = getattr(query, "_keras_mask", None)
        for t, _ in carried:
            t._keras_mask = None
        try:
            return self._attend(query, value, key, query_mask, value_mask, key_mask, attention_mask, return_attention_scores, training, use_causal_mask)
        finally:
            for t, m in carried:
                t._keras_mask = m

    def _attend(self, query, value, key, query_mask, value_mask, key_mask, attention_mask, return_attention_scores, training, use_causal_mask):
        causal_only = (use_causal_mask and query_mask is None and value_mask is None and key_mask is None and attention_mask is None
                       and self._sliding_window is None and type(self)._compute_attention is MultiHeadAttention._compute_attention)
        if causal_only:
            attention_mask = None
        else:
            attention_mask = self._compute_attention_mask(query, value, query_mask=query_mask, value_mask=value_mask, key_mask=key_mask,
                                                          attention_mask=attention_mask, use_causal_mask=use_causal_mask)
        tp = None
        if getattr(self._query_dense._kernel, "_shard_slices", None) is not None:
            from keras_b200.parallel import tensor_parallel

            projections = [self._query_dense, self._key_dense, self._value_dense] + ([self._gate_dense] if self._use_gate else [])
            tp = tensor_parallel.mark_attention(self, projections, self._output_dense)
        gate = self._gate_dense(query) if self._use_gate else None
        q = self._query_dense(query)
        k = self._key_dense(key)
        v = self._value_dense(value)
        extra = {"use_causal_mask": True} if causal_only else {}
        out, scores = self._compute_attention(q, k, v, attention_mask, training, return_attention_scores, **extra)
        if gate is not None:
            out = ops.multiply(out, gate)
        out = self._output_dense(out)
        if query_mask is not None:
            try:
                out._keras_mask = query_mask
            except AttributeError:
                pass
        if return_attention_scores:
            if tp is not None and scores is not None:
                scores = tensor_parallel.gather_dim(scores, 1, *tp[1:])
            return out, scores
        return out

    def _compute_attention_mask(self, query, value, query_mask=None, value_mask=None, key_mask=None, attention_mask=None, use_causal_mask=False):
        auto = None
        if query_mask is not None:
            auto = ops.expand_dims(ops.cast(query_mask, "bool"), -1)
        for m in (value_mask, key_mask):
            if m is not None:
                mm = ops.expand_dims(ops.cast(m, "bool"), -2)
                auto = mm if auto is None else ops.logical_and(auto, mm)
        if use_causal_mask:
            mm = self._compute_causal_mask(query, value)
            auto = mm if auto is None else ops.logical_and(auto, mm)
        if self._sliding_window is not None:
            mm = self._compute_sliding_window_mask(query, value)
            auto = mm if auto is None else ops.logical_and(auto, mm)
        if attention_mask is not None:
            attention_mask = ops.cast(attention_mask, "bool")
        if auto is not None:
            attention_mask = auto if attention_mask is None else ops.logical_and(attention_mask, auto)
        return attention_mask

    def _compute_causal_mask(self, query, value=None):
        t = ops.shape(query)[1]
        s = t if value is None else ops.shape(value)[1]
        rows = ops.reshape(ops.arange(t, dtype="int32"), (1, t, 1))
        cols = ops.reshape(ops.arange(s, dtype="int32"), (1, 1, s))
        return ops.greater_equal(rows, cols)

    def _compute_sliding_window_mask(self, query, value=None):
        t = ops.shape(query)[1]
        s = t if value is None else ops.shape(value)[1]
        rows = ops.reshape(ops.arange(t, dtype="int32"), (1, t, 1))
        cols = ops.reshape(ops.arange(s, dtype="int32"), (1, 1, s))
        return ops.less(ops.abs(ops.subtract(rows, cols)), self._sliding_window)

    def compute_mask(self, inputs, previous_mask=None):
        return None

    def compute_output_shape(self, query_shape, value_shape, key_shape=None):
        query_shape, value_shape = tuple(query_shape), tuple(value_shape)
        key_shape = value_shape if key_shape is None else tuple(key_shape)
        if value_shape[1:-1] != key_shape[1:-1]:
            raise ValueError(f"All dimensions of `value` and `key`, except the last one, must be equal. Received: value_shape={value_shape} and key_shape={key_shape}")
        if self._output_shape:
            query_shape = query_shape[:-1] + self._output_shape
        return query_shape

    def compute_output_spec(self, query, value, key=None, query_mask=None, value_mask=None, key_mask=None, attention_mask=None,
                            return_attention_scores=False, training=None, use_causal_mask=False):
        from keras_b200.core.keras_tensor import KerasTensor

        key_shape = key.shape if key is not None else None
        out_shape = self.compute_output_shape(query.shape, value.shape, key_shape)
        out = KerasTensor(out_shape, dtype=self.compute_dtype)
        if return_attention_scores:
            length = query.shape[1]
            scores_shape = (query.shape[0], self._num_heads, length, value.shape[1])
            return out, KerasTensor(scores_shape, dtype=self.compute_dtype)
        return out


@keras_export(["keras.layers.GroupQueryAttention", "keras.layers.GroupedQueryAttention"])
class GroupedQueryAttention(Layer):
    """Grouped-query attention (keras/src/layers/attention/grouped_query_attention.py): ``num_query_heads`` query
    heads share ``num_key_value_heads`` key/value heads.  K/V are never repeated in memory on the fused path."""

    def __init__(self, head_dim, num_query_heads, num_key_value_heads, dropout=0.0, use_bias=True, flash_attention=None,
                 kernel_initializer="glorot_uniform", bias_initializer="zeros", kernel_regularizer=None, bias_regularizer=None,
                 activity_regularizer=None, kernel_constraint=None, bias_constraint=None, use_gate=False, seed=None, **kwargs):
        super().__init__(**kwargs)
        self.supports_masking = True
        self.head_dim, self.num_query_heads, self.num_key_value_heads = head_dim, num_query_heads, num_key_value_heads
        if num_query_heads % num_key_value_heads != 0:
            raise ValueError("`num_query_heads` must be divisible by `num_key_value_heads`.")
        self.num_repeats = num_query_heads // num_key_value_heads
        self.dropout, self.use_bias, self.use_gate = dropout, use_bias, use_gate
        self._flash_attention = flash_attention or config.is_flash_attention_enabled()
        self.kernel_initializer = initializers.get(kernel_initializer)
        self.bias_initializer = initializers.get(bias_initializer)
        self.kernel_regularizer = regularizers.get(kernel_regularizer)
        self.bias_regularizer = regularizers.get(bias_regularizer)
        self.activity_regularizer = regularizers.get(activity_regularizer)
        self.kernel_constraint = constraints.get(kernel_constraint)
        self.bias_constraint = constraints.get(bias_constraint)
        self.seed = seed
        self._inverse_sqrt_head_dim = 1.0 / math.sqrt(float(head_dim))
        self._return_attention_scores = False
        if self._flash_attention and self.dropout > 0.0:
            raise ValueError("Dropout is not supported when flash attention is enabled. Please set dropout to 0.0 to use flash attention.")

    def _kw(self):
        return dict(kernel_initializer=self.kernel_initializer.__class__.from_config(self.kernel_initializer.get_config()),
                    bias_initializer=self.bias_initializer.__class__.from_config(self.bias_initializer.get_config()),
                    kernel_regularizer=self.kernel_regularizer, bias_regularizer=self.bias_regularizer,
                    activity_regularizer=self.activity_regularizer, kernel_constraint=self.kernel_constraint,
                    bias_constraint=self.bias_constraint, dtype=self.dtype_policy)

    def build(self, query_shape, value_shape, key_shape=None):
        key_shape = value_shape if key_shape is None else key_shape
        self.feature_dim = query_shape[-1]
        self._query_dense = EinsumDense("bqm,muh->bquh", output_shape=(None, self.num_query_heads, self.head_dim),
                                        bias_axes="uh" if self.use_bias else None, name="query", **self._kw())
        self._query_dense.build(query_shape)
        self._key_dense = EinsumDense("bkm,mvh->bkvh", output_shape=(None, self.num_key_value_heads, self.head_dim),
                                      bias_axes="vh" if self.use_bias else None, name="key", **self._kw())
        self._key_dense.build(key_shape)
        self._value_dense = EinsumDense("bkm,mvh->bkvh", output_shape=(None, self.num_key_value_heads, self.head_dim),
                                        bias_axes="vh" if self.use_bias else None, name="value", **self._kw())
        self._value_dense.build(value_shape)
        if self.use_gate:
            self._gate_dense = EinsumDense("bqm,muh->bquh", output_shape=(None, self.num_query_heads, self.head_dim),
                                           bias_axes="uh" if self.use_bias else None, activation="sigmoid", name="gate", **self._kw())
            self._gate_dense.build(query_shape)
        self._softmax = Softmax(axis=-1, dtype=self.dtype_policy)
        self._dropout_layer = Dropout(rate=self.dropout, dtype=self.dtype_policy, seed=self.seed)
        self._dot_product_equation = "bquh,bkuh->buqk"
        self._combine_equation = "buqk,bkuh->bquh"
        self._output_dense = EinsumDense("bquh,uhm->bqm", output_shape=(None, self.feature_dim), bias_axes="m" if self.use_bias else None,
                                         name="attention_output", **self._kw())
        self._output_dense.build((None, None, self.num_query_heads, self.head_dim))

    query_dense = property(lambda self: self._query_dense)
    key_dense = property(lambda self: self._key_dense)
    value_dense = property(lambda self: self._value_dense)
    output_dense = property(lambda self: self._output_dense)

    def call(self, query, value, key=None, query_mask=None, value_mask=None, key_mask=None, attention_mask=None, return_attention_scores=False,
             training=None, use_causal_mask=False):
        self._return_attention_scores = return_attention_scores
        if key is None:
            key = value
        # a purely causal mask is passed to the fused attention kernel as a flag instead of a [T, T] tensor
        self._causal_only = bool(use_causal_mask and query_mask is None and value_mask is None and key_mask is None and attention_mask is None
                                 and self.dropout == 0.0 and not return_attention_scores and self._flash_attention is not False)
        if not self._causal_only:
            attention_mask = self._compute_attention_mask(query, value, query_mask=query_mask, value_mask=value_mask, key_mask=key_mask,
                                                          attention_mask=attention_mask, use_causal_mask=use_causal_mask)
        tp = None
        if getattr(self._query_dense._kernel, "_shard_slices", None) is not None:
            from keras_b200.parallel import tensor_parallel

            projections = [self._query_dense, self._key_dense, self._value_dense] + ([self._gate_dense] if self.use_gate else [])
            tp = tensor_parallel.mark_attention(self, projections, self._output_dense)
        gate = self._gate_dense(query) if self.use_gate else None
        q = self._query_dense(query)
        k = self._key_dense(key)
        v = self._value_dense(value)
        out, scores = self._compute_attention(q, k, v, attention_mask=attention_mask, training=training)
        if gate is not None:
            out = ops.multiply(out, gate)
        out = self._output_dense(out)
        if return_attention_scores:
            if tp is not None and scores is not None:
                scores = tensor_parallel.gather_dim(scores, 1, *tp[1:])
            return out, scores
        return out

    _compute_attention_mask = MultiHeadAttention._compute_attention_mask
    _compute_causal_mask = MultiHeadAttention._compute_causal_mask
    _sliding_window = None

    def _masked_softmax(self, scores, attention_mask=None):
        if attention_mask is not None:
            for _ in range(len(scores.shape) - len(attention_mask.shape)):
                attention_mask = ops.expand_dims(attention_mask, axis=-3)
        return self._softmax(scores, mask=attention_mask)

    def _compute_attention(self, query, key, value, attention_mask=None, training=None):
        if self._flash_attention and self._return_attention_scores:
            raise ValueError("Returning attention scores is not supported when flash attention is enabled. Please disable flash attention to access attention scores.")
        if self.dropout == 0.0 and not self._return_attention_scores and self._flash_attention is not False:
            if attention_mask is not None:
                for _ in range(4 - len(attention_mask.shape)):
                    attention_mask = ops.expand_dims(attention_mask, axis=-3)
                attention_mask = ops.cast(attention_mask, "bool")
            out = ops.dot_product_attention(query, key, value, mask=attention_mask, scale=self._inverse_sqrt_head_dim,
                                            is_causal=bool(getattr(self, "_causal_only", False)) and attention_mask is None,
                                            flash_attention=self._flash_attention or None)
            return out, None
        key = ops.repeat(key, self.num_repeats, axis=2)
        value = ops.repeat(value, self.num_repeats, axis=2)
        query = ops.multiply(query, ops.cast(self._inverse_sqrt_head_dim, query.dtype))
        scores = ops.einsum(self._dot_product_equation, query, key)
        scores = self._masked_softmax(scores, attention_mask)
        dropped = self._dropout_layer(scores, training=training) if self.dropout > 0.0 else scores
        return ops.einsum(self._combine_equation, dropped, value), scores

    def compute_mask(self, inputs, previous_mask=None):
        return None

    def compute_output_shape(self, query_shape, value_shape, key_shape=None):
        key_shape = value_shape if key_shape is None else key_shape
        if tuple(value_shape[1:-1]) != tuple(key_shape[1:-1]):
            raise ValueError(f"All dimensions of `value` and `key`, except the last one, must be equal. Received: value_shape={value_shape} and key_shape={key_shape}")
        return tuple(query_shape)

    def get_config(self):
        return {
            **super().get_config(),
            "head_dim": self.head_dim, "num_query_heads": self.num_query_heads, "num_key_value_heads": self.num_key_value_heads,
            "use_bias": self.use_bias, "dropout": self.dropout, "use_gate": self.use_gate,
            "kernel_initializer": initializers.serialize(self.kernel_initializer), "bias_initializer": initializers.serialize(self.bias_initializer),
            "kernel_regularizer": regularizers.serialize(self.kernel_regularizer), "bias_regularizer": regularizers.serialize(self.bias_regularizer),
            "activity_regularizer": regularizers.serialize(self.activity_regularizer),
            "kernel_constraint": constraints.serialize(self.kernel_constraint), "bias_constraint": constraints.serialize(self.bias_constraint),
            "seed": self.seed,
        }


GroupQueryAttention = GroupedQueryAttention


@keras_export("keras.layers.Attention")
class Attention(Layer):
    """Dot-product (Luong) attention over ``[query, value, key?]`` (keras/src/layers/attention/attention.py)."""

    def __init__(self, use_scale=False, score_mode="dot", dropout=0.0, seed=None, **kwargs):
        super().__init__(**kwargs)
        self.use_scale, self.score_mode, self.dropout = use_scale, score_mode, dropout
        if self.dropout > 0:
            from keras_b200.random.seed_generator import SeedGenerator

            self.seed_generator = SeedGenerator(seed=seed)
        if score_mode not in ("dot", "concat"):
            raise ValueError(f"Invalid value for argument score_mode. Expected one of {{'dot', 'concat'}}. Received: score_mode={score_mode}")
        self._return_attention_scores = False

    def build(self, input_shape):
        self._validate_inputs(input_shape)
        self.scale = None
        self.concat_score_weight = None
        if self.use_scale:
            self.scale = self.add_weight(name="scale", shape=(), initializer="ones", dtype=self.dtype, trainable=True)
        if self.score_mode == "concat":
            self.concat_score_weight = self.add_weight(name="concat_score_weight", shape=(), initializer="ones", dtype=self.dtype, trainable=True)

    def _calculate_scores(self, query, key):
        if self.score_mode == "dot":
            scores = ops.matmul(query, ops.transpose(key, axes=[0, 2, 1]))
            if self.scale is not None:
                scores = ops.multiply(scores, self.scale)
        else:
            q = ops.expand_dims(query, axis=-2)
            k = ops.expand_dims(key, axis=-3)
            if self.scale is not None:
                scores = self.concat_score_weight * ops.sum(ops.tanh(self.scale * (q + k)), axis=-1)
            else:
                scores = self.concat_score_weight * ops.sum(ops.tanh(q + k), axis=-1)
        return scores

    def _apply_scores(self, scores, value, scores_mask=None, training=False):
        if scores_mask is not None:
            padding_mask = ops.logical_not(scores_mask)
            max_value = 65504.0 if str(scores.dtype).endswith("float16") and "bfloat" not in str(scores.dtype) else 1.0e9
            if len(padding_mask.shape) == 2:
                padding_mask = ops.expand_dims(padding_mask, axis=-2)
            scores = ops.subtract(scores, ops.multiply(max_value, ops.cast(padding_mask, dtype=scores.dtype)))
        weights = ops.softmax(scores, axis=-1)
        if training and self.dropout > 0:
            from keras_b200 import random

            weights = random.dropout(weights, self.dropout, seed=self.seed_generator)
        return ops.matmul(weights, value), weights

    def _calculate_score_mask(self, scores, v_mask, use_causal_mask):
        if use_causal_mask:
            shape = ops.shape(scores)
            t, s = shape[-2], shape[-1]
            rows = ops.reshape(ops.arange(t, dtype="int32"), (1, t, 1))
            cols = ops.reshape(ops.arange(s, dtype="int32"), (1, 1, s))
            causal = ops.greater_equal(rows, cols)
            if v_mask is not None:
                v_mask = ops.expand_dims(v_mask, axis=-2)
                return ops.logical_and(v_mask, causal)
            return causal
        return v_mask

    def call(self, inputs, mask=None, training=False, return_attention_scores=False, use_causal_mask=False):
        self._validate_inputs(inputs=inputs, mask=mask)
        self._return_attention_scores = return_attention_scores
        q, v = inputs[0], inputs[1]
        k = inputs[2] if len(inputs) > 2 else v
        q_mask = mask[0] if mask else None
        v_mask = mask[1] if mask else None
        scores = self._calculate_scores(query=q, key=k)
        scores_mask = self._calculate_score_mask(scores, v_mask, use_causal_mask)
        result, attention_scores = self._apply_scores(scores=scores, value=v, scores_mask=scores_mask, training=training)
        if q_mask is not None:
            q_mask = ops.expand_dims(q_mask, axis=-1)
            result = ops.multiply(result, ops.cast(q_mask, dtype=result.dtype))
        if return_attention_scores:
            return result, attention_scores
        return result

    def compute_mask(self, inputs, mask=None):
        self._validate_inputs(inputs=inputs, mask=mask)
        if mask is None or mask[0] is None:
            return None
        return ops.convert_to_tensor(mask[0])

    def compute_output_shape(self, input_shape):
        output_shape = (*input_shape[0][:-1], input_shape[1][-1])
        if self._return_attention_scores:
            return output_shape, (*input_shape[0][:-1], input_shape[1][1])
        return output_shape

    def compute_output_spec(self, inputs, mask=None, return_attention_scores=False, training=None, use_causal_mask=False):
        from keras_b200.core.keras_tensor import KerasTensor

        shapes = [i.shape for i in inputs]
        self._return_attention_scores = False
        out = KerasTensor(self.compute_output_shape(shapes), dtype=self.compute_dtype)
        if return_attention_scores:
            return out, KerasTensor((*shapes[0][:-1], shapes[1][1]), dtype=self.compute_dtype)
        return out

    def _validate_inputs(self, inputs, mask=None):
        cls = self.__class__.__name__
        if not isinstance(inputs, (list, tuple)):
            raise ValueError(f"{cls} layer must be called on a list of inputs, namely [query, value] or [query, value, key]. Received: inputs={inputs}.")
        if len(inputs) < 2 or len(inputs) > 3:
            raise ValueError(f"{cls} layer accepts inputs list of length 2 or 3, namely [query, value] or [query, value, key]. Received length: {len(inputs)}.")
        if mask is not None:
            if not isinstance(mask, (list, tuple)):
                raise ValueError(f"{cls} layer mask must be a list, namely [query_mask, value_mask]. Received: mask={mask}.")
            if len(mask) < 2 or len(mask) > 3:
                raise ValueError(f"{cls} layer accepts mask list of length 2 or 3. Received: inputs={inputs}, mask={mask}.")

    def get_config(self):
        return {**super().get_config(), "use_scale": self.use_scale, "score_mode": self.score_mode, "dropout": self.dropout}


@keras_export("keras.layers.AdditiveAttention")
class AdditiveAttention(Attention):
    """Bahdanau attention: ``scores = sum(scale * tanh(query + key))`` (keras/src/layers/attention/additive_attention.py)."""

    def __init__(self, use_scale=True, dropout=0.0, **kwargs):
        super().__init__(use_scale=use_scale, dropout=dropout, **kwargs)

    def build(self, input_shape):
        self._validate_inputs(input_shape)
        dim = input_shape[0][-1]
        self.scale = None
        if self.use_scale:
            self.scale = self.add_weight(name="scale", shape=[dim], initializer="glorot_uniform", dtype=self.dtype, trainable=True)

    def _calculate_scores(self, query, key):
        q = ops.expand_dims(query, axis=-2)
        k = ops.expand_dims(key, axis=-3)
        scale = self.scale if self.use_scale else 1.0
        return ops.sum(scale * ops.tanh(q + k), axis=-1)

    def get_config(self):
        cfg = super().get_config()
        del cfg["score_mode"]
        return cfg
