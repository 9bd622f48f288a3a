"""Recurrent layers: ``RNN``, ``SimpleRNN``/``LSTM``/``GRU`` (+cells), ``StackedRNNCells``, ``Bidirectional``,
``TimeDistributed`` and ``ConvLSTM1D/2D/3D``.

Weights, gate order and configs follow keras/src/layers/rnn/{rnn,simple_rnn,lstm,gru,stacked_rnn_cells,
bidirectional,time_distributed,conv_lstm}.py.  LSTM and GRU without dropout hoist the input projection of all
time steps into one GEMM (``[B*T, in] x [in, gates]``) and leave only the recurrent GEMM inside the time loop.
"""

import torch

from keras_b200 import activations, constraints, initializers, ops, regularizers, tree
from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_tensor
from keras_b200.layers.input_spec import InputSpec
from keras_b200.layers.layer import Layer
from keras_b200.layers.rnn.rnn_loop import rnn as rnn_loop
from keras_b200.saving import serialization_lib


class DropoutRNNCell:
    """Mixin giving a cell its input-dropout and recurrent-dropout masks, drawn once per sequence and reused at every step
    (keras/src/layers/rnn/dropout_rnn_cell.py).  A cell that sets ``dropout_mask_count`` gets that many independent masks, one per
    gate, drawn one after the other from the cell's seed generator."""

    def _mask(self, attr, rate, like):
        if rate == 0:
            return None
        m = getattr(self, attr, None)
        if m is None:
            from keras_b200 import random

            count = getattr(self, "dropout_mask_count", None)
            ones = ops.ones_like(like)
            if count is None:
                m = random.dropout(ones, rate=rate, seed=self.seed_generator)
            else:
                m = [random.dropout(ones, rate=rate, seed=self.seed_generator) for _ in range(count)]
            object.__setattr__(self, attr, m)
        return m

    def get_dropout_mask(self, step_input):
        return self._mask("_dropout_mask", self.dropout, step_input)

    def get_recurrent_dropout_mask(self, step_input):
        return self._mask("_recurrent_dropout_mask", self.recurrent_dropout, step_input)

    def reset_dropout_mask(self):
        object.__setattr__(self, "_dropout_mask", None)

    def reset_recurrent_dropout_mask(self):
        object.__setattr__(self, "_recurrent_dropout_mask", None)


def _gate_matmul(x, masks, weight, gates):
    """``x @ weight`` where gate ``g`` (a block of columns of ``weight``) sees ``x * masks[g]``."""
    if masks is None:
        return ops.matmul(x, weight)
    w = weight.value if hasattr(weight, "value") else weight
    u = w.shape[1] // gates
    return ops.concatenate([ops.matmul(x * masks[g], w[:, g * u:(g + 1) * u]) for g in range(gates)], axis=-1)


def _use_gate_masks(cell, implementation):
    """Recurrent dropout forces the per-gate formulation, which draws one mask per gate (keras/src/layers/rnn/lstm.py:136-139)."""
    cell.implementation = 1 if cell.recurrent_dropout != 0.0 else implementation
    if cell.implementation == 1:
        cell.dropout_mask_count = cell.GATES


class _BaseCell(Layer, DropoutRNNCell):
    GATES = 1

    def __init__(self, units, activation="tanh", use_bias=True, kernel_initializer="glorot_uniform", recurrent_initializer="orthogonal",
                 bias_initializer="zeros", kernel_regularizer=None, recurrent_regularizer=None, bias_regularizer=None, kernel_constraint=None,
                 recurrent_constraint=None, bias_constraint=None, dropout=0.0, recurrent_dropout=0.0, seed=None, **kwargs):
        if units <= 0:
            raise ValueError(f"Received an invalid value for argument `units`, expected a positive integer, got {units}.")
        super().__init__(**kwargs)
        from keras_b200.random.seed_generator import SeedGenerator

        self.seed = seed
        self.seed_generator = SeedGenerator(seed)
        self.units = units
        self.activation = activations.get(activation)
        self.use_bias = use_bias
        self.kernel_initializer = initializers.get(kernel_initializer)
        self.recurrent_initializer = initializers.get(recurrent_initializer)
        self.bias_initializer = initializers.get(bias_initializer)
        self.kernel_regularizer = regularizers.get(kernel_regularizer)
        self.recurrent_regularizer = regularizers.get(recurrent_regularizer)
        self.bias_regularizer = regularizers.get(bias_regularizer)
        self.kernel_constraint = constraints.get(kernel_constraint)
        self.recurrent_constraint = constraints.get(recurrent_constraint)
        self.bias_constraint = constraints.get(bias_constraint)
        self.dropout = min(1.0, max(0.0, dropout))
        self.recurrent_dropout = min(1.0, max(0.0, recurrent_dropout))
        self.state_size = units
        self.output_size = units

    def _bias_shape(self):
        return (self.GATES * self.units,)

    def _bias_init(self):
        return self.bias_initializer

    def build(self, input_shape):
        g = self.GATES * self.units
        self.kernel = self.add_weight(shape=(input_shape[-1], g), name="kernel", initializer=self.kernel_initializer,
                                      regularizer=self.kernel_regularizer, constraint=self.kernel_constraint)
        self.recurrent_kernel = self.add_weight(shape=(self.units, g), name="recurrent_kernel", initializer=self.recurrent_initializer,
                                                regularizer=self.recurrent_regularizer, constraint=self.recurrent_constraint)
        if self.use_bias:
            self.bias = self.add_weight(shape=self._bias_shape(), name="bias", initializer=self._bias_init(), regularizer=self.bias_regularizer,
                                        constraint=self.bias_constraint)
        else:
            self.bias = None

    def get_initial_state(self, batch_size=None):
        return [ops.zeros((batch_size, self.state_size), dtype=self.compute_dtype)]

    def _base_config(self):
        return {
            "units": self.units, "activation": activations.serialize(self.activation), "use_bias": self.use_bias,
            "kernel_initializer": initializers.serialize(self.kernel_initializer),
            "recurrent_initializer": initializers.serialize(self.recurrent_initializer),
            "bias_initializer": initializers.serialize(self.bias_initializer),
            "kernel_regularizer": regularizers.serialize(self.kernel_regularizer),
            "recurrent_regularizer": regularizers.serialize(self.recurrent_regularizer),
            "bias_regularizer": regularizers.serialize(self.bias_regularizer),
            "kernel_constraint": constraints.serialize(self.kernel_constraint),
            "recurrent_constraint": constraints.serialize(self.recurrent_constraint),
            "bias_constraint": constraints.serialize(self.bias_constraint),
            "dropout": self.dropout, "recurrent_dropout": self.recurrent_dropout, "seed": self.seed,
        }

    def get_config(self):
        return {**super().get_config(), **self._base_config()}


@keras_export("keras.layers.SimpleRNNCell")
class SimpleRNNCell(_BaseCell):
    def call(self, sequence, states, training=False):
        prev = states[0] if isinstance(states, (list, tuple)) else states
        dp = self.get_dropout_mask(sequence) if training else None
        rdp = self.get_recurrent_dropout_mask(prev) if training else None
        if dp is not None:
            sequence = sequence * dp
        h = ops.matmul(sequence, self.kernel)
        if self.bias is not None:
            h = ops.add(h, self.bias)
        if rdp is not None:
            prev = prev * rdp
        out = h + ops.matmul(prev, self.recurrent_kernel)
        if self.activation is not None:
            out = self.activation(out)
        new_state = [out] if isinstance(states, (list, tuple)) else out
        return out, new_state


@keras_export("keras.layers.LSTMCell")
class LSTMCell(_BaseCell):
    GATES = 4

    def __init__(self, units, activation="tanh", recurrent_activation="sigmoid", use_bias=True, kernel_initializer="glorot_uniform",
                 recurrent_initializer="orthogonal", bias_initializer="zeros", unit_forget_bias=True, kernel_regularizer=None,
                 recurrent_regularizer=None, bias_regularizer=None, kernel_constraint=None, recurrent_constraint=None, bias_constraint=None,
                 dropout=0.0, recurrent_dropout=0.0, seed=None, **kwargs):
        implementation = kwargs.pop("implementation", 2)
        super().__init__(units, activation, use_bias, kernel_initializer, recurrent_initializer, bias_initializer, kernel_regularizer,
                         recurrent_regularizer, bias_regularizer, kernel_constraint, recurrent_constraint, bias_constraint, dropout,
                         recurrent_dropout, seed, **kwargs)
        self.recurrent_activation = activations.get(recurrent_activation)
        self.unit_forget_bias = unit_forget_bias
        _use_gate_masks(self, implementation)
        self.state_size = [units, units]

    def _bias_init(self):
        if not self.unit_forget_bias:
            return self.bias_initializer
        u = self.units
        base = self.bias_initializer

        def init(shape, dtype=None, **kw):
            return ops.concatenate([base((u,), dtype=dtype), initializers.get("ones")((u,), dtype=dtype), base((u * 2,), dtype=dtype)])

        return init

    def gates(self, z, c_prev):
        u = self.units
        i = self.recurrent_activation(z[:, :u])
        f = self.recurrent_activation(z[:, u:2 * u])
        c = f * c_prev + i * self.activation(z[:, 2 * u:3 * u])
        o = self.recurrent_activation(z[:, 3 * u:])
        return o * self.activation(c), c

    def call(self, sequence, states, training=False):
        h_prev, c_prev = states[0], states[1]
        dp = self.get_dropout_mask(sequence) if training and 0.0 < self.dropout < 1.0 else None
        if self.implementation == 1:
            rdp = self.get_recurrent_dropout_mask(h_prev) if training and 0.0 < self.recurrent_dropout < 1.0 else None
            z = _gate_matmul(sequence, dp, self.kernel, 4) + _gate_matmul(h_prev, rdp, self.recurrent_kernel, 4)
        else:
            if dp is not None:
                sequence = sequence * dp
            z = ops.matmul(sequence, self.kernel) + ops.matmul(h_prev, self.recurrent_kernel)
        if self.bias is not None:
            z = ops.add(z, self.bias)
        h, c = self.gates(z, c_prev)
        return h, [h, c]

    def get_initial_state(self, batch_size=None):
        return [ops.zeros((batch_size, d), dtype=self.compute_dtype) for d in self.state_size]

    def get_config(self):
        cfg = super().get_config()
        cfg.update({"recurrent_activation": activations.serialize(self.recurrent_activation), "unit_forget_bias": self.unit_forget_bias})
        return cfg


@keras_export("keras.layers.GRUCell")
class GRUCell(_BaseCell):
    GATES = 3

    def __init__(self, units, activation="tanh", recurrent_activation="sigmoid", use_bias=True, kernel_initializer="glorot_uniform",
                 recurrent_initializer="orthogonal", bias_initializer="zeros", kernel_regularizer=None, recurrent_regularizer=None,
                 bias_regularizer=None, kernel_constraint=None, recurrent_constraint=None, bias_constraint=None, dropout=0.0,
                 recurrent_dropout=0.0, reset_after=True, seed=None, **kwargs):
        implementation = kwargs.pop("implementation", 2)
        super().__init__(units, activation, use_bias, kernel_initializer, recurrent_initializer, bias_initializer, kernel_regularizer,
                         recurrent_regularizer, bias_regularizer, kernel_constraint, recurrent_constraint, bias_constraint, dropout,
                         recurrent_dropout, seed, **kwargs)
        self.recurrent_activation = activations.get(recurrent_activation)
        self.reset_after = reset_after
        _use_gate_masks(self, implementation)

    def _bias_shape(self):
        return (2, 3 * self.units) if self.reset_after else (3 * self.units,)

    def step_from_projection(self, xz, h_prev, recurrent_bias):
        """One GRU step given the input projection ``xz = x @ kernel + input_bias``."""
        u = self.units
        if self.reset_after:
            inner = ops.matmul(h_prev, self.recurrent_kernel)
            if recurrent_bias is not None:
                inner = inner + recurrent_bias
            z = self.recurrent_activation(xz[:, :u] + inner[:, :u])
            r = self.recurrent_activation(xz[:, u:2 * u] + inner[:, u:2 * u])
            hh = self.activation(xz[:, 2 * u:] + r * inner[:, 2 * u:])
        else:
            rk = self.recurrent_kernel
            rk = rk.value if hasattr(rk, "value") else rk
            zr = ops.matmul(h_prev, rk[:, :2 * u])
            z = self.recurrent_activation(xz[:, :u] + zr[:, :u])
            r = self.recurrent_activation(xz[:, u:2 * u] + zr[:, u:])
            hh = self.activation(xz[:, 2 * u:] + ops.matmul(r * h_prev, rk[:, 2 * u:]))
        return z * h_prev + (1 - z) * hh

    def _step_with_gate_masks(self, xz, h_prev, recurrent_bias, masks):
        """The per-gate formulation: each gate sees the previous state under its own recurrent-dropout mask; the state carried
        over by the update gate is the unmasked one (keras/src/layers/rnn/gru.py:196-254)."""
        u = self.units
        rk = self.recurrent_kernel
        rk = rk.value if hasattr(rk, "value") else rk
        hz, hr, hh_in = (h_prev * m for m in masks) if masks is not None else (h_prev, h_prev, h_prev)
        rz, rr = ops.matmul(hz, rk[:, :u]), ops.matmul(hr, rk[:, u:2 * u])
        if recurrent_bias is not None:
            rz, rr = rz + recurrent_bias[:u], rr + recurrent_bias[u:2 * u]
        z = self.recurrent_activation(xz[:, :u] + rz)
        r = self.recurrent_activation(xz[:, u:2 * u] + rr)
        if self.reset_after:
            rh = ops.matmul(hh_in, rk[:, 2 * u:])
            if recurrent_bias is not None:
                rh = rh + recurrent_bias[2 * u:]
            rh = r * rh
        else:
            rh = ops.matmul(r * hh_in, rk[:, 2 * u:])
        hh = self.activation(xz[:, 2 * u:] + rh)
        return z * h_prev + (1 - z) * hh

    def _split_bias(self):
        if self.bias is None:
            return None, None
        b = self.bias.value if hasattr(self.bias, "value") else self.bias
        if self.reset_after:
            return b[0], b[1]
        return b, None

    def call(self, sequence, states, training=False):
        h_prev = states[0] if isinstance(states, (list, tuple)) else states
        dp = self.get_dropout_mask(sequence) if training and 0.0 < self.dropout < 1.0 else None
        ib, rb = self._split_bias()
        if self.implementation == 1:
            rdp = self.get_recurrent_dropout_mask(h_prev) if training and 0.0 < self.recurrent_dropout < 1.0 else None
            xz = _gate_matmul(sequence, dp, self.kernel, 3)
            if ib is not None:
                xz = xz + ib
            h = self._step_with_gate_masks(xz, h_prev, rb, rdp)
        else:
            xz = ops.matmul(sequence * dp if dp is not None else sequence, self.kernel)
            if ib is not None:
                xz = xz + ib
            h = self.step_from_projection(xz, h_prev, rb)
        new_state = [h] if isinstance(states, (list, tuple)) else h
        return h, new_state

    def get_config(self):
        cfg = super().get_config()
        cfg.update({"recurrent_activation": activations.serialize(self.recurrent_activation), "reset_after": self.reset_after})
        return cfg


@keras_export("keras.layers.StackedRNNCells")
class StackedRNNCells(Layer):
    def __init__(self, cells, **kwargs):
        super().__init__(**kwargs)
        for cell in cells:
            if "call" not in dir(cell):
                raise ValueError(f"All cells must have a `call` method. Received cell without a `call` method: {cell}")
            if "state_size" not in dir(cell):
                raise ValueError(f"All cells must have a `state_size` attribute. Received cell without a `state_size` attribute: {cell}")
        self.cells = cells

    @property
    def state_size(self):
        return [c.state_size for c in self.cells]

    @property
    def output_size(self):
        last = self.cells[-1]
        if getattr(last, "output_size", None) is not None:
            return last.output_size
        if tree.is_nested(last.state_size):
            return last.state_size[0]
        return last.state_size

    def get_initial_state(self, batch_size=None):
        out = []
        for cell in self.cells:
            fn = getattr(cell, "get_initial_state", None)
            if fn:
                out.append(fn(batch_size=batch_size))
            elif tree.is_nested(cell.state_size):
                out.append([ops.zeros((batch_size, d), dtype=self.compute_dtype) for d in cell.state_size])
            else:
                out.append(ops.zeros((batch_size, cell.state_size), dtype=self.compute_dtype))
        return out

    def call(self, inputs, states, training=False, **kwargs):
        new_states = []
        for cell, st in zip(self.cells, states):
            nested = tree.is_nested(st)
            st = list(st) if nested else [st]
            if isinstance(cell, Layer):
                kw = dict(kwargs)
                if cell._call_has_training_arg:
                    kw["training"] = training
                inputs, st = cell(inputs, st, **kw)
            else:
                inputs, st = cell.call(inputs, st, **kwargs)
            if len(st) == 1 and not nested:
                st = st[0]
            new_states.append(st)
        return inputs, new_states

    def build(self, input_shape):
        for cell in self.cells:
            if isinstance(cell, Layer) and not cell.built:
                cell.build(input_shape)
                cell.built = True
            out_dim = getattr(cell, "output_size", None)
            if out_dim is None:
                out_dim = cell.state_size[0] if tree.is_nested(cell.state_size) else cell.state_size
            input_shape = (input_shape[0], out_dim)

    def get_config(self):
        return {**super().get_config(), "cells": [serialization_lib.serialize_keras_object(c) for c in self.cells]}

    @classmethod
    def from_config(cls, config, custom_objects=None):
        cells = [serialization_lib.deserialize_keras_object(c, custom_objects=custom_objects) for c in config.pop("cells")]
        return cls(cells, **config)


@keras_export("keras.layers.RNN")
class RNN(Layer):
    def __init__(self, cell, return_sequences=False, return_state=False, go_backwards=False, stateful=False, unroll=False,
                 zero_output_for_mask=False, **kwargs):
        if isinstance(cell, (list, tuple)):
            cell = StackedRNNCells(cell)
        if "call" not in dir(cell):
            raise ValueError(f"Argument `cell` should have a `call` method. Received: cell={cell}")
        if "state_size" not in dir(cell):
            raise ValueError(f"The RNN cell should have a `state_size` attribute (single integer or list of integers, one integer per RNN state). Received: cell={cell}")
        super().__init__(**kwargs)
        self.zero_output_for_mask = zero_output_for_mask
        self.cell = cell
        self.return_sequences, self.return_state, self.go_backwards = return_sequences, return_state, go_backwards
        self.stateful, self.unroll = stateful, unroll
        # the mask steers the recurrence (through the ``mask`` argument) but is not attached to the output
        # (keras/src/layers/rnn/rnn.py:212)
        self.supports_masking = False
        self.input_spec = None
        self.states = None
        self._expected_batch_size = None
        state_size = getattr(self.cell, "state_size", None)
        if state_size is None:
            raise ValueError("state_size must be specified as property on the RNN cell.")
        if not isinstance(state_size, (list, tuple, int)):
            raise ValueError("state_size must be an integer, or a list/tuple of integers (one for each state tensor).")
        if isinstance(state_size, int):
            self.state_size, self.single_state = [state_size], True
        else:
            self.state_size, self.single_state = list(state_size), False

    def compute_output_shape(self, sequences_shape, initial_state_shape=None):
        batch, length = sequences_shape[0], sequences_shape[1]
        states_shape = []
        for s in self.state_size:
            if isinstance(s, int):
                states_shape.append((batch, s))
            else:
                states_shape.append([(batch, d) for d in s])
        out_size = getattr(self.cell, "output_size", None)
        if out_size is None:
            out_size = self.state_size[0]
        if not isinstance(out_size, int):
            raise ValueError("output_size must be an integer.")
        out_shape = (batch, length, out_size) if self.return_sequences else (batch, out_size)
        if self.return_state:
            return (out_shape, *states_shape)
        return out_shape

    def compute_mask(self, _, mask):
        mask = tree.flatten(mask)[0] if mask is not None else None
        out_mask = mask if self.return_sequences else None
        if self.return_state:
            return [out_mask] + [None for _ in self.state_size]
        return out_mask

    def build(self, sequences_shape, initial_state_shape=None):
        step_shape = (sequences_shape[0],) + tuple(sequences_shape[2:])
        if isinstance(self.cell, Layer) and not self.cell.built:
            self.cell.build(step_shape)
            self.cell.built = True
        if self.stateful:
            if self.states is not None:
                self.reset_state()
            else:
                if sequences_shape[0] is None:
                    raise ValueError(f"When using `stateful=True` in a RNN, the batch size must be static. Found dynamic batch size: sequence.shape={sequences_shape}")
                self._create_state_variables(sequences_shape[0])
                self._expected_batch_size = sequences_shape[0]

    def _create_state_variables(self, batch_size):
        from keras_b200.core.scopes import name_scope
        from keras_b200.core.variables import Variable

        with name_scope(self.name, caller=self):
            states = tree.map_structure(lambda v: Variable(v, trainable=False, dtype=self.variable_dtype, name="rnn_state"),
                                        self.get_initial_state(batch_size))
        object.__setattr__(self, "states", states)

    def get_initial_state(self, batch_size):
        fn = getattr(self.cell, "get_initial_state", None)
        if fn:
            init = fn(batch_size=batch_size)
        else:
            return [ops.zeros((batch_size, d), dtype=self.cell.compute_dtype) for d in self.state_size]
        if not tree.is_nested(init):
            init = [init]
        return list(init)

    def reset_states(self):
        self.reset_state()

    def reset_state(self):
        if self.states is not None:
            for v in tree.flatten(self.states):
                v.assign(ops.zeros_like(v.value))

    def inner_loop(self, sequences, initial_state, mask, training=False):
        kw = {}
        if isinstance(self.cell, Layer) and self.cell._call_has_training_arg:
            kw["training"] = training

        def step(inputs, states):
            if self.stateful:
                states = tree.map_structure(lambda s: s.clone() if isinstance(s, torch.Tensor) else s, list(states))
            out, new_states = self.cell(inputs, list(states), **kw)
            if not tree.is_nested(new_states):
                new_states = [new_states]
            return out, new_states

        if not tree.is_nested(initial_state):
            initial_state = [initial_state]
        return rnn_loop(step, sequences, initial_state, go_backwards=self.go_backwards, mask=mask, unroll=self.unroll,
                        input_length=sequences.shape[1], zero_output_for_mask=self.zero_output_for_mask, return_all_outputs=self.return_sequences)

    def call(self, sequences, initial_state=None, mask=None, training=False):
        if self.unroll and sequences.shape[1] is None:
            raise ValueError("Cannot unroll a RNN if the time dimension is undefined.")
        if initial_state is None:
            if self.stateful:
                initial_state = self.states
            else:
                initial_state = self.get_initial_state(batch_size=ops.shape(sequences)[0])
        if self.stateful and self._expected_batch_size is not None and sequences.shape[0] is not None and sequences.shape[0] != self._expected_batch_size:
            raise ValueError(f"If an RNN is stateful, the batch size of the input sequences must be the same as the batch size of the initial state. \n"
                             f"- Expected batch size: {self._expected_batch_size}\n- Received batch size: {sequences.shape[0]}")
        if not tree.is_nested(initial_state):
            initial_state = [initial_state]
        initial_state = tree.map_structure(lambda x: convert_to_tensor(x, dtype=self.cell.compute_dtype), list(initial_state))
        self._maybe_config_dropout_masks(self.cell, sequences[:, 0], initial_state)
        last, outputs, states = self.inner_loop(sequences=sequences, initial_state=initial_state, mask=mask, training=training)
        last = ops.cast(last, self.compute_dtype)
        outputs = ops.cast(outputs, self.compute_dtype)
        states = tree.map_structure(lambda x: ops.cast(x, dtype=self.compute_dtype), states)
        self._maybe_reset_dropout_masks(self.cell)
        if self.stateful:
            for var, st in zip(tree.flatten(self.states), tree.flatten(states)):
                var.assign(st.detach() if isinstance(st, torch.Tensor) else st)
        out = outputs if self.return_sequences else last
        if self.return_state:
            return (out, *states)
        return out

    def _maybe_config_dropout_masks(self, cell, input_sequence, input_state):
        state = input_state[0] if isinstance(input_state, (list, tuple)) else input_state
        if isinstance(cell, DropoutRNNCell):
            cell.get_dropout_mask(input_sequence)
            cell.get_recurrent_dropout_mask(state)
        if isinstance(cell, StackedRNNCells):
            for c, s in zip(cell.cells, input_state):
                self._maybe_config_dropout_masks(c, input_sequence, s)
                s = list(s) if tree.is_nested(s) else [s]
                fn = c.__call__ if callable(c) else c.call
                input_sequence, _ = fn(input_sequence, s)

    def _maybe_reset_dropout_masks(self, cell):
        if isinstance(cell, DropoutRNNCell):
            cell.reset_dropout_mask()
            cell.reset_recurrent_dropout_mask()
        if isinstance(cell, StackedRNNCells):
            for c in cell.cells:
                self._maybe_reset_dropout_masks(c)

    def get_config(self):
        cfg = {"return_sequences": self.return_sequences, "return_state": self.return_state, "go_backwards": self.go_backwards,
               "stateful": self.stateful, "unroll": self.unroll, "zero_output_for_mask": self.zero_output_for_mask,
               "cell": serialization_lib.serialize_keras_object(self.cell)}
        return {**super().get_config(), **cfg}

    @classmethod
    def from_config(cls, config, custom_objects=None):
        cell = serialization_lib.deserialize_keras_object(config.pop("cell"), custom_objects=custom_objects)
        return cls(cell, **config)


_RNN_KW = ("return_sequences", "return_state", "go_backwards", "stateful", "unroll")


class _CellRNN(RNN):
    """RNN layer that owns exactly one cell and mirrors its hyper-parameters as properties."""

    CELL = None
    _MIRRORED = ("units", "activation", "use_bias", "kernel_initializer", "recurrent_initializer", "bias_initializer", "kernel_regularizer",
                 "recurrent_regularizer", "bias_regularizer", "kernel_constraint", "recurrent_constraint", "bias_constraint", "dropout",
                 "recurrent_dropout")

    def __getattr__(self, name):
        if name in type(self)._MIRRORED and "cell" in self.__dict__:
            return getattr(self.__dict__["cell"], name)
        raise AttributeError(f"'{type(self).__name__}' object has no attribute '{name}'")

    def _cell_config(self):
        cfg = self.cell._base_config()
        return cfg

    def get_config(self):
        base = super().get_config()
        del base["cell"]
        cfg = {**self._cell_config(), **base, "activity_regularizer": regularizers.serialize(self.activity_regularizer)}
        cfg.pop("zero_output_for_mask", None)
        return cfg

    @classmethod
    def from_config(cls, config):
        return cls(**config)

    def _hoisted(self, sequences, initial_state, mask, training):
        return None

    def inner_loop(self, sequences, initial_state, mask, training=False):
        out = self._hoisted(sequences, initial_state, mask, training)
        if out is not None:
            return out
        return super().inner_loop(sequences, initial_state, mask, training=training)


@keras_export("keras.layers.SimpleRNN")
class SimpleRNN(_CellRNN):
    def __init__(self, units, activation="tanh", use_bias=True, kernel_initializer="glorot_uniform", recurrent_initializer="orthogonal",
                 bias_initializer="zeros", kernel_regularizer=None, recurrent_regularizer=None, bias_regularizer=None, activity_regularizer=None,
                 kernel_constraint=None, recurrent_constraint=None, bias_constraint=None, dropout=0.0, recurrent_dropout=0.0,
                 return_sequences=False, return_state=False, go_backwards=False, stateful=False, unroll=False, seed=None, **kwargs):
        cell = SimpleRNNCell(units, activation=activation, use_bias=use_bias, kernel_initializer=kernel_initializer,
                             recurrent_initializer=recurrent_initializer, bias_initializer=bias_initializer, kernel_regularizer=kernel_regularizer,
                             recurrent_regularizer=recurrent_regularizer, bias_regularizer=bias_regularizer, kernel_constraint=kernel_constraint,
                             recurrent_constraint=recurrent_constraint, bias_constraint=bias_constraint, dropout=dropout,
                             recurrent_dropout=recurrent_dropout, seed=seed, dtype=kwargs.get("dtype", None), trainable=kwargs.get("trainable", True),
                             name="simple_rnn_cell")
        super().__init__(cell, return_sequences=return_sequences, return_state=return_state, go_backwards=go_backwards, stateful=stateful,
                         unroll=unroll, activity_regularizer=activity_regularizer, **kwargs)
        self.input_spec = [InputSpec(ndim=3)]

    def call(self, sequences, initial_state=None, mask=None, training=False):
        return super().call(sequences, mask=mask, training=training, initial_state=initial_state)


def _time_major_projection(cell, sequences, bias):
    """``x @ kernel + bias`` for all time steps at once, returned time-major ``[T, B, gates]``."""
    k = cell.kernel
    xz = ops.matmul(sequences, k)
    if bias is not None:
        xz = xz + bias
    return xz.transpose(0, 1)


@keras_export("keras.layers.LSTM")
class LSTM(_CellRNN):
    _MIRRORED = _CellRNN._MIRRORED + ("recurrent_activation", "unit_forget_bias")

    def __init__(self, units, activation="tanh", recurrent_activation="sigmoid", use_bias=True, kernel_initializer="glorot_uniform",
                 recurrent_initializer="orthogonal", bias_initializer="zeros", unit_forget_bias=True, kernel_regularizer=None,
                 recurrent_regularizer=None, bias_regularizer=None, activity_regularizer=None, kernel_constraint=None, recurrent_constraint=None,
                 bias_constraint=None, dropout=0.0, recurrent_dropout=0.0, seed=None, return_sequences=False, return_state=False,
                 go_backwards=False, stateful=False, unroll=False, use_cudnn="auto", **kwargs):
        cell = LSTMCell(units, activation=activation, recurrent_activation=recurrent_activation, use_bias=use_bias,
                        kernel_initializer=kernel_initializer, unit_forget_bias=unit_forget_bias, recurrent_initializer=recurrent_initializer,
                        bias_initializer=bias_initializer, kernel_regularizer=kernel_regularizer, recurrent_regularizer=recurrent_regularizer,
                        bias_regularizer=bias_regularizer, kernel_constraint=kernel_constraint, recurrent_constraint=recurrent_constraint,
                        bias_constraint=bias_constraint, dropout=dropout, recurrent_dropout=recurrent_dropout,
                        dtype=kwargs.get("dtype", None), trainable=kwargs.get("trainable", True), name="lstm_cell", seed=seed,
                        implementation=kwargs.pop("implementation", 2))
        super().__init__(cell, return_sequences=return_sequences, return_state=return_state, go_backwards=go_backwards, stateful=stateful,
                         unroll=unroll, activity_regularizer=activity_regularizer, **kwargs)
        self.input_spec = InputSpec(ndim=3)
        if use_cudnn not in ("auto", True, False):
            raise ValueError(f"Invalid valid received for argument `use_cudnn`. Expected one of {{'auto', True, False}}. Received: use_cudnn={use_cudnn}")
        self.use_cudnn = use_cudnn

    def _hoisted(self, sequences, initial_state, mask, training):
        cell = self.cell
        if mask is not None or (training and (cell.dropout > 0 or cell.recurrent_dropout > 0)) or not isinstance(sequences, torch.Tensor):
            return None
        xz = _time_major_projection(cell, sequences, cell.bias.value if cell.bias is not None else None)
        h, c = initial_state[0], initial_state[1]
        rk = cell.recurrent_kernel.value
        steps = range(xz.shape[0] - 1, -1, -1) if self.go_backwards else range(xz.shape[0])
        outs = []
        for t in steps:
            h, c = cell.gates(xz[t] + torch.matmul(h, rk), c)
            if self.return_sequences:
                outs.append(h)
        outputs = torch.stack(outs, dim=1) if self.return_sequences else h.unsqueeze(1)
        return h, outputs, [h, c]

    def call(self, sequences, initial_state=None, mask=None, training=False):
        return super().call(sequences, mask=mask, training=training, initial_state=initial_state)

    def _cell_config(self):
        cfg = self.cell._base_config()
        cfg.update({"recurrent_activation": activations.serialize(self.cell.recurrent_activation), "unit_forget_bias": self.cell.unit_forget_bias})
        return cfg


@keras_export("keras.layers.GRU")
class GRU(_CellRNN):
    _MIRRORED = _CellRNN._MIRRORED + ("recurrent_activation", "reset_after")

    def __init__(self, units, activation="tanh", recurrent_activation="sigmoid", use_bias=True, kernel_initializer="glorot_uniform",
                 recurrent_initializer="orthogonal", bias_initializer="zeros", kernel_regularizer=None, recurrent_regularizer=None,
                 bias_regularizer=None, activity_regularizer=None, kernel_constraint=None, recurrent_constraint=None, bias_constraint=None,
                 dropout=0.0, recurrent_dropout=0.0, seed=None, return_sequences=False, return_state=False, go_backwards=False, stateful=False,
                 unroll=False, reset_after=True, use_cudnn="auto", **kwargs):
        cell = GRUCell(units, activation=activation, recurrent_activation=recurrent_activation, use_bias=use_bias,
                       kernel_initializer=kernel_initializer, recurrent_initializer=recurrent_initializer, bias_initializer=bias_initializer,
                       kernel_regularizer=kernel_regularizer, recurrent_regularizer=recurrent_regularizer, bias_regularizer=bias_regularizer,
                       kernel_constraint=kernel_constraint, recurrent_constraint=recurrent_constraint, bias_constraint=bias_constraint,
                       dropout=dropout, recurrent_dropout=recurrent_dropout, reset_after=reset_after, dtype=kwargs.get("dtype", None),
                       trainable=kwargs.get("trainable", True), name="gru_cell", seed=seed, implementation=kwargs.pop("implementation", 2))
        super().__init__(cell, return_sequences=return_sequences, return_state=return_state, go_backwards=go_backwards, stateful=stateful,
                         unroll=unroll, activity_regularizer=activity_regularizer, **kwargs)
        self.input_spec = InputSpec(ndim=3)
        if use_cudnn not in ("auto", True, False):
            raise ValueError(f"Invalid valid received for argument `use_cudnn`. Expected one of {{'auto', True, False}}. Received: use_cudnn={use_cudnn}")
        self.use_cudnn = use_cudnn

    def _hoisted(self, sequences, initial_state, mask, training):
        cell = self.cell
        if mask is not None or (training and (cell.dropout > 0 or cell.recurrent_dropout > 0)) or not isinstance(sequences, torch.Tensor):
            return None
        ib, rb = cell._split_bias()
        xz = _time_major_projection(cell, sequences, ib)
        h = initial_state[0]
        steps = range(xz.shape[0] - 1, -1, -1) if self.go_backwards else range(xz.shape[0])
        outs = []
        for t in steps:
            h = cell.step_from_projection(xz[t], h, rb)
            if self.return_sequences:
                outs.append(h)
        outputs = torch.stack(outs, dim=1) if self.return_sequences else h.unsqueeze(1)
        return h, outputs, [h]

    def call(self, sequences, initial_state=None, mask=None, training=False):
        return super().call(sequences, mask=mask, training=training, initial_state=initial_state)

    def _cell_config(self):
        cfg = self.cell._base_config()
        cfg.update({"recurrent_activation": activations.serialize(self.cell.recurrent_activation), "reset_after": self.cell.reset_after})
        return cfg


@keras_export("keras.layers.Bidirectional")
class Bidirectional(Layer):
    def __init__(self, layer, merge_mode="concat", weights=None, backward_layer=None, **kwargs):
        if not isinstance(layer, Layer):
            raise ValueError(f"Please initialize `Bidirectional` layer with a `keras.layers.Layer` instance. Received: {layer}")
        if backward_layer is not None and not isinstance(backward_layer, Layer):
            raise ValueError(f"`backward_layer` need to be a `keras.layers.Layer` instance. Received: {backward_layer}")
        if merge_mode not in ["sum", "mul", "ave", "concat", None]:
            raise ValueError(f'Invalid merge mode. Received: {merge_mode}. Merge mode should be one of {{"sum", "mul", "ave", "concat", None}}')
        super().__init__(**kwargs)

        def strip(name, prefix):
            return name[len(prefix):] if name.startswith(prefix) else name

        cfg = serialization_lib.serialize_keras_object(layer)
        cfg["config"]["name"] = "forward_" + strip(layer.name, "forward_")
        self.forward_layer = serialization_lib.deserialize_keras_object(cfg)
        if backward_layer is None:
            cfg = serialization_lib.serialize_keras_object(layer)
            cfg["config"]["go_backwards"] = True
            cfg["config"]["name"] = "backward_" + strip(layer.name, "backward_")
            self.backward_layer = serialization_lib.deserialize_keras_object(cfg)
        else:
            self.backward_layer = backward_layer
        self._verify_layer_config()
        for lyr in (self.forward_layer, self.backward_layer):
            if getattr(lyr, "zero_output_for_mask", None) is not None:
                lyr.zero_output_for_mask = lyr.return_sequences
        self.merge_mode = merge_mode
        if weights:
            nw = len(weights)
            self.forward_layer.initial_weights = weights[: nw // 2]
            self.backward_layer.initial_weights = weights[nw // 2:]
        self.stateful = layer.stateful
        self.return_sequences = layer.return_sequences
        self.return_state = layer.return_state
        # The mask reaches both directions through the ``mask`` argument, but the merged output carries none
        # (keras/src/layers/rnn/bidirectional.py:153).
        self.supports_masking = False
        self.input_spec = layer.input_spec

    def _verify_layer_config(self):
        if self.forward_layer.go_backwards == self.backward_layer.go_backwards:
            raise ValueError("Forward layer and backward layer should have different `go_backwards` value. Received: forward_layer.go_backwards "
                             f"{self.forward_layer.go_backwards}, backward_layer.go_backwards={self.backward_layer.go_backwards}")
        for a in ("stateful", "return_sequences", "return_state"):
            fv, bv = getattr(self.forward_layer, a), getattr(self.backward_layer, a)
            if fv != bv:
                raise ValueError(f'Forward layer and backward layer are expected to have the same value for attribute "{a}", got "{fv}" for forward layer and "{bv}" for backward layer')

    def compute_output_shape(self, sequences_shape, initial_state_shape=None):
        out = self.forward_layer.compute_output_shape(sequences_shape)
        state_shape = ()
        if self.return_state:
            out, state_shape = out[0], tuple(out[1:])
        if self.merge_mode == "concat":
            out = list(out)
            out[-1] *= 2
            out = tuple(out)
        elif self.merge_mode is None:
            out = [out, out]
        if self.return_state:
            if self.merge_mode is None:
                return tuple(out) + state_shape + state_shape
            return (out,) + state_shape + state_shape
        return tuple(out)

    def call(self, sequences, initial_state=None, mask=None, training=None):
        kw = {}
        if self.forward_layer._call_has_training_arg:
            kw["training"] = training
        if self.forward_layer._plan.has_mask:
            kw["mask"] = mask
        fs = bs = None
        if initial_state is not None:
            half = len(initial_state) // 2
            fs, bs = initial_state[:half], initial_state[half:]
        y = self.forward_layer(sequences, initial_state=fs, **kw)
        y_rev = self.backward_layer(sequences, initial_state=bs, **kw)
        states = ()
        if self.return_state:
            states = tuple(y[1:]) + tuple(y_rev[1:])
            y, y_rev = y[0], y_rev[0]
        y = ops.cast(y, self.compute_dtype)
        y_rev = ops.cast(y_rev, self.compute_dtype)
        if self.return_sequences:
            y_rev = ops.flip(y_rev, axis=1)
        if self.merge_mode == "concat":
            out = ops.concatenate([y, y_rev], axis=-1)
        elif self.merge_mode == "sum":
            out = y + y_rev
        elif self.merge_mode == "ave":
            out = (y + y_rev) / 2
        elif self.merge_mode == "mul":
            out = y * y_rev
        elif self.merge_mode is None:
            out = (y, y_rev)
        else:
            raise ValueError(f"Unrecognized value for `merge_mode`. Received: {self.merge_mode}")
        if self.return_state:
            if self.merge_mode is None:
                return out + states
            return (out,) + states
        return out

    def reset_states(self):
        self.reset_state()

    def reset_state(self):
        if not self.stateful:
            raise AttributeError("Layer must be stateful.")
        self.forward_layer.reset_state()
        self.backward_layer.reset_state()

    @property
    def states(self):
        if self.forward_layer.states and self.backward_layer.states:
            return tuple(self.forward_layer.states + self.backward_layer.states)
        return None

    def build(self, sequences_shape, initial_state_shape=None):
        if not self.forward_layer.built:
            self.forward_layer.build(sequences_shape)
        if not self.backward_layer.built:
            self.backward_layer.build(sequences_shape)

    def compute_mask(self, _, mask):
        if isinstance(mask, list):
            mask = mask[0]
        out_mask = mask if self.return_sequences else None
        if self.merge_mode is None:
            out_mask = (out_mask, out_mask)
        if self.return_state and self.states is not None:
            state_mask = tuple(None for _ in self.states)
            if isinstance(out_mask, tuple):
                return out_mask + state_mask * 2
            return (out_mask,) + state_mask * 2
        return out_mask

    def get_config(self):
        cfg = {"merge_mode": self.merge_mode, "layer": serialization_lib.serialize_keras_object(self.forward_layer),
               "backward_layer": serialization_lib.serialize_keras_object(self.backward_layer)}
        return {**super().get_config(), **cfg}

    @classmethod
    def from_config(cls, config, custom_objects=None):
        import copy

        config = copy.deepcopy(config)
        config["layer"] = serialization_lib.deserialize_keras_object(config["layer"], custom_objects=custom_objects)
        bl = config.pop("backward_layer", None)
        if bl is not None:
            config["backward_layer"] = serialization_lib.deserialize_keras_object(bl, custom_objects=custom_objects)
        return cls(**config)


@keras_export("keras.layers.TimeDistributed")
class TimeDistributed(Layer):
    """Apply ``layer`` to every temporal slice: ``[B, T, ...]`` is folded to ``[B*T, ...]`` for one call."""

    def __init__(self, layer, **kwargs):
        if not isinstance(layer, Layer):
            raise ValueError(f"Please initialize `TimeDistributed` layer with a `keras.layers.Layer` instance. Received: {layer}")
        super().__init__(**kwargs)
        self.layer = layer
        self.supports_masking = False  # keras/src/layers/rnn/time_distributed.py:54: the output carries no mask

    def _child_shape(self, input_shape):
        if not isinstance(input_shape, (tuple, list)) or len(input_shape) < 3:
            raise ValueError(f"`TimeDistributed` Layer should be passed an `input_shape` with at least 3 dimensions, received: {input_shape}")
        return (input_shape[0], *input_shape[2:])

    def compute_output_shape(self, input_shape):
        child = self.layer.compute_output_shape(self._child_shape(input_shape))
        return (child[0], input_shape[1], *child[1:])

    def build(self, input_shape):
        if not self.layer.built:
            self.layer.build(self._child_shape(input_shape))
            self.layer.built = True

    def call(self, inputs, training=None, mask=None):
        shape = ops.shape(inputs)
        b, t = shape[0], shape[1]
        kw = {}
        if self.layer._call_has_training_arg:
            kw["training"] = training
        if mask is not None and self.layer._plan.has_mask:
            kw["mask"] = ops.reshape(mask, (-1,) + tuple(ops.shape(mask)[2:]))
        flat = ops.reshape(inputs, (-1,) + tuple(shape[2:]))
        out = self.layer(flat, **kw)
        return tree.map_structure(lambda o: ops.reshape(o, (b, t) + tuple(ops.shape(o)[1:])), out)

    def get_config(self):
        return {**super().get_config(), "layer": serialization_lib.serialize_keras_object(self.layer)}

    @classmethod
    def from_config(cls, config, custom_objects=None):
        layer = serialization_lib.deserialize_keras_object(config.pop("layer"), custom_objects=custom_objects)
        return cls(layer, **config)


# ------------------------------------------------------------------------------------- ConvLSTM
class ConvLSTMCell(Layer, DropoutRNNCell):
    def __init__(self, rank, filters, kernel_size, strides=1, padding="valid", data_format=None, dilation_rate=1, activation="tanh",
                 recurrent_activation="sigmoid", use_bias=True, kernel_initializer="glorot_uniform", recurrent_initializer="orthogonal",
                 bias_initializer="zeros", unit_forget_bias=True, kernel_regularizer=None, recurrent_regularizer=None, bias_regularizer=None,
                 kernel_constraint=None, recurrent_constraint=None, bias_constraint=None, dropout=0.0, recurrent_dropout=0.0, seed=None, **kwargs):
        super().__init__(**kwargs)
        from keras_b200.core import config as _config
        from keras_b200.random.seed_generator import SeedGenerator

        def tup(v, name):
            if isinstance(v, int):
                return (v,) * rank
            v = tuple(v)
            if len(v) != rank:
                raise ValueError(f"The `{name}` argument must be a tuple of {rank} integers. Received: {v}")
            return v

        self.seed = seed
        self.seed_generator = SeedGenerator(seed=seed)
        self.rank, self.filters = rank, filters
        self.kernel_size = tup(kernel_size, "kernel_size")
        self.strides = tup(strides, "strides")
        self.padding = padding.lower()
        self.data_format = _config.standardize_data_format(data_format)
        self.dilation_rate = tup(dilation_rate, "dilation_rate")
        self.activation = activations.get(activation)
        self.recurrent_activation = activations.get(recurrent_activation)
        self.use_bias = use_bias
        self.kernel_initializer = initializers.get(kernel_initializer)
        self.recurrent_initializer = initializers.get(recurrent_initializer)
        self.bias_initializer = initializers.get(bias_initializer)
        self.unit_forget_bias = unit_forget_bias
        self.kernel_regularizer = regularizers.get(kernel_regularizer)
        self.recurrent_regularizer = regularizers.get(recurrent_regularizer)
        self.bias_regularizer = regularizers.get(bias_regularizer)
        self.kernel_constraint = constraints.get(kernel_constraint)
        self.recurrent_constraint = constraints.get(recurrent_constraint)
        self.bias_constraint = constraints.get(bias_constraint)
        self.dropout_mask_count = 4
        self.dropout = min(1.0, max(0.0, dropout))
        self.recurrent_dropout = min(1.0, max(0.0, recurrent_dropout))
        self.input_spec = InputSpec(ndim=rank + 2)
        self.state_size = -1  # resolved in build

    def build(self, inputs_shape, states_shape=None):
        if self.data_format == "channels_first":
            channel_axis = 1
            self.spatial_dims = tuple(inputs_shape[2:])
        else:
            channel_axis = -1
            self.spatial_dims = tuple(inputs_shape[1:-1])
        if None in self.spatial_dims:
            raise ValueError(f"ConvLSTM layers only support static input shapes for the spatial dimension. Received invalid input shape: input_shape={inputs_shape}")
        if inputs_shape[channel_axis] is None:
            raise ValueError(f"The channel dimension of the inputs (last axis) should be defined. Found None. Full input shape received: input_shape={inputs_shape}")
        self.input_spec = InputSpec(ndim=self.rank + 3, shape=(None,) + tuple(inputs_shape[1:]))
        in_dim = inputs_shape[channel_axis]
        self.kernel_shape = self.kernel_size + (in_dim, self.filters * 4)
        rk_shape = self.kernel_size + (self.filters, self.filters * 4)
        self.kernel = self.add_weight(shape=self.kernel_shape, initializer=self.kernel_initializer, name="kernel", regularizer=self.kernel_regularizer,
                                      constraint=self.kernel_constraint)
        self.recurrent_kernel = self.add_weight(shape=rk_shape, initializer=self.recurrent_initializer, name="recurrent_kernel",
                                                regularizer=self.recurrent_regularizer, constraint=self.recurrent_constraint)
        if self.use_bias:
            if self.unit_forget_bias:
                f, base = self.filters, self.bias_initializer

                def bias_init(_, *args, **kw):
                    return ops.concatenate([base((f,), *args, **kw), initializers.get("ones")((f,), *args, **kw), base((f * 2,), *args, **kw)])
            else:
                bias_init = self.bias_initializer
            self.bias = self.add_weight(shape=(self.filters * 4,), name="bias", initializer=bias_init, regularizer=self.bias_regularizer,
                                        constraint=self.bias_constraint)
        else:
            self.bias = None

    def call(self, inputs, states, training=False):
        h_prev, c_prev = states[0], states[1]
        dp = self.get_dropout_mask(inputs) if training and 0.0 < self.dropout < 1.0 else None
        rdp = self.get_recurrent_dropout_mask(h_prev) if training and 0.0 < self.recurrent_dropout < 1.0 else None
        caxis = -1 if self.data_format == "channels_last" else 1

        def gate_conv(x, masks, kernel, **kw):
            # one mask per gate (keras/src/layers/rnn/conv_lstm.py:244-266): gate g convolves x * masks[g] with its block of filters
            if masks is None:
                return ops.conv(x, kernel, **kw)
            k = kernel.value if hasattr(kernel, "value") else kernel
            f = self.filters
            return ops.concatenate([ops.conv(x * masks[g], k[..., g * f:(g + 1) * f], **kw) for g in range(4)], axis=caxis)

        x = gate_conv(inputs, dp, self.kernel, strides=self.strides, padding=self.padding, data_format=self.data_format, dilation_rate=self.dilation_rate)
        if self.bias is not None:
            shape = (1,) * (self.rank + 1) + (self.filters * 4,) if self.data_format == "channels_last" else (1, self.filters * 4) + (1,) * self.rank
            x = x + ops.reshape(self.bias, shape)
        hc = gate_conv(h_prev, rdp, self.recurrent_kernel, strides=1, padding="same", data_format=self.data_format)
        z = x + hc
        zi, zf, zc, zo = ops.split(z, 4, axis=caxis)
        i = self.recurrent_activation(zi)
        f = self.recurrent_activation(zf)
        c = f * c_prev + i * self.activation(zc)
        o = self.recurrent_activation(zo)
        h = o * self.activation(c)
        return h, [h, c]

    def compute_output_shape(self, inputs_shape, states_shape=None):
        from keras_b200.ops.operation_utils import compute_conv_output_shape

        out = compute_conv_output_shape(inputs_shape, self.filters, self.kernel_size, strides=self.strides, padding=self.padding,
                                        data_format=self.data_format, dilation_rate=self.dilation_rate)
        return out, [out, out]

    def get_initial_state(self, batch_size=None):
        if self.data_format == "channels_last":
            in_shape = (batch_size,) + self.spatial_dims + (self.kernel_shape[-2],)
        else:
            in_shape = (batch_size, self.kernel_shape[-2]) + self.spatial_dims
        state_shape = self.compute_output_shape(in_shape)[0]
        return [ops.zeros(state_shape, dtype=self.compute_dtype), ops.zeros(state_shape, dtype=self.compute_dtype)]

    def get_config(self):
        cfg = {
            "filters": self.filters, "kernel_size": self.kernel_size, "strides": self.strides, "padding": self.padding,
            "data_format": self.data_format, "dilation_rate": self.dilation_rate, "activation": activations.serialize(self.activation),
            "recurrent_activation": activations.serialize(self.recurrent_activation), "use_bias": self.use_bias,
            "kernel_initializer": initializers.serialize(self.kernel_initializer),
            "recurrent_initializer": initializers.serialize(self.recurrent_initializer),
            "bias_initializer": initializers.serialize(self.bias_initializer), "unit_forget_bias": self.unit_forget_bias,
            "kernel_regularizer": regularizers.serialize(self.kernel_regularizer),
            "recurrent_regularizer": regularizers.serialize(self.recurrent_regularizer),
            "bias_regularizer": regularizers.serialize(self.bias_regularizer),
            "kernel_constraint": constraints.serialize(self.kernel_constraint),
            "recurrent_constraint": constraints.serialize(self.recurrent_constraint),
            "bias_constraint": constraints.serialize(self.bias_constraint),
            "dropout": self.dropout, "recurrent_dropout": self.recurrent_dropout, "seed": self.seed,
        }
        return {**super().get_config(), **cfg}


class ConvLSTM(RNN):
    def __init__(self, rank, filters, kernel_size, strides=1, padding="valid", data_format=None, dilation_rate=1, activation="tanh",
                 recurrent_activation="sigmoid", use_bias=True, kernel_initializer="glorot_uniform", recurrent_initializer="orthogonal",
                 bias_initializer="zeros", unit_forget_bias=True, kernel_regularizer=None, recurrent_regularizer=None, bias_regularizer=None,
                 kernel_constraint=None, recurrent_constraint=None, bias_constraint=None, dropout=0.0, recurrent_dropout=0.0, seed=None,
                 return_sequences=False, return_state=False, go_backwards=False, stateful=False, **kwargs):
        cell = ConvLSTMCell(rank=rank, filters=filters, kernel_size=kernel_size, strides=strides, padding=padding, data_format=data_format,
                            dilation_rate=dilation_rate, activation=activation, recurrent_activation=recurrent_activation, use_bias=use_bias,
                            kernel_initializer=kernel_initializer, recurrent_initializer=recurrent_initializer, bias_initializer=bias_initializer,
                            unit_forget_bias=unit_forget_bias, kernel_regularizer=kernel_regularizer, recurrent_regularizer=recurrent_regularizer,
                            bias_regularizer=bias_regularizer, kernel_constraint=kernel_constraint, recurrent_constraint=recurrent_constraint,
                            bias_constraint=bias_constraint, dropout=dropout, recurrent_dropout=recurrent_dropout, seed=seed, name="conv_lstm_cell",
                            dtype=kwargs.get("dtype"))
        super().__init__(cell, return_sequences=return_sequences, return_state=return_state, go_backwards=go_backwards, stateful=stateful, **kwargs)
        self.input_spec = InputSpec(ndim=rank + 3)

    def call(self, sequences, initial_state=None, mask=None, training=False):
        return super().call(sequences, initial_state=initial_state, mask=mask, training=training)

    def compute_output_shape(self, sequences_shape, initial_state_shape=None):
        batch, steps = sequences_shape[0], sequences_shape[1]
        step_shape = (batch,) + tuple(sequences_shape[2:])
        state_shape = self.cell.compute_output_shape(step_shape)[0][1:]
        if self.return_sequences:
            out = (batch, steps) + tuple(state_shape)
        else:
            out = (batch,) + tuple(state_shape)
        if self.return_state:
            batched = (batch,) + tuple(state_shape)
            return out, batched, batched
        return out

    def compute_mask(self, _, mask):
        mask = tree.flatten(mask)[0] if mask is not None else None
        out_mask = mask if self.return_sequences else None
        if self.return_state:
            return [out_mask, None, None]
        return out_mask

    def __getattr__(self, name):
        if name in ("filters", "kernel_size", "strides", "padding", "data_format", "dilation_rate", "activation", "recurrent_activation", "use_bias",
                    "kernel_initializer", "recurrent_initializer", "bias_initializer", "unit_forget_bias", "kernel_regularizer",
                    "recurrent_regularizer", "bias_regularizer", "kernel_constraint", "recurrent_constraint", "bias_constraint", "dropout",
                    "recurrent_dropout") and "cell" in self.__dict__:
            return getattr(self.__dict__["cell"], name)
        raise AttributeError(f"'{type(self).__name__}' object has no attribute '{name}'")

    def get_config(self):
        base = super().get_config()
        cell_cfg = self.cell.get_config()
        for k in ("name", "trainable", "dtype"):
            cell_cfg.pop(k, None)
        del base["cell"]
        base.pop("unroll", None)
        base.pop("zero_output_for_mask", None)
        cfg = {**cell_cfg, **base, "activity_regularizer": regularizers.serialize(self.activity_regularizer)}
        return cfg

    @classmethod
    def from_config(cls, config):
        return cls(**config)


def _make_conv_lstm(name, rank):
    def __init__(self, filters, kernel_size, strides=1, padding="valid", data_format=None, dilation_rate=1, activation="tanh",
                 recurrent_activation="sigmoid", use_bias=True, kernel_initializer="glorot_uniform", recurrent_initializer="orthogonal",
                 bias_initializer="zeros", unit_forget_bias=True, kernel_regularizer=None, recurrent_regularizer=None, bias_regularizer=None,
                 activity_regularizer=None, kernel_constraint=None, recurrent_constraint=None, bias_constraint=None, dropout=0.0,
                 recurrent_dropout=0.0, seed=None, return_sequences=False, return_state=False, go_backwards=False, stateful=False, **kwargs):
        ConvLSTM.__init__(self, rank, filters, kernel_size, strides=strides, padding=padding, data_format=data_format, dilation_rate=dilation_rate,
                          activation=activation, recurrent_activation=recurrent_activation, use_bias=use_bias,
                          kernel_initializer=kernel_initializer, recurrent_initializer=recurrent_initializer, bias_initializer=bias_initializer,
                          unit_forget_bias=unit_forget_bias, kernel_regularizer=kernel_regularizer, recurrent_regularizer=recurrent_regularizer,
                          bias_regularizer=bias_regularizer, activity_regularizer=activity_regularizer, kernel_constraint=kernel_constraint,
                          recurrent_constraint=recurrent_constraint, bias_constraint=bias_constraint, return_sequences=return_sequences,
                          return_state=return_state, go_backwards=go_backwards, stateful=stateful, dropout=dropout,
                          recurrent_dropout=recurrent_dropout, seed=seed, **kwargs)

    cls = type(name, (ConvLSTM,), {"__init__": __init__})
    cls.__module__ = __name__
    return keras_export(f"keras.layers.{name}")(cls)


ConvLSTM1D = _make_conv_lstm("ConvLSTM1D", 1)
ConvLSTM2D = _make_conv_lstm("ConvLSTM2D", 2)
ConvLSTM3D = _make_conv_lstm("ConvLSTM3D", 3)
