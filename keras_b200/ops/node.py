"""Graph edges: ``Node`` records one call of an operation on symbolic tensors.

Semantics of keras/src/ops/node.py:8-143 and symbolic_arguments.py; the argument container
additionally pre-computes a *fill plan* so that replaying a node does not walk nested
structures again.
"""

import collections

from keras_b200 import tree
from keras_b200.core.keras_tensor import KerasTensor

KerasHistory = collections.namedtuple("KerasHistory", ["operation", "node_index", "tensor_index"])


class SymbolicArguments:
    def __init__(self, *args, **kwargs):
        self.args = tree.map_structure(lambda x: x, args)
        self.kwargs = tree.map_structure(lambda x: x, kwargs)
        self._flat = tree.flatten((self.args, self.kwargs))
        self.keras_tensors = [x for x in self._flat if isinstance(x, KerasTensor)]
        self._slots = [i for i, x in enumerate(self._flat) if isinstance(x, KerasTensor)]
        # Fast path: one positional KerasTensor and nothing nested around it.
        self._single = (
            len(self.args) >= 1
            and isinstance(self.args[0], KerasTensor)
            and len(self.keras_tensors) == 1
        )

    def convert(self, conversion_fn):
        return tree.map_structure(
            lambda x: conversion_fn(x) if isinstance(x, KerasTensor) else x, (self.args, self.kwargs)
        )

    def fill_in(self, tensor_dict):
        """Replace each KerasTensor by ``tensor_dict[id(kt)]`` (left as is when absent)."""
        if self._single:
            v = tensor_dict.get(id(self.args[0]), None)
            return (v,) + tuple(self.args[1:]), self.kwargs
        flat = list(self._flat)
        for i in self._slots:
            v = tensor_dict.get(id(flat[i]), None)
            flat[i] = v
        return tree.pack_sequence_as((self.args, self.kwargs), flat)


class Node:
    def __init__(self, operation, call_args=None, call_kwargs=None, outputs=None):
        self.operation = operation
        self.arguments = SymbolicArguments(*(call_args or ()), **(call_kwargs or {}))
        self.outputs = [] if outputs is None else tree.flatten(outputs)
        for x in self.outputs:
            if not isinstance(x, KerasTensor):
                raise ValueError(
                    "All operation outputs must be tensors. "
                    f"Operation {operation} returned a non-tensor. Non-tensor received: {x}"
                )
        inputs = self.arguments.keras_tensors
        untracked = any(not t.record_history for t in inputs)
        if not untracked:
            for t in inputs:
                if not hasattr(t, "_keras_history"):
                    t._keras_history = KerasHistory(None, 0, 0)
        operation._inbound_nodes.append(self)
        for t in inputs:
            hist = getattr(t, "_keras_history", None)
            if hist is not None and hist.operation is not None:
                hist.operation._outbound_nodes.append(self)
        if not untracked:
            index = len(operation._inbound_nodes) - 1
            for i, t in enumerate(self.outputs):
                t._keras_history = KerasHistory(operation, index, i)
        self.is_input = not inputs

    def __repr__(self):
        return f"<Node operation={self.operation.name}, id={id(self)}>"

    @property
    def input_tensors(self):
        return self.arguments.keras_tensors

    @property
    def output_tensors(self):
        return self.outputs

    @property
    def parent_nodes(self):
        out = []
        for t in self.arguments.keras_tensors:
            hist = t._keras_history
            if hist.operation is not None:
                out.append(hist.operation._inbound_nodes[hist.node_index])
        return out


def is_keras_tensor(obj):
    return hasattr(obj, "_keras_history")
