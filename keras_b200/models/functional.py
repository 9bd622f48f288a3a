"""``Functional``: a ``Model`` defined by a DAG of layers between ``Input`` tensors and outputs.

Behaviour of keras/src/models/functional.py:27-940: input standardisation (:256-373), config
schema with ``inbound_nodes`` as serialised ``args``/``kwargs`` (:430-504), two-pass node replay
on load (:507-687).
"""

import copy
import inspect
import warnings

import torch

from keras_b200 import ops, tree
from keras_b200.core.dtypes import standardize_dtype
from keras_b200.core.keras_tensor import KerasTensor
from keras_b200.layers.core.input_layer import Input, InputLayer
from keras_b200.layers.input_spec import InputSpec
from keras_b200.layers.layer import Layer
from keras_b200.models.model import Model
from keras_b200.ops.function import Function, make_node_key
from keras_b200.ops.node import KerasHistory, Node
from keras_b200.ops.operation import Operation


class Functional(Function, Model):
    def __new__(cls, *args, **kwargs):
        return Model.__new__(cls)

    def __init__(self, inputs, outputs, name=None, **kwargs):
        if isinstance(inputs, dict):
            for k, v in inputs.items():
                if isinstance(v, KerasTensor) and k != v.name:
                    warnings.warn(
                        "When providing `inputs` as a dict, all keys in the dict must match the names of the "
                        f"corresponding tensors. Received key '{k}' mapping to value {v} which has name '{v.name}'. "
                        "Change the tensor name to '{k}' (via `Input(..., name='{k}')`)"
                    )
        trainable = kwargs.pop("trainable", None)
        flat_inputs = tree.flatten(inputs)
        flat_outputs = tree.flatten(outputs)
        for x in flat_inputs:
            if not isinstance(x, KerasTensor):
                raise ValueError(f"All `inputs` values must be KerasTensors. Received: inputs={inputs} including invalid value {x} of type {type(x)}")
        for x in flat_outputs:
            if not isinstance(x, KerasTensor):
                raise ValueError(f"All `outputs` values must be KerasTensors. Received: outputs={outputs} including invalid value {x} of type {type(x)}")
        if not all(is_input_keras_tensor(t) for t in flat_inputs):
            inputs, outputs = clone_graph_nodes(inputs, outputs)
        if "_compute_loss_has_training_arg" not in self.__dict__:
            from keras_b200.trainers.trainer import Trainer

            Trainer.__init__(self)
        Layer.__init__(self, name=name, **kwargs)
        Function.__init__(self, inputs, outputs, name=self.name)
        if trainable is not None:
            self.trainable = trainable
        self._layers = self.layers
        self.build(None)
        self._convert_input_args = False
        self._allow_non_tensor_positional_args = True
        output_layers = [x._keras_history[0] for x in self.outputs]
        self.output_names = [x.name for x in output_layers]
        self._init_trainer_state()

    def _lock_state(self):
        pass

    def _obj_type(self):
        return "Functional"

    @property
    def layers(self):
        return [op for op in self._operations if isinstance(op, Layer)]

    @layers.setter
    def layers(self, _):
        raise AttributeError("`Model.layers` attribute is reserved and should not be used. Please use another name.")

    def call(self, inputs, training=None, mask=None, **kwargs):
        inputs = self._standardize_inputs(inputs)
        if mask is None:
            masks = [None] * len(inputs)
        else:
            masks = tree.flatten(mask)
            for x, m in zip(inputs, masks):
                if m is not None:
                    try:
                        x._keras_mask = m
                    except AttributeError:
                        pass
        fusion = None
        if inputs and isinstance(inputs[0], torch.Tensor) and inputs[0].is_cuda:
            from keras_b200.core import config as _config

            if _config.fused_kernels_enabled():
                from keras_b200.models import fusion as fusion_mod

                fusion = _FusionCtx(fusion_mod, training)
        outputs = self._run_through_graph(inputs, operation_fn=lambda op: operation_fn(op, training=training, **kwargs), fusion=fusion)
        return unpack_singleton(outputs)

    def compute_output_spec(self, inputs, training=None, mask=None):
        return Function.compute_output_spec(self, inputs)

    def compute_output_shape(self, input_shape):
        return Function.compute_output_shape(self, input_shape)

    def build(self, input_shape):
        self.built = True

    @property
    def input_shape(self):
        shapes = tree.map_structure(lambda x: x.shape, self.inputs)
        if isinstance(shapes, list) and len(shapes) == 1:
            return shapes[0]
        return shapes

    @property
    def output_shape(self):
        shapes = tree.map_structure(lambda x: x.shape, self.outputs)
        if isinstance(shapes, list) and len(shapes) == 1:
            return shapes[0]
        return shapes

    def _assert_input_compatibility(self, *args):
        return Function._assert_input_compatibility(self, *args)

    def _maybe_warn_inputs_struct_mismatch(self, inputs, raise_exception=False):
        try:
            tree.assert_same_structure(tree.lists_to_tuples(inputs), tree.lists_to_tuples(self._inputs_struct))
        except Exception:
            model_struct = tree.map_structure(lambda x: x.name, self._inputs_struct)
            in_struct = tree.map_structure(lambda x: f"Tensor(shape={tuple(x.shape)})" if hasattr(x, "shape") else str(x), inputs)
            msg = f"The structure of `inputs` doesn't match the expected structure.\nExpected: {model_struct}\nReceived: inputs={in_struct}"
            if raise_exception:
                raise ValueError(msg)
            warnings.warn(msg)

    def _convert_inputs_to_tensors(self, flat_inputs):
        out = []
        for x, ref in zip(flat_inputs, self._inputs):
            if x is None:
                out.append(None)
            else:
                out.append(ops.convert_to_tensor(x, dtype=ref.dtype) if not isinstance(x, KerasTensor) else x)
        return out

    def _adjust_input_rank(self, flat_inputs):
        adjusted = []
        for x, ref in zip(flat_inputs, self._inputs):
            if x is None:
                adjusted.append(x)
                continue
            x_rank, ref_rank = len(x.shape), len(ref.shape)
            if x_rank == ref_rank:
                adjusted.append(x)
            elif x_rank == ref_rank + 1 and x.shape[-1] == 1:
                adjusted.append(ops.squeeze(x, axis=-1))
            elif x_rank == ref_rank - 1 and ref.shape[-1] == 1:
                adjusted.append(ops.expand_dims(x, axis=-1))
            else:
                raise ValueError(f"Invalid input shape for input {x}. Expected shape {ref.shape}, but input has incompatible shape {tuple(x.shape)}")
        for i, x in enumerate(flat_inputs):
            m = getattr(x, "_keras_mask", None)
            if m is not None and adjusted[i] is not x:
                try:
                    adjusted[i]._keras_mask = m
                except AttributeError:
                    pass
        return adjusted

    def _standardize_inputs(self, inputs):
        raise_exception = False
        if isinstance(self._inputs_struct, list) and len(self._inputs_struct) == 1 and isinstance(inputs, (torch.Tensor, KerasTensor)):
            inputs = [inputs]
        elif isinstance(inputs, dict) and not isinstance(self._inputs_struct, dict):
            if hasattr(self._inputs_struct, "__len__") and all(isinstance(i, KerasTensor) for i in self._inputs_struct):
                expected = set(i.name for i in self._inputs_struct)
                if expected.issubset(inputs.keys()):
                    inputs = [inputs[i.name] for i in self._inputs_struct]
                else:
                    raise_exception = True
            elif isinstance(self._inputs_struct, KerasTensor):
                if self._inputs_struct.name in inputs:
                    inputs = [inputs[self._inputs_struct.name]]
                else:
                    raise_exception = True
            else:
                raise_exception = True
        if isinstance(self._inputs_struct, dict) and not isinstance(inputs, dict) and list(self._inputs_struct.keys()) != sorted(self._inputs_struct.keys()):
            raise_exception = True
        if isinstance(inputs, dict) and isinstance(self._inputs_struct, dict):
            flat = [inputs[k] for k in sorted(self._inputs_struct.keys())] if set(self._inputs_struct).issubset(inputs) else tree.flatten(inputs)
            if len(flat) != len(self._inputs):
                self._maybe_warn_inputs_struct_mismatch(inputs, raise_exception=True)
        else:
            flat = tree.flatten(inputs)
            if len(flat) != len(self._inputs) or raise_exception:
                self._maybe_warn_inputs_struct_mismatch(inputs, raise_exception=True)
        flat = self._convert_inputs_to_tensors(flat)
        return self._adjust_input_rank(flat)

    @property
    def input(self):
        return self._inputs_struct

    @property
    def output(self):
        return self._outputs_struct

    def add_loss(self, loss):
        raise NotImplementedError

    @property
    def input_spec(self):
        if hasattr(self, "_manual_input_spec"):
            return self._manual_input_spec

        def shape_with_no_batch_size(x):
            x = list(x)
            if x:
                x[0] = None
            return tuple(x)

        def make_spec_for_tensor(x, name=None):
            optional = False
            hist = x._keras_history
            if isinstance(hist[0], InputLayer):
                if hist[0].optional:
                    optional = True
            return InputSpec(shape=shape_with_no_batch_size(x.shape), allow_last_axis_squeeze=True, name=x._keras_history[0].name if name is None else name, optional=optional)

        if isinstance(self._inputs_struct, dict):
            if all(isinstance(x, KerasTensor) for x in self._inputs_struct.values()):
                names = sorted(self._inputs_struct.keys())
                return [make_spec_for_tensor(self._inputs_struct[n], name=n) for n in names]
            return None
        return [make_spec_for_tensor(x) for x in self.inputs]

    @input_spec.setter
    def input_spec(self, value):
        self._manual_input_spec = value

    # -- config --------------------------------------------------------------------------
    def get_config(self):
        from keras_b200.saving import serialization_lib

        if not functional_like_constructor(self.__class__):
            return Model.get_config(self)
        config = {"name": self.name, "trainable": self.trainable}
        node_reindexing = {}
        for operation in self.operations:
            kept = 0
            for i, node in enumerate(operation._inbound_nodes):
                key = make_node_key(operation, i)
                if key in self._nodes:
                    node_reindexing[key] = kept
                    kept += 1
        layer_configs = []
        for operation in self.operations:
            filtered = []
            for i, node in enumerate(operation._inbound_nodes):
                key = make_node_key(operation, i)
                if key in self._nodes:
                    node_data = serialize_node(node, own_nodes=self._nodes)
                    if node_data is not None:
                        filtered.append(node_data)
            layer_config = serialization_lib.serialize_keras_object(operation)
            layer_config["name"] = operation.name
            layer_config["inbound_nodes"] = filtered
            layer_configs.append(layer_config)
        config["layers"] = layer_configs

        def get_tensor_config(tensor):
            operation, node_index, tensor_index = tensor._keras_history
            key = make_node_key(operation, node_index)
            assert key in self._nodes
            return [operation.name, node_reindexing[key], tensor_index]

        def map_tensors(tensors):
            if isinstance(tensors, KerasTensor):
                return [get_tensor_config(tensors)]
            return tree.map_structure(lambda t: get_tensor_config(t) if isinstance(t, KerasTensor) else t, tensors)

        config["input_layers"] = map_tensors(self._inputs_struct)
        config["output_layers"] = map_tensors(self._outputs_struct)
        return copy.deepcopy(config)


class _FusionCtx:
    __slots__ = ("mod", "training", "Deferred", "NoBias", "run_bn", "run_conv_nobias", "run_pool_padded", "Padded", "build_plan", "applicable")

    def __init__(self, mod, training):
        self.mod, self.training = mod, training
        self.Deferred, self.NoBias, self.run_bn, self.build_plan, self.applicable = mod.Deferred, mod.NoBias, mod.run_bn, mod.build_plan, mod.applicable
        self.run_conv_nobias, self.run_pool_padded, self.Padded = mod.run_conv_nobias, mod.run_pool_padded, mod.Padded


class _NotReady(Exception):
    """A recorded call refers to an output that has not been produced yet."""


class _GraphReplayer:
    """Rebuilds a functional graph from its config by replaying the recorded layer calls.

    Every layer of the config is created first.  Its recorded calls ("inbound nodes") wait in a queue, in config order, and
    a call runs as soon as all tensors it names exist, i.e. as soon as the producing layers have been called often enough.
    The queue is swept until it is empty; a sweep that runs nothing means the config names a tensor nobody produces.
    Calls of one layer keep their recorded order, because node indices are positions in that order."""

    def __init__(self, custom_objects):
        self.custom_objects = custom_objects
        self.layers = {}          # name -> layer
        self.pending = []         # [layer, [recorded call, ...]] in config order

    def add_layer(self, layer_config):
        from keras_b200.saving import serialization_lib

        if "module" in layer_config:
            layer = serialization_lib.deserialize_keras_object(layer_config, custom_objects=self.custom_objects)
        else:  # a Keras 2 config: only class_name / config
            layer = _legacy_layer(layer_config, self.custom_objects)
        if not isinstance(layer, Operation):
            raise ValueError(f"Unexpected object from deserialization, expected a layer or operation, got a {type(layer)}")
        self.layers[layer_config["name"]] = layer
        calls = list(layer_config["inbound_nodes"])
        if calls:
            self.pending.append([layer, calls])

    def output_of(self, layer_name, node_index, tensor_index):
        layer = self.layers.get(layer_name)
        if layer is None:
            raise ValueError(f"Unknown layer: {layer_name}")
        if node_index >= len(layer._inbound_nodes):
            raise _NotReady(layer_name)
        return layer._inbound_nodes[node_index].output_tensors[tensor_index]

    def _arguments(self, call):
        """(args, kwargs) of a recorded call with tensor references replaced by the live tensors."""
        from keras_b200.saving import serialization_lib

        if not call:
            return [], {}
        if isinstance(call, list):
            # Keras 2: [[layer_name, node_index, tensor_index, kwargs?], ...]
            tensors, kwargs = [], {}
            for entry in call:
                tensors.append(self.output_of(entry[0], entry[1], entry[2]))
                if len(entry) == 4:
                    kwargs = entry[3]
            return [unpack_singleton(tensors)], kwargs

        def revive(x):
            history = getattr(x, "_pre_serialization_keras_history", None) if isinstance(x, KerasTensor) else None
            return x if history is None else self.output_of(history[0], history[1], history[2])

        args = tree.map_structure(revive, serialization_lib.deserialize_keras_object(call["args"]))
        kwargs = tree.map_structure(revive, serialization_lib.deserialize_keras_object(call["kwargs"]))
        return args, kwargs

    def replay(self):
        while self.pending:
            ran_any = False
            for entry in self.pending:
                layer, calls = entry
                while calls:
                    try:
                        args, kwargs = self._arguments(calls[0])
                    except _NotReady:
                        break
                    layer(*args, **kwargs)
                    calls.pop(0)
                    ran_any = True
            self.pending = [entry for entry in self.pending if entry[1]]
            if self.pending and not ran_any:
                raise ValueError("Could not rebuild the model graph from its config: some nodes depend on tensors that are never produced.")

    def endpoints(self, spec):
        """Tensors named by an ``input_layers`` / ``output_layers`` entry: ``[name, node, tensor]`` triples in any nesting."""
        if isinstance(spec, list) and len(spec) == 3 and isinstance(spec[0], str):
            name, node_index, tensor_index = spec
            if isinstance(self.layers.get(name), Functional):
                node_index -= 1  # a nested model was called once more when it was built
            return self.output_of(name, node_index, tensor_index)
        if isinstance(spec, dict):
            return {key: self.endpoints(value) for key, value in spec.items()}
        if isinstance(spec, tuple):
            return tuple(self.endpoints(value) for value in spec)
        return [self.endpoints(value) for value in spec]


def functional_from_config(cls, config, custom_objects=None):
    """``cls`` instance rebuilt from ``Functional.get_config()`` output (schema of keras/src/models/functional.py:430-504)."""
    layer_configs = config.pop("layers")
    inputs_spec, outputs_spec = config.pop("input_layers"), config.pop("output_layers")
    name, trainable = config.pop("name", None), config.pop("trainable", None)
    replayer = _GraphReplayer(custom_objects)
    for layer_config in layer_configs:
        replayer.add_layer(layer_config)
    replayer.replay()
    inputs = unpack_singleton(replayer.endpoints(inputs_spec)) if isinstance(inputs_spec, list) else replayer.endpoints(inputs_spec)
    outputs = unpack_singleton(replayer.endpoints(outputs_spec)) if isinstance(outputs_spec, list) else replayer.endpoints(outputs_spec)
    return cls(inputs=inputs, outputs=outputs, name=name, trainable=trainable, **config)


def _legacy_layer(layer_data, custom_objects):
    from keras_b200.legacy.saving import legacy_serialization

    return legacy_serialization.deserialize_layer(layer_data, custom_objects=custom_objects)


def operation_fn(operation, **call_context_args):
    """Bind call-context args (``training`` …) the operation accepts."""

    def call(*args, **kwargs):
        if isinstance(operation, Layer):
            plan = operation._plan
            for name, value in call_context_args.items():
                if value is not None and (name in plan.arg_names or plan.has_var_kw) and name not in kwargs:
                    kwargs[name] = value
        return operation(*args, **kwargs)

    return call


def functional_like_constructor(cls):
    init_args = inspect.getfullargspec(cls.__init__).args[1:]
    functional_init_args = inspect.getfullargspec(Functional.__init__).args[1:]
    return init_args == functional_init_args


def unpack_singleton(x):
    if isinstance(x, (list, tuple)) and len(x) == 1:
        return x[0]
    return x


def serialize_node(node, own_nodes=()):
    from keras_b200.saving import serialization_lib

    if not node.input_tensors:
        return
    def serialize_keras_tensor(x):
        if isinstance(x, KerasTensor):
            operation, node_index, tensor_index = x._keras_history
            irrelevant = 0
            for i, n in enumerate(operation._inbound_nodes[:node_index]):
                if make_node_key(operation, i) not in own_nodes:
                    irrelevant += 1
            x._keras_history = KerasHistory(operation, node_index - irrelevant, tensor_index)
            serialized = serialization_lib.serialize_keras_object(x)
            x._keras_history = KerasHistory(operation, node_index, tensor_index)
            return serialized
        return x

    args = tree.map_structure(serialize_keras_tensor, node.arguments.args)
    kwargs = tree.map_structure(serialize_keras_tensor, node.arguments.kwargs)
    return {"args": serialization_lib.serialize_keras_object(args), "kwargs": serialization_lib.serialize_keras_object(kwargs)}


def is_input_keras_tensor(x):
    op, node_index, _ = x._keras_history
    node = op._inbound_nodes[node_index]
    return node.is_input


def clone_single_keras_tensor(x):
    return KerasTensor(shape=x.shape, dtype=x.dtype, sparse=x.sparse, name=f"{x.name}_clone")


def clone_keras_tensors(tensors, kt_id_mapping):
    def swap(x):
        if not isinstance(x, KerasTensor):
            return x
        if id(x) in kt_id_mapping:
            return kt_id_mapping[id(x)]
        new_x = clone_single_keras_tensor(x)
        kt_id_mapping[id(x)] = new_x
        return new_x

    return tree.map_structure(swap, tensors)


def find_nodes_by_inputs_and_outputs(inputs, outputs):
    from keras_b200.ops.function import _find_between

    return _find_between(inputs, outputs)


def clone_graph_nodes(inputs, outputs):
    """Make a sub-graph defined by intermediate tensors self-contained by cloning its inputs."""
    from keras_b200.ops.function import nodes_between

    nodes_to_clone = nodes_between(inputs, outputs)
    cloned_inputs = []
    cloned_outputs = []
    kt_id_mapping = {}
    op_id_mapping = {}
    for kt_input in tree.flatten(inputs):
        if is_input_keras_tensor(kt_input):
            cloned_inputs.append(kt_input)
            kt_id_mapping[id(kt_input)] = kt_input
        else:
            cloned_input = Input(batch_shape=kt_input.shape, dtype=kt_input.dtype, sparse=kt_input.sparse, name=f"{kt_input.name}CLONE")
            cloned_inputs.append(cloned_input)
            kt_id_mapping[id(kt_input)] = cloned_input
            op_id_mapping[id(kt_input._keras_history[0])] = cloned_input._keras_history[0]
    cloned_inputs = tree.pack_sequence_as(inputs, cloned_inputs)
    for kt_output in tree.flatten(outputs):
        cpy = clone_single_keras_tensor(kt_output)
        cpy._keras_history = kt_output._keras_history
        cloned_outputs.append(cpy)
        kt_id_mapping[id(kt_output)] = cpy
    cloned_outputs = tree.pack_sequence_as(outputs, cloned_outputs)
    for node in nodes_to_clone:
        if id(node.operation) in op_id_mapping:
            operation = op_id_mapping[id(node.operation)]
        else:
            operation = node.operation
        output_copy = clone_keras_tensors(node.output_tensors, kt_id_mapping)
        if not isinstance(operation, InputLayer):
            call_args_copy = clone_keras_tensors(node.arguments.args, kt_id_mapping)
            call_kwargs_copy = clone_keras_tensors(node.arguments.kwargs, kt_id_mapping)
        else:
            call_args_copy = ()
            call_kwargs_copy = {}
        Node(operation, call_args=call_args_copy, call_kwargs=call_kwargs_copy, outputs=output_copy)
    return cloned_inputs, cloned_outputs
