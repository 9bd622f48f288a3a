"""``clone_model`` (keras/src/models/cloning.py:14-425)."""

from keras_b200 import tree
from keras_b200.core.export_registry import keras_export
from keras_b200.core.keras_tensor import KerasTensor
from keras_b200.layers.core.input_layer import Input, InputLayer
from keras_b200.layers.layer import Layer


def _clone_layer(layer):
    from keras_b200.saving import serialization_lib

    return layer.__class__.from_config(layer.get_config())


@keras_export("keras.models.clone_model")
def clone_model(model, input_tensors=None, clone_function=None, call_function=None, recursive=False, **kwargs):
    from keras_b200.models.functional import Functional
    from keras_b200.models.model import Model
    from keras_b200.models.sequential import Sequential

    cache = kwargs.pop("cache", None)
    if kwargs:
        raise ValueError(f"Unexpected keyword argument(s): {tuple(kwargs.keys())}")
    clone_function = clone_function or _clone_layer
    if isinstance(model, Sequential):
        if call_function is not None:
            raise ValueError("`call_function` argument is not supported with Sequential models. Received: call_function=" f"{call_function}")
        return _clone_sequential(model, clone_function, input_tensors, recursive)
    if isinstance(model, Functional):
        if getattr(type(model), "get_config", None) is not None and not _functional_like(model):
            if clone_function is not _clone_layer or input_tensors is not None:
                raise ValueError("Arguments `clone_function` and `input_tensors` are only supported for Sequential models or Functional models.")
        return _clone_functional(model, clone_function, call_function, input_tensors, recursive)
    if clone_function is not _clone_layer or input_tensors is not None:
        raise ValueError(
            "Arguments `clone_function` and `input_tensors` are only supported for Sequential models or Functional models. "
            f"Received model of type '{model.__class__.__name__}', with clone_function={clone_function} and input_tensors={input_tensors}")
    if call_function is not None:
        raise ValueError(f"Argument `call_function` is only supported for Functional models. Received model of type '{model.__class__.__name__}', with call_function={call_function}")
    return model.__class__.from_config(model.get_config())


def _functional_like(model):
    from keras_b200.models.functional import functional_like_constructor

    return functional_like_constructor(model.__class__)


def _clone_sequential(model, clone_function, input_tensors, recursive):
    from keras_b200.models.sequential import Sequential

    new_layers = []
    for layer in model._stack:
        if isinstance(layer, InputLayer):
            continue
        if recursive and isinstance(layer, (Sequential,)) or (recursive and hasattr(layer, "_operations")):
            new_layers.append(clone_model(layer, clone_function=clone_function, recursive=True))
        else:
            new_layers.append(clone_function(layer))
    ref_input = model._stack[0] if model._stack and isinstance(model._stack[0], InputLayer) else None
    if input_tensors is not None:
        if isinstance(input_tensors, (list, tuple)):
            if len(input_tensors) != 1:
                raise ValueError("Argument `input_tensors` must contain a single tensor.")
            input_tensors = input_tensors[0]
        if not isinstance(input_tensors, KerasTensor):
            raise ValueError(f"Argument `input_tensors` must be a KerasTensor. Received invalid value: input_tensors={input_tensors}")
        inputs = Input(tensor=input_tensors, name=ref_input.name if ref_input else None)
        new_layers = [inputs] + new_layers
    elif ref_input is not None:
        inputs = Input(batch_shape=ref_input.batch_shape, dtype=ref_input.dtype, name=ref_input.name)
        new_layers = [inputs] + new_layers
    cloned = Sequential(new_layers, name=model.name, trainable=model.trainable)
    return cloned


def _clone_functional(model, clone_function, call_function, input_tensors, recursive):
    from keras_b200.models.functional import Functional
    from keras_b200.models.model import Model

    if input_tensors is not None:
        if not all(isinstance(x, KerasTensor) for x in tree.flatten(input_tensors)):
            raise ValueError(f"All entries in `input_tensors` must be KerasTensors. Received invalid values: inputs_tensors={input_tensors}")
        try:
            tree.assert_same_structure(input_tensors, model.input, check_types=False)
        except ValueError as e:
            raise ValueError(f"`input_tensors` must have the same structure as model.input\nReference structure: {model.input}\nReceived structure: {input_tensors}") from e
    else:
        input_tensors = tree.map_structure(lambda x: Input(batch_shape=x.shape, dtype=x.dtype, name=x.name), model.input)

    layer_map = {}

    def get_clone(op):
        if id(op) not in layer_map:
            if isinstance(op, InputLayer):
                layer_map[id(op)] = op
            elif recursive and isinstance(op, Model):
                layer_map[id(op)] = clone_model(op, clone_function=clone_function, call_function=call_function, recursive=True)
            elif isinstance(op, Layer):
                layer_map[id(op)] = clone_function(op)
            else:
                layer_map[id(op)] = op
        return layer_map[id(op)]

    def op_fn(op):
        clone = get_clone(op)
        if call_function is not None:
            return lambda *a, **k: call_function(clone, *a, **k)
        return clone

    output_tensors = model._run_through_graph(input_tensors, operation_fn=op_fn)
    if _functional_like(model) and type(model) not in (Functional, Model):
        new_model = model.__class__(input_tensors, output_tensors, name=model.name)
    else:
        new_model = Functional(input_tensors, output_tensors, name=model.name)
    if model.compiled:
        compiled_config = model.get_compile_config()
        new_model.compile_from_config(compiled_config)
    return new_model
