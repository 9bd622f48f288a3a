"""``model_to_dot`` / ``plot_model`` (keras/src/utils/model_visualization.py).  Both need ``pydot`` and graphviz;
without them they raise the same ``ImportError`` as the reference.  ``model_to_dot_source`` gives the DOT text
without any dependency."""

import os

from keras_b200 import tree
from keras_b200.core.export_registry import keras_export

try:
    import pydot
except ImportError:
    pydot = None


def check_pydot():
    return pydot is not None


def check_graphviz():
    if not check_pydot():
        return False
    try:
        pydot.Dot.create(pydot.Dot())
        return True
    except (OSError, Exception):
        return False


def _label(layer, show_layer_names, show_shapes, show_dtype, show_layer_activations, show_trainable):
    cls = layer.__class__.__name__
    parts = [f"{layer.name} ({cls})" if show_layer_names else cls]
    if show_layer_activations and getattr(layer, "activation", None) is not None:
        act = layer.activation
        parts.append("Activation: " + (getattr(act, "__name__", None) or act.__class__.__name__))
    if show_shapes:
        from keras_b200.utils.summary_utils import format_layer_shape

        parts.append("Output shape: " + str(format_layer_shape(layer)))
    if show_dtype:
        parts.append("Output dtype: " + str(getattr(layer, "compute_dtype", "?")))
    if show_trainable and hasattr(layer, "trainable") and layer.weights:
        parts.append("Trainable" if layer.trainable else "Non-trainable")
    return "\\n".join(parts)


def _edges(model):
    from keras_b200.models import Functional, Sequential

    if isinstance(model, Sequential):
        layers = model.layers
        return layers, [(layers[i], layers[i + 1]) for i in range(len(layers) - 1)]
    if isinstance(model, Functional):
        layers = list(model._operations)
        edges = []
        for layer in layers:
            for node in layer._inbound_nodes:
                if node not in [n for d in model._nodes_by_depth.values() for n in d]:
                    continue
                for kt in tree.flatten(node.input_tensors):
                    src = kt._keras_history.operation
                    if (src, layer) not in edges:
                        edges.append((src, layer))
        return layers, edges
    return list(model.layers), []


def model_to_dot_source(model, show_shapes=False, show_dtype=False, show_layer_names=True, rankdir="TB", show_layer_activations=False,
                        show_trainable=False, dpi=200):
    """DOT source of the layer graph as a string."""
    layers, edges = _edges(model)
    lines = ["digraph G {", f'  rankdir={rankdir}; dpi={dpi}; node [shape=record, fontname="Helvetica"];']
    for layer in layers:
        lines.append(f'  n{id(layer)} [label="{_label(layer, show_layer_names, show_shapes, show_dtype, show_layer_activations, show_trainable)}"];')
    for a, b in edges:
        lines.append(f"  n{id(a)} -> n{id(b)};")
    lines.append("}")
    return "\n".join(lines)


@keras_export("keras.utils.model_to_dot")
def model_to_dot(model, show_shapes=False, show_dtype=False, show_layer_names=True, rankdir="TB", expand_nested=False, dpi=200, subgraph=False,
                 show_layer_activations=False, show_trainable=False, **kwargs):
    if not model.built:
        raise ValueError("This model has not yet been built. Build the model first by calling `build()` or by calling the model on a batch of data.")
    if not check_pydot():
        raise ImportError("You must install pydot (`pip install pydot`) for model_to_dot to work.")
    src = model_to_dot_source(model, show_shapes, show_dtype, show_layer_names, rankdir, show_layer_activations, show_trainable, dpi)
    return pydot.graph_from_dot_data(src)[0]


@keras_export("keras.utils.plot_model")
def plot_model(model, to_file="model.png", show_shapes=False, show_dtype=False, show_layer_names=False, rankdir="TB", expand_nested=False, dpi=200,
               show_layer_activations=False, show_trainable=False, **kwargs):
    if not model.built:
        raise ValueError("This model has not yet been built. Build the model first by calling `build()` or by calling the model on a batch of data.")
    if not check_pydot():
        message = "You must install pydot (`pip install pydot`) for `plot_model` to work."
        raise ImportError(message)
    if not check_graphviz():
        message = "You must install graphviz (see instructions at https://graphviz.gitlab.io/download/) for `plot_model` to work."
        raise ImportError(message)
    dot = model_to_dot(model, show_shapes=show_shapes, show_dtype=show_dtype, show_layer_names=show_layer_names, rankdir=rankdir,
                       expand_nested=expand_nested, dpi=dpi, show_layer_activations=show_layer_activations, show_trainable=show_trainable)
    to_file = str(to_file)
    _, extension = os.path.splitext(to_file)
    extension = extension[1:] if extension else "png"
    dot.write(to_file, format=extension)
    if extension != "pdf":
        try:
            from IPython import display

            return display.Image(filename=to_file)
        except ImportError:
            pass
