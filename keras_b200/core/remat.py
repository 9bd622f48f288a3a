"""Rematerialisation (activation recomputation) scopes.

Behaviour of keras/src/backend/common/remat.py:9-186: ``RematScope(mode=...)`` with modes
``full``, ``activations``, ``larger_than`` (+ ``output_size_threshold``), ``list_of_layers``
(+ ``layer_names``) decides which layers recompute their forward pass during backward.
"""

import collections

from keras_b200.core import global_state
from keras_b200.core.export_registry import keras_export

RematMode = collections.namedtuple("RematMode", ["mode", "output_size_threshold", "layer_names"])


@keras_export("keras.RematScope")
class RematScope:
    def __init__(self, mode="full", output_size_threshold=1024, layer_names=None):
        if mode not in {"full", "activations", "larger_than", "list_of_layers", None}:
            raise ValueError(
                f"Invalid mode '{mode}'. Supported modes are: 'full', 'activations', 'larger_than', 'list_of_layers', or None."
            )
        self.mode = mode
        self.output_size_threshold = output_size_threshold
        self.layer_names = layer_names or []
        self._pop = False

    def __enter__(self):
        stack = global_state.get_global_attribute("remat_scope_stack", default=[], set_to_default=True)
        stack.append(self)
        self._pop = True
        return self

    def __exit__(self, *exc):
        if self._pop:
            global_state.get_global_attribute("remat_scope_stack").pop()
            self._pop = False


def get_current_remat_mode():
    stack = global_state.get_global_attribute("remat_scope_stack")
    if not stack:
        return None
    top = stack[-1]
    if top.mode is None:
        return None
    return RematMode(top.mode, top.output_size_threshold, top.layer_names)


@keras_export("keras.remat")
def remat(f):
    import torch.utils.checkpoint as ckpt

    def wrapped(*args, **kwargs):
        return ckpt.checkpoint(f, *args, use_reentrant=False, **kwargs)

    return wrapped


def wrap_for_mode(layer, layer_call, mode, args, kwargs):
    """Return the callable to use for this call according to the remat mode."""
    if mode is None:
        return layer_call
    import torch

    if not torch.is_grad_enabled():
        return layer_call
    if mode.mode == "full":
        return remat(layer_call)
    if mode.mode == "list_of_layers":
        return remat(layer_call) if layer.name in mode.layer_names else layer_call
    if mode.mode == "larger_than":
        try:
            import math

            from keras_b200 import tree
            from keras_b200.core.tensor import compute_output_spec
            from keras_b200.core.keras_tensor import KerasTensor
            from keras_b200.core.dtypes import standardize_dtype

            spec_args, spec_kwargs = tree.map_structure(
                lambda x: KerasTensor(tuple(x.shape), standardize_dtype(x.dtype)) if isinstance(x, torch.Tensor) else x, (args, kwargs)
            )
            out = compute_output_spec(layer_call, *spec_args, **spec_kwargs)
            size = sum(math.prod(d for d in o.shape if d is not None) for o in tree.flatten(out) if isinstance(o, KerasTensor))
            return remat(layer_call) if size > mode.output_size_threshold else layer_call
        except Exception:
            return layer_call
    if mode.mode == "activations":
        has_act = getattr(layer, "activation", None) is not None and getattr(layer.activation, "__name__", "linear") != "linear"
        return remat(layer_call) if has_act else layer_call
    return layer_call
