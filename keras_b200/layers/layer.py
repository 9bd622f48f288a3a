"""``Layer``: state (variables, sub-layers) + computation (``call``).

Behaviour follows keras/src/layers/layer.py:71-1888 (tracking, ``build`` wrapper, ``add_weight``,
the ``__call__`` pipeline with autocast / masks / ``training`` resolution, losses, stateless
call, variable (de)serialization by index).  Differences by design: a layer is not a
``torch.nn.Module``; the per-call argument handling is compiled once per class into a *call
plan* (argument names, whether ``training`` / ``mask`` are accepted) so the hot path does no
``inspect.Signature.bind``; and sharded variables (``ModelParallel``) are first class.
"""

import collections
import inspect
import os
import warnings

import torch

from keras_b200 import constraints, dtype_policies, initializers, regularizers, tree
from keras_b200.core import config, global_state
from keras_b200.core.dtypes import standardize_dtype, to_torch_dtype
from keras_b200.core.export_registry import keras_export
from keras_b200.core.keras_tensor import KerasTensor, any_symbolic_tensors
from keras_b200.core.naming import auto_name
from keras_b200.core.scopes import StatelessScope, current_path, in_stateless_scope, name_scope
from keras_b200.core.tensor import convert_to_tensor, get_device
from keras_b200.core.variables import AutocastScope, Variable
from keras_b200.layers.input_spec import InputSpec, assert_input_compatibility
from keras_b200.ops.node import Node
from keras_b200.ops.operation import Operation

_TENSOR_TYPES = (torch.Tensor, KerasTensor)


# KERAS_B200_NVTX=1: every eager layer call opens an NVTX range named by the layer's path (for profiler timelines).
_NVTX_RANGES = os.environ.get("KERAS_B200_NVTX", "0") == "1" and torch.cuda.is_available()


class _TrackedList(list):
    """List that reports inserted values to its owner layer (so appended sub-layers are tracked)."""

    _tree_rebuild_as_list = True

    def __init__(self, owner, values=()):
        self._owner = owner
        super().__init__(owner._track_value(v) for v in values)

    def append(self, v):
        super().append(self._owner._track_value(v))

    def extend(self, vs):
        super().extend(self._owner._track_value(v) for v in vs)

    def insert(self, i, v):
        super().insert(i, self._owner._track_value(v))

    def __setitem__(self, i, v):
        if isinstance(i, slice):
            v = [self._owner._track_value(e) for e in v]
        else:
            v = self._owner._track_value(v)
        super().__setitem__(i, v)

    def __iadd__(self, vs):
        self.extend(vs)
        return self

    def __reduce__(self):
        return (list, (list(self),))


class _TrackedDict(dict):
    _tree_rebuild_as_dict = True

    def __init__(self, owner, values=None):
        self._owner = owner
        super().__init__()
        for k, v in (values or {}).items():
            self[k] = v

    def __setitem__(self, k, v):
        super().__setitem__(k, self._owner._track_value(v))

    def update(self, other=(), **kw):
        for k, v in dict(other, **kw).items():
            self[k] = v

    def setdefault(self, k, default=None):
        if k not in self:
            self[k] = default
        return self[k]

    def __reduce__(self):
        return (dict, (dict(self),))


class _CallPlan:
    """Per-class facts about ``call`` / ``build`` signatures, computed once."""

    _tree_rebuild_as_dict = True

    __slots__ = ("arg_names", "has_training", "has_mask", "has_var_kw", "build_names", "build_by_name", "signature", "context_args", "n_positional", "mask_pairs")

    def __init__(self, cls):
        sig = inspect.signature(cls.call)
        self.signature = sig
        params = list(sig.parameters.values())[1:]
        self.arg_names = [p.name for p in params if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD, p.KEYWORD_ONLY)]
        self.n_positional = len([p for p in params if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)])
        self.has_var_kw = any(p.kind == p.VAR_KEYWORD for p in params)
        self.has_training = "training" in self.arg_names
        self.has_mask = "mask" in self.arg_names
        self.mask_pairs = [(n, f"{n}_mask") for n in self.arg_names if f"{n}_mask" in self.arg_names]
        try:
            bparams = list(inspect.signature(cls.build).parameters.values())[1:]
        except (TypeError, ValueError):
            bparams = []
        self.build_names = [p.name for p in bparams if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD, p.KEYWORD_ONLY)]
        self.build_by_name = len(self.build_names) > 0 and all(n.endswith("_shape") or n.endswith("_shapes") for n in self.build_names) and not (len(self.build_names) == 1 and self.build_names[0] in ("input_shape", "inputs_shape", "input_shapes"))


_PLANS = {}


def _plan_for(cls):
    plan = _PLANS.get(cls)
    if plan is None:
        plan = _CallPlan(cls)
        _PLANS[cls] = plan
    return plan


class CallContext:
    __slots__ = ("entry_layer", "training", "extra")

    def __init__(self, entry_layer):
        self.entry_layer = entry_layer
        self.training = None
        self.extra = {}

    def get_value(self, arg_name, default=None):
        if arg_name == "training":
            return self.training if self.training is not None else default
        return self.extra.get(arg_name, default)

    def set_value(self, arg_name, value):
        if arg_name == "training":
            self.training = value
        else:
            self.extra[arg_name] = value


def _wrap_build(build_fn):
    if getattr(build_fn, "_is_build_wrapper", False):
        return build_fn

    def build(self, *args, **kwargs):
        if self.built and getattr(self, "_build_lock_shapes", None) is not None and not getattr(self, "_allow_rebuild", False):
            return
        depth = self.__dict__.get("_build_depth", 0)
        object.__setattr__(self, "_build_depth", depth + 1)
        try:
            with _StateUnlock(self), self._open_name_scope():
                self._path = current_path()
                build_fn(self, *args, **kwargs)
        finally:
            object.__setattr__(self, "_build_depth", depth)
        if depth > 0:
            return  # a parent class's build called through super(): the outermost build finishes and locks the state
        names = _plan_for(type(self)).build_names
        shapes = dict(zip(names, args))
        shapes.update(kwargs)
        self._build_shapes_dict = shapes
        self.built = True
        self._build_lock_shapes = True
        self._post_build()
        self._lock_state()

    build._is_build_wrapper = True
    build.__wrapped__ = build_fn
    build.__doc__ = build_fn.__doc__
    return build


def _wrap_quantize(fn):
    if getattr(fn, "_is_quantize_wrapper", False):
        return fn

    def quantize(self, mode=None, config=None, **kwargs):
        from keras_b200.quantizers.quantization_config import validate_and_resolve_config

        config = validate_and_resolve_config(mode, config)
        mode = config.mode
        self._check_quantize_args(mode, self.compute_dtype)
        self._tracker_unlock()
        try:
            result = fn(self, mode, config=config, **kwargs) if _accepts_config(fn) else fn(self, mode, **kwargs)
        finally:
            self._lock_state()
        self._post_quantize(mode, **kwargs)
        return result

    quantize._is_quantize_wrapper = True
    quantize.__wrapped__ = fn
    return quantize


def _accepts_config(fn):
    try:
        return "config" in inspect.signature(fn).parameters
    except (TypeError, ValueError):
        return False


class _StateUnlock:
    def __init__(self, layer):
        self.layer = layer

    def __enter__(self):
        self.prev = self.layer._locked
        object.__setattr__(self.layer, "_locked", False)

    def __exit__(self, *exc):
        object.__setattr__(self.layer, "_locked", self.prev)


@keras_export(["keras.Layer", "keras.layers.Layer"])
class Layer(Operation):
    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        if "build" in cls.__dict__:
            cls.build = _wrap_build(cls.__dict__["build"])
        if "quantize" in cls.__dict__:
            cls.quantize = _wrap_quantize(cls.__dict__["quantize"])

    def __init__(self, *, activity_regularizer=None, trainable=True, dtype=None, autocast=True, name=None, **kwargs):
        object.__setattr__(self, "_locked", False)
        object.__setattr__(self, "_layers", [])
        object.__setattr__(self, "_trainable_variables", [])
        object.__setattr__(self, "_non_trainable_variables", [])
        object.__setattr__(self, "_metrics", [])
        object.__setattr__(self, "_seed_generators", [])
        Operation.__init__(self, name=name)
        self.activity_regularizer = regularizers.get(activity_regularizer)
        input_dim_arg = kwargs.pop("input_dim", None)
        if input_dim_arg is not None:
            input_shape_arg = (input_dim_arg,)
        else:
            input_shape_arg = kwargs.pop("input_shape", None)
        if kwargs:
            raise ValueError(f"Unrecognized keyword arguments passed to {self.__class__.__name__}: {kwargs}")
        self._input_shape_arg = input_shape_arg
        if input_shape_arg is not None:
            warnings.warn(
                "Do not pass an `input_shape`/`input_dim` argument to a layer. When using Sequential "
                "models, prefer using an `Input(shape)` object as the first layer in the model instead.",
                stacklevel=2,
            )
        self._path = None
        self.built = False
        self.autocast = autocast
        self._dtype_policy = dtype_policies.get(dtype)
        self._input_spec = None
        self._called = False
        self.supports_jit = True
        self._trainable = trainable
        self._losses = []
        self._loss_ids = set()
        self._losses_override = []
        self._supports_masking = not _is_default(type(self), "compute_mask")
        self._convert_input_args = True
        self._allow_non_tensor_positional_args = False
        self._build_shapes_dict = None
        self._parent_path = None
        self._remat_mode = _current_remat_mode()
        self._plan = _plan_for(type(self))
        self._call_context_args = {"training"}
        self._cached_vars = None
        self._autocast_cache = None

    # -- attribute tracking --------------------------------------------------------------
    def _track_value(self, value):
        if isinstance(value, Layer):
            if value is not self and not any(value is l for l in self._layers):
                self._layers.append(value)
                self._invalidate()
        elif isinstance(value, Variable):
            self._track_variable(value)
        elif isinstance(value, _TRACK_EXTRA):
            self._track_extra(value)
        elif type(value) is list or type(value) is collections.deque:
            return _TrackedList(self, value) if type(value) is list else value
        elif type(value) is dict or type(value) is collections.OrderedDict:
            return _TrackedDict(self, value)
        elif isinstance(value, tuple) and not hasattr(value, "_fields"):
            for v in value:
                if isinstance(v, (Layer, Variable) + _TRACK_EXTRA) or type(v) in (list, dict):
                    return tuple(self._track_value(e) for e in value)
        return value

    def _track_extra(self, value):
        from keras_b200.metrics.metric import Metric
        from keras_b200.random.seed_generator import SeedGenerator

        if isinstance(value, Metric):
            if not any(value is m for m in self._metrics):
                self._metrics.append(value)
                self._invalidate()
        elif isinstance(value, SeedGenerator):
            if not any(value is s for s in self._seed_generators):
                self._seed_generators.append(value)
                self._invalidate()

    def _track_variable(self, variable):
        if variable.trainable:
            target = self._trainable_variables
        else:
            target = self._non_trainable_variables
        if not any(variable is v for v in self._trainable_variables) and not any(variable is v for v in self._non_trainable_variables):
            if self._locked:
                raise ValueError(
                    "You cannot add new elements of state (variables or sub-layers) to a layer that is "
                    "already built. All state must be created in the `__init__()` method or in the "
                    "`build()` method."
                )
            target.append(variable)
            if not self.trainable:
                variable.trainable = False
            self._invalidate()

    def _untrack_variable(self, variable):
        for lst in (self._trainable_variables, self._non_trainable_variables):
            for i, v in enumerate(lst):
                if v is variable:
                    del lst[i]
                    break
        self._invalidate()

    def _invalidate(self):
        object.__setattr__(self, "_cached_vars", None)

    def __setattr__(self, name, value):
        if name in _UNTRACKED_ATTRS:
            object.__setattr__(self, name, value)
            return
        if name[0] != "_" or not isinstance(value, (bool, int, float, str, type(None))):
            try:
                value = self._track_value(value)
            except AttributeError:
                # attribute assigned before Layer.__init__ ran
                if isinstance(value, (Layer, Variable)):
                    raise RuntimeError(
                        f"In layer {self.__class__.__name__}, you forgot to call `super().__init__()` as the "
                        "first statement in the `__init__()` method. Go add it!"
                    )
        object.__setattr__(self, name, value)

    def __delattr__(self, name):
        value = self.__dict__.get(name)
        if isinstance(value, Variable):
            self._untrack_variable(value)
        elif isinstance(value, Layer):
            self._layers[:] = [l for l in self._layers if l is not value]
            self._invalidate()
        object.__delattr__(self, name)

    def _lock_state(self):
        object.__setattr__(self, "_locked", True)

    def _tracker_unlock(self):
        object.__setattr__(self, "_locked", False)

    def _post_build(self):
        pass

    def _post_track_variable(self, variable):
        pass

    def _check_super_called(self):
        if "_layers" not in self.__dict__:
            raise RuntimeError(
                f"In layer '{self.__class__.__name__}', you forgot to call `super().__init__()` as the "
                "first statement in the `__init__()` method. Go add it!"
            )

    # -- naming --------------------------------------------------------------------------
    def _open_name_scope(self):
        if self._parent_path is None:
            self._parent_path = current_path()
        return name_scope(self.name, caller=self, override_parent=self._parent_path)

    @property
    def path(self):
        return self._path

    # -- build ---------------------------------------------------------------------------
    def build(self, input_shape):
        self._check_super_called()
        if _is_default(type(self), "call") is False and _might_have_unbuilt_state(self):
            warnings.warn(
                f"`build()` was called on layer '{self.name}', however the layer does not have a "
                "`build()` method implemented and it looks like it has unbuilt state. This will cause "
                "the layer to be marked as built, despite not being actually built, which may cause "
                "failures down the line. Make sure to implement a proper `build()` method."
            )
        self.built = True

    def get_build_config(self):
        if self._build_shapes_dict is not None:
            if len(self._build_shapes_dict) == 1:
                return {"input_shape": tuple(self._build_shapes_dict.values())[0]}
            return {"shapes_dict": self._build_shapes_dict}

    def build_from_config(self, config):
        if config:
            if "input_shape" in config:
                self.build(config["input_shape"])
            elif "shapes_dict" in config:
                self.build(**config["shapes_dict"])

    def add_variable(self, shape, initializer, dtype=None, trainable=True, autocast=True, regularizer=None, constraint=None, name=None):
        return self.add_weight(shape=shape, initializer=initializer, dtype=dtype, trainable=trainable, autocast=autocast, regularizer=regularizer, constraint=constraint, name=name)

    def add_weight(self, shape=None, initializer=None, dtype=None, trainable=True, autocast=True, regularizer=None, constraint=None, aggregation="none", overwrite_with_gradient=False, name=None):
        self._check_super_called()
        if shape is None:
            shape = ()
        if dtype is not None:
            dtype = standardize_dtype(dtype)
        else:
            dtype = self.variable_dtype
        if initializer is None:
            initializer = "glorot_uniform" if "float" in dtype else "zeros"
        initializer = initializers.get(initializer)
        with self._open_name_scope():
            variable = Variable(initializer=initializer, shape=shape, dtype=dtype, trainable=trainable, autocast=autocast, aggregation=aggregation, name=name)
        variable.regularizer = regularizers.get(regularizer)
        variable.constraint = constraints.get(constraint)
        variable.overwrite_with_gradient = overwrite_with_gradient
        self._track_variable(variable)
        return variable

    # -- trainable / variables -----------------------------------------------------------
    @property
    def trainable(self):
        return self._trainable

    @trainable.setter
    def trainable(self, value):
        value = bool(value)
        object.__setattr__(self, "_trainable", value)
        for v in self._trainable_variables:
            v.trainable = value
        for layer in self._layers:
            layer.trainable = value
        self._invalidate()

    def _collect(self):
        """(variables, trainable, non_trainable) over this layer and all sub-layers, deduplicated."""
        cache = self._cached_vars
        if cache is not None and cache[0] == self._tracking_signature():
            return cache[1]
        seen = set()
        all_vars, trainable, non_trainable = [], [], []

        def visit(layer, ancestors_trainable):
            layer_trainable = ancestors_trainable and layer._trainable
            for v in layer._trainable_variables:
                if id(v) not in seen:
                    seen.add(id(v))
                    all_vars.append(v)
                    (trainable if (layer_trainable and v.trainable) else non_trainable).append(v)
            for v in layer._non_trainable_variables:
                if id(v) not in seen:
                    seen.add(id(v))
                    all_vars.append(v)
                    non_trainable.append(v)
            for sg in layer._seed_generators:
                v = sg.state
                if id(v) not in seen:
                    seen.add(id(v))
                    all_vars.append(v)
                    non_trainable.append(v)

        # own variables first, then metrics, then sub-layers depth-first (reference order)
        def walk(layer, anc):
            visit(layer, anc)
            for m in layer._metrics:
                for v in m.variables:
                    if id(v) not in seen:
                        seen.add(id(v))
                        all_vars.append(v)
                        non_trainable.append(v)
            for sub in layer._layers:
                walk(sub, anc and layer._trainable)

        walk(self, True)
        result = (all_vars, trainable, non_trainable)
        object.__setattr__(self, "_cached_vars", (self._tracking_signature(), result))
        return result

    def _tracking_signature(self):
        # cheap structural fingerprint: sums of list lengths across the tree
        total = 0
        stack = [self]
        while stack:
            l = stack.pop()
            total += len(l._trainable_variables) * 1000003 + len(l._non_trainable_variables) * 10007 + len(l._layers) * 101 + (7 if l._trainable else 0) + len(l._metrics) + len(l._seed_generators) * 13
            stack.extend(l._layers)
        return total

    @property
    def variables(self):
        return list(self._collect()[0])

    @property
    def trainable_variables(self):
        if not self._trainable:
            return []
        return list(self._collect()[1])

    @property
    def non_trainable_variables(self):
        if not self._trainable:
            return list(self._collect()[0])
        return list(self._collect()[2])

    @property
    def weights(self):
        """Weight variables in layer order: a layer's own trainable then non-trainable variables, followed by those of its
        sub-layers, depth first (keras/src/layers/layer.py:713-731).  ``get_weights`` / ``set_weights`` use this order, so
        BatchNormalization contributes gamma, beta, moving_mean, moving_variance in one run."""
        skip = {id(v) for v in self._all_aux_variables()}
        out, seen = [], set()

        def walk(layer):
            for v in layer._trainable_variables + layer._non_trainable_variables:
                if id(v) not in seen and id(v) not in skip:
                    seen.add(id(v))
                    out.append(v)
            for sub in layer._layers:
                walk(sub)

        walk(self)
        return out

    @property
    def trainable_weights(self):
        return self.trainable_variables

    @property
    def non_trainable_weights(self):
        skip = {id(v) for v in self._all_aux_variables()}
        return [v for v in self.non_trainable_variables if id(v) not in skip]

    def _all_aux_variables(self):
        """Seed-generator and metric state: variables that are not weights."""
        out = []
        for layer in self._flatten_layers(include_self=True):
            for sg in layer._seed_generators:
                out.append(sg.state)
            for m in layer._metrics:
                out.extend(m.variables)
        return out

    @property
    def metrics(self):
        out = list(self._metrics)
        for layer in self._flatten_layers(include_self=False):
            out.extend(layer._metrics)
        return out

    @property
    def metrics_variables(self):
        vars_ = []
        for m in self.metrics:
            vars_.extend(m.variables)
        return vars_

    def get_weights(self):
        return [v.numpy() for v in self.weights]

    def set_weights(self, weights):
        layer_weights = self.weights
        if len(layer_weights) != len(weights):
            raise ValueError(
                f"You called `set_weights(weights)` on layer '{self.name}' with a weight list of length "
                f"{len(weights)}, but the layer was expecting {len(layer_weights)} weights."
            )
        for variable, value in zip(layer_weights, weights):
            if tuple(variable.shape) != tuple(value.shape):
                raise ValueError(f"Layer {self.name} weight shape {variable.shape} is not compatible with provided weight shape {value.shape}.")
            variable.assign(value)

    def parameters(self):
        """Underlying ``torch.nn.Parameter`` objects (for interop with torch optimizers)."""
        return [v._value for v in self.variables if v._value is not None]

    def count_params(self):
        if not self.built:
            raise ValueError(
                f"You tried to call `count_params` on layer '{self.name}', but the layer isn't built. "
                "You can build it manually via: `layer.build(input_shape)`."
            )
        import math

        return int(sum(math.prod(v.shape) for v in self.weights))

    def _flatten_layers(self, include_self=True, recursive=True):
        out = [self] if include_self else []
        seen = {id(self)}
        queue = collections.deque(self._layers)
        while queue:
            layer = queue.popleft()
            if id(layer) in seen:
                continue
            seen.add(id(layer))
            out.append(layer)
            if recursive:
                queue.extendleft(reversed(layer._layers))
        return out

    # -- dtype ---------------------------------------------------------------------------
    @property
    def dtype_policy(self):
        return self._dtype_policy

    @dtype_policy.setter
    def dtype_policy(self, value):
        policy = dtype_policies.get(value)
        from keras_b200.dtype_policies.dtype_policy_map import DTypePolicyMap

        if isinstance(self._dtype_policy, DTypePolicyMap) and self.path:
            if self.path in self._dtype_policy:
                del self._dtype_policy[self.path]
            self._dtype_policy[self.path] = policy
        else:
            self._dtype_policy = policy
        if policy.quantization_mode is not None:
            if self.built and not getattr(self, "_is_quantized", False):
                self.quantize(policy.quantization_mode)

    def _resolved_policy(self):
        from keras_b200.dtype_policies.dtype_policy_map import DTypePolicyMap

        p = self._dtype_policy
        if isinstance(p, DTypePolicyMap):
            return p[self.path] if self.path else p.default_policy
        return p

    @property
    def dtype(self):
        return self.variable_dtype

    @property
    def compute_dtype(self):
        return self._resolved_policy().compute_dtype

    @property
    def variable_dtype(self):
        return self._resolved_policy().variable_dtype

    @property
    def quantization_mode(self):
        return self._resolved_policy().quantization_mode

    @property
    def input_dtype(self):
        return self.compute_dtype

    @property
    def supports_masking(self):
        return self._supports_masking

    @supports_masking.setter
    def supports_masking(self, value):
        self._supports_masking = value

    @property
    def input_spec(self):
        return self._input_spec

    @input_spec.setter
    def input_spec(self, value):
        self._input_spec = value

    # -- the call pipeline ---------------------------------------------------------------
    def __call__(self, *args, **kwargs):
        self._check_super_called()
        self._called = True
        plan = self._plan

        # 1. input conversion + autocast
        if self._convert_input_args:
            compute_td = None
            if args:
                first = args[0]
                if type(first) is torch.Tensor:
                    if self.autocast and first.dtype.is_floating_point:
                        compute_td = self._compute_torch_dtype()
                        if first.dtype != compute_td and compute_td.is_floating_point:
                            args = (first.to(compute_td),) + args[1:]
                elif not isinstance(first, KerasTensor):
                    args = (self._convert_structure(first),) + args[1:]
                if len(args) > 1:
                    args = (args[0],) + tuple(self._convert_structure(a) for a in args[1:])
            if kwargs:
                for k, v in kwargs.items():
                    if v is not None and k != "training" and not isinstance(v, (bool, int, float, str)):
                        kwargs[k] = self._convert_structure(v)

        if not self._allow_non_tensor_positional_args and args:
            for a in args:
                if not isinstance(a, _TENSOR_TYPES) and a is not None and not _only_tensors(a):
                    raise ValueError(
                        "Only input tensors may be passed as positional arguments. The following argument "
                        f"value should be passed as a keyword argument: {a} (of type {type(a)})"
                    )

        symbolic = any_symbolic_tensors(args, kwargs)

        # 2. map positional arguments to names when needed (build by name, masks on extra args)
        first_arg = args[0] if args else (kwargs.get(plan.arg_names[0]) if plan.arg_names and plan.arg_names[0] in kwargs else None)

        # 3. input spec + build
        if self._input_spec is not None and first_arg is not None and (symbolic or not getattr(self, "_tp_local_input", False)):
            if type(first_arg) is torch.Tensor:
                # eager tensors: a (spec, shape, dtype) combination that passed once passes again
                sig = (id(self._input_spec), first_arg.shape, first_arg.dtype)
                if sig != self.__dict__.get("_spec_checked"):
                    assert_input_compatibility(self._input_spec, first_arg, self.name)
                    self.__dict__["_spec_checked"] = sig
            else:
                assert_input_compatibility(self._input_spec, first_arg, self.name)
        if not self.built:
            with self._open_name_scope():
                self._maybe_build(plan, args, kwargs)

        # 4. training flag
        ctx = global_state.get_global_attribute("current_call_ctx")
        entered = False
        if ctx is None:
            ctx = CallContext(self)
            global_state.set_global_attribute("current_call_ctx", ctx)
            entered = True
        try:
            prev_training = ctx.training
            training = kwargs.get("training") if "training" in kwargs else None
            if training is None and plan.has_training and len(args) > plan.arg_names.index("training") >= 0 and plan.arg_names.index("training") < plan.n_positional:
                training = args[plan.arg_names.index("training")]
            if training is None:
                training = ctx.training
                if training is None:
                    default = plan.signature.parameters["training"].default if plan.has_training else None
                    training = None if default is inspect.Parameter.empty else default
            else:
                ctx.training = training
            implicit = ()
            if plan.has_training:
                if not (len(args) > plan.arg_names.index("training") and plan.arg_names.index("training") < plan.n_positional):
                    if kwargs.get("training") is None:
                        implicit = ("training",)  # resolved from the context or the default, not chosen by the caller
                    kwargs["training"] = training
            elif "training" in kwargs and not plan.has_var_kw:
                kwargs.pop("training")
            for extra in self._call_context_args:
                if extra != "training":
                    self._resolve_context_arg(extra, ctx, plan, kwargs)

            # 5. masks
            if plan.has_mask:
                if kwargs.get("mask") is None and not (len(args) > plan.arg_names.index("mask") and plan.arg_names.index("mask") < plan.n_positional):
                    m = _get_mask(first_arg)
                    if m is not None:
                        kwargs["mask"] = m
            if plan.mask_pairs:
                # an argument ``x`` with a companion ``x_mask`` gets the mask attached to its value, once the call has more
                # than one tensor argument (with a single one only ``mask`` is filled, above)
                bound = dict(zip(plan.arg_names, args))
                bound.update(kwargs)
                if sum(1 for v in bound.values() if isinstance(v, (torch.Tensor, KerasTensor))) > 1:
                    for nm, mk in plan.mask_pairs:
                        if bound.get(mk) is None and bound.get(nm) is not None:
                            m = _get_mask(bound[nm])
                            if m is not None:
                                kwargs[mk] = m

            # 6. run
            with self._open_name_scope():
                if self.autocast and self.compute_dtype != self.variable_dtype:
                    scope = self._autocast_cache
                    if scope is None or scope.dtype != self.compute_dtype:
                        scope = AutocastScope(self.compute_dtype)
                        object.__setattr__(self, "_autocast_cache", scope)
                    outer = global_state.get_global_attribute("autocast_scope")
                    global_state.set_global_attribute("autocast_scope", scope)
                else:
                    outer = global_state.get_global_attribute("autocast_scope")
                    global_state.set_global_attribute("autocast_scope", _NO_AUTOCAST)
                try:
                    if symbolic:
                        # a graph node remembers only what the caller chose: an implicit `training` stays open so that the
                        # model's own call can set it later
                        outputs = self._symbolic_call(*args, _implicit=implicit, **kwargs) if implicit else self._symbolic_call(*args, **kwargs)
                    elif _NVTX_RANGES:
                        # one profiler range per layer call, named by the layer's path: a timeline then reads in model terms
                        torch.cuda.nvtx.range_push(getattr(self, "path", None) or self.name)
                        try:
                            outputs = self._eager_call(*args, **kwargs)
                        finally:
                            torch.cuda.nvtx.range_pop()
                    else:
                        outputs = self._eager_call(*args, **kwargs)
                finally:
                    global_state.set_global_attribute("autocast_scope", outer)

                # distribution: relayout outputs when the active distribution asks for it
                dist = global_state.get_global_attribute("distribution")
                if dist is not None and not symbolic:
                    outputs = _apply_output_layout(dist, self, outputs)

                if self.activity_regularizer is not None and not symbolic:
                    for out in tree.flatten(outputs):
                        if isinstance(out, torch.Tensor):
                            loss = self.activity_regularizer(out)
                            if out.ndim > 0 and out.shape[0]:
                                loss = loss / out.shape[0]
                            self.add_loss(loss)

            # 7. output masks
            if self._supports_masking:
                prev = _get_mask(first_arg) if first_arg is not None else None
                if prev is not None or not _is_default(type(self), "compute_mask"):
                    mask_arg = kwargs.get("mask", prev) if plan.has_mask else prev
                    self._set_output_mask(first_arg, outputs, mask_arg)
            elif first_arg is not None and _any_mask(first_arg):
                warnings.warn(f"Layer '{self.name}' (of type {self.__class__.__name__}) was passed an input with a mask attached to it. However, this layer "
                              "does not support masking and will therefore destroy the mask information. Downstream layers will not see the mask.")
            return outputs
        finally:
            ctx.training = prev_training if not entered else None
            if entered:
                global_state.set_global_attribute("current_call_ctx", None)

    def _resolve_context_arg(self, name, ctx, plan, kwargs):
        value = kwargs.get(name)
        if value is None:
            value = ctx.get_value(name)
        else:
            ctx.set_value(name, value)
        if name in plan.arg_names or plan.has_var_kw:
            if value is not None:
                kwargs[name] = value
        else:
            kwargs.pop(name, None)

    def _register_call_context_args(self, *names):
        if self._called:
            raise RuntimeError("Cannot add call-context args after the layer has been called.")
        self._call_context_args = self._call_context_args | set(names)

    def _compute_torch_dtype(self):
        return to_torch_dtype(self.compute_dtype)

    def _convert_structure(self, x):
        if type(x) is torch.Tensor or isinstance(x, KerasTensor):
            if self.autocast and type(x) is torch.Tensor and x.dtype.is_floating_point:
                td = self._compute_torch_dtype()
                return x if x.dtype == td or not td.is_floating_point else x.to(td)  # never truncate floats to an integer policy
            return x
        policy = self._resolved_policy()
        autocast, dtype = self.autocast, self.input_dtype
        if isinstance(x, (list, tuple, dict)):
            return tree.map_structure(lambda v: policy.convert_input(v, autocast, dtype) if v is not None else None, x)
        return policy.convert_input(x, autocast, dtype)

    def _eager_call(self, *args, **kwargs):
        if self.quantization_mode is not None and getattr(self, "_is_quantized", False):
            return self.quantized_call(*args, **kwargs)
        if self._remat_mode is not None:
            return self.rematerialized_call(self.call, *args, **kwargs)(*args, **kwargs)
        return self.call(*args, **kwargs)

    def _symbolic_call(self, *args, _implicit=(), **kwargs):
        outputs = self.compute_output_spec(*args, **kwargs)
        recorded = {k: v for k, v in kwargs.items() if k not in _implicit} if _implicit else kwargs
        Node(operation=self, call_args=args, call_kwargs=recorded, outputs=outputs)
        return outputs

    def symbolic_call(self, *args, **kwargs):
        return self._symbolic_call(*args, **kwargs)

    def call(self, *args, **kwargs):
        raise self._not_implemented_error(self.call)

    def quantized_call(self, *args, **kwargs):
        mode = self.quantization_mode
        fn = {"int8": "_int8_call", "float8": "_float8_call", "int4": "_int4_call", "gptq": "_gptq_call", "awq": "_awq_call", "ternary": "_ternary_call"}.get(mode)
        if fn is None or not hasattr(self, fn):
            raise self._quantization_mode_error(mode)
        return getattr(self, fn)(*args, **kwargs)

    def _maybe_build(self, plan, args, kwargs):
        if self.built:
            return
        names = plan.arg_names
        bound = dict(zip(names, args))
        bound.update(kwargs)
        shapes = {}
        for k, v in bound.items():
            if k in ("training", "mask"):
                continue
            s = _shape_structure(v)
            if s is not None:
                shapes[f"{k}_shape"] = s
        if not _is_default(type(self), "build"):
            if plan.build_by_name or len(plan.build_names) > 1:
                kw = {}
                for bn in plan.build_names:
                    if bn in shapes:
                        kw[bn] = shapes[bn]
                    elif bn in ("input_shape", "inputs_shape") and shapes:
                        kw[bn] = next(iter(shapes.values()))
                    else:
                        p = inspect.signature(type(self).build).parameters.get(bn)
                        if p is not None and p.default is inspect.Parameter.empty:
                            raise ValueError(
                                f"For a `build()` method with more than one argument, all arguments should have a "
                                f"`_shape` suffix and match an argument from `call()`. E.g. `build(self, foo_shape, "
                                f"bar_shape)`. For layer '{self.__class__.__name__}', Received `build()` argument "
                                f"`{bn}`, which does not end in `_shape`."
                            )
                self.build(**kw)
            else:
                self.build(next(iter(shapes.values())) if shapes else None)
            self._check_super_called()
            self.built = True
        elif _might_have_unbuilt_state(self):
            # no custom build: build sub-layers by running `call` symbolically
            try:
                spec_args, spec_kwargs = tree.map_structure(_to_spec, (args, kwargs))
                from keras_b200.core.tensor import compute_output_spec

                with _StateUnlock(self):
                    compute_output_spec(self.call, *spec_args, **spec_kwargs)
            except Exception as e:
                if not tree.flatten(self._layers):
                    pass
                else:
                    warnings.warn(
                        f"Layer '{self.name}' looks like it has unbuilt state, but Keras is not able to trace the "
                        "layer `call()` in order to build it automatically. Possible causes:\n1. The `call()` "
                        "method of your layer may be crashing. Try to `__call__()` the layer eagerly on some "
                        "test input first to see if it works. E.g. `x = np.random.random((3, 4)); y = layer(x)`\n"
                        "2. If the `call()` method is correct, then you may need to implement the "
                        "`def build(self, input_shape)` method on your layer. It should create all variables "
                        f"used by the layer (e.g. by calling `layer.build()` on all its children layers).\nException encountered: ''{e}''"
                    )
            self.build(next(iter(shapes.values())) if shapes else None)
        else:
            self._build_shapes_dict = shapes
            self.built = True
            self._lock_state()

    # -- masks ---------------------------------------------------------------------------
    def compute_mask(self, inputs, previous_mask):
        return previous_mask

    @property
    def _call_has_training_arg(self):
        return self._plan.has_training

    @property
    def _call_has_mask_arg(self):
        return self._plan.has_mask

    def _set_output_mask(self, inputs, outputs, previous_mask):
        flat_out = tree.flatten(outputs)
        mask_already = all(getattr(o, "_keras_mask", None) is not None for o in flat_out if o is not None) and bool(flat_out)
        if mask_already:
            return
        try:
            out_masks = self.compute_mask(inputs, previous_mask)
        except Exception:
            return
        if out_masks is None:
            return
        flat_masks = tree.flatten(out_masks)
        for t, m in zip(flat_out, flat_masks):
            if t is not None and m is not None and getattr(t, "_keras_mask", None) is None:
                try:
                    t._keras_mask = m
                except AttributeError:
                    pass

    # -- stateless -----------------------------------------------------------------------
    def stateless_call(self, trainable_variables, non_trainable_variables, *args, return_losses=False, **kwargs):
        self._check_super_called()
        if not self.built:
            raise ValueError(
                f"To call stateless_call, {self.__class__.__name__} must be built (i.e. its variables must have "
                "been already created). You can build it by calling it on some data."
            )
        tv, ntv = self.trainable_variables, self.non_trainable_variables
        if len(trainable_variables) != len(tv):
            raise ValueError(
                "Argument `trainable_variables` must be a list of tensors corresponding 1:1 to "
                f"{self.__class__.__name__}().trainable_variables. Received list with length "
                f"{len(trainable_variables)}, but expected {len(tv)} variables."
            )
        if len(non_trainable_variables) != len(ntv):
            raise ValueError(
                "Argument `non_trainable_variables` must be a list of tensors corresponding 1:1 to "
                f"{self.__class__.__name__}().non_trainable_variables. Received list with length "
                f"{len(non_trainable_variables)}, but expected {len(ntv)} variables."
            )
        mapping = list(zip(tv, trainable_variables)) + list(zip(ntv, non_trainable_variables))
        with StatelessScope(state_mapping=mapping, collect_losses=return_losses) as scope:
            outputs = self.__call__(*args, **kwargs) if self.quantization_mode is None else self.__call__(*args, **kwargs)
            if return_losses:
                losses = self.losses
        new_ntv = []
        for v in ntv:
            nv = scope.get_current_value(v)
            new_ntv.append(nv if nv is not None else v.value)
        if return_losses:
            return outputs, new_ntv, losses
        return outputs, new_ntv

    # -- shape inference -----------------------------------------------------------------
    def compute_output_shape(self, *args, **kwargs):
        raise self._not_implemented_error(
            self.compute_output_shape,
            "Should implement `def compute_output_shape(self, input_shape)`.",
        )

    def compute_output_spec(self, *args, **kwargs):
        if _is_default(type(self), "compute_output_shape"):
            from keras_b200.core.tensor import compute_output_spec

            call_kwargs = dict(kwargs)

            def run(*a, **k):
                return self._eager_call(*a, **k)

            return compute_output_spec(run, *args, **call_kwargs)
        plan = self._plan
        pos_names = plan.arg_names[: plan.n_positional] if plan.n_positional < len(args) else plan.arg_names
        bound = dict(zip(pos_names, args))
        for i in range(len(pos_names), len(args)):
            bound[f"arg{i}"] = args[i]  # call(*args): positional inputs beyond the named parameters
        bound.update(kwargs)
        sig_params = inspect.signature(self.compute_output_shape).parameters
        shape_params = list(sig_params)
        required = [p for p, v in sig_params.items() if v.default is inspect.Parameter.empty and p.endswith("_shape")]
        shapes = {f"{k}_shape": _shape_structure(v) for k, v in bound.items() if _shape_structure(v) is not None and k not in ("training", "mask")}
        if len(shape_params) == 1 or not all(p in shapes for p in required):
            out_shape = self.compute_output_shape(next(iter(shapes.values())))
        else:
            out_shape = self.compute_output_shape(**{p: shapes[p] for p in shape_params if p in shapes})
        dtype = self.compute_dtype
        first = next((v for v in tree.flatten(list(bound.values())) if isinstance(v, KerasTensor)), None)
        if first is not None and "float" not in first.dtype and not self.autocast:
            dtype = first.dtype
        if _is_shape_tuple(out_shape):
            return KerasTensor(out_shape, dtype=dtype)
        return tree.map_shape_structure(lambda s: KerasTensor(s, dtype=dtype), out_shape)

    # -- losses --------------------------------------------------------------------------
    def add_loss(self, loss):
        losses = tree.flatten(loss)
        for x in losses:
            if not isinstance(x, (torch.Tensor, KerasTensor)):
                raise ValueError(f"`add_loss()` can only be called from inside `build()` or `call()`, on a tensor input. Received invalid value: {x}")
        if in_stateless_scope():
            scope = global_state.get_global_attribute("stateless_scope")
            if scope.collect_losses:
                for x in losses:
                    scope.add_loss(x)
                    self._loss_ids.add(id(x))
        else:
            self._losses.extend(losses)

    def _get_own_losses(self):
        if in_stateless_scope():
            scope = global_state.get_global_attribute("stateless_scope")
            return [l for l in scope.losses if id(l) in self._loss_ids]
        return self._losses[:]

    def _get_regularization_losses(self):
        out = []
        for v in self.trainable_weights:
            if v.regularizer is not None:
                out.append(v.regularizer(v.value))
        return out

    @property
    def losses(self):
        if self._losses_override:
            return self._losses_override
        losses = self._get_own_losses()
        for layer in self._flatten_layers(include_self=False):
            losses.extend(layer._get_own_losses())
        weight_losses = self._get_regularization_losses()
        losses.extend(weight_losses)
        return losses

    def _clear_losses(self):
        if in_stateless_scope():
            scope = global_state.get_global_attribute("stateless_scope")
            if scope.collect_losses:
                for x in scope.losses:
                    if id(x) in self._loss_ids:
                        scope.losses.remove(x)
        self._losses.clear()
        self._loss_ids.clear()
        for layer in self._layers:
            layer._clear_losses()

    # -- quantization --------------------------------------------------------------------
    def quantized_build(self, input_shape, mode):
        raise self._not_implemented_error(self.quantized_build)

    def quantize(self, mode=None, type_check=True, config=None):
        raise self._not_implemented_error(self.quantize)

    def _check_quantize_args(self, mode, compute_dtype):
        if not self.built:
            raise ValueError(f"Cannot quantize a layer that isn't yet built. Layer '{self.name}' (of type '{self.__class__.__name__}') is not built yet.")
        if getattr(self, "_is_quantized", False):
            raise ValueError(f"Layer '{self.name}' is already quantized with dtype_policy='{self.dtype_policy.name}'. Received: mode={mode}")
        if mode not in dtype_policies.QUANTIZATION_MODES:
            raise ValueError(f"Invalid quantization mode. Expected one of {dtype_policies.QUANTIZATION_MODES}. Received: mode={mode}")
        if mode == "int8" and compute_dtype == "float16":
            raise ValueError(f"Quantization mode='{mode}' doesn't work well with compute_dtype='float16'. Consider loading model/layer with another dtype policy such as 'mixed_bfloat16' or 'float32' before calling `quantize()`.")

    def _post_quantize(self, mode, **kwargs):
        pass

    def _quantization_mode_error(self, mode):
        return NotImplementedError(f"Invalid quantization mode. Expected one of {dtype_policies.QUANTIZATION_MODES}. Received: quantization_mode={mode}")

    # -- persistence ---------------------------------------------------------------------
    def save_own_variables(self, store):
        for i, v in enumerate(self._trainable_variables + self._non_trainable_variables):
            store[f"{i}"] = v

    def load_own_variables(self, store):
        all_vars = self._trainable_variables + self._non_trainable_variables
        if len(store.keys()) != len(all_vars):
            if len(all_vars) == 0 and not self.built:
                raise ValueError(
                    f"Layer '{self.name}' was never built and thus it doesn't have any variables. However the "
                    f"weights file lists {len(store.keys())} variables for this layer.\nIn most cases, this error "
                    "indicates that either:\n\n1. The layer is owned by a parent layer that implements a `build()` "
                    "method, but calling the parent's `build()` method did NOT create the state of the child "
                    "layer. A `build()` method must create ALL state for the layer, including the state of any "
                    "children layers.\n\n2. You need to implement the `def build_from_config(self, config)` method "
                    f"on layer '{self.name}', to specify how to rebuild it during loading. In this case, you might "
                    "also want to implement the method that generates the build config at saving time, "
                    "`def get_build_config(self)`. The method `build_from_config()` is meant to create the state "
                    "of the layer (i.e. its variables) upon deserialization."
                )
            raise ValueError(
                f"Layer '{self.name}' expected {len(all_vars)} variables, but received {len(store.keys())} "
                f"variables during loading. Expected: {[v.name for v in all_vars]}"
            )
        for i, v in enumerate(all_vars):
            v.assign(store[f"{i}"])

    def save_assets(self, dir_path):
        pass

    def load_assets(self, dir_path):
        pass

    # -- config --------------------------------------------------------------------------
    def get_config(self):
        self._check_super_called()
        base = {"name": self.name, "trainable": self.trainable, "dtype": dtype_policies.serialize(self.dtype_policy)}
        if self.activity_regularizer is not None:
            base["activity_regularizer"] = regularizers.serialize(self.activity_regularizer)
        auto = getattr(self, "_auto_config", None)
        if type(self).get_config is Layer.get_config and type(self).__init__ is not Layer.__init__:
            # no custom get_config: use captured constructor args when serializable
            if auto is None:
                raise NotImplementedError(
                    f"Layer {self.__class__.__name__} was created by passing non-serializable argument values in "
                    "`__init__()`, and therefore the layer must override `get_config()` in order to be serializable."
                )
            from keras_b200.saving import serialization_lib

            cfg = dict(base)
            for k, v in auto.items():
                if k in ("name", "trainable", "dtype", "activity_regularizer"):
                    continue
                try:
                    cfg[k] = serialization_lib.serialize_keras_object(v)
                except Exception:
                    raise NotImplementedError(
                        f"Layer {self.__class__.__name__} was created by passing non-serializable argument values in "
                        f"`__init__()` (argument `{k}`), and therefore the layer must override `get_config()` in "
                        "order to be serializable."
                    )
            return cfg
        return base

    def _not_implemented_error(self, attr, msg=None):
        name = attr.__name__ if callable(attr) else str(attr)
        text = f"Layer {self.__class__.__name__} does not have a `{name}` method implemented."
        if msg:
            text += f" {msg}"
        return NotImplementedError(text)

    def rematerialized_call(self, layer_call, *args, **kwargs):
        from keras_b200.core.remat import wrap_for_mode

        return wrap_for_mode(self, layer_call, self._remat_mode, args, kwargs)

    def __repr__(self):
        return f"<{self.__class__.__name__} name={self.name}, built={self.built}>"

    def __str__(self):
        return self.__repr__()

    def _obj_type(self):
        return "Layer"


class _NoAutocast:
    dtype = None
    torch_dtype = None


_NO_AUTOCAST = None
# Trainer-owned objects that are reported through `Model.metrics` explicitly.
_UNTRACKED_ATTRS = frozenset({"_loss_tracker", "_compile_metrics", "_compile_loss", "_compile_config", "_parallel_engine", "_grad_arena", "_device_stager", "_graphed_step", "history"})
_TRACK_EXTRA = ()


def _late_bind():
    global _TRACK_EXTRA
    from keras_b200.metrics.metric import Metric
    from keras_b200.random.seed_generator import SeedGenerator

    _TRACK_EXTRA = (Metric, SeedGenerator)


def _is_default(cls, name):
    return getattr(cls, name, None) is getattr(Layer, name) or (
        name == "build" and getattr(getattr(cls, name, None), "__wrapped__", None) is getattr(Layer.build, "__wrapped__", Layer.build)
    )


def _might_have_unbuilt_state(layer):
    return any(not l.built for l in layer._layers)


def _only_tensors(x):
    flat = tree.flatten(x)
    return bool(flat) and all(isinstance(v, _TENSOR_TYPES) or v is None for v in flat)


def _get_mask(x):
    if isinstance(x, (list, tuple, dict)):
        masks = tree.map_structure(lambda v: getattr(v, "_keras_mask", None), x)
        return masks if any(m is not None for m in tree.flatten(masks)) else None
    return getattr(x, "_keras_mask", None)


def _any_mask(x):
    return _get_mask(x) is not None


def _is_shape_tuple(s):
    return isinstance(s, (list, tuple)) and all(d is None or isinstance(d, int) for d in s)


def _shape_structure(v):
    if isinstance(v, _TENSOR_TYPES):
        return tuple(v.shape)
    if isinstance(v, (list, tuple, dict)):
        flat = tree.flatten(v)
        if flat and all(isinstance(e, _TENSOR_TYPES) or e is None for e in flat):
            return tree.map_structure(lambda e: tuple(e.shape) if e is not None else None, v)
    return None


def _to_spec(x):
    if isinstance(x, torch.Tensor):
        from keras_b200.core.dtypes import standardize_dtype as sd

        return KerasTensor(tuple(x.shape), dtype=sd(x.dtype))
    return x


def _current_remat_mode():
    from keras_b200.core.remat import get_current_remat_mode

    return get_current_remat_mode()


def _apply_output_layout(dist, layer, outputs):
    try:
        path = layer.path
        if path is None:
            return outputs
        layout = dist.get_tensor_layout(path + "/output") if hasattr(dist, "get_tensor_layout") else None
        if layout is None:
            return outputs
        from keras_b200.distribution import distribution_lib

        return distribution_lib.distribute_tensor(outputs, layout)
    except Exception:
        return outputs
