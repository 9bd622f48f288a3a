"""Scoped global state: name scopes, stateless scope, symbolic scope.

Reference behaviour: keras/src/backend/common/name_scope.py:4-74,
stateless_scope.py:6-105, symbolic_scope.py.
"""

from keras_b200.core import global_state
from keras_b200.core.export_registry import keras_export


@keras_export("keras.name_scope")
class name_scope:
    """Context manager that prefixes the ``path`` of variables created inside it."""

    def __init__(self, name, caller=None, deduplicate=False, override_parent=None):
        if not isinstance(name, str) or "/" in name:
            raise ValueError(
                "Argument `name` must be a string and cannot contain character `/`. "
                f"Received: name={name}"
            )
        self.name = name
        self.caller = caller
        self.deduplicate = deduplicate
        self.override_parent = override_parent
        if override_parent is None and deduplicate and getattr(caller, "_parent_path", None):
            self.override_parent = caller._parent_path
        self._pop = False

    def __enter__(self):
        stack = global_state.get_global_attribute("name_scope_stack", default=[], set_to_default=True)
        if self.deduplicate and stack:
            top = stack[-1]
            if top.caller is not None and top.caller is self.caller and top.name == self.name:
                return self
        stack.append(self)
        self._pop = True
        return self

    def __exit__(self, *exc):
        if self._pop:
            stack = global_state.get_global_attribute("name_scope_stack")
            if stack:
                stack.pop()
            self._pop = False


def current_path():
    stack = global_state.get_global_attribute("name_scope_stack")
    if not stack:
        return ""
    parts = []
    for entry in stack:
        if entry.override_parent is not None:
            parts = [p for p in entry.override_parent.split("/") if p]
        parts.append(entry.name)
    return "/".join(parts)


@keras_export("keras.StatelessScope")
class StatelessScope:
    """Run code without mutating variables: reads come from ``state_mapping``, writes are
    collected and can be read back with ``get_current_value``."""

    def __init__(self, state_mapping=None, collect_losses=False, initialize_variables=True):
        from keras_b200.core.variables import Variable

        self.collect_losses = collect_losses
        self.initialize_variables = initialize_variables
        self.losses = []
        self.state_mapping = {}
        for k, v in state_mapping or {}:
            if not isinstance(k, Variable):
                raise ValueError(
                    "Invalid reference variable in StatelessScope: all keys in argument "
                    f"`mapping` must be Variable instances. Received instead: {k}"
                )
            if isinstance(v, Variable):
                v = v.value
            from keras_b200.core.tensor import convert_to_tensor

            v = convert_to_tensor(v, dtype=k.dtype)
            if tuple(k.shape) != tuple(v.shape):
                raise ValueError(
                    "Invalid variable value in StatelessScope: all values in argument `mapping` "
                    "must be tensors with a shape that matches the corresponding variable shape. "
                    f"For variable {k}, received invalid value {v} with shape {tuple(v.shape)}."
                )
            self.state_mapping[id(k)] = v

    def __enter__(self):
        self._outer = global_state.get_global_attribute("stateless_scope")
        global_state.set_global_attribute("stateless_scope", self)
        return self

    def add_loss(self, loss):
        self.losses.append(loss)

    def add_update(self, update):
        variable, value = update
        self.state_mapping[id(variable)] = value

    def get_current_value(self, variable):
        return self.state_mapping.get(id(variable))

    def __exit__(self, *exc):
        global_state.set_global_attribute("stateless_scope", self._outer)
        if self._outer is None and self.initialize_variables:
            from keras_b200.core.variables import initialize_all_variables

            initialize_all_variables()


def in_stateless_scope():
    return global_state.get_global_attribute("stateless_scope") is not None


def get_stateless_scope():
    return global_state.get_global_attribute("stateless_scope")


@keras_export("keras.SymbolicScope")
class SymbolicScope:
    """Marks code that runs on placeholder (meta) tensors to infer output shapes."""

    def __enter__(self):
        self._outer = global_state.get_global_attribute("symbolic_scope")
        global_state.set_global_attribute("symbolic_scope", self)
        return self

    def __exit__(self, *exc):
        global_state.set_global_attribute("symbolic_scope", self._outer)


def in_symbolic_scope():
    return global_state.get_global_attribute("symbolic_scope") is not None
