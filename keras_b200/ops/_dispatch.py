"""Glue that turns a plain eager function into a public op.

A public op (a) runs its torch implementation when called on concrete values, and (b) records a
graph ``Node`` when any argument is a ``KerasTensor``, inferring the output spec by tracing the
same implementation on the meta device.  The reference writes one ``Operation`` subclass with a
hand-written ``compute_output_spec`` per op (keras/src/ops/numpy.py etc.); tracing the single
implementation keeps eager and symbolic results consistent by construction.
"""

import functools

from keras_b200.core.export_registry import keras_export
from keras_b200.core.keras_tensor import any_symbolic_tensors
from keras_b200.ops.operation import Operation


def _camel(name):
    return "".join(p.capitalize() for p in name.split("_"))


_OP_CLASSES = {}


class FunctionOp(Operation):
    """Operation whose behaviour is a module-level function of ``keras.ops``."""

    op_name = None
    fn = None

    def __init__(self, name=None):
        super().__init__(name=name)

    def call(self, *args, **kwargs):
        return type(self).fn(*args, **kwargs)

    def get_config(self):
        return {"name": self.name}

    @classmethod
    def from_config(cls, config):
        return cls(name=config.get("name"))


def op_class_for(fn_name):
    return _OP_CLASSES.get(fn_name)


def make_op(*export_names):
    """Decorator: register ``fn`` as a public op under the given ``keras.ops.*`` names."""

    def deco(fn):
        fn_name = fn.__name__
        cls = type(_camel(fn_name), (FunctionOp,), {"fn": staticmethod(fn), "op_name": fn_name})
        cls.__module__ = "keras_b200.ops"
        _OP_CLASSES[fn_name] = cls
        # Graphs written by reference Keras name the op class from a private module
        # (e.g. module "keras.src.ops.numpy", class "Add"); index by class name for loading.
        keras_export(f"keras.ops.{_camel(fn_name)}__op")(cls)

        @functools.wraps(fn)
        def public(*args, **kwargs):
            if any_symbolic_tensors(args, kwargs):
                return cls()(*args, **kwargs)
            return fn(*args, **kwargs)

        public._eager = fn
        public._op_class = cls
        if export_names:
            keras_export(list(export_names))(public)
        return public

    return deco


def op(namespace=None, also=()):
    """Shorthand: ``@op("nn")`` exports as ``keras.ops.<name>`` and ``keras.ops.nn.<name>``."""

    def deco(fn):
        names = [f"keras.ops.{fn.__name__}"]
        if namespace:
            names.append(f"keras.ops.{namespace}.{fn.__name__}")
        names.extend(also)
        return make_op(*names)(fn)

    return deco
