"""Distillation objectives: ``LogitsDistillation`` (temperature-softened outputs) and ``FeatureDistillation``
(intermediate activations), keras/src/distillation/distillation_loss.py."""

from keras_b200 import losses, ops, tree
from keras_b200.core.export_registry import keras_export
from keras_b200.saving import serialization_lib


def _as_loss_fn(item):
    if item is None:
        return None
    if isinstance(item, str):
        fn = losses.get(item)
        if fn is None:
            raise ValueError(f"Unknown loss function: '{item}'.")
        return fn
    return item


def _sum_of(loss_values):
    flat = [ops.convert_to_tensor(v, dtype="float32") if not hasattr(v, "shape") else v for v in tree.flatten(loss_values)]
    return ops.sum(ops.stack(flat))


@keras_export("keras.distillation.DistillationLoss")
class DistillationLoss:
    """Base class: ``compute_loss(teacher_outputs, student_outputs) -> scalar``."""

    def compute_loss(self, teacher_outputs, student_outputs, **kwargs):
        raise NotImplementedError("Subclasses must implement compute_loss")

    def validate_outputs(self, teacher_outputs, student_outputs):
        tree.assert_same_structure(teacher_outputs, student_outputs)

    def validate_model_compatibility(self, teacher, student):
        pass


@keras_export("keras.distillation.FeatureDistillation")
class FeatureDistillation(DistillationLoss):
    def __init__(self, loss="mse", teacher_layer_name=None, student_layer_name=None):
        self.teacher_layer_name, self.student_layer_name = teacher_layer_name, student_layer_name
        self.loss = tree.map_structure(_as_loss_fn, loss)
        if all(l is None for l in tree.flatten(self.loss)):
            raise ValueError("The `loss` argument in `FeatureDistillation` must contain at least one non-`None` value.")

    def validate_model_compatibility(self, teacher, student):
        if self.teacher_layer_name is not None or self.student_layer_name is not None:
            sub = [n for n, m in (("teacher", teacher), ("student", student)) if getattr(m, "inputs", None) is None]
            if sub:
                raise ValueError(f"FeatureDistillation with specific layer names requires Functional or Sequential models. The {' and '.join(sub)} "
                                 "model(s) appear to be subclassed (no symbolic inputs/outputs). Either use Functional/Sequential models, or use "
                                 "FeatureDistillation without layer names (to distill final outputs only), or use LogitsDistillation instead.")
        for which, model, name in (("teacher", teacher, self.teacher_layer_name), ("student", student, self.student_layer_name)):
            if name is not None:
                try:
                    model.get_layer(name=name)
                except ValueError as e:
                    raise ValueError(f"In {which} model: {e}")

    def validate_outputs(self, teacher_outputs, student_outputs):
        super().validate_outputs(teacher_outputs, student_outputs)
        try:
            tree.assert_same_structure(self.loss, teacher_outputs)
        except ValueError as e:
            raise ValueError(f"Loss structure mismatch. Loss structure: {self.loss}, Output structure: {teacher_outputs}. Error: {e}")

    def compute_loss(self, teacher_outputs, student_outputs, **kwargs):
        def apply(fn, t, s):
            return 0.0 if fn is None else ops.mean(fn(t, s))

        return _sum_of(tree.map_structure(apply, self.loss, teacher_outputs, student_outputs))

    def get_config(self):
        return {"loss": losses.serialize(self.loss), "teacher_layer_name": self.teacher_layer_name, "student_layer_name": self.student_layer_name}

    @classmethod
    def from_config(cls, config):
        config = config.copy()
        config["loss"] = losses.deserialize(config["loss"])
        return cls(**config)


@keras_export("keras.distillation.LogitsDistillation")
class LogitsDistillation(DistillationLoss):
    def __init__(self, temperature=3.0, loss="kl_divergence"):
        self.temperature = temperature
        self.loss = tree.map_structure(_as_loss_fn, loss)
        if all(l is None for l in tree.flatten(self.loss)):
            raise ValueError("At least one loss must be non-`None`.")
        if not isinstance(temperature, (int, float)):
            raise ValueError(f"temperature must be a number, got {type(temperature)}")
        if temperature <= 0.0:
            raise ValueError("temperature must be positive.")

    def compute_loss(self, teacher_outputs, student_outputs, **kwargs):
        t_scaled = tree.map_structure(lambda x: ops.divide(x, self.temperature), teacher_outputs)
        s_scaled = tree.map_structure(lambda x: ops.divide(x, self.temperature), student_outputs)

        def apply(fn, t, s):
            if fn is None:
                return 0.0
            if isinstance(fn, losses.KLDivergence) or getattr(fn, "__name__", "") in ("kl_divergence", "kld"):
                value = ops.mean(fn(ops.softmax(t, axis=-1), ops.softmax(s, axis=-1)))
                return value * (self.temperature ** 2)
            return ops.mean(fn(t, s))

        return _sum_of(tree.map_structure(apply, self.loss, t_scaled, s_scaled))

    def get_config(self):
        return {"temperature": self.temperature, "loss": serialization_lib.serialize_keras_object(self.loss)}

    @classmethod
    def from_config(cls, config):
        config = config.copy()
        config["loss"] = losses.deserialize(config["loss"])
        return cls(**config)
