"""``Distiller``: trains a student against a frozen teacher with a weighted sum of the student's own loss and one
or more distillation losses (keras/src/distillation/distiller.py)."""

from keras_b200 import metrics as metrics_module
from keras_b200 import ops, tree
from keras_b200.core.export_registry import keras_export
from keras_b200.distillation.distillation_loss import _as_loss_fn
from keras_b200.models.model import Model
from keras_b200.models.sequential import Sequential
from keras_b200.saving import serialization_lib


@keras_export("keras.distillation.Distiller")
class Distiller(Model):
    def __init__(self, teacher, student, distillation_losses, distillation_loss_weights=None, student_loss_weight=0.5, name="distiller", **kwargs):
        super().__init__(name=name, **kwargs)
        self._validate_models(teacher, student)
        self.teacher, self.student = teacher, student
        if not isinstance(student_loss_weight, (int, float)):
            raise ValueError(f"student_loss_weight must be a number, got {type(student_loss_weight)}")
        if student_loss_weight < 0.0 or student_loss_weight > 1.0:
            raise ValueError(f"student_loss_weight must be between 0.0 and 1.0, got {student_loss_weight}")
        self.student_loss_weight = student_loss_weight
        if distillation_losses is None:
            raise ValueError("'distillation_losses' cannot be `None`. Provide a distillation loss (e.g., LogitsDistillation or FeatureDistillation) or a list of distillation losses.")
        if not isinstance(distillation_losses, (list, tuple)):
            self.distillation_losses, self.distillation_loss_weights = [distillation_losses], [1.0]
        else:
            self.distillation_losses = list(distillation_losses)
            if distillation_loss_weights is None:
                self.distillation_loss_weights = [1.0] * len(distillation_losses)
            else:
                if len(distillation_loss_weights) != len(distillation_losses):
                    raise ValueError(f"Number of distillation_loss_weights ({len(distillation_loss_weights)}) must match number of distillation_losses ({len(distillation_losses)})")
                self.distillation_loss_weights = list(distillation_loss_weights)
        for dl in self.distillation_losses:
            dl.validate_model_compatibility(teacher, student)
        self._create_multi_feature_extractors()
        self.teacher.trainable = False
        self.student_loss_tracker = metrics_module.Mean(name="student_loss")
        self.distillation_loss_tracker = metrics_module.Mean(name="distillation_loss")
        self.total_loss_tracker = metrics_module.Mean(name="total_loss")

    # -- validation ----------------------------------------------------------------------
    def _validate_models(self, teacher, student):
        if not isinstance(teacher, Model):
            raise ValueError(f"Teacher must be a keras.Model, got {type(teacher)}")
        if not isinstance(student, Model):
            raise ValueError(f"Student must be a keras.Model, got {type(student)}")
        for attr, ctx in (("inputs", "input"), ("outputs", "output")):
            t, s = getattr(teacher, attr, None), getattr(student, attr, None)
            if t is None or s is None:
                continue
            tree.map_structure(lambda a, b: self._assert_shapes_are_compatible(a.shape, b.shape, ctx), t, s)
            tree.map_structure(lambda a, b: self._assert_same_dtype(a.dtype, b.dtype, ctx), t, s)

    def _assert_shapes_are_compatible(self, shape1, shape2, context):
        if len(shape1) != len(shape2):
            raise ValueError(f"Teacher and student {context} shapes have different dimensions. Teacher: {shape1}, Student: {shape2}.")
        for d1, d2 in zip(shape1, shape2):
            if d1 is not None and d2 is not None and d1 != d2:
                raise ValueError(f"Teacher and student {context} shapes are incompatible. Teacher: {shape1}, Student: {shape2}. All dimensions must match.")

    def _assert_same_dtype(self, teacher_dtype, student_dtype, context):
        if teacher_dtype != student_dtype:
            raise ValueError(f"Teacher and student {context} dtypes must match. Teacher: {teacher_dtype}, Student: {student_dtype}.")

    # -- feature extraction --------------------------------------------------------------
    def _create_multi_feature_extractors(self):
        t_names, s_names = [], []
        for dl in self.distillation_losses:
            for attr, names in (("teacher_layer_name", t_names), ("student_layer_name", s_names)):
                n = getattr(dl, attr, None)
                if n and n not in names:
                    names.append(n)
        self._teacher_feature_extractor = self._create_feature_extractor(self.teacher, t_names)
        self._student_feature_extractor = self._create_feature_extractor(self.student, s_names)

    def _create_feature_extractor(self, model, layer_names):
        if not layer_names:
            return None
        if getattr(model, "inputs", None) is None:
            raise ValueError(f"Cannot create feature extractor for {model.name}. The model has no symbolic inputs attribute.")
        final_output = model.layers[-1].output if isinstance(model, Sequential) else model.output
        outputs = {"final_output": final_output}
        for n in layer_names:
            outputs[n] = model.get_layer(name=n).output
        return Model(inputs=model.inputs, outputs=outputs, name=f"{model.name}_multi_feature_extractor")

    def _extract_all_teacher_features(self, x):
        if self._teacher_feature_extractor is not None:
            return self._teacher_feature_extractor(x, training=False)
        return {"final_output": self.teacher(x, training=False)}

    def _extract_all_student_features(self, x, y_pred):
        if self._student_feature_extractor is not None:
            return self._student_feature_extractor(x, training=True)
        return {"final_output": y_pred}

    def _get_distillation_loss_features(self, distillation_loss, all_features, is_teacher):
        name = (distillation_loss.teacher_layer_name if is_teacher else distillation_loss.student_layer_name) or "final_output"
        if name not in all_features:
            raise ValueError(f"Layer '{name}' not found in extracted features. Available: {list(all_features.keys())}")
        return all_features[name]

    # -- training ------------------------------------------------------------------------
    def compile(self, optimizer="adam", loss=None, metrics=None, **kwargs):
        if loss is None:
            raise ValueError("'loss' cannot be `None`.")
        self._student_loss = tree.map_structure(_as_loss_fn, loss)
        self._student_loss_for_serialization = loss
        if metrics is not None and not isinstance(metrics, (list, tuple)):
            raise ValueError(f"metrics must be a list or tuple, got {type(metrics)}")
        super().compile(optimizer=optimizer, loss=None, metrics=metrics, **kwargs)

    def call(self, inputs, training=None, **kwargs):
        return self.student(inputs, training=training, **kwargs)

    def compute_loss(self, x=None, y=None, y_pred=None, sample_weight=None, training=True):
        import torch

        if y_pred is None:
            y_pred = self(x, training=training)
        student_loss = 0.0
        if self.student_loss_weight > 0.0 and y is not None:
            values = tree.flatten(tree.map_structure(lambda l, o, p: l(o, p), self._student_loss, y, y_pred))
            student_loss = ops.sum(ops.stack(values)) if len(values) > 1 else values[0]
            if hasattr(student_loss, "shape") and len(student_loss.shape) > 0:
                student_loss = ops.mean(student_loss)
        distillation_loss = 0.0
        if self.student_loss_weight < 1.0:
            with torch.no_grad():
                teacher_features = self._extract_all_teacher_features(x)
            student_features = self._extract_all_student_features(x, y_pred)
            for fn, weight in zip(self.distillation_losses, self.distillation_loss_weights):
                if getattr(fn, "teacher_layer_name", None) is not None:
                    try:
                        t_out = self._get_distillation_loss_features(fn, teacher_features, is_teacher=True)
                        s_out = self._get_distillation_loss_features(fn, student_features, is_teacher=False)
                    except ValueError as e:
                        raise RuntimeError(f"Failed to extract features for {type(fn).__name__} targeting teacher layer '{fn.teacher_layer_name}' "
                                           f"and student layer '{fn.student_layer_name}'. Original error: {e}") from e
                else:
                    t_out, s_out = teacher_features["final_output"], y_pred
                fn.validate_outputs(t_out, s_out)
                current = fn.compute_loss(t_out, s_out)
                if hasattr(current, "shape") and len(current.shape) > 0:
                    raise ValueError(f"Distillation loss {fn.__class__.__name__} returned a non-scalar loss with shape {current.shape}. The compute_loss method must return a scalar tensor.")
                distillation_loss = ops.add(distillation_loss, ops.multiply(weight, current))
        total = ops.add(ops.multiply(self.student_loss_weight, student_loss), ops.multiply(1.0 - self.student_loss_weight, distillation_loss))
        self.student_loss_tracker.update_state(student_loss)
        self.distillation_loss_tracker.update_state(distillation_loss)
        self.total_loss_tracker.update_state(total)
        return total

    def reset_metrics(self):
        super().reset_metrics()
        self.student_loss_tracker.reset_state()
        self.distillation_loss_tracker.reset_state()
        self.total_loss_tracker.reset_state()

    def get_config(self):
        cfg = super().get_config()
        cfg.update({"teacher": serialization_lib.serialize_keras_object(self.teacher), "student": serialization_lib.serialize_keras_object(self.student),
                    "distillation_losses": [serialization_lib.serialize_keras_object(d) for d in self.distillation_losses],
                    "distillation_loss_weights": self.distillation_loss_weights, "student_loss_weight": self.student_loss_weight})
        return cfg

    @classmethod
    def from_config(cls, config):
        config = config.copy()
        config["teacher"] = serialization_lib.deserialize_keras_object(config["teacher"])
        config["student"] = serialization_lib.deserialize_keras_object(config["student"])
        config["distillation_losses"] = [serialization_lib.deserialize_keras_object(d) for d in config["distillation_losses"]]
        return cls(**config)
