from keras_b200.distillation.distillation_loss import DistillationLoss, FeatureDistillation, LogitsDistillation  # noqa: F401
from keras_b200.distillation.distiller import Distiller  # noqa: F401
