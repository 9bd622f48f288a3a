from keras_b200.dtype_policies import DTypePolicy, dtype_policy, set_dtype_policy  # noqa: F401
from keras_b200.optimizers.loss_scale_optimizer import LossScaleOptimizer  # noqa: F401

Policy = DTypePolicy
global_policy = dtype_policy
set_global_policy = set_dtype_policy
