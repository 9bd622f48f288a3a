"""keras_b200: a deep-learning framework with the Keras 3 API, built for NVIDIA B200.

``import keras_b200 as keras`` gives the public namespace (layers, models, ops, optimizers, losses,
metrics, callbacks, distribution, saving, …).  Tensors are PyTorch tensors; hot paths run
hand-written sm_100a kernels (``keras_b200.kernels``) and NVLink collectives fused with their
compute (``keras_b200.parallel``).
"""

import torch as _torch  # noqa: F401  (imported first: initialises CUDA runtime state once)

from keras_b200.version import __version__, version  # noqa: F401
from keras_b200.core import config as _core_config  # noqa: F401
from keras_b200 import tree  # noqa: F401
from keras_b200 import ops  # noqa: F401
from keras_b200 import random  # noqa: F401
from keras_b200 import initializers, regularizers, constraints, activations  # noqa: F401
from keras_b200 import dtype_policies, quantizers  # noqa: F401
from keras_b200 import losses, metrics  # noqa: F401
from keras_b200 import layers  # noqa: F401
from keras_b200 import optimizers  # noqa: F401
from keras_b200 import models  # noqa: F401
from keras_b200 import callbacks  # noqa: F401
from keras_b200 import saving  # noqa: F401
from keras_b200 import distribution  # noqa: F401
from keras_b200 import config  # noqa: F401
from keras_b200 import utils  # noqa: F401
from keras_b200 import mixed_precision  # noqa: F401
from keras_b200 import backend  # noqa: F401

from keras_b200.core.variables import Variable  # noqa: F401
from keras_b200.core.keras_tensor import KerasTensor  # noqa: F401
from keras_b200.core.scopes import StatelessScope, SymbolicScope, name_scope  # noqa: F401
from keras_b200.core.remat import RematScope, remat  # noqa: F401
from keras_b200.core.tensor import device_scope as device  # noqa: F401
from keras_b200.dtype_policies import DTypePolicy, FloatDTypePolicy  # noqa: F401
from keras_b200.initializers import Initializer  # noqa: F401
from keras_b200.layers import Input, InputSpec, Layer  # noqa: F401
from keras_b200.losses import Loss  # noqa: F401
from keras_b200.metrics import Metric  # noqa: F401
from keras_b200.models import Model, Sequential  # noqa: F401
from keras_b200.ops.function import Function  # noqa: F401
from keras_b200.ops.operation import Operation  # noqa: F401
from keras_b200.optimizers import Optimizer  # noqa: F401
from keras_b200.quantizers import Quantizer  # noqa: F401
from keras_b200.regularizers import Regularizer  # noqa: F401


def __getattr__(name):
    import importlib

    if name in ("applications", "datasets", "export", "legacy", "preprocessing", "visualization", "wrappers", "distillation", "parallel", "kernels", "testing"):
        return importlib.import_module(f"keras_b200.{name}")
    raise AttributeError(f"module 'keras_b200' has no attribute {name!r}")
