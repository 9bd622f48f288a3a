"""``keras.callbacks``."""

from keras_b200.callbacks.base import Callback, CallbackList  # noqa: F401
from keras_b200.callbacks.watch import MonitorCallback  # noqa: F401
from keras_b200.callbacks.reporting import CSVLogger, History, LambdaCallback, ProgbarLogger, RemoteMonitor  # noqa: F401
from keras_b200.callbacks.training_control import EarlyStopping, LearningRateScheduler, ReduceLROnPlateau, TerminateOnNaN  # noqa: F401
from keras_b200.callbacks.checkpointing import BackupAndRestore, ModelCheckpoint, SwapEMAWeights  # noqa: F401
from keras_b200.callbacks.tensorboard import TensorBoard  # noqa: F401
from keras_b200.callbacks.orbax_checkpoint import OrbaxCheckpoint  # noqa: F401
from keras_b200.callbacks.failure_detection import FailureDetection  # noqa: F401
