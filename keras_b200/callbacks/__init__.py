from keras_b200.callbacks.callbacks import (  # noqa: F401
    BackupAndRestore, Callback, CallbackList, CSVLogger, EarlyStopping, History, LambdaCallback, LearningRateScheduler,
    ModelCheckpoint, MonitorCallback, ProgbarLogger, ReduceLROnPlateau, RemoteMonitor, SwapEMAWeights, TerminateOnNaN,
)
from keras_b200.callbacks.tensorboard import TensorBoard  # noqa: F401
from keras_b200.callbacks.orbax_checkpoint import OrbaxCheckpoint  # noqa: F401
from keras_b200.callbacks.failure_detection import FailureDetection  # noqa: F401
