"""Re-export of the ``KerasSaveable`` base (keras/src/saving/keras_saveable.py)."""

from keras_b200.ops.operation import KerasSaveable  # noqa: F401
