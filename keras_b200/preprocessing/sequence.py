"""``keras.preprocessing.sequence`` (keras/api/preprocessing/sequence/__init__.py)."""

from keras_b200.utils.misc_utils import pad_sequences  # noqa: F401
