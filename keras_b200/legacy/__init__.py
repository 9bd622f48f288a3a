"""``keras.legacy``: Keras 2 file formats and serialisation."""

from keras_b200.legacy import saving  # noqa: F401
