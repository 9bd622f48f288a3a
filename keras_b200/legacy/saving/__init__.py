from keras_b200.legacy.saving.legacy_serialization import deserialize_keras_object, serialize_keras_object  # noqa: F401
