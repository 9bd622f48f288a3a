"""``keras.optimizers.legacy.*``: placeholders that explain the removal (keras/src/optimizers/__init__.py:107-121)."""

from keras_b200.core.export_registry import keras_export


@keras_export(["keras.optimizers.legacy.Adagrad", "keras.optimizers.legacy.Adam", "keras.optimizers.legacy.Ftrl", "keras.optimizers.legacy.RMSprop",
               "keras.optimizers.legacy.SGD", "keras.optimizers.legacy.Optimizer"])
class LegacyOptimizerWarning:
    def __init__(self, *args, **kwargs):
        raise ImportError("`keras.optimizers.legacy` is not supported in Keras 3. When using `tf.keras`, to continue using a "
                          "`tf.keras.optimizers.legacy` optimizer, you can install the `tf_keras` package (Keras 2) and set the environment "
                          "variable `TF_USE_LEGACY_KERAS=True` to configure TensorFlow to use `tf_keras` when accessing `tf.keras`.")


Adagrad = Adam = Ftrl = RMSprop = SGD = Optimizer = LegacyOptimizerWarning
