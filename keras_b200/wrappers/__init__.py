from keras_b200.wrappers.sklearn_wrapper import SKLearnClassifier, SKLearnRegressor, SKLearnTransformer  # noqa: F401
