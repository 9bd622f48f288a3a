"""scikit-learn estimator wrappers around models: ``SKLearnClassifier``, ``SKLearnRegressor``, ``SKLearnTransformer``
(keras/src/wrappers/sklearn_wrapper.py).  The wrapped ``model`` is either a compiled model (cloned per ``fit``
unless ``warm_start``) or a callable ``model(X, y, **model_kwargs) -> compiled model``."""

import copy

import numpy as np

from keras_b200.core.export_registry import keras_export
from keras_b200.models.cloning import clone_model
from keras_b200.models.model import Model

try:
    import sklearn
    import sklearn.pipeline
    import sklearn.preprocessing
    from sklearn.base import BaseEstimator, ClassifierMixin, RegressorMixin, TransformerMixin
except ImportError:  # pragma: no cover
    sklearn = None

    class BaseEstimator:
        pass

    ClassifierMixin = RegressorMixin = TransformerMixin = BaseEstimator


def _need_sklearn(symbol):
    if sklearn is None:
        raise ImportError(f"{symbol} requires `scikit-learn` to be installed. Run `pip install scikit-learn` to install it.")


def _validate(estimator, *args, **kwargs):
    try:
        from sklearn.utils.validation import validate_data
    except ImportError:
        return estimator._validate_data(*args, **kwargs)
    return validate_data(estimator, *args, **kwargs)


def _target_type(y):
    from sklearn.utils.multiclass import type_of_target

    kind = type_of_target(y)
    if kind == "unknown":
        raise ValueError(f"Unknown label type for data: {y!r}")
    return kind


def _routing_enabled():
    if sklearn is None:
        return False
    return bool(sklearn.get_config().get("enable_metadata_routing", False))


class TargetReshaper(TransformerMixin, BaseEstimator):
    """1-D targets become a column for the model and are squeezed back on the way out."""

    def fit(self, y):
        self.ndim_ = y.ndim
        return self

    def transform(self, y):
        return y.reshape(-1, 1) if y.ndim == 1 else y

    def inverse_transform(self, y):
        from sklearn.utils.validation import check_is_fitted

        check_is_fitted(self)
        if self.ndim_ == 1 and y.ndim == 2:
            return np.squeeze(y, axis=1)
        return y


class SKLBase(BaseEstimator):
    def __init__(self, model, warm_start=False, model_kwargs=None, fit_kwargs=None):
        _need_sklearn(self.__class__.__name__)
        self.model = model
        self.warm_start = warm_start
        self.model_kwargs = model_kwargs
        self.fit_kwargs = fit_kwargs

    def _more_tags(self):
        return {"non_deterministic": True}

    def __sklearn_tags__(self):
        tags = super().__sklearn_tags__()
        tags.non_deterministic = True
        return tags

    def __sklearn_clone__(self):
        model = self.model if callable(self.model) and not isinstance(self.model, Model) else copy.deepcopy(self.model)
        return type(self)(model=model, warm_start=self.warm_start, model_kwargs=self.model_kwargs)

    @property
    def epoch_(self):
        return getattr(self, "history_", {}).get("epoch", 0) if isinstance(getattr(self, "history_", None), dict) else 0

    def set_fit_request(self, **kwargs):
        if not _routing_enabled():
            raise RuntimeError("This method is only available when metadata routing is enabled. You can enable it using sklearn.set_config(enable_metadata_routing=True).")
        self._metadata_request = sklearn.utils.metadata_routing.MetadataRequest(owner=self.__class__.__name__)
        for param, alias in kwargs.items():
            self._metadata_request.score.add_request(param=param, alias=alias)
        return self

    def _get_model(self, X, y):
        if self.warm_start and hasattr(self, "model_"):
            return self.model_
        if isinstance(self.model, Model):
            if self.warm_start:
                return self.model
            clone = clone_model(self.model)
            if self.model.compiled:
                clone.compile_from_config(self.model.get_compile_config())
            return clone
        return self.model(X=X, y=y, **(self.model_kwargs or {}))

    def fit(self, X, y, **kwargs):
        X, y = _validate(self, X, y)
        y = self._process_target(y, reset=True)
        model = self._get_model(X, y)
        if not model.compiled or not model.loss or not model.optimizer:
            raise RuntimeError("Given model needs to be compiled, and have a loss and an optimizer.")
        fit_kwargs = dict(self.fit_kwargs or {})
        fit_kwargs.update(kwargs)
        self.history_ = model.fit(X, y, **fit_kwargs)
        self.model_ = model
        return self

    def predict(self, X):
        from sklearn.utils.validation import check_is_fitted

        check_is_fitted(self)
        X = _validate(self, X, reset=False)
        return self._reverse_process_target(self.model_.predict(X, verbose=0))

    def _process_target(self, y, reset=False):
        _target_type(y)
        if reset:
            self._target_encoder = TargetReshaper().fit(y)
        return self._target_encoder.transform(y)

    def _reverse_process_target(self, y):
        return self._target_encoder.inverse_transform(y)


@keras_export("keras.wrappers.SKLearnClassifier")
class SKLearnClassifier(ClassifierMixin, SKLBase):
    def decision_function(self, X):
        from sklearn.utils.validation import check_is_fitted

        check_is_fitted(self)
        X = _validate(self, X, reset=False)
        return self.model_.predict(X, verbose=0)

    def _process_target(self, y, reset=False):
        kind = _target_type(y)
        if kind not in ["binary", "multiclass"]:
            raise ValueError(f"Only binary and multiclass target types are supported. Target type: {kind}")
        if reset:
            self._target_encoder = sklearn.pipeline.make_pipeline(TargetReshaper(), sklearn.preprocessing.OneHotEncoder(sparse_output=False)).fit(y)
            self.classes_ = np.unique(y)
            if len(self.classes_) == 1:
                raise ValueError("Classifier can't train when only one class is present.")
        return self._target_encoder.transform(y)

    def _more_tags(self):
        return {"poor_score": True}

    def __sklearn_tags__(self):
        tags = super().__sklearn_tags__()
        tags.classifier_tags.poor_score = True
        return tags


@keras_export("keras.wrappers.SKLearnRegressor")
class SKLearnRegressor(RegressorMixin, SKLBase):
    def _more_tags(self):
        return {"poor_score": True}

    def __sklearn_tags__(self):
        tags = super().__sklearn_tags__()
        tags.regressor_tags.poor_score = True
        return tags


@keras_export("keras.wrappers.SKLearnTransformer")
class SKLearnTransformer(TransformerMixin, SKLBase):
    def transform(self, X):
        from sklearn.utils.validation import check_is_fitted

        check_is_fitted(self)
        X = _validate(self, X, reset=False)
        return self.model_.predict(X, verbose=0)

    def _more_tags(self):
        return {"preserves_dtype": []}

    def __sklearn_tags__(self):
        tags = super().__sklearn_tags__()
        tags.transformer_tags.preserves_dtype = []
        return tags
