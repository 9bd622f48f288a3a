"""``FeatureSpace``: one-stop preprocessing of structured (dict) data
(keras/src/layers/preprocessing/feature_space.py:83-866)."""

import numpy as np

from keras_b200 import tree
from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import convert_to_tensor, is_tensor
from keras_b200.layers.layer import Layer
from keras_b200.saving import saving_lib, serialization_lib
from keras_b200.saving.keras_saveable import KerasSaveable


class Cross(KerasSaveable):
    def __init__(self, feature_names, crossing_dim, output_mode="one_hot"):
        if output_mode not in {"int", "one_hot"}:
            raise ValueError(f"Invalid value for argument `output_mode`. Expected one of {{'int', 'one_hot'}}. Received: output_mode={output_mode}")
        self.feature_names = tuple(feature_names)
        self.crossing_dim = crossing_dim
        self.output_mode = output_mode

    def _obj_type(self):
        return "Cross"

    @property
    def name(self):
        return "_X_".join(self.feature_names)

    def get_config(self):
        return {"feature_names": self.feature_names, "crossing_dim": self.crossing_dim, "output_mode": self.output_mode}

    @classmethod
    def from_config(cls, config):
        return cls(**config)


class Feature(KerasSaveable):
    def __init__(self, dtype, preprocessor, output_mode):
        if output_mode not in {"int", "one_hot", "float"}:
            raise ValueError(f"Invalid value for argument `output_mode`. Expected one of {{'int', 'one_hot', 'float'}}. Received: output_mode={output_mode}")
        self.dtype = dtype
        if isinstance(preprocessor, dict):
            preprocessor = serialization_lib.deserialize_keras_object(preprocessor)
        self.preprocessor = preprocessor
        self.output_mode = output_mode

    def _obj_type(self):
        return "Feature"

    def get_config(self):
        return {"dtype": self.dtype, "preprocessor": serialization_lib.serialize_keras_object(self.preprocessor), "output_mode": self.output_mode}

    @classmethod
    def from_config(cls, config):
        return cls(**config)


@keras_export("keras.utils.FeatureSpace")
class FeatureSpace(Layer):
    @classmethod
    def cross(cls, feature_names, crossing_dim, output_mode="one_hot"):
        return Cross(feature_names, crossing_dim, output_mode=output_mode)

    @classmethod
    def feature(cls, dtype, preprocessor, output_mode):
        return Feature(dtype, preprocessor, output_mode)

    @classmethod
    def float(cls, name=None):
        from keras_b200 import layers
        from keras_b200.core.naming import auto_name

        name = name or auto_name("float")
        return Feature(dtype="float32", preprocessor=layers.Identity(dtype="float32", name=f"{name}_preprocessor"), output_mode="float")

    @classmethod
    def float_rescaled(cls, scale=1.0, offset=0.0, name=None):
        from keras_b200 import layers
        from keras_b200.core.naming import auto_name

        name = name or auto_name("float_rescaled")
        return Feature(dtype="float32", preprocessor=layers.Rescaling(scale=scale, offset=offset, name=f"{name}_preprocessor"), output_mode="float")

    @classmethod
    def float_normalized(cls, name=None):
        from keras_b200 import layers
        from keras_b200.core.naming import auto_name

        name = name or auto_name("float_normalized")
        return Feature(dtype="float32", preprocessor=layers.Normalization(axis=-1, name=f"{name}_preprocessor"), output_mode="float")

    @classmethod
    def float_discretized(cls, num_bins, bin_boundaries=None, output_mode="one_hot", name=None):
        from keras_b200 import layers
        from keras_b200.core.naming import auto_name

        name = name or auto_name("float_discretized")
        return Feature(dtype="float32", preprocessor=layers.Discretization(num_bins=num_bins, bin_boundaries=bin_boundaries, name=f"{name}_preprocessor"),
                       output_mode=output_mode)

    @classmethod
    def integer_categorical(cls, max_tokens=None, num_oov_indices=1, output_mode="one_hot", name=None):
        from keras_b200 import layers
        from keras_b200.core.naming import auto_name

        name = name or auto_name("integer_categorical")
        return Feature(dtype="int32", preprocessor=layers.IntegerLookup(name=f"{name}_preprocessor", max_tokens=max_tokens, num_oov_indices=num_oov_indices),
                       output_mode=output_mode)

    @classmethod
    def string_categorical(cls, max_tokens=None, num_oov_indices=1, output_mode="one_hot", name=None):
        from keras_b200 import layers
        from keras_b200.core.naming import auto_name

        name = name or auto_name("string_categorical")
        return Feature(dtype="string", preprocessor=layers.StringLookup(name=f"{name}_preprocessor", max_tokens=max_tokens, num_oov_indices=num_oov_indices),
                       output_mode=output_mode)

    @classmethod
    def string_hashed(cls, num_bins, output_mode="one_hot", name=None):
        from keras_b200 import layers
        from keras_b200.core.naming import auto_name

        name = name or auto_name("string_hashed")
        return Feature(dtype="string", preprocessor=layers.Hashing(name=f"{name}_preprocessor", num_bins=num_bins), output_mode=output_mode)

    @classmethod
    def integer_hashed(cls, num_bins, output_mode="one_hot", name=None):
        from keras_b200 import layers
        from keras_b200.core.naming import auto_name

        name = name or auto_name("integer_hashed")
        return Feature(dtype="int32", preprocessor=layers.Hashing(name=f"{name}_preprocessor", num_bins=num_bins), output_mode=output_mode)

    def __init__(self, features, output_mode="concat", crosses=None, crossing_dim=32, hashing_dim=32, num_discretization_bins=32, name=None):
        super().__init__(name=name)
        if not features:
            raise ValueError("The `features` argument cannot be None or empty.")
        self.crossing_dim, self.hashing_dim, self.num_discretization_bins = crossing_dim, hashing_dim, num_discretization_bins
        self.features = {name: self._standardize_feature(name, value) for name, value in features.items()}
        self.crosses = []
        if crosses:
            feature_set = set(features.keys())
            for cross in crosses:
                if isinstance(cross, dict):
                    cross = serialization_lib.deserialize_keras_object(cross)
                if isinstance(cross, Cross):
                    self.crosses.append(cross)
                else:
                    if not crossing_dim:
                        raise ValueError("When specifying `crosses`, the argument `crossing_dim` (dimensionality of the crossing space) should be specified as well.")
                    for key in cross:
                        if key not in feature_set:
                            raise ValueError(f"All features referenced in the `crosses` argument should be present in the `features` dict. Received unknown features: {cross}")
                    self.crosses.append(Cross(cross, crossing_dim=crossing_dim))
        self.crosses_by_name = {cross.name: cross for cross in self.crosses}
        if output_mode not in {"dict", "concat"}:
            raise ValueError(f"Invalid value for argument `output_mode`. Expected one of {{'dict', 'concat'}}. Received: output_mode={output_mode}")
        self.output_mode = output_mode
        from keras_b200 import layers

        self.inputs = {name: layers.Input(shape=(1,), dtype=value.dtype, name=name) for name, value in self.features.items()}
        self.preprocessors = {name: value.preprocessor for name, value in self.features.items()}
        self.encoded_features = None
        self.crossers = {cross.name: layers.HashedCrossing(cross.crossing_dim, name=cross.name) for cross in self.crosses}
        self.one_hot_encoders = {}
        self._is_adapted = False
        self.concat = None
        self._preprocessed_features_names = None
        self._crossed_features_names = None
        self._sublayers_built = False
        self._convert_input_args = False
        self._allow_non_tensor_positional_args = True

    def _standardize_feature(self, name, feature):
        if isinstance(feature, Feature):
            return feature
        if isinstance(feature, dict):
            return serialization_lib.deserialize_keras_object(feature)
        if feature == "float":
            return self.float(name=name)
        if feature == "float_normalized":
            return self.float_normalized(name=name)
        if feature == "float_rescaled":
            return self.float_rescaled(name=name)
        if feature == "float_discretized":
            return self.float_discretized(name=name, num_bins=self.num_discretization_bins)
        if feature == "integer_categorical":
            return self.integer_categorical(name=name)
        if feature == "string_categorical":
            return self.string_categorical(name=name)
        if feature == "integer_hashed":
            return self.integer_hashed(self.hashing_dim, name=name)
        if feature == "string_hashed":
            return self.string_hashed(self.hashing_dim, name=name)
        raise ValueError(f"Invalid feature type: {feature}")

    def _list_adaptable_preprocessors(self):
        from keras_b200 import layers

        out = []
        for name in self.features.keys():
            p = self.preprocessors[name]
            if isinstance(p, layers.Normalization):
                if p.input_mean is not None:
                    continue
            elif isinstance(p, layers.TextVectorization):
                if p._has_input_vocabulary:
                    continue
            elif hasattr(p, "_has_input_vocabulary") and p._has_input_vocabulary:
                continue
            if hasattr(p, "adapt"):
                out.append(name)
        return out

    def adapt(self, dataset, verbose=1):
        """``dataset``: a dict of arrays, or an iterable of dict batches."""
        if isinstance(dataset, dict):
            dataset = [dataset]
        elif not hasattr(dataset, "__iter__"):
            raise ValueError(f"`adapt()` can only be called on a dict of arrays or an iterable of dict batches. Received instead: {dataset} (of type {type(dataset)})")
        batches = list(dataset)
        for name in self._list_adaptable_preprocessors():
            def feature_batches(name=name):
                for b in batches:
                    x = b[name]
                    arr = x if is_tensor(x) else np.asarray(x)
                    if arr.ndim in (0, 1):
                        arr = arr.reshape(-1, 1)
                    yield arr

            self.preprocessors[name].adapt(list(feature_batches()))
        self._is_adapted = True
        self._build_encoders()
        self.built = True
        self._sublayers_built = True

    def get_inputs(self):
        self._check_if_built()
        return self.inputs

    def get_encoded_features(self):
        self._check_if_adapted()
        if self.encoded_features is None:
            pre = self._preprocess_features(self.inputs)
            crossed = self._cross_features(pre)
            self.encoded_features = self._merge_features(pre, crossed)
        return self.encoded_features

    def _preprocess_features(self, features):
        return {name: self.preprocessors[name](features[name]) for name in features.keys()}

    def _cross_features(self, features):
        out = {}
        for cross in self.crosses:
            out[cross.name] = self.crossers[cross.name]([features[name] for name in cross.feature_names])
        return out

    def _cardinality(self, name, preprocessor):
        from keras_b200 import layers

        if isinstance(preprocessor, (layers.IntegerLookup, layers.StringLookup)):
            return preprocessor.vocabulary_size()
        if isinstance(preprocessor, layers.CategoryEncoding):
            return preprocessor.num_tokens
        if isinstance(preprocessor, layers.Discretization):
            return preprocessor.num_bins
        if isinstance(preprocessor, (layers.HashedCrossing, layers.Hashing)):
            return preprocessor.num_bins
        raise ValueError(f"Feature '{name}' has `output_mode='one_hot'`. However it isn't a standard feature and the dimensionality of its "
                         "output space is not known, thus it cannot be one-hot encoded. Try using `output_mode='int'`.")

    def _build_encoders(self):
        from keras_b200 import layers

        self._preprocessed_features_names = sorted(self.features.keys())
        self._crossed_features_names = sorted(self.crosses_by_name.keys())
        specs = [self.features[n] for n in self._preprocessed_features_names] + [self.crosses_by_name[n] for n in self._crossed_features_names]
        for name, spec in zip(self._preprocessed_features_names + self._crossed_features_names, specs):
            if spec.output_mode == "one_hot":
                pre = self.preprocessors.get(name) or self.crossers.get(name)
                self.one_hot_encoders[name] = layers.CategoryEncoding(num_tokens=self._cardinality(name, pre), output_mode="multi_hot")
        if self.output_mode == "concat":
            self.concat = layers.Concatenate(axis=-1)

    def _merge_features(self, preprocessed, crossed):
        from keras_b200 import ops

        if not self._sublayers_built and not self.one_hot_encoders and self.concat is None:
            self._build_encoders()
        names = self._preprocessed_features_names + self._crossed_features_names
        feats = [preprocessed[n] for n in self._preprocessed_features_names] + [crossed[n] for n in self._crossed_features_names]
        out = {}
        to_concat = []
        for name, f in zip(names, feats):
            enc = self.one_hot_encoders.get(name)
            if enc is not None:
                f = enc(f)
            if self.output_mode == "dict":
                out[name] = f
            else:
                dtype = str(getattr(f, "dtype", "float32"))
                if "float" not in dtype:
                    f = ops.cast(f, "float32")
                to_concat.append(f)
        if self.output_mode == "dict":
            return out
        return self.concat(to_concat)

    def _check_if_adapted(self):
        if not self._is_adapted:
            if not self._list_adaptable_preprocessors():
                self._is_adapted = True
            else:
                raise ValueError("You need to call `.adapt(dataset)` on the FeatureSpace before you can start using it.")

    def _check_if_built(self):
        if not self._sublayers_built:
            self._check_if_adapted()
            self.get_encoded_features()
            self._sublayers_built = True

    def _convert_input(self, x):
        if isinstance(x, (list, tuple)) or np.isscalar(x) or isinstance(x, (str, bytes)):
            x = np.asarray(x)
        if isinstance(x, np.ndarray) and x.dtype.kind in "USO":
            return x
        if isinstance(x, np.ndarray):
            return x
        return x

    def __call__(self, data):
        self._check_if_built()
        if not isinstance(data, dict):
            raise ValueError(f"A FeatureSpace can only be called with a dict. Received: data={data} (of type {type(data)}")
        data = {key: self._convert_input(value) for key, value in data.items()}
        rebatched = False
        for name, x in data.items():
            ndim = x.ndim if hasattr(x, "ndim") else np.ndim(x)
            if ndim == 0:
                data[name] = x.reshape((1, 1))
                rebatched = True
            elif ndim == 1:
                data[name] = x.reshape(-1, 1) if isinstance(x, np.ndarray) else x.unsqueeze(-1)
        pre = self._preprocess_features(data)
        pre = tree.map_structure(lambda t: convert_to_tensor(t) if not (isinstance(t, np.ndarray) and t.dtype.kind in "USO") else t, pre)
        crossed = self._cross_features(pre)
        merged = self._merge_features(pre, crossed)
        if rebatched:
            if self.output_mode == "concat":
                assert merged.shape[0] == 1
                merged = merged[0]
            else:
                merged = {k: (v[0] if v.shape[0] == 1 else v) for k, v in merged.items()}
        return merged

    def get_config(self):
        return {"features": serialization_lib.serialize_keras_object(self.features), "output_mode": self.output_mode,
                "crosses": serialization_lib.serialize_keras_object(self.crosses), "crossing_dim": self.crossing_dim,
                "hashing_dim": self.hashing_dim, "num_discretization_bins": self.num_discretization_bins}

    @classmethod
    def from_config(cls, config):
        return cls(**config)

    def get_build_config(self):
        return {name: feature.preprocessor.get_build_config() for name, feature in self.features.items()}

    def build_from_config(self, config):
        for name in config.keys():
            preprocessor = self.features[name].preprocessor
            if not preprocessor.built:
                preprocessor.build_from_config(config[name])
        self._is_adapted = True

    def save(self, filepath):
        """Save the ``FeatureSpace`` as a ``.keras`` archive; reload with ``keras.models.load_model``."""
        saving_lib.save_model(self, filepath)

    def save_own_variables(self, store):
        return

    def load_own_variables(self, store):
        return
