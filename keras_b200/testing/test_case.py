"""``keras.testing.TestCase``: array assertions plus ``run_layer_test`` / ``run_class_serialization_test``, the harness
that checks a layer end to end: config round trip, symbolic and eager shapes/dtypes, weight counts, masks, a training
step, and the mixed-precision policy (keras/src/testing/test_case.py:22-640)."""

import json
import shutil
import tempfile
import unittest

import numpy as np
import torch

from keras_b200 import tree
from keras_b200.core.keras_tensor import KerasTensor
from keras_b200.core.tensor import convert_to_numpy, is_tensor
from keras_b200.core.variables import Variable
from keras_b200.saving import serialization_lib


def torch_uses_gpu():
    from keras_b200.core.tensor import get_device

    return get_device().type == "cuda"


uses_gpu = torch_uses_gpu


def _np(x):
    if isinstance(x, Variable):
        x = x.value
    if is_tensor(x):
        return convert_to_numpy(x)
    return np.asarray(x)


class TestCase(unittest.TestCase):
    maxDiff = None

    def setUp(self):
        from keras_b200.core import global_state

        global_state.clear_session(free_memory=False)

    def get_temp_dir(self):
        d = tempfile.mkdtemp()
        self.addCleanup(lambda: shutil.rmtree(d, ignore_errors=True))
        return d

    def convert_to_numpy(self, x):
        return _np(x)

    def assertAllClose(self, x1, x2, atol=1e-6, rtol=1e-6, msg=None):
        np.testing.assert_allclose(_np(x1).astype("float64") if _np(x1).dtype.kind in "fiub" else _np(x1),
                                   _np(x2).astype("float64") if _np(x2).dtype.kind in "fiub" else _np(x2), atol=atol, rtol=rtol, err_msg=msg or "")

    def assertNotAllClose(self, x1, x2, atol=1e-6, rtol=1e-6, msg=None):
        try:
            self.assertAllClose(x1, x2, atol=atol, rtol=rtol)
        except AssertionError:
            return
        raise AssertionError(msg or f"The two values are close at all elements. \n\nx1={x1} \nx2={x2}")

    def assertAlmostEqual(self, x1, x2, decimal=3, tpu_decimal=None, msg=None):
        np.testing.assert_almost_equal(_np(x1), _np(x2), decimal=decimal, err_msg=msg or "")

    def assertAllEqual(self, actual, desired, msg=None):
        tree.assert_same_structure(tree.map_structure(lambda x: 0, actual), tree.map_structure(lambda x: 0, desired)) if tree.is_nested(actual) else None
        for a, d in zip(tree.flatten(actual), tree.flatten(desired)):
            np.testing.assert_array_equal(_np(a), _np(d), err_msg=msg or "")

    def assertLen(self, iterable, expected_len, msg=None):
        self.assertEqual(len(iterable), expected_len, msg=msg)

    def assertSparse(self, x, sparse=True):
        is_sparse = isinstance(x, torch.Tensor) and x.is_sparse or getattr(x, "sparse", False)
        self.assertEqual(bool(is_sparse), sparse)

    def assertRagged(self, x, ragged=True):
        self.assertEqual(bool(getattr(x, "ragged", False)), ragged)

    def assertDType(self, x, dtype, msg=None):
        from keras_b200.core.dtypes import standardize_dtype

        actual = standardize_dtype(x.dtype) if hasattr(x, "dtype") else standardize_dtype(type(x))
        self.assertEqual(actual, standardize_dtype(dtype), msg or f"Expected dtype {dtype}, got {actual}")

    def assertFileExists(self, path):
        import os

        if not os.path.exists(path):
            raise AssertionError(f"File {path} does not exist")

    # -- serialisation -------------------------------------------------------------------
    def run_class_serialization_test(self, instance, custom_objects=None):
        cls = instance.__class__
        config = instance.get_config()
        config_json = json.dumps(config, sort_keys=True, indent=4, default=str)
        from keras_b200.saving.object_registration import custom_object_scope

        with custom_object_scope(custom_objects or {}):
            revived = cls.from_config(json.loads(json.dumps(config, default=str)) if _jsonable(config) else config)
        revived_json = json.dumps(revived.get_config(), sort_keys=True, indent=4, default=str)
        self.assertEqual(config_json, revived_json)
        self.assertEqual(set(dir(instance)), set(dir(revived)))
        serialized = serialization_lib.serialize_keras_object(instance)
        with custom_object_scope(custom_objects or {}):
            revived2 = serialization_lib.deserialize_keras_object(json.loads(json.dumps(serialized, default=str)) if _jsonable(serialized) else serialized,
                                                                  custom_objects=custom_objects)
        self.assertEqual(json.dumps(revived2.get_config(), sort_keys=True, indent=4, default=str), config_json)
        return revived

    # -- layers --------------------------------------------------------------------------
    def run_layer_test(self, layer_cls, init_kwargs, input_shape=None, input_dtype=None, input_sparse=False, input_ragged=False, input_data=None,
                       call_kwargs=None, expected_output_shape=None, expected_output_dtype=None, expected_output_sparse=False,
                       expected_output_ragged=False, expected_output=None, expected_num_trainable_weights=None,
                       expected_num_non_trainable_weights=None, expected_num_non_trainable_variables=None, expected_num_seed_generators=None,
                       expected_num_losses=None, supports_masking=None, expected_mask_shape=None, custom_objects=None, run_training_check=True,
                       run_mixed_precision_check=True, assert_built_after_instantiation=False, tpu_atol=None, tpu_rtol=None):
        if input_shape is not None and input_data is not None:
            raise ValueError("input_shape and input_data cannot be passed at the same time.")
        if expected_output_shape is not None and expected_output is not None:
            raise ValueError("expected_output_shape and expected_output cannot be passed at the same time.")
        if expected_output is not None and input_data is None:
            raise ValueError("In order to use expected_output, input_data must be provided.")
        if expected_mask_shape is not None and supports_masking is not True:
            raise ValueError("In order to use expected_mask_shape, supports_masking must be True.")
        call_kwargs = call_kwargs or {}
        from keras_b200 import backend, layers, losses, models, optimizers  # noqa: F401

        if input_dtype is None:
            if input_data is not None:
                input_dtype = tree.map_structure(lambda x: str(_np(x).dtype), input_data)
            else:
                input_dtype = tree.map_shape_structure(lambda s: "float32", input_shape)

        layer = layer_cls(**init_kwargs)
        self.run_class_serialization_test(layer, custom_objects)
        if assert_built_after_instantiation:
            self.assertTrue(layer.built)
        if supports_masking is not None:
            self.assertEqual(layer.supports_masking, supports_masking)

        def build_asserts(lyr):
            self.assertTrue(lyr.built)
            if expected_num_trainable_weights is not None:
                self.assertLen(lyr.trainable_weights, expected_num_trainable_weights)
            if expected_num_non_trainable_weights is not None:
                self.assertLen(lyr.non_trainable_weights, expected_num_non_trainable_weights)
            if expected_num_non_trainable_variables is not None:
                self.assertLen(lyr.non_trainable_variables, expected_num_non_trainable_variables)
            if expected_num_seed_generators is not None:
                self.assertLen(get_seed_generators(lyr), expected_num_seed_generators)

        def output_asserts(lyr, output, eager=False):
            if expected_output_shape is not None:
                for shape, out in zip(_flat_shapes(expected_output_shape), tree.flatten(output)):
                    self.assertEqual(tuple(shape), tuple(out.shape))
            if expected_output_dtype is not None:
                for dt, out in zip(tree.flatten(expected_output_dtype), tree.flatten(output)):
                    self.assertDType(out, dt)
            if eager:
                if expected_output is not None:
                    for ref, out in zip(tree.flatten(expected_output), tree.flatten(output)):
                        self.assertAllClose(ref, out, atol=1e-5, rtol=1e-5)
                if expected_num_losses is not None:
                    self.assertLen(lyr.losses, expected_num_losses)

        # symbolic call
        if input_shape is not None:
            symbolic_inputs = map_shape_dtype_structure(lambda s, d: KerasTensor(s, dtype=d), input_shape, input_dtype)
            lyr = layer_cls(**init_kwargs)
            if isinstance(symbolic_inputs, dict):
                out = lyr(**symbolic_inputs, **call_kwargs)
            else:
                out = lyr(symbolic_inputs, **call_kwargs)
            build_asserts(lyr)
            output_asserts(lyr, out)
            if expected_mask_shape is not None:
                mask = lyr.compute_mask(symbolic_inputs)
                self.assertEqual(tuple(expected_mask_shape), tuple(mask.shape))

        # eager call
        if input_data is None and input_shape is not None:
            input_data = map_shape_dtype_structure(_random_array, input_shape, input_dtype)
        if input_data is not None:
            lyr = layer_cls(**init_kwargs)
            if isinstance(input_data, dict):
                out = lyr(**input_data, **call_kwargs)
            else:
                out = lyr(input_data, **call_kwargs)
            build_asserts(lyr)
            output_asserts(lyr, out, eager=True)
            if run_training_check and all("float" in str(d) for d in tree.flatten(input_dtype)):
                self._training_step(lyr, input_data, out, call_kwargs)
            if run_mixed_precision_check and all("float" in str(d) for d in tree.flatten(input_dtype)):
                self._mixed_precision(layer_cls, init_kwargs, input_data, call_kwargs)

    def _training_step(self, layer, input_data, output_data, call_kwargs):
        from keras_b200 import models, optimizers

        class TestModel(models.Model):
            def __init__(self, lyr):
                super().__init__()
                self.layer = lyr

            def call(self, x, training=False):
                if isinstance(x, dict):
                    return self.layer(**x, **call_kwargs)
                return self.layer(x, **call_kwargs)

        model = TestModel(layer)
        flat_out = tree.flatten(output_data)

        def loss_fn(y_true, y_pred, sample_weight=None):
            total = 0.0
            for o in tree.flatten(y_pred):
                if isinstance(o, torch.Tensor) and o.dtype.is_floating_point:
                    total = total + o.float().mean()
            return total

        class Loss:
            def __call__(self, y_true, y_pred, sample_weight=None):
                return loss_fn(y_true, y_pred)

        if not any(isinstance(o, torch.Tensor) and o.dtype.is_floating_point for o in flat_out):
            return
        model.compile(optimizer=optimizers.SGD(0.0), loss=None)
        model.compute_loss = lambda x=None, y=None, y_pred=None, sample_weight=None, training=True: loss_fn(y, y_pred)
        if not model.trainable_weights:
            return
        model.train_on_batch(input_data, None) if False else model.train_step((input_data, tree.map_structure(lambda o: _np(o), output_data)))

    def _mixed_precision(self, layer_cls, init_kwargs, input_data, call_kwargs):
        from keras_b200 import dtype_policies

        kwargs = dict(init_kwargs)
        kwargs["dtype"] = dtype_policies.DTypePolicy("mixed_float16")
        layer = layer_cls(**kwargs)
        half = tree.map_structure(lambda x: _np(x).astype("float16") if _np(x).dtype.kind == "f" else _np(x), input_data)
        if isinstance(half, dict):
            out = layer(**half, **call_kwargs)
        else:
            out = layer(half, **call_kwargs)
        for o in tree.flatten(out):
            if isinstance(o, torch.Tensor) and o.dtype.is_floating_point:
                self.assertIn(str(o.dtype), ("torch.float16", "torch.float32"))
        for w in layer.weights:
            if "float" in str(w.dtype):
                self.assertEqual(str(w.dtype), "float32")


def _jsonable(obj):
    try:
        json.dumps(obj)
        return True
    except TypeError:
        return False


def _flat_shapes(shapes):
    if is_shape_tuple(shapes):
        return [shapes]
    if isinstance(shapes, dict):
        return [s for k in sorted(shapes) for s in _flat_shapes(shapes[k])]
    return [s for item in shapes for s in _flat_shapes(item)]


def _random_array(shape, dtype):
    shape = tuple(2 if d is None else d for d in shape)
    if "int" in dtype:
        return np.random.randint(0, 3, size=shape).astype(dtype)
    if dtype == "bool":
        return np.random.rand(*shape) > 0.5
    return np.random.standard_normal(shape).astype(dtype)


def is_shape_tuple(x):
    return isinstance(x, (list, tuple)) and all(isinstance(e, (int, type(None))) for e in x)


def map_shape_dtype_structure(fn, shape, dtype):
    if is_shape_tuple(shape):
        return fn(tuple(shape), dtype)
    if isinstance(shape, list):
        return [map_shape_dtype_structure(fn, s, d) for s, d in zip(shape, dtype)]
    if isinstance(shape, tuple):
        return tuple(map_shape_dtype_structure(fn, s, d) for s, d in zip(shape, dtype))
    if isinstance(shape, dict):
        return {k: map_shape_dtype_structure(fn, v, dtype[k]) for k, v in shape.items()}
    raise ValueError(f"Cannot map function to unknown objects {shape} and {dtype}")


def get_seed_generators(layer):
    from keras_b200.random.seed_generator import SeedGenerator

    seen, out = set(), []
    for lyr in layer._flatten_layers():
        for v in vars(lyr).values():
            if isinstance(v, SeedGenerator) and id(v) not in seen:
                seen.add(id(v))
                out.append(v)
    return out
