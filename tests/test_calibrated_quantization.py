"""GPTQ and AWQ: the solvers against the reference's on the same matrices, and ``model.quantize`` end to end (calibration,
accuracy against round-to-nearest, checkpoint round trip)."""

import os

import numpy as np
import pytest
import torch

import keras_b200 as keras
from keras_b200.quantizers import weight_only
from tests import oracle


def _problem(seed, out_features=24, in_features=96, rows=400):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(out_features, in_features, generator=g) * 0.3
    x = torch.randn(rows, in_features, generator=g) * (torch.rand(in_features, generator=g) * 2 + 0.1)
    return w, x


@pytest.mark.parametrize("bits,group,symmetric,order", [(4, -1, False, False), (4, 32, False, False), (4, 32, True, True), (8, -1, False, True),
                                                         (2, 16, False, False), (3, 32, False, True)])
def test_gptq_solver_matches_reference(bits, group, symmetric, order):
    oracle.ref()
    from keras.src.quantizers import gptq as ref_gptq
    from keras.src.quantizers.gptq_config import GPTQConfig
    from keras.src.quantizers.quantizers import GPTQQuantizer

    w, x = _problem(bits * 7 + group)
    estimate = weight_only.HessianEstimate(w.shape[1])
    estimate.add(x[:150])
    estimate.add(x[150:])
    h = estimate.damped(0.01)
    # the reference keeps one grid per block when group_size is -1: compare on a single block there
    block = 32 if group != -1 else 128
    finder = GPTQQuantizer(GPTQConfig(dataset=None, tokenizer=None, weight_bits=bits, group_size=group, symmetric=symmetric, activation_order=order),
                           compute_dtype="float32")
    want = ref_gptq.gptq_quantize_matrix(w.clone(), h.clone(), blocksize=block, group_size=group, activation_order=order,
                                         order_metric=torch.diagonal(h), compute_scale_zero=finder.find_params)
    got = weight_only.gptq_solve(w, h, bits=bits, group_size=group, symmetric=symmetric, activation_order=order, block=block)
    assert float((got[0] != want[0].cpu()).float().mean()) < 0.005
    torch.testing.assert_close(got[1], want[1].cpu(), rtol=1e-5, atol=1e-7)
    assert torch.equal(got[2], want[2].cpu()) and torch.equal(got[3], want[3].cpu().to(torch.int32))


def test_hessian_estimate_matches_reference_running_average():
    rk = oracle.ref()
    from keras.src.quantizers.gptq import GPTQ

    layer = rk.layers.Dense(8)
    layer.build((None, 20))
    theirs = GPTQ(layer)
    ours = weight_only.HessianEstimate(20)
    g = torch.Generator().manual_seed(4)
    for rows in (7, 31, 3):
        x = torch.randn(rows, 20, generator=g)
        theirs.update_hessian_with_batch(x)
        ours.add(x)
    torch.testing.assert_close(ours.matrix, theirs.hessian.cpu(), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("group,clip", [(-1, False), (32, False), (32, True), (-1, True)])
def test_awq_solver_matches_reference(group, clip):
    oracle.ref()
    from keras.src.quantizers import awq as ref_awq

    w, x = _problem(11 + group)
    profile = weight_only.ActivationProfile(w.shape[1], keep_sample=clip)
    profile.add(x[:100])
    profile.add(x[100:])
    want = ref_awq.awq_quantize_matrix(w.clone(), profile.magnitudes.clone(), num_grid_points=20, group_size=group, apply_clip=clip,
                                       activation_sample=profile.sample)
    got = weight_only.awq_solve(w, profile.magnitudes, num_grid_points=20, group_size=group, activation_sample=profile.sample if clip else None)
    assert float((got[0] != want[0].cpu()).float().mean()) < 0.005
    torch.testing.assert_close(got[3], want[3].cpu(), rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(got[1], want[1].cpu(), rtol=1e-5, atol=1e-7)


# --------------------------------------------------------------------------------------------- end to end
class _Tokenizer:
    def tokenize(self, text):
        return np.array([(ord(c) * 7) % 50 for c in text], dtype="int32")


@keras.saving.register_keras_serializable(package="calib_test")
class Block(keras.layers.Layer):
    PARTS = ("norm", "query", "out", "up", "down")

    def __init__(self, width=32, parts=None, **kwargs):
        super().__init__(**kwargs)
        self.width = width
        if parts is None:
            parts = {"norm": keras.layers.LayerNormalization(), "query": keras.layers.EinsumDense("btd,dhk->bthk", output_shape=(None, 4, width // 4)),
                     "out": keras.layers.EinsumDense("bthk,hkd->btd", output_shape=(None, width)),
                     "up": keras.layers.Dense(2 * width, activation="gelu"), "down": keras.layers.Dense(width)}
        for name in self.PARTS:  # a restored block gets its sub-layers back with their (quantised) dtype policies
            setattr(self, name, parts[name])

    def call(self, x):
        h = self.norm(x)
        x = x + self.out(self.query(h))
        return x + self.down(self.up(x))

    def get_config(self):
        parts = {name: keras.saving.serialize_keras_object(getattr(self, name)) for name in self.PARTS}
        return {**super().get_config(), "width": self.width, "parts": parts}

    @classmethod
    def from_config(cls, config):
        config = dict(config)
        config["parts"] = {name: keras.saving.deserialize_keras_object(part) for name, part in config["parts"].items()}
        return cls(**config)


def _model(seed):
    keras.utils.set_random_seed(seed)
    tokens = keras.Input((16,), dtype="int32")
    embed = keras.layers.Embedding(50, 32, name="embed")
    blocks = [Block(name=f"block_{i}") for i in range(2)]
    h = embed(tokens)
    for block in blocks:
        h = block(h)
    out = keras.layers.Dense(50, name="head")(h)
    return keras.Model(tokens, out), {"pre_block_layers": [embed], "sequential_blocks": blocks}


def _config(mode, structure, **kwargs):
    data = ["the quick brown fox jumps over the lazy dog " * 3, "pack my box with five dozen liquor jugs " * 3, "sphinx of black quartz judge my vow " * 3]
    cls = keras.quantizers.GPTQConfig if mode == "gptq" else keras.quantizers.AWQConfig
    return cls(dataset=data, tokenizer=_Tokenizer(), num_samples=16, sequence_length=16, group_size=16, quantization_layer_structure=structure, **kwargs)


@pytest.mark.parametrize("mode", ["gptq", "awq"])
def test_model_quantize_calibrates_blocks_and_round_trips(mode, tmp_path):
    model, structure = _model(3)
    x = np.random.default_rng(0).integers(0, 50, size=(8, 16)).astype("int32")
    before = keras.ops.convert_to_numpy(model(x))
    model.quantize(mode, config=_config(mode, structure))
    projections = [layer for block in structure["sequential_blocks"] for layer in (block.query, block.out, block.up, block.down)]
    for layer in projections:
        assert layer.quantization_mode == mode and layer._calibrated and not hasattr(layer, "_kernel")
        assert layer.quantized_kernel.dtype == "uint8" and layer.dtype_policy.name.startswith(f"{mode}/4/16_from_")
    head = model.get_layer("head")
    assert head.quantization_mode is None  # outside the blocks: untouched
    after = keras.ops.convert_to_numpy(model(x))
    rel = np.linalg.norm(after - before) / np.linalg.norm(before)
    assert rel < 0.2, rel
    path = os.path.join(tmp_path, f"{mode}.keras")
    model.save(path)
    restored = keras.saving.load_model(path, custom_objects={"Block": Block})
    np.testing.assert_allclose(keras.ops.convert_to_numpy(restored(x)), after, rtol=1e-5, atol=1e-5)


def test_gptq_beats_round_to_nearest_on_the_calibration_distribution():
    w, x = _problem(21, out_features=48, in_features=128, rows=800)
    g = torch.Generator().manual_seed(9)
    # correlated input features: that is what lets the error of one feature be compensated by the others
    x = torch.randn(800, 24, generator=g) @ torch.randn(24, 128, generator=g) + 0.05 * x
    estimate = weight_only.HessianEstimate(128)
    estimate.add(x)
    codes, scale, zero, g_idx = weight_only.gptq_solve(w, estimate.damped(0.01), bits=3, group_size=32)
    gptq_error = float(((x @ (weight_only.dequantize(codes.float(), scale, zero, g_idx) - w).T) ** 2).mean())
    rtn = weight_only.round_to_nearest(w, 3, 32)
    rtn_error = float(((x @ (weight_only.dequantize(rtn[0], rtn[1], rtn[2], rtn[3]) - w).T) ** 2).mean())
    assert gptq_error < 0.7 * rtn_error, (gptq_error, rtn_error)


def test_calibrated_modes_need_data_and_structure():
    model, structure = _model(5)
    with pytest.raises(ValueError, match="must pass a `GPTQConfig`"):
        model.quantize("gptq")
    with pytest.raises(ValueError, match="requires a dataset and a tokenizer"):
        model.quantize("gptq", config=keras.quantizers.GPTQConfig(dataset=None, tokenizer=None, quantization_layer_structure=structure))
    with pytest.raises(ValueError, match="valid quantization structure"):
        model.quantize("awq", config=keras.quantizers.AWQConfig(dataset=["abc"], tokenizer=_Tokenizer()))
