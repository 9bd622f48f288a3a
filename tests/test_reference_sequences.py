"""Masks and seeded dropout through recurrent and attention layers, against the reference (CPU, float32)."""

import warnings

import numpy as np
import pytest
import torch

import keras_b200 as keras
from tests import oracle

IDS = np.array([[3, 4, 5, 0, 0], [1, 2, 0, 0, 0], [6, 7, 8, 9, 1]], "int32")


def _both(build, run):
    """``build(k)`` makes a layer or model in either framework; ours takes the reference's weights; ``run`` gives the outputs."""
    rk = oracle.ref()
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        theirs, ours = build(rk), build(keras)
        ours.set_weights(theirs.get_weights())
        return run(rk, theirs), run(keras, ours)


def _same(got, expected, what, rtol=1e-5, atol=1e-5):
    got = list(got) if isinstance(got, (list, tuple)) else [got]
    expected = list(expected) if isinstance(expected, (list, tuple)) else [expected]
    assert len(got) == len(expected), what
    for a, b in zip(got, expected):
        oracle.assert_same(a, b, what, rtol=rtol, atol=atol)


RNN_OPTIONS = [dict(), dict(return_sequences=True), dict(go_backwards=True, return_sequences=True), dict(unroll=True),
               dict(return_sequences=True, zero_output_for_mask=True), dict(return_state=True)]


@pytest.mark.parametrize("kind", ["LSTM", "GRU", "SimpleRNN"])
@pytest.mark.parametrize("options", RNN_OPTIONS, ids=["last", "sequences", "backwards", "unrolled", "zero_output", "state"])
def test_masked_recurrent_layers_match_reference(kind, options):
    def build(k):
        return k.Sequential([k.Input((5,), dtype="int32"), k.layers.Embedding(12, 4, mask_zero=True), getattr(k.layers, kind)(3, **options)])

    expected, got = _both(build, lambda k, m: m(IDS))
    _same(got, expected, f"{kind} {options}")


def test_mask_propagation_follows_the_reference_layer_by_layer():
    """Which layers attach the incoming mask to their output decides what a masked loss averages over."""
    rk = oracle.ref()
    for name, make in [("LSTM", lambda k: k.layers.LSTM(3, return_sequences=True)), ("GRU", lambda k: k.layers.GRU(3, return_sequences=True)),
                       ("Bidirectional", lambda k: k.layers.Bidirectional(k.layers.GRU(3, return_sequences=True))),
                       ("TimeDistributed", lambda k: k.layers.TimeDistributed(k.layers.Dense(3))), ("Dense", lambda k: k.layers.Dense(3)),
                       ("Dropout", lambda k: k.layers.Dropout(0.5)), ("LayerNormalization", lambda k: k.layers.LayerNormalization()),
                       ("Conv1D", lambda k: k.layers.Conv1D(3, 1))]:
        carried = []
        for k in (rk, keras):
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                layer = make(k)
                out = layer(k.layers.Embedding(12, 4, mask_zero=True)(IDS))
            carried.append(getattr(out, "_keras_mask", None) is not None)
            assert layer.supports_masking == carried[-1] or name in ("Conv1D",), name
        assert carried[0] == carried[1], f"{name}: the reference {'keeps' if carried[0] else 'drops'} the mask"


def test_layer_without_mask_support_warns_that_the_mask_is_lost():
    masked = keras.layers.Embedding(12, 4, mask_zero=True)(IDS)
    with pytest.warns(UserWarning, match="does not support masking"):
        keras.layers.Conv1D(3, 1)(masked)


def test_masked_models_match_reference():
    def bidirectional(k):
        return k.Sequential([k.Input((5,), dtype="int32"), k.layers.Embedding(12, 4, mask_zero=True),
                             k.layers.Bidirectional(k.layers.GRU(3, return_sequences=True)), k.layers.GlobalAveragePooling1D()])

    def attention(k):
        inp = k.Input((5,), dtype="int32")
        e = k.layers.Embedding(12, 6, mask_zero=True)(inp)
        return k.Model(inp, k.layers.MultiHeadAttention(2, 3)(e, e, use_causal_mask=True))

    def distributed(k):
        inp = k.Input((5,), dtype="int32")
        e = k.layers.Embedding(12, 6, mask_zero=True)(inp)
        return k.Model(inp, k.layers.LSTM(2)(k.layers.TimeDistributed(k.layers.Dense(3))(e)))

    def pooled(k):
        return k.Sequential([k.Input((5,), dtype="int32"), k.layers.Embedding(12, 4, mask_zero=True), k.layers.Dense(3), k.layers.GlobalAveragePooling1D()])

    for build in (bidirectional, attention, distributed, pooled):
        expected, got = _both(build, lambda k, m: m(IDS))
        _same(got, expected, build.__name__)


def test_attention_keeps_input_masks_for_other_consumers_and_masks_its_output():
    e = keras.layers.Embedding(12, 6, mask_zero=True)(IDS)
    out = keras.layers.MultiHeadAttention(2, 3)(e, e)
    assert getattr(e, "_keras_mask", None) is not None
    np.testing.assert_array_equal(oracle.to_np(out._keras_mask), IDS != 0)


def test_fit_with_a_masked_sequence_loss_matches_reference():
    y = np.random.default_rng(5).normal(size=(3, 5, 2)).astype("float32")

    def build(k):
        return k.Sequential([k.Input((5,), dtype="int32"), k.layers.Embedding(12, 4, mask_zero=True), k.layers.Dense(3, activation="tanh"), k.layers.Dense(2)])

    def run(k, m):
        m.compile(optimizer=k.optimizers.SGD(0.1), loss="mse", metrics=["mae"])
        h = m.fit(IDS, y, epochs=2, batch_size=3, verbose=0, shuffle=False)
        return [np.array(h.history["loss"], "float32"), np.array(h.history["mae"], "float32")]

    expected, got = _both(build, run)
    _same(got, expected, "masked loss and metric", rtol=1e-4, atol=1e-5)
    masked_mean = ((oracle.to_np(build(keras)(IDS)) * 0).sum())  # shape check only: the model runs eagerly too
    assert masked_mean == 0


DROPOUT_LAYERS = [
    ("lstm", lambda k: k.layers.LSTM(3, dropout=0.3, recurrent_dropout=0.2, seed=5), (2, 4, 3)),
    ("lstm_input_only", lambda k: k.layers.LSTM(3, dropout=0.4, seed=1), (2, 4, 3)),
    ("lstm_recurrent_only", lambda k: k.layers.LSTM(3, recurrent_dropout=0.4, seed=1, return_sequences=True), (2, 4, 3)),
    ("gru", lambda k: k.layers.GRU(3, dropout=0.3, recurrent_dropout=0.2, seed=5, return_sequences=True), (2, 4, 3)),
    ("gru_reset_before", lambda k: k.layers.GRU(3, dropout=0.4, recurrent_dropout=0.3, reset_after=False, seed=1), (2, 4, 3)),
    ("gru_per_gate_without_dropout", lambda k: k.layers.GRU(3, implementation=1), (2, 4, 3)),
    ("simple_rnn", lambda k: k.layers.SimpleRNN(3, dropout=0.4, recurrent_dropout=0.3, seed=1), (2, 4, 3)),
    ("conv_lstm", lambda k: k.layers.ConvLSTM2D(2, 3, padding="same", dropout=0.4, recurrent_dropout=0.3, seed=1), (2, 3, 5, 5, 2)),
    ("stacked_cells", lambda k: k.layers.RNN([k.layers.LSTMCell(3, dropout=0.3, seed=1), k.layers.GRUCell(2, recurrent_dropout=0.3, seed=2)]), (2, 4, 3)),
    ("bidirectional", lambda k: k.layers.Bidirectional(k.layers.LSTM(3, dropout=0.3, recurrent_dropout=0.2, seed=1)), (2, 4, 3)),
    ("attention", lambda k: k.layers.MultiHeadAttention(2, 3, dropout=0.5, seed=9), (2, 4, 6)),
]


@pytest.mark.parametrize("spec", DROPOUT_LAYERS, ids=[s[0] for s in DROPOUT_LAYERS])
def test_seeded_dropout_inside_layers_draws_the_reference_masks(spec):
    """Same seed, same masks: one mask per gate where the reference draws one per gate, and a new draw at every call."""
    name, make, shape = spec
    x = np.random.default_rng(1).normal(size=shape).astype("float32")

    def build(k):
        layer = make(k)
        layer.build(shape, shape) if name == "attention" else layer.build(shape)
        return layer

    def run(k, layer):
        args = (torch.tensor(x), torch.tensor(x)) if name == "attention" else (torch.tensor(x),)
        return [layer(*args, training=True), layer(*args, training=True)]

    expected, got = _both(build, run)
    _same(got, expected, name)
    assert not np.allclose(oracle.to_np(got[0]), oracle.to_np(got[1])) or name == "gru_per_gate_without_dropout"


def test_stateful_rnn_and_initial_state_match_reference():
    x = np.random.default_rng(1).normal(size=(2, 4, 3)).astype("float32")
    h0 = np.random.default_rng(2).normal(size=(2, 3)).astype("float32")

    def stateful(k):
        layer = k.layers.LSTM(3, stateful=True, return_sequences=True)
        layer.build((2, 4, 3))
        return layer

    def run_stateful(k, layer):
        first, second = layer(torch.tensor(x)), layer(torch.tensor(x))
        layer.reset_state()
        return [first, second, layer(torch.tensor(x))]

    expected, got = _both(stateful, run_stateful)
    _same(got, expected, "stateful LSTM")
    np.testing.assert_allclose(oracle.to_np(got[0]), oracle.to_np(got[2]), rtol=1e-6)

    def with_state(k):
        layer = k.layers.GRU(3, return_state=True)
        layer.build((2, 4, 3))
        return layer

    expected, got = _both(with_state, lambda k, layer: list(layer(torch.tensor(x), initial_state=[torch.tensor(h0)])))
    _same(got, expected, "GRU with an initial state")


def test_fully_masked_attention_rows_are_finite_and_uniform():
    """A query row whose every key is masked attends uniformly, as in the reference (a large finite negative, not -inf)."""
    rk = oracle.ref()
    r = np.random.default_rng(0)
    q, k_, v = (r.normal(size=s).astype("float32") for s in ((2, 4, 2, 3), (2, 5, 2, 3), (2, 5, 2, 3)))
    mask = r.integers(0, 2, (2, 1, 4, 5)).astype(bool)
    mask[0, 0, 1] = False
    got = keras.ops.dot_product_attention(q, k_, v, mask=mask)
    oracle.assert_same(got, rk.ops.dot_product_attention(q, k_, v, mask=mask), "dot_product_attention with a fully masked row")
    np.testing.assert_allclose(oracle.to_np(got)[0, 1], v[0].mean(0), rtol=1e-5, atol=1e-6)
