"""The captured (CUDA graph) training step against the eager one: same losses, same weights, learning-rate changes
honoured between replays, odd batches and random layers handled."""

import numpy as np
import pytest
import torch

import keras_b200 as keras

pytestmark = pytest.mark.gpu


def _mlp(seed, dropout_seed=None):
    keras.utils.set_random_seed(seed)
    layers = [keras.layers.Input((64,)), keras.layers.Dense(256, activation="relu"), keras.layers.LayerNormalization()]
    if dropout_seed is not None:
        layers.append(keras.layers.Dropout(0.25, seed=dropout_seed))
    layers += [keras.layers.Dense(128, activation="gelu"), keras.layers.Dense(10)]
    return keras.Sequential(layers)


def _data(n, seed=0):
    rng = np.random.default_rng(seed)
    return rng.standard_normal((n, 64)).astype("float32"), rng.integers(0, 10, size=(n,)).astype("int64")


@pytest.mark.parametrize("policy", ["float32", "mixed_bfloat16"])
@pytest.mark.parametrize("optimizer", ["adam", "sgd"])
def test_captured_step_matches_eager(policy, optimizer):
    keras.config.set_dtype_policy(policy)
    try:
        def make(jit):
            model = _mlp(7)
            opt = keras.optimizers.AdamW(1e-3, weight_decay=0.01) if optimizer == "adam" else keras.optimizers.SGD(0.05, momentum=0.9)
            model.compile(optimizer=opt, loss=keras.losses.SparseCategoricalCrossentropy(from_logits=True), metrics=["accuracy"], jit_compile=jit)
            return model

        eager, graphed = make(False), make("auto")
        graphed.set_weights(eager.get_weights())
        x, y = _data(256)
        losses = {"eager": [], "graphed": []}
        for step in range(10):
            xb, yb = x[(step % 2) * 128:(step % 2 + 1) * 128], y[(step % 2) * 128:(step % 2 + 1) * 128]
            if step == 6:  # a new learning rate must reach the captured update without a re-capture
                eager.optimizer.learning_rate = 0.01
                graphed.optimizer.learning_rate = 0.01
            losses["eager"].append(eager.train_on_batch(xb, yb))
            losses["graphed"].append(graphed.train_on_batch(xb, yb))
        assert eager._graphed_step.replays == 0
        assert graphed._graphed_step.disabled is None, graphed._graphed_step.failure_traceback
        assert graphed._graphed_step.replays == 7
        np.testing.assert_allclose(np.array(losses["graphed"]), np.array(losses["eager"]), rtol=1e-5, atol=1e-6)
        for a, b in zip(graphed.get_weights(), eager.get_weights()):
            np.testing.assert_allclose(a, b, rtol=1e-5, atol=1e-6)
        assert int(graphed.optimizer.iterations.numpy()) == 10
        assert graphed.optimizer._step() == 10
    finally:
        keras.config.set_dtype_policy("float32")


def test_fit_with_short_last_batch_and_metrics():
    model = _mlp(3)
    model.compile(optimizer=keras.optimizers.Adam(1e-3), loss=keras.losses.SparseCategoricalCrossentropy(from_logits=True), metrics=["accuracy"])
    x, y = _data(128 * 5 + 48)
    history = model.fit(x, y, batch_size=128, epochs=3, verbose=0, shuffle=False)
    stepper = model._graphed_step
    assert stepper.disabled is None, stepper.failure_traceback
    assert stepper.replays == 3 * 5 - 3          # three eager steps first; the short batches run eagerly as well
    assert int(model.optimizer.iterations.numpy()) == 3 * 6
    loss = history.history["loss"]
    assert np.all(np.isfinite(loss)) and loss[-1] < loss[0]

    reference = _mlp(3)
    reference.compile(optimizer=keras.optimizers.Adam(1e-3), loss=keras.losses.SparseCategoricalCrossentropy(from_logits=True), metrics=["accuracy"],
                      jit_compile=False)
    ref_history = reference.fit(x, y, batch_size=128, epochs=3, verbose=0, shuffle=False)
    np.testing.assert_allclose(loss, ref_history.history["loss"], rtol=1e-5)
    np.testing.assert_allclose(history.history["accuracy"], ref_history.history["accuracy"], rtol=1e-6)


def test_seeded_random_layer_stays_eager():
    model = _mlp(5, dropout_seed=11)
    model.compile(optimizer="adam", loss=keras.losses.SparseCategoricalCrossentropy(from_logits=True))
    x, y = _data(128)
    values = [model.train_on_batch(x, y) for _ in range(6)]
    stepper = model._graphed_step
    assert stepper.replays == 0 and "CaptureUnsafe" in stepper.disabled
    assert np.all(np.isfinite(values))
    assert int(model.optimizer.iterations.numpy()) == 6
    assert model.optimizer._step() == 6
    # the masks still differ from step to step: the same batch gives different losses at a tiny learning rate
    model.optimizer.learning_rate = 0.0
    a, b = model.train_on_batch(x, y), model.train_on_batch(x, y)
    assert a != b


def test_adam_step_scalars_from_device_match_host_formula():
    from keras_b200.kernels import ops as kops

    torch.manual_seed(0)
    n = 5000
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    m, v = torch.rand(n, device="cuda"), torch.rand(n, device="cuda")
    lr, b1, b2, eps, wd, t = 3e-3, 0.9, 0.999, 1e-7, 0.1, 41
    alpha = lr * np.sqrt(1 - b2 ** (t + 1)) / (1 - b1 ** (t + 1))
    want_m = m + (g - m) * (1 - b1)
    want_v = v + (g * g - v) * (1 - b2)
    want_p = p * (1 - lr * wd) - alpha * want_m / (want_v.sqrt() + eps)
    for on_device in (False, True):
        pp, gg, mm, vv = p.clone(), g.clone(), m.clone(), v.clone()
        plan = kops.OptimizerPlan([pp], [gg], [mm], [vv], None, [wd])
        if on_device:
            plan.adam(0.0, b1, b2, eps, lr_tensor=torch.tensor(lr, device="cuda"), step_tensor=torch.tensor(t, device="cuda", dtype=torch.int32))
        else:
            plan.adam(alpha, b1, b2, eps, lr=lr)
        torch.testing.assert_close(pp, want_p, rtol=2e-6, atol=2e-6)
        torch.testing.assert_close(mm, want_m, rtol=2e-6, atol=2e-6)
        torch.testing.assert_close(vv, want_v, rtol=2e-6, atol=2e-6)
        assert float(gg.abs().max()) == 0.0


def test_unused_variable_is_skipped_like_a_missing_gradient():
    """A variable the loss never reaches gets no update (no weight decay either) although gradients live in the arena."""

    class WithSpare(keras.layers.Layer):
        def build(self, input_shape):
            self.used = self.add_weight(shape=(input_shape[-1], 8), initializer="glorot_uniform", name="used")
            self.spare = self.add_weight(shape=(4, 4), initializer="ones", name="spare")

        def call(self, x):
            return keras.ops.matmul(x, self.used)

    model = keras.Sequential([keras.layers.Input((64,)), keras.layers.Dense(32, activation="relu"), WithSpare(), keras.layers.Dense(10)])
    model.compile(optimizer=keras.optimizers.AdamW(1e-2, weight_decay=0.1), loss=keras.losses.SparseCategoricalCrossentropy(from_logits=True))
    x, y = _data(128)
    spare = model.layers[1].spare
    used_before = model.layers[1].used.numpy().copy()
    with pytest.warns(UserWarning, match="Gradients do not exist"):
        model.train_on_batch(x, y)
    for _ in range(6):
        model.train_on_batch(x, y)
    assert model._graphed_step.replays == 4
    np.testing.assert_array_equal(spare.numpy(), np.ones((4, 4), "float32"))
    assert np.abs(model.layers[1].used.numpy() - used_before).max() > 1e-4


def test_assigned_weights_reach_the_captured_step():
    """``set_weights`` between replays: the recorded step reads the bf16 shadows, which must follow the assignment at once."""
    keras.config.set_dtype_policy("mixed_bfloat16")
    try:
        def make(jit):
            m = _mlp(9)
            m.compile(optimizer=keras.optimizers.SGD(0.05), loss=keras.losses.SparseCategoricalCrossentropy(from_logits=True), jit_compile=jit)
            return m

        eager, graphed = make(False), make("auto")
        graphed.set_weights(eager.get_weights())
        x, y = _data(128)
        for _ in range(5):
            eager.train_on_batch(x, y)
            graphed.train_on_batch(x, y)
        assert graphed._graphed_step.replays == 2
        fresh = [w * 0.5 for w in eager.get_weights()]
        eager.set_weights(fresh)
        graphed.set_weights(fresh)
        a, b = eager.train_on_batch(x, y), graphed.train_on_batch(x, y)
        assert graphed._graphed_step.replays == 3
        np.testing.assert_allclose(b, a, rtol=1e-5, atol=1e-6)
        for u, v in zip(graphed.get_weights(), eager.get_weights()):
            np.testing.assert_allclose(u, v, rtol=1e-5, atol=1e-6)
    finally:
        keras.config.set_dtype_policy("float32")
