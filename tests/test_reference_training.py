"""Optimizers, losses, metrics, random ops and a short ``fit`` against the reference (CPU, float32)."""

import numpy as np
import pytest
import torch

import keras_b200 as keras
from tests import oracle

OPTIMIZERS = [
    ("SGD", dict(learning_rate=0.1)),
    ("SGD", dict(learning_rate=0.1, momentum=0.9, nesterov=True)),
    ("Adam", dict(learning_rate=0.01)),
    ("Adam", dict(learning_rate=0.01, amsgrad=True)),
    ("Adam", dict(learning_rate=0.1, gradient_accumulation_steps=2)),
    ("Adam", dict(learning_rate=0.01, use_ema=True, ema_momentum=0.9)),
    ("Adam", dict(learning_rate=0.01, clipnorm=0.5)),
    ("Adam", dict(learning_rate=0.01, global_clipnorm=0.5)),
    ("AdamW", dict(learning_rate=0.01, weight_decay=0.1)),
    ("Adamax", dict(learning_rate=0.01)),
    ("Adadelta", dict(learning_rate=1.0)),
    ("Adagrad", dict(learning_rate=0.1)),
    ("Adafactor", dict(learning_rate=0.01)),
    ("Ftrl", dict(learning_rate=0.1, l1_regularization_strength=0.01)),
    ("Lamb", dict(learning_rate=0.01)),
    ("Lion", dict(learning_rate=0.01)),
    ("Nadam", dict(learning_rate=0.01)),
    ("RMSprop", dict(learning_rate=0.01, momentum=0.5, centered=True)),
    ("Muon", dict(learning_rate=0.01)),
    ("ScheduleFreeAdamW", dict(learning_rate=0.01, warmup_steps=2)),
]


def _opt_ids():
    return [f"{n}_{i}" for i, (n, _) in enumerate(OPTIMIZERS)]


@pytest.mark.parametrize("spec", OPTIMIZERS, ids=_opt_ids())
def test_optimizer_trajectory_matches_reference(spec):
    rk = oracle.ref()
    name, kwargs = spec
    if not hasattr(rk.optimizers, name):
        pytest.skip("optimizer absent from this reference version")
    rng = np.random.default_rng(0)
    init = [rng.normal(size=(4, 3)).astype("float32"), rng.normal(size=(3,)).astype("float32")]
    grads = [[rng.normal(size=a.shape).astype("float32") for a in init] for _ in range(5)]

    def run(k):
        variables = [k.Variable(a.copy(), name=f"v{i}") for i, a in enumerate(init)]
        opt = getattr(k.optimizers, name)(**kwargs)
        for step in grads:
            opt.apply([torch.tensor(g) for g in step], variables)
        if kwargs.get("use_ema"):
            opt.finalize_variable_values(variables)
        return [oracle.to_np(v.value) for v in variables], int(oracle.to_np(getattr(opt.iterations, "value", opt.iterations)))

    (theirs, their_it), (ours, our_it) = run(rk), run(keras)
    assert our_it == their_it
    for a, b in zip(ours, theirs):
        np.testing.assert_allclose(a, b, rtol=2e-5, atol=2e-6, err_msg=name)


LOSSES = ["BinaryCrossentropy", "BinaryFocalCrossentropy", "CategoricalCrossentropy", "CategoricalFocalCrossentropy", "CategoricalHinge",
          "CosineSimilarity", "Dice", "Hinge", "Huber", "KLDivergence", "LogCosh", "MeanAbsoluteError", "MeanAbsolutePercentageError",
          "MeanSquaredError", "MeanSquaredLogarithmicError", "Poisson", "SquaredHinge", "Tversky", "Circle", "CategoricalGeneralizedCrossEntropy"]


@pytest.mark.parametrize("name", LOSSES)
def test_loss_matches_reference(name):
    rk = oracle.ref()
    if not hasattr(rk.losses, name):
        pytest.skip("loss absent from this reference version")
    rng = np.random.default_rng(1)
    p = rng.uniform(0.05, 0.95, (6, 4)).astype("float32")
    p = p / p.sum(-1, keepdims=True)
    t = np.eye(4, dtype="float32")[rng.integers(0, 4, 6)]
    weights = rng.uniform(0.5, 1.5, (6,)).astype("float32")
    if name in ("Circle", "CategoricalGeneralizedCrossEntropy"):
        t_arg = t.argmax(-1).astype("int32")
    else:
        t_arg = t
    expected = getattr(rk.losses, name)()(t_arg, p, sample_weight=weights)
    got = getattr(keras.losses, name)()(t_arg, p, sample_weight=weights)
    oracle.assert_same(got, expected, name, rtol=1e-5, atol=1e-6)


def test_sparse_categorical_crossentropy_with_ignore_class_and_logits():
    rk = oracle.ref()
    rng = np.random.default_rng(2)
    logits = rng.normal(size=(5, 7, 4)).astype("float32")
    labels = rng.integers(0, 4, (5, 7)).astype("int32")
    labels[0, :3] = -1
    for k_args in (dict(from_logits=True), dict(from_logits=True, ignore_class=-1), dict(from_logits=True, reduction="sum")):
        oracle.assert_same(keras.losses.SparseCategoricalCrossentropy(**k_args)(labels, logits) if "ignore_class" in k_args or labels.min() >= 0 else 0,
                           rk.losses.SparseCategoricalCrossentropy(**k_args)(labels, logits) if "ignore_class" in k_args or labels.min() >= 0 else 0,
                           str(k_args), rtol=1e-5, atol=1e-6, check_dtype=False)


METRICS = [
    ("Accuracy", {}, "labels"), ("BinaryAccuracy", dict(threshold=0.4), "binary"), ("CategoricalAccuracy", {}, "onehot"),
    ("SparseCategoricalAccuracy", {}, "sparse"), ("TopKCategoricalAccuracy", dict(k=2), "onehot"), ("SparseTopKCategoricalAccuracy", dict(k=2), "sparse"),
    ("AUC", dict(num_thresholds=20), "binary"), ("Precision", {}, "binary"), ("Recall", dict(thresholds=0.3), "binary"),
    ("F1Score", dict(average="macro"), "onehot"), ("FBetaScore", dict(beta=2.0, average="weighted"), "onehot"),
    ("MeanIoU", dict(num_classes=4), "labels"), ("IoU", dict(num_classes=4, target_class_ids=[1, 2]), "labels"), ("BinaryIoU", {}, "binary"),
    ("OneHotMeanIoU", dict(num_classes=4), "onehot"), ("MeanSquaredError", {}, "real"), ("RootMeanSquaredError", {}, "real"),
    ("MeanAbsoluteError", {}, "real"), ("LogCoshError", {}, "real"), ("CosineSimilarity", {}, "real"), ("R2Score", {}, "real"),
    ("PearsonCorrelation", {}, "real"), ("ConcordanceCorrelation", {}, "real"), ("KLDivergence", {}, "onehot"), ("Poisson", {}, "onehot"),
    ("Hinge", {}, "onehot"), ("CategoricalCrossentropy", {}, "onehot"), ("SparseCategoricalCrossentropy", {}, "sparse"),
    ("BinaryCrossentropy", {}, "binary"), ("TruePositives", {}, "binary"), ("FalseNegatives", dict(thresholds=[0.3, 0.7]), "binary"),
    ("PrecisionAtRecall", dict(recall=0.5, num_thresholds=20), "binary"), ("SensitivityAtSpecificity", dict(specificity=0.5, num_thresholds=20), "binary"),
    ("Mean", {}, "values"), ("Sum", {}, "values"),
]


@pytest.mark.parametrize("spec", METRICS, ids=[m[0] for m in METRICS])
def test_metric_matches_reference(spec):
    rk = oracle.ref()
    name, kwargs, kind = spec
    if not hasattr(rk.metrics, name):
        pytest.skip("metric absent from this reference version")
    rng = np.random.default_rng(3)

    def batch():
        p = rng.uniform(0.05, 0.95, (8, 4)).astype("float32")
        p = p / p.sum(-1, keepdims=True)
        lab = rng.integers(0, 4, 8).astype("int32")
        if kind == "labels":
            return lab, p.argmax(-1).astype("int32")
        if kind == "binary":
            return (rng.uniform(size=(8, 1)) > 0.5).astype("float32"), rng.uniform(size=(8, 1)).astype("float32")
        if kind == "onehot":
            return np.eye(4, dtype="float32")[lab], p
        if kind == "sparse":
            return lab, p
        if kind == "real":
            return rng.normal(size=(8, 3)).astype("float32"), rng.normal(size=(8, 3)).astype("float32")
        return (rng.normal(size=(8,)).astype("float32"),)

    batches = [batch() for _ in range(3)]
    theirs, ours = getattr(rk.metrics, name)(**kwargs), getattr(keras.metrics, name)(**kwargs)
    for b in batches:
        theirs.update_state(*b)
        ours.update_state(*b)
    oracle.assert_same(ours.result(), theirs.result(), name, rtol=1e-5, atol=1e-6, check_dtype=False)


def test_positional_k_of_sparse_top_k_accuracy():
    m = keras.metrics.SparseTopKCategoricalAccuracy(3)
    assert m.k == 3 and isinstance(m.name, str)


def test_random_ops_follow_the_reference_generator_rule():
    rk = oracle.ref()
    x = torch.ones((4, 6))
    for seed in (7, 1234):
        oracle.assert_same(keras.random.dropout(x, 0.4, seed=seed), rk.random.dropout(x, 0.4, seed=seed), "dropout")
        oracle.assert_same(keras.random.normal((3, 4), seed=seed), rk.random.normal((3, 4), seed=seed), "normal")
        oracle.assert_same(keras.random.uniform((3, 4), seed=seed), rk.random.uniform((3, 4), seed=seed), "uniform")
        oracle.assert_same(keras.random.truncated_normal((3, 4), seed=seed), rk.random.truncated_normal((3, 4), seed=seed), "truncated_normal")
        oracle.assert_same(keras.random.randint((3, 4), 0, 9, seed=seed), rk.random.randint((3, 4), 0, 9, seed=seed), "randint")
    theirs, ours = rk.random.SeedGenerator(5), keras.random.SeedGenerator(5)
    for _ in range(3):
        oracle.assert_same(keras.random.dropout(x, 0.5, seed=ours), rk.random.dropout(x, 0.5, seed=theirs), "dropout with a SeedGenerator")
    theirs_layer, ours_layer = rk.layers.Dropout(0.3, seed=11), keras.layers.Dropout(0.3, seed=11)
    oracle.assert_same(ours_layer(x, training=True), theirs_layer(x, training=True), "Dropout layer")


def _small_convnet(k):
    return k.Sequential([
        k.Input((12, 12, 1)), k.layers.Conv2D(4, 3, activation="relu"), k.layers.MaxPooling2D(2), k.layers.Conv2D(6, 3, activation="relu"),
        k.layers.GlobalAveragePooling2D(), k.layers.Dropout(0.25, seed=3), k.layers.Dense(5, activation="softmax")])


@pytest.mark.parametrize("options", [dict(), dict(steps_per_execution=2), dict(gradient_accumulation_steps=2), dict(shuffle=True), dict(shuffle="batch")],
                         ids=["plain", "steps_per_execution", "accumulation", "shuffled", "shuffled_in_batches"])
def test_fit_history_matches_reference(options):
    rk = oracle.ref()
    rng = np.random.default_rng(4)
    x = rng.normal(size=(64, 12, 12, 1)).astype("float32")
    y = rng.integers(0, 5, (64,)).astype("int32")
    theirs, ours = _small_convnet(rk), _small_convnet(keras)
    ours.set_weights(theirs.get_weights())
    accumulation = options.get("gradient_accumulation_steps")
    spe = options.get("steps_per_execution", 1)
    histories = []
    for k, model in ((rk, theirs), (keras, ours)):
        opt = k.optimizers.Adam(1e-2, gradient_accumulation_steps=accumulation) if accumulation else k.optimizers.Adam(1e-2)
        model.compile(optimizer=opt, loss="sparse_categorical_crossentropy", metrics=["accuracy"], steps_per_execution=spe)
        h = model.fit(x, y, batch_size=16, epochs=3 if options.get("shuffle") else 2, shuffle=options.get("shuffle", False), verbose=0, validation_split=0.25)
        histories.append(h.history)
    for key in histories[0]:
        np.testing.assert_allclose(histories[1][key], histories[0][key], rtol=2e-3, atol=2e-4, err_msg=key)
    scores_theirs = theirs.evaluate(x, y, batch_size=32, verbose=0)
    scores_ours = ours.evaluate(x, y, batch_size=32, verbose=0)
    assert len(scores_ours) == len(scores_theirs)
    np.testing.assert_allclose(scores_ours, scores_theirs, rtol=2e-3, atol=2e-4)


def test_evaluate_with_metric_instance_returns_each_metric_once():
    rk = oracle.ref()
    rng = np.random.default_rng(5)
    x, y = rng.normal(size=(16, 4)).astype("float32"), rng.integers(0, 3, (16,)).astype("int32")
    out = []
    for k in (rk, keras):
        model = k.Sequential([k.Input((4,)), k.layers.Dense(3, activation="softmax")])
        model.compile(optimizer="sgd", loss="sparse_categorical_crossentropy", metrics=[k.metrics.SparseCategoricalAccuracy(name="acc"), "accuracy"])
        out.append(model.evaluate(x, y, verbose=0))
    assert len(out[1]) == len(out[0])


def test_multi_optimizer_routing_matches_reference():
    rk = oracle.ref()
    if not hasattr(rk.optimizers, "MultiOptimizer"):
        pytest.skip("MultiOptimizer absent from this reference version")
    rng = np.random.default_rng(6)
    init = {"enc/kernel": rng.normal(size=(3, 2)), "enc/bias": rng.normal(size=(2,)), "head/kernel": rng.normal(size=(2, 2))}
    grads = [[rng.normal(size=a.shape).astype("float32") for a in init.values()] for _ in range(4)]

    def run(k):
        variables = [k.Variable(a.astype("float32"), name=n.split("/")[1]) for n, a in init.items()]
        for v, n in zip(variables, init):
            v._path = n if hasattr(v, "_path") else None
            try:
                v.path = n
            except Exception:
                pass
        omap = k.optimizers.OptimizerMap(k.optimizers.SGD(0.1), {"enc/.*": k.optimizers.Adam(0.01)})
        omap["head/kernel"] = k.optimizers.SGD(0.5, momentum=0.9)
        opt = k.optimizers.MultiOptimizer(omap)
        for step in grads:
            opt.apply([torch.tensor(g) for g in step], variables)
        return [oracle.to_np(v.value) for v in variables], [type(o).__name__ for o in opt.optimizers], len(opt.variables)

    theirs, ours = run(rk), run(keras)
    assert ours[1:] == theirs[1:]
    for a, b in zip(ours[0], theirs[0]):
        np.testing.assert_allclose(a, b, rtol=2e-5, atol=2e-6)
    with pytest.raises(ValueError):
        keras.optimizers.OptimizerMap(keras.optimizers.SGD(0.1), {"a.*": keras.optimizers.SGD(0.1), "ab.*": keras.optimizers.SGD(0.2)})["abc"]


def test_to_categorical_types_follow_the_reference():
    rk = oracle.ref()
    import torch

    for labels in ([0, 2, 1, 3], np.array([[0], [2], [1]]), np.array([[0, 2], [1, 3]])):
        theirs, ours = rk.utils.to_categorical(labels, num_classes=5), keras.utils.to_categorical(labels, num_classes=5)
        assert type(ours) is type(theirs) and ours.dtype == theirs.dtype and ours.shape == theirs.shape
        np.testing.assert_array_equal(ours, theirs)
    theirs, ours = rk.utils.to_categorical(torch.tensor([[1], [3]]), 4), keras.utils.to_categorical(torch.tensor([[1], [3]]), 4)
    assert isinstance(ours, torch.Tensor) and ours.dtype == theirs.dtype and tuple(ours.shape) == tuple(theirs.shape)
    np.testing.assert_array_equal(ours.numpy(), theirs.numpy())


def test_multi_output_fit_evaluate_match_reference_keys_and_values():
    """Two inputs, two outputs, per-output losses, loss weights, metrics and sample weights: histories, evaluate dicts and
    train_on_batch dicts carry the reference's keys in the reference's order with the reference's numbers."""
    rk = oracle.ref()
    rng = np.random.default_rng(0)
    xa, xb = rng.normal(size=(64, 8)).astype("float32"), rng.normal(size=(64, 5)).astype("float32")
    y1, y2 = rng.integers(0, 3, (64,)), rng.normal(size=(64, 1)).astype("float32")

    def build(k):
        a, b = k.Input((8,), name="a"), k.Input((5,), name="b")
        h = k.layers.Concatenate()([k.layers.Dense(16, activation="relu", name="da")(a), k.layers.Dense(16, activation="tanh", name="db")(b)])
        return k.Model({"a": a, "b": b}, {"cls": k.layers.Dense(3, name="cls")(h), "reg": k.layers.Dense(1, name="reg")(h)})

    rk.utils.set_random_seed(1)
    start = build(rk).get_weights()

    def run(k):
        m = build(k)
        m.set_weights(start)
        m.compile(optimizer=k.optimizers.Adam(1e-2), loss={"cls": k.losses.SparseCategoricalCrossentropy(from_logits=True), "reg": "mse"},
                  loss_weights={"cls": 1.0, "reg": 0.5},
                  metrics={"cls": ["accuracy", k.metrics.SparseTopKCategoricalAccuracy(2, name="top2")], "reg": [k.metrics.MeanAbsoluteError()]})
        hist = m.fit({"a": xa, "b": xb}, {"cls": y1, "reg": y2}, batch_size=16, epochs=2, verbose=0, shuffle=False, validation_split=0.25,
                     sample_weight={"cls": np.linspace(0.5, 1.5, 64).astype("float32"), "reg": np.ones(64, "float32")}).history
        ev = m.evaluate({"a": xa, "b": xb}, {"cls": y1, "reg": y2}, batch_size=32, verbose=0, return_dict=True)
        flat = m.evaluate({"a": xa, "b": xb}, {"cls": y1, "reg": y2}, batch_size=32, verbose=0)
        step = m.train_on_batch({"a": xa[:8], "b": xb[:8]}, {"cls": y1[:8], "reg": y2[:8]}, return_dict=True)
        return hist, ev, flat, step

    theirs, ours = run(rk), run(keras)
    for a, b in zip(ours, theirs):
        if isinstance(b, dict):
            assert list(a) == list(b)
            for key in b:
                np.testing.assert_allclose(a[key], b[key], rtol=3e-4, atol=3e-5, err_msg=key)
        else:
            np.testing.assert_allclose(a, b, rtol=3e-4, atol=3e-5)


def test_random_shuffle_orders_like_the_reference():
    rk = oracle.ref()
    x = np.arange(24).reshape(4, 3, 2)
    for seed in (0, 7):
        for axis in (0, 1, -1):
            np.testing.assert_array_equal(keras.random.shuffle(x, axis=axis, seed=seed).numpy(), rk.random.shuffle(x, axis=axis, seed=seed).numpy())


INITIALIZERS = ["GlorotUniform", "GlorotNormal", "HeUniform", "HeNormal", "LecunUniform", "LecunNormal", "RandomNormal", "RandomUniform", "TruncatedNormal", "Orthogonal",
                "VarianceScaling"]


@pytest.mark.parametrize("name", INITIALIZERS)
def test_seeded_initializers_draw_the_reference_values(name):
    rk = oracle.ref()
    for shape in [(6, 6), (3, 3, 4, 8)]:
        for dtype in ("float32", "float16"):
            if name == "Orthogonal" and dtype == "float16":
                continue  # no half-precision QR on the CPU
            theirs = getattr(rk.initializers, name)(seed=7)(shape, dtype=dtype)
            ours = getattr(keras.initializers, name)(seed=7)(shape, dtype=dtype)
            oracle.assert_same(ours, theirs, f"{name} {shape} {dtype}")
    again = getattr(keras.initializers, name)(seed=7)
    oracle.assert_same(again((4, 4)), again((4, 4)), "an integer seed gives the same values at every call")


def test_fixed_initializers_regularizers_and_constraints_match_reference():
    rk = oracle.ref()
    w = np.random.default_rng(0).normal(size=(4, 5, 3)).astype("float32")
    for make in (lambda k: k.initializers.Identity(gain=2.0)((5, 5)), lambda k: k.initializers.Constant(2.5)((3, 2)),
                 lambda k: k.initializers.STFT(side="real", window="hann")((16, 1, 9)),
                 lambda k: k.initializers.VarianceScaling(2.0, "fan_out", "untruncated_normal", seed=3)((5, 7)),
                 lambda k: k.initializers.Orthogonal(gain=2.0, seed=1)((4, 10)),
                 lambda k: k.regularizers.L1L2(l1=0.1, l2=0.2)(torch.tensor(w)),
                 lambda k: k.regularizers.OrthogonalRegularizer(factor=0.1, mode="rows")(torch.tensor(w[0])),
                 lambda k: k.regularizers.OrthogonalRegularizer(factor=0.1, mode="columns")(torch.tensor(w[0])),
                 lambda k: k.constraints.MaxNorm(max_value=1.0, axis=0)(torch.tensor(w)),
                 lambda k: k.constraints.MinMaxNorm(min_value=0.5, max_value=1.0, rate=0.7, axis=[0, 1])(torch.tensor(w)),
                 lambda k: k.constraints.NonNeg()(torch.tensor(w)), lambda k: k.constraints.UnitNorm(axis=1)(torch.tensor(w))):
        oracle.assert_same(make(keras), make(rk), "fixed initializer, regularizer or constraint", rtol=1e-5, atol=1e-6)


SCHEDULES = [
    ("ExponentialDecay", dict(initial_learning_rate=0.1, decay_steps=10, decay_rate=0.5)),
    ("ExponentialDecay", dict(initial_learning_rate=0.1, decay_steps=10, decay_rate=0.5, staircase=True)),
    ("PiecewiseConstantDecay", dict(boundaries=[5, 10], values=[1.0, 0.5, 0.1])),
    ("PolynomialDecay", dict(initial_learning_rate=0.1, decay_steps=20, end_learning_rate=0.01, power=2.0)),
    ("PolynomialDecay", dict(initial_learning_rate=0.1, decay_steps=7, end_learning_rate=0.01, power=0.5, cycle=True)),
    ("InverseTimeDecay", dict(initial_learning_rate=0.1, decay_steps=5, decay_rate=0.5, staircase=True)),
    ("CosineDecay", dict(initial_learning_rate=0.0, decay_steps=20, alpha=0.1, warmup_target=0.2, warmup_steps=5)),
    ("CosineDecayRestarts", dict(initial_learning_rate=0.1, first_decay_steps=5, t_mul=2.0, m_mul=0.9, alpha=0.05)),
]


@pytest.mark.parametrize("spec", SCHEDULES, ids=[f"{n}_{i}" for i, (n, _) in enumerate(SCHEDULES)])
def test_learning_rate_schedules_match_reference(spec):
    rk = oracle.ref()
    name, kwargs = spec
    theirs, ours = getattr(rk.optimizers.schedules, name)(**kwargs), getattr(keras.optimizers.schedules, name)(**kwargs)
    assert sorted(ours.get_config()) == sorted(theirs.get_config())
    for step in range(30):
        np.testing.assert_allclose(float(oracle.to_np(ours(step))), float(oracle.to_np(theirs(step))), rtol=1e-6, err_msg=f"{name} at step {step}")
