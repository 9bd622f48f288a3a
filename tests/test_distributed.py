"""Multi-process paths on CPU (gloo, world size 2): data-parallel training equals large-batch training,
packed metric reduction, sharded variables, host-side failure detection."""

import os
import socket
import sys
import tempfile

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp


_PORT_STATE = {"next": None}


def _free_port():
    """A listening port below the ephemeral range (so no outgoing connection of a worker can grab it between the probe
    and the rendezvous), different for every call of this process."""
    if _PORT_STATE["next"] is None:
        _PORT_STATE["next"] = 20000 + (os.getpid() * 37) % 8000
    for _ in range(200):
        port = _PORT_STATE["next"]
        _PORT_STATE["next"] = 20000 + (port - 20000 + 1) % 8000
        s = socket.socket()
        try:
            s.bind(("127.0.0.1", port))
        except OSError:
            continue
        finally:
            s.close()
        return port
    raise RuntimeError("no free rendezvous port found")


def _run(fn, world, *args, timeout=240):
    port = _free_port()
    ctx = mp.get_context("spawn")
    with tempfile.TemporaryDirectory() as tmp:
        procs = [ctx.Process(target=_entry, args=(fn.__name__, r, world, port, tmp) + args) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout)
        codes = [p.exitcode for p in procs]
        for p in procs:
            if p.is_alive():
                p.kill()
        out = {}
        for r in range(world):
            f = os.path.join(tmp, f"out{r}.npz")
            if os.path.exists(f):
                out[r] = dict(np.load(f, allow_pickle=True))
        return codes, out


def _entry(fn_name, rank, world, port, tmp, *args):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                       "KERAS_TORCH_DEVICE": "cpu", "CUDA_VISIBLE_DEVICES": ""})
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    torch.set_num_threads(1)
    result = globals()[fn_name](rank, world, *args)
    if result is not None:
        np.savez(os.path.join(tmp, f"out{rank}.npz"), **result)


def _make_model(keras):
    keras.utils.set_random_seed(7)
    inp = keras.Input((6,))
    x = keras.layers.Dense(8, activation="relu")(inp)
    out = keras.layers.Dense(3)(x)
    m = keras.Model(inp, out)
    m.compile(optimizer=keras.optimizers.SGD(0.1, momentum=0.9), loss=keras.losses.MeanSquaredError(), metrics=[keras.metrics.MeanAbsoluteError()])
    return m


def _data():
    rng = np.random.RandomState(0)
    return rng.randn(32, 6).astype("float32"), rng.randn(32, 3).astype("float32")


def _dp_worker(rank, world):
    import keras_b200 as keras

    keras.distribution.initialize()
    dist = keras.distribution.DataParallel()
    keras.distribution.set_distribution(dist)
    m = _make_model(keras)
    x, y = _data()
    hist = m.fit(x, y, batch_size=4, epochs=2, shuffle=False, verbose=0)
    w = {f"w{i}": v for i, v in enumerate(m.get_weights())}
    w["loss"] = np.array(hist.history["loss"])
    w["mae"] = np.array(hist.history["mean_absolute_error"])
    return w


def test_data_parallel_matches_large_batch():
    codes, out = _run(_dp_worker, 2)
    assert codes == [0, 0], codes
    import keras_b200 as keras

    m = _make_model(keras)
    x, y = _data()
    hist = m.fit(x, y, batch_size=8, epochs=2, shuffle=False, verbose=0)
    ref = m.get_weights()
    for r in (0, 1):
        for i, w in enumerate(ref):
            np.testing.assert_allclose(out[r][f"w{i}"], w, rtol=1e-5, atol=1e-6)
        # metrics and loss are reduced over replicas: both ranks report the global values
        np.testing.assert_allclose(out[r]["mae"], hist.history["mean_absolute_error"], rtol=1e-5)
        np.testing.assert_allclose(out[r]["loss"], hist.history["loss"], rtol=1e-5)


def _tp_worker(rank, world):
    import keras_b200 as keras

    keras.distribution.initialize()
    mesh = keras.distribution.DeviceMesh((1, 2), ["batch", "model"], devices=keras.distribution.list_devices())
    lm = keras.distribution.LayoutMap(mesh)
    lm["dense.*kernel"] = (None, "model")
    lm["dense.*bias"] = ("model",)
    keras.distribution.set_distribution(keras.distribution.ModelParallel(layout_map=lm, batch_dim_name="batch"))
    keras.utils.set_random_seed(3)
    inp = keras.Input((6,))
    out = keras.layers.Dense(8, name="dense")(inp)
    m = keras.Model(inp, out)
    m.compile(optimizer=keras.optimizers.SGD(0.05), loss="mse")
    x, y = np.ones((4, 6), "float32"), np.zeros((4, 8), "float32")
    k = m.layers[-1].kernel
    local_shape = tuple(k._value.shape)
    before = np.array(k.numpy(), copy=True)
    m.train_on_batch(x, y)
    after = k.numpy()
    return {"local": np.array(local_shape), "global": np.array(tuple(k.shape)), "before": before, "after": after, "pred": m.predict(x, verbose=0)}


def test_model_parallel_sharded_variables_match_unsharded():
    codes, out = _run(_tp_worker, 2)
    assert codes == [0, 0], codes
    import keras_b200 as keras

    keras.utils.set_random_seed(3)
    inp = keras.Input((6,))
    m = keras.Model(inp, keras.layers.Dense(8, name="dense")(inp))
    m.compile(optimizer=keras.optimizers.SGD(0.05), loss="mse")
    x, y = np.ones((4, 6), "float32"), np.zeros((4, 8), "float32")
    before = np.array(m.layers[-1].kernel.numpy(), copy=True)
    m.train_on_batch(x, y)
    for r in (0, 1):
        assert tuple(out[r]["local"]) == (6, 4) and tuple(out[r]["global"]) == (6, 8)
        np.testing.assert_allclose(out[r]["before"], before, rtol=1e-6)
        np.testing.assert_allclose(out[r]["after"], m.layers[-1].kernel.numpy(), rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(out[r]["pred"], m.predict(x, verbose=0), rtol=1e-5, atol=1e-6)


def _tp_mlp(keras):
    keras.utils.set_random_seed(11)
    inp = keras.Input((6,))
    x = keras.layers.Dense(16, activation="relu", name="up")(inp)
    x = keras.layers.Dropout(0.0)(x)
    x = keras.layers.Dense(6, name="down")(x)
    x = keras.layers.EinsumDense("ab,bcd->acd", output_shape=(4, 2), bias_axes="cd", name="heads")(x)
    x = keras.layers.EinsumDense("acd,cde->ae", output_shape=(5,), bias_axes="e", name="merge")(x)
    out = keras.layers.Dense(3, name="plain")(x)
    m = keras.Model(inp, out)
    m.compile(optimizer=keras.optimizers.Adam(0.01), loss="mse")
    return m


def _tp_pair_worker(rank, world):
    import keras_b200 as keras

    keras.distribution.initialize()
    mesh = keras.distribution.DeviceMesh((1, 2), ["batch", "model"], devices=keras.distribution.list_devices())
    lm = keras.distribution.LayoutMap(mesh)
    lm["up/kernel"] = (None, "model")
    lm["up/bias"] = ("model",)
    lm["down/kernel"] = ("model", None)
    lm["heads/kernel"] = (None, "model", None)
    lm["heads/bias"] = ("model", None)
    lm["merge/kernel"] = ("model", None, None)
    keras.distribution.set_distribution(keras.distribution.ModelParallel(layout_map=lm, batch_dim_name="batch"))
    m = _tp_mlp(keras)
    x, y = _data()
    losses = [float(m.train_on_batch(x[:8], y[:8])) for _ in range(3)]
    out = {f"w{i}": w for i, w in enumerate(m.get_weights())}
    out["losses"] = np.array(losses)
    out["pred"] = m.predict(x[:8], verbose=0)
    out["kept"] = np.array(sorted(m._parallel_engine.plan["kept_sharded"]))
    out["up_local"] = np.array(tuple(m.get_layer("up").kernel._value.shape))
    return out


def test_tensor_parallel_column_row_layers_match_unsharded():
    codes, out = _run(_tp_pair_worker, 2)
    assert codes == [0, 0], codes
    import keras_b200 as keras

    m = _tp_mlp(keras)
    x, y = _data()
    losses = [float(m.train_on_batch(x[:8], y[:8])) for _ in range(3)]
    for r in (0, 1):
        assert tuple(out[r]["up_local"]) == (6, 8)
        assert [str(s) for s in out[r]["kept"]] == ["up"], out[r]["kept"]
        np.testing.assert_allclose(out[r]["losses"], losses, rtol=1e-5)
        for i, w in enumerate(m.get_weights()):
            np.testing.assert_allclose(out[r][f"w{i}"], w, rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(out[r]["pred"], m.predict(x[:8], verbose=0), rtol=1e-4, atol=1e-6)


def _tp_attention_model(keras):
    keras.utils.set_random_seed(5)
    inp = keras.Input((5, 8))
    x = keras.layers.MultiHeadAttention(num_heads=4, key_dim=3, name="mha")(inp, inp, use_causal_mask=True)
    x = keras.layers.LayerNormalization(name="ln")(x + inp)
    x = keras.layers.GroupedQueryAttention(head_dim=4, num_query_heads=4, num_key_value_heads=2, name="gqa")(x, x)
    out = keras.layers.Dense(2, name="head")(x)
    m = keras.Model(inp, out)
    m.compile(optimizer=keras.optimizers.SGD(0.1), loss="mse")
    return m


def _tp_attention_worker(rank, world):
    import keras_b200 as keras

    keras.distribution.initialize()
    mesh = keras.distribution.DeviceMesh((1, 2), ["batch", "model"], devices=keras.distribution.list_devices())
    lm = keras.distribution.LayoutMap(mesh)
    lm["(mha|gqa)/(query|key|value)/kernel"] = (None, "model", None)
    lm["(mha|gqa)/(query|key|value)/bias"] = ("model", None)
    lm["(mha|gqa)/attention_output/kernel"] = ("model", None, None)
    keras.distribution.set_distribution(keras.distribution.ModelParallel(layout_map=lm, batch_dim_name="batch"))
    m = _tp_attention_model(keras)
    rng = np.random.RandomState(1)
    x, y = rng.randn(4, 5, 8).astype("float32"), rng.randn(4, 5, 2).astype("float32")
    losses = [float(m.train_on_batch(x, y)) for _ in range(3)]
    out = {f"w{i}": w for i, w in enumerate(m.get_weights())}
    out["losses"] = np.array(losses)
    out["q_local"] = np.array(tuple(m.get_layer("mha")._query_dense.kernel._value.shape))
    out["kept"] = np.array([bool(getattr(m.get_layer(n)._query_dense, "_tp_keep_sharded", False)) for n in ("mha", "gqa")])
    return out


def test_tensor_parallel_attention_heads_match_unsharded():
    codes, out = _run(_tp_attention_worker, 2)
    assert codes == [0, 0], codes
    import keras_b200 as keras

    m = _tp_attention_model(keras)
    rng = np.random.RandomState(1)
    x, y = rng.randn(4, 5, 8).astype("float32"), rng.randn(4, 5, 2).astype("float32")
    losses = [float(m.train_on_batch(x, y)) for _ in range(3)]
    for r in (0, 1):
        assert tuple(out[r]["q_local"]) == (8, 2, 3)
        assert out[r]["kept"].all()
        np.testing.assert_allclose(out[r]["losses"], losses, rtol=1e-5)
        for i, w in enumerate(m.get_weights()):
            np.testing.assert_allclose(out[r][f"w{i}"], w, rtol=1e-4, atol=1e-6)


def _sp_model(keras):
    keras.utils.set_random_seed(21)
    inp = keras.Input((5, 8))
    h = keras.layers.Dense(8, name="embed")(inp)
    for i in range(2):
        a = keras.layers.LayerNormalization(name=f"ln1_{i}")(h)
        a = keras.layers.MultiHeadAttention(num_heads=4, key_dim=2, name=f"attn_{i}")(a, a, use_causal_mask=True)
        h = keras.layers.Add(name=f"res1_{i}")([h, a])
        m = keras.layers.LayerNormalization(name=f"ln2_{i}")(h)
        m = keras.layers.Dense(16, activation="relu", name=f"up_{i}")(m)
        m = keras.layers.Dense(8, name=f"down_{i}")(m)
        h = keras.layers.Add(name=f"res2_{i}")([h, m])
    h = keras.layers.LayerNormalization(name="ln_f")(h)
    out = keras.layers.Dense(3, name="head")(h)
    m = keras.Model(inp, out)
    m.compile(optimizer=keras.optimizers.SGD(0.1), loss="mse")
    return m


def _sp_worker(rank, world):
    os.environ["KERAS_B200_TP_SP_EMULATE"] = "1"
    import keras_b200 as keras
    from keras_b200.core import global_state

    keras.distribution.initialize()
    mesh = keras.distribution.DeviceMesh((1, 2), ["batch", "model"], devices=keras.distribution.list_devices())
    lm = keras.distribution.LayoutMap(mesh)
    lm["attn_.*/(query|key|value)/kernel"] = (None, "model", None)
    lm["attn_.*/(query|key|value)/bias"] = ("model", None)
    lm["attn_.*/attention_output/kernel"] = ("model", None, None)
    lm["up_.*/kernel"] = (None, "model")
    lm["up_.*/bias"] = ("model",)
    lm["down_.*/kernel"] = ("model", None)
    keras.distribution.set_distribution(keras.distribution.ModelParallel(layout_map=lm, batch_dim_name="batch"))
    m = _sp_model(keras)
    rng = np.random.RandomState(2)
    x, y = rng.randn(4, 5, 8).astype("float32"), rng.randn(4, 5, 3).astype("float32")
    losses = [float(m.train_on_batch(x, y)) for _ in range(3)]
    sp = global_state.get_global_attribute("tp_sequence_parallel")
    out = {f"w{i}": w for i, w in enumerate(m.get_weights())}
    out["losses"] = np.array(losses)
    out["partial"] = np.array(sorted(v.path for v in sp.partial_variables.values())) if sp is not None else np.array([])
    out["pred"] = m.predict(x, verbose=0)
    return out


def test_sequence_parallel_executor_matches_unsharded():
    codes, out = _run(_sp_worker, 2)
    assert codes == [0, 0], codes
    import keras_b200 as keras

    m = _sp_model(keras)
    rng = np.random.RandomState(2)
    x, y = rng.randn(4, 5, 8).astype("float32"), rng.randn(4, 5, 3).astype("float32")
    losses = [float(m.train_on_batch(x, y)) for _ in range(3)]
    for r in (0, 1):
        partial = [str(p) for p in out[r]["partial"]]
        # the per-sample layers between the blocks ran on batch shards
        assert any("ln2_0" in p for p in partial) and any("ln_f" in p for p in partial), partial
        np.testing.assert_allclose(out[r]["losses"], losses, rtol=1e-5)
        for i, w in enumerate(m.get_weights()):
            np.testing.assert_allclose(out[r][f"w{i}"], w, rtol=2e-4, atol=1e-6)
        np.testing.assert_allclose(out[r]["pred"], m.predict(x, verbose=0), rtol=1e-4, atol=1e-6)


def _dp_tp_worker(rank, world):
    os.environ["KERAS_B200_TP_SP_EMULATE"] = "1"
    import keras_b200 as keras

    keras.distribution.initialize()
    mesh = keras.distribution.DeviceMesh((2, 2), ["data", "model"], devices=keras.distribution.list_devices())
    lm = keras.distribution.LayoutMap(mesh)
    lm["attn_.*/(query|key|value)/kernel"] = (None, "model", None)
    lm["attn_.*/(query|key|value)/bias"] = ("model", None)
    lm["attn_.*/attention_output/kernel"] = ("model", None, None)
    lm["up_.*/kernel"] = (None, "model")
    lm["up_.*/bias"] = ("model",)
    lm["down_.*/kernel"] = ("model", None)
    keras.distribution.set_distribution(keras.distribution.ModelParallel(layout_map=lm, batch_dim_name="data"))
    m = _sp_model(keras)  # SGD: Adam would amplify the rounding noise of gradients that are zero in exact arithmetic (key bias)
    rng = np.random.RandomState(2)
    x, y = rng.randn(8, 5, 8).astype("float32"), rng.randn(8, 5, 3).astype("float32")
    data_index = rank // 2  # ranks (0, 1) form the first model-parallel group and read the first half of the batch
    xs, ys = x[data_index * 4:(data_index + 1) * 4], y[data_index * 4:(data_index + 1) * 4]
    losses = [float(m.train_on_batch(xs, ys)) for _ in range(3)]
    out = {f"w{i}": w for i, w in enumerate(m.get_weights())}
    out["losses"] = np.array(losses)
    return out


def test_data_and_model_parallel_mesh_matches_single_process():
    codes, out = _run(_dp_tp_worker, 4, timeout=300)
    assert codes == [0, 0, 0, 0], codes
    import keras_b200 as keras

    m = _sp_model(keras)  # SGD: Adam would amplify the rounding noise of gradients that are zero in exact arithmetic (key bias)
    rng = np.random.RandomState(2)
    x, y = rng.randn(8, 5, 8).astype("float32"), rng.randn(8, 5, 3).astype("float32")
    for _ in range(3):
        m.train_on_batch(x, y)
    for r in range(4):
        for i, w in enumerate(m.get_weights()):
            np.testing.assert_allclose(out[r][f"w{i}"], w, rtol=5e-4, atol=2e-6)
    assert abs(out[0]["losses"][-1] - out[2]["losses"][-1]) < 1e-6  # the loss is reduced over the data axis


def _watchdog_worker(rank, world, scenario):
    import time

    import keras_b200 as keras
    from keras_b200.parallel.watchdog import RankFailure, RankWatchdog

    keras.distribution.initialize()
    wd = RankWatchdog(interval_s=0.1, timeout_s=1.0).start()
    detected, step_reached = [], 0
    try:
        for step in range(40):
            wd.check()  # between steps: no collective in flight
            step_reached = step
            if rank == 1 and step == 3:
                if scenario == "leave":
                    wd.leave("simulated departure")
                    return {"detected": np.array([]), "step": np.array(step)}
                if scenario == "silent":
                    wd.pause_heartbeat()  # the process stays alive but looks wedged from outside
                if scenario == "raise":
                    wd.report_failure(ValueError("injected on the host"))
                    wd.stop()
                    return {"detected": np.array([]), "step": np.array(step)}
            time.sleep(0.1)
    except RankFailure as e:
        detected = e.ranks
        reason = e.reasons[e.ranks[0]]
        wd.stop()
        return {"detected": np.array(detected), "step": np.array(step_reached), "reason": np.array(reason)}
    wd.stop()
    return {"detected": np.array(detected), "step": np.array(step_reached)}


@pytest.mark.parametrize("scenario", ["leave", "silent", "raise"])
def test_rank_watchdog_detects_lost_rank_on_the_host(scenario):
    codes, out = _run(_watchdog_worker, 3, scenario, timeout=120)
    assert codes == [0, 0, 0], codes
    for r in (0, 2):
        assert list(out[r]["detected"]) == [1], (r, out[r])
        assert 3 <= int(out[r]["step"]) < 39
    expected = {"leave": "simulated departure", "silent": "no heartbeat", "raise": "ValueError"}[scenario]
    assert expected in str(out[0]["reason"])


def _restart_worker(rank, world, backup_dir, fail):
    import keras_b200 as keras
    from keras_b200.parallel.watchdog import RankFailure

    keras.distribution.initialize()
    keras.distribution.set_distribution(keras.distribution.DataParallel())
    m = _make_model(keras)
    x, y = _data()

    class Leave(keras.callbacks.Callback):
        def on_epoch_begin(self, epoch, logs=None):
            if fail and rank == 1 and epoch == 2:
                fd.watchdog.leave("simulated crash before epoch 2")
                raise SystemExit(0)

    fd = keras.callbacks.FailureDetection(interval_s=0.1, timeout_s=2.0)
    backup = keras.callbacks.BackupAndRestore(os.path.join(backup_dir, f"rank{rank}"))
    epochs_run = []

    class Record(keras.callbacks.Callback):
        def on_epoch_begin(self, epoch, logs=None):
            import time

            epochs_run.append(epoch)
            time.sleep(0.5)  # let a departure that happened at this epoch boundary be seen before the first batch

    outcome = "finished"
    try:
        m.fit(x, y, batch_size=4, epochs=4, shuffle=False, verbose=0, callbacks=[backup, fd, Leave(), Record()])
    except RankFailure as e:
        outcome = f"lost {e.ranks}"
    return {"outcome": np.array(outcome), "epochs": np.array(epochs_run)}


def test_failure_detection_aborts_fit_and_backup_restores_the_epoch():
    with tempfile.TemporaryDirectory() as d:
        codes, out = _run(_restart_worker, 2, d, True, timeout=180)
        assert codes[0] == 0, codes
        assert "lost [1]" in str(out[0]["outcome"]), out[0]
        assert list(out[0]["epochs"])[:2] == [0, 1]
        # restart with fresh processes: training resumes at the interrupted epoch instead of epoch 0
        codes, out = _run(_restart_worker, 2, d, False, timeout=180)
        assert codes == [0, 0], codes
        assert str(out[0]["outcome"]) == "finished"
        assert list(out[0]["epochs"])[0] >= 2 and list(out[0]["epochs"])[-1] == 3, out[0]["epochs"]


def test_gradient_buckets_cover_the_arena_in_backward_order():
    """Buckets of the overlapped data-parallel reduction: contiguous, at variable boundaries, in arena order, nothing left out."""
    from keras_b200.parallel.overlap import plan_buckets

    sizes = [32, 320, 64, 4096, 64, 64, 64, 2048]          # arena order (last layer first)
    offsets, at = {}, 0
    for position, size in enumerate(sizes):
        offsets[len(sizes) - 1 - position] = at            # variable indices run in creation order: the reverse
        at += size
    buckets, bucket_of = plan_buckets(offsets, at, target_bytes=4096, max_buckets=8)
    assert buckets[0][0] == 0 and sum(n for _, n in buckets) == at
    assert all(buckets[i][0] + buckets[i][1] == buckets[i + 1][0] for i in range(len(buckets) - 1))
    starts = {start for start, _ in buckets}
    assert starts <= set(offsets.values())                 # cut at variable boundaries only
    assert bucket_of == sorted(bucket_of, reverse=True)    # later variables (earlier in backward) sit in earlier buckets
    assert 2 <= len(buckets) <= 8
    one, _ = plan_buckets(offsets, at, target_bytes=1 << 30, max_buckets=8)
    assert one == [(0, at)]
