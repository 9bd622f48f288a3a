"""Multi-GPU paths: peer-memory all-reduce kernel vs NCCL, data-parallel ResNet block training, bounded waits."""

import ctypes
import os
import sys

import numpy as np
import pytest
import torch

from tests.test_distributed import _free_port  # noqa: F401  (helper reuse)

pytestmark = pytest.mark.gpu


def _spawn(fn_name, world, timeout=150):
    import tempfile

    import torch.multiprocessing as mp

    port = _free_port()
    ctx = mp.get_context("spawn")
    with tempfile.TemporaryDirectory() as tmp:
        procs = [ctx.Process(target=_gpu_entry, args=(fn_name, r, world, port, tmp)) for r in range(world)]
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


def _gpu_entry(fn_name, rank, world, port, tmp):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                       "NCCL_NVLS_ENABLE": "0", "KERAS_B200_COMM_TIMEOUT_MS": "20000", "KERAS_B200_PG_TIMEOUT_S": "90"})
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    torch.cuda.set_device(rank)
    result = globals()[fn_name](rank, world)
    if result is not None:
        np.savez(os.path.join(tmp, f"out{rank}.npz"), **result)


def _allreduce_worker(rank, world):
    import torch.distributed as dist

    import keras_b200 as keras
    from keras_b200.parallel.collectives import P2PAllReducer

    keras.distribution.initialize()
    n = 3 * 1024 * 1024 + 4 * 37
    red = P2PAllReducer(n)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    errs = []
    for it in range(3):
        src = torch.randn(red.numel, device="cuda", generator=g)
        red.flat.copy_(src)
        ref = src.clone()
        dist.all_reduce(ref)
        torch.cuda.synchronize()
        dist.barrier()
        red.all_reduce(scale=0.5)
        torch.cuda.synchronize()
        errs.append(float((red.flat - 0.5 * ref).abs().max()))
        dist.barrier()
    # skewed starts: each rank in turn launches late (no barrier in between); the flag protocol has to absorb it
    import time

    for late in range(world):
        src = torch.randn(red.numel, device="cuda", generator=g)
        red.flat.copy_(src)
        ref = src.clone()
        dist.all_reduce(ref)
        torch.cuda.synchronize()
        if rank == late:
            time.sleep(0.3)
        red.all_reduce()
        red.all_reduce(scale=0.5)  # back to back: the second call's entry flags must not be mistaken for the first's exit
        torch.cuda.synchronize()
        errs.append(float((red.flat - 0.5 * world * ref).abs().max() / world))
    dist.barrier()
    # the other collectives of the same kernel: reduce-scatter, all-gather, broadcast
    per = ((red.numel // 4 + world - 1) // world) * 4
    lo, hi = per * rank, min(red.numel, per * (rank + 1))
    src = torch.randn(red.numel, device="cuda", generator=g)
    red.flat.copy_(src)
    ref = src.clone()
    dist.all_reduce(ref)
    torch.cuda.synchronize()
    dist.barrier()
    red.reduce_scatter()
    torch.cuda.synchronize()
    errs.append(float((red.flat[lo:hi] - ref[lo:hi]).abs().max()))
    dist.barrier()
    red.all_gather()
    torch.cuda.synchronize()
    errs.append(float((red.flat - ref).abs().max()))
    dist.barrier()
    red.flat.fill_(float(rank + 1))
    torch.cuda.synchronize()
    dist.barrier()
    red.broadcast(root=world - 1)
    torch.cuda.synchronize()
    errs.append(float((red.flat - float(world)).abs().max()))
    dist.barrier()
    red.check(wait=True)
    red.close()
    return {"errs": np.array(errs)}


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_p2p_allreduce_matches_nccl():
    codes, out = _spawn("_allreduce_worker", 2)
    assert codes == [0, 0], codes
    for r in (0, 1):
        assert out[r]["errs"].max() < 1e-5, out[r]["errs"]


def _dp_worker(rank, world):
    import keras_b200 as keras

    keras.distribution.initialize()
    keras.distribution.set_distribution(keras.distribution.DataParallel())
    keras.utils.set_random_seed(11)
    inp = keras.Input((16, 16, 8))
    x = keras.layers.Conv2D(16, 3, padding="same")(inp)
    x = keras.layers.BatchNormalization()(x)
    x = keras.layers.Activation("relu")(x)
    x = keras.layers.GlobalAveragePooling2D()(x)
    out = keras.layers.Dense(5)(x)
    m = keras.Model(inp, out)
    m.compile(optimizer=keras.optimizers.SGD(0.05, momentum=0.9), loss=keras.losses.SparseCategoricalCrossentropy(from_logits=True))
    rng = np.random.RandomState(rank)
    xs, ys = rng.randn(8, 16, 16, 8).astype("float32"), rng.randint(0, 5, (8,))
    losses = [float(m.train_on_batch(xs, ys)) for _ in range(3)]
    m._parallel_engine.check(wait=True)
    used_p2p = m._parallel_engine._reducer is not None
    w = {f"w{i}": v for i, v in enumerate(m.get_weights())}
    w["losses"] = np.array(losses)
    w["p2p"] = np.array(used_p2p)
    m._parallel_engine.close()
    return w


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_data_parallel_replicas_stay_identical():
    codes, out = _spawn("_dp_worker", 2)
    assert codes == [0, 0], codes
    assert bool(out[0]["p2p"]) and bool(out[1]["p2p"])
    keys = [k for k in out[0] if k.startswith("w")]
    trainable_like = 0
    for k in keys:
        a, b = out[0][k], out[1][k]
        if a.shape == b.shape and np.array_equal(a, b):
            trainable_like += 1
    # kernels, biases, gamma, beta are bit-identical across replicas (moving statistics are per replica)
    assert trainable_like >= 6, trainable_like
    np.testing.assert_allclose(out[0]["losses"], out[1]["losses"], rtol=1e-5)


def _dp_graph_worker(rank, world):
    import keras_b200 as keras

    keras.distribution.initialize()
    keras.distribution.set_distribution(keras.distribution.DataParallel())

    def make(jit):
        keras.utils.set_random_seed(11)
        m = keras.Sequential([keras.layers.Input((32,)), keras.layers.Dense(64, activation="relu"), keras.layers.LayerNormalization(),
                              keras.layers.Dense(5)])
        m.compile(optimizer=keras.optimizers.Adam(1e-2), loss=keras.losses.SparseCategoricalCrossentropy(from_logits=True), metrics=["accuracy"],
                  jit_compile=jit)
        return m

    eager, graphed = make(False), make("auto")
    rng = np.random.RandomState(rank)
    xs, ys = rng.randn(4, 16, 32).astype("float32"), rng.randint(0, 5, (4, 16))
    rows = {"eager": [], "graphed": []}
    for step in range(8):
        rows["eager"].append(eager.train_on_batch(xs[step % 4], ys[step % 4]))
        rows["graphed"].append(graphed.train_on_batch(xs[step % 4], ys[step % 4]))
    for m in (eager, graphed):
        m._parallel_engine.check(wait=True)
    out = {"eager": np.array(rows["eager"]), "graphed": np.array(rows["graphed"]), "replays": np.array(graphed._graphed_step.replays),
           "disabled": np.array(str(graphed._graphed_step.failure_traceback or graphed._graphed_step.disabled)),
           "eager_replays": np.array(eager._graphed_step.replays)}
    for i, (a, b) in enumerate(zip(eager.get_weights(), graphed.get_weights())):
        out[f"e{i}"], out[f"g{i}"] = a, b
    for m in (eager, graphed):
        m._parallel_engine.close()
    return out


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_data_parallel_step_replays_as_cuda_graph():
    codes, out = _spawn("_dp_graph_worker", 2)
    assert codes == [0, 0], codes
    for r in (0, 1):
        assert str(out[r]["disabled"]) == "None", str(out[r]["disabled"])
        assert int(out[r]["replays"]) == 5 and int(out[r]["eager_replays"]) == 0
        np.testing.assert_allclose(out[r]["graphed"], out[r]["eager"], rtol=1e-5, atol=1e-6)
        for k in [k for k in out[r] if k.startswith("e") and k[1:].isdigit()]:
            np.testing.assert_allclose(out[r]["g" + k[1:]], out[r][k], rtol=1e-5, atol=1e-6)
    # loss and accuracy are the replica means: both ranks log the same numbers
    np.testing.assert_allclose(out[0]["graphed"], out[1]["graphed"], rtol=1e-6)


def _dp_overlap_worker(rank, world):
    """The same model trained with the gradient reduction after the backward pass and overlapped with it in small buckets."""
    import keras_b200 as keras

    keras.distribution.initialize()
    keras.distribution.set_distribution(keras.distribution.DataParallel())
    out = {}
    for policy in ("float32", "mixed_bfloat16"):
        keras.config.set_dtype_policy(policy)
        for overlap in ("0", "1"):
            os.environ["KERAS_B200_DP_OVERLAP"] = overlap
            os.environ["KERAS_B200_DP_BUCKET_BYTES"] = "4096"
            keras.utils.set_random_seed(31)
            m = keras.Sequential([keras.layers.Input((32,)), keras.layers.Dense(64, activation="relu"), keras.layers.LayerNormalization(),
                                  keras.layers.Dense(64, activation="gelu"), keras.layers.Dense(5)])
            m.compile(optimizer=keras.optimizers.SGD(0.05, momentum=0.9), loss=keras.losses.SparseCategoricalCrossentropy(from_logits=True))
            rng = np.random.RandomState(7 + rank)
            xs, ys = rng.randn(4, 32, 32).astype("float32"), rng.randint(0, 5, (4, 32))
            losses = [float(m.train_on_batch(xs[i % 4], ys[i % 4])) for i in range(9)]
            engine = m._parallel_engine
            engine.check(wait=True)
            schedule = getattr(engine, "_overlap", None)
            key = f"{policy}_{overlap}"
            out[key + "_losses"] = np.array(losses)
            out[key + "_buckets"] = np.array(len(schedule.buckets) if schedule is not None else 0)
            out[key + "_launched"] = np.array(schedule.launched if schedule is not None else 0)
            out[key + "_replays"] = np.array(m._graphed_step.replays if m._graphed_step is not None else -1)
            out[key + "_why"] = np.array(str(m._graphed_step.failure_traceback or m._graphed_step.disabled) if m._graphed_step is not None else "no stepper")
            for i, w in enumerate(m.get_weights()):
                out[f"{key}_w{i}"] = w
            engine.close()
    keras.config.set_dtype_policy("float32")
    return out


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_gradient_reduction_overlapped_with_backward_gives_the_same_weights():
    codes, out = _spawn("_dp_overlap_worker", 2)
    assert codes == [0, 0], codes
    for r in (0, 1):
        for policy in ("float32", "mixed_bfloat16"):
            assert int(out[r][f"{policy}_0_buckets"]) == 0
            assert int(out[r][f"{policy}_1_buckets"]) >= 2 and int(out[r][f"{policy}_1_launched"]) == int(out[r][f"{policy}_1_buckets"])
            assert int(out[r][f"{policy}_1_replays"]) >= 5, str(out[r][f"{policy}_1_why"])  # the overlapped step is recorded and replayed as well
            np.testing.assert_array_equal(out[r][f"{policy}_1_losses"], out[r][f"{policy}_0_losses"])
            for k in [k for k in out[r] if k.startswith(f"{policy}_0_w")]:
                np.testing.assert_array_equal(out[r][k.replace("_0_w", "_1_w")], out[r][k])


def _equivalence_model(keras):
    keras.utils.set_random_seed(23)
    m = keras.Sequential([keras.layers.Input((32,)), keras.layers.Dense(64, activation="relu"), keras.layers.LayerNormalization(),
                          keras.layers.Dense(64, activation="gelu"), keras.layers.Dense(5)])
    m.compile(optimizer=keras.optimizers.SGD(0.05, momentum=0.9), loss=keras.losses.SparseCategoricalCrossentropy(from_logits=True))
    return m


def _equivalence_data():
    rng = np.random.RandomState(5)
    return rng.randn(6, 64, 32).astype("float32"), rng.randint(0, 5, (6, 64))


def _dp_equivalence_worker(rank, world):
    import keras_b200 as keras

    keras.distribution.initialize()
    keras.distribution.set_distribution(keras.distribution.DataParallel())
    m = _equivalence_model(keras)
    xs, ys = _equivalence_data()
    per = xs.shape[1] // world
    losses = [float(m.train_on_batch(xs[i][rank * per:(rank + 1) * per], ys[i][rank * per:(rank + 1) * per])) for i in range(6)]
    m._parallel_engine.check(wait=True)
    out = {"losses": np.array(losses)}
    for i, w in enumerate(m.get_weights()):
        out[f"w{i}"] = w
    m._parallel_engine.close()
    return out


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_replicas_at_equal_global_batch_follow_the_single_gpu_run():
    """Mean loss and mean gradient over two half batches are those of the whole batch: the curves agree to fp32 reordering."""
    import keras_b200 as keras

    codes, out = _spawn("_dp_equivalence_worker", 2)
    assert codes == [0, 0], codes
    single = _equivalence_model(keras)
    xs, ys = _equivalence_data()
    losses = [float(single.train_on_batch(xs[i], ys[i])) for i in range(6)]
    np.testing.assert_allclose(out[0]["losses"], losses, rtol=2e-4, atol=2e-5)
    for i, w in enumerate(single.get_weights()):
        np.testing.assert_allclose(out[0][f"w{i}"], w, rtol=2e-3, atol=2e-5)
        np.testing.assert_array_equal(out[0][f"w{i}"], out[1][f"w{i}"])


def test_bounded_wait_reports_timeout_and_context_survives():
    from keras_b200.kernels import ops as kops

    lib = kops._lib()
    flag = torch.zeros(64, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.kb200_wait_selftest(ctypes.c_void_p(flag.data_ptr()), ctypes.c_void_p(status.data_ptr()), ctypes.c_longlong(200), kops._stream())
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) != 0  # the wait ran out and said so
    # the context is still usable
    assert float((torch.ones(8, device="cuda") * 2).sum().item()) == 16.0
    # and a flag that is set lets the wait pass
    flag.fill_(1)
    status.zero_()
    lib.kb200_wait_selftest(ctypes.c_void_p(flag.data_ptr()), ctypes.c_void_p(status.data_ptr()), ctypes.c_longlong(200), kops._stream())
    torch.cuda.synchronize()
    assert int(status.item()) == 0


def _fused_gemm_worker(rank, world):
    import torch.distributed as dist

    import keras_b200 as keras
    from keras_b200.parallel.fused_gemm import ColumnParallelLinear, FusedGemmContext, RowParallelLinear

    keras.distribution.initialize()
    fused = FusedGemmContext()
    g = torch.Generator(device="cuda").manual_seed(7 + rank)
    errs = []
    for Ms, K, N in [(256, 512, 768), (1024, 1024, 2048), (256, 512, 768)]:
        M = Ms * world
        # all-gather -> GEMM
        x_rows = torch.randn(Ms, K, device="cuda", generator=g).bfloat16()
        w = (torch.randn(K, N, device="cuda", generator=g) * 0.05).bfloat16()
        parts = [torch.empty_like(x_rows) for _ in range(world)]
        dist.all_gather(parts, x_rows)
        ref = torch.cat(parts).float() @ w.float()
        out, gathered = fused.all_gather_gemm(x_rows, w)
        torch.cuda.synchronize()
        errs.append(float((out.float() - ref).abs().max() / ref.abs().max()))
        errs.append(float((gathered.float() - torch.cat(parts).float()).abs().max()))
        # GEMM -> reduce-scatter
        a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        full = a.float() @ w.float()
        dist.all_reduce(full)
        got = fused.gemm_reduce_scatter(a, w)
        torch.cuda.synchronize()
        ref_rows = full[rank * Ms:(rank + 1) * Ms]
        errs.append(float((got.float() - ref_rows).abs().max() / ref_rows.abs().max()))
        dist.barrier()
    # autograd pair: column-parallel up projection, row-parallel down projection on row-sharded activations
    Ms, D, F = 256, 512, 1024
    x_rows = torch.randn(Ms, D, device="cuda", generator=g).bfloat16().requires_grad_(True)
    w1 = (torch.randn(D, F, device="cuda", generator=g) * 0.05).bfloat16().requires_grad_(True)
    w2 = (torch.randn(F, D, device="cuda", generator=g) * 0.05).bfloat16().requires_grad_(True)
    h = ColumnParallelLinear.apply(x_rows, w1, None, fused)
    y_rows = RowParallelLinear.apply(torch.relu(h), w2, fused)
    dy = torch.randn(Ms, D, device="cuda", generator=g).bfloat16()
    y_rows.backward(dy)
    torch.cuda.synchronize()
    # reference with NCCL collectives and fp32 math
    parts = [torch.empty_like(x_rows) for _ in range(world)]
    dist.all_gather(parts, x_rows.detach())
    xf = torch.cat(parts).float().requires_grad_(True)
    w1f, w2f = w1.detach().float().requires_grad_(True), w2.detach().float().requires_grad_(True)
    yf = torch.relu(xf @ w1f) @ w2f
    dist.all_reduce(yf.data)
    dparts = [torch.empty_like(dy) for _ in range(world)]
    dist.all_gather(dparts, dy)
    yf.backward(torch.cat(dparts).float())
    dxf = xf.grad.clone()
    dist.all_reduce(dxf)
    rel = lambda a, b: float((a.float() - b).abs().max() / (b.abs().max() + 1e-6))
    errs.append(rel(y_rows, yf.data[rank * Ms:(rank + 1) * Ms]))
    errs.append(rel(x_rows.grad, dxf[rank * Ms:(rank + 1) * Ms]))
    errs.append(rel(w1.grad, w1f.grad))
    errs.append(rel(w2.grad, w2f.grad))
    fused.check()
    dist.barrier()
    fused.close()
    return {"errs": np.array(errs)}


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_allgather_gemm_and_gemm_reduce_scatter_match_nccl(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    codes, out = _spawn("_fused_gemm_worker", world)
    assert codes == [0] * world, codes
    for r in range(world):
        assert (out[r]["errs"] < 3e-2).all(), out[r]["errs"]


@pytest.mark.parametrize("world", [4, 8])
def test_p2p_collectives_match_nccl_on_more_ranks(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    codes, out = _spawn("_allreduce_worker", world)
    assert codes == [0] * world, codes
    for r in range(world):
        assert out[r]["errs"].max() < 1e-5, out[r]["errs"]


def _sp_gpu_worker(rank, world):
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
    keras.config.set_dtype_policy("mixed_bfloat16")
    keras.utils.set_random_seed(5)
    d, T, B = 256, 128, 8
    inp = keras.Input((T, d))
    h = inp
    for i in range(2):
        a = keras.layers.LayerNormalization(name=f"ln1_{i}")(h)
        a = keras.layers.MultiHeadAttention(num_heads=4, key_dim=64, name=f"attn_{i}")(a, a, use_causal_mask=True)
        h = keras.layers.Add(name=f"res1_{i}")([h, a])
        m = keras.layers.LayerNormalization(name=f"ln2_{i}")(h)
        m = keras.layers.Dense(1024, activation="relu", name=f"up_{i}")(m)
        m = keras.layers.Dense(d, name=f"down_{i}")(m)
        h = keras.layers.Add(name=f"res2_{i}")([h, m])
    out = keras.layers.Dense(8, name="head")(keras.layers.LayerNormalization(name="ln_f")(h))
    model = keras.Model(inp, out)
    model.compile(optimizer=keras.optimizers.SGD(0.002), loss="mse")
    rng = np.random.RandomState(3)
    x, y = rng.randn(B, T, d).astype("float32"), rng.randn(B, T, 8).astype("float32")
    losses = [float(model.train_on_batch(x, y)) for _ in range(4)]
    sp = global_state.get_global_attribute("tp_sequence_parallel")
    used = 0 if sp is None or sp.fused is None else sp.fused.epoch
    model._parallel_engine.check(wait=True)
    torch.cuda.synchronize()
    import torch.distributed as dist

    dist.barrier()
    model._parallel_engine.close()
    return {"losses": np.array(losses), "fused_calls": np.array(used)}


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sequence_parallel_training_uses_fused_gemms_and_matches_unfused():
    codes, fused = _spawn("_sp_gpu_worker", 2)
    assert codes == [0, 0], codes
    os.environ["KERAS_B200_TP_FUSED"] = "0"
    try:
        codes, plain = _spawn("_sp_gpu_worker", 2)
    finally:
        del os.environ["KERAS_B200_TP_FUSED"]
    assert codes == [0, 0], codes
    assert int(fused[0]["fused_calls"]) > 0 and int(plain[0]["fused_calls"]) == 0
    np.testing.assert_allclose(fused[0]["losses"], fused[1]["losses"], rtol=1e-6)
    np.testing.assert_allclose(fused[0]["losses"], plain[0]["losses"], rtol=3e-2)
