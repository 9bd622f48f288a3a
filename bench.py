"""Headline benchmark: ResNet-50 v1 training throughput (images/sec), mixed_bfloat16, SGD momentum.

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference] [--config resnet50]

For N>1 launch one rank per GPU with ``python -m torch.distributed.run``.  Rank 0 prints one JSON
line.  ``value`` is the job-wide images/sec timed on the device (CUDA events, max over ranks) through
``Model.train_on_batch`` on device-resident synthetic inputs; ``e2e`` is the same metric through
``Model.fit`` over a generator of pinned host batches: every step copies its batch host→device and a
callback reads the step's loss back to the host.  Both arms (``--impl ours`` and ``--impl reference``,
the unmodified reference Keras on its torch backend from ``baseline/_ref``) make the same calls.

At N=4 and N=8 the line also carries ``"secondary"``: the 8B decoder under ``ModelParallel`` (tp4, dp2 x tp4), measured
the same way for 10 steps, with the same model on library collectives as its baseline.  A watchdog prints the primary
line without it if that measurement does not finish in time.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))

CONFIGS = {
    "resnet50": {"kind": "resnet", "model": "ResNet-50 v1", "per_gpu_batch": 256, "image": 224, "classes": 1000},
    "resnet50_small": {"kind": "resnet", "model": "ResNet-50 v1 (smoke size)", "per_gpu_batch": 16, "image": 64, "classes": 1000},
    "gpt2": {"kind": "decoder", "model": "GPT-2 small (12 x 768, 12 heads, MLP 3072, vocab 50257)", "per_gpu_batch": 16, "seq": 1024, "vocab": 50257,
             "layers": 12, "d": 768, "heads": 12, "ffn": 3072},
    "llama8b": {"kind": "llama", "model": "Llama-style 8B decoder (32 x 4096, 32 query / 8 KV heads, SwiGLU 14336, vocab 128256, RoPE theta 5e5)",
                "global_batch": 16, "seq": 4096, "vocab": 128256, "layers": 32, "d": 4096, "q_heads": 32, "kv_heads": 8, "ffn": 14336,
                "rope_theta": 5e5, "model_axis": 4},
    "llama8b_4layer": {"kind": "llama", "model": "4 layers of the Llama-style 8B decoder (4096 wide, 32 query / 8 KV heads, SwiGLU 14336, vocab 128256)",
                       "global_batch": 2, "seq": 4096, "vocab": 128256, "layers": 4, "d": 4096, "q_heads": 32, "kv_heads": 8, "ffn": 14336,
                       "rope_theta": 5e5, "model_axis": 1},
    "llama_small": {"kind": "llama", "model": "Llama-style decoder (smoke size)", "global_batch": 8, "seq": 256, "vocab": 2048, "layers": 2, "d": 512,
                    "q_heads": 8, "kv_heads": 4, "ffn": 1536, "rope_theta": 5e5, "model_axis": 4},
    "gpt_fp8": {"kind": "decoder", "model": "1.3B decoder (24 x 2048, 16 heads, MLP 8192, vocab 50257), float8 policy on Dense/EinsumDense",
                "per_gpu_batch": 8, "seq": 2048, "vocab": 50257, "layers": 24, "d": 2048, "heads": 16, "ffn": 8192, "float8": True},
    "gpt_bf16_1b3": {"kind": "decoder", "model": "1.3B decoder (24 x 2048, 16 heads, MLP 8192, vocab 50257), bf16", "per_gpu_batch": 8, "seq": 2048,
                     "vocab": 50257, "layers": 24, "d": 2048, "heads": 16, "ffn": 8192},
    "gpt_int8_predict": {"kind": "decoder", "model": "1.3B decoder (24 x 2048, 16 heads, MLP 8192, vocab 50257), quantize('int8'), predict", "per_gpu_batch": 64,
                         "seq": 128, "vocab": 50257, "layers": 24, "d": 2048, "heads": 16, "ffn": 8192, "predict": True, "int8": True},
    "gpt_int8_predict_small": {"kind": "decoder", "model": "decoder (smoke size), quantize('int8'), predict", "per_gpu_batch": 8, "seq": 64, "vocab": 1024,
                               "layers": 2, "d": 128, "heads": 4, "ffn": 512, "predict": True, "int8": True},
    "gpt2_small": {"kind": "decoder", "model": "GPT-2 shaped (smoke size)", "per_gpu_batch": 4, "seq": 128, "vocab": 1024, "layers": 2, "d": 128,
                   "heads": 4, "ffn": 512},
}


def build_model(keras, cfg):
    """Model + optimizer of a config, written against the public Keras API only (both arms call this)."""
    if cfg["kind"] == "resnet":
        img = cfg["image"]
        model = keras.applications.ResNet50(weights=None, input_shape=(img, img, 3), classes=cfg["classes"])
        model.compile(optimizer=keras.optimizers.SGD(learning_rate=0.1, momentum=0.9), loss="sparse_categorical_crossentropy")
        return model
    if cfg["kind"] == "llama":
        return build_llama(keras, cfg)
    seq, d = cfg["seq"], cfg["d"]

    class PositionEmbedding(keras.layers.Layer):
        def build(self, input_shape):
            self.table = self.add_weight(shape=(seq, d), initializer="random_normal", name="table")

        def call(self, x):
            return x + keras.ops.cast(self.table, x.dtype)

    tokens = keras.Input((seq,), dtype="int32")
    h = keras.layers.Embedding(cfg["vocab"], d, name="wte")(tokens)
    h = PositionEmbedding(name="wpe")(h)
    for i in range(cfg["layers"]):
        a = keras.layers.LayerNormalization(epsilon=1e-5, name=f"ln1_{i}")(h)
        a = keras.layers.MultiHeadAttention(cfg["heads"], d // cfg["heads"], name=f"attn_{i}")(a, a, use_causal_mask=True)
        h = keras.layers.Add(name=f"res1_{i}")([h, a])
        m = keras.layers.LayerNormalization(epsilon=1e-5, name=f"ln2_{i}")(h)
        m = keras.layers.Dense(cfg["ffn"], activation="gelu", name=f"up_{i}")(m)
        m = keras.layers.Dense(d, name=f"down_{i}")(m)
        h = keras.layers.Add(name=f"res2_{i}")([h, m])
    h = keras.layers.LayerNormalization(epsilon=1e-5, name="ln_f")(h)
    logits = keras.layers.Dense(cfg["vocab"], use_bias=False, name="lm_head")(h)
    model = keras.Model(tokens, logits)
    if cfg.get("int8"):
        # post-training quantisation of every Dense / EinsumDense kernel to int8 (per-channel scales, activations quantised per row at run time)
        model.quantize("int8")
    if cfg.get("float8"):
        # the float8 dtype policy on every Dense / EinsumDense (e4m3 operands, e5m2 output gradients, delayed scaling)
        model.quantize("float8")
    model.compile(optimizer=keras.optimizers.AdamW(learning_rate=3e-4, weight_decay=0.1),
                  loss=keras.losses.SparseCategoricalCrossentropy(from_logits=True))
    return model


def build_llama(keras, cfg):
    """Llama-style decoder from Keras layers: RMSNormalization, GroupedQueryAttention (rotary embedding added by
    overriding its attention hook), SwiGLU MLP from three bias-free Dense layers."""
    ops = keras.ops
    seq, d, hd = cfg["seq"], cfg["d"], cfg["d"] // cfg["q_heads"]

    class RotaryGQA(keras.layers.GroupedQueryAttention):
        def _rope(self, x):
            half = hd // 2
            pos = ops.cast(ops.arange(seq), "float32")
            inv = ops.exp(ops.cast(ops.arange(half), "float32") * (-float(np_log(cfg["rope_theta"])) / half))
            ang = ops.expand_dims(ops.expand_dims(pos, -1) * ops.expand_dims(inv, 0), 1)  # [T, 1, half]
            cos, sin = ops.cast(ops.cos(ang), x.dtype), ops.cast(ops.sin(ang), x.dtype)
            x1, x2 = x[..., :half], x[..., half:]
            return ops.concatenate([x1 * cos - x2 * sin, x2 * cos + x1 * sin], axis=-1)

        def _compute_attention(self, query, key, value, attention_mask=None, training=None):
            return super()._compute_attention(self._rope(query), self._rope(key), value, attention_mask=attention_mask, training=training)

    tokens = keras.Input((seq,), dtype="int32")
    h = keras.layers.Embedding(cfg["vocab"], d, name="embed")(tokens)
    for i in range(cfg["layers"]):
        a = keras.layers.RMSNormalization(epsilon=1e-5, name=f"attn_norm_{i}")(h)
        a = RotaryGQA(head_dim=hd, num_query_heads=cfg["q_heads"], num_key_value_heads=cfg["kv_heads"], use_bias=False, name=f"attn_{i}")(
            a, a, use_causal_mask=True)
        h = keras.layers.Add(name=f"res1_{i}")([h, a])
        m = keras.layers.RMSNormalization(epsilon=1e-5, name=f"mlp_norm_{i}")(h)
        g = keras.layers.Dense(cfg["ffn"], use_bias=False, name=f"gate_{i}")(m)
        u = keras.layers.Dense(cfg["ffn"], use_bias=False, name=f"up_{i}")(m)
        m = keras.layers.Multiply(name=f"glu_{i}")([keras.layers.Activation("silu", name=f"silu_{i}")(g), u])
        m = keras.layers.Dense(d, use_bias=False, name=f"down_{i}")(m)
        h = keras.layers.Add(name=f"res2_{i}")([h, m])
    h = keras.layers.RMSNormalization(epsilon=1e-5, name="final_norm")(h)
    logits = keras.layers.Dense(cfg["vocab"], use_bias=False, name="lm_head")(h)
    model = keras.Model(tokens, logits)
    model.compile(optimizer=keras.optimizers.AdamW(learning_rate=3e-4, weight_decay=0.1),
                  loss=keras.losses.SparseCategoricalCrossentropy(from_logits=True))
    return model


def np_log(x):
    import math

    return math.log(x)


def llama_layout(keras, cfg, world):
    """(distribution, data replicas) for the decoder: DeviceMesh (data, model), q/k/v/gate/up sharded by columns (heads /
    hidden units), o/down by rows."""
    model_axis = min(cfg["model_axis"], world)
    data_axis = world // model_axis
    mesh = keras.distribution.DeviceMesh((data_axis, model_axis), ["data", "model"], devices=keras.distribution.list_devices())
    lm = keras.distribution.LayoutMap(mesh)
    lm["attn_.*/(query|key|value)/kernel"] = (None, "model", None)
    lm["attn_.*/attention_output/kernel"] = ("model", None, None)
    lm["(gate|up)_.*/kernel"] = (None, "model")
    lm["down_.*/kernel"] = ("model", None)
    if cfg.get("shard_head", True):
        lm["lm_head/kernel"] = (None, "model")  # each rank computes its slice of the vocabulary; the logits are gathered
    return keras.distribution.ModelParallel(layout_map=lm, batch_dim_name="data"), data_axis


def make_batches(torch, cfg, rank, n_buf=3):
    """Pinned host batches of the config's shape (synthetic)."""
    gen = torch.Generator().manual_seed(1234 + rank)
    bs = cfg["per_gpu_batch"]  # for the llama configs: the batch of this rank's data replica (set by run_ours)
    if cfg["kind"] == "resnet":
        img, classes = cfg["image"], cfg["classes"]
        xs = [torch.randn((bs, img, img, 3), generator=gen, dtype=torch.float32).pin_memory() for _ in range(n_buf)]
        ys = [torch.randint(0, classes, (bs,), generator=gen, dtype=torch.int64).pin_memory() for _ in range(n_buf)]
    else:
        xs = [torch.randint(0, cfg["vocab"], (bs, cfg["seq"]), generator=gen, dtype=torch.int32).pin_memory() for _ in range(n_buf)]
        ys = [torch.randint(0, cfg["vocab"], (bs, cfg["seq"]), generator=gen, dtype=torch.int64).pin_memory() for _ in range(n_buf)]
    return xs, ys


def describe(cfg, world):
    """(metric, unit, samples per step per GPU, config dict) for the JSON line."""
    bs = cfg["per_gpu_batch"]
    if cfg["kind"] == "resnet":
        return ("ResNet-50 training throughput", "images/sec", bs,
                {"model": cfg["model"], "global_batch": bs * world, "per_gpu_batch": bs, "image_size": cfg["image"], "seq_len": None,
                 "parallelism": f"dp{world}", "optimizer": "SGD(momentum=0.9, lr=0.1)", "policy": "mixed_bfloat16",
                 "l2_hygiene": "inputs_larger_than_L2 (per-step batch and activations exceed 126 MB)"})
    if cfg["kind"] == "llama":
        model_axis = min(cfg["model_axis"], world)
        data_axis = world // model_axis
        return ("decoder training throughput (ModelParallel)", "tokens/sec", cfg["global_batch"] * cfg["seq"] / world,
                {"model": cfg["model"], "global_batch": cfg["global_batch"], "seq_len": cfg["seq"], "parallelism": f"dp{data_axis}xtp{model_axis}",
                 "sharding": "q/k/v/gate/up and the vocabulary projection by columns, o/down by rows; batch-sharded activations between blocks (fused all-gather->GEMM, GEMM->reduce-scatter)",
                 "optimizer": "AdamW(lr=3e-4, weight_decay=0.1)", "policy": "mixed_bfloat16",
                 "l2_hygiene": "inputs_larger_than_L2 (weights and activations of a step exceed 126 MB)"})
    return ("decoder training throughput", "tokens/sec", bs * cfg["seq"],
            {"model": cfg["model"], "global_batch": bs * world, "per_gpu_batch": bs, "seq_len": cfg["seq"], "parallelism": f"dp{world}",
             "optimizer": "AdamW(lr=3e-4, weight_decay=0.1)", "policy": "mixed_bfloat16" + (" + float8 quantization of Dense/EinsumDense" if cfg.get("float8") else ""),
             "l2_hygiene": "inputs_larger_than_L2 (weights, logits and activations of a step exceed 126 MB)"})


class ClockSampler:
    """SM clock and throttle reasons of this rank's GPU while timing runs.

    One ``nvidia-smi`` process per rank, started before the timed region, loops on its own (``-lms``) and appends to a file;
    it is ended by PID afterwards and the file is read.  Nothing is spawned and no Python thread runs during the timed region:
    forking a process that maps a hundred gigabytes of device memory stalls the interpreter for milliseconds, and under data
    parallelism every rank waits for the slowest."""

    FIELDS = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    PERIOD_MS = 250

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.path = None

    def _command(self, loop):
        cmd = ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.index)]
        return cmd + ["-lms", str(self.PERIOD_MS)] if loop else cmd

    def start(self):
        import tempfile

        fd, self.path = tempfile.mkstemp(prefix=f"clocks_gpu{self.index}_", suffix=".csv")
        try:
            self.proc = subprocess.Popen(self._command(loop=True), stdout=fd, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        finally:
            os.close(fd)

    def stop(self):
        text = ""
        if self.proc is not None:
            self.proc.terminate()  # this process only, by its PID
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        if self.path is not None:
            try:
                with open(self.path) as f:
                    text = f.read()
                os.unlink(self.path)
            except OSError:
                pass
        if not text.strip():
            # the looping process wrote nothing (buffered output lost with it): one sample right after the region
            try:
                text = subprocess.run(self._command(loop=False), capture_output=True, text=True, timeout=5).stdout
            except Exception:
                text = ""
        clocks, reasons, maxc = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in text.strip().splitlines():
            s = [p.strip() for p in line.split(",")]
            try:
                clocks.append(float(s[0]))
                maxc = float(s[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": maxc, "reasons": sorted(reasons), "samples": len(clocks)}


def _dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def _timed(torch, dist, world, steps, step_fn):
    """Barrier + sync, K steps between CUDA events, sync; returns max-over-ranks milliseconds."""
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        step_fn(i)
    end.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = start.elapsed_time(end)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def run_e2e(keras, torch, dist, world, steps, warmup, model, host_x, host_y, last):
    """K training steps through ``Model.fit`` on a generator of pinned host batches, the loss read back to the host after
    every step by a callback.  Falls back to a ``train_on_batch`` loop when ``fit`` refuses the generator (the reference
    rejects generators under a multi-process distribution).  Returns (milliseconds, api description)."""
    n_buf = len(host_x)

    class LossReader(keras.callbacks.Callback):
        def on_train_batch_end(self, batch, logs=None):
            last["loss"] = float(logs["loss"])  # 4 bytes device -> host every step

    def batches():
        i = 0
        while True:
            yield host_x[i % n_buf], host_y[i % n_buf]
            i += 1

    def fit_steps(n):
        model.fit(batches(), steps_per_epoch=n, epochs=1, verbose=0, callbacks=[LossReader()])

    def batch_steps(n):
        for i in range(n):
            last["loss"] = model.train_on_batch(host_x[i % n_buf], host_y[i % n_buf])
            if isinstance(last["loss"], (list, tuple)):
                last["loss"] = last["loss"][0]

    runner, api = fit_steps, "Model.fit(generator of pinned host batches, steps_per_epoch=K) + loss read in on_train_batch_end"
    try:
        fit_steps(max(1, min(warmup, 3)))
    except Exception as e:
        runner, api = batch_steps, f"Model.train_on_batch(pinned host tensors) -> float loss (fit refused the generator: {type(e).__name__})"
        batch_steps(max(1, min(warmup, 3)))
    ms = _timed(torch, dist, world, 1, lambda i: runner(steps))
    return ms, api


def measure_predict(keras, torch, args, cfg, local, impl, launch_count=None):
    """Inference throughput of a quantised model on one GPU, through the public API only (both arms run this function):
    ``value`` times ``model(tokens, training=False)`` on device-resident batches; ``e2e`` times ``model.predict_on_batch`` on
    pinned host batches, which copies the tokens in and the logits out every step."""
    model = build_model(keras, cfg)
    n_buf = 3
    host_x, _ = make_batches(torch, cfg, 0, n_buf)
    dev_x = [t.cuda() for t in host_x]
    bs, seq = cfg["per_gpu_batch"], cfg["seq"]
    last = {}

    def dev_step(i):
        with torch.no_grad():
            last["out"] = model(dev_x[i % n_buf], training=False)

    def host_step(i):
        last["np"] = model.predict_on_batch(host_x[i % n_buf])

    for i in range(max(args.warmup, 3)):
        dev_step(i)
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = launch_count() if launch_count else 0
    ms = _timed(torch, None, 1, args.steps, dev_step)
    launches = (launch_count() - launches0) if launch_count else 0
    clocks = sampler.stop()
    for i in range(3):
        host_step(i)
    e2e_steps = max(3, args.steps // 4)
    ms_e2e = _timed(torch, None, 1, e2e_steps, host_step)
    out_bytes = int(last["np"].nbytes)
    tokens = bs * seq
    return {
        "metric": "decoder int8 predict throughput", "value": tokens * args.steps / (ms / 1e3), "unit": "tokens/sec", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 weights and activations, bf16 elsewhere", "data": "synthetic", "impl": impl,
        "config": {"model": cfg["model"], "global_batch": bs, "per_gpu_batch": bs, "seq_len": seq, "parallelism": "dp1", "policy": "mixed_bfloat16 + quantize('int8')",
                   "l2_hygiene": "inputs_larger_than_L2 (1.3 GB of int8 weights and the logits of a step exceed 126 MB)"},
        "clocks": clocks,
        "e2e": {"value": tokens * e2e_steps / (ms_e2e / 1e3), "unit": "tokens/sec", "ms_per_step": ms_e2e / e2e_steps, "steps": e2e_steps,
                "h2d_bytes_per_step": int(host_x[0].numel() * host_x[0].element_size()), "d2h_bytes_per_step": out_bytes,
                "api": "Model.predict_on_batch(pinned host tokens) -> numpy logits"},
        "gpu_launches": int(launches),
    }


def measure_ours(keras, torch, dist, args, cfg, rank, world, local, steps, warmup):
    """Build the config's model under the distribution that is set, time ``steps`` training steps twice (device-resident
    inputs through ``train_on_batch``; pinned host batches through ``fit``) and return the result row (every rank returns
    it; rank 0 prints)."""
    from keras_b200.kernels import ops as kops

    data_rank = rank
    if cfg["kind"] == "llama":
        model_axis = min(cfg["model_axis"], world)
        data_axis = max(1, world // model_axis)
        cfg = dict(cfg, per_gpu_batch=cfg["global_batch"] // data_axis)
        data_rank = rank // (world // data_axis)  # ranks of one model-parallel group read the same batch
    model = build_model(keras, cfg)
    n_buf = 3
    host_x, host_y = make_batches(torch, cfg, data_rank, n_buf)
    dev_x = [t.cuda() for t in host_x]
    dev_y = [t.cuda() for t in host_y]
    metric, unit, per_step, cfg_out = describe(cfg, world)

    last = {}
    model.train_on_batch(host_x[0], host_y[0])  # builds model, optimizer, kernels

    def dev_step(i):
        last["loss"] = model.train_on_batch(dev_x[i % n_buf], dev_y[i % n_buf])

    for i in range(warmup):
        dev_step(i)
    if args.profile_range:
        # one step between cudaProfilerStart/Stop for `ncu --profile-from-start off`
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        dev_step(0)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        return None, model
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = kops.launch_count()
    replays0 = getattr(getattr(model, "_graphed_step", None), "replays", 0)
    ms = _timed(torch, dist, world, steps, dev_step)
    launches = kops.launch_count() - launches0
    replays_value = getattr(getattr(model, "_graphed_step", None), "replays", 0) - replays0
    clocks = sampler.stop()
    replays_before_e2e = getattr(getattr(model, "_graphed_step", None), "replays", 0)
    ms_e2e, e2e_api = run_e2e(keras, torch, dist, world, steps, warmup, model, host_x, host_y, last)
    total = per_step * world * steps
    value = total / (ms / 1e3)
    out = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": cfg_out,
        "clocks": clocks,
        "e2e": {"value": total / (ms_e2e / 1e3), "unit": unit, "ms_per_step": ms_e2e / steps,
                "h2d_bytes_per_step": int(host_x[0].numel() * host_x[0].element_size() + host_y[0].numel() * host_y[0].element_size()),
                "d2h_bytes_per_step": 4,
                "api": e2e_api},
        "gpu_launches": int(launches),
        "final_loss": float(last["loss"]) if not isinstance(last["loss"], (list, tuple)) else float(last["loss"][0]),
    }
    stepper = getattr(model, "_graphed_step", None)
    if stepper is not None:
        # how the steps were issued: replays of the captured CUDA graph of the step, or eagerly (and why)
        out["step_graph"] = {"replays": int(stepper.replays), "replays_in_value_region": int(replays_value), "replays_in_e2e_region": int(stepper.replays - replays_before_e2e),
                             "eager_reason": stepper.disabled}
    return out, model


def _release(torch, model):
    """Close the model's parallel engine (peer buffers), drop what keeps its device memory alive (the captured step graph
    and its pool, the gradient arena, optimizer state) and give the memory back before the next model is built."""
    import gc

    torch.cuda.synchronize()
    engine = getattr(model, "_parallel_engine", None)
    if engine is not None:
        engine.check(wait=True)
        engine.close()
        model._parallel_engine = None
    # whatever else still refers to the model or its optimizer (callbacks, histories), the device memory goes now
    opt = getattr(model, "optimizer", None)
    variables = list(getattr(model, "variables", []))
    if opt is not None:
        variables += list(getattr(opt, "variables", []))
        for attr in ("_fused_plan", "_momentums", "_velocities", "momentums"):
            if hasattr(opt, attr):
                try:
                    setattr(opt, attr, None)
                except Exception:
                    pass
    for v in variables:
        for attr in ("_value", "_shadow", "_shadow_tensor"):
            try:
                object.__setattr__(v, attr, None)
            except Exception:
                pass
    arena = getattr(model, "_grad_arena", None)
    if arena is not None:
        arena.flat, arena.views = None, []
    for attr in ("_graphed_step", "train_function", "test_function", "predict_function", "_grad_arena", "optimizer", "_device_stager"):
        try:
            setattr(model, attr, None)
        except Exception:
            pass
    gc.collect()
    torch.cuda.empty_cache()


SECONDARY_CONFIG = "llama8b"
SECONDARY_STEPS = 10


def run_secondary(keras, torch, dist, args, rank, world, local):
    """The ModelParallel half of the headline: the 8B decoder's training throughput at this N (tp4 at N=4, dp2 x tp4 at N=8)
    through the fused all-gather->GEMM / GEMM->reduce-scatter kernels, and the same model with those collectives on the
    library path (``KERAS_B200_TP_FUSED=0``) as its stated baseline: the reference has no torch-backend model parallelism
    to compare with."""
    cfg = CONFIGS[args.secondary_config]
    # weak scaling over the data axis: each model-parallel group of `model_axis` GPUs keeps the per-replica batch of the
    # 8-GPU layout (global batch 16 over 2 replicas), so N=4 (one replica) runs global batch 8
    model_axis = min(cfg["model_axis"], world)
    replicas = max(1, world // model_axis)
    cfg = dict(cfg, global_batch=max(1, cfg["global_batch"] // 2) * replicas)
    rows, failure = {}, None
    for label, fused in (("fused", "1"), ("library_collectives", "0")):
        os.environ["KERAS_B200_TP_FUSED"] = fused
        distribution, _ = llama_layout(keras, cfg, world)
        keras.distribution.set_distribution(distribution)
        free0 = torch.cuda.mem_get_info()[0] / 2**30
        held0 = torch.cuda.memory_allocated() / 2**30
        try:
            row, model = measure_ours(keras, torch, dist, args, cfg, rank, world, local, SECONDARY_STEPS, 3)
        except Exception as e:
            failure = (f"{label}: {type(e).__name__}: {str(e)[:160]} [free before build {free0:.1f} GiB, still allocated before it "
                       f"{held0:.1f} GiB, peak {torch.cuda.max_memory_allocated() / 2**30:.1f} GiB]")
            if label == "fused":
                raise RuntimeError(failure) from None
            break  # the product's number stands; its baseline is reported as unavailable
        row["free_gib_before_build"] = round(free0, 1)
        row["peak_allocated_gib"] = round(torch.cuda.max_memory_allocated() / 2**30, 1)
        rows[label] = row
        _release(torch, model)
        del model
        torch.cuda.reset_peak_memory_stats()
    os.environ["KERAS_B200_TP_FUSED"] = "1"
    out = dict(rows["fused"])
    base = rows.get("library_collectives")
    what = "same model and layout, tensor-parallel collectives through torch.distributed/NCCL (KERAS_B200_TP_FUSED=0)"
    if base is None:
        out["baseline"] = {"what": what, "unavailable": failure}
    else:
        out["baseline"] = {"what": what, "value": base["value"], "ms_per_step": base["ms_per_step"], "e2e": base["e2e"], "clocks": base["clocks"]}
        out["vs_library_collectives"] = out["value"] / base["value"] if base["value"] else None
    return out


def run_ours(args, cfg):
    import torch

    rank, world, local = _dist_env()
    torch.cuda.set_device(local)
    sys.path.insert(0, ROOT)
    import keras_b200 as keras

    dist = None
    if world > 1:
        keras.distribution.initialize()
        import torch.distributed as dist

        if cfg["kind"] == "llama":
            distribution, _ = llama_layout(keras, cfg, world)
            keras.distribution.set_distribution(distribution)
        else:
            keras.distribution.set_distribution(keras.distribution.DataParallel())
    keras.config.set_dtype_policy("mixed_bfloat16")
    if cfg.get("predict"):
        from keras_b200.kernels import ops as kops

        if world > 1:
            raise SystemExit("the predict configs run on one GPU")
        print(json.dumps(measure_predict(keras, torch, args, cfg, local, "ours", kops.launch_count)), flush=True)
        return
    out, model = measure_ours(keras, torch, dist, args, cfg, rank, world, local, args.steps, args.warmup)
    if out is None:
        return
    baseline = _published_baseline()
    out["vs_baseline"] = (out["value"] / baseline) if baseline else None

    printed = threading.Event()

    def emit():
        if rank == 0 and not printed.is_set():
            printed.set()
            print(json.dumps(out), flush=True)

    want_secondary = (args.secondary == "on" and world > 1) or (args.secondary == "auto" and args.config == "resnet50" and world in (4, 8))
    if want_secondary:
        _release(torch, model)
        del model
        budget = float(os.environ.get("KERAS_B200_SECONDARY_BUDGET_S", "480"))

        def watchdog():
            # the primary line is never lost to the secondary measurement: past the budget every rank prints/exits on its own
            if not done.wait(budget):
                out["secondary"] = {"unavailable": f"not finished within {budget:.0f} s"}
                emit()
                os._exit(0)

        done = threading.Event()
        threading.Thread(target=watchdog, daemon=True).start()
        try:
            out["secondary"] = run_secondary(keras, torch, dist, args, rank, world, local)
        except Exception as e:
            out["secondary"] = {"unavailable": f"{type(e).__name__}: {str(e)[:300]}"}
        done.set()
        emit()
    else:
        emit()
        _release(torch, model)
    if world > 1:
        torch.cuda.synchronize()
        try:
            dist.barrier()
            dist.destroy_process_group()
        except Exception:
            pass


def run_reference(args, cfg):
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "keras")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed (pip install --target baseline/_ref of the reference did not run)"}))
        return
    os.environ["KERAS_BACKEND"] = "torch"
    os.environ.setdefault("KERAS_HOME", "/tmp/keras_ref_home")
    sys.path.insert(0, ref)
    import torch

    rank, world, local = _dist_env()
    if cfg["kind"] == "llama" and (world > 1 or cfg["layers"] > 8):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the reference's torch backend never applies ModelParallel layouts to variables "
                              "(keras/src/backend/torch/core.py creates plain tensors), so every GPU would hold the whole model: 8B parameters "
                              "with fp32 master weights and Adam state plus activations do not fit 180 GB"}))
        return
    if cfg["kind"] == "llama":
        cfg = dict(cfg, per_gpu_batch=cfg["global_batch"])
    torch.cuda.set_device(local)
    try:
        import keras
    except Exception as e:  # pragma: no cover
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"reference import failed: {type(e).__name__}: {str(e)[:200]}"}))
        return
    dist = None
    if world > 1:
        keras.distribution.initialize()
        import torch.distributed as dist

        keras.distribution.set_distribution(keras.distribution.DataParallel())
    keras.config.set_dtype_policy("mixed_bfloat16")
    if cfg.get("predict"):
        out = measure_predict(keras, torch, args, cfg, local, "reference")
        out["framework"] = f"keras {keras.__version__} (torch backend, stock code path)"
        print(json.dumps(out))
        return
    model = build_model(keras, cfg)
    n_buf = 3
    host_x, host_y = make_batches(torch, cfg, rank, n_buf)
    dev_x = [t.cuda() for t in host_x]
    dev_y = [t.cuda() for t in host_y]
    metric, unit, per_step, cfg_out = describe(cfg, world)
    last = {}

    def dev_step(i):
        last["loss"] = model.train_on_batch(dev_x[i % n_buf], dev_y[i % n_buf])

    for i in range(max(args.warmup, 1)):
        dev_step(i)
    sampler = ClockSampler(local)
    sampler.start()
    ms = _timed(torch, dist, world, args.steps, dev_step)
    clocks = sampler.stop()
    ms_e2e, e2e_api = run_e2e(keras, torch, dist, world, args.steps, args.warmup, model, host_x, host_y, last)
    if rank == 0:
        total = per_step * world * args.steps
        loss = last["loss"]
        out = {
            "metric": metric, "value": total / (ms / 1e3), "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "impl": "reference", "framework": f"keras {keras.__version__} (torch backend, stock code path)",
            "config": cfg_out,
            "clocks": clocks,
            "e2e": {"value": total / (ms_e2e / 1e3), "unit": unit, "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": int(host_x[0].numel() * host_x[0].element_size() + host_y[0].numel() * host_y[0].element_size()),
                    "d2h_bytes_per_step": 4,
                    "api": e2e_api},
            "gpu_launches": 0,
            "final_loss": float(loss if not isinstance(loss, (list, tuple)) else loss[0]),
        }
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _published_baseline():
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            pub = json.load(f).get("published") or {}
        for v in pub.values():
            if isinstance(v, (int, float)):
                return float(v)
    except Exception:
        pass
    return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="resnet50", choices=sorted(CONFIGS))
    ap.add_argument("--model-axis", type=int, default=0, help="llama configs: ranks per model-parallel group (default: the config's, at most N)")
    ap.add_argument("--profile-range", action="store_true", help="run warm-up, then one step inside cudaProfilerStart/Stop, and exit")
    ap.add_argument("--secondary-config", default=SECONDARY_CONFIG, choices=sorted(k for k, v in CONFIGS.items() if v["kind"] == "llama"))
    ap.add_argument("--secondary", default="auto", choices=["auto", "on", "off"],
                    help="at N=4 and N=8, also measure the 8B ModelParallel decoder and report it under \"secondary\" (auto: with the default config)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    cfg = CONFIGS[args.config]
    if args.model_axis > 0 and cfg["kind"] == "llama":
        cfg = dict(cfg, model_axis=args.model_axis)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus != world and world == 1 and args.gpus > 1:
        # convenience: re-launch under torchrun when asked for N>1 from a plain python call
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1",
               "--master-port", os.environ.get("MASTER_PORT", "29533"), os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    if args.impl == "reference":
        try:
            run_reference(args, cfg)
        except Exception as e:  # the reference arm never fails the run: it reports why it has no number
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"reference run raised {type(e).__name__}: {str(e)[:200]}"}))
    else:
        run_ours(args, cfg)


if __name__ == "__main__":
    main()
