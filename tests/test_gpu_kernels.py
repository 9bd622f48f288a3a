"""Numerics of the sm_100a kernels against plain PyTorch fp32 references (needs a B200)."""

import numpy as np
import pytest
import torch

import keras_b200 as keras

pytestmark = pytest.mark.gpu


def _ops():
    from keras_b200.kernels import ops

    return ops


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("relu,res", [(False, False), (True, False), (True, True)])
def test_fused_batchnorm_forward_backward(dtype, tol, relu, res):
    torch.manual_seed(0)
    N, H, W, C = 6, 9, 7, 64
    x = (torch.randn(N, H, W, C, device="cuda") * 2 + 0.5).to(dtype).requires_grad_(True)
    r = torch.randn(N, H, W, C, device="cuda").to(dtype).requires_grad_(True) if res else None
    gamma = (torch.rand(C, device="cuda") + 0.5).requires_grad_(True)
    beta = torch.randn(C, device="cuda").requires_grad_(True)
    mm, mv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
    y = _ops().FusedBatchNormAct.apply(x, gamma, beta, r, mm, mv, 0.9, 1e-3, relu)
    dy = torch.randn_like(y)
    y.backward(dy)
    # fp32 reference
    xf = x.detach().float().requires_grad_(True)
    rf = r.detach().float().requires_grad_(True) if res else None
    gf, bf = gamma.detach().clone().requires_grad_(True), beta.detach().clone().requires_grad_(True)
    mean = xf.mean((0, 1, 2))
    var = (xf * xf).mean((0, 1, 2)) - mean * mean
    ref = (xf - mean) * torch.rsqrt(var + 1e-3) * gf + bf
    if res:
        ref = ref + rf
    if relu:
        ref = torch.relu(ref)
    ref.backward(dy.float())
    assert torch.allclose(y.float(), ref, atol=tol * 4, rtol=tol)
    assert torch.allclose(x.grad.float(), xf.grad, atol=tol * 4, rtol=tol * 4)
    assert torch.allclose(gamma.grad, gf.grad, atol=tol * 40, rtol=tol * 4)
    assert torch.allclose(beta.grad, bf.grad, atol=tol * 40, rtol=tol * 4)
    if res:
        assert torch.allclose(r.grad.float(), rf.grad, atol=tol * 4, rtol=tol)
    assert torch.allclose(mm, 0.1 * mean.detach(), atol=1e-2, rtol=1e-2)
    assert torch.allclose(mv, 0.9 + 0.1 * var.detach(), atol=1e-2, rtol=2e-2)


@pytest.mark.parametrize("rows,C", [(40000 + 37, 64), (9000 + 5, 256), (1500 + 3, 2048), (300000 + 1, 8)])
@pytest.mark.parametrize("relu,res", [(True, True), (True, False), (False, False)])
def test_batchnorm_streaming_passes(rows, C, relu, res):
    """Shapes large enough for the bulk-copy ring kernels (two-input passes), with a ragged last tile."""
    from keras_b200.kernels import ops as kops

    torch.manual_seed(3)
    x = (torch.randn(rows, C, device="cuda") * 1.5 + 0.25).bfloat16().requires_grad_(True)
    r = torch.randn(rows, C, device="cuda").bfloat16().requires_grad_(True) if res else None
    gamma = (torch.rand(C, device="cuda") + 0.5).requires_grad_(True)
    beta = torch.randn(C, device="cuda").requires_grad_(True)
    mm, mv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
    y = kops.FusedBatchNormAct.apply(x, gamma, beta, r, mm, mv, 0.9, 1e-3, relu)
    dy = torch.randn_like(y)
    y.backward(dy)
    xf = x.detach().float().requires_grad_(True)
    rf = r.detach().float().requires_grad_(True) if res else None
    gf, bf = gamma.detach().clone().requires_grad_(True), beta.detach().clone().requires_grad_(True)
    mean = xf.mean(0)
    var = (xf * xf).mean(0) - mean * mean
    ref = (xf - mean) * torch.rsqrt(var + 1e-3) * gf + bf
    if res:
        ref = ref + rf
    # where the pre-activation is within rounding of zero the two sides may disagree about the ReLU mask: leave those out
    sure = (ref.detach().abs() > 3e-2) if relu else torch.ones_like(ref, dtype=torch.bool)
    if relu:
        ref = torch.relu(ref)
    ref.backward(dy.float())
    assert kops._lib().kb200_bn_stream_status() == 0
    torch.testing.assert_close(y.float(), ref, atol=6e-2, rtol=2e-2)
    assert float(sure.float().mean()) > 0.95
    torch.testing.assert_close(torch.where(sure, x.grad.float(), xf.grad), xf.grad, atol=6e-2, rtol=6e-2)
    scale = float(rows) ** 0.5
    torch.testing.assert_close(gamma.grad, gf.grad, atol=0.05 * scale, rtol=3e-2)
    torch.testing.assert_close(beta.grad, bf.grad, atol=0.05 * scale, rtol=3e-2)
    if res:
        # the residual branch receives the masked gradient unchanged, bit for bit
        assert torch.equal(r.grad, torch.where(y > 0, dy, torch.zeros_like(dy)) if relu else dy)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("D", [64, 768, 1000, 1001, 2048, 4096, 8192])
def test_fused_norm(dtype, tol, rms, D):
    torch.manual_seed(1)
    x = torch.randn(37, D, device="cuda").to(dtype).requires_grad_(True)
    g = (torch.rand(D, device="cuda") + 0.5).requires_grad_(True)
    b = None if rms else torch.randn(D, device="cuda").requires_grad_(True)
    y = _ops().FusedNorm.apply(x, g, b, 1e-5, rms)
    dy = torch.randn_like(y)
    y.backward(dy)
    xf = x.detach().float().requires_grad_(True)
    gf = g.detach().clone().requires_grad_(True)
    if rms:
        ref = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + 1e-5) * gf
    else:
        bf = b.detach().clone().requires_grad_(True)
        ref = torch.nn.functional.layer_norm(xf, (D,), gf, bf, 1e-5)
    ref.backward(dy.float())
    assert torch.allclose(y.float(), ref, atol=tol * 4, rtol=tol)
    assert torch.allclose(x.grad.float(), xf.grad, atol=tol * 4, rtol=tol * 4)
    assert torch.allclose(g.grad, gf.grad, atol=tol * 40, rtol=tol * 4)
    if not rms:
        assert torch.allclose(b.grad, bf.grad, atol=tol * 40, rtol=tol * 4)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("V", [1000, 50257])
def test_fused_softmax_cross_entropy(dtype, tol, V):
    torch.manual_seed(2)
    logits = (torch.randn(19, V, device="cuda") * 3).to(dtype).requires_grad_(True)
    labels = torch.randint(0, V, (19,), device="cuda")
    loss = _ops().FusedSoftmaxXent.apply(logits, labels)
    w = torch.rand(19, device="cuda")
    (loss.float() * w).sum().backward()
    lf = logits.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lf, labels, reduction="none")
    (ref * w).sum().backward()
    assert torch.allclose(loss.float(), ref, atol=tol * 4, rtol=tol)
    assert torch.allclose(logits.grad.float(), lf.grad, atol=tol, rtol=tol * 4)


def test_fused_optimizers_match_eager_rules():
    torch.manual_seed(3)
    shapes = [(64, 33), (7,), (3, 3, 16, 32), (1000,)]
    for kind in ("adam", "sgd"):
        vs = [keras.Variable(torch.randn(s).numpy()) for s in shapes]
        ref = [v.numpy().astype("float64") for v in vs]
        if kind == "adam":
            opt = keras.optimizers.AdamW(1e-2, weight_decay=0.1)
        else:
            opt = keras.optimizers.SGD(1e-2, momentum=0.9, nesterov=True)
        m = [np.zeros_like(r) for r in ref]
        vv = [np.zeros_like(r) for r in ref]
        grads = [torch.zeros(s, device="cuda") for s in shapes]
        for t in range(1, 4):
            gs = [torch.randn(s, device="cuda") for s in shapes]
            for dst, src in zip(grads, gs):
                dst.copy_(src)
            if t == 2:
                # the training step's own gradient storage is consumed (zeroed) by the update kernel ...
                opt._gradients_are_step_storage = True
                opt.apply(grads, vs)
                opt._gradients_are_step_storage = False
                assert opt._fused_zeroed_grads and all(float(g.abs().sum()) == 0.0 for g in grads)
            else:
                # ... gradients that user code hands to apply() are left as they are
                opt.apply(grads, vs)
                assert opt._fused_plan is not None and not opt._fused_zeroed_grads
                assert all(torch.equal(g, src) for g, src in zip(grads, gs))
            for i, g in enumerate(gs):
                g = g.cpu().numpy().astype("float64")
                if kind == "adam":
                    ref[i] *= 1 - 0.1 * 1e-2
                    m[i] += (g - m[i]) * 0.1
                    vv[i] += (g * g - vv[i]) * 0.001
                    alpha = 1e-2 * np.sqrt(1 - 0.999 ** t) / (1 - 0.9 ** t)
                    ref[i] -= alpha * m[i] / (np.sqrt(vv[i]) + 1e-7)
                else:
                    m[i] = 0.9 * m[i] - 1e-2 * g
                    ref[i] += 0.9 * m[i] - 1e-2 * g
        for v, r in zip(vs, ref):
            np.testing.assert_allclose(v.numpy(), r, rtol=2e-4, atol=2e-5)


@pytest.mark.parametrize("make", [
    lambda k: k.optimizers.RMSprop(1e-2, rho=0.9),
    lambda k: k.optimizers.RMSprop(1e-2, rho=0.9, momentum=0.8),
    lambda k: k.optimizers.RMSprop(1e-2, centered=True, weight_decay=0.05),
    lambda k: k.optimizers.Adagrad(0.05),
    lambda k: k.optimizers.Adadelta(1.0),
    lambda k: k.optimizers.Adamax(2e-2, weight_decay=0.01),
    lambda k: k.optimizers.Nadam(2e-2),
    lambda k: k.optimizers.Lion(1e-3, weight_decay=0.1),
], ids=["rmsprop", "rmsprop_momentum", "rmsprop_centered_decay", "adagrad", "adadelta", "adamax_decay", "nadam", "lion_decay"])
def test_rule_kernel_matches_the_per_variable_update(make, monkeypatch):
    """One launch of the rule kernel over all variables against the same optimizer stepping variable by variable with torch ops."""
    shapes = [(64, 33), (7,), (3, 3, 16, 32), (1000,), (8193,)]
    torch.manual_seed(5)
    init = [torch.randn(s) for s in shapes]
    steps = [[torch.randn(s, device="cuda") for s in shapes] for _ in range(5)]

    def run(fused):
        monkeypatch.setenv("KERAS_B200_DISABLE_FUSED_KERNELS", "0" if fused else "1")
        opt = make(keras)
        vs = [keras.Variable(t.numpy()) for t in init]
        grads = [torch.zeros(s, device="cuda") for s in shapes]
        for gs in steps:
            for dst, src in zip(grads, gs):
                dst.copy_(src)
            opt.apply(grads, vs)
            assert (getattr(opt, "_fused_plan", None) is not None) == fused
        return [v.numpy() for v in vs], [v.numpy() for v in opt.variables]

    fused_params, fused_state = run(True)
    eager_params, eager_state = run(False)
    monkeypatch.setenv("KERAS_B200_DISABLE_FUSED_KERNELS", "0")
    for a, b in zip(fused_params, eager_params):
        np.testing.assert_allclose(a, b, rtol=2e-4, atol=2e-5)
    for a, b in zip(fused_state, eager_state):
        np.testing.assert_allclose(a, b, rtol=2e-4, atol=2e-6)


def _residual_net(keras, width=64):
    """Stem convolution, one projection block and one identity block (bottlenecks with BatchNorm), classifier."""
    L = keras.layers

    def bottleneck(x, filters, stride, project, name):
        shortcut = x
        if project:
            shortcut = L.Conv2D(4 * filters, 1, strides=stride, name=name + "_0_conv")(x)
            shortcut = L.BatchNormalization(epsilon=1.001e-5, name=name + "_0_bn")(shortcut)
        y = L.Conv2D(filters, 1, strides=stride, name=name + "_1_conv")(x)
        y = L.Activation("relu")(L.BatchNormalization(epsilon=1.001e-5, name=name + "_1_bn")(y))
        y = L.Conv2D(filters, 3, padding="same", name=name + "_2_conv")(y)
        y = L.Activation("relu")(L.BatchNormalization(epsilon=1.001e-5, name=name + "_2_bn")(y))
        y = L.BatchNormalization(epsilon=1.001e-5, name=name + "_3_bn")(L.Conv2D(4 * filters, 1, name=name + "_3_conv")(y))
        return L.Activation("relu")(L.Add()([shortcut, y]))

    inp = keras.Input((32, 32, 8))
    x = L.Conv2D(width, 3, padding="same", name="stem")(inp)
    x = L.Activation("relu")(L.BatchNormalization(name="stem_bn")(x))
    x = bottleneck(x, width, 2, True, "a")
    x = bottleneck(x, width, 1, False, "b")
    x = L.GlobalAveragePooling2D()(x)
    return keras.Model(inp, L.Dense(10, name="predictions")(x))


def test_residual_step_fused_matches_unfused(monkeypatch):
    """Same weights, same batch, three SGD steps: the losses agree and so do the gradients of the first and the last layer
    (seen as the first step's weight change), with this package's kernels and graph fusion against the library path."""
    keras.config.set_dtype_policy("mixed_bfloat16")
    rng = np.random.default_rng(0)
    x = rng.normal(size=(64, 32, 32, 8)).astype("float32")
    y = rng.integers(0, 10, size=(64,))

    def run(disable):
        keras.backend.clear_session(free_memory=False)
        keras.config.set_dtype_policy("mixed_bfloat16")
        keras.utils.set_random_seed(7)
        monkeypatch.setenv("KERAS_B200_DISABLE_FUSED_KERNELS", "1" if disable else "0")
        model = _residual_net(keras)
        model.compile(optimizer=keras.optimizers.SGD(0.01, momentum=0.9), loss=keras.losses.SparseCategoricalCrossentropy(from_logits=True),
                      jit_compile=False)
        first, last = model.get_layer("stem").kernel, model.get_layer("predictions").kernel
        before = [first.numpy().copy(), last.numpy().copy()]
        losses = [model.train_on_batch(x, y)]
        deltas = [first.numpy() - before[0], last.numpy() - before[1]]  # -lr * gradient of the first step
        losses += [model.train_on_batch(x, y) for _ in range(2)]
        return losses, deltas

    from keras_b200.kernels import ops

    launches_before = ops.launch_count()
    fused, fused_deltas = run(False)
    assert ops.launch_count() > launches_before
    plain, plain_deltas = run(True)
    np.testing.assert_allclose(fused, plain, rtol=0.03, atol=0.03)
    for name, a, b in zip(("first convolution", "classifier"), fused_deltas, plain_deltas):
        a, b = a.ravel().astype("float64"), b.ravel().astype("float64")
        cosine = float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-30))
        assert cosine > 0.98, (name, cosine)
        assert abs(np.linalg.norm(a) / np.linalg.norm(b) - 1.0) < 0.1, (name, np.linalg.norm(a), np.linalg.norm(b))
    keras.config.set_dtype_policy("float32")


def test_resnet_step_fused_matches_unfused(monkeypatch):
    """The full ResNet-50 at a tiny size: fifty BatchNorm layers over 8 samples amplify bf16 rounding, so only the first loss
    is compared closely; gradients are compared on the shallow network above."""
    keras.config.set_dtype_policy("mixed_bfloat16")
    rng = np.random.default_rng(0)
    x = rng.normal(size=(8, 64, 64, 3)).astype("float32")
    y = rng.integers(0, 10, size=(8,))

    def run(disable):
        keras.backend.clear_session(free_memory=False)
        keras.config.set_dtype_policy("mixed_bfloat16")
        keras.utils.set_random_seed(7)
        monkeypatch.setenv("KERAS_B200_DISABLE_FUSED_KERNELS", "1" if disable else "0")
        model = keras.applications.ResNet50(weights=None, input_shape=(64, 64, 3), classes=10)
        model.compile(optimizer=keras.optimizers.SGD(0.01, momentum=0.9), loss="sparse_categorical_crossentropy")
        return [model.train_on_batch(x, y) for _ in range(3)]

    from keras_b200.kernels import ops

    launches_before = ops.launch_count()
    fused = run(False)
    assert ops.launch_count() > launches_before
    plain = run(True)
    assert all(np.isfinite(fused)) and all(np.isfinite(plain))
    assert abs(fused[0] - plain[0]) < 0.05 * abs(plain[0]) + 0.05
    keras.config.set_dtype_policy("float32")


def test_training_on_gpu_transformer_block():
    keras.config.set_dtype_policy("mixed_bfloat16")
    inp = keras.Input((64,), dtype="int32")
    h = keras.layers.Embedding(1000, 128)(inp)
    h = keras.layers.LayerNormalization()(h)
    h = keras.layers.Dense(256, activation="gelu")(h)
    out = keras.layers.Dense(1000)(h)
    model = keras.Model(inp, out)
    model.compile(optimizer=keras.optimizers.AdamW(1e-3, weight_decay=0.01), loss=keras.losses.SparseCategoricalCrossentropy(from_logits=True))
    rng = np.random.default_rng(0)
    x = rng.integers(0, 1000, size=(16, 64))
    y = rng.integers(0, 1000, size=(16, 64))
    losses = [model.train_on_batch(x, y) for _ in range(8)]
    assert np.isfinite(losses).all() and losses[-1] < losses[0]


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 384, 192), (1000, 264, 520), (4096, 1024, 768), (136, 8, 8), (5000, 1000, 520), (9504, 520, 72)])
def test_tcgen05_gemm_all_operand_majors(M, N, K):
    from keras_b200.kernels import gemm

    torch.manual_seed(0)
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(K, N, device="cuda") * 0.5).bfloat16()
    bias = torch.randn(N, device="cuda")
    ref = a.float() @ b.float()
    out = gemm.gemm(a, b, 0, 1, M, N, K)                       # A K-major, B MN-major
    gemm.check_errors()
    assert torch.allclose(out.float(), ref, atol=0.06 * K ** 0.5, rtol=2e-2)
    out = gemm.gemm(a, b.t().contiguous(), 0, 0, M, N, K, bias=bias, act=1, out_dtype=torch.float32)   # B K-major, fused bias+relu
    gemm.check_errors()
    assert torch.allclose(out, torch.relu(ref + bias), atol=0.06 * K ** 0.5, rtol=2e-2)
    out = gemm.gemm(a.t().contiguous(), b, 1, 1, M, N, K)       # A MN-major, B MN-major
    gemm.check_errors()
    assert torch.allclose(out.float(), ref, atol=0.06 * K ** 0.5, rtol=2e-2)


def test_tcgen05_gemm_autograd_matches_torch():
    from keras_b200.kernels import gemm

    torch.manual_seed(1)
    x = torch.randn(512, 256, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(256, 384, device="cuda") * 0.1).bfloat16().requires_grad_(True)
    b = torch.randn(384, device="cuda").requires_grad_(True)
    y = gemm.GemmFn.apply(x, w, b)
    dy = torch.randn_like(y)
    y.backward(dy)
    gemm.check_errors()
    xf, wf, bf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True), b.detach().clone().requires_grad_(True)
    ref = xf @ wf + bf
    ref.backward(dy.float())
    assert torch.allclose(y.float(), ref, atol=0.3, rtol=2e-2)
    assert torch.allclose(x.grad.float(), xf.grad, atol=0.3, rtol=3e-2)
    assert torch.allclose(w.grad.float(), wf.grad, atol=1.0, rtol=3e-2)
    assert torch.allclose(b.grad, bf.grad, atol=0.5, rtol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", ["zero_pad", "same", "valid", "two_by_two"])
def test_fused_max_pool_matches_torch(dtype, case):
    import torch.nn.functional as F

    from keras_b200.kernels import dispatch

    torch.manual_seed(0)
    x = torch.randn(3, 13, 17, 16, device="cuda").to(dtype).requires_grad_(True)
    xr = x.detach().float().requires_grad_(True)
    if case == "zero_pad":
        y = dispatch.max_pool2d(x, (3, 3), (2, 2), "valid", zero_pad=((1, 1), (1, 1)))
        ref = F.max_pool2d(F.pad(xr.permute(0, 3, 1, 2), (1, 1, 1, 1)), 3, 2).permute(0, 2, 3, 1)
    elif case == "same":
        y = dispatch.max_pool2d(x, (3, 3), (2, 2), "same")
        ref = F.max_pool2d(F.pad(xr.permute(0, 3, 1, 2), (1, 1, 1, 1), value=-float("inf")), 3, 2).permute(0, 2, 3, 1)
    elif case == "two_by_two":
        y = dispatch.max_pool2d(x, (2, 2), (2, 2), "valid")
        ref = F.max_pool2d(xr.permute(0, 3, 1, 2), 2, 2).permute(0, 2, 3, 1)
    else:
        y = dispatch.max_pool2d(x, (2, 3), (2, 1), "valid")
        ref = F.max_pool2d(xr.permute(0, 3, 1, 2), (2, 3), (2, 1)).permute(0, 2, 3, 1)
    assert y is not None and y.shape == ref.shape
    torch.testing.assert_close(y.float(), ref, rtol=0, atol=0)
    g = torch.randn_like(ref)
    y.backward(g.to(dtype))
    ref.backward(g.to(dtype).float())
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=1e-2 if dtype == torch.bfloat16 else 1e-6, atol=1e-2 if dtype == torch.bfloat16 else 1e-6)


@pytest.mark.gpu
def test_custom_layer_with_weight_traces_symbolically_on_gpu():
    class Shift(keras.layers.Layer):
        def build(self, input_shape):
            self.offset = self.add_weight(shape=(input_shape[-1],), initializer="ones", name="offset")

        def call(self, x):
            return x + keras.ops.cast(self.offset, x.dtype)

    keras.config.set_dtype_policy("float32")
    inp = keras.Input((5,))
    model = keras.Model(inp, Shift()(inp))
    out = model(np.zeros((2, 5), "float32"))
    assert out.device.type == "cuda" and float(out.sum()) == 10.0


@pytest.mark.gpu
def test_tcgen05_gemm_padded_width_and_split_k_gradients():
    from keras_b200.kernels import gemm

    torch.manual_seed(2)
    for M, K, N in [(8192, 256, 1001), (8192, 256, 384)]:
        x = torch.randn(M, K, device="cuda").bfloat16().requires_grad_(True)
        w = (torch.randn(K, N, device="cuda") * 0.1).bfloat16().requires_grad_(True)
        b = torch.randn(N, device="cuda").requires_grad_(True)
        assert gemm.split_k_for(K, (N + 7) // 8 * 8, M, x.device) > 1
        y = gemm.GemmFn.apply(x, w, b)
        assert tuple(y.shape) == (M, N)
        dy = torch.randn(M, N, device="cuda").bfloat16()
        y.backward(dy)
        gemm.check_errors()
        xf, wf, bf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True), b.detach().clone().requires_grad_(True)
        ref = xf @ wf + bf
        ref.backward(dy.float())
        assert torch.allclose(y.float(), ref, atol=0.3, rtol=2e-2)
        assert torch.allclose(x.grad.float(), xf.grad, atol=0.3, rtol=3e-2)
        assert tuple(w.grad.shape) == (K, N)
        assert torch.allclose(w.grad.float(), wf.grad, atol=2.0, rtol=3e-2)
        assert torch.allclose(b.grad, bf.grad, atol=1.0, rtol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_softmax_xent_on_padded_logits_view(dtype):
    import torch.nn.functional as F

    from keras_b200.kernels import ops as kops

    torch.manual_seed(3)
    rows, V, ld = 64, 1001, 1008
    buf = (torch.randn(rows, ld, device="cuda") * 3).to(dtype)
    for logits in (buf[:, :V], buf[:, :V].contiguous()):
        logits = logits.detach().requires_grad_(True)
        labels = torch.randint(0, V, (rows,), device="cuda")
        loss = kops.FusedSoftmaxXent.apply(logits.reshape(8, 8, V), labels.reshape(8, 8))
        assert loss.dtype == torch.float32
        g = torch.rand(8, 8, device="cuda")
        (loss * g).sum().backward()
        ref_in = logits.detach().float().requires_grad_(True)
        ref = F.cross_entropy(ref_in, labels, reduction="none")
        (ref * g.reshape(-1)).sum().backward()
        assert torch.allclose(loss.reshape(-1), ref, atol=2e-3, rtol=1e-3)
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        assert torch.allclose(logits.grad.float(), ref_in.grad, atol=tol, rtol=2e-2)


@pytest.mark.gpu
def test_fp8_quantize_and_gemm_match_torch_float8():
    from keras_b200.kernels import fp8

    torch.manual_seed(4)
    M, K, N = 512, 384, 640
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(K, N, device="cuda") * 0.2).bfloat16()
    sx, sw = torch.tensor(0.01, device="cuda"), torch.tensor(0.002, device="cuda")
    qx, qxt, amax = fp8.quantize(x, sx, False, row_major=True, transposed=True)
    ref_q = torch.clip(x.float() / sx, -448, 448).to(torch.float8_e4m3fn)
    assert torch.equal(qx[:, :K].view(torch.float8_e4m3fn).float(), ref_q.float())
    assert torch.equal(qxt[:, :M].view(torch.float8_e4m3fn).float(), ref_q.float().t())
    assert float(amax) == float(x.float().abs().max())
    _, qwt, _ = fp8.quantize(w, sw, False, row_major=False, transposed=True)
    ref_w = torch.clip(w.float() / sw, -448, 448).to(torch.float8_e4m3fn)
    y = fp8.gemm(qx, qwt, (sx * sw).reshape(1), M, N, K)
    ref = (ref_q.float() @ ref_w.float()) * float(sx * sw)
    from keras_b200.kernels import gemm

    gemm.check_errors()
    assert torch.allclose(y.float(), ref, atol=2e-2 * float(ref.abs().max()), rtol=2e-2)
    # ragged tile edges of the vector quantisation kernel, both input types
    for dt in (torch.bfloat16, torch.float32):
        xr = torch.randn(520, 392, device="cuda").to(dt)
        qr, qrt, ar = fp8.quantize(xr, sx, True, row_major=True, transposed=True)
        ref_r = torch.clip(xr.float() / sx, -57344, 57344).to(torch.float8_e5m2).float()
        assert torch.equal(qr[:, :392].view(torch.float8_e5m2).float(), ref_r)
        assert torch.equal(qrt[:, :520].view(torch.float8_e5m2).float(), ref_r.t())
        assert float(ar) == float(xr.float().abs().max())
    # e5m2 x e4m3 (gradient product)
    g = torch.randn(M, N, device="cuda").bfloat16()
    sg = torch.tensor(0.001, device="cuda")
    qg, _, _ = fp8.quantize(g, sg, True, row_major=True, transposed=False)
    _, _, _ = qg, None, None
    qw, _, _ = fp8.quantize(w, sw, False, row_major=True, transposed=False)
    dx = fp8.gemm(qg, qw, (sg * sw).reshape(1), M, K, N, a_e5m2=True)
    ref_g = torch.clip(g.float() / sg, -57344, 57344).to(torch.float8_e5m2)
    ref_dx = (ref_g.float() @ ref_w.float().t()) * float(sg * sw)
    gemm.check_errors()
    assert torch.allclose(dx.float(), ref_dx, atol=2e-2 * float(ref_dx.abs().max()), rtol=2e-2)


@pytest.mark.gpu
def test_float8_policy_dense_trains_on_fp8_gemm():
    keras.config.set_dtype_policy("mixed_bfloat16")
    try:
        keras.utils.set_random_seed(0)
        inp = keras.Input((256,))
        h = keras.layers.Dense(512, activation="relu", name="d1")(inp)
        out = keras.layers.Dense(256, name="d2")(h)
        model = keras.Model(inp, out)
        model.quantize("float8")
        model.compile(optimizer=keras.optimizers.Adam(1e-3), loss="mse")
        rng = np.random.default_rng(0)
        x = rng.standard_normal((512, 256)).astype("float32")
        y = (x @ rng.standard_normal((256, 256)).astype("float32")) * 0.05
        from keras_b200.kernels import ops as kops

        before = kops.launch_count()
        losses = [float(model.train_on_batch(x, y)) for _ in range(30)]
        assert kops.launch_count() > before
        assert np.isfinite(losses).all() and losses[-1] < 0.7 * losses[0], losses[::5]
        d1 = model.get_layer("d1")
        assert float(d1.inputs_amax_history.numpy()[0]) > 0.0 and float(d1.outputs_grad_amax_history.numpy()[0]) > 0.0
    finally:
        keras.config.set_dtype_policy("float32")


@pytest.mark.gpu
def test_int8_tensor_core_gemm_matches_integer_reference():
    from keras_b200.kernels import dispatch, gemm

    torch.manual_seed(5)
    M, K, N = 384, 512, 768
    a = torch.randint(-127, 128, (M, K), device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (K, N), device="cuda", dtype=torch.int8)
    a_scale = torch.rand(M, 1, device="cuda") * 50 + 1
    w_scale = torch.rand(N, device="cuda") * 50 + 1
    out = dispatch.int8_matmul(a, w, a_scale, w_scale, out_dtype=torch.float32)
    gemm.check_errors()
    assert out is not None
    ref = (a.double() @ w.double()) / (a_scale.double() * w_scale.double())
    assert torch.allclose(out.double(), ref, rtol=1e-5, atol=1e-6 * float(ref.abs().max()))


@pytest.mark.gpu
def test_int8_quantized_model_predicts_on_int8_gemm():
    keras.config.set_dtype_policy("float32")
    keras.utils.set_random_seed(1)
    inp = keras.Input((256,))
    out = keras.layers.Dense(128, name="d2")(keras.layers.Dense(512, activation="relu", name="d1")(inp))
    model = keras.Model(inp, out)
    x = np.random.default_rng(0).standard_normal((64, 256)).astype("float32")
    ref = model.predict(x, verbose=0)
    model.quantize("int8")
    from keras_b200.kernels import ops as kops

    before = kops.launch_count()
    got = model.predict(x, verbose=0)
    assert kops.launch_count() > before
    assert np.abs(got - ref).max() < 0.05 * np.abs(ref).max()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_column_sum_kernel(dtype):
    from keras_b200.kernels import ops as kops

    torch.manual_seed(6)
    for rows, cols, pitch in [(4096, 768, 768), (1000, 1000, 1008), (300, 8, 8)]:
        buf = torch.randn(rows, pitch, device="cuda").to(dtype)
        x = buf[:, :cols]
        got = kops.column_sum(x)
        ref = x.double().sum(0)
        assert got.dtype == torch.float32
        assert torch.allclose(got.double(), ref, rtol=1e-4, atol=1e-3)


def _attention_reference(q, k, v, scale, causal):
    qf, kf, vf = q.float().transpose(1, 2), k.float().transpose(1, 2), v.float().transpose(1, 2)
    if kf.shape[1] != qf.shape[1]:
        rep = qf.shape[1] // kf.shape[1]
        kf, vf = kf.repeat_interleave(rep, dim=1), vf.repeat_interleave(rep, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        Tq, Tk = s.shape[-2:]
        s = s.masked_fill(torch.triu(torch.ones(Tq, Tk, dtype=torch.bool, device=s.device), diagonal=1), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    return torch.matmul(torch.softmax(s, dim=-1), vf).transpose(1, 2), lse


@pytest.mark.gpu
@pytest.mark.parametrize("B,Tq,Tk,H,Hkv,D,causal", [(2, 256, 256, 4, 4, 64, True), (1, 200, 333, 4, 2, 128, False), (2, 1024, 1024, 3, 1, 64, True),
                                                     (1, 384, 384, 2, 2, 128, True), (3, 128, 640, 2, 2, 64, False)])
def test_flash_attention_forward_matches_fp32_reference(B, Tq, Tk, H, Hkv, D, causal):
    from keras_b200.kernels import attention

    torch.manual_seed(7)
    q = torch.randn(B, Tq, H, D, device="cuda").bfloat16()
    k = torch.randn(B, Tk, Hkv, D, device="cuda").bfloat16()
    v = torch.randn(B, Tk, Hkv, D, device="cuda").bfloat16()
    scale = D ** -0.5
    out, lse = attention.forward(q, k, v, scale, causal)
    attention.check_errors()
    ref, ref_lse = _attention_reference(q, k, v, scale, causal)
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2), float((out.float() - ref).abs().max())
    assert torch.allclose(lse, ref_lse, atol=2e-2, rtol=1e-3)


@pytest.mark.gpu
def test_flash_attention_training_path_gradients(monkeypatch):
    from keras_b200.kernels import attention

    monkeypatch.setenv("KERAS_B200_FLASH_ATTENTION", "1")
    torch.manual_seed(8)
    q, k, v = (torch.randn(2, 256, 4, 64, device="cuda").bfloat16().requires_grad_(True) for _ in range(3))
    out = attention.flash_attention(q, k, v, None, 0.125, True)
    assert out is not None
    g = torch.randn_like(out)
    out.backward(g)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref, _ = _attention_reference(qf, kf, vf, 0.125, True)
    ref.backward(g.float())
    for a, b in ((q.grad, qf.grad), (k.grad, kf.grad), (v.grad, vf.grad)):
        assert torch.allclose(a.float(), b, atol=5e-2, rtol=5e-2)


@pytest.mark.gpu
def test_fp8_delayed_scaling_kernel_matches_reference_formulas():
    from keras_b200 import quantizers
    from keras_b200.kernels import fp8

    torch.manual_seed(0)
    for length, fill in [(1024, "random"), (16, "random"), (1024, "zeros"), (7, "inf")]:
        hist = torch.rand(length, device="cuda") * 3 if fill == "random" else torch.zeros(length, device="cuda")
        if fill == "inf":
            hist[3] = float("inf")
        scale = torch.tensor(0.37, device="cuda")
        amax = torch.tensor([2.5], device="cuda")
        new_scale, new_hist = fp8.delayed_scaling(hist, scale, amax, 448.0)
        want_scale = quantizers.compute_float8_scale(torch.amax(hist, dim=0), scale, 448.0)
        want_hist = torch.roll(hist, shifts=-1).clone()
        want_hist[0] = 2.5
        torch.testing.assert_close(new_scale, want_scale, rtol=1e-6, atol=0)
        assert torch.equal(new_hist, want_hist)


@pytest.mark.gpu
@pytest.mark.parametrize("n,with_bias", [(512, True), (1001, False), (1001, True)])
def test_float8_dense_with_bias_and_odd_width_matches_emulation(n, with_bias):
    """The fp8 tensor-core path (bias in the epilogue, zero-padded width) against quantise-dequantise around a float matmul."""
    keras.config.set_dtype_policy("mixed_bfloat16")
    try:
        keras.utils.set_random_seed(3)
        layer = keras.layers.Dense(n, use_bias=with_bias, bias_initializer="random_normal")
        layer.build((None, 256))
        layer.quantize("float8")
        x = torch.randn(64, 256, device="cuda").bfloat16().requires_grad_(True)
        y = layer(x, training=True)
        assert tuple(y.shape) == (64, n) and y.dtype == torch.bfloat16
        g = torch.randn_like(y)
        y.backward(g)
        w = layer.kernel.value.float() if hasattr(layer.kernel, "value") else layer.kernel.float()
        q = lambda t, m: torch.clip(t.float(), -m, m).to(torch.float8_e4m3fn if m == 448 else torch.float8_e5m2).float()  # noqa: E731
        ref = q(x.detach(), 448) @ q(w, 448)
        if with_bias:
            ref = ref + layer.bias.value.float()
        torch.testing.assert_close(y.float(), ref, atol=0.15, rtol=3e-2)
        ref_dx = q(g, 57344) @ q(w, 448).t()
        torch.testing.assert_close(x.grad.float(), ref_dx, atol=0.3, rtol=5e-2)
    finally:
        keras.config.set_dtype_policy("float32")
