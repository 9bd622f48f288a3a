"""Softmax, embedding, average / global-average pooling and resize kernels against plain PyTorch fp32 math (needs a B200)."""

import pytest
import torch
import torch.nn.functional as F

import keras_b200 as keras

pytestmark = pytest.mark.gpu


def _bf16_close(a, b, atol=2e-2, rtol=2e-2):
    torch.testing.assert_close(a.float(), b.float(), atol=atol, rtol=rtol)


@pytest.mark.parametrize("shape", [(37, 10), (16, 12, 64, 64), (5, 1000), (3, 50257), (9, 2049), (4, 4096)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("log", [False, True])
def test_softmax_forward_backward(shape, dtype, log):
    from keras_b200.kernels import dispatch

    torch.manual_seed(0)
    x = (torch.randn(*shape, device="cuda") * 3).to(dtype).requires_grad_(True)
    y = dispatch.softmax(x, log=log)
    assert y is not None and y.dtype == dtype
    ref_in = x.detach().float().requires_grad_(True)
    ref = torch.log_softmax(ref_in, -1) if log else torch.softmax(ref_in, -1)
    g = torch.randn(*shape, device="cuda").to(dtype)
    y.backward(g)
    ref.backward(g.float())
    if dtype == torch.float32:
        torch.testing.assert_close(y, ref, atol=2e-5, rtol=1e-4)
        torch.testing.assert_close(x.grad, ref_in.grad, atol=2e-5, rtol=1e-4)
    else:
        _bf16_close(y, ref)
        _bf16_close(x.grad, ref_in.grad, atol=6e-2, rtol=3e-2)


def test_softmax_mask_axes_and_layer():
    torch.manual_seed(1)
    x = torch.randn(4, 8, 33, 40, device="cuda")
    mask = torch.rand(4, 1, 33, 40, device="cuda") > 0.3
    mask[0, 0, 0] = False  # a fully masked row
    layer = keras.layers.Softmax(axis=-1)
    out = layer(x, mask=mask)
    big = -1e9
    ref = torch.softmax(x + (1.0 - mask.float()) * big, -1) * mask.float()
    torch.testing.assert_close(out, ref, atol=2e-6, rtol=1e-5)
    # axes other than the last, and several axes
    y = keras.ops.softmax(x, axis=1)
    torch.testing.assert_close(y, torch.softmax(x, 1), atol=2e-6, rtol=1e-5)
    y = keras.ops.softmax(x, axis=(2, 3))
    torch.testing.assert_close(y, torch.softmax(x.reshape(4, 8, -1), -1).reshape(x.shape), atol=2e-6, rtol=1e-5)
    y = keras.ops.log_softmax(x.bfloat16(), axis=-1)
    assert y.dtype == torch.bfloat16
    _bf16_close(y, torch.log_softmax(x.bfloat16().float(), -1), atol=5e-2)


@pytest.mark.parametrize("table_dtype,out_dtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16), (torch.bfloat16, torch.bfloat16)])
def test_embedding_gather_and_scatter_add(table_dtype, out_dtype):
    from keras_b200.kernels import dispatch

    torch.manual_seed(2)
    V, D = 1003, 72
    table = torch.randn(V, D, device="cuda").to(table_dtype).requires_grad_(True)
    ids = torch.randint(0, V, (7, 129), device="cuda")
    ids[0, :40] = 5  # many hits on one row
    out = dispatch.embedding(None, table, ids, out_dtype)
    assert out is not None and out.dtype == out_dtype and out.shape == (7, 129, D)
    torch.testing.assert_close(out.float(), table.detach()[ids].to(out_dtype).float())
    g = torch.randn(7, 129, D, device="cuda").to(out_dtype)
    out.backward(g)
    ref = torch.zeros(V, D, device="cuda").index_add_(0, ids.reshape(-1), g.float().reshape(-1, D))
    torch.testing.assert_close(table.grad.float(), ref.to(table_dtype).float(), atol=2e-2 if table_dtype == torch.bfloat16 else 1e-4, rtol=2e-2)


def test_embedding_layer_trains_like_the_library_path(monkeypatch):
    def run(fused):
        monkeypatch.setenv("KERAS_B200_DISABLE_FUSED_KERNELS", "0" if fused else "1")
        keras.utils.set_random_seed(3)
        model = keras.Sequential([keras.layers.Embedding(500, 64), keras.layers.GlobalAveragePooling1D(), keras.layers.Dense(8)])
        model.compile(optimizer=keras.optimizers.SGD(0.5), loss=keras.losses.SparseCategoricalCrossentropy(from_logits=True))
        x = torch.randint(0, 500, (64, 20))
        y = torch.randint(0, 8, (64,))
        hist = model.fit(x, y, batch_size=32, epochs=3, verbose=0, shuffle=False)
        return hist.history["loss"], model.layers[0].embeddings.value.detach().float().cpu()

    from keras_b200.core import config

    loss_a, emb_a = run(True)
    loss_b, emb_b = run(False)
    monkeypatch.setenv("KERAS_B200_DISABLE_FUSED_KERNELS", "0")
    assert config.fused_kernels_enabled()
    torch.testing.assert_close(torch.tensor(loss_a), torch.tensor(loss_b), atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(emb_a, emb_b, atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("n,h,w,c,k,s,padding", [(3, 17, 19, 16, 3, 2, "same"), (2, 14, 14, 64, 2, 2, "valid"), (2, 9, 11, 8, 3, 1, "same"), (1, 7, 7, 32, 7, 7, "valid")])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_average_pooling(n, h, w, c, k, s, padding, dtype):
    torch.manual_seed(4)
    x = torch.randn(n, h, w, c, device="cuda").to(dtype).requires_grad_(True)
    y = keras.ops.average_pool(x, k, s, padding)
    xr = x.detach().float().permute(0, 3, 1, 2).requires_grad_(True)
    if padding == "same":
        oh, ow = -(-h // s), -(-w // s)
        th, tw = max((oh - 1) * s + k - h, 0), max((ow - 1) * s + k - w, 0)
        pads = (tw // 2, tw - tw // 2, th // 2, th - th // 2)
        num = F.avg_pool2d(F.pad(xr, pads), k, s)
        den = F.avg_pool2d(F.pad(torch.ones(1, 1, h, w, device="cuda"), pads), k, s)
        ref = num / den
    else:
        ref = F.avg_pool2d(xr, k, s)
    ref = ref.permute(0, 2, 3, 1)
    g = torch.randn_like(ref)
    y.backward(g.to(dtype))
    ref.backward(g.to(dtype).float())
    tol = dict(atol=1e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    torch.testing.assert_close(y.float(), ref, **tol)
    torch.testing.assert_close(x.grad.float(), xr.grad.permute(0, 2, 3, 1), **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_global_average_pooling_layer(dtype):
    torch.manual_seed(5)
    x = torch.randn(6, 7, 7, 2048, device="cuda").to(dtype).requires_grad_(True)
    layer = keras.layers.GlobalAveragePooling2D()
    y = layer(x)
    ref_in = x.detach().float().requires_grad_(True)
    ref = ref_in.mean((1, 2))
    g = torch.randn(6, 2048, device="cuda").to(dtype)
    y.backward(g)
    ref.backward(g.float())
    tol = dict(atol=1e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(y.float(), ref, **tol)
    torch.testing.assert_close(x.grad.float(), ref_in.grad, **tol)
    assert keras.layers.GlobalAveragePooling2D(keepdims=True)(x).shape == (6, 1, 1, 2048)


@pytest.mark.parametrize("interpolation", ["bilinear", "nearest"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.uint8, torch.bfloat16])
@pytest.mark.parametrize("size", [(224, 224), (50, 37), (97, 131)])
def test_resize_matches_interpolate(interpolation, dtype, size):
    torch.manual_seed(6)
    x = (torch.rand(3, 97, 131, 3, device="cuda") * 255)
    x = x.to(dtype) if dtype != torch.uint8 else x.round().to(torch.uint8)
    y = keras.ops.image.resize(x, size, interpolation=interpolation)
    assert y.dtype == dtype and y.shape == (3, size[0], size[1], 3)
    xc = x.float().permute(0, 3, 1, 2)
    if interpolation == "nearest":
        ref = F.interpolate(xc, size=size, mode="nearest-exact")
    else:
        ref = F.interpolate(xc, size=size, mode="bilinear", align_corners=False)
    ref = ref.permute(0, 2, 3, 1)
    if dtype == torch.uint8:
        assert (y.float() - ref.round().clip(0, 255)).abs().max() <= 1.0  # a tie in the rounding may fall either way
        assert ((y.float() - ref.round().clip(0, 255)).abs() > 0).float().mean() < 1e-3
    elif dtype == torch.bfloat16:
        torch.testing.assert_close(y.float(), ref, atol=1.5, rtol=1e-2)
    else:
        torch.testing.assert_close(y, ref, atol=1e-3, rtol=1e-5)


@pytest.mark.parametrize("rows,k", [(64, 2048), (1000, 72), (33, 8192), (17, 100)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_int8_row_quantisation_gives_the_codes_of_the_op_chain(rows, k, dtype):
    from keras_b200 import quantizers
    from keras_b200.kernels import dispatch

    torch.manual_seed(7)
    x = (torch.randn(rows, k, device="cuda") * torch.rand(rows, 1, device="cuda") * 5).to(dtype)
    x[3] = 0  # a row of zeros: the scale is qmax / epsilon
    quantizer = quantizers.AbsMaxQuantizer(axis=-1)
    q, scale, inv = dispatch.int8_quantize_rows(x, quantizer)
    ref_q, ref_scale = quantizer(x, axis=-1)
    assert q.dtype == torch.int8 and scale.dtype == dtype
    torch.testing.assert_close(scale.float(), ref_scale.float(), rtol=0, atol=0)
    assert torch.equal(q, ref_q)
    torch.testing.assert_close(inv, 1.0 / ref_scale.reshape(-1).float(), rtol=1e-6, atol=0)


def test_int8_layers_on_the_kernels_match_the_library_ops(monkeypatch):
    keras.utils.set_random_seed(8)
    for make, shape in [(lambda: keras.layers.Dense(96), (4, 33, 64)),
                        (lambda: keras.layers.EinsumDense("abc,cde->abde", output_shape=(None, 4, 24), bias_axes="de"), (4, 33, 64)),
                        (lambda: keras.layers.EinsumDense("abcd,cde->abe", output_shape=(None, 64), bias_axes="e"), (4, 33, 4, 16))]:
        layer = make()
        x = torch.randn(*shape, device="cuda")
        layer(x)
        layer.quantize("int8")
        monkeypatch.setenv("KERAS_B200_DISABLE_FUSED_KERNELS", "1")
        library = layer(x)
        monkeypatch.setenv("KERAS_B200_DISABLE_FUSED_KERNELS", "0")
        fused = layer(x)
        torch.testing.assert_close(fused, library, rtol=1e-4, atol=1e-4)
