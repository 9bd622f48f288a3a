"""Memory-safety and determinism checks of the kernels without a sanitizer: every buffer the Python wrappers allocate is
placed between guard zones that must come back untouched, on shapes that do not divide the tiles; kernels whose algorithm
is order-independent must return the same bits twice."""

import contextlib

import pytest
import torch

import keras_b200 as keras  # noqa: F401  (loads the kernel library)

pytestmark = pytest.mark.gpu

GUARD_BYTES = 4096
GUARD_BYTE = 0xA5


class _GuardedAllocator:
    """Stands in for the ``torch`` module inside a wrapper module: ``empty`` / ``zeros`` / ``empty_like`` / ``zeros_like`` hand
    out views that sit between two guard zones."""

    def __init__(self):
        self.blocks = []

    def __getattr__(self, name):
        return getattr(torch, name)

    def _guarded(self, shape, dtype, device, fill_zero):
        if isinstance(shape, int):
            shape = (shape,)
        shape = tuple(int(s) for s in shape)
        dtype = dtype or torch.get_default_dtype()
        numel = 1
        for s in shape:
            numel *= s
        payload = numel * torch.empty((), dtype=dtype).element_size()
        padded = (payload + 255) // 256 * 256
        raw = torch.full((GUARD_BYTES + padded + GUARD_BYTES,), GUARD_BYTE, dtype=torch.uint8, device=device)
        view = raw[GUARD_BYTES:GUARD_BYTES + payload].view(dtype).view(shape)
        if fill_zero:
            view.zero_()
        self.blocks.append((raw, payload))
        return view

    def empty(self, *shape, dtype=None, device=None, **kwargs):
        shape = shape[0] if len(shape) == 1 and not isinstance(shape[0], int) else shape
        if device is None or torch.device(device).type != "cuda":
            return torch.empty(shape, dtype=dtype, device=device, **kwargs)
        return self._guarded(shape, dtype, device, False)

    def zeros(self, *shape, dtype=None, device=None, **kwargs):
        shape = shape[0] if len(shape) == 1 and not isinstance(shape[0], int) else shape
        if device is None or torch.device(device).type != "cuda":
            return torch.zeros(shape, dtype=dtype, device=device, **kwargs)
        return self._guarded(shape, dtype, device, True)

    def empty_like(self, t, dtype=None, **kwargs):
        if not t.is_cuda:
            return torch.empty_like(t, dtype=dtype, **kwargs)
        return self._guarded(tuple(t.shape), dtype or t.dtype, t.device, False)

    def zeros_like(self, t, dtype=None, **kwargs):
        if not t.is_cuda:
            return torch.zeros_like(t, dtype=dtype, **kwargs)
        return self._guarded(tuple(t.shape), dtype or t.dtype, t.device, True)

    def check(self):
        torch.cuda.synchronize()
        assert self.blocks, "the guarded allocator was never used: the wrappers allocate somewhere else"
        for raw, payload in self.blocks:
            head = raw[:GUARD_BYTES]
            tail = raw[GUARD_BYTES + (payload + 255) // 256 * 256:]
            slack = raw[GUARD_BYTES + payload:GUARD_BYTES + (payload + 255) // 256 * 256]
            assert bool((head == GUARD_BYTE).all()), "write before a buffer"
            assert bool((tail == GUARD_BYTE).all()), "write past a buffer"
            assert bool((slack == GUARD_BYTE).all()), "write into the alignment slack after a buffer"


@contextlib.contextmanager
def guarded_allocations(monkeypatch):
    from keras_b200.kernels import conv, gemm, ops

    allocator = _GuardedAllocator()
    for module in (conv, gemm, ops):
        monkeypatch.setattr(module, "torch", allocator)
    try:
        yield allocator
    finally:
        monkeypatch.undo()


@pytest.mark.parametrize("n,h,w,cin,cout,k,stride", [(3, 57, 57, 72, 64, 3, 1), (2, 56, 56, 64, 256, 1, 1), (5, 7, 7, 512, 2048, 1, 1), (2, 57, 29, 64, 128, 3, 2),
                                                    (2, 28, 28, 256, 512, 1, 2), (2, 33, 31, 3, 64, 7, 2)])
def test_convolution_stays_inside_its_buffers(monkeypatch, n, h, w, cin, cout, k, stride):
    from keras_b200.kernels import conv as kconv

    torch.manual_seed(0)
    x = torch.randn(n, h, w, cin, device="cuda").bfloat16().requires_grad_(True)
    kernel = (torch.randn(k, k, cin, cout, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    with guarded_allocations(monkeypatch) as allocator:
        y = kconv.conv(x, kernel, (stride, stride), "same", "channels_last", (1, 1))
        if y is None:
            pytest.skip("this geometry is served by the library convolution")
        y.backward(torch.randn_like(y))
        allocator.check()
    ref = torch.nn.functional.conv2d(x.detach().float().permute(0, 3, 1, 2), kernel.detach().float().permute(3, 2, 0, 1), stride=stride,
                                     padding=0 if k == 1 else None) if k == 1 else None
    if ref is not None:
        torch.testing.assert_close(y.float(), ref.permute(0, 2, 3, 1), atol=0.1, rtol=3e-2)


@pytest.mark.parametrize("m,n,k", [(1000, 264, 520), (136, 8, 8), (5000, 1000, 520), (4096, 50257, 64)])
def test_gemm_stays_inside_its_buffers(monkeypatch, m, n, k):
    from keras_b200.kernels import gemm as kgemm

    torch.manual_seed(0)
    x = torch.randn(m, k, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(k, n, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    b = torch.randn(n, device="cuda").bfloat16().requires_grad_(True)
    with guarded_allocations(monkeypatch) as allocator:
        out = kgemm.GemmFn.apply(x, w, b, None, None)
        out.backward(torch.randn_like(out))
        allocator.check()
    torch.testing.assert_close(out.float(), x.detach().float() @ w.detach().float() + b.detach().float(), atol=0.2, rtol=3e-2)


@pytest.mark.parametrize("rows,c", [(40037, 64), (1503, 2048), (333, 24), (9005, 256)])
@pytest.mark.parametrize("residual", [False, True])
def test_batchnorm_layernorm_xent_pool_stay_inside_their_buffers(monkeypatch, rows, c, residual):
    from keras_b200.kernels import dispatch
    from keras_b200.kernels import ops as kops

    torch.manual_seed(1)
    x = torch.randn(rows, c, device="cuda").bfloat16().requires_grad_(True)
    r = torch.randn(rows, c, device="cuda").bfloat16().requires_grad_(True) if residual else None
    gamma, beta = torch.ones(c, device="cuda", requires_grad=True), torch.zeros(c, device="cuda", requires_grad=True)
    mm, mv = torch.zeros(c, device="cuda"), torch.ones(c, device="cuda")
    labels = torch.randint(0, c, (rows,), device="cuda")
    with guarded_allocations(monkeypatch) as allocator:
        y = kops.FusedBatchNormAct.apply(x, gamma, beta, r, mm, mv, 0.9, 1e-3, True)
        z = kops.FusedNorm.apply(y, gamma, beta, 1e-5, False)
        loss = kops.FusedSoftmaxXent.apply(z, labels)
        loss.sum().backward()
        if c % 8 == 0 and rows % 7 == 0:
            pass
        allocator.check()
    assert kops._lib().kb200_bn_stream_status() == 0
    assert torch.isfinite(loss).all() and torch.isfinite(x.grad.float()).all()
    img = torch.randn(3, 37, 41, 16, device="cuda").bfloat16().requires_grad_(True)
    with guarded_allocations(monkeypatch) as allocator:
        pooled = dispatch.max_pool2d(img, (3, 3), (2, 2), "valid", zero_pad=((1, 1), (1, 1)))
        pooled.backward(torch.randn_like(pooled))
        allocator.check()


def test_order_independent_kernels_return_the_same_bits_twice():
    from keras_b200.kernels import conv as kconv
    from keras_b200.kernels import dispatch
    from keras_b200.kernels import gemm as kgemm
    from keras_b200.kernels import ops as kops

    torch.manual_seed(2)
    x = torch.randn(4, 29, 29, 64, device="cuda").bfloat16()
    kernel = (torch.randn(3, 3, 64, 128, device="cuda") * 0.05).bfloat16()
    a = torch.randn(1000, 520, device="cuda").bfloat16()
    b = (torch.randn(520, 264, device="cuda") * 0.05).bfloat16()
    rows = torch.randn(777, 768, device="cuda").bfloat16()
    gamma, beta = torch.rand(768, device="cuda") + 0.5, torch.randn(768, device="cuda")
    img = torch.randn(3, 37, 41, 16, device="cuda").bfloat16()

    def once():
        return (kconv.conv(x, kernel, (1, 1), "same", "channels_last", (1, 1)), kgemm.gemm(a, b, 0, 1, 1000, 264, 520),
                kops.FusedNorm.apply(rows, gamma, beta, 1e-5, False), dispatch.max_pool2d(img, (3, 3), (2, 2), "same"))

    first, second = once(), once()
    for u, v in zip(first, second):
        assert torch.equal(u, v)
