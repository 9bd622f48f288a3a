"""Routing of hot ops to the sm_100a kernels.

Each function returns ``None`` when the call does not qualify (CPU tensor, unsupported dtype or
shape, kernels disabled by ``KERAS_B200_DISABLE_FUSED_KERNELS=1``); the caller then uses its
library path.  On a CUDA device the extension must be loadable: a missing build raises instead
of silently falling back.
"""

from keras_b200.core import config


def _ext():
    from keras_b200.kernels import loader

    return loader.get()


def enabled(t):
    return t.is_cuda and config.fused_kernels_enabled()


def matmul(a, b):
    return None


def conv(x, kernel, strides, padding, data_format, dilation):
    return None


def softmax_cross_entropy(logits, labels):
    return None


def layer_norm(x, gamma, beta, eps):
    return None


def rms_norm(x, scale, eps):
    return None


def flash_attention(q, k, v, mask, scale, is_causal):
    return None


def dense(x, kernel, bias, activation_name):
    return None


def int8_matmul(q_inputs, kernel, out_scale):
    return None


def fp8_matmul(layer, inputs, kernel, equation, training):
    return None


def batch_norm(layer, inputs, training):
    return None


def fused_sgd(opt, grads, variables, lr):
    return False


def fused_adam(opt, grads, variables, lr):
    return False
