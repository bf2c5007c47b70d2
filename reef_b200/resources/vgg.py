"""VGG-16 schedule graph (13 conv3x3+bias+ReLU, 5 max-pools 2x2/2, three dense layers, softmax).

Follows the op families of the reference's CNN resources (conv2d_add_nn_relu, max_pool2d,
batch_flatten, dense_add_nn_relu / dense_add, softmax; reference: resource/resnet152/resnet152.cu:2-33,
365-374,775-841).  Activations are channels-last, so the flatten order is (h, w, c) and the first
dense weight is laid out accordingly — it is random anyway."""
from __future__ import annotations

import numpy as np

from .layers import Builder

_CFG = [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"]


def build_vgg16(*, name: str = "vgg16", image: int = 224, classes: int = 1000, seed: int = 4001,
                conv_impl: str = "auto", fc: int = 4096) -> Builder:
    b = Builder(name, seed, conv_impl)
    g = b.g
    data = g.input("data", 3 * image * image)
    from .graph import Tensor
    x = Tensor(data, image, image, 3)
    first = True
    for v in _CFG:
        if v == "M":
            x = b.pool(x, "max", 2, 2, 0)
            continue
        bias = b.rng().normal(0.0, 0.05, v).astype(np.float32)
        if first:
            x = b.stem_conv(data, 3, image, image, v, 3, 1, 1, bias=bias, relu=True)
        else:
            x = b.conv(x, v, 3, 1, 1, bias=bias, relu=True)
        first = False
    flat = b.flatten(x)
    h = b.dense(flat, fc, relu=True)
    h = b.dense(h, fc, relu=True)
    logits = b.dense(h, classes, w_std=float(np.sqrt(1.0 / fc)) * 0.5)
    b.softmax_output(logits)
    b.logits_idx = logits.idx
    return b
