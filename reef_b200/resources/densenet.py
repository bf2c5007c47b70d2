"""DenseNet schedule graphs (DenseNet-121/169/201; growth 32, bottleneck 4x).

A dense layer is BN-ReLU-conv1x1-BN-ReLU-conv3x3 whose 32 output channels are appended to the block's
feature map.  The concatenation is never materialised as a copy (the reference's TVM build emits
`fused_concatenate_N` kernels, reference: resource/inception/inception.cu:288): every producer writes its
channels at an offset of one shared channels-last buffer (`ocs`/`ooff` in the kernel name) and every
consumer reads a channel prefix of it (`ics`/`ioff`).  The first BN-ReLU of a layer acts on that prefix
(`fused_add_nn_relu` with the folded shift; its positive scale moves into the 1x1 weights), the second is
folded into the 1x1 conv (`conv2d_add_nn_relu`).  Transitions: BN-ReLU, 1x1 conv, 2x2/2 average pool."""
from __future__ import annotations

import numpy as np

from .graph import Tensor
from .layers import Builder

_BLOCKS = {121: [6, 12, 24, 16], 169: [6, 12, 32, 32], 201: [6, 12, 48, 32]}


def build_densenet(depth: int = 201, *, name: str | None = None, image: int = 224, classes: int = 1000,
                   growth: int = 32, seed: int = 4002, conv_impl: str = "auto") -> Builder:
    blocks = _BLOCKS[depth]
    b = Builder(name or f"densenet{depth}", seed, conv_impl)
    g = b.g
    data = g.input("data", 3 * image * image)
    s0, t0 = b.bn(64)
    x = b.stem_conv(data, 3, image, image, 64, 7, 2, 3, out_scale=s0, bias=t0, relu=True)
    x = b.pool(x, "max", 3, 2, 1)
    c = 64
    for bi, n_layers in enumerate(blocks):
        c_total = c + n_layers * growth
        buf = Tensor(g.temp(x.h * x.w * c_total), x.h, x.w, c_total)
        # the block's input becomes the first channels of its concat buffer
        # (a 1x1 identity-free copy: bias+ReLU of the previous stage already wrote a dense tensor, so
        # copy through the strided-output conv is avoided by letting the producer below write here)
        _copy_into(b, x, b.slice_of(buf, 0, c))
        for li in range(n_layers):
            cin = c + li * growth
            s1, t1 = b.bn(cin)
            act = b.bias_relu_slice(b.slice_of(buf, 0, cin), t1 / s1)
            s2, t2 = b.bn(4 * growth)
            mid = b.conv(act, 4 * growth, 1, 1, 0, in_scale=s1, out_scale=s2, bias=t2, relu=True)
            b.conv(mid, growth, 3, 1, 1, out=b.slice_of(buf, cin, growth), w_gain=0.5)
        c = c_total
        x = buf
        if bi != len(blocks) - 1:
            s, t = b.bn(c)
            act = b.bias_relu_slice(x, t / s)
            y = b.conv(act, c // 2, 1, 1, 0, in_scale=s)
            x = b.pool(y, "avg", 2, 2, 0, count_include_pad=True)
            c = c // 2
    s, t = b.bn(c)
    act = b.bias_relu_slice(x, t / s)        # final BN-ReLU (scale dropped: it only rescales the logits' input)
    pooled = b.global_avg_pool(act)
    flat = b.flatten(pooled)
    logits = b.dense(flat, classes, w_std=float(np.sqrt(1.0 / c)) * 0.5)
    b.softmax_output(logits)
    b.logits_idx = logits.idx
    return b


def _copy_into(b: Builder, x: Tensor, dst: Tensor) -> None:
    """Place a dense tensor into a channel slice of a concat buffer with the pooling kernel's strided
    output (a 1x1/1 max-pool is a copy): no extra kernel family needed."""
    b.pool(x, "max", 1, 1, 0, out=dst)
