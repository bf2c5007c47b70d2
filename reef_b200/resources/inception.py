"""Inception-v3 schedule graph (299x299 input; blocks A x3, B, C x4, D, E x2).

Every convolution is conv+BN+ReLU folded to `fused_nn_conv2d_add_nn_relu`; the padded 3x3/1 average pool
counts the padding, as the reference's kernel does (reference: resource/inception/inception.cu:578-587).
Branch outputs are written straight into their channel range of the block's output buffer (kernel-name
attributes `ocs`/`ooff`) instead of through the reference's `fused_concatenate_N` copy kernels
(reference: resource/inception/inception.cu:288,825,2918)."""
from __future__ import annotations

import numpy as np

from .graph import Tensor
from .layers import Builder


def build_inception_v3(*, name: str = "inception_v3", image: int = 299, classes: int = 1000, seed: int = 4000,
                       conv_impl: str = "auto") -> Builder:
    b = Builder(name, seed, conv_impl)
    g = b.g

    def cbr(x, co, k, stride=1, pad=0, out=None, nchw=False):
        s, t = b.bn(co)
        return b.conv(x, co, k, stride, pad, out_scale=s, bias=t, relu=True, out=out, nchw_in=nchw)

    def concat_buf(h, w, c):
        return Tensor(g.temp(h * w * c), h, w, c)

    data = g.input("data", 3 * image * image)
    s_in, t_in = b.bn(32)
    x = b.stem_conv(data, 3, image, image, 32, 3, 2, 0, out_scale=s_in, bias=t_in, relu=True)
    x = cbr(x, 32, 3)
    x = cbr(x, 64, 3, 1, 1)
    x = b.pool(x, "max", 3, 2, 0)
    x = cbr(x, 80, 1)
    x = cbr(x, 192, 3)
    x = b.pool(x, "max", 3, 2, 0)

    def block_a(x, pf):
        out = concat_buf(x.h, x.w, 64 + 64 + 96 + pf)
        cbr(x, 64, 1, out=b.slice_of(out, 0, 64))
        cbr(cbr(x, 48, 1), 64, 5, 1, 2, out=b.slice_of(out, 64, 64))
        cbr(cbr(cbr(x, 64, 1), 96, 3, 1, 1), 96, 3, 1, 1, out=b.slice_of(out, 128, 96))
        cbr(b.pool(x, "avg", 3, 1, 1), pf, 1, out=b.slice_of(out, 224, pf))
        return out

    def block_b(x):
        ho = (x.h - 3) // 2 + 1
        out = concat_buf(ho, ho, 384 + 96 + x.c)
        cbr(x, 384, 3, 2, 0, out=b.slice_of(out, 0, 384))
        cbr(cbr(cbr(x, 64, 1), 96, 3, 1, 1), 96, 3, 2, 0, out=b.slice_of(out, 384, 96))
        b.pool(x, "max", 3, 2, 0, out=b.slice_of(out, 480, x.c))
        return out

    def block_c(x, c7):
        out = concat_buf(x.h, x.w, 768)
        cbr(x, 192, 1, out=b.slice_of(out, 0, 192))
        t = cbr(cbr(x, c7, 1), c7, (1, 7), 1, (0, 3))
        cbr(t, 192, (7, 1), 1, (3, 0), out=b.slice_of(out, 192, 192))
        t = cbr(cbr(x, c7, 1), c7, (7, 1), 1, (3, 0))
        t = cbr(cbr(t, c7, (1, 7), 1, (0, 3)), c7, (7, 1), 1, (3, 0))
        cbr(t, 192, (1, 7), 1, (0, 3), out=b.slice_of(out, 384, 192))
        cbr(b.pool(x, "avg", 3, 1, 1), 192, 1, out=b.slice_of(out, 576, 192))
        return out

    def block_d(x):
        ho = (x.h - 3) // 2 + 1
        out = concat_buf(ho, ho, 320 + 192 + x.c)
        cbr(cbr(x, 192, 1), 320, 3, 2, 0, out=b.slice_of(out, 0, 320))
        t = cbr(cbr(cbr(x, 192, 1), 192, (1, 7), 1, (0, 3)), 192, (7, 1), 1, (3, 0))
        cbr(t, 192, 3, 2, 0, out=b.slice_of(out, 320, 192))
        b.pool(x, "max", 3, 2, 0, out=b.slice_of(out, 512, x.c))
        return out

    def block_e(x):
        out = concat_buf(x.h, x.w, 2048)
        cbr(x, 320, 1, out=b.slice_of(out, 0, 320))
        t = cbr(x, 384, 1)
        cbr(t, 384, (1, 3), 1, (0, 1), out=b.slice_of(out, 320, 384))
        cbr(t, 384, (3, 1), 1, (1, 0), out=b.slice_of(out, 704, 384))
        t = cbr(cbr(x, 448, 1), 384, 3, 1, 1)
        cbr(t, 384, (1, 3), 1, (0, 1), out=b.slice_of(out, 1088, 384))
        cbr(t, 384, (3, 1), 1, (1, 0), out=b.slice_of(out, 1472, 384))
        cbr(b.pool(x, "avg", 3, 1, 1), 192, 1, out=b.slice_of(out, 1856, 192))
        return out

    for pf in (32, 64, 64):
        x = block_a(x, pf)
    x = block_b(x)
    for c7 in (128, 160, 160, 192):
        x = block_c(x, c7)
    x = block_d(x)
    x = block_e(x)
    x = block_e(x)
    pooled = b.global_avg_pool(x)
    flat = b.flatten(pooled)
    logits = b.dense(flat, classes, w_std=float(np.sqrt(1.0 / 2048)) * 0.5)
    b.softmax_output(logits)
    b.logits_idx = logits.idx
    return b
