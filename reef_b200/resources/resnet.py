"""Pre-activation ResNet schedule graphs (ResNet-18/34 basic units, ResNet-50/101/152 bottleneck units).

Graph shape follows the reference's shipped ResNet resources (reference:
resource/resnet18/resnet18.json kernels 0-56; resource/resnet/resnet.json for
the bottleneck variant): per-channel bias on the input, 7x7/2 stem conv with
bias+ReLU, 3x3/2 max-pool with the first unit's folded pre-activation bias+ReLU,
pre-activation units whose first unit per stage has a 1x1 projection shortcut
taken from the activated input, stride on the first conv of the unit, a final
scale-shift-ReLU fused into the last conv, global average pool, flatten, dense
and softmax.
"""
from __future__ import annotations

import numpy as np

from .graph import Tensor
from .layers import Builder

# The last conv of every residual branch is damped: with fixed (not batch-computed) BatchNorm
# statistics nothing renormalises the residual sum, and He-normal branches would double the
# variance per unit (x1e15 over ResNet-152's 50 units, a one-hot softmax).  0.2 keeps activations
# and logits O(1..100) so that logits and probabilities are both meaningful parity signals.
RES_BRANCH_GAIN = 0.2

_CFG = {
    18: ("basic", [2, 2, 2, 2], [64, 64, 128, 256, 512]),
    34: ("basic", [3, 4, 6, 3], [64, 64, 128, 256, 512]),
    50: ("bottleneck", [3, 4, 6, 3], [64, 256, 512, 1024, 2048]),
    101: ("bottleneck", [3, 4, 23, 3], [64, 256, 512, 1024, 2048]),
    152: ("bottleneck", [3, 8, 36, 3], [64, 256, 512, 1024, 2048]),
}


def build_resnet(depth: int, *, name: str | None = None, image: int = 224, classes: int = 1000,
                 seed: int = 1000, conv_impl: str = "auto", fuse_preact: bool = False) -> Builder:
    kind, units, widths = _CFG[depth]
    b = Builder(name or f"resnet{depth}", seed, conv_impl)
    g = b.g
    data = g.input("data", 3 * image * image)

    # BN on the input image: scale folds into the stem weights, shift stays as a bias op.
    s0, t0 = b.bn(3)
    s_stem, t_stem = b.bn(widths[0])
    x1 = b.stem_conv(data, 3, image, image, widths[0], 7, 2, 3, input_bias=t0 / s0, in_scale=s0, out_scale=s_stem,
                     bias=t_stem, relu=True)

    # first unit's pre-activation BN rides on the max-pool (positive scale commutes with max and ReLU)
    s_pre, t_pre = b.bn(widths[0])
    act = b.pool(x1, "max", 3, 2, 1, bias=t_pre / s_pre)
    act_scale = s_pre          # scale still owed to the consumers of `act`
    x_raw: Tensor | None = None

    n_stage = len(units)
    for si in range(n_stage):
        co = widths[si + 1]
        for ui in range(units[si]):
            stride = 1 if (si == 0 or ui > 0) else 2
            first = ui == 0
            last_unit = si == n_stage - 1 and ui == units[si] - 1
            if kind == "basic":
                s2, t2 = b.bn(co)
                t = b.conv(act, co, 3, stride, 1, in_scale=act_scale, out_scale=s2, bias=t2, relu=True)
                sc = b.conv(act, co, 1, stride, 0, in_scale=act_scale) if first else x_raw
                final = dict(residual=sc)
                if last_unit:
                    sf, tf = b.bn(co)
                    final.update(gamma_beta=(sf, tf), relu=True)
                last = (t, co, 3, 1, 1)
            else:
                mid = co // 4
                s2, t2 = b.bn(mid)
                t_a = b.conv(act, mid, 1, stride, 0, in_scale=act_scale, out_scale=s2, bias=t2, relu=True)
                s3, t3 = b.bn(mid)
                t_b = b.conv(t_a, mid, 3, 1, 1, out_scale=s3, bias=t3, relu=True)
                sc = b.conv(act, co, 1, stride, 0, in_scale=act_scale) if first else x_raw
                final = dict(residual=sc)
                if last_unit:
                    sf, tf = b.bn(co)
                    final.update(gamma_beta=(sf, tf), relu=True)
                last = (t_b, co, 1, 1, 0)
            # the unit's last convolution adds the shortcut; the next unit's pre-activation relu(x + t/s) rides
            # on its epilogue where the tensor-core variant exists (weights are drawn before that unit's BN, so
            # both schedules hold the same model)
            wgt = b.he_conv(co, last[2], last[2], last[0].c)
            if last_unit:
                x_raw = b.conv(*last, weight=wgt, w_gain=RES_BRANCH_GAIN, **final)
            else:
                s_n, t_n = b.bn(co)
                x_raw, act = b.conv(*last, weight=wgt, w_gain=RES_BRANCH_GAIN, preact_bias=t_n / s_n, **final)
                act_scale = s_n

    pooled = b.global_avg_pool(x_raw)
    flat = b.flatten(pooled)
    logits = b.dense(flat, classes, w_std=float(np.sqrt(1.0 / flat.c)) * 0.5)
    b.softmax_output(logits)
    b.logits_idx = logits.idx
    return b
