"""BERT encoder schedule graph (BERT-base: 12 layers, hidden 768, 12 heads, FFN 3072, vocab 30522).

The reference's BERT resource is a TVM kernel list of ~30 small kernels per layer (batch_matmul, four-pass
softmax, five-launch LayerNorm, transposes, bias/GELU elementwise; reference: resource/bert/bert.json,
resource/bert/bert.cu:3-395).  The per-element math is kept (oracle/reef_oracle.c) and the fusion
boundaries are ours: per layer
    QKV projection (+bias)            reef_matmul_nt_bias        A, W[3H][H], out, bias
    attention (scale, softmax, PV)    reef_attention             qkv, out
    output projection (+bias, +x)     reef_matmul_nt_bias_residual   A, W, out, bias, residual
    LayerNorm                         reef_layernorm             out, x, gamma, beta
    FFN-1 (+bias, GELU)               reef_matmul_nt_bias_gelu   A, W, out, bias
    FFN-2 (+bias, +x)                 reef_matmul_nt_bias_residual
    LayerNorm                         reef_layernorm
after   embedding gather + position   reef_embedding             out, word, ids(int64), pos
        LayerNorm                     reef_layernorm
Input storage ``input0`` (int64 token ids), output ``output`` = final hidden states [S][H].
Weights ~ N(0, 0.02) as in the benchmark config; LayerNorm gamma = 1 + N(0, 0.02), beta = N(0, 0.02).
"""
from __future__ import annotations

import numpy as np

from .graph import Graph, kname, tuned_plan
from .layers import round_tf32


class _B:
    def __init__(self, name, seed, impl):
        self.g = Graph(name)
        self.seed, self._n, self.impl = seed, 0, impl

    def rng(self):
        self._n += 1
        return np.random.default_rng([self.seed, self._n])

    def normal(self, *shape, std=0.02):
        return self.rng().normal(0.0, std, shape).astype(np.float32)

    def matmul(self, x, m, n, k, *, gelu=False, residual=None, out=None, round_out=False):
        from .. import capi
        op = "reef_matmul_nt_bias" + ("_gelu" if gelu else "") + ("_residual" if residual is not None else "")
        w = self.normal(n, k)
        attrs = dict(m=m, n=n, k=k)
        if self.impl != "simt":
            try:
                capi.kernel_plan(kname(op, **attrs, v=1))
                attrs["v"] = 1
                attrs.update(tuned_plan(kname(op, **attrs)))
                w = round_tf32(w)
                if round_out:
                    attrs["rt"] = 1   # the consumer is a tensor-core kernel: store the nearest TF32 value, not fp32 it would truncate
            except capi.ReefError:
                pass
        out = self.g.temp(m * n) if out is None else out
        args = [x, self.g.param(w), out, self.g.param(self.normal(n))]
        if residual is not None:
            args.append(residual)
        self.g.kernel(kname(op, **attrs), args)
        return out

    def layernorm(self, x, rows, h, out=None):
        out = self.g.temp(rows * h) if out is None else out
        gamma = (1.0 + self.normal(h)).astype(np.float32)
        self.g.kernel(kname("reef_layernorm", rows=rows, h=h), [out, x, self.g.param(gamma), self.g.param(self.normal(h))])
        return out


def build_bert(*, name: str = "bert_base", layers: int = 12, hidden: int = 768, heads: int = 12, ffn: int = 3072,
               vocab: int = 30522, seq: int = 128, seed: int = 5000, conv_impl: str = "auto") -> _B:
    assert hidden == heads * 64, "the attention kernel is written for head dimension 64"
    from .. import capi
    b = _B(name, seed, conv_impl)
    g = b.g
    ids = g.input("input0", seq, "int64")
    word = g.param(b.normal(vocab, hidden))
    pos = g.param(b.normal(seq, hidden))
    emb = g.temp(seq * hidden)
    g.kernel(kname("reef_embedding", s=seq, h=hidden, vocab=vocab), [emb, word, ids, pos])
    x = b.layernorm(emb, seq, hidden)
    for li in range(layers):
        att_attrs = dict(s=seq, heads=heads, d=hidden // heads)
        att_tc = False
        if conv_impl != "simt":
            try:   # both attention products on the tensor cores where the registry has the shape (<= 128 tokens)
                capi.kernel_plan(kname("reef_attention", **att_attrs, v=1))
                att_attrs["v"] = 1
                att_tc = True
            except capi.ReefError:
                pass
        qkv = b.matmul(x, seq, 3 * hidden, hidden, round_out=att_tc)
        ctx = g.temp(seq * hidden)
        g.kernel(kname("reef_attention", **att_attrs), [qkv, ctx])
        att = b.matmul(ctx, seq, hidden, hidden, residual=x)
        x1 = b.layernorm(att, seq, hidden)
        h1 = b.matmul(x1, seq, ffn, hidden, gelu=True)
        h2 = b.matmul(h1, seq, hidden, ffn, residual=x1)
        last = li == layers - 1
        out = g.add_storage("output", seq * hidden) if last else None
        x = b.layernorm(h2, seq, hidden, out=out)
    return b
