"""Cases that pin the C oracle against the reference's OWN kernels (resource/<model>/<model>.cu of the reference,
compiled unchanged and run on the CPU: oracle/_ref, oracle/ref_kernels.py).

Every case names one reference kernel (or the short chain of kernels that makes one operator: the five LayerNorm
launches, the four softmax launches, QK^T -> mask -> softmax -> PV), its shapes in the reference's layouts (NCHW
activations, OIHW weights, [head][token][d] attention operands) and the oracle call that stands for it in this
repository's layouts (NHWC, OHWI, fused [token][3H] QKV).  ``ref_output`` needs the compiled reference kernels;
``oracle_output`` does not.  tests/golden/make_ref_kernel_golden.py stores ``ref_output`` of every case as a fixture.
"""
from __future__ import annotations

import numpy as np

from oracle import oracle

SUBSAMPLE_LIMIT = 32768   # fixtures keep at most this many values per case (a fixed stride over the flat output)


def _rng(case_id):
    return np.random.default_rng(abs(hash_str(case_id)) % (2 ** 31))


def hash_str(s):
    h = 0
    for ch in s:
        h = (h * 131 + ord(ch)) & 0x7FFFFFFF
    return h


def subsample(y):
    y = np.asarray(y).reshape(-1)
    stride = max(1, -(-y.size // SUBSAMPLE_LIMIT))
    return y[::stride].copy()


# ---- ResNet-152 (reference resource/resnet152: 64x64 input) --------------------------------------------------------
def _conv(ref, ci, hi, co, k, s, p, tail):
    """tail: '' | '_add' (residual) | '_add_nn_relu' (bias) | '_add_add_nn_relu' (residual, bias) |
    '_add_multiply_add_nn_relu' (residual, gamma, beta); argument order of both sides: in, W, out, rest..."""
    ho = (hi + 2 * p - k) // s + 1

    def inputs(rng):
        d = dict(x=rng.normal(0, 1, (ci, hi, hi)), w=rng.normal(0, (2.0 / (ci * k * k)) ** 0.5, (co, ci, k, k)))
        if tail in ("_add", "_add_add_nn_relu", "_add_multiply_add_nn_relu"):
            d["res"] = rng.normal(0, 1, (co, ho, ho))
        if tail in ("_add_nn_relu", "_add_add_nn_relu"):
            d["bias"] = rng.normal(0, 0.5, co)
        if tail == "_add_multiply_add_nn_relu":
            d["gamma"] = rng.uniform(0.5, 1.5, co)
            d["beta"] = rng.normal(0, 0.5, co)
        return {k_: v.astype(np.float32) for k_, v in d.items()}

    order = [n for n in ("res", "bias", "gamma", "beta")]

    def ref_run(R, d):
        y = np.zeros(co * ho * ho, np.float32)
        bufs = [d["x"].reshape(-1).copy(), d["w"].reshape(-1).copy(), y] + [d[n].reshape(-1).copy() for n in order if n in d]
        R.launch("resnet152", ref, bufs)
        return y.reshape(co, ho, ho)

    def oracle_run(d):
        name = f"fused_nn_conv2d{tail}__ci{ci}_hi{hi}_wi{hi}_co{co}_kh{k}_kw{k}_sh{s}_sw{s}_ph{p}_pw{p}"
        y = np.zeros(ho * ho * co, np.float32)
        bufs = [np.ascontiguousarray(d["x"].transpose(1, 2, 0)).reshape(-1),
                np.ascontiguousarray(d["w"].transpose(0, 2, 3, 1)).reshape(-1), y]
        for n in order:
            if n in d:
                bufs.append(np.ascontiguousarray(d[n].transpose(1, 2, 0)).reshape(-1) if n == "res" else d[n])
        oracle.run_kernel(name, bufs)
        return y.reshape(ho, ho, co).transpose(2, 0, 1)

    return dict(inputs=inputs, ref=ref_run, oracle=oracle_run)


def _simple(model, ref, make_inputs, ref_bufs, oracle_name, oracle_bufs, out_shape, ref_post=None, oracle_post=None):
    def ref_run(R, d):
        bufs, out = ref_bufs(d)
        R.launch(model, ref, bufs)
        return ref_post(out) if ref_post else out.reshape(out_shape)

    def oracle_run(d):
        bufs, out = oracle_bufs(d)
        oracle.run_kernel(oracle_name, bufs)
        return oracle_post(out) if oracle_post else out.reshape(out_shape)

    return dict(inputs=make_inputs, ref=ref_run, oracle=oracle_run)


def _f32(**kw):
    return {k: np.asarray(v, dtype=np.float32) for k, v in kw.items()}


CASES = {
    # reference kernel (resource/resnet152/resnet152.cu) -> the oracle call that restates it
    "conv7x7_s2_stem_bias_relu": _conv("fused_nn_conv2d_add_nn_relu_12_kernel0", 3, 64, 64, 7, 2, 3, "_add_nn_relu"),
    "conv3x3_bias_relu": _conv("fused_nn_conv2d_add_nn_relu_9_kernel0", 64, 16, 64, 3, 1, 1, "_add_nn_relu"),
    "conv1x1_residual": _conv("fused_nn_conv2d_add_1_kernel0", 256, 4, 1024, 1, 1, 0, "_add"),
    "conv1x1_residual_bias_relu": _conv("fused_nn_conv2d_add_add_nn_relu_kernel0", 256, 4, 1024, 1, 1, 0, "_add_add_nn_relu"),
    # (the shipped fused_nn_conv2d_add_nn_relu_8_kernel0, the first stride-2 1x1 of stage 2, is hand-edited and
    # inconsistent with itself — resnet152.cu:3399 against :3410 — so the stride-2 1x1 of stage 3 stands for the family)
    "conv1x1_s2_bias_relu": _conv("fused_nn_conv2d_add_nn_relu_5_kernel0", 512, 8, 256, 1, 2, 0, "_add_nn_relu"),
    "conv1x1_s2_projection": _conv("fused_nn_conv2d_2_kernel0", 512, 8, 1024, 1, 2, 0, ""),
    "conv1x1_residual_scale_shift_relu": _conv("fused_nn_conv2d_add_multiply_add_nn_relu_kernel0", 512, 2, 2048, 1, 1, 0,
                                               "_add_multiply_add_nn_relu"),
    "conv3x3_deep_bias_relu": _conv("fused_nn_conv2d_add_nn_relu_kernel0", 512, 2, 512, 3, 1, 1, "_add_nn_relu"),
    "max_pool3x3_s2_bias_relu": _simple(
        "resnet152", "fused_nn_max_pool2d_add_nn_relu_kernel0",
        lambda rng: _f32(x=-np.abs(rng.normal(0, 1, (64, 32, 32))) - 0.5, bias=rng.normal(1.0, 0.5, 64)),   # all-negative image: the pad value shows
        lambda d: (lambda y: ([d["x"].reshape(-1).copy(), y, d["bias"]], y))(np.zeros(64 * 16 * 16, np.float32)),
        "fused_nn_max_pool2d_add_nn_relu__c64_hi32_wi32_k3_s2_p1_ho16_wo16",
        lambda d: (lambda y: ([np.ascontiguousarray(d["x"].transpose(1, 2, 0)).reshape(-1), y, d["bias"]], y))(np.zeros(16 * 16 * 64, np.float32)),
        (64, 16, 16), oracle_post=lambda y: y.reshape(16, 16, 64).transpose(2, 0, 1)),
    "input_bias_add": _simple(
        "resnet152", "fused_add_14_kernel0",
        lambda rng: _f32(x=rng.normal(0, 1, (3, 64, 64)), bias=rng.normal(0, 1, 3)),
        lambda d: (lambda y: ([y, d["x"].reshape(-1).copy(), d["bias"]], y))(np.zeros(3 * 64 * 64, np.float32)),
        "fused_add__c3_hw4096",
        lambda d: (lambda y: ([y, d["x"].reshape(-1).copy(), d["bias"]], y))(np.zeros(3 * 64 * 64, np.float32)),
        (3, 64, 64)),
    "bias_relu": _simple(
        "resnet152", "fused_add_nn_relu_1_kernel0",
        lambda rng: _f32(x=rng.normal(0, 1, (1024, 4, 4)), bias=rng.normal(0, 1, 1024)),
        lambda d: (lambda y: ([y, d["x"].reshape(-1).copy(), d["bias"]], y))(np.zeros(1024 * 16, np.float32)),
        "fused_add_nn_relu__c1024_n16",
        lambda d: (lambda y: ([y, np.ascontiguousarray(d["x"].transpose(1, 2, 0)).reshape(-1), d["bias"]], y))(np.zeros(16 * 1024, np.float32)),
        (1024, 4, 4), oracle_post=lambda y: y.reshape(4, 4, 1024).transpose(2, 0, 1)),
    "global_avg_pool": _simple(
        "resnet152", "fused_nn_global_avg_pool2d_kernel0",
        lambda rng: _f32(x=rng.normal(0, 1, (2048, 2, 2))),
        lambda d: (lambda y: ([d["x"].reshape(-1).copy(), y], y))(np.zeros(2048, np.float32)),
        "fused_nn_global_avg_pool2d__c2048_hw4",
        lambda d: (lambda y: ([np.ascontiguousarray(d["x"].transpose(1, 2, 0)).reshape(-1), y], y))(np.zeros(2048, np.float32)),
        (2048,)),
    "batch_flatten": _simple(
        "resnet152", "fused_nn_batch_flatten_kernel0",
        lambda rng: _f32(x=rng.normal(0, 1, 2048)),
        lambda d: (lambda y: ([y, d["x"].copy()], y))(np.zeros(2048, np.float32)),
        "fused_nn_batch_flatten__n2048",
        lambda d: (lambda y: ([y, d["x"].copy()], y))(np.zeros(2048, np.float32)),
        (2048,)),
    "dense_bias": _simple(
        "resnet152", "fused_nn_dense_add_kernel0",
        lambda rng: _f32(x=rng.normal(0, 1, 2048), w=rng.normal(0, 0.03, (1000, 2048)), bias=rng.normal(0, 1, 1000)),
        lambda d: (lambda y: ([d["x"].copy(), d["w"].reshape(-1).copy(), y, d["bias"]], y))(np.zeros(1000, np.float32)),
        "fused_nn_dense_add__k2048_n1000",
        lambda d: (lambda y: ([d["x"].copy(), d["w"].reshape(-1).copy(), y, d["bias"]], y))(np.zeros(1000, np.float32)),
        (1000,)),
    "softmax_1000": _simple(
        "resnet152", "fused_nn_softmax_kernel0",
        lambda rng: _f32(x=rng.normal(0, 3, 1000)),
        lambda d: (lambda y: ([np.concatenate([d["x"], np.zeros(1048, np.float32)]), y], y))(np.zeros(2048, np.float32)),
        "fused_nn_softmax__n1000",
        lambda d: (lambda y: ([d["x"].copy(), y], y))(np.zeros(1000, np.float32)),
        (1000,), ref_post=lambda y: y[:1000].copy()),
    # reference resource/inception/inception.cu: 3x3 stride-1 average pool that counts the padding (x 1/9 everywhere)
    "avg_pool3x3_s1_count_include_pad": _simple(
        "inception", "fused_nn_avg_pool2d_7_kernel0",
        lambda rng: _f32(x=rng.normal(1.0, 1, (192, 35, 35))),
        lambda d: (lambda y: ([d["x"].reshape(-1).copy(), y], y))(np.zeros(192 * 35 * 35, np.float32)),
        "fused_nn_avg_pool2d__c192_hi35_wi35_k3_s1_p1_ho35_wo35_cip1",
        lambda d: (lambda y: ([np.ascontiguousarray(d["x"].transpose(1, 2, 0)).reshape(-1), y], y))(np.zeros(35 * 35 * 192, np.float32)),
        (192, 35, 35), oracle_post=lambda y: y.reshape(35, 35, 192).transpose(2, 0, 1)),
}


# ---- BERT (reference resource/bert: 480 tokens, hidden 480, 12 heads x 40) -----------------------------------------
T, H, HEADS, D = 480, 480, 12, 40


def _bert_ln():
    def inputs(rng):
        return _f32(x=rng.normal(0.3, 1.5, (T, H)), gamma=rng.uniform(0.5, 1.5, H), beta=rng.normal(0, 0.5, H))

    def ref_run(R, d):
        x = d["x"].reshape(-1).copy()
        red = np.zeros(T * 32, np.float32)      # scratch of the two-stage reductions
        mu, var = np.zeros(T, np.float32), np.zeros(T, np.float32)
        out = np.zeros(T * H, np.float32)
        R.launch("bert", "fused_mean_1_kernel0", [x, red])
        R.launch("bert", "fused_mean_1_kernel1", [mu, red])
        R.launch("bert", "fused_variance_1_kernel0", [x, mu, red])
        R.launch("bert", "fused_variance_1_kernel1", [var, red])
        R.launch("bert", "fused_subtract_add_sqrt_divide_multiply_add_1_kernel0", [out, x, mu, var, d["gamma"], d["beta"]])
        return out.reshape(T, H)

    def oracle_run(d):
        out = np.zeros(T * H, np.float32)
        oracle.run_kernel(f"reef_layernorm__rows{T}_h{H}", [out, d["x"].reshape(-1).copy(), d["gamma"], d["beta"]])
        return out.reshape(T, H)

    return dict(inputs=inputs, ref=ref_run, oracle=oracle_run)


def _bert_gelu():
    def inputs(rng):
        return _f32(x=rng.normal(0, 2, (H, T)), bias=rng.normal(0, 1, H))

    def ref_run(R, d):
        # the reference's tensor is feature-major here: the bias runs along the FIRST axis (bert.cu:170, index / 480)
        out = np.zeros(T * H, np.float32)
        R.launch("bert", "fused_reshape_add_multiply_erf_multiply_add_multiply_reshape_kernel0", [out, d["x"].reshape(-1).copy(), d["bias"]])
        return out.reshape(H, T)

    def oracle_run(d):
        # the oracle has bias + GELU as the epilogue of its matmul: x * I + bias is exact, so this is the epilogue alone
        out = np.zeros(T * H, np.float32)
        eye = np.eye(H, dtype=np.float32).reshape(-1)
        oracle.run_kernel(f"reef_matmul_nt_bias_gelu__m{T}_n{H}_k{H}", [np.ascontiguousarray(d["x"].T).reshape(-1), eye, out, d["bias"]])
        return out.reshape(T, H).T

    return dict(inputs=inputs, ref=ref_run, oracle=oracle_run)


def _bert_matmul():
    def inputs(rng):
        return _f32(a=rng.normal(0, 1, (T, H)), b=rng.normal(0, 0.05, (H, H)))

    def ref_run(R, d):
        out = np.zeros(T * H, np.float32)
        R.launch("bert", "fused_nn_batch_matmul_3_kernel0", [d["a"].reshape(-1).copy(), d["b"].reshape(-1).copy(), out])
        return out.reshape(T, H)

    def oracle_run(d):
        out = np.zeros(T * H, np.float32)
        oracle.run_kernel(f"reef_matmul_nt__m{T}_n{H}_k{H}", [d["a"].reshape(-1).copy(), d["b"].reshape(-1).copy(), out])
        return out.reshape(T, H)

    return dict(inputs=inputs, ref=ref_run, oracle=oracle_run)


def _ref_softmax(R, scores):
    """The reference's four softmax launches on [rows][480] scores (max, exp, sum, divide)."""
    rows = scores.size // T
    mx, sm = np.zeros(rows, np.float32), np.zeros(rows, np.float32)
    ex, out = np.zeros(scores.size, np.float32), np.zeros(scores.size, np.float32)
    R.launch("bert", "fused_nn_softmax_1_kernel0", [mx, scores])
    R.launch("bert", "fused_nn_softmax_1_kernel1", [ex, scores, mx])
    R.launch("bert", "fused_nn_softmax_1_kernel2", [sm, ex])
    R.launch("bert", "fused_nn_softmax_1_kernel3", [out, ex, sm])
    return out


def _bert_softmax():
    def inputs(rng):
        return _f32(x=rng.normal(0, 3, (HEADS * T, T)))

    def ref_run(R, d):
        return _ref_softmax(R, d["x"].reshape(-1).copy()).reshape(HEADS * T, T)

    def oracle_run(d):
        out = np.zeros(HEADS * T * T, np.float32)
        oracle.run_kernel(f"fused_nn_softmax__rows{HEADS * T}_n{T}", [d["x"].reshape(-1).copy(), out])
        return out.reshape(HEADS * T, T)

    return dict(inputs=inputs, ref=ref_run, oracle=oracle_run)


def _bert_attention(masked):
    """QK^T (batch_matmul_5) -> masked fill (where) -> softmax (4 launches) -> PV (batch_matmul_4) of the reference,
    fed with Q already divided by sqrt(d) as its graph does in an earlier kernel, against the oracle's one attention
    call on the fused [token][Q|K|V] buffer."""
    def inputs(rng):
        d = _f32(q=rng.normal(0, 1, (HEADS, T, D)), k=rng.normal(0, 1, (HEADS, T, D)), v=rng.normal(0, 1, (HEADS, T, D)))
        m = np.ones(T, np.int8)
        if masked:
            m[rng.choice(T, 77, replace=False)] = 0
        d["mask"] = m
        return d

    def ref_run(R, d):
        qs = (d["q"] / np.float32(np.sqrt(np.float32(D)))).astype(np.float32)
        scores = np.zeros(HEADS * T * T, np.float32)
        R.launch("bert", "fused_nn_batch_matmul_5_kernel0", [qs.reshape(-1).copy(), d["k"].reshape(-1).copy(), scores])
        filled = np.zeros_like(scores)
        # the reference's `where` takes the INVERTED mask (non-zero = fill with -inf, bert.cu:384; its graph builds it
        # with an `equal` kernel from the attention mask), the oracle takes the attention mask itself (0 = masked)
        R.launch("bert", "fused_reshape_cast_broadcast_to_like_where_kernel0", [filled, (1 - d["mask"]).astype(np.int8), scores])
        p = _ref_softmax(R, filled)
        vt = np.ascontiguousarray(d["v"].transpose(0, 2, 1)).reshape(-1)      # [head][d][token]
        ctx = np.zeros(HEADS * T * D, np.float32)
        R.launch("bert", "fused_nn_batch_matmul_4_kernel0", [p, vt, ctx])
        return ctx.reshape(HEADS, T, D)

    def oracle_run(d):
        qkv = np.zeros((T, 3, HEADS, D), np.float32)
        qkv[:, 0], qkv[:, 1], qkv[:, 2] = d["q"].transpose(1, 0, 2), d["k"].transpose(1, 0, 2), d["v"].transpose(1, 0, 2)
        out = np.zeros(T * HEADS * D, np.float32)
        name = f"reef_attention__s{T}_heads{HEADS}_d{D}" + ("_mask1" if masked else "")
        bufs = [qkv.reshape(-1)] + ([d["mask"].astype(np.float32)] if masked else []) + [out]
        oracle.run_kernel(name, bufs)
        return out.reshape(T, HEADS, D).transpose(1, 0, 2)

    return dict(inputs=inputs, ref=ref_run, oracle=oracle_run)


def _bert_embedding():
    vocab, npos = 30522, 1024

    def inputs(rng):
        ids = rng.integers(0, vocab, T).astype(np.int64)
        ids[:4] = [-5, vocab + 9, 0, vocab - 1]          # outside the table on both sides: clamped
        return dict(word=rng.normal(0, 0.02, (vocab, H)).astype(np.float32), pos=rng.normal(0, 0.02, (npos, H)).astype(np.float32),
                    ids=ids, pos_ids=np.arange(T, dtype=np.int64))

    def ref_run(R, d):
        out = np.zeros(T * H, np.float32)
        R.launch("bert", "fused_cast_take_broadcast_to_like_cast_take_add_1_kernel0",
                 [out, d["word"].reshape(-1), d["ids"].copy(), d["pos"].reshape(-1), d["pos_ids"].copy()])
        return out.reshape(T, H)

    def oracle_run(d):
        out = np.zeros(T * H, np.float32)
        oracle.run_kernel(f"reef_embedding__s{T}_h{H}_vocab{vocab}", [out, d["word"].reshape(-1), d["ids"].copy(), d["pos"].reshape(-1)])
        return out.reshape(T, H)

    return dict(inputs=inputs, ref=ref_run, oracle=oracle_run)


CASES.update({
    "bert_layernorm_5_launches": _bert_ln(),
    "bert_bias_gelu": _bert_gelu(),
    "bert_matmul_nt": _bert_matmul(),
    "bert_softmax_4_launches": _bert_softmax(),
    "bert_attention": _bert_attention(False),
    "bert_attention_masked": _bert_attention(True),
    "bert_embedding": _bert_embedding(),
})


def case_inputs(case_id):
    return CASES[case_id]["inputs"](_rng(case_id))


def input_checksum(d):
    """Detects a change of the random generator between the machine that wrote a fixture and the one that reads it."""
    return float(sum(np.asarray(v, dtype=np.float64).sum() for _, v in sorted(d.items())))
