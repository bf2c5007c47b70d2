"""CPU tests that pin the oracle: the reference's mocked_kernel known-answer, an independent PyTorch fp32
interpretation of the same schedule graphs, and the committed golden fixtures."""
import json
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from conftest import rel_err, seeded_input
from oracle import oracle
from oracle.torch_ref import run_graph

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_mocked_kernel_known_answer(gen):
    # reference: src/reef/test/test.cpp:102-116 — inputs == 3 -> every output == (3+3)*3 = 18
    base = gen("mocked_kernel")
    o = oracle.OracleExecutor(base + ".json")
    three = np.full(8192, 3.0, np.float32)
    for n in ("a", "b", "c"):
        o.set_input(n, three)
    o.execute()
    assert np.all(o.get_output() == 18.0)


def test_mocked_kernel_indexing_matches_reference_kernel(gen):
    # reference: resource/mocked_kernel/mocked_kernel.cu:20-29 — first operand indexed by thread offset only
    base = gen("mocked_kernel")
    o = oracle.OracleExecutor(base + ".json")
    a, b, c = (seeded_input(8192, s) for s in (1, 2, 3))
    o.set_input("a", a); o.set_input("b", b); o.set_input("c", c)
    o.execute()
    temp = np.tile(b[:128], 64) + a          # add(args = b, a): temp[i] = b[i % 128] + a[i]
    want = np.tile(temp[:128], 64) * c       # multiply(temp, c)
    assert np.array_equal(o.get_output(), want)


def test_set_input_out_of_range(gen):
    # reference: executor_base.cpp:110 — len < storage size -> OutOfRange
    base = gen("mocked_kernel")
    o = oracle.OracleExecutor(base + ".json")
    with pytest.raises(IndexError):
        o.set_input("a", np.zeros(10, np.float32))


@pytest.mark.parametrize("ci,hi,wi,co,k,s,p", [(16, 9, 11, 8, 3, 1, 1), (32, 14, 14, 64, 1, 2, 0), (3, 20, 20, 16, 7, 2, 3),
                                                (48, 8, 8, 32, (1, 7), 1, (0, 3)), (16, 7, 7, 24, 3, 2, 1)])
def test_oracle_conv_vs_torch(ci, hi, wi, co, k, s, p):
    kh, kw = (k, k) if isinstance(k, int) else k
    ph, pw = (p, p) if isinstance(p, int) else p
    rng = np.random.default_rng(0)
    x = rng.normal(size=(hi, wi, ci)).astype(np.float32)
    w = rng.normal(size=(co, kh, kw, ci)).astype(np.float32)
    ho, wo = (hi + 2 * ph - kh) // s + 1, (wi + 2 * pw - kw) // s + 1
    res = rng.normal(size=(ho * wo, co)).astype(np.float32)
    bias = rng.normal(size=co).astype(np.float32)
    out = np.zeros(ho * wo * co, np.float32)
    name = (f"fused_nn_conv2d_add_add_nn_relu__ci{ci}_hi{hi}_wi{wi}_co{co}_kh{kh}_kw{kw}_sh{s}_sw{s}_ph{ph}_pw{pw}")
    oracle.run_kernel(name, [x.reshape(-1), w.reshape(-1), out, res.reshape(-1), bias])
    y = F.conv2d(torch.from_numpy(x).permute(2, 0, 1)[None], torch.from_numpy(w).permute(0, 3, 1, 2), None, s, (ph, pw))
    y = torch.relu(y[0].permute(1, 2, 0).reshape(-1, co) + torch.from_numpy(res) + torch.from_numpy(bias)).numpy()
    assert rel_err(out, y.reshape(-1)) < 1e-5


def test_oracle_pool_edge_values():
    # max-pool pads with -3.402823e38 (reference: resnet152.cu:367,370): an all-negative image keeps its values
    x = -np.abs(seeded_input(6 * 6 * 4)) - 1.0
    out = np.zeros(3 * 3 * 4, np.float32)
    oracle.run_kernel("fused_nn_max_pool2d__c4_hi6_wi6_k3_s2_p1_ho3_wo3", [x, out])
    y = F.max_pool2d(torch.from_numpy(x).reshape(6, 6, 4).permute(2, 0, 1)[None], 3, 2, 1)[0].permute(1, 2, 0)
    assert np.array_equal(out, y.reshape(-1).numpy())
    # avg-pool 3x3 s1 p1 counts the padding (reference: inception.cu:578-587)
    x = np.ones(4 * 4 * 4, np.float32)
    out = np.zeros(4 * 4 * 4, np.float32)
    oracle.run_kernel("fused_nn_avg_pool2d__c4_hi4_wi4_k3_s1_p1_ho4_wo4_cip1", [x, out])
    assert abs(out.reshape(4, 4, 4)[0, 0, 0] - 4.0 / 9.0) < 1e-6 and abs(out.reshape(4, 4, 4)[1, 1, 0] - 1.0) < 1e-6


@pytest.mark.parametrize("model", ["resnet18_64", "resnet50_64"])
def test_oracle_graph_vs_torch(gen, model):
    base = gen(model)
    x = seeded_input(3 * 64 * 64)
    o = oracle.OracleExecutor(base + ".json", base + ".param")
    o.set_input("data", x)
    o.execute()
    st, names = run_graph(base + ".json", base + ".param", {"data": x})
    for i, n in enumerate(names):
        if n in ("null", "output"):
            assert rel_err(o.storage[i], st[i]) < 2e-5, f"storage {i}"
    assert abs(float(o.get_output().sum()) - 1.0) < 1e-4


def test_golden_resnet18_64(gen):
    """Committed fixture (tests/golden/make_golden.py): logits and probabilities of resnet18_64 (fp32 schedule) for the
    constant input 10.0 — the input the reference's own DNN test uses (reference: test.cpp:44-46)."""
    base = gen("resnet18_64", variant="_fp32")
    g = np.load(os.path.join(GOLDEN, "resnet18_64_fp32_const10.npz"))
    o = oracle.OracleExecutor(base + ".json", base + ".param")
    o.set_input("data", np.full(3 * 64 * 64, 10.0, np.float32))
    o.execute()
    j = json.load(open(base + ".json"))
    logits = o.storage[j["kernels"][-1]["args"][0]]
    assert rel_err(logits, g["logits"]) < 1e-4
    assert rel_err(o.get_output(), g["probs"]) < 1e-4


def test_oracle_bert_vs_torch(gen):
    """BERT families (embedding, LayerNorm eps 1e-12, matmul+bias(+GELU)(+residual), attention) against an
    independent float64 PyTorch encoder built from the same .param blobs."""
    from reef_b200.resources.graph import read_param_file
    base = gen("bert_tiny")
    j = json.load(open(base + ".json"))
    ids = np.random.default_rng(1).integers(0, 1000, 48).astype(np.int64)
    o = oracle.OracleExecutor(base + ".json", base + ".param")
    o.set_input("input0", ids)
    o.execute()
    P = read_param_file(base + ".param")
    names = [s["name"] for s in j["storage"]]

    def T(i):
        return torch.from_numpy(P[names[i]].copy()).double()

    it = iter(j["kernels"])
    k = next(it)
    x = T(k["args"][1]).reshape(1000, 128)[torch.from_numpy(ids)] + T(k["args"][3]).reshape(48, 128)

    def ln(x, k):
        return F.layer_norm(x, (128,), T(k["args"][2]), T(k["args"][3]), eps=1e-12)

    x = ln(x, next(it))
    for _ in range(2):
        k = next(it)
        qkv = x @ T(k["args"][1]).reshape(384, 128).T + T(k["args"][3])
        next(it)
        q, kk, v = [t.reshape(48, 2, 64).permute(1, 0, 2) for t in qkv.split(128, dim=1)]
        ctx = (torch.softmax(q @ kk.transpose(1, 2) / 8.0, -1) @ v).permute(1, 0, 2).reshape(48, 128)
        k = next(it)
        a = ctx @ T(k["args"][1]).reshape(128, 128).T + T(k["args"][3]) + x
        x1 = ln(a, next(it))
        k = next(it)
        h = x1 @ T(k["args"][1]).reshape(256, 128).T + T(k["args"][3])
        h = h * (0.5 * torch.erf(h * 0.7071067811865476) + 0.5)
        k = next(it)
        x = ln(h @ T(k["args"][1]).reshape(128, 256).T + T(k["args"][3]) + x1, next(it))
    assert rel_err(o.get_output(), x.reshape(-1).numpy()) < 1e-5


@pytest.mark.parametrize("model,n", [("vgg16_32", 32), ("densenet121_64", 64), ("inception_v3_139", 139)])
def test_oracle_more_cnn_graphs_vs_torch(gen, model, n):
    base = gen(model)
    x = seeded_input(3 * n * n)
    o = oracle.OracleExecutor(base + ".json", base + ".param")
    o.set_input("data", x)
    o.execute()
    st, names = run_graph(base + ".json", base + ".param", {"data": x})
    assert rel_err(o.get_output(), st[names.index("output")]) < 2e-5


def test_oracle_bert_graph_vs_torch_executor(gen):
    """The schedule interpreter built on PyTorch operators (oracle/torch_ref.py, the second CPU baseline of the bench)
    agrees with the plain-C oracle on every buffer of a BERT schedule, as it does on the CNN schedules above."""
    base = gen("bert_tiny")
    ids = np.random.default_rng(4).integers(0, 1000, 48).astype(np.int64)
    o = oracle.OracleExecutor(base + ".json", base + ".param")
    o.set_input("input0", ids)
    o.execute()
    st, names = run_graph(base + ".json", base + ".param", {"input0": ids})
    for i, n in enumerate(names):
        if n in ("null", "output"):
            assert rel_err(o.storage[i], st[i]) < 2e-5, f"storage {i}"
