"""GPU parity tests of the executor layers, through the C-ABI (libreef_host -> libreef_cuda).
Pyramid as in the reference's test.cpp: raw executor -> dispatcher (rt_executor) -> best-effort flavour
(hybrid_executor), same fixtures at every level; plus per-layer parity against the CPU oracle."""
import json

import numpy as np
import pytest

from conftest import rel_err, seeded_input
from gpu_util import FP32_TOL, TF32_TOL, all_storage, compare_layers, load_executor, single_kernel_model, tol_for
from oracle import oracle
from reef_b200 import capi

pytestmark = pytest.mark.gpu


def _mocked(e):
    three = np.full(8192, 3.0, np.float32)
    for n in ("a", "b", "c"):
        e.set_input(n, three)


@pytest.mark.parametrize("flavour", ["execute", "execute_dispatch", "execute_preemptable", "execute_graph"])
def test_mocked_kernel_all_flavours(gen, flavour):
    # reference: test.cpp:102-116 (executor_base), :246-261 (rt_executor), :296-311 (hybrid_executor)
    e = load_executor(gen("mocked_kernel"))
    _mocked(e)
    getattr(e, flavour)()
    out = e.get_output()
    assert out.shape == (8192,) and np.all(out == 18.0)


def test_set_input_errors(gen):
    e = load_executor(gen("mocked_kernel"))
    with pytest.raises(capi.ReefError) as ex:
        e.set_input("a", np.zeros(16, np.float32))          # shorter than the storage entry
    assert ex.value.status == capi.OUT_OF_RANGE
    with pytest.raises(capi.ReefError) as ex:
        e.set_input("nope", np.zeros(8192, np.float32))
    assert ex.value.status == capi.NOT_FOUND
    with pytest.raises(capi.ReefError) as ex:
        e.execute_kernel(5)
    assert ex.value.status == capi.OUT_OF_RANGE


def test_unknown_kernel_name_is_not_found(tmp_path):
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps({"storage": [{"name": "a", "size": 4, "stype": "float32"}],
                               "kernels": [{"name": "no_such_kernel", "launch_params": [1, 1, 1, 1, 1, 1], "args": [0]}],
                               "args": [0], "shared_memory": {}}))
    e = capi.HybridExecutor(0)
    with pytest.raises(capi.ReefError) as ex:
        e.load_model_from_file(str(bad))
    assert ex.value.status == capi.NOT_FOUND


CONV_CASES = [
    # (family, ci, hi, wi, co, kh, kw, s, ph, pw)   ragged pixel/out-channel tiles, strides, asymmetric taps
    ("fused_nn_conv2d", 16, 9, 11, 8, 3, 3, 1, 1, 1),
    ("fused_nn_conv2d_add", 64, 14, 14, 100, 1, 1, 1, 0, 0),
    ("fused_nn_conv2d_add_nn_relu", 32, 15, 15, 72, 3, 3, 2, 1, 1),
    ("fused_nn_conv2d_add_add_nn_relu", 48, 7, 7, 64, 1, 1, 2, 0, 0),
    ("fused_nn_conv2d_add_multiply_add_nn_relu", 128, 7, 7, 256, 3, 3, 1, 1, 1),
    ("fused_nn_conv2d_nn_relu", 80, 8, 8, 32, 1, 7, 1, 0, 3),
    ("fused_nn_conv2d_add_nn_relu", 20, 10, 10, 12, 5, 5, 1, 2, 2),    # ci not a multiple of 16: generic gather
]


# tensor-core variant (v1): flat 1x1, spatial 3x3, stride-2 sub-lattices, cluster split-K, ragged tiles,
# fewer than 128 output channels, a K range that does not divide evenly over the cluster
TC_CASES = [
    ("fused_nn_conv2d", 64, 8, 8, 128, 1, 1, 1, 0, 0),
    ("fused_nn_conv2d_add_nn_relu", 32, 8, 8, 64, 1, 1, 1, 0, 0),
    ("fused_nn_conv2d_add", 256, 14, 14, 1024, 1, 1, 1, 0, 0),
    ("fused_nn_conv2d_add_nn_relu", 1024, 14, 14, 256, 1, 1, 1, 0, 0),
    ("fused_nn_conv2d_add_nn_relu", 256, 14, 14, 256, 3, 3, 1, 1, 1),
    ("fused_nn_conv2d_add_nn_relu", 64, 56, 56, 64, 3, 3, 1, 1, 1),
    ("fused_nn_conv2d_add_add_nn_relu", 64, 56, 56, 256, 1, 1, 1, 0, 0),
    ("fused_nn_conv2d_add_nn_relu", 256, 56, 56, 128, 1, 1, 2, 0, 0),
    ("fused_nn_conv2d_add_nn_relu", 128, 28, 28, 256, 3, 3, 2, 1, 1),
    ("fused_nn_conv2d_add_multiply_add_nn_relu", 512, 7, 7, 2048, 1, 1, 1, 0, 0),
    ("fused_nn_conv2d_add_nn_relu", 512, 7, 7, 512, 3, 3, 1, 1, 1),
    ("fused_nn_conv2d_nn_relu", 96, 17, 17, 160, 1, 7, 1, 0, 3),
    ("fused_nn_conv2d_add_nn_relu", 160, 9, 13, 72, 5, 5, 1, 2, 2),
    ("fused_nn_conv2d_add_nn_relu", 64, 15, 15, 96, 3, 3, 2, 0, 0),
    ("fused_nn_conv2d_add_nn_relu", 32, 69, 69, 32, 3, 3, 1, 0, 0),      # one channel block per tap, prime output width
    ("fused_nn_conv2d_add_nn_relu", 48, 35, 35, 64, 5, 5, 1, 2, 2),      # Cin not a multiple of 32: ragged last channel block
    ("fused_nn_conv2d_add_nn_relu", 80, 19, 19, 192, 3, 3, 1, 0, 0),
    ("fused_nn_conv2d_add", 20, 12, 12, 40, 1, 1, 1, 0, 0),              # a single ragged channel block
]


@pytest.mark.parametrize("case", TC_CASES, ids=[c[0][9:] + f"_{c[1]}x{c[4]}k{c[5]}{c[6]}s{c[7]}h{c[2]}" for c in TC_CASES])
def test_conv_tensor_core_parity(tmp_path, case):
    from gpu_util import TF32_TOL
    _conv_case(tmp_path, case, "_v1", TF32_TOL)


@pytest.mark.parametrize("shape", [(256, 14, 14, 1024, 1), (64, 9, 11, 96, 3), (512, 7, 7, 2048, 1), (128, 28, 28, 128, 3)])
def test_conv_preact_dual_output(tmp_path, shape):
    """reef_conv2d_add_preact: conv + residual -> out, relu(out + bias2) -> out2 in one launch, against the
    oracle's two reference kernels (fused_nn_conv2d_add, then fused_add_nn_relu), every flavour bit-identical."""
    from gpu_util import TF32_TOL, all_storage
    ci, hi, wi, co, k = shape
    pad = k // 2
    name = f"reef_conv2d_add_preact__ci{ci}_hi{hi}_wi{wi}_co{co}_kh{k}_kw{k}_sh1_sw1_ph{pad}_pw{pad}_v1"
    specs = [("in", ci * hi * wi), ("param", co * k * k * ci), ("out", hi * wi * co), ("in", hi * wi * co),
             ("param", co), ("out", hi * wi * co)]
    base, inputs = single_kernel_model(tmp_path, "one", name, specs)
    j = json.load(open(base + ".json"))
    e = load_executor(base)
    o = oracle.OracleExecutor(base + ".json", base + ".param")
    for kk, v in inputs.items():
        e.set_input(kk, v)
        o.set_input(kk, v)
    e.execute()
    o.execute()
    got = all_storage(e, j)
    for idx in (2, 5):
        err = rel_err(got[idx], o.storage[idx])
        print(name, "storage", idx, "rel err", err)
        assert err < TF32_TOL
    assert capi.device_error() == 0
    for f in ("execute_preemptable", "execute_dispatch", "execute_graph"):
        getattr(e, f)()
        again = all_storage(e, j)
        assert np.array_equal(again[2], got[2]) and np.array_equal(again[5], got[5]), f


def test_tensor_core_stem_variant(tmp_path):
    """conv_impl="tc_stem": reef_nchw_to_nhwc4 (input + bias, planar -> 4-channel channels-last) feeds a 4-channel
    tensor-core stem convolution (ragged channel blocks are zero-filled by TMA); every buffer against the oracle."""
    from reef_b200 import resources
    d = resources.generate("resnet18_64", str(tmp_path), conv_impl="tc_stem")
    base = d + "/resnet18_64"
    j = json.load(open(base + ".json"))
    names = [k["name"] for k in j["kernels"]]
    assert names[0].startswith("reef_nchw_to_nhwc4__c3") and "_ci4_" in names[1] and names[1].endswith("_v1")
    x = seeded_input(3 * 64 * 64, seed=5)
    e = load_executor(base)
    o = oracle.OracleExecutor(base + ".json", base + ".param")
    e.set_input("data", x)
    o.set_input("data", x)
    e.execute()
    o.execute()
    worst = compare_layers(e, o, j, lambda n: TF32_TOL)
    print("tc_stem worst layer", worst)
    assert capi.device_error() == 0
    raw = e.get_output().copy()
    for f in ("execute_preemptable", "execute_dispatch", "execute_graph"):
        getattr(e, f)()
        assert np.array_equal(e.get_output(), raw), f


IM2COL_CASES = [  # c, hi, wi, kh, kw, sh, sw, ph, pw, kp
    (3, 64, 64, 7, 7, 2, 2, 3, 3, 160), (3, 33, 47, 3, 3, 1, 1, 1, 1, 32), (3, 41, 41, 3, 3, 2, 2, 0, 0, 32),
    (1, 20, 24, 5, 3, 1, 2, 2, 0, 32), (4, 17, 17, 3, 3, 3, 3, 1, 1, 64), (3, 8, 8, 7, 7, 1, 1, 3, 3, 148)]


@pytest.mark.parametrize("case", IM2COL_CASES, ids=["c%d_%dx%d_k%dx%d_s%d%d_p%d%d_kp%d" % c for c in IM2COL_CASES])
def test_im2col_kernel_matches_oracle(tmp_path, case):
    """reef_im2col_nchw (planar input + bias -> im2col matrix, rounded to TF32): against the oracle's gather, with
    ragged borders, strides, padding wider than a tap's reach and columns beyond K; all launch flavours bit-identical."""
    c, hi, wi, kh, kw, sh, sw, ph, pw, kp = case
    ho, wo = (hi + 2 * ph - kh) // sh + 1, (wi + 2 * pw - kw) // sw + 1
    name = f"reef_im2col_nchw__c{c}_hi{hi}_wi{wi}_kh{kh}_kw{kw}_sh{sh}_sw{sw}_ph{ph}_pw{pw}_kp{kp}"
    base, inputs = single_kernel_model(tmp_path, "one", name, [("out", ho * wo * kp), ("in", c * hi * wi), ("param", c)])
    e = load_executor(base)
    o = oracle.OracleExecutor(base + ".json", base + ".param")
    for k, v in inputs.items():
        e.set_input(k, v)
        o.set_input(k, v)
    e.execute()
    o.execute()
    got, want = e.get_output(), o.get_output()
    assert capi.device_error() == 0
    # TF32 rounding of the stored values: 2^-11 relative; zeros (padding, columns beyond K) are exact
    assert np.array_equal(got == 0.0, want == 0.0)
    assert np.all(np.abs(got - want) <= np.abs(want) * 2.0 ** -11 + 1e-30)
    raw = got.copy()
    for f in ("execute_preemptable", "execute_dispatch", "execute_graph"):
        getattr(e, f)()
        assert np.array_equal(e.get_output(), raw), f


def test_im2col_stem_against_the_planar_stem(tmp_path):
    """The default schedule runs the first convolution as reef_im2col_nchw + a 1x1 tensor-core convolution over the
    flattened taps; the `_simtstem` variant keeps the planar CUDA-core convolution.  Same seed, same weights: the two
    networks agree within the TF32 tolerance on the logits and the output, and the default one against the oracle
    buffer by buffer."""
    from reef_b200 import resources
    d1 = resources.generate("resnet18_64", str(tmp_path))
    d0 = resources.generate("resnet18_64", str(tmp_path), variant="_simtstem")
    b1, b0 = d1 + "/resnet18_64", d0 + "/resnet18_64_simtstem"
    j1, j0 = json.load(open(b1 + ".json")), json.load(open(b0 + ".json"))
    n1, n0 = [k["name"] for k in j1["kernels"]], [k["name"] for k in j0["kernels"]]
    assert n1[0].startswith("reef_im2col_nchw__c3") and "_ci160_" in n1[1] and "_kh1_kw1_" in n1[1] and "_v1" in n1[1]
    assert "_nchw1" in n0[1] and not any(n.startswith("reef_im2col") for n in n0)
    x = seeded_input(3 * 64 * 64, seed=6)
    outs = []
    for b in (b1, b0):
        e = load_executor(b)
        e.set_input("data", x)
        e.execute()
        outs.append(e.get_output().copy())
        assert capi.device_error() == 0
    assert rel_err(outs[0], outs[1]) < TF32_TOL
    e = load_executor(b1)
    o = oracle.OracleExecutor(b1 + ".json", b1 + ".param")
    e.set_input("data", x)
    o.set_input("data", x)
    e.execute()
    o.execute()
    worst = compare_layers(e, o, j1, lambda n: TF32_TOL)
    print("im2col stem worst layer", worst)


@pytest.mark.parametrize("case", CONV_CASES, ids=[c[0][9:] + f"_{c[1]}x{c[4]}k{c[5]}{c[6]}s{c[7]}" for c in CONV_CASES])
def test_conv_kernel_parity(tmp_path, case):
    _conv_case(tmp_path, case, "", FP32_TOL)


def _conv_case(tmp_path, case, suffix, tol):
    fam, ci, hi, wi, co, kh, kw, s, ph, pw = case
    ho, wo = (hi + 2 * ph - kh) // s + 1, (wi + 2 * pw - kw) // s + 1
    name = f"{fam}__ci{ci}_hi{hi}_wi{wi}_co{co}_kh{kh}_kw{kw}_sh{s}_sw{s}_ph{ph}_pw{pw}{suffix}"
    specs = [("in", ci * hi * wi), ("param", co * kh * kw * ci), ("out", ho * wo * co)]
    tail = fam[len("fused_nn_conv2d"):].replace("_nn_relu", "")
    if tail == "_add":
        specs.append(("param", co) if fam.endswith("_nn_relu") else ("in", ho * wo * co))
    elif tail == "_add_add":
        specs += [("in", ho * wo * co), ("param", co)]
    elif tail == "_add_multiply_add":
        specs += [("in", ho * wo * co), ("param", co), ("param", co)]
    base, inputs = single_kernel_model(tmp_path, "one", name, specs)
    e = load_executor(base)
    o = oracle.OracleExecutor(base + ".json", base + ".param")
    for k, v in inputs.items():
        e.set_input(k, v)
        o.set_input(k, v)
    e.execute()
    o.execute()
    err = rel_err(e.get_output(), o.get_output())
    print(name, "rel err", err, "launch", capi.kernel_plan(name)[0])
    assert capi.device_error() == 0
    assert err < tol
    # the best-effort flavour and the dispatcher run the same body: bit-identical to the raw launch
    raw = e.get_output()
    e.execute_preemptable()
    assert np.array_equal(e.get_output(), raw)
    e.execute_dispatch()
    assert np.array_equal(e.get_output(), raw)
    e.execute_graph()
    assert np.array_equal(e.get_output(), raw)
    assert capi.device_error() == 0


@pytest.mark.parametrize("variant", ["", "_fp32"])
@pytest.mark.parametrize("model", ["resnet18_64", "resnet50_64"])
def test_small_resnet_layer_by_layer(gen, model, variant):
    base = gen(model, variant=variant)
    tol = tol_for(base)
    assert tol == (TF32_TOL if variant == "" else FP32_TOL)
    j = json.load(open(base + ".json"))
    x = seeded_input(3 * 64 * 64)
    e = load_executor(base)
    o = oracle.OracleExecutor(base + ".json", base + ".param")
    e.set_input("data", x)
    o.set_input("data", x)
    e.execute()
    o.execute()
    worst = compare_layers(e, o, j, lambda kname: tol)
    print(model + variant, "worst layer rel err", worst)
    assert capi.device_error() == 0
    assert abs(float(e.get_output().sum()) - 1.0) < 1e-4


def test_resnet18_golden_const10(gen):
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "resnet18_64_fp32_const10.npz"))
    base = gen("resnet18_64", variant="_fp32")
    tol = tol_for(base)
    j = json.load(open(base + ".json"))
    e = load_executor(base)
    e.set_input("data", np.full(3 * 64 * 64, 10.0, np.float32))
    e.execute()
    li = j["kernels"][-1]["args"][0]
    assert rel_err(e.get_data(li, 4000), g["logits"]) < tol
    assert rel_err(e.get_output(), g["probs"]) < tol


@pytest.mark.parametrize("model,variant", [("resnet18", ""), ("resnet18", "_fp32"), ("resnet152", ""), ("resnet152", "_fp32")])
def test_full_size_resnet_logits_and_probs(gen, model, variant):
    base = gen(model, variant=variant)
    tol = tol_for(base)
    j = json.load(open(base + ".json"))
    x = seeded_input(3 * 224 * 224, seed=11)
    e = load_executor(base)
    o = oracle.OracleExecutor(base + ".json", base + ".param")
    e.set_input("data", x)
    o.set_input("data", x)
    e.execute()
    o.execute()
    li = j["kernels"][-1]["args"][0]
    err_logits = rel_err(e.get_data(li, 4000), o.storage[li])
    err_probs = rel_err(e.get_output(), o.get_output())
    print(model + variant, "logits rel err", err_logits, "probs rel err", err_probs, "tol", tol)
    assert capi.device_error() == 0
    assert err_logits < tol and err_probs < tol
    # graph replay, dispatcher and best-effort flavour give the same bytes as the raw launches
    raw = e.get_output()
    for f in ("execute_graph", "execute_dispatch", "execute_preemptable"):
        getattr(e, f)()
        assert np.array_equal(e.get_output(), raw), f


@pytest.mark.parametrize("model,delays", [("resnet50_64", [10, 20, 40, 60, 100, 150, 250]), ("resnet152", [100, 400, 900, 1500])])
def test_preempted_and_rerun_is_bit_identical(gen, model, delays):
    """A best-effort run that is preempted (flag raised mid-flight) and resumed from the first kernel whose
    completion counter is short must leave every buffer bit-identical to an uninterrupted GPU run."""
    base = gen(model)
    j = json.load(open(base + ".json"))
    n_in = j["storage"][0]["size"]
    x = seeded_input(n_in, seed=5)
    ref = load_executor(base)
    ref.set_input("data", x)
    ref.execute_preemptable()
    want = all_storage(ref, j)
    slots, blocks = ref.task_slots()
    assert slots == blocks                      # every kernel's counter reached its block count
    hit = 0
    for rep in range(3):          # where a delay lands depends on the host's launch rate: a second and third round if none did
        for d in delays:
            e = load_executor(base)
            e.set_input("data", x)
            restarts, first = e.execute_preempt_resume(d)
            hit += restarts > 0
            got = all_storage(e, j)
            for i, (a, b) in enumerate(zip(got, want)):
                assert np.array_equal(a, b), f"delay {d}us: storage {i} differs after {restarts} restarts (first {first})"
            print(model, "delay", d, "us -> restarts", restarts, "first incomplete kernel", first)
        if hit > 0:
            break
    assert hit > 0, "no delay landed inside the run; preemption was not exercised"


def test_profiler_writes_reference_schema(gen, tmp_path):
    """The measured profile parses with the reference-schema reader and has a positive latency for every
    distinct kernel (reference: test.cpp:79-91 parser.parse_profile)."""
    import ctypes as C
    import shutil
    from reef_b200 import profiler
    base = gen("resnet18_64")
    for ext in (".json", ".param"):
        shutil.copy(base + ext, str(tmp_path / ("m" + ext)))
    out = profiler.profile_model(str(tmp_path / "m"), iters=3)
    j = json.load(open(base + ".json"))
    prof = json.load(open(out))
    assert prof["latency_unit_ns"] == 1 and prof["model_latency"] > 0
    assert set(prof["kernel_latency"]) == {k["name"] for k in j["kernels"]}
    n, ml, mn = C.c_size_t(), C.c_int(), C.c_int()
    assert capi.host_lib().reef_profile_parse(out.encode(), C.byref(n), C.byref(ml), C.byref(mn)) == capi.SUCC
    assert n.value == len(prof["kernel_latency"]) and mn.value > 0
    # the executor accepts it
    e = capi.HybridExecutor(0)
    e.load_model_from_file(str(tmp_path / "m.json"), out)


@pytest.mark.parametrize("model,inp,n", [("vgg16_32", "data", 3 * 32 * 32), ("densenet121_64", "data", 3 * 64 * 64),
                                         ("inception_v3_139", "data", 3 * 139 * 139), ("bert_tiny", "input0", 48)])
def test_more_models_layer_by_layer(gen, model, inp, n):
    """VGG (conv+bias+ReLU, 2x2 max-pool, dense+ReLU), DenseNet (concat by channel offset, 2x2 avg-pool) and
    BERT (embedding, LayerNorm, tensor-core matmul with bias/GELU/residual, attention), every buffer."""
    base = gen(model)
    j = json.load(open(base + ".json"))
    x = seeded_input(n) if inp == "data" else np.random.default_rng(3).integers(0, 1000, n).astype(np.int64)
    e = load_executor(base)
    o = oracle.OracleExecutor(base + ".json", base + ".param")
    e.set_input(inp, x)
    o.set_input(inp, x)
    e.execute()
    o.execute()
    tol = tol_for(base)
    worst = compare_layers(e, o, j, lambda kname: tol)
    print(model, "worst layer rel err", worst)
    assert capi.device_error() == 0
    raw = e.get_output()
    for f in ("execute_graph", "execute_preemptable", "execute_dispatch"):
        getattr(e, f)()
        assert np.array_equal(e.get_output(), raw), f


@pytest.mark.parametrize("model,inp", [("vgg16", "data"), ("densenet201", "data"), ("inception_v3", "data"),
                                       ("bert_base", "input0")])
def test_more_models_full_size(gen, model, inp):
    """Full-size VGG-16, DenseNet-201, Inception-v3 and BERT-base: EVERY buffer a kernel writes (logits included),
    not only the normalised output, against the oracle."""
    base = gen(model)
    j = json.load(open(base + ".json"))
    if inp == "data":
        x = seeded_input(j["storage"][0]["size"], seed=12)
    else:
        x = np.random.default_rng(12).integers(0, 30522, 128).astype(np.int64)
    e = load_executor(base)
    o = oracle.OracleExecutor(base + ".json", base + ".param")
    e.set_input(inp, x)
    o.set_input(inp, x)
    e.execute()
    o.execute()
    tol = tol_for(base)
    worst = compare_layers(e, o, j, lambda kname: tol)
    err = rel_err(e.get_output(), o.get_output())
    if inp == "data":
        li = j["kernels"][-1]["args"][0]      # input of the final softmax = logits
        err_logits = rel_err(e.get_data(li, j["storage"][li]["size"] * 4), o.storage[li])
        print(model, "logits rel err", err_logits)
        assert err_logits < tol
    print(model, "worst layer", worst, "output rel err", err, "tol", tol, "graph ms", e.time(1, 3, 10))
    assert capi.device_error() == 0 and err < tol


def _unrounded_reference(gen, model, inp, x):
    """Oracle run of the `_fp32` variant of the same seed: the same architecture with the weights as drawn (not
    rounded to TF32) and every convolution / matmul in fp32.  Returns (logits or hidden states, output)."""
    base32 = gen(model, variant="_fp32")
    j32 = json.load(open(base32 + ".json"))
    o = oracle.OracleExecutor(base32 + ".json", base32 + ".param")
    o.set_input(inp, x)
    o.execute()
    li = j32["kernels"][-1]["args"][0] if inp == "data" else None
    return (o.storage[li].copy() if li is not None else None), o.get_output().copy()


@pytest.mark.parametrize("model,inp", [("resnet18", "data"), ("resnet152", "data"), ("inception_v3", "data"),
                                       ("bert_base", "input0")])
def test_tf32_schedule_against_the_unrounded_fp32_model(gen, model, inp):
    """The comparison the accuracy bound is stated for: the default schedule on the GPU (TF32 tensor cores, weights
    stored pre-rounded to TF32, activations rounded between layers) against the fp32 model with UNROUNDED weights of
    the same seed, through the whole depth of the network: max relative error <= 1e-2 on logits and on the output."""
    base = gen(model)
    j = json.load(open(base + ".json"))
    if inp == "data":
        x = seeded_input(j["storage"][0]["size"], seed=13)
    else:
        x = np.random.default_rng(13).integers(0, 30522, 128).astype(np.int64)
    want_logits, want_out = _unrounded_reference(gen, model, inp, x)
    # the two parameter files hold different weights for the tensor-core layers (rounded / as drawn)
    from reef_b200.resources.graph import read_param_file
    pa, pb = read_param_file(base + ".param"), read_param_file(gen(model, variant="_fp32") + ".param")
    rounded = 0
    # the two builds draw the same parameters in the same order; the default schedule holds a few arrays the fp32 one
    # does not (the im2col bias, the first convolution's weights flattened and padded), so the lists are walked side
    # by side and an array without a partner of its size among the next few is skipped
    la, lb = list(pa.values()), list(pb.values())
    i = 0
    for b in lb:
        j2 = next((q for q in range(i, min(i + 4, len(la))) if la[q].size == b.size), None)
        if j2 is None:
            continue
        a, i = la[j2], j2 + 1
        if not np.array_equal(a, b):
            assert np.abs(a - b).max() <= 2.0 ** -10 * np.abs(b).max()    # a rounded copy, not another tensor
            rounded += 1
    assert rounded > 10, "the default schedule's tensor-core weights should be rounded copies of the fp32 model's"
    e = load_executor(base)
    e.set_input(inp, x)
    e.execute()
    err_out = rel_err(e.get_output(), want_out)
    print(model, "TF32 GPU vs unrounded fp32 oracle: output rel err", err_out)
    assert capi.device_error() == 0
    assert err_out < TF32_TOL
    if want_logits is not None:
        li = j["kernels"][-1]["args"][0]
        err_logits = rel_err(e.get_data(li, j["storage"][li]["size"] * 4), want_logits)
        print(model, "logits rel err", err_logits)
        assert err_logits < TF32_TOL


MID_KERNEL_CASES = [
    # a kernel whose blocks are ALL resident from the start (fewer blocks than the GPU holds at once): with polls at
    # block entry only, a flag raised after the launch could stop nothing and the counter would reach the block count
    ("dense", "fused_nn_dense_add_nn_relu__k25088_n4096", [("in", 25088), ("param", 4096 * 25088), ("out", 4096), ("param", 4096)],
     [10, 20, 30, 45, 60], 30),
    ("conv3x3_tc", "fused_nn_conv2d_add_nn_relu__ci1024_hi14_wi14_co1024_kh3_kw3_sh1_sw1_ph1_pw1_v1",
     [("in", 1024 * 14 * 14), ("param", 1024 * 9 * 1024), ("out", 1024 * 14 * 14), ("param", 1024)], [1, 2, 3, 4, 5, 6, 8, 10, 12], 6),
]


@pytest.mark.parametrize("case", MID_KERNEL_CASES, ids=[c[0] for c in MID_KERNEL_CASES])
def test_best_effort_kernel_leaves_mid_kernel(tmp_path, case):
    """Loop-head polls of the preempt flag (VGG-16's first dense layer, a GEMV of 411 MB; a 3x3 tensor-core
    convolution): the flag goes up while the single kernel of the model runs, with all of its blocks resident since
    the launch.  In some attempt the completion counter stays short of the block count — blocks left in the middle —
    and after every attempt the resumed run leaves output bit-identical to an uninterrupted one."""
    tag, name, specs, delays, started_by = case   # started_by: a delay (us) by which the kernel's blocks are surely running
    base, inputs = single_kernel_model(tmp_path, "one", name, specs)
    j = json.load(open(base + ".json"))
    dims = capi.kernel_plan(name)[0]
    nblocks = dims[0] * dims[1] * dims[2]
    assert nblocks <= 2 * 148, "the case is meant to be resident as a whole"
    ref = load_executor(base)
    for k, v in inputs.items():
        ref.set_input(k, v)
    ref.execute_preemptable()
    want = all_storage(ref, j)
    assert ref.task_slots()[0] == ref.task_slots()[1]
    e = load_executor(base)
    for k, v in inputs.items():
        e.set_input(k, v)
    seen = []
    for rep in range(6):
        for d in delays:
            restarts, first, count = e.execute_preempt_resume(d, with_count=True)
            if restarts > 0:
                seen.append((d, count))
            got = all_storage(e, j)
            for i, (a, b) in enumerate(zip(got, want)):
                assert np.array_equal(a, b), f"{tag} delay {d}us: storage {i} differs after {restarts} restarts"
        if any(c < nblocks for _, c in seen) and rep >= 1:
            break
    print(tag, "blocks", nblocks, "preempted attempts (delay us, counter when found short):", seen[:12])
    assert capi.device_error() == 0
    assert seen, "no attempt was preempted"
    # a launch reaches the SMs within a few microseconds: an attempt preempted at `started_by` or later was stopped
    # while its blocks were running, and its counter short of the block count says they left before their end
    assert any(d >= started_by and 0 <= c < nblocks for d, c in seen), "the kernel never left in the middle"


@pytest.mark.parametrize("s,heads,mask", [(128, 12, 0), (48, 2, 0), (100, 3, 1), (128, 4, 1), (1, 1, 0)])
def test_attention_tensor_core_parity(tmp_path, s, heads, mask):
    """reef_attention _v1: QK^T and PV on tcgen05 (one CTA per head, up to 128 tokens), softmax in registers, against the
    oracle; ragged sequence lengths (rows and keys beyond the sequence), a key mask, every launch flavour bit-identical;
    and against the CUDA-core variant of the same kernel."""
    H = heads * 64
    name = f"reef_attention__s{s}_heads{heads}_d64" + ("_mask1" if mask else "")
    specs = [("in", s * 3 * H)] + ([("in", s)] if mask else []) + [("out", s * H)]
    outs = {}
    for variant in ("_v1", ""):
        base, inputs = single_kernel_model(tmp_path / ("m" + variant), "one", name + variant, specs, seed=s + heads)
        if mask:
            m = (np.random.default_rng(5).random(s) > 0.3).astype(np.float32)
            m[0] = 1.0
            inputs["in1"] = m
        e = load_executor(base, params=False)      # the kernel has no parameters
        o = oracle.OracleExecutor(base + ".json")
        for k, v in inputs.items():
            e.set_input(k, v)
            o.set_input(k, v)
        e.execute()
        o.execute()
        got = e.get_output()
        err = rel_err(got, o.get_output())
        print(name + variant, "rel err", err)
        assert capi.device_error() == 0
        assert not np.isnan(got).any() and err < (TF32_TOL if variant else FP32_TOL)
        for f in ("execute_preemptable", "execute_dispatch", "execute_graph"):
            getattr(e, f)()
            assert np.array_equal(e.get_output(), got), f
        outs[variant] = got
    assert rel_err(outs["_v1"], outs[""]) < TF32_TOL


@pytest.mark.parametrize("model,clusters", [("resnet18_64", 0), ("resnet50_64", 4), ("resnet152", 0), ("resnet152", 9), ("bert_base", 0),
                                            ("inception_v3_139", 0), ("vgg16_32", 0), ("densenet121_64", 0)])
def test_persistent_chain_is_bit_identical(gen, model, clusters):
    """Runs of consecutive tensor-core layers as ONE persistent kernel (8-CTA clusters walking the layer list, layers
    ordered by completion counters): every buffer bit-identical to the per-kernel launches, directly and as a CUDA
    graph, for every K split the plans use and for several grid sizes (the tile -> CTA mapping changes with the
    number of clusters, the arithmetic must not)."""
    base = gen(model)
    j = json.load(open(base + ".json"))
    st = j["storage"][0]
    x = seeded_input(st["size"], seed=17) if st["stype"] == "float32" else np.random.default_rng(17).integers(0, 1000, st["size"]).astype(np.int64)
    ref = load_executor(base)
    ref.set_input(st["name"], x)
    ref.execute()
    want = all_storage(ref, j)
    e = load_executor(base)
    n = e.build_chains(clusters)
    assert n >= 1
    e.set_input(st["name"], x)
    for rep in range(3):
        e.execute_chained()
        got = all_storage(e, j)
        for i, (a, b) in enumerate(zip(got, want)):
            assert np.array_equal(a, b), f"{model}: storage {i} differs (chained run {rep})"
    assert capi.device_error() == 0
    e.execute_graph()
    e.execute_graph()
    got = all_storage(e, j)
    for i, (a, b) in enumerate(zip(got, want)):
        assert np.array_equal(a, b), f"{model}: storage {i} differs (graph with chains)"
    assert capi.device_error() == 0
    print(model, "chains", n, "clusters asked", clusters, "chain 0 (begin, end, clusters, max)", e.chain_info(0), "graph ms plain", ref.time(1, 3, 20), "with chains", e.time(1, 3, 20))


@pytest.mark.parametrize("model,clusters,delays", [("resnet50_64", 2, [30, 80, 200]), ("resnet152", 4, [200, 700, 2500]),
                                                   ("resnet152", 0, [100, 400, 1200])])
def test_best_effort_chain_preempted_and_resumed_is_bit_identical(gen, model, clusters, delays):
    """The best-effort form of a persistent chain: the preempt flag goes up while the chain walks its layers, every
    cluster leaves at its next tile boundary, the completion counters give the first incomplete layer and the chain is
    restarted there.  Every buffer ends bit-identical to an uninterrupted per-kernel run, for a chain that runs on a
    few clusters (the padding configuration) as well as on the default grid."""
    base = gen(model)
    j = json.load(open(base + ".json"))
    x = seeded_input(j["storage"][0]["size"], seed=23)
    ref = load_executor(base)
    ref.set_input("data", x)
    ref.execute()
    want = all_storage(ref, j)
    e = load_executor(base)
    assert e.build_chains(0) >= 1
    e.set_input("data", x)
    hit = []
    b, en, _, _ = e.chain_info(0)
    for rep in range(3):      # where a delay lands depends on the host's launch rate: up to three rounds
        for d in delays:
            restarts, first = e.execute_preempt_resume_chained(d, clusters)
            hit.append((d, restarts, first))
            got = all_storage(e, j)
            for i, (a, bb) in enumerate(zip(got, want)):
                assert np.array_equal(a, bb), f"{model} delay {d}us: storage {i} differs after {restarts} restarts (first {first})"
        if any(b < f < en for _, r, f in hit if r > 0):
            break
    print(model, "clusters", clusters, "(delay us, restarts, first incomplete kernel):", hit)
    assert capi.device_error() == 0
    assert any(r > 0 for _, r, _ in hit), "no delay landed inside the run"
    assert any(b < f < en for _, r, f in hit if r > 0), "no preemption stopped the chain in the middle of its layers"


def test_stream_latency_probe_and_untimed_events():
    """reef_probe_stream_latency returns positive medians, and a completion-only event is seen complete by the host no
    later than a timed one (the reason the scheduler tracks completion with reef_event_create_untimed)."""
    w, wc, ev, evt = capi.probe_stream_latency(200, 0)
    print("write call", w, "write+completion", wc, "untimed event", ev, "timed event", evt)
    assert 0 < w < wc and 0 < ev <= evt * 1.5 and wc < 1000 and evt < 1000
    assert capi.device_error() == 0
