"""CPU tests of the resource layout: json schema, .param byte format, profile schema, the C++ parsers
(mirrors reference src/reef/test/test.cpp:59-91 parser.*) and the C-ABI export list."""
import ctypes as C
import json
import os
import re
import struct

import numpy as np
import pytest

from reef_b200 import capi, resources
from reef_b200.resources.graph import PARAM_MAGIC, kname, parse_kname, read_param_file, write_param_file

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_kname_roundtrip():
    n = kname("fused_nn_conv2d_add_nn_relu", ci=64, hi=56, wi=56, co=256, kh=1, kw=1, sh=1, sw=1, ph=0, pw=0)
    op, a = parse_kname(n)
    assert op == "fused_nn_conv2d_add_nn_relu" and a["co"] == 256 and a["pw"] == 0
    assert parse_kname("add") == ("add", {})


def test_mocked_kernel_json_matches_reference_schema(gen):
    base = gen("mocked_kernel")
    j = json.load(open(base + ".json"))
    # reference: resource/mocked_kernel/mocked_kernel.json:1-72
    assert [s["name"] for s in j["storage"]] == ["a", "b", "temp", "c", "output"]
    assert all(s["size"] == 8192 and s["stype"] == "float32" for s in j["storage"])
    assert [k["name"] for k in j["kernels"]] == ["add", "multiply"]
    assert j["kernels"][0]["launch_params"] == [64, 1, 1, 4, 8, 4]
    assert j["kernels"][0]["args"] == [1, 0, 2] and j["kernels"][1]["args"] == [2, 3, 4]
    assert j["args"] == [0, 1, 3]
    assert set(j["shared_memory"]) == {"add", "multiply"}


def test_param_format_bytes(tmp_path):
    p = tmp_path / "x.param"
    write_param_file(str(p), {"p0": np.arange(3, dtype=np.float32), "p22": np.ones(5, np.float32)})
    raw = p.read_bytes()
    # reference writer: script/tvm_generate_model.py:66-76
    assert raw[:17] == PARAM_MAGIC and len(PARAM_MAGIC) == 17
    assert struct.unpack("<Q", raw[17:25])[0] == 2
    assert raw[25:28] == b"p0\0" and struct.unpack("<Q", raw[28:36])[0] == 3
    back = read_param_file(str(p))
    assert back["p22"].tolist() == [1.0] * 5


def test_cpp_parsers_resnet18(gen, libs):
    base = gen("resnet18")
    L = capi.host_lib()
    ns, nk, na = C.c_size_t(), C.c_size_t(), C.c_size_t()
    assert L.reef_model_parse((base + ".json").encode(), C.byref(ns), C.byref(nk), C.byref(na)) == capi.SUCC
    j = json.load(open(base + ".json"))
    assert nk.value == len(j["kernels"]) != 0 and ns.value == len(j["storage"]) and na.value == len(j["args"])
    # parser.parse_params (reference test.cpp:68-77 expects p22 = 256*128*3*3 = 294912 for its ResNet-18):
    # our ResNet-18 has the same 3x3/2 128->256 conv; find it by size
    params = read_param_file(base + ".param")
    key = [k for k, v in params.items() if v.size == 294912][0]
    ke, nb = C.c_size_t(), C.c_size_t()
    assert L.reef_param_parse((base + ".param").encode(), key.encode(), C.byref(ke), C.byref(nb)) == capi.SUCC
    assert ke.value == 294912 and nb.value == len(params)
    # parser.parse_profile (reference test.cpp:79-91): every kernel has latencies > 0
    nkp, ml, mn = C.c_size_t(), C.c_int(), C.c_int()
    assert L.reef_profile_parse((base + ".profile.json").encode(), C.byref(nkp), C.byref(ml), C.byref(mn)) == capi.SUCC
    assert nkp.value == len({k["name"] for k in j["kernels"]}) and mn.value > 0


def test_cpp_parsers_reject_bad_files(tmp_path, libs):
    L = capi.host_lib()
    bad = tmp_path / "bad.json"
    bad.write_text('{"storage": [{"name": "a", "size": 4, "stype": "float32"}], "kernels": [{"name": "add", '
                   '"launch_params": [1,1,1,1,1,1], "args": [7]}], "args": [], "shared_memory": {}}')
    assert L.reef_model_parse(str(bad).encode(), None, None, None) == capi.NOT_FOUND   # index outside the table
    assert L.reef_model_parse(b"/nonexistent.json", None, None, None) == capi.NOT_FOUND
    short = tmp_path / "short.param"
    short.write_bytes(PARAM_MAGIC + struct.pack("<Q", 1) + b"p0\0" + struct.pack("<Q", 100) + b"\0" * 8)
    assert L.reef_param_parse(str(short).encode(), b"p0", None, None) == capi.NOT_FOUND  # truncated array
    wrong = tmp_path / "wrong.param"
    wrong.write_bytes(b"NOT_A_PARAM_FILE\0" + struct.pack("<Q", 1))
    assert L.reef_param_parse(str(wrong).encode(), b"p0", None, None) == capi.NOT_FOUND


def test_json_launch_params_come_from_registry(gen):
    base = gen("resnet18_64")
    j = json.load(open(base + ".json"))
    for k in j["kernels"]:
        dims, smem, nargs = capi.kernel_plan(k["name"])
        assert dims == k["launch_params"] and smem == j["shared_memory"][k["name"]] and nargs == len(k["args"])
    with pytest.raises(capi.ReefError) as e:
        capi.kernel_plan("fused_nn_unknown_op__n4")
    assert e.value.status == capi.NOT_FOUND


def test_no_storage_reuse_in_generated_schedules(gen):
    """Re-running a best-effort kernel must be exact: no kernel writes a buffer an earlier kernel still
    needs (the reference disables reuse for the same reason, script/generate_final_schedule.py:37-40)."""
    base = gen("resnet50_64")
    j = json.load(open(base + ".json"))
    written = set()
    for k in j["kernels"]:
        op, _ = parse_kname(k["name"])
        out = k["args"][0] if op in ("fused_add", "fused_add_nn_relu", "fused_nn_batch_flatten") else \
            (k["args"][2] if "conv2d" in op or "dense" in op else k["args"][1])
        assert out not in written, f"{k['name']} overwrites storage {out}"
        written.add(out)


def _declared(header):
    txt = open(os.path.join(ROOT, "include", header)).read()
    return sorted(set(re.findall(r"REEF_(?:HOST_)?API\s+[\w\s\*]+?\b(reef_[a-z0-9_]+)\s*\(", txt)))


def test_cabi_exports_every_declared_symbol(libs):
    cuda = C.CDLL(os.path.join(ROOT, "reef_b200", "libreef_cuda.so"), mode=C.RTLD_GLOBAL)
    names = _declared("reef_cuda.h")      # (reef_debug_aids.h declares what only a -DREEF_DEBUG_AIDS build exports)
    assert len(names) > 35
    for n in names:
        assert hasattr(cuda, n), f"libreef_cuda.so does not export {n}"
    host = C.CDLL(os.path.join(ROOT, "reef_b200", "libreef_host.so"))
    names = _declared("reef_host.h")
    assert len(names) > 40
    for n in names:
        assert hasattr(host, n), f"libreef_host.so does not export {n}"


def test_product_fails_loudly_without_gpu(libs):
    """No CPU fallback: on a machine without a GPU the executor refuses to start."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(capi.ReefError):
        capi.HybridExecutor(0)


def test_model_totals_match_the_published_architectures(libs, tmp_path):
    """flops.py: ResNet-18 3.65 GFLOP / 46.8 MB of weights, ResNet-50 7.72 GFLOP / 102 MB at 224x224, batch 1 (53 tensor-core
    kernels: 52 convolutions plus the first one, which runs as an im2col gather and a 1x1 tensor-core convolution)."""
    from reef_b200 import flops
    t18 = flops.model_totals("resnet18", str(tmp_path))["totals"]
    assert abs(t18["flops"] / 1e9 - 3.65) < 0.05 and abs(t18["weight_bytes"] / 1e6 - 46.8) < 0.5
    t50 = flops.model_totals("resnet50", str(tmp_path))["totals"]
    assert abs(t50["flops"] / 1e9 - 7.72) < 0.05 and abs(t50["weight_bytes"] / 1e6 - 102.1) < 0.5
    assert t50["tensor_core_kernels"] == 53 and t50["hbm_floor_us_nominal"] > t50["tf32_floor_us_nominal"]


def test_tuned_plan_table_is_consistent(libs):
    """Every measured plan in the table resolves in the registry, keeps the family's argument count, and is what
    the generator writes into the schedule; REEF_UNTUNED keeps the bare names."""
    import json
    import os
    from reef_b200 import capi, resources, tune
    from reef_b200.resources.graph import tuned_plan
    path = os.path.join(os.path.dirname(resources.__file__), "tuned_plans.json")
    table = json.load(open(path))
    assert table["plans"], "the committed table holds the measured plans"
    for name, (tp, ts) in table["plans"].items():
        assert name in table["measured_us"] and table["measured_us"][name][1] <= table["measured_us"][name][0]
        d0, _, n0 = capi.kernel_plan(name)
        d1, smem, n1 = capi.kernel_plan(f"{name}_tp{tp}_ts{ts}")
        assert n0 == n1 and smem <= 112 * 1024 and d1[3] == 256
        assert tuned_plan(name) == dict(tp=tp, ts=ts)
    # candidates(): the default plan first, then distinct (grid, shared memory) alternatives within 24..300 CTAs
    c = tune.candidates("fused_nn_conv2d_add_nn_relu__ci256_hi14_wi14_co256_kh3_kw3_sh1_sw1_ph1_pw1_v1")
    assert c[0][0] is None and len(c) > 4 and len({(g, s) for _, g, s in c[1:]}) == len(c) - 1
    assert all(24 <= g[0] * g[1] <= 300 for _, g, _ in c[1:])
    # the helper that sizes a timing model knows every tensor-core family
    assert tune._arg_sizes("reef_matmul_nt_bias_gelu", dict(m=128, n=3072, k=768))[:3] == (128 * 768, 3072 * 768, 128 * 3072)
    assert tune._arg_sizes("reef_conv2d_add_preact", dict(ci=64, hi=8, wi=8, co=128, kh=1, kw=1, sh=1, sw=1, ph=0, pw=0))[3] == \
        [("temp", 64 * 128), ("param", 128), ("temp", 64 * 128)]


def test_estimate_slot_usage(libs, tmp_path):
    from reef_b200 import estimate, resources
    d = resources.generate("resnet18_64", str(tmp_path))
    r = estimate.estimate(d)
    assert r["kernels"] > 20 and 0 < r["busy_pct"] <= r["busy_with_parked_successor_pct"] <= 100


REF_FIXTURES = os.path.join(ROOT, "tests", "golden", "ref")


@pytest.mark.parametrize("model,storage,kernels,args,profile_kernels,model_latency", [
    ("mocked_kernel", 5, 2, 3, 2, 30),
    ("resnet18", 101, 57, 44, 54, 2189),
    ("resnet152", 317, 207, 312, 35, 13233),
    ("bert", 112, 205, 102, 23, 5426),
    ("inception", 204, 146, 191, 75, 8273),
])
def test_cpp_parsers_read_the_reference_shipped_resources(libs, model, storage, kernels, args, profile_kernels, model_latency):
    """The reference's own <model>.json and <model>.profile.json (copied unchanged from its resource/ directory into
    tests/golden/ref) go through the C++ parsers with the expectations of the reference's parser tests
    (src/reef/test/test.cpp:59-65 parse_model: kernels != 0; :79-91 parse_profile: 54 kernels for resnet18, every kernel
    has a latency table and every latency is > 0).  Counts are those of the files themselves."""
    L = capi.host_lib()
    jpath = os.path.join(REF_FIXTURES, model + ".json")
    ns, nk, na = C.c_size_t(), C.c_size_t(), C.c_size_t()
    assert L.reef_model_parse(jpath.encode(), C.byref(ns), C.byref(nk), C.byref(na)) == capi.SUCC
    j = json.load(open(jpath))
    assert (ns.value, nk.value, na.value) == (len(j["storage"]), len(j["kernels"]), len(j["args"])) == (storage, kernels, args)
    assert nk.value != 0
    ppath = os.path.join(REF_FIXTURES, model + ".profile.json")
    nkp, ml, mn = C.c_size_t(), C.c_int(), C.c_int()
    assert L.reef_profile_parse(ppath.encode(), C.byref(nkp), C.byref(ml), C.byref(mn)) == capi.SUCC
    assert nkp.value == profile_kernels and ml.value == model_latency
    assert mn.value > 0          # every kernel has a non-empty latency table with entries > 0
    # the reference's kernels are TVM symbols of a per-model code object: the registry here does not know them
    # and says so instead of guessing
    if model != "mocked_kernel":
        err = C.create_string_buffer(512)
        assert L.reef_model_check(jpath.encode(), err, C.c_size_t(512)) == capi.NOT_FOUND
        assert b"kernel" in err.value


def test_reference_mocked_kernel_json_is_loadable_as_is(libs):
    """The reference's mocked_kernel.json (two kernels `add`, `multiply`, launch [64,1,1,4,8,4]) passes every check the
    loader makes before it touches the GPU: same names, same launch geometry, same storage sizes."""
    L = capi.host_lib()
    err = C.create_string_buffer(512)
    rc = L.reef_model_check(os.path.join(REF_FIXTURES, "mocked_kernel.json").encode(), err, C.c_size_t(512))
    assert rc == capi.SUCC, err.value


def test_loader_refuses_a_storage_entry_smaller_than_the_kernel_needs(gen, libs, tmp_path):
    """A json whose storage entry is smaller than what the shape in the kernel name makes the kernel touch is refused
    with OutOfRange before any device memory is allocated."""
    L = capi.host_lib()
    base = gen("resnet18_64")
    j = json.load(open(base + ".json"))
    err = C.create_string_buffer(512)
    assert L.reef_model_check((base + ".json").encode(), err, C.c_size_t(512)) == capi.SUCC, err.value
    # shrink the output buffer of a convolution in the middle of the network by one element
    k = [k for k in j["kernels"] if "conv2d" in k["name"]][5]
    victim = k["args"][2]
    j["storage"][victim]["size"] -= 1
    bad = tmp_path / "shrunk.json"
    bad.write_text(json.dumps(j))
    assert L.reef_model_check(str(bad).encode(), err, C.c_size_t(512)) == capi.OUT_OF_RANGE
    assert b"smaller than argument 2" in err.value and k["name"].encode() in err.value
    # and a weight buffer
    j = json.load(open(base + ".json"))
    j["storage"][k["args"][1]]["size"] //= 2
    bad.write_text(json.dumps(j))
    assert L.reef_model_check(str(bad).encode(), err, C.c_size_t(512)) == capi.OUT_OF_RANGE
    assert b"argument 1" in err.value


@pytest.mark.parametrize("model", ["resnet18", "resnet50_64", "vgg16_32", "densenet121_64", "inception_v3_139", "bert_tiny",
                                   "resnet18_64_fp32"])
def test_generated_schedules_pass_the_storage_size_check(gen, libs, model):
    """Every generated schedule binds each kernel argument to a storage entry of at least the size the kernel needs
    (one model per family here; the full-size schedules pass the same check whenever a GPU test loads them)."""
    L = capi.host_lib()
    if model.endswith("_fp32"):
        base = gen(model[:-5], variant="_fp32")
    else:
        base = gen(model)
    err = C.create_string_buffer(512)
    assert L.reef_model_check((base + ".json").encode(), err, C.c_size_t(512)) == capi.SUCC, err.value
