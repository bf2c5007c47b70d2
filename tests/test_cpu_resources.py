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
    names = _declared("reef_cuda.h")
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
    """flops.py: ResNet-18 3.65 GFLOP / 46.8 MB of weights, ResNet-50 7.72 GFLOP / 102 MB at 224x224, batch 1."""
    from reef_b200 import flops
    t18 = flops.model_totals("resnet18", str(tmp_path))["totals"]
    assert abs(t18["flops"] / 1e9 - 3.65) < 0.05 and abs(t18["weight_bytes"] / 1e6 - 46.8) < 0.5
    t50 = flops.model_totals("resnet50", str(tmp_path))["totals"]
    assert abs(t50["flops"] / 1e9 - 7.72) < 0.05 and abs(t50["weight_bytes"] / 1e6 - 102.1) < 0.5
    assert t50["tensor_core_kernels"] == 52 and t50["hbm_floor_us_nominal"] > t50["tf32_floor_us_nominal"]


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
