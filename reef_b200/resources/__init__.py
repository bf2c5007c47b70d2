"""Generator of REEF model resources (``<model>.json`` + ``.param`` + ``.profile.json``).

Replaces the reference's TVM export + schedule merge (reference: script/tvm_generate_model.py,
script/generate_final_schedule.py) for the synthetic benchmark configs: the architectures are
authored here, the kernel list is chosen here, and launch geometry comes from the kernel registry
through the C-ABI (``reef_kernel_plan``), so the json cannot disagree with the library.
"""
from __future__ import annotations

import os

from .graph import Graph, kname, parse_kname, read_param_file, write_param_file  # noqa: F401
from .mocked import build_mocked_kernel
from .bert import build_bert
from .densenet import build_densenet
from .inception import build_inception_v3
from .resnet import build_resnet
from .vgg import build_vgg16

DEFAULT_DIR = os.environ.get("REEF_RESOURCE_DIR", "/tmp/reef_b200_resources")

# seeds: 1000 * (index of the benchmark config the model first appears in) + model ordinal
_BUILDERS = {
    "resnet18": lambda **kw: build_resnet(18, seed=1000, **kw),
    "resnet50": lambda **kw: build_resnet(50, seed=5001, **kw),
    "resnet152": lambda **kw: build_resnet(152, seed=2000, **kw),
    # small variants for fast parity tests (same builders, 64x64 input like the reference's shipped resnet152)
    "resnet18_64": lambda **kw: build_resnet(18, name="resnet18_64", image=64, seed=1064, **kw),
    "resnet50_64": lambda **kw: build_resnet(50, name="resnet50_64", image=64, seed=5064, **kw),
    "bert_base": lambda **kw: build_bert(**kw),
    "bert_tiny": lambda **kw: build_bert(name="bert_tiny", layers=2, hidden=128, heads=2, ffn=256, vocab=1000, seq=48,
                                         seed=5048, **kw),
    "inception_v3": lambda **kw: build_inception_v3(**kw),
    "inception_v3_139": lambda **kw: build_inception_v3(name="inception_v3_139", image=139, seed=4139, **kw),
    "vgg16": lambda **kw: build_vgg16(**kw),
    "vgg16_32": lambda **kw: build_vgg16(name="vgg16_32", image=32, fc=256, seed=4032, **kw),
    "densenet201": lambda **kw: build_densenet(201, **kw),
    "densenet121_64": lambda **kw: build_densenet(121, name="densenet121_64", image=64, seed=4064, **kw),
}


def _generator_stamp() -> str:
    """Changes whenever the generator sources or the kernel library (launch plans) change, so cached
    resource directories written by an older build are regenerated instead of silently reused."""
    import glob
    import hashlib
    h = hashlib.sha256()
    here = os.path.dirname(os.path.abspath(__file__))
    h.update(os.environ.get("REEF_UNTUNED", "").encode())
    for f in sorted(glob.glob(os.path.join(here, "*.py")) + glob.glob(os.path.join(here, "tuned_plans.json"))):
        with open(f, "rb") as fh:
            h.update(fh.read())
    stamp = os.path.join(os.path.dirname(here), "libreef_cuda.so.stamp")
    if os.path.exists(stamp):
        with open(stamp, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def available():
    return ["mocked_kernel"] + sorted(_BUILDERS)


def generate(model: str, out_root: str | None = None, *, force: bool = False, variant: str = "", **kw) -> str:
    """Write the resources of `model` under <out_root>/<model><variant>/ and return that directory.

    ``variant="_fp32"`` selects the exact-fp32 schedule (CUDA-core convolutions only); the default
    schedule uses the tcgen05 TF32 convolution wherever the registry supports the shape."""
    if variant == "_fp32":
        kw.setdefault("conv_impl", "simt")
    elif variant == "_simtstem":
        kw.setdefault("conv_impl", "simt_stem")   # tensor-core schedule with the first convolution left on CUDA cores
    from .. import capi
    out_root = out_root or DEFAULT_DIR
    name = model + variant
    out_dir = os.path.join(out_root, name)
    base = os.path.join(out_dir, name)
    exts = (".json", ".profile.json") if model == "mocked_kernel" else (".json", ".param", ".profile.json")
    stamp_path = base + ".generator"
    stamp = _generator_stamp() + repr(sorted(kw.items()))
    if not force and all(os.path.exists(base + ext) for ext in exts) and os.path.exists(stamp_path) \
            and open(stamp_path).read() == stamp:
        return out_dir
    if model == "mocked_kernel":
        g = build_mocked_kernel()
        g.name = name
        # mocked_kernel has no parameters; the reference ships no .param for it
        os.makedirs(out_dir, exist_ok=True)
        import json
        j = g.finalize(capi.plan_fn)
        with open(base + ".json", "w") as f:
            json.dump(j, f, indent=1)
        from .graph import default_profile
        with open(base + ".profile.json", "w") as f:
            json.dump(default_profile(j), f)
        with open(stamp_path, "w") as f:
            f.write(stamp)
        return out_dir
    b = _BUILDERS[model](**kw)
    b.g.name = name
    b.g.write(out_dir, capi.plan_fn)
    with open(stamp_path, "w") as f:
        f.write(stamp)
    return out_dir
