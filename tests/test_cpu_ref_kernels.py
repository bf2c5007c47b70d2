"""Pins the C oracle against the reference's OWN kernels.

`tests/golden/ref_kernels.npz` holds outputs of the reference's generated kernel sources (resource/resnet152/resnet152.cu,
resource/bert/bert.cu, resource/inception/inception.cu), compiled unchanged and executed on the CPU (oracle/refkernels,
`make -C oracle ref`), for the cases of tests/ref_cases.py.  Here the oracle's restatement of each of those kernels
runs on the same seeded inputs and must agree with the reference's arithmetic: convolutions (7x7 stem, 3x3, 1x1,
stride 2, every epilogue variant), pooling with its pad value, average pooling that counts the padding, bias add,
bias + ReLU, global average pool, flatten, the GEMV, the 1000-way softmax, and BERT's LayerNorm (five launches in the
reference), bias + exact-erf GELU, X W^T, row softmax (four launches), QK^T -> masked fill -> softmax -> PV, and the
clamped embedding gather.  Tolerance 1e-5 of the largest output (fp32 sums in another order); the copies and
comparisons that involve no arithmetic must be bit-exact.
Where the compiled reference kernels are present (oracle/_ref) the same comparison also runs live on fresh seeds."""
import os

import numpy as np
import pytest

from conftest import rel_err
import ref_cases as RC
from oracle import ref_kernels as R

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_kernels.npz")
TOL = 1e-5
EXACT = {"input_bias_add", "bias_relu", "batch_flatten", "max_pool3x3_s2_bias_relu", "bert_embedding"}


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


@pytest.mark.parametrize("cid", sorted(RC.CASES))
def test_oracle_matches_the_reference_kernel(golden, cid):
    d = RC.case_inputs(cid)
    assert abs(RC.input_checksum(d) - float(golden[cid + "__input_checksum"][0])) <= 1e-6 * max(1.0, abs(float(golden[cid + "__input_checksum"][0]))), \
        "the seeded inputs differ from those the fixture was made with (random generator changed?)"
    y = RC.CASES[cid]["oracle"](d)
    assert tuple(y.shape) == tuple(golden[cid + "__shape"])
    got, want = RC.subsample(y), golden[cid]
    assert not np.isnan(got).any()
    if cid in EXACT:
        assert np.array_equal(got, want), cid
    else:
        err = rel_err(got, want)
        assert err < TOL, f"{cid}: rel err {err}"


def test_fixture_covers_every_case(golden):
    assert {k for k in golden.files if "__" not in k} == set(RC.CASES)


@pytest.mark.skipif(not all(R.available(m) for m in ("resnet152", "bert", "inception")),
                    reason="the compiled reference kernels (oracle/_ref) are not present on this machine")
@pytest.mark.parametrize("cid", sorted(RC.CASES))
def test_live_reference_kernel_against_oracle_and_fixture(golden, cid):
    """With oracle/_ref present: the reference kernel itself runs here, reproduces the committed fixture bit for bit
    (the fixture is what the reference computes, not something edited) and agrees with the oracle on other inputs."""
    d = RC.case_inputs(cid)
    y = RC.CASES[cid]["ref"](R, d)
    assert np.array_equal(RC.subsample(y).astype(np.float32), golden[cid])
    d2 = RC.CASES[cid]["inputs"](np.random.default_rng(RC.hash_str(cid) % 1000 + 77))
    yr, yo = RC.CASES[cid]["ref"](R, d2), RC.CASES[cid]["oracle"](d2)
    assert rel_err(yo, yr) < TOL
