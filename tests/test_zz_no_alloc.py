"""reef_dispatch_static: the dispatcher entry point that allocates nothing.

Some callers of this library may not allocate device memory at the moment they need to launch a padded
kernel pair: a scheduler loop that is serving a real-time request (cudaMalloc would synchronise the device
under it) or code inside an open CUDA stream capture (where cudaMalloc is not allowed at all).  For them the
dispatcher's ticket counters live in a static device array inside libreef_cuda instead of in caller-owned
memory.  This test drives the entry point through the C-ABI exactly as such a caller would — the test itself
allocates the input/output buffers up front, the calls under test allocate nothing — and checks, on two
calls in a row on the same lane, that the outputs are bit-identical to those of the existing reef_dispatch
(same kernels, same bodies, so the tolerance is zero).  It is collected last so that a failure here cannot
hide the result of any other test.
"""
import ctypes as C

import numpy as np
import pytest

from reef_b200 import capi

pytestmark = pytest.mark.gpu

RT_NAME = "fused_nn_conv2d_add_nn_relu__ci32_hi15_wi15_co72_kh3_kw3_sh2_sw2_ph1_pw1"   # 8x8x72 out, 2 blocks
BE_NAME = "fused_add_nn_relu__c64_n3136"                                               # 49 blocks


class _Dev:
    """Raw C-ABI helper: device buffers and kernel handles (set-up, not the code under test)."""

    def __init__(self):
        self.L = capi.cuda_lib()
        assert self.L.reef_gpu_init(C.c_int(0)) == capi.SUCC, capi.last_error()
        self.mod = C.c_void_p()
        assert self.L.reef_module_open(None, C.byref(self.mod)) == capi.SUCC
        self.stream = C.c_void_p()
        assert self.L.reef_stream_create(C.byref(self.stream), C.c_int(0)) == capi.SUCC
        self.bufs = []

    def kernel(self, name):
        k = C.c_void_p()
        assert self.L.reef_module_get_kernel(self.mod, name.encode(), C.byref(k)) == capi.SUCC, capi.last_error()
        return k

    def buf(self, host=None, n=None):
        nbytes = host.nbytes if host is not None else n * 4
        p = C.c_uint64()
        assert self.L.reef_malloc(C.byref(p), C.c_size_t(nbytes)) == capi.SUCC
        if host is not None:
            h = np.ascontiguousarray(host)
            assert self.L.reef_memcpy_h2d(p, h.ctypes.data_as(C.c_void_p), C.c_size_t(nbytes)) == capi.SUCC
        else:
            assert self.L.reef_memset(p, C.c_int(0), C.c_size_t(nbytes)) == capi.SUCC
        self.bufs.append(p)
        return p

    def read(self, p, n):
        out = np.empty(n, np.float32)
        assert self.L.reef_memcpy_d2h(out.ctypes.data_as(C.c_void_p), p, C.c_size_t(n * 4)) == capi.SUCC
        return out

    def close(self):
        for p in self.bufs:
            self.L.reef_free(p)
        self.L.reef_stream_destroy(self.stream)
        self.L.reef_module_close(self.mod)


def _args(ptrs):
    """void** of pointers to 8-byte device pointers, as GPUModuleLaunchKernel took them."""
    arr = (C.c_void_p * len(ptrs))(*[C.cast(C.pointer(p), C.c_void_p) for p in ptrs])
    return arr


def test_dispatch_static_matches_dispatch_on_two_calls_in_a_row():
    d = _Dev()
    L = d.L
    rng = np.random.default_rng(42)
    # real-time kernel: conv 32->72, 3x3/2 on 15x15 (+bias, ReLU); best-effort kernel: bias+ReLU on 3136x64
    x = d.buf(rng.normal(size=15 * 15 * 32).astype(np.float32))
    w = d.buf(rng.normal(size=72 * 9 * 32).astype(np.float32))
    b = d.buf(rng.normal(size=72).astype(np.float32))
    be_in = d.buf(rng.normal(size=3136 * 64).astype(np.float32))
    be_bias = d.buf(rng.normal(size=64).astype(np.float32))
    rt_k, be_k = d.kernel(RT_NAME), d.kernel(BE_NAME)
    n_rt_out, n_be_out = 8 * 8 * 72, 3136 * 64
    be_blocks = 49

    def run(static, lane=3):
        rt_out, be_out = d.buf(n=n_rt_out), d.buf(n=n_be_out)
        slot = d.buf(n=1)
        rt_args, be_args = _args([x, w, rt_out, b]), _args([be_out, be_in, be_bias])
        if static:
            rc = L.reef_dispatch_static(rt_k, rt_args, be_k, be_args, C.c_int(0), C.c_int(be_blocks), C.c_int(64),
                                        C.c_int(2), slot, C.c_int(lane), d.stream)
        else:
            ctrl = d.buf(n=4)
            rc = L.reef_dispatch(rt_k, rt_args, be_k, be_args, C.c_int(0), C.c_int(be_blocks), C.c_int(64), C.c_int(2),
                                 slot, ctrl, C.c_uint64(0), d.stream, None)
        assert rc == capi.SUCC, capi.last_error()
        assert L.reef_stream_sync(d.stream) == capi.SUCC, capi.last_error()
        done = d.read(slot, 1).view(np.int32)[0]
        return d.read(rt_out, n_rt_out), d.read(be_out, n_be_out), int(done)

    want_rt, want_be, want_done = run(static=False)
    assert want_done == be_blocks and np.abs(want_rt).max() > 0 and np.abs(want_be).max() > 0
    for call in range(2):                       # two calls in a row, same lane: the lane is re-cleared each time
        got_rt, got_be, done = run(static=True)
        assert done == be_blocks, f"call {call}: completion counter {done}"
        assert np.array_equal(got_rt, want_rt), f"call {call}: real-time output differs from reef_dispatch"
        assert np.array_equal(got_be, want_be), f"call {call}: best-effort output differs from reef_dispatch"

    # a lane beyond the static maximum is refused with a clear error, nothing is launched
    slot = d.buf(n=1)
    rc = L.reef_dispatch_static(rt_k, _args([x, w, d.buf(n=n_rt_out), b]), None, None, C.c_int(0), C.c_int(0),
                                C.c_int(148), C.c_int(1), slot, C.c_int(64), d.stream)
    assert rc == capi.OUT_OF_RANGE and "64" in capi.last_error()
    d.close()
