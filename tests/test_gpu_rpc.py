"""Request API on a B200: the reference's client calls against the real scheduler, checked with the oracle."""
import os

import numpy as np
import pytest

from conftest import rel_err
from oracle import oracle

pytestmark = pytest.mark.gpu


def test_rpc_real_time_and_best_effort_clients(gen):
    from reef_b200.rpc import REEFClient, REEFServer
    server = REEFServer("127.0.0.1:0")
    server.run()
    try:
        addr = f"127.0.0.1:{server.port}"
        # mocked_kernel: inputs a = b = c = 3 -> every output 18 (reference: src/reef/test/test.cpp:102-116)
        be = REEFClient(addr)
        be.init(False)
        d = os.path.dirname(gen("mocked_kernel"))
        mk = be.load_model(d, "mocked_kernel")
        for name in ("a", "b", "c"):
            blob = mk._register(name)[0]
            blob.array(np.float32)[:] = 3.0
            assert mk._stub.call("SetBlob", key=f"{mk.get_mid()}_{name}").succ
        mk.infer()
        out = mk.get_output_blob()
        mk.get_output()
        assert np.all(out.array(np.float32) == 18.0)

        # a real-time ResNet client with its input and output in shared memory
        rt = REEFClient(addr)
        rt.init(True)
        base = gen("resnet18_64")
        m = rt.load_model(os.path.dirname(base), "resnet18_64")
        x = np.random.default_rng(3).normal(0, 1, 3 * 64 * 64).astype(np.float32)
        m.get_input_blob().array(np.float32)[:] = x
        m.load_input()
        lat = [m.infer().latency_ms for _ in range(5)]
        m.get_output_blob()
        m.get_output()
        o = oracle.OracleExecutor(base + ".json", base + ".param")
        o.set_input("data", x)
        o.execute()
        err = rel_err(m.get_output_blob().array(np.float32), o.get_output())
        print("rpc resnet18_64 rel err", err, "latencies ms", lat)
        assert err < 1e-2
        rt.close(); be.close()
    finally:
        server.shutdown()
