"""Request API without a GPU: wire format, shared-memory blobs, and the six RPCs against a stand-in scheduler."""
import os

import numpy as np
import pytest

from reef_b200.rpc import REEFClient, REEFServer, SharedMemory, wire


def test_wire_known_encodings():
    # bytes protoc-generated code produces for the same messages (proto3: defaults are not written)
    assert wire.encode(wire.make("LoadModelRequest", dir="a", name="b", qid=3)).hex() == "0a01611201621803"
    assert wire.encode(wire.make("SetPriorityRequest", rt=True)).hex() == "0801"
    assert wire.encode(wire.make("SetPriorityRequest", rt=False)) == b""
    assert wire.encode(wire.make("RegisterBlobReply", succ=True, key="7_data", size=602112)).hex() == \
        "08011206375f646174611880e024"
    assert wire.encode(wire.make("InferReply", succ=True, tid=300)).hex() == "080110ac02"
    # negative int32: ten-byte sign-extended varint
    assert wire.encode(wire.make("InferReply", tid=-1)).hex() == "10ffffffffffffffffff01"


def test_wire_round_trip_and_unknown_fields():
    for kind, fields in [("LoadModelRequest", dict(dir="/m/resnet", name="resnet152", qid=5)),
                         ("RegisterBlobReply", dict(succ=True, key="12_output", size=1 << 40)),
                         ("InferRequest", dict(mid=7, **{"async": True})), ("InferReply", dict(tid=-3))]:
        m = wire.decode(kind, wire.encode(wire.make(kind, **fields)))
        for k, v in fields.items():
            assert getattr(m, k) == v
    m = wire.decode("GetBlobReply", bytes.fromhex("0801") + bytes.fromhex("7a03616263") + bytes.fromhex("a00105"))
    assert m.succ is True                      # fields 15 (string) and 20 (varint) are skipped
    assert wire.decode("LoadModelReply", b"").succ is False and wire.decode("LoadModelReply", b"").mid == 0
    with pytest.raises(ValueError):
        wire.decode("GetBlobRequest", bytes.fromhex("0a05616263"))     # truncated string
    with pytest.raises(KeyError):
        wire.make("InferRequest", nope=1)


def test_shared_memory_blob_is_the_posix_object():
    key = f"reef_test_{os.getpid()}"
    a = SharedMemory(key, 4096, create=True)
    assert os.path.exists("/dev/shm/" + key)   # what shm_open(key) of a C++ client would map
    b = SharedMemory(key, 4096)
    a.array(np.float32)[:4] = [1, 2, 3, 4]
    assert b.array(np.float32)[:4].tolist() == [1, 2, 3, 4]
    del b
    a.close()
    assert not os.path.exists("/dev/shm/" + key)


class FakeScheduler:
    """Stands in for REEFScheduler: one "model" that adds 1 to its input."""
    def __init__(self):
        self.queues, self.models, self.data, self.tasks, self.running = [], [], {}, 0, False

    def run(self): self.running = True
    def shutdown(self): self.running = False
    def create_queue(self, qtype):
        self.queues.append(qtype)
        return len(self.queues) - 1
    def load_model(self, d, name):
        if name == "missing":
            raise RuntimeError("no such model")
        self.models.append((d, name))
        mid = len(self.models) - 1
        self.data[mid] = {"data": np.zeros(64, np.float32), "output": np.zeros(64, np.float32)}
        return mid
    def bind_model_queue(self, qid, mid):
        if qid >= len(self.queues):
            raise RuntimeError("no such queue")
    def get_data_size(self, mid, name): return self.data[mid][name].nbytes
    def set_input(self, mid, arr, name): self.data[mid][name][:] = np.frombuffer(arr, np.float32)
    def get_output_into(self, mid, out, name): out[:] = self.data[mid][name].view(np.uint8)
    def new_task(self, mid):
        if mid not in self.data:
            raise RuntimeError("bad model")
        self.data[mid]["output"][:] = self.data[mid]["data"] + 1
        self.tasks += 1
        return self.tasks
    def wait_task(self, tid): pass


def test_six_rpcs_end_to_end_over_grpc():
    sched = FakeScheduler()
    server = REEFServer("127.0.0.1:0", scheduler=sched)
    server.run()
    try:
        assert sched.running
        addr = f"127.0.0.1:{server.port}"
        rt, be = REEFClient(addr), REEFClient(addr)
        assert rt.init(True) and be.init(False)
        assert sched.queues == [0, 1] and rt.qid == 0 and be.qid == 1      # RealTimeQueue = 0, BestEffortQueue = 1
        m = rt.load_model("/models/x", "x")
        assert sched.models == [("/models/x", "x")] and m.get_mid() == 0
        with pytest.raises(RuntimeError):
            be.load_model("/models", "missing")
        inp = m.get_input_blob()
        assert inp.key == "0_data" and inp.size == 256
        inp.array(np.float32)[:] = np.arange(64)
        m.load_input()
        t = m.infer()
        assert t.tid == 1 and t.finish >= t.submit
        out = m.get_output_blob()
        m.get_output()
        assert np.array_equal(out.array(np.float32), np.arange(64, dtype=np.float32) + 1)
        # unknown blob key, unknown model: succ = false with gRPC status OK (the client raises)
        from reef_b200.rpc.client import _Stub
        import grpc
        stub = _Stub(grpc.insecure_channel(addr))
        assert stub.call("GetBlob", key="nope").succ is False
        assert stub.call("Infer", mid=99).succ is False
        assert stub.call("RegisterBlob", mid=99, name="data").succ is False
        rt.close(); be.close()
    finally:
        server.shutdown()
    assert not sched.running and not os.path.exists("/dev/shm/0_data")
