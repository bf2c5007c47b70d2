"""Client side of REEF's request API (reference: src/reef/client/client.h:25-93, client.cpp).

``REEFClient(addr).init(real_time)`` obtains a task queue (real-time clients share one, every best-effort client
gets its own), ``load_model(dir, name)`` returns a ``ModelHandle`` whose ``infer()`` submits a request and waits
for it; inputs and outputs go through shared-memory blobs that ``get_input_blob`` / ``get_output_blob`` map and
``load_input`` / ``get_output`` move to and from the device.  A failed call raises ``RuntimeError`` where the
reference aborts on an ASSERT.
"""
from __future__ import annotations

import argparse
import time
from dataclasses import dataclass

import grpc

from . import wire
from .shm import SharedMemory

DEFAULT_REEF_ADDR = "localhost:34543"


@dataclass
class TaskHandle:
    tid: int = -1
    submit: float = 0.0       # seconds (time.time()) at submission and at completion
    finish: float = 0.0

    @property
    def latency_ms(self) -> float:
        return 1e3 * (self.finish - self.submit)


class _Stub:
    def __init__(self, channel):
        self._calls = {}
        for method, (req_kind, rep_kind) in wire.METHODS.items():
            self._calls[method] = channel.unary_unary(
                f"/{wire.SERVICE}/{method}", request_serializer=wire.encode,
                response_deserializer=(lambda k: (lambda b: wire.decode(k, b)))(rep_kind))

    def call(self, method: str, **fields):
        req_kind, _ = wire.METHODS[method]
        return self._calls[method](wire.make(req_kind, **fields))


class ModelHandle:
    def __init__(self, stub: _Stub, mid: int, model_dir: str, name: str):
        self._stub, self.mid, self.dir, self.name = stub, mid, model_dir, name
        self._input = self._output = None
        self._input_key = self._output_key = ""

    def infer(self) -> TaskHandle:
        """Submit an inference task and wait for its completion (client.cpp:67-81)."""
        t = TaskHandle(submit=time.time())
        rep = self._stub.call("Infer", mid=self.mid)
        if not rep.succ:
            raise RuntimeError(f"Infer failed for model {self.mid}")
        t.finish = time.time()
        t.tid = rep.tid
        return t

    def infer_async(self) -> TaskHandle:
        """Declared by the reference and left empty there (client.cpp:83-86); kept for the same surface."""
        return TaskHandle()

    def _register(self, name: str):
        rep = self._stub.call("RegisterBlob", mid=self.mid, name=name)
        if not rep.succ:
            raise RuntimeError(f"RegisterBlob failed for tensor {name!r} of model {self.mid}")
        return SharedMemory(rep.key, rep.size), rep.key

    def get_input_blob(self, name: str = "data") -> SharedMemory:
        if self._input is None:
            self._input, self._input_key = self._register(name)
        return self._input

    def get_output_blob(self, name: str = "output") -> SharedMemory:
        if self._output is None:
            self._output, self._output_key = self._register(name)
        return self._output

    def load_input(self):
        """Move the input blob to the device (SetBlob); returns when it is there."""
        if self._input is None:
            raise RuntimeError("get_input_blob() first")
        if not self._stub.call("SetBlob", key=self._input_key).succ:
            raise RuntimeError("SetBlob failed")

    def get_output(self):
        """Move the model output into the output blob (GetBlob)."""
        if self._output is None:
            raise RuntimeError("get_output_blob() first")
        if not self._stub.call("GetBlob", key=self._output_key).succ:
            raise RuntimeError("GetBlob failed")

    def get_mid(self) -> int:
        return self.mid


class REEFClient:
    def __init__(self, server_addr: str = DEFAULT_REEF_ADDR):
        self._channel = grpc.insecure_channel(server_addr)
        self._stub = _Stub(self._channel)
        self.models = []
        self.qid = None

    def init(self, real_time: bool = False, timeout: float = 10.0) -> bool:
        grpc.channel_ready_future(self._channel).result(timeout=timeout)
        rep = self._stub.call("SetPriority", rt=bool(real_time))
        if not rep.succ:
            raise RuntimeError("SetPriority failed")
        self.qid = rep.qid
        return True

    def load_model(self, model_dir: str, name: str) -> ModelHandle:
        if self.qid is None:
            raise RuntimeError("init() first")
        rep = self._stub.call("LoadModel", dir=model_dir, name=name, qid=self.qid)
        if not rep.succ:
            raise RuntimeError(f"LoadModel failed for {model_dir}/{name}")
        m = ModelHandle(self._stub, rep.mid, model_dir, name)
        self.models.append(m)
        return m

    def close(self):
        self._channel.close()


def main(argv=None):
    """The reference's ``reef_client`` (one request, src/example/rpc_client.cpp) and, with a sleep time,
    ``reef_client_cont`` (requests until killed, src/example/rpc_client_cont.cpp)."""
    ap = argparse.ArgumentParser(description="REEF client: model_dir model_name real_time [sleep_ms]")
    ap.add_argument("model_dir")
    ap.add_argument("model_name")
    ap.add_argument("real_time", type=int)
    ap.add_argument("sleep_ms", type=int, nargs="?", default=None,
                    help="continuous mode: pause between requests (the reference's reef_client_cont)")
    ap.add_argument("--addr", default=DEFAULT_REEF_ADDR)
    ap.add_argument("--count", type=int, default=0, help="continuous mode: stop after this many requests (0: never)")
    args = ap.parse_args(argv)
    client = REEFClient(args.addr)
    client.init(bool(args.real_time))
    print(f"loading '{args.model_name}' from '{args.model_dir}'", flush=True)
    model = client.load_model(args.model_dir, args.model_name)
    if args.sleep_ms is None:
        print("submit inference request")
        print(f"inference latency: {model.infer().latency_ms:.3f} ms")
        return
    print("submit inference requests")
    n = 0
    while args.count == 0 or n < args.count:
        print(f"client {model.get_mid()} inference latency: {model.infer().latency_ms:.3f} ms", flush=True)
        time.sleep(args.sleep_ms / 1e3)
        n += 1


if __name__ == "__main__":
    main()
