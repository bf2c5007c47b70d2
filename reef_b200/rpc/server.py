"""REEF's request API served over gRPC: the six RPCs of ``reef.rpc.REEFService`` in front of the scheduler.

Mirrors ``REEFServer`` of the reference (src/reef/server/server.cpp:8-199): the same service and method names,
the same messages on the wire (``wire.py``), tensors through POSIX shared memory keyed ``"<mid>_<name>"``
(``shm.py``).  The handlers do what the reference's do, line for line in behaviour:

  SetPriority   create_queue(RealTime | BestEffort)                              (server.cpp:34-54)
  LoadModel     load <dir>/<name>.json/.profile.json[/.param], bind to the queue  (server.cpp:56-93)
  RegisterBlob  size of the named tensor, create the blob once                   (server.cpp:95-121)
  SetBlob       blob -> device (set_input)                                       (server.cpp:148-170)
  GetBlob       device -> blob (get_output)                                      (server.cpp:123-146)
  Infer         new_task + wait_task                                             (server.cpp:172-195)

Every failure is reported as ``succ = false`` in the reply with gRPC status OK, as the reference does.
The service is registered with grpcio's generic handlers, so no generated code is involved.
"""
from __future__ import annotations

import argparse
import os
import threading
from concurrent import futures

import grpc

from . import wire
from .shm import SharedMemory

DEFAULT_REEF_ADDR = "localhost:34543"      # reference: src/reef/util/common.h:8


class REEFServer:
    def __init__(self, addr: str = DEFAULT_REEF_ADDR, scheduler=None, mode: int | None = None, device: int = 0,
                 max_workers: int = 16):
        """``scheduler``: an object with the REEFScheduler methods (default: the CUDA one; it needs a GPU)."""
        if scheduler is None:
            from .. import capi
            scheduler = capi.REEFScheduler(capi.REEFScheduler.REEF if mode is None else mode, device)
        self.scheduler = scheduler
        self.addr = addr
        self.port = None
        self._shms = {}                      # key -> (mid, tensor name, SharedMemory)
        self._shm_mtx = threading.Lock()
        self._server = grpc.server(futures.ThreadPoolExecutor(max_workers=max_workers))
        handlers = {}
        for method, (req_kind, _) in wire.METHODS.items():
            fn = getattr(self, method)
            handlers[method] = grpc.unary_unary_rpc_method_handler(
                (lambda f: (lambda request, context: f(request)))(fn),
                request_deserializer=(lambda k: (lambda b: wire.decode(k, b)))(req_kind),
                response_serializer=wire.encode)
        self._server.add_generic_rpc_handlers((grpc.method_handlers_generic_handler(wire.SERVICE, handlers),))

    # ---- life cycle (reference: server.cpp:14-32) -------------------------------------------------
    def run(self):
        self.port = self._server.add_insecure_port(self.addr)
        if self.port == 0:
            raise RuntimeError(f"cannot listen on {self.addr}")
        self._server.start()
        self.scheduler.run()

    def wait(self):
        self._server.wait_for_termination()

    def shutdown(self):
        self._server.stop(grace=None).wait()
        self.scheduler.shutdown()
        with self._shm_mtx:
            for _, _, shm in self._shms.values():
                shm.close()
            self._shms.clear()

    # ---- the six RPCs ----------------------------------------------------------------------------------
    def SetPriority(self, req):
        from ..capi import REEFScheduler as S
        try:
            qid = self.scheduler.create_queue(S.RealTimeQueue if req.rt else S.BestEffortQueue)
        except Exception:
            return wire.make("SetPriorityReply", succ=False)
        return wire.make("SetPriorityReply", succ=True, qid=qid)

    def LoadModel(self, req):
        try:
            mid = self.scheduler.load_model(req.dir, req.name)
        except Exception:
            return wire.make("LoadModelReply", succ=False)
        try:
            self.scheduler.bind_model_queue(req.qid, mid)
        except Exception:
            return wire.make("LoadModelReply", succ=False, mid=mid)
        return wire.make("LoadModelReply", succ=True, mid=mid)

    def RegisterBlob(self, req):
        try:
            size = self.scheduler.get_data_size(req.mid, req.name)
        except Exception:
            return wire.make("RegisterBlobReply", succ=False)
        key = f"{req.mid}_{req.name}"
        with self._shm_mtx:
            if key not in self._shms:
                self._shms[key] = (req.mid, req.name, SharedMemory(key, size, create=True))
        return wire.make("RegisterBlobReply", succ=True, key=key, size=size)

    def _blob(self, key):
        with self._shm_mtx:
            return self._shms.get(key)

    def GetBlob(self, req):
        info = self._blob(req.key)
        if info is None:
            return wire.make("GetBlobReply", succ=False)
        mid, name, shm = info
        try:
            self.scheduler.get_output_into(mid, shm.array("u1"), name)
        except Exception:
            return wire.make("GetBlobReply", succ=False)
        return wire.make("GetBlobReply", succ=True)

    def SetBlob(self, req):
        info = self._blob(req.key)
        if info is None:
            return wire.make("SetBlobReply", succ=False)
        mid, name, shm = info
        try:
            self.scheduler.set_input(mid, shm.array("u1"), name)
        except Exception:
            return wire.make("SetBlobReply", succ=False)
        return wire.make("SetBlobReply", succ=True)

    def Infer(self, req):
        try:
            tid = self.scheduler.new_task(req.mid)
        except Exception:
            return wire.make("InferReply", succ=False)
        try:
            self.scheduler.wait_task(tid)
        except Exception:
            return wire.make("InferReply", succ=False, tid=tid)
        return wire.make("InferReply", succ=True, tid=tid)


def main(argv=None):
    """The reference's ``reef_server`` executable (src/example/rpc_server.cpp): serve until killed."""
    ap = argparse.ArgumentParser(description="REEF server on a B200 (gRPC request API + shared-memory blobs)")
    ap.add_argument("--addr", default=DEFAULT_REEF_ADDR)
    ap.add_argument("--device", type=int, default=int(os.environ.get("LOCAL_RANK", "0")))
    ap.add_argument("--mode", type=int, default=3, help="0 NoPreempt, 1 MultiStream, 2 WaitPreempt, 3 REEF, 4 Reset")
    args = ap.parse_args(argv)
    server = REEFServer(args.addr, mode=args.mode, device=args.device)
    server.run()
    print(f"reef server listening on {args.addr} (port {server.port}), device {args.device}", flush=True)
    try:
        server.wait()
    except KeyboardInterrupt:
        server.shutdown()


if __name__ == "__main__":
    main()
