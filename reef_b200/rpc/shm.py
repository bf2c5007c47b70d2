"""POSIX shared-memory blobs, the data plane of REEF's request API.

Tensors never travel inside an RPC: the server creates one shared-memory object per (model, tensor), keyed
``"<mid>_<name>"``, and client and server map it (reference: src/reef/util/shared_memory.cpp:13-26,
src/reef/server/server.cpp:95-121).  ``shm_open(key)`` of the reference and this class open the same object:
on Linux a POSIX shared-memory object named ``key`` is the file ``/dev/shm/key``.
"""
from __future__ import annotations

import mmap
import os

import numpy as np

_ROOT = "/dev/shm"


class SharedMemory:
    def __init__(self, key: str, size: int, create: bool = False):
        if not key or "/" in key.strip("/"):
            raise ValueError(f"bad shared-memory key {key!r}")
        self.key, self.size, self.create = key, int(size), create
        path = os.path.join(_ROOT, key.strip("/"))
        flags = os.O_RDWR | (os.O_CREAT if create else 0)
        self._fd = os.open(path, flags, 0o777)
        try:
            os.ftruncate(self._fd, self.size)       # the reference sizes the object on both sides too (:22)
            self._map = mmap.mmap(self._fd, self.size, mmap.MAP_SHARED, mmap.PROT_READ | mmap.PROT_WRITE)
        except Exception:
            os.close(self._fd)
            raise
        self._path = path

    def data(self) -> memoryview:
        return memoryview(self._map)

    def array(self, dtype=np.float32) -> np.ndarray:
        """The blob as a numpy array that aliases the mapping (no copy)."""
        return np.frombuffer(self._map, dtype=dtype)

    def close(self):
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:
                pass                  # a numpy view is still alive: the mapping goes with it
            self._map = None
            os.close(self._fd)
            if self.create:
                try:
                    os.unlink(self._path)       # the creator unlinks (reference :29-33)
                except FileNotFoundError:
                    pass

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
