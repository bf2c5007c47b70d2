"""REEF's request API: gRPC service ``reef.rpc.REEFService`` + shared-memory blobs (server and client).

``python -m reef_b200.rpc.server`` / ``python -m reef_b200.rpc.client`` are the reference's ``reef_server`` /
``reef_client`` / ``reef_client_cont`` executables (src/example/*.cpp).
"""
_EXPORTS = {"ModelHandle": "client", "REEFClient": "client", "TaskHandle": "client", "DEFAULT_REEF_ADDR": "server",
            "REEFServer": "server", "SharedMemory": "shm"}

__all__ = sorted(_EXPORTS)


def __getattr__(name):      # submodules load on first use, so that `python -m reef_b200.rpc.server` runs it once
    if name in _EXPORTS:
        import importlib
        return getattr(importlib.import_module(f"{__name__}.{_EXPORTS[name]}"), name)
    raise AttributeError(name)
