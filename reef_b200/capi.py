"""ctypes bindings over ``libreef_cuda.so`` (include/reef_cuda.h) and ``libreef_host.so``
(include/reef_host.h).  Class and method names follow the reference's C++ classes
(reference: src/reef/executor/executor_base.h, hybrid_executor.h, src/reef/server/scheduler.h:68-126)
so tests read like the reference's own (reference: src/reef/test/test.cpp)."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

SUCC, FAIL, NOT_FOUND, OUT_OF_RANGE, FULL, TIMEOUT = range(6)
STATUS_NAMES = ["Succ", "Fail", "NotFound", "OutOfRange", "Full", "Timeout"]

_cuda = None
_host = None


class ReefError(RuntimeError):
    def __init__(self, status: int, what: str, detail: str = ""):
        self.status = status
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__(f"{what}: Status::{name}" + (f" ({detail})" if detail else ""))


class KernelAttrs(C.Structure):
    _fields_ = [("num_blocks", C.c_int), ("threads", C.c_int), ("regs_per_thread", C.c_int),
                ("static_smem", C.c_int), ("dyn_smem", C.c_int), ("local_mem", C.c_int),
                ("max_blocks_per_sm", C.c_int), ("flops", C.c_double), ("bytes", C.c_double),
                ("tensor_core", C.c_int), ("cluster", C.c_int), ("chainable", C.c_int)]


class TaskInfo(C.Structure):
    _fields_ = [("state", C.c_int), ("preempted", C.c_int), ("padded", C.c_int), ("padded_to_complete", C.c_int),
                ("submit_ns", C.c_int64), ("start_ns", C.c_int64), ("end_ns", C.c_int64), ("failed", C.c_int)]


class SchedStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("preempt_count", "preempt_ns_sum", "preempt_ns_max", "rt_tasks", "be_tasks",
                                          "be_tasks_padded_to_finish", "padded_kernels", "padded_blocks",
                                          "drain_count", "drain_ns_sum", "drain_ns_max",
                                          "dev_count", "dev_ns_sum", "dev_ns_max", "drain_ns_p50", "drain_ns_p99")]


class Client(C.Structure):
    _fields_ = [("mid", C.c_uint32), ("max_requests", C.c_uint32), ("warmup_requests", C.c_uint32),
                ("input", C.c_void_p), ("input_len", C.c_size_t), ("input_name", C.c_char_p),
                ("output", C.c_void_p), ("output_len", C.c_size_t), ("latencies_ms", C.POINTER(C.c_float)),
                ("completed", C.c_uint64), ("elapsed_s", C.c_double), ("think_us", C.c_uint32), ("failed", C.c_uint32)]


def cuda_lib():
    """The C-ABI device library.  Loads without a GPU (for reef_kernel_plan); compute calls need one."""
    global _cuda
    if _cuda is None:
        path = os.path.join(_build.PKG, "libreef_cuda.so")
        if not os.path.exists(path):
            raise ReefError(NOT_FOUND, "libreef_cuda.so is not built (run reef_b200.build.build_all())")
        _cuda = C.CDLL(path, mode=C.RTLD_GLOBAL)
        _cuda.reef_last_error.restype = C.c_char_p
        _cuda.reef_launch_count.restype = C.c_uint64
    return _cuda


def host_lib():
    global _host
    if _host is None:
        cuda_lib()
        path = os.path.join(_build.PKG, "libreef_host.so")
        if not os.path.exists(path):
            raise ReefError(NOT_FOUND, "libreef_host.so is not built (run reef_b200.build.build_all())")
        _host = C.CDLL(path)
        _host.reef_executor_error.restype = C.c_char_p
        _host.reef_sched_error.restype = C.c_char_p
        _host.reef_sched_avg_preempt_latency.restype = C.c_int64
        _host.reef_sched_avg_kernel_sel_latency.restype = C.c_int64
    return _host


def last_error() -> str:
    return (cuda_lib().reef_last_error() or b"").decode()


def _check(rc: int, what: str, detail: str = ""):
    if rc != SUCC:
        raise ReefError(rc, what, detail or last_error())


def kernel_plan(name: str):
    """(dims[6], dyn_smem, num_args) of a kernel name; raises ReefError(NotFound) for unknown names."""
    dims = (C.c_uint32 * 6)()
    smem = C.c_uint32()
    nargs = C.c_int()
    _check(cuda_lib().reef_kernel_plan(name.encode(), dims, C.byref(smem), C.byref(nargs)), f"reef_kernel_plan({name})")
    return list(dims), int(smem.value), int(nargs.value)


def kernel_cost(name: str):
    """(flops, bytes, tensor_core) of one launch of a kernel name; needs no GPU."""
    fl, by, tc = C.c_double(), C.c_double(), C.c_int()
    _check(cuda_lib().reef_kernel_cost(name.encode(), C.byref(fl), C.byref(by), C.byref(tc)), f"reef_kernel_cost({name})")
    return fl.value, by.value, tc.value


def plan_fn(name: str):
    d, s, _ = kernel_plan(name)
    return d, s


def device_count() -> int:
    n = C.c_int()
    _check(cuda_lib().reef_device_count(C.byref(n)), "reef_device_count")
    return n.value


def probe_stream_latency(iters: int = 2000, device: int = 0):
    """(write call, write + completion as the host sees it, completion-only event round trip, timed event round trip)
    in microseconds, medians."""
    lib = cuda_lib()
    _check(lib.reef_gpu_init(C.c_int(device)), "reef_gpu_init")
    a, b, c, d = C.c_double(), C.c_double(), C.c_double(), C.c_double()
    _check(lib.reef_probe_stream_latency(C.c_int(iters), C.byref(a), C.byref(b), C.byref(c), C.byref(d)), "reef_probe_stream_latency")
    return a.value, b.value, c.value, d.value


def device_error() -> int:
    """Reads and clears the device error word (non-zero: a bounded device-side wait expired)."""
    v = C.c_int()
    _check(cuda_lib().reef_device_error(C.byref(v)), "reef_device_error")
    return v.value


def device_error_set(value: int):
    """Stores a value into the device error word from the host (failure injection without any device wait)."""
    _check(cuda_lib().reef_device_error_set(C.c_int(value)), "reef_device_error_set")


def launch_count() -> int:
    return int(cuda_lib().reef_launch_count())


def _buf(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class HybridExecutor:
    """reference: src/reef/executor/hybrid_executor.h (with ExecutorBase's set_input/execute/get_output)."""

    def __init__(self, device: int = 0):
        self._h = C.c_void_p()
        self._lib = host_lib()
        _check(self._lib.reef_executor_create(C.c_int(device), C.byref(self._h)), "reef_executor_create")

    def close(self):
        if self._h:
            self._lib.reef_executor_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _err(self):
        return (self._lib.reef_executor_error(self._h) or b"").decode()

    def load_model_from_file(self, json_path: str, profile_path: str | None = None):
        rc = self._lib.reef_executor_load(self._h, json_path.encode(), (profile_path or "").encode())
        _check(rc, "load_hybrid_model_from_file", self._err())

    def load_param_from_file(self, param_path: str):
        _check(self._lib.reef_executor_load_param(self._h, param_path.encode()), "load_param_from_file", self._err())

    def num_kernels(self) -> int:
        n = C.c_size_t()
        self._lib.reef_executor_num_kernels(self._h, C.byref(n))
        return n.value

    def get_data_size(self, name: str) -> int:
        n = C.c_size_t()
        _check(self._lib.reef_executor_get_data_size(self._h, name.encode(), C.byref(n)), f"get_data_size({name})")
        return n.value

    def set_input(self, name: str, value: np.ndarray):
        v = np.ascontiguousarray(value)
        _check(self._lib.reef_executor_set_input(self._h, name.encode(), _buf(v), C.c_size_t(v.nbytes)),
               f"set_input({name})")

    def get_output(self, dtype=np.float32) -> np.ndarray:
        n = self.get_data_size("output")
        out = np.empty(n // np.dtype(dtype).itemsize, dtype=dtype)
        _check(self._lib.reef_executor_get_output(self._h, _buf(out), C.c_size_t(out.nbytes)), "get_output")
        return out

    def get_data(self, idx: int, nbytes: int, dtype=np.float32) -> np.ndarray:
        out = np.empty(nbytes // np.dtype(dtype).itemsize, dtype=dtype)
        _check(self._lib.reef_executor_get_data(self._h, C.c_int(idx), _buf(out), C.c_size_t(out.nbytes)),
               f"get_data({idx})")
        return out

    def execute(self):
        _check(self._lib.reef_executor_execute(self._h), "execute", self._err())

    def execute_to(self, idx: int):
        _check(self._lib.reef_executor_execute_to(self._h, C.c_int(idx)), "execute_to", self._err())

    def execute_kernel(self, idx: int):
        _check(self._lib.reef_executor_execute_kernel(self._h, C.c_int(idx)), "execute_kernel", self._err())

    def execute_preemptable(self):
        _check(self._lib.reef_executor_execute_preemptable(self._h), "execute_preemptale", self._err())

    def execute_graph(self):
        _check(self._lib.reef_executor_execute_graph(self._h), "execute_graph", self._err())

    def execute_dispatch(self):
        _check(self._lib.reef_executor_execute_dispatch(self._h), "execute_dispatch", self._err())

    def build_chains(self, clusters: int = 0) -> int:
        """Runs of consecutive tensor-core layers become persistent kernels; returns the number of runs."""
        n = C.c_size_t()
        _check(self._lib.reef_executor_build_chains(self._h, C.c_int(clusters), C.byref(n)), "build_chains", self._err())
        return int(n.value)

    def chain_info(self, idx: int = 0):
        """(first kernel, end kernel, clusters of the grid, most clusters the GPU holds at once) of chain ``idx``."""
        b, e, c, m = C.c_int(), C.c_int(), C.c_int(), C.c_int()
        _check(self._lib.reef_executor_chain_info(self._h, C.c_size_t(idx), C.byref(b), C.byref(e), C.byref(c), C.byref(m)),
               "chain_info", self._err())
        return b.value, e.value, c.value, m.value

    def execute_preempt_resume_chained(self, delay_us: int, clusters: int = 0):
        restarts, first = C.c_int(), C.c_int()
        _check(self._lib.reef_executor_execute_preempt_resume_chained(self._h, C.c_int(delay_us), C.c_int(clusters),
                                                                      C.byref(restarts), C.byref(first)),
               "execute_preempt_resume_chained", self._err())
        return restarts.value, first.value

    def execute_preemptable_chained(self, clusters: int = 0):
        _check(self._lib.reef_executor_execute_preemptable_chained(self._h, C.c_int(clusters)), "execute_preemptable_chained", self._err())

    def set_stream_priority(self, high: bool):
        _check(self._lib.reef_executor_set_stream_priority(self._h, C.c_int(int(high))), "set_stream_priority", self._err())

    def execute_chained(self):
        _check(self._lib.reef_executor_execute_chained(self._h), "execute_chained", self._err())

    def execute_preempt_resume(self, delay_us: int, with_count: bool = False):
        """Best-effort run, flag raised ``delay_us`` after the first launch, resumed until done.  Returns (restarts,
        first incomplete kernel) and, with ``with_count``, that kernel's completion counter when it was found short."""
        restarts, first, count = C.c_int(), C.c_int(), C.c_int()
        _check(self._lib.reef_executor_execute_preempt_resume(self._h, C.c_int(delay_us), C.byref(restarts),
                                                              C.byref(first), C.byref(count)), "execute_preempt_resume",
               self._err())
        return (restarts.value, first.value, count.value) if with_count else (restarts.value, first.value)

    def task_slots(self):
        n = self.num_kernels()
        slots = (C.c_int * n)()
        blocks = (C.c_int * n)()
        _check(self._lib.reef_executor_task_slots(self._h, slots, blocks, C.c_size_t(n)), "task_slots")
        return list(slots), list(blocks)

    def time(self, mode: int, warmup: int, iters: int) -> float:
        ms = C.c_float()
        _check(self._lib.reef_executor_time(self._h, C.c_int(mode), C.c_int(warmup), C.c_int(iters), C.byref(ms)),
               "reef_executor_time", self._err())
        return ms.value

    def time_tensor_core(self, warmup: int = 3, iters: int = 20):
        """(ms per replay, launches) of a graph with only the tensor-core kernels of the schedule."""
        ms = C.c_float()
        n = C.c_int()
        _check(self._lib.reef_executor_time_tensor_core(self._h, C.c_int(warmup), C.c_int(iters), C.byref(ms), C.byref(n)),
               "time_tensor_core", self._err())
        return float(ms.value), int(n.value)

    def time_kernel(self, idx: int, reps: int = 20, warmup: int = 3, iters: int = 20) -> float:
        """Microseconds per launch of kernel ``idx`` alone (a CUDA graph of ``reps`` launches, CUDA events)."""
        us = C.c_float()
        _check(self._lib.reef_executor_time_kernel(self._h, C.c_int(idx), C.c_int(reps), C.c_int(warmup), C.c_int(iters),
                                                   C.byref(us)), "time_kernel", self._err())
        return float(us.value)

    def profile_kernels(self, iters: int = 20):
        n = self.num_kernels()
        us = (C.c_float * n)()
        flops = (C.c_double * n)()
        nbytes = (C.c_double * n)()
        tc = (C.c_int * n)()
        blocks = (C.c_int * n)()
        occ = (C.c_int * n)()
        _check(self._lib.reef_executor_profile_kernels(self._h, C.c_int(iters), us, flops, nbytes, tc, blocks, occ,
                                                       C.c_size_t(n)), "profile_kernels", self._err())
        return [dict(us=us[i], flops=flops[i], bytes=nbytes[i], tensor_core=tc[i], blocks=blocks[i],
                     max_blocks_per_sm=occ[i]) for i in range(n)]

    def write_profile(self, out_path: str, iters: int = 20):
        _check(self._lib.reef_executor_write_profile(self._h, C.c_int(iters), out_path.encode()), "write_profile",
               self._err())

    def profile_wave(self, idx: int, occupancy: int, iters: int = 10) -> float:
        us = C.c_float()
        _check(self._lib.reef_executor_profile_wave(self._h, C.c_int(idx), C.c_int(occupancy), C.c_int(iters),
                                                    C.byref(us)), "profile_wave", self._err())
        return us.value


class REEFScheduler:
    """reference: src/reef/server/scheduler.h:68-126."""
    NoPreempt, MultiStream, WaitPreempt, REEF, Reset = range(5)
    RealTimeQueue, BestEffortQueue = 0, 1
    Init, Waiting, Executing, Finish = range(4)

    def __init__(self, mode: int = 3, device: int = 0):
        self._h = C.c_void_p()
        self._lib = host_lib()
        _check(self._lib.reef_sched_create(C.c_int(mode), C.c_int(device), C.byref(self._h)), "REEFScheduler")

    def close(self):
        if self._h:
            self._lib.reef_sched_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _err(self):
        return (self._lib.reef_sched_error(self._h) or b"").decode()

    def load_model(self, model_dir: str, model_name: str) -> int:
        mid = C.c_uint32()
        _check(self._lib.reef_sched_load_model(self._h, model_dir.encode(), model_name.encode(), C.byref(mid)),
               "load_model", self._err())
        return mid.value

    def load_model_files(self, json_path: str, profile_path: str = "", param_path: str = "") -> int:
        mid = C.c_uint32()
        _check(self._lib.reef_sched_load_model_files(self._h, json_path.encode(), profile_path.encode(),
                                                     param_path.encode(), C.byref(mid)), "load_model", self._err())
        return mid.value

    def create_queue(self, qtype: int) -> int:
        qid = C.c_uint32()
        _check(self._lib.reef_sched_create_queue(self._h, C.c_int(qtype), C.byref(qid)), "create_queue")
        return qid.value

    def bind_model_queue(self, qid: int, mid: int):
        _check(self._lib.reef_sched_bind_model_queue(self._h, C.c_uint32(qid), C.c_uint32(mid)), "bind_model_queue")

    def get_data_size(self, mid: int, name: str) -> int:
        n = C.c_size_t()
        _check(self._lib.reef_sched_get_data_size(self._h, C.c_uint32(mid), name.encode(), C.byref(n)), "get_data_size")
        return n.value

    def set_input(self, mid: int, data: np.ndarray, name: str = "data"):
        v = np.ascontiguousarray(data)
        _check(self._lib.reef_sched_set_input(self._h, C.c_uint32(mid), _buf(v), C.c_size_t(v.nbytes), name.encode()),
               "set_input")

    def get_output(self, mid: int, name: str = "output", dtype=np.float32) -> np.ndarray:
        n = self.get_data_size(mid, name)
        out = np.empty(n // np.dtype(dtype).itemsize, dtype=dtype)
        _check(self._lib.reef_sched_get_output(self._h, C.c_uint32(mid), _buf(out), C.c_size_t(out.nbytes),
                                               name.encode()), "get_output")
        return out

    def get_output_into(self, mid: int, out: np.ndarray, name: str = "output"):
        """Copy the named tensor into ``out`` (a contiguous array of exactly the tensor's size in bytes)."""
        _check(self._lib.reef_sched_get_output(self._h, C.c_uint32(mid), _buf(out), C.c_size_t(out.nbytes),
                                               name.encode()), "get_output")

    def new_task(self, mid: int) -> int:
        tid = C.c_uint32()
        _check(self._lib.reef_sched_new_task(self._h, C.c_uint32(mid), C.byref(tid)), "new_task")
        return tid.value

    def wait_task(self, tid: int):
        _check(self._lib.reef_sched_wait_task(self._h, C.c_uint32(tid)), "wait_task")

    def inject_launch_failures(self, mid: int, n: int):
        """Host-side failure injection: the next ``n`` kernel launches of model ``mid`` return an error."""
        _check(self._lib.reef_sched_inject_launch_failures(self._h, C.c_uint32(mid), C.c_int(n)), "inject_launch_failures")

    def get_task(self, tid: int) -> TaskInfo:
        info = TaskInfo()
        _check(self._lib.reef_sched_task_info(self._h, C.c_uint32(tid), C.byref(info)), "get_task")
        return info

    def set_wait_sync(self, v: bool):
        self._lib.reef_sched_set_wait_sync(self._h, C.c_int(int(v)))

    def use_mapped_flag(self):
        _check(self._lib.reef_sched_use_mapped_flag(self._h), "use_mapped_flag", self._err())

    def set_sm_partition(self, be_sms: int, flags: int = 0):
        """Best-effort streams get ``be_sms`` SMs of their own, the real-time stream the rest (before any queue is
        created).  Returns (real-time SMs, best-effort SMs) as provisioned by the driver."""
        a, b = C.c_int(), C.c_int()
        _check(self._lib.reef_sched_set_sm_partition(self._h, C.c_int(be_sms), C.c_int(flags), C.byref(a), C.byref(b)),
               "set_sm_partition", self._err())
        return a.value, b.value

    def set_device_stamps(self, on: bool):
        _check(self._lib.reef_sched_set_device_stamps(self._h, C.c_int(int(on))), "set_device_stamps", self._err())

    def set_pad_slowdown_target(self, v: float):
        self._lib.reef_sched_set_pad_slowdown_target(self._h, C.c_double(v))

    def set_cpu_slice(self, first_cpu: int, n_cpus: int):
        self._lib.reef_sched_set_cpu_slice(self._h, C.c_int(first_cpu), C.c_int(n_cpus))

    def set_be_stream_cap(self, v: int):
        self._lib.reef_sched_set_be_stream_cap(self._h, C.c_int(v))

    def set_rt_chains(self, clusters: int):
        self._lib.reef_sched_set_rt_chains(self._h, C.c_int(clusters))

    def set_rt_graph(self, v: bool):
        self._lib.reef_sched_set_rt_graph(self._h, C.c_int(int(v)))

    def run(self):
        _check(self._lib.reef_sched_run(self._h), "run", self._err())

    def shutdown(self):
        _check(self._lib.reef_sched_shutdown(self._h), "shutdown")

    def avg_preempt_latency(self) -> int:
        return int(self._lib.reef_sched_avg_preempt_latency(self._h))

    def avg_kernel_sel_latency(self) -> int:
        return int(self._lib.reef_sched_avg_kernel_sel_latency(self._h))

    def stats(self) -> dict:
        st = SchedStats()
        self._lib.reef_sched_stats(self._h, C.byref(st))
        return {n: int(getattr(st, n)) for n, _ in SchedStats._fields_}

    def run_clients(self, clients: list, allow_failed: bool = False) -> list:
        """clients: dicts(mid, max_requests, warmup, input (ndarray|None), input_name, want_output, think_us).
        Returns per client dict(latencies_ms ndarray, completed, elapsed_s, output)."""
        arr = (Client * len(clients))()
        keep = []
        for i, c in enumerate(clients):
            arr[i].mid = c["mid"]
            arr[i].max_requests = c.get("max_requests", 0)
            arr[i].warmup_requests = c.get("warmup", 0)
            inp = c.get("input")
            if inp is not None:
                inp = np.ascontiguousarray(inp)
                arr[i].input = inp.ctypes.data
                arr[i].input_len = inp.nbytes
            nm = c.get("input_name", "data").encode()
            arr[i].input_name = nm
            out = None
            if c.get("want_output", True):
                out = np.zeros(self.get_data_size(c["mid"], "output") // 4, dtype=np.float32)
                arr[i].output = out.ctypes.data
                arr[i].output_len = out.nbytes
            lat = np.zeros(max(1, arr[i].max_requests), dtype=np.float32)
            arr[i].latencies_ms = lat.ctypes.data_as(C.POINTER(C.c_float))
            arr[i].think_us = c.get("think_us", 0)
            keep.append((inp, nm, out, lat))
        rc = self._lib.reef_run_clients(self._h, arr, C.c_size_t(len(clients)))
        if rc != SUCC and not allow_failed:
            _check(rc, "reef_run_clients", self._err())
        res = []
        for i, (inp, nm, out, lat) in enumerate(keep):
            n = int(arr[i].completed)
            res.append(dict(latencies_ms=lat[:n] if arr[i].max_requests else lat[:0], completed=n,
                            elapsed_s=float(arr[i].elapsed_s), output=out, failed=bool(arr[i].failed)))
        return res
