#!/usr/bin/env python
"""Benchmark of the REEF executor kernel path on B200.

Workload (BASELINE.json configs[2], the configuration the headline metric is quoted on): one
real-time (RT) client issuing back-to-back ResNet-152 batch-1 requests while 4 best-effort (BE)
clients run ResNet-152 batch-1 closed-loop, all on one GPU through REEFScheduler in REEF mode
(flag preemption + dynamic kernel padding).  Synthetic, seeded weights and inputs.

A "step" is a block of 100 RT requests (so the default 20 steps after 3 warm-up steps are 2000 timed RT
requests after 300 warm-up requests: percentiles over 2000 samples, the padding controller in steady state).
`value` is whole-job inferences/s = RT inf/s + BE inf/s over ONE window (the BE clients start counting when the
RT client has finished its warm-up), inputs resident in HBM; `e2e` is the same measured through the scheduler's
public request calls with pinned HOST buffers (set_input H2D + new_task + wait_task + get_output D2H inside the
timed region).  RT p50/p99, RT-alone p99, BE inf/s, BE-alone inf/s and the preemption latencies ride along in
`rt_be`.

N > 1 (torchrun, one rank per GPU): one scheduler + full weight replica per GPU, requests are
independent, no data-path collective ("scaling": "weak").

`--impl reference` times the CPU arm: the reference's own kernels cannot run here (HIP/gfx906,
TVM-generated), so the arm is the plain-C oracle port of the same schedule graph on all host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

UNIT = "inf/s"
REQS_PER_STEP = 100     # one step = this many back-to-back RT requests
# DRAM traffic of the dominant kernel per launch, from an ncu capture of all 154 tensor-core launches of one
# ResNet-152 pass (dram__bytes_read.sum + dram__bytes_write.sum; summary committed as
# profiles/conv_tc_resnet152_dram.md).  A constant of that capture: it is NOT measured in a bench run.
CONV_TC_TRAFFIC_PER_LAUNCH = {"c2": 2407620, "c1": 2407620}
# BASELINE.json configs; "c2" is the configuration the headline metric is quoted on and the default
WORKLOADS = {
    "c0": dict(metric="resnet18_b1_inferences_per_s_rt_only", rt="resnet18", be=[],
               desc="configs[0]: ResNet-18 b1, single RT client, no contention"),
    "c1": dict(metric="resnet152_b1_inferences_per_s_rt_only", rt="resnet152", be=[],
               desc="configs[1]: ResNet-152 b1, RT-only closed-loop requests"),
    "c2": dict(metric="resnet152_b1_inferences_per_s_rt_plus_4be", rt="resnet152", be=["resnet152"] * 4,
               desc="configs[2]: ResNet-152 b1 RT client back-to-back + 4 BE ResNet-152 b1 closed-loop clients, REEF mode"),
    "c3": dict(metric="inception_v3_b1_inferences_per_s_rt_plus_vgg16_densenet201_be", rt="inception_v3",
               be=["vgg16", "densenet201"],
               desc="configs[3]: RT Inception-v3 b1 (299x299) + BE VGG-16 b1 + BE DenseNet-201 b1, REEF mode (kernel padding mix)"),
    "c4": dict(metric="bert_base_s128_inferences_per_s_rt_plus_4be_resnet50", rt="bert_base", be=["resnet50"] * 4,
               desc="configs[4]: RT BERT-base b1 seq 128 + 4 BE ResNet-50 b1 per GPU, REEF mode"),
}
METRIC = WORKLOADS["c2"]["metric"]
WORKLOAD = WORKLOADS["c2"]["desc"]
MODEL = WORKLOADS["c2"]["rt"]


def model_input(base, seed):
    """(input storage name, seeded synthetic input) of the model at `base`: images ~ N(0,1), token ids uniform."""
    st = json.load(open(base + ".json"))["storage"][0]
    rng = np.random.default_rng(seed)
    if st["stype"] == "int64":
        return st["name"], rng.integers(0, 30522, st["size"]).astype(np.int64)
    return st["name"], rng.normal(0, 1, st["size"]).astype(np.float32)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock/throttle samples during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu):
        self.gpu, self.proc, self.lines = gpu, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def pct(a, q):
    return float(np.percentile(a, q)) if len(a) else None


def pinned_array(capi, nbytes, dtype=np.float32):
    import ctypes as C
    p = C.c_void_p()
    rc = capi.cuda_lib().reef_host_alloc_pinned(C.byref(p), C.c_size_t(nbytes))
    if rc != 0:
        raise RuntimeError("reef_host_alloc_pinned failed: " + capi.last_error())
    buf = (C.c_char * nbytes).from_address(p.value)
    return np.frombuffer(buf, dtype=dtype)


def run_reference_arm(args, rank, world):
    """CPU arm: the oracle port of the ResNet-152 schedule on all host cores; a step = one inference."""
    if rank != 0:
        return
    from oracle import oracle
    from reef_b200 import resources
    d = resources.generate(MODEL)
    base = os.path.join(d, MODEL)
    x = np.random.default_rng(2001).normal(0, 1, 3 * 224 * 224).astype(np.float32)
    o = oracle.OracleExecutor(base + ".json", base + ".param")
    o.set_input("data", x)
    oracle.set_threads(os.cpu_count() or 1)   # torchrun exports OMP_NUM_THREADS=1; the CPU arm uses every host core
    cores = oracle.num_threads()
    for _ in range(max(1, min(args.warmup, 3))):
        o.execute()
    steps = max(1, min(args.steps, 20))   # bounded sample: about 10-30 s of CPU work
    t0 = time.perf_counter()
    for _ in range(steps):
        o.execute()
    dt = time.perf_counter() - t0
    v = steps / dt
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": args.warmup, "ms_per_step": 1000.0 * dt / steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD + " (CPU arm: the same ResNet-152 schedule, one client, sequential)"},
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                             "sample": f"{steps} ResNet-152 b1 inferences, OpenMP on {cores} threads"},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20, help="timed steps; one step = %d RT requests" % REQS_PER_STEP)
    ap.add_argument("--warmup", type=int, default=3, help="warm-up steps (at least 3)")
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--be-cap", type=int, default=int(os.environ.get("REEF_BE_CAP", "2")),
                    help="kernels a BE task keeps on its stream (reference: 2, scheduler.cpp:32)")
    ap.add_argument("--pad-target", type=float, default=None,
                    help="slowdown the padding controller may cost a real-time task (default: the scheduler's 0.065)")
    ap.add_argument("--mapped-flag", action="store_true", help="also measure preemption with the flag in mapped host memory")
    ap.add_argument("--be-sms", type=int, default=int(os.environ.get("REEF_BE_SMS", "0")),
                    help="SMs set aside for the best-effort streams (spatial partition; 0 = none, all streams share the GPU)")
    ap.add_argument("--partition-flags", type=int, default=0, help="flags of reef_partition_create")
    ap.add_argument("--no-pin", action="store_true", help="do not pin the scheduler and client threads to CPU cores")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--profile-out", default="")
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    n_be = len(wl["be"])
    args.warmup = max(args.warmup, 3)
    n_req, n_warm = args.steps * REQS_PER_STEP, args.warmup * REQS_PER_STEP

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: no CUDA device is visible and there is no CPU fallback")
    from reef_b200 import build, capi, resources
    if rank == 0:
        build.build_all()
    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        import datetime
        # a rank that fails must not keep the others waiting at a barrier for the default ten minutes
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=150))
        dist.barrier()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # CPU placement: every rank takes an equal slice of the cores this process may run on; inside it the scheduler
    # thread and the RT client get a core each, the BE clients share the rest (the scheduler thread and the RT client
    # both spin: left unpinned, eight ranks of them fight over the same cores and the RT tail grows)
    cpu_slice = None
    try:
        cores = sorted(os.sched_getaffinity(0))
    except AttributeError:
        cores = list(range(os.cpu_count() or 1))
    per_rank = len(cores) // max(1, int(os.environ.get("LOCAL_WORLD_SIZE", world)))
    if not args.no_pin and per_rank >= 3 and cores == list(range(cores[0], cores[0] + len(cores))):
        cpu_slice = (cores[0] + local_rank * per_rank, per_rank)
    torch.set_num_threads(1)

    models = sorted(set([wl["rt"]] + wl["be"]))
    if rank == 0:
        from reef_b200 import profiler
        for m in models:
            d = resources.generate(m)
            # latency tables for the padding policy, measured on this GPU (the reference ships them per model)
            profiler.profile_model(os.path.join(d, m), iters=10, device=local_rank)
    barrier()
    bases = {m: os.path.join(resources.generate(m), m) for m in models}
    inputs = {m: model_input(bases[m], 2001 + rank) for m in models}
    base = bases[wl["rt"]]
    in_name, x = inputs[wl["rt"]]
    S = capi.REEFScheduler

    def load(s, m, qtype):
        b = bases[m]
        mid = s.load_model_files(b + ".json", b + ".profile.json", b + ".param")
        s.bind_model_queue(s.create_queue(qtype), mid)
        s.set_input(mid, inputs[m][1], inputs[m][0])
        return mid

    extra_cfg = {}

    def make_sched(n_be_clients, rt=True, mapped_flag=False, stamps=False, partition=True):
        s = S(S.REEF, local_rank)
        if partition and args.be_sms > 0:
            extra_cfg["sm_partition_rt_be"] = list(s.set_sm_partition(args.be_sms, args.partition_flags))
        s.set_be_stream_cap(args.be_cap)
        if args.pad_target is not None:
            s.set_pad_slowdown_target(args.pad_target)
        if cpu_slice is not None:
            s.set_cpu_slice(*cpu_slice)
        if mapped_flag:
            s.use_mapped_flag()
        if stamps:
            s.set_device_stamps(True)
        s.run()
        ids = {"rt": None, "be": [], "be_models": wl["be"][:n_be_clients]}
        if rt:
            ids["rt"] = load(s, wl["rt"], S.RealTimeQueue)
        for m in wl["be"][:n_be_clients]:
            ids["be"].append(load(s, m, S.BestEffortQueue))
        return s, ids

    extra = {}
    # ---- phase A: RT alone (on the whole GPU: with a spatial partition the baselines of both kinds stay unpartitioned) (closed loop, inputs resident) -------------------------------------
    s, ids = make_sched(0, partition=False)
    r = s.run_clients([dict(mid=ids["rt"], max_requests=n_req, warmup=n_warm, want_output=False)])[0]
    extra["rt_alone_p50_ms"] = pct(r["latencies_ms"], 50)
    extra["rt_alone_p99_ms"] = pct(r["latencies_ms"], 99)
    extra["rt_alone_inf_s"] = r["completed"] / r["elapsed_s"]
    s.shutdown(); s.close()
    if args.be_sms > 0:
        s, ids = make_sched(0)
        r = s.run_clients([dict(mid=ids["rt"], max_requests=max(200, n_req // 4), warmup=n_warm, want_output=False)])[0]
        extra["rt_alone_on_its_partition_p50_ms"] = pct(r["latencies_ms"], 50)
        extra["rt_alone_on_its_partition_p99_ms"] = pct(r["latencies_ms"], 99)
        s.shutdown(); s.close()

    # ---- phase B: BE alone ---------------------------------------------------------------------
    if n_be:
        s, ids = make_sched(n_be, rt=False, partition=False)
        be_req = max(20, n_req // 8)
        rs = s.run_clients([dict(mid=m, max_requests=be_req, warmup=max(3, n_warm // 8), want_output=False)
                            for m in ids["be"]])
        extra["be_alone_inf_s"] = sum(r["completed"] / r["elapsed_s"] for r in rs)
        s.shutdown(); s.close()

    # ---- phase C (timed region of `value`): RT + 4 BE, inputs resident in HBM --------------------
    s, ids = make_sched(n_be)
    clients = [dict(mid=ids["rt"], max_requests=n_req, warmup=n_warm, want_output=False)] + \
              [dict(mid=m, max_requests=0, want_output=False) for m in ids["be"]]
    sampler = ClockSampler(local_rank)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.start()
    launches0 = capi.launch_count()
    ev0.record()
    rs = s.run_clients(clients)
    torch.cuda.synchronize()
    ev1.record()
    torch.cuda.synchronize()
    launches = capi.launch_count() - launches0
    clocks = sampler.stop()
    barrier()
    rt_r, be_r = rs[0], rs[1:]
    # the timed region of the K steps is the RT client's recorded window; the BE clients count over the same window
    # (they start counting when the RT client has finished its warm-up), so the two throughputs add up
    region_s = rt_r["elapsed_s"]
    be_inf_s = sum(r["completed"] / r["elapsed_s"] for r in be_r if r["elapsed_s"] > 0)
    st = s.stats()
    extra.update({"rt_p50_ms": pct(rt_r["latencies_ms"], 50), "rt_p99_ms": pct(rt_r["latencies_ms"], 99),
                  "be_inf_s": be_inf_s, "rt_inf_s": rt_r["completed"] / region_s,
                  "preempt_count_back_to_back": st["preempt_count"],
                  "padded_kernels": st["padded_kernels"], "be_tasks_padded_to_finish": st["be_tasks_padded_to_finish"],
                  "device_event_ms_incl_warmup": ev0.elapsed_time(ev1), "be_stream_cap": args.be_cap})
    s.shutdown(); s.close()

    if n_be:
        # ---- phase D: reset-based preemption.  The RT client pauses 2 ms between requests, so the BE clients run at
        # full speed on their own streams and every RT arrival preempts them (under a back-to-back RT client the BE
        # tasks only advance as padding and there is nothing to preempt).  Three figures per preemption:
        #   flag    host clock: flag raised, queued launches dropped, tasks rolled back
        #   drain   host clock: flag write -> BE streams idle and completion counters read.  This is the figure to
        #           hold against the 20 us target: the reference's switch also ends with no BE wavefront running
        #           (scheduler.cpp:305-346, 374-439: flag, clear queues, kill wavefronts, measured around the whole)
        #   device  %globaltimer: first BE block that saw the flag -> last BE block that left
        # --mapped-flag repeats the drain phase with the flag in mapped host memory raised by a host store (every
        # device-side poll then crosses PCIe: measured 20 times slower, hence not the default).
        n_pre = max(200, n_req // 8)

        def preempt_phase(wait_sync, mapped, be_cap=None):
            s, ids = make_sched(n_be, mapped_flag=mapped, stamps=wait_sync)
            s.set_wait_sync(wait_sync)
            if be_cap is not None:
                s.set_be_stream_cap(be_cap)
            clients = [dict(mid=ids["rt"], max_requests=n_pre, warmup=5, want_output=False, think_us=2000)] + \
                      [dict(mid=m, max_requests=0, want_output=False) for m in ids["be"]]
            rs = s.run_clients(clients)
            st = s.stats()
            s.shutdown(); s.close()
            return rs, st

        rs, st = preempt_phase(False, False)
        extra["preempt_flag_avg_us"] = st["preempt_ns_sum"] / max(1, st["preempt_count"]) / 1e3
        extra["preempt_flag_max_us"] = st["preempt_ns_max"] / 1e3
        extra["preempt_flag_count"] = st["preempt_count"]
        extra["be_inf_s_rt_every_2ms"] = sum(r["completed"] / r["elapsed_s"] for r in rs[1:] if r["elapsed_s"] > 0)
        for tag, mapped in [("", False)] + ([("mapped_flag_", True)] if args.mapped_flag else []):
            rs, st = preempt_phase(True, mapped)
            extra["preempt_%sdrain_avg_us" % tag] = st["drain_ns_sum"] / max(1, st["drain_count"]) / 1e3
            extra["preempt_%sdrain_p50_us" % tag] = st["drain_ns_p50"] / 1e3
            extra["preempt_%sdrain_p99_us" % tag] = st["drain_ns_p99"] / 1e3
            extra["preempt_%sdrain_max_us" % tag] = st["drain_ns_max"] / 1e3
            extra["preempt_%sdevice_avg_us" % tag] = st["dev_ns_sum"] / max(1, st["dev_count"]) / 1e3
            extra["preempt_%sdevice_max_us" % tag] = st["dev_ns_max"] / 1e3
            extra["preempt_%sdrain_count" % tag] = st["drain_count"]
            extra["preempt_%sdevice_samples" % tag] = st["dev_count"]
            extra["be_inf_s_%srt_every_2ms_with_drain" % tag] = sum(r["completed"] / r["elapsed_s"] for r in rs[1:] if r["elapsed_s"] > 0)
            if not mapped:
                extra["rt_after_preempt_p50_ms"] = pct(rs[0]["latencies_ms"], 50)
                extra["rt_after_preempt_p99_ms"] = pct(rs[0]["latencies_ms"], 99)
        if args.be_cap != 1:
            # the in-flight cap trades free-running best-effort throughput against the drain: with one kernel per stream
            # in flight (the reference's default is 2, scheduler.cpp:29-33) nothing is queued behind the kernel that leaves
            rs, st = preempt_phase(True, False, be_cap=1)
            extra["preempt_cap1_drain_avg_us"] = st["drain_ns_sum"] / max(1, st["drain_count"]) / 1e3
            extra["preempt_cap1_drain_p99_us"] = st["drain_ns_p99"] / 1e3
            extra["preempt_cap1_drain_max_us"] = st["drain_ns_max"] / 1e3
            extra["be_inf_s_cap1_rt_every_2ms_with_drain"] = sum(r["completed"] / r["elapsed_s"] for r in rs[1:] if r["elapsed_s"] > 0)
        extra["preempt_target_metric"] = "preempt_drain_avg_us (flag write -> best-effort streams drained, host clock) < 20"

    # ---- phase E (e2e): same workload through the request calls with pinned host buffers ---------
    s, ids = make_sched(n_be)
    in_bytes = x.nbytes
    pins = []
    clients = []
    for i, (mid, mname) in enumerate(zip([ids["rt"]] + ids["be"], [wl["rt"]] + ids["be_models"])):
        nm, arr = inputs[mname]
        pin = pinned_array(capi, arr.nbytes, arr.dtype)
        pin[:] = arr
        pins.append(pin)
        clients.append(dict(mid=mid, max_requests=n_req if i == 0 else 0, warmup=n_warm if i == 0 else 0,
                            input=pin, input_name=nm, want_output=True))
    barrier()
    rs = s.run_clients(clients)
    barrier()
    e2e_region = rs[0]["elapsed_s"]
    e2e_total = rs[0]["completed"] / e2e_region + sum(r["completed"] / r["elapsed_s"] for r in rs[1:] if r["elapsed_s"] > 0)
    out_bytes = int(rs[0]["output"].nbytes)
    extra["e2e_rt_p50_ms"] = pct(rs[0]["latencies_ms"], 50)
    extra["e2e_rt_p99_ms"] = pct(rs[0]["latencies_ms"], 99)
    s.shutdown(); s.close()

    # ---- kernel profile -> roofline of the dominant kernel family (conv2d) ------------------------
    e = capi.HybridExecutor(local_rank)
    e.load_model_from_file(base + ".json", base + ".profile.json")
    e.load_param_from_file(base + ".param")
    e.set_input(in_name, x)
    prof = e.profile_kernels(20)
    names = [k["name"] for k in json.load(open(base + ".json"))["kernels"]]
    conv = [(n, p) for n, p in zip(names, prof) if p["tensor_core"]]   # reef_conv_tc_kernel launches
    conv_us = sum(p["us"] for _, p in conv)
    conv_bytes = sum(p["bytes"] for _, p in conv)
    conv_flops = sum(p["flops"] for _, p in conv)
    all_us = sum(p["us"] for p in prof)
    peak, peak_kind = measured_peaks()
    # launch duration of the dominant kernel: a CUDA graph holding only the tensor-core launches of one pass, in
    # schedule order, replayed back to back and timed with CUDA events on its stream (events between single
    # kernels would add several microseconds of serialisation to every launch)
    tc_ms, tc_n = e.time_tensor_core(5, 50)
    achieved = conv_bytes / (tc_ms * 1e-3) / 1e9
    traffic = CONV_TC_TRAFFIC_PER_LAUNCH.get(args.workload)
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "peak_kind": peak_kind,
                "traffic_source": ("constant from an ncu capture of the 154 ResNet-152 launches (dram bytes read + written "
                                   "per launch, profiles/conv_tc_resnet152_dram.md); not measured in this run"
                                   if traffic is not None else None),
                "kernel": "reef_conv_tc_kernel (tcgen05 TF32 convolution/matmul: the %d launches of one %s pass as a CUDA "
                          "graph of their own, timed with CUDA events over 50 replays)" % (tc_n, wl["rt"]),
                "algorithmic_bytes_per_pass": conv_bytes, "algorithmic_bytes_per_launch": conv_bytes / max(1, tc_n),
                "avg_launch_us": 1e3 * tc_ms / max(1, tc_n),
                "avg_launch_us_with_events_between_kernels": conv_us / max(1, len(conv)),
                "conv_tflops": conv_flops / (tc_ms * 1e-3) / 1e12, "conv_share_of_kernel_time": conv_us / all_us}
    graph_ms = e.time(1, 5, 50)
    extra["rt_graph_device_ms"] = graph_ms
    # model-level fraction: sum over all kernels of (algorithmic bytes / HBM peak) over the replay time; at batch 1
    # every kernel's floor is its HBM time, and launch gaps dominate the rest
    roofline["model_hbm_floor_us"] = sum(p["bytes"] for p in prof) / (peak * 1e9) * 1e6
    roofline["model_frac"] = roofline["model_hbm_floor_us"] / (graph_ms * 1e3)
    if args.profile_out and rank == 0:
        with open(args.profile_out, "w") as f:
            json.dump([dict(name=n, **p) for n, p in zip(names, prof)], f, indent=1)
    e.close()

    # ---- aggregate over ranks --------------------------------------------------------------------
    value = rt_r["completed"] / region_s + be_inf_s
    ms_per_step = 1000.0 * region_s / max(1, args.steps)
    e2e_value = e2e_total
    from reef_b200 import replicas
    sums, maxes = replicas.aggregate(dist, {"value": value, "e2e": e2e_value, "launches": float(launches)},
                                     {"ms_per_step": ms_per_step, "rt_p99_ms": extra["rt_p99_ms"],
                                      "rt_alone_p99_ms": extra["rt_alone_p99_ms"]},
                                     device="cuda" if dist is not None else None)
    value, e2e_value, launches = sums["value"], sums["e2e"], int(sums["launches"])
    ms_per_step = maxes["ms_per_step"]
    if dist is not None:
        extra["rt_p99_ms_max_over_ranks"] = maxes["rt_p99_ms"]
        extra["rt_alone_p99_ms_max_over_ranks"] = maxes["rt_alone_p99_ms"]

    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        from oracle import oracle
        oracle.set_threads(os.cpu_count() or 1)
        o = oracle.OracleExecutor(base + ".json", base + ".param")
        o.set_input(in_name, x)
        o.execute()
        n_cpu = 0
        t0 = time.perf_counter()
        while n_cpu < 3 or (time.perf_counter() - t0 < 10.0 and n_cpu < 40):
            o.execute()
            n_cpu += 1
        dt = time.perf_counter() - t0
        cpu = {"value": n_cpu / dt, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
               "sample": f"{n_cpu} sequential {wl['rt']} b1 inferences of the same schedule (plain-C oracle, OpenMP)"}
        # second CPU row: the same schedule interpreted with PyTorch's CPU operators on all host cores
        try:
            from oracle import torch_ref
            torch.set_num_threads(os.cpu_count() or 1)
            te = torch_ref.TorchExecutor(base + ".json", base + ".param")
            te.set_input(in_name, x)
            te.execute()
            n_t = 0
            t0 = time.perf_counter()
            while n_t < 3 or (time.perf_counter() - t0 < 8.0 and n_t < 200):
                te.execute()
                n_t += 1
            dt = time.perf_counter() - t0
            cpu["pytorch_cpu"] = {"value": n_t / dt, "unit": UNIT, "cores": torch.get_num_threads(),
                                  "sample": f"{n_t} sequential {wl['rt']} b1 inferences, PyTorch {torch.__version__} CPU operators "
                                            "over the same schedule and weights"}
        except Exception as ex:   # the row is informative; the port above is the baseline
            cpu["pytorch_cpu"] = {"unavailable": repr(ex)[:200]}

    if rank == 0:
        line = {"metric": wl["metric"], "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "tf32", "data": "synthetic",
                "config": {"workload": wl["desc"], "inputs": "seeded synthetic: images N(0,1), token ids uniform",
                           "arithmetic": "convolutions and matmuls multiply in TF32 on tcgen05 with fp32 accumulation; everything else fp32",
                           "clients": "1 RT + %d BE per GPU" % n_be,
                           "step": "%d back-to-back RT requests (%d timed after %d warm-up)" % (REQS_PER_STEP, n_req, n_warm),
                           "cpu_slice": list(cpu_slice) if cpu_slice else None,
                           **extra_cfg,
                           "l2": "every client owns a weight replica; the replicas streamed per pass exceed the 126 MB L2"},
                "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes},
                "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
                "rt_be": extra}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
