"""GPU tests of REEFScheduler through the C entry points (mirrors reference test.cpp:346-535)."""
import json
import time

import numpy as np
import pytest

from conftest import rel_err, seeded_input
from gpu_util import FP32_TOL, tol_for
from oracle import oracle
from reef_b200 import capi

pytestmark = pytest.mark.gpu
S = capi.REEFScheduler


def _oracle_out(base, x):
    o = oracle.OracleExecutor(base + ".json", base + ".param")
    o.set_input("data", x)
    o.execute()
    return o.get_output()


@pytest.mark.parametrize("qtype", [S.RealTimeQueue, S.BestEffortQueue])
def test_scheduler_mocked_kernel(gen, qtype):
    # reference: test.cpp:346-369 (rt), :397-420 (be)
    base = gen("mocked_kernel")
    s = S(S.REEF)
    s.run()
    mid = s.load_model_files(base + ".json", base + ".profile.json")
    qid = s.create_queue(qtype)
    s.bind_model_queue(qid, mid)
    three = np.full(8192, 3.0, np.float32)
    for n in ("a", "b", "c"):
        s.set_input(mid, three, n)
    tid = s.new_task(mid)
    s.wait_task(tid)
    assert np.all(s.get_output(mid) == 18.0)
    assert s.get_task(tid).state == S.Finish
    s.shutdown()
    s.close()


def test_scheduler_errors(gen):
    base = gen("mocked_kernel")
    s = S(S.REEF)
    with pytest.raises(capi.ReefError) as e:
        s.new_task(0)                                   # no such model
    assert e.value.status == capi.OUT_OF_RANGE
    mid = s.load_model_files(base + ".json", base + ".profile.json")
    with pytest.raises(capi.ReefError) as e:
        s.bind_model_queue(7, mid)                      # no such queue
    assert e.value.status == capi.OUT_OF_RANGE
    qids = [s.create_queue(S.BestEffortQueue) for _ in range(32)]
    assert qids == list(range(32))
    with pytest.raises(capi.ReefError) as e:
        s.create_queue(S.BestEffortQueue)               # reference: max_num_be_queues = 32 -> Full
    assert e.value.status == capi.FULL
    with pytest.raises(capi.ReefError) as e:
        s.load_model_files("/nonexistent.json")
    assert e.value.status == capi.NOT_FOUND
    s.close()


@pytest.mark.parametrize("mode", [S.NoPreempt, S.MultiStream, S.WaitPreempt, S.REEF, S.Reset])
def test_scheduler_resnet18_rt_and_be_all_modes(gen, mode):
    base = gen("resnet18")
    x = seeded_input(3 * 224 * 224, seed=3)
    want = _oracle_out(base, x)
    FP32_TOL = tol_for(base)
    s = S(mode)
    s.run()
    rt = s.load_model_files(base + ".json", base + ".profile.json", base + ".param")
    be = s.load_model_files(base + ".json", base + ".profile.json", base + ".param")
    s.bind_model_queue(s.create_queue(S.RealTimeQueue), rt)
    s.bind_model_queue(s.create_queue(S.BestEffortQueue), be)
    s.set_input(rt, x)
    s.set_input(be, x)
    for _ in range(3):
        t_be = s.new_task(be)
        t_rt = s.new_task(rt)
        s.wait_task(t_rt)
        s.wait_task(t_be)
        assert rel_err(s.get_output(rt), want) < FP32_TOL
        assert rel_err(s.get_output(be), want) < FP32_TOL
    s.shutdown()
    s.close()


def test_scheduler_preempt_and_resume(gen):
    """reference: test.cpp:448-489 — a best-effort task is running when a real-time task arrives: the
    real-time task starts later and ends earlier, the best-effort task reports preempted and/or padded,
    and its output is still right (here: bit-identical to an uninterrupted best-effort run)."""
    base = gen("resnet152")
    x = seeded_input(3 * 224 * 224, seed=4)
    for wait_sync in (False, True):
        s = S(S.REEF)
        s.set_wait_sync(wait_sync)
        s.run()
        rt = s.load_model_files(base + ".json", base + ".profile.json", base + ".param")
        be = s.load_model_files(base + ".json", base + ".profile.json", base + ".param")
        s.bind_model_queue(s.create_queue(S.RealTimeQueue), rt)
        s.bind_model_queue(s.create_queue(S.BestEffortQueue), be)
        s.set_input(rt, x)
        s.set_input(be, x)
        t0 = s.new_task(be)
        s.wait_task(t0)
        uninterrupted = s.get_output(be).copy()
        seen = 0
        for delay in (0.0002, 0.0005, 0.001, 0.002):
            t_be = s.new_task(be)
            time.sleep(delay)
            t_rt = s.new_task(rt)
            s.wait_task(t_rt)
            s.wait_task(t_be)
            ib, ir = s.get_task(t_be), s.get_task(t_rt)
            assert ir.submit_ns >= ib.submit_ns
            if ib.preempted or ib.padded:
                seen += 1
                assert ib.end_ns >= ir.start_ns
            assert np.array_equal(s.get_output(be), uninterrupted), f"delay {delay}: resumed output differs"
            assert np.array_equal(s.get_output(rt), uninterrupted)
        st = s.stats()
        print("wait_sync", wait_sync, "preempted/padded tasks", seen, st, "avg preempt us", s.avg_preempt_latency())
        assert seen > 0 and st["preempt_count"] > 0
        s.shutdown()
        s.close()


def test_scheduler_mocked_kernel_padded_to_complete(gen):
    # reference: test.cpp:491-535 — BE and RT queued before run(): the BE task finishes inside the padding
    base = gen("mocked_kernel")
    s = S(S.REEF)
    rt = s.load_model_files(base + ".json", base + ".profile.json")
    be = s.load_model_files(base + ".json", base + ".profile.json")
    s.bind_model_queue(s.create_queue(S.RealTimeQueue), rt)
    s.bind_model_queue(s.create_queue(S.BestEffortQueue), be)
    three = np.full(8192, 3.0, np.float32)
    for m in (rt, be):
        for n in ("a", "b", "c"):
            s.set_input(m, three, n)
    t_be = s.new_task(be)
    t_rt = s.new_task(rt)
    s.run()
    s.wait_task(t_rt)
    s.wait_task(t_be)
    assert s.get_task(t_be).padded_to_complete == 1 and s.get_task(t_be).padded == 1
    assert np.all(s.get_output(rt) == 18.0) and np.all(s.get_output(be) == 18.0)
    s.shutdown()
    s.close()


def test_closed_loop_clients_rt_with_be(gen):
    base = gen("resnet18")
    x = seeded_input(3 * 224 * 224, seed=9)
    want = _oracle_out(base, x)
    FP32_TOL = tol_for(base)
    s = S(S.REEF)
    s.run()
    rt = s.load_model_files(base + ".json", base + ".profile.json", base + ".param")
    s.bind_model_queue(s.create_queue(S.RealTimeQueue), rt)
    bes = []
    for _ in range(2):
        m = s.load_model_files(base + ".json", base + ".profile.json", base + ".param")
        s.bind_model_queue(s.create_queue(S.BestEffortQueue), m)
        bes.append(m)
    clients = [dict(mid=rt, max_requests=200, warmup=5, input=x)] + [dict(mid=m, max_requests=0, input=x) for m in bes]
    res = s.run_clients(clients)
    assert res[0]["completed"] == 200 and res[0]["latencies_ms"].min() > 0
    assert rel_err(res[0]["output"], want) < FP32_TOL
    for r in res[1:]:
        assert r["completed"] > 0 and rel_err(r["output"], want) < FP32_TOL
    s.shutdown()
    s.close()


def test_padding_segments_keep_best_effort_results_exact(gen):
    """Four best-effort ResNet-152 clients advance only as padding under a back-to-back real-time client
    (padding segments, several pieces per stream, tasks completed inside the window): every client finishes
    requests, most of them entirely by padding, and every output is bit-identical to an unpadded run."""
    base = gen("resnet152")
    x = seeded_input(3 * 224 * 224, seed=21)
    e = capi.HybridExecutor(0)
    e.load_model_from_file(base + ".json", base + ".profile.json")
    e.load_param_from_file(base + ".param")
    e.set_input("data", x)
    e.execute()
    want = e.get_output().copy()
    e.close()
    s = S(S.REEF)
    s.set_pad_slowdown_target(0.5)      # a generous slowdown budget: pad as much as fits
    s.run()
    rt = s.load_model_files(base + ".json", base + ".profile.json", base + ".param")
    s.bind_model_queue(s.create_queue(S.RealTimeQueue), rt)
    bes = []
    for _ in range(4):
        m = s.load_model_files(base + ".json", base + ".profile.json", base + ".param")
        s.bind_model_queue(s.create_queue(S.BestEffortQueue), m)
        bes.append(m)
    res = s.run_clients([dict(mid=rt, max_requests=150, warmup=10, input=x)] +
                        [dict(mid=m, max_requests=0, input=x) for m in bes])
    st = s.stats()
    print("padding stats", st, "be completed", [r["completed"] for r in res[1:]])
    assert capi.device_error() == 0
    assert np.array_equal(res[0]["output"], want)
    for r in res[1:]:
        assert r["completed"] > 0 and np.array_equal(r["output"], want)
    assert st["padded_kernels"] > 1000 and st["be_tasks_padded_to_finish"] > 0
    s.shutdown()
    s.close()


def test_failed_launch_and_device_error_end_in_a_failed_task(gen):
    """A task whose kernel launch returns an error, or during which the device error word was set, ends in Finish
    with the failed mark and wait_task returns Fail (the reference aborts the process, hip_impl.h:34-41).  Both
    failures are injected on the host: the launch call is made to return an error before it reaches the device, and
    the error word is stored from the host; no device-side wait is made to expire."""
    base = gen("resnet18_64")
    x = seeded_input(3 * 64 * 64, seed=2)
    for qtype in (S.RealTimeQueue, S.BestEffortQueue):
        s = S(S.REEF)
        s.run()
        mid = s.load_model_files(base + ".json", base + ".profile.json", base + ".param")
        s.bind_model_queue(s.create_queue(qtype), mid)
        s.set_input(mid, x)
        t = s.new_task(mid)
        s.wait_task(t)
        good = s.get_output(mid).copy()
        assert s.get_task(t).failed == 0
        # 1. the launch call fails (once)
        s.inject_launch_failures(mid, 1)
        t = s.new_task(mid)
        with pytest.raises(capi.ReefError) as ex:
            s.wait_task(t)
        assert ex.value.status == capi.FAIL
        info = s.get_task(t)
        assert info.state == S.Finish and info.failed == 1
        # 2. the next task is clean again and right
        t = s.new_task(mid)
        s.wait_task(t)
        assert s.get_task(t).failed == 0 and np.array_equal(s.get_output(mid), good)
        # 3. the device error word is found set when the task's stream has drained
        capi.device_error_set(1)
        t = s.new_task(mid)
        with pytest.raises(capi.ReefError) as ex:
            s.wait_task(t)
        assert ex.value.status == capi.FAIL and s.get_task(t).failed == 1
        assert capi.device_error() == 0          # the scheduler cleared the word
        t = s.new_task(mid)
        s.wait_task(t)
        assert s.get_task(t).failed == 0 and np.array_equal(s.get_output(mid), good)
        # a closed-loop client stops at the first failed request and says so
        s.inject_launch_failures(mid, 1)
        res = s.run_clients([dict(mid=mid, max_requests=5, warmup=0, input=x)], allow_failed=True)
        assert res[0]["failed"] and res[0]["completed"] == 0
        s.shutdown()
        s.close()


def test_scheduler_sm_partition_keeps_results(gen):
    """Best-effort streams confined to SMs of their own (a green-context partition; the real-time stream keeps the
    whole GPU with flag 4, or takes the other side of the split with flag 0): outputs are unchanged."""
    base = gen("resnet18")
    x = seeded_input(3 * 224 * 224, seed=11)
    want = _oracle_out(base, x)
    tol = tol_for(base)
    for flags in (4, 0):
        s = S(S.REEF)
        rt_sms, be_sms = s.set_sm_partition(32, flags)
        assert be_sms >= 8 and rt_sms >= 8 and rt_sms + be_sms <= 148
        s.run()
        rt = s.load_model_files(base + ".json", base + ".profile.json", base + ".param")
        be = s.load_model_files(base + ".json", base + ".profile.json", base + ".param")
        s.bind_model_queue(s.create_queue(S.RealTimeQueue), rt)
        s.bind_model_queue(s.create_queue(S.BestEffortQueue), be)
        res = s.run_clients([dict(mid=rt, max_requests=40, warmup=5, input=x), dict(mid=be, max_requests=0, input=x)])
        assert rel_err(res[0]["output"], want) < tol
        # (how many best-effort requests finish inside 40 short real-time requests depends on the padding throttle: the
        # best-effort result is checked on a request of its own afterwards, whatever was preempted or padded before)
        t = s.new_task(be)
        s.wait_task(t)
        assert s.get_task(t).failed == 0 and rel_err(s.get_output(be), want) < tol
        assert capi.device_error() == 0
        s.shutdown()
        s.close()
