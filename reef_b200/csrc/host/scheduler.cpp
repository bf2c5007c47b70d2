#include "scheduler.h"

#include <pthread.h>
#include <sched.h>

#include <algorithm>
#include <cassert>
#include <cstdlib>

namespace reef {
namespace server {

using executor::HybridExecutor;
typedef std::chrono::steady_clock sclock;

static inline uint64_t ns_since(sclock::time_point t0) {
    return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(sclock::now() - t0).count();
}

REEFScheduler::REEFScheduler(ScheduleMode _mode, int _device)
    : mode(_mode),
      device(_device),
      model_pool_size(0),
      model_pool(model_pool_capacity),
      task_idx_pool(0),
      be_queues(max_num_be_queues),
      be_queue_cnt(0),
      wait_sync(false),
      rt_graph(true),
      preempted(false),
      _shutdown(false),
      pending_tasks(0),
      preempt_count(0),
      preempt_latency_sum(0),
      preempt_latency_max(0),
      kernel_sel_count(0),
      kernel_sel_latency_sum(0),
      n_rt_tasks(0),
      n_be_tasks(0),
      n_be_padded_finish(0),
      n_padded_kernels(0),
      n_padded_blocks(0) {
    // reference: scheduler.cpp:24-33
    if (reef_gpu_init(device) != REEF_SUCC || reef_device_num_sms(&num_sms) != REEF_SUCC ||
        reef_stream_create(&preempt_stream, 1) != REEF_SUCC || reef_malloc(&preempt_flag, 4) != REEF_SUCC ||
        reef_write32_async(preempt_stream, preempt_flag, 0) != REEF_SUCC ||
        reef_stream_sync(preempt_stream) != REEF_SUCC) {
        err_ = reef_last_error();
        fprintf(stderr, "[reef] scheduler: device layer failed: %s\n", err_.c_str());
        num_sms = 0;   // run()/load_model() refuse to work
    }
    be_stream_device_queue_cap = mode == WaitPreempt ? 1024 : 2;
#ifdef REEF_DEBUG_AIDS
    // development builds: the padding parameters can be set from the environment for sweeps
    if (const char* v = getenv("REEF_PAD_DEPTH")) set_pad_limits(atoi(v), pad_overcommit, pad_quantum);
    if (const char* v = getenv("REEF_PAD_OVERCOMMIT")) set_pad_limits(pad_depth, atoi(v), pad_quantum);
    if (const char* v = getenv("REEF_PAD_QUANTUM")) set_pad_limits(pad_depth, pad_overcommit, atoi(v));
    if (const char* v = getenv("REEF_PAD_WINDOW")) set_pad_window(atoi(v));
    if (const char* v = getenv("REEF_RT_GRACE_US")) set_rt_grace_us(atoi(v));
    if (const char* v = getenv("REEF_PAD_PIECE_CAP")) pad_piece_cap = atoi(v);
    if (const char* v = getenv("REEF_PAD_PIECE_MB")) pad_piece_bytes = atof(v) * 1e6;
    if (const char* v = getenv("REEF_PAD_TARGET")) set_pad_slowdown_target(atof(v));
#endif
}

REEFScheduler::~REEFScheduler() {
    if (scheduler && scheduler->joinable()) shutdown();
#ifdef REEF_DEBUG_AIDS
    if (getenv("REEF_PAD_TRACE") && pad_trace.calls) {
        const PadTrace& t = pad_trace;
        fprintf(stderr,
                "[reef] timeline padding: %llu windows avg %.1f us (graph launch %.1f us), per window: %.1f iterations, "
                "%.1f pieces (launch %.2f us, turnaround %.1f us), iterations skipped: rate-limited %.1f, no free slots %.1f, no queue could take a piece %.1f\n",
                (unsigned long long)t.calls, t.window_ns / 1e3 / t.calls, t.graph_launch_ns / 1e3 / t.calls,
                (double)t.iters / t.calls, (double)t.launched / t.calls, t.launched ? t.launch_ns / 1e3 / t.launched : 0.0,
                t.retired ? t.turnaround_ns / 1e3 / t.retired : 0.0, (double)t.no_slot / t.calls, (double)t.no_sms / t.calls,
                (double)t.no_queue / t.calls);
        fprintf(stderr, "[reef]   per window: segments %.1f, single pieces %.1f; queue visits skipped: empty %.1f, draining %.1f, "
                "depth full %.1f, fully issued %.1f, no fit %.1f\n", (double)t.segments / t.calls, (double)t.singles / t.calls,
                (double)t.q_empty / t.calls, (double)t.q_draining / t.calls, (double)t.q_full / t.calls,
                (double)t.q_issued / t.calls, (double)t.q_nofit / t.calls);
        fprintf(stderr, "[reef]   slowdown controller: target %.3f, smoothed ratio %.3f, rate %.1f kernels per window\n", pad_target,
                pad_ratio_ema, pad_rate);
    }
#endif
    reef_gpu_init(device);
    reef_device_sync();
    model_pool.clear();
    for (auto& q : be_queues)
        if (q) {
            for (auto& f : q->inflight) reef_event_destroy(f.ev);
            for (auto& po : q->pad_out) reef_event_destroy(po.ev);
            for (auto e : q->free_events) reef_event_destroy(e);
            if (q->stream) reef_stream_destroy(q->stream);
        }
    if (rt_queue && rt_queue->stream) reef_stream_destroy(rt_queue->stream);
    if (preempt_stream) reef_stream_destroy(preempt_stream);
    if (device_stamps) reef_preempt_stamps_arm(0);
    if (partition) reef_partition_destroy(partition);
    if (mapped_flag_host) reef_flag_free_mapped(mapped_flag_host);
    else if (preempt_flag) reef_free(preempt_flag);
}

Status REEFScheduler::use_mapped_flag() {
    if (model_pool_size.load() != 0 || mapped_flag_host != nullptr) return Status::Fail;   // executors already hold the flag
    GPU_RETURN_STATUS(reef_gpu_init(device));
    uint32_t* h = nullptr;
    executor::GPUDevicePtr_t d = 0;
    GPU_RETURN_STATUS(reef_flag_alloc_mapped(&h, &d));
    if (preempt_flag) reef_free(preempt_flag);
    mapped_flag_host = h;
    preempt_flag = d;
    return Status::Succ;
}

Status REEFScheduler::set_sm_partition(int be_sms, int flags, int* rt_sms_out, int* be_sms_out) {
    if (partition != nullptr || rt_queue.get() != nullptr || be_queue_cnt.load() != 0) return Status::Fail;   // streams exist already
    GPU_RETURN_STATUS(reef_gpu_init(device));
    if (reef_partition_create(be_sms, flags, &partition) != REEF_SUCC) {
        err_ = reef_last_error();
        partition = nullptr;
        return Status::Fail;
    }
    reef_partition_info(partition, rt_sms_out, be_sms_out);
    partition_rt_whole_gpu = (flags & 4) != 0;
    return Status::Succ;
}

Status REEFScheduler::set_device_stamps(bool on) {
    GPU_RETURN_STATUS(reef_gpu_init(device));
    GPU_RETURN_STATUS(reef_preempt_stamps_arm(on ? 1 : 0));
    device_stamps = on;
    if (on) wait_sync = true;
    return Status::Succ;
}

// raises or clears the preempt flag; returns when the new value is on its way (mapped flag: stored)
void REEFScheduler::write_flag(uint32_t v) {
    if (mapped_flag_host) reef_flag_set(mapped_flag_host, v);
    else reef_write32_async(preempt_stream, preempt_flag, v);
}

Status REEFScheduler::create_task_queue(std::shared_ptr<TaskQueue>& ret, bool rt) {
    executor::GPUStream_t stream;
    GPU_RETURN_STATUS(reef_gpu_init(device));
    if (partition && !(rt && partition_rt_whole_gpu)) {
        GPU_RETURN_STATUS(reef_partition_stream_create(partition, rt ? 0 : 1, rt ? 1 : 0, &stream));
    } else {
        GPU_RETURN_STATUS(reef_stream_create(&stream, rt ? 1 : 0));
    }
    ret = std::make_shared<TaskQueue>();
    ret->stream = stream;
    return Status::Succ;
}

Status REEFScheduler::load_model(const std::string& model_dir, const std::string& model_name, ModelID& mid) {
    std::string base = model_dir + "/" + model_name;
    // the reference's two-argument form loads no parameters (scheduler.cpp:57-68); a .param beside
    // the json is loaded here when it exists
    std::string param = base + ".param";
    FILE* f = fopen(param.c_str(), "rb");
    if (f) fclose(f); else param.clear();
    return load_model(base + ".trans.co", base + ".be.co", base + ".json", base + ".profile.json", param, mid);
}

Status REEFScheduler::load_model(const std::string& rt_co_path, const std::string& be_co_path,
                                 const std::string& json_path, const std::string& profile_path,
                                 const std::string& param_path, ModelID& mid) {
    if (num_sms == 0) RETURN_STATUS(Status::Fail);
    GPU_RETURN_STATUS(reef_gpu_init(device));
    std::shared_ptr<Model> model(new Model);
    Status st = model->executor.load_hybrid_model_from_file(json_path.c_str(), profile_path.c_str(),
                                                            rt_co_path.c_str(), be_co_path.c_str());
    if (st != Status::Succ) {
        err_ = model->executor.error();
        RETURN_STATUS(st);
    }
    model->qid = rt_queue_id;   // real-time queue by default
    if (!param_path.empty()) {
        st = model->executor.load_param_from_file(param_path.c_str());
        if (st != Status::Succ) {
            err_ = model->executor.error();
            RETURN_STATUS(st);
        }
    }
    auto idx = model_pool_size.load();
    if (idx >= model_pool_capacity) RETURN_STATUS(Status::Full);
    model->executor.set_preempt_flag(preempt_flag);
    model_pool[idx] = std::move(model);
    model_pool_size.store(idx + 1);
    mid = idx;
    return Status::Succ;
}

Status REEFScheduler::create_queue(const TaskQueueType& qtp, QueueID& qid) {
    if (qtp == TaskQueueType::RealTimeQueue) {
        qid = rt_queue_id;
        std::unique_lock<std::mutex> lock(be_queues_mtx);
        if (rt_queue.get() == nullptr) RETURN_STATUS(create_task_queue(rt_queue, true));
        return Status::Succ;
    }
    std::shared_ptr<TaskQueue> q;
    RETURN_STATUS(create_task_queue(q, false));
    {
        std::unique_lock<std::mutex> lock(be_queues_mtx);
        auto idx = be_queue_cnt.load();
        if (idx >= max_num_be_queues) {
            reef_stream_destroy(q->stream);
            return Status::Full;
        }
        be_queues[idx] = std::move(q);
        be_queue_cnt.store(idx + 1);
        qid = idx;
    }
    return Status::Succ;
}

Status REEFScheduler::bind_model_queue(const QueueID& qid, const ModelID& mid) {
    if (model_pool_size.load() <= mid) return Status::OutOfRange;
    if (be_queue_cnt.load() <= qid && qid != rt_queue_id) return Status::OutOfRange;
    model_pool[mid]->qid = qid;
    if (qid == rt_queue_id && rt_chain_clusters >= 0) {
        reef_gpu_init(device);
        if (model_pool[mid]->executor.build_chains(rt_chain_clusters) != Status::Succ) {
            err_ = "persistent chains: " + model_pool[mid]->executor.error();
            return Status::Fail;
        }
    }
    if (mode == ScheduleMode::REEF && qid != rt_queue_id) {
        // best-effort model under dynamic kernel padding: capture its padding segments now, not inside a
        // real-time window
        reef_gpu_init(device);
        if (model_pool[mid]->executor.build_pad_segments() != Status::Succ) {
            err_ = "padding segments: " + model_pool[mid]->executor.error();
            return Status::Fail;
        }
    }
    return Status::Succ;
}

Status REEFScheduler::new_task(const ModelID& mid, TaskID& tid) {
    if (model_pool_size.load() <= mid) return Status::OutOfRange;
    auto& model = model_pool[mid];
    if (model->qid == rt_queue_id && rt_queue.get() == nullptr) return Status::Fail;
    std::shared_ptr<Task> task(new Task);
    task->model = model;
    task->id = task_idx_pool.fetch_add(1);
    task->qid = model->qid;
    task->block_offset = 0;
    task->kernel_offset = 0;
    task->launch_offset = 0;
    task->state.store(TaskState::Init);
    task->submit = std::chrono::system_clock::now();
    task->preempted = false;
    task->padding = false;
    task->padding_to_finish = false;
    task->needs_recover = false;
    task->all_issued_by_padding = false;
    task->failed = false;
    tid = task->id;
    {
        std::unique_lock<std::mutex> lock(task_pool_mtx);
        task_pool.insert({tid, task});
    }
    bool ok = model->qid == rt_queue_id ? rt_queue->task_queue.push(task) : be_queues[model->qid]->task_queue.push(task);
    if (!ok) {
        std::unique_lock<std::mutex> lock(task_pool_mtx);
        task_pool.erase(tid);
        return Status::Full;
    }
    if (pending_tasks.fetch_add(1) == 0) {
        std::unique_lock<std::mutex> lock(task_cnt_mtx);
        task_cnt_cv.notify_all();
    }
    return Status::Succ;
}

Status REEFScheduler::get_task(TaskID tid, std::shared_ptr<Task>& t) {
    std::unique_lock<std::mutex> lock(task_pool_mtx);
    auto res = task_pool.find(tid);
    if (res == task_pool.end()) return Status::NotFound;
    t = res->second;
    return Status::Succ;
}

Status REEFScheduler::wait_task(TaskID tid) {
    std::shared_ptr<Task> task;
    Status st = get_task(tid, task);
    if (st != Status::Succ) return st;
    // a real-time caller spins briefly (its inference takes well under a millisecond), then blocks on the task's
    // condvar; a best-effort caller blocks at once and leaves its core to the threads that are on the critical path
    if (task->qid == rt_queue_id) {
        auto t0 = sclock::now();
        while (task->state.load(std::memory_order_acquire) != TaskState::Finish) {
            if (ns_since(t0) > 2000000ull) break;
        }
    }
    {
        std::unique_lock<std::mutex> lock(task->mtx);
        while (task->state.load() != TaskState::Finish) task->cv.wait_for(lock, std::chrono::milliseconds(50));
    }
    {
        // the reference never erases finished tasks (scheduler.cpp:199-205 is commented out) and its pool
        // grows without bound; finished tasks stay queryable through the caller's shared_ptr instead
        std::unique_lock<std::mutex> lock(task_pool_mtx);
        if (task_pool.size() > 4096) task_pool.erase(tid);
    }
    return task->failed ? Status::Fail : Status::Succ;
}

Status REEFScheduler::inject_launch_failures(ModelID mid, int n) {
    if (mid >= model_pool_size.load()) return Status::OutOfRange;
    model_pool[mid]->executor.inject_launch_failures(n);
    return Status::Succ;
}

// The device error word is read after a task's stream has been synchronised (or seen drained): non-zero means a
// bounded wait of some kernel expired since the last look, so what ran since then did not produce valid output.
bool REEFScheduler::device_error_seen(const char* where) {
    int v = 0;
    if (reef_device_error_peek(&v) != REEF_SUCC || v == 0) return false;
    reef_device_error(&v);   // clear: the next task starts clean
    err_ = std::string("device error word set (a bounded device-side wait expired) seen after ") + where;
    fprintf(stderr, "[reef] %s\n", err_.c_str());
    return true;
}

// Diagnostics for the first CUDA error of a run: a device fault is reported by whichever call comes next, not by the
// kernel that caused it, so the kernels every best-effort stream had in flight at that moment are listed once.
void REEFScheduler::dump_streams_once(const char* why) {
    if (streams_dumped) return;
    streams_dumped = true;
    fprintf(stderr, "[reef] first error (%s): preempted=%d wait_sync=%d; best-effort streams:\n", why, (int)preempted, (int)wait_sync);
    const uint32_t nq = be_queue_cnt.load();
    for (uint32_t i = 0; i < nq; i++) {
        auto& q = *be_queues[i];
        if (q.task_queue.empty()) {
            fprintf(stderr, "[reef]   queue %u: idle, %zu padded pieces out\n", i, q.pad_out.size());
            continue;
        }
        auto t = q.task_queue.front();
        auto& exe = t->model->executor;
        fprintf(stderr, "[reef]   queue %u: task %u state %d kernel_offset %d launch_offset %d block_offset %d padded pieces out %zu\n", i,
                t->id, (int)t->get_state(), t->kernel_offset, t->launch_offset, t->block_offset, q.pad_out.size());
        for (auto& f : q.inflight) fprintf(stderr, "[reef]     in flight (best-effort flavour): %d %s\n", f.kernel, exe.kernel_name(f.kernel));
        for (int k : q.preempted_kernels) fprintf(stderr, "[reef]     in flight at the last preemption: %d %s\n", k, exe.kernel_name(k));
        if (q.inflight.empty() && t->kernel_offset < (int)exe.num_kernels())
            fprintf(stderr, "[reef]     next kernel: %d %s\n", t->kernel_offset, exe.kernel_name(t->kernel_offset));
    }
}

// a best-effort task whose launch failed: ended as failed, off its queue, nothing left in the window
void REEFScheduler::fail_be_task(TaskQueue& q, std::shared_ptr<Task>& t, const std::string& why) {
    dump_streams_once(why.c_str());
    err_ = why;
    fprintf(stderr, "[reef] best-effort task %u failed: %s\n", t->id, why.c_str());
    for (auto& f : q.inflight) q.free_events.push_back(f.ev);
    q.inflight.clear();
    t->failed = true;
    t->end = std::chrono::system_clock::now();
    t->kernel_offset = 0;
    t->block_offset = 0;
    t->state.store(TaskState::Finish);
    if (!q.task_queue.empty() && q.task_queue.front() == t) q.task_queue.pop();
    n_be_tasks++;
    finish_task(t);
}

Status REEFScheduler::get_data_size(ModelID mid, const std::string& name, size_t& size) {
    if (mid >= model_pool_size.load()) return Status::OutOfRange;
    return model_pool[mid]->executor.get_data_size(name, size);
}

Status REEFScheduler::set_input(ModelID mid, const void* data, size_t len, const std::string& name) {
    if (mid >= model_pool_size.load()) return Status::OutOfRange;
    GPU_RETURN_STATUS(reef_gpu_init(device));
    return model_pool[mid]->executor.set_input(name, data, len);
}

Status REEFScheduler::get_output(ModelID mid, void* data, size_t len, const std::string& name) {
    if (mid >= model_pool_size.load()) return Status::OutOfRange;
    GPU_RETURN_STATUS(reef_gpu_init(device));
    if (name == "output") return model_pool[mid]->executor.get_output(data, len);
    size_t idx = 0;
    auto& exe = model_pool[mid]->executor;
    for (; idx < exe.model->storage.size(); idx++)
        if (exe.model->storage[idx].name == name) break;
    if (idx == exe.model->storage.size()) return Status::NotFound;
    return exe.get_data((int)idx, data, len);
}

Status REEFScheduler::run() {
    if (scheduler.get() != nullptr || num_sms == 0) return Status::Fail;
    {
        std::unique_lock<std::mutex> lock(be_queues_mtx);
        if (rt_queue.get() == nullptr) RETURN_STATUS(create_task_queue(rt_queue, true));
    }
    _shutdown.store(false);
    scheduler.reset(new std::thread([this] {
        if (cpu_first >= 0 && cpu_count >= 3) {
            cpu_set_t set;
            CPU_ZERO(&set);
            CPU_SET(cpu_first, &set);
            pthread_setaffinity_np(pthread_self(), sizeof(set), &set);   // best effort: a refusal changes nothing else
        }
        reef_gpu_init(device);
        auto last_busy = sclock::now();
        while (!this->_shutdown.load()) {
            this->loop_body();
            if (pending_tasks.load() != 0) {
                last_busy = sclock::now();
            } else if (ns_since(last_busy) > 5000000ull) {
                // idle for 5 ms: stop spinning until a task arrives
                std::unique_lock<std::mutex> lock(task_cnt_mtx);
                task_cnt_cv.wait_for(lock, std::chrono::milliseconds(1),
                                     [this] { return pending_tasks.load() != 0 || _shutdown.load(); });
            }
        }
    }));
    return Status::Succ;
}

Status REEFScheduler::shutdown() {
    if (!scheduler) return Status::Fail;
    _shutdown.store(true);
    {
        std::unique_lock<std::mutex> lock(task_cnt_mtx);
        task_cnt_cv.notify_all();
    }
    if (scheduler->joinable()) scheduler->join();
    scheduler.reset();
    return Status::Succ;
}

void REEFScheduler::finish_task(std::shared_ptr<Task>& t) {
    {
        std::unique_lock<std::mutex> lock(t->mtx);
        t->state.store(TaskState::Finish, std::memory_order_release);
        t->cv.notify_all();
    }
    pending_tasks.fetch_sub(1);
}

// reference: scheduler.cpp:262-303 — strict priority: drain the real-time queue (preempting first), else
// walk the best-effort queues, re-checking the real-time queue after every step.
void REEFScheduler::loop_body() {
    for (;;) {
        while (!rt_queue->task_queue.empty()) {
            auto rt_task = rt_queue->task_queue.front();
            rt_queue->task_queue.pop();
            execute_rt_task(rt_task);   // preempts the best-effort tasks first (or right after its graph launch)
            last_rt_finish = sclock::now();
            rt_recent = true;
        }
        // A closed-loop real-time client submits its next request a few microseconds after the previous one
        // completes.  Best-effort work started in that gap would be preempted at once, and every launch made
        // for it delays the moment the new request is seen, so the queue is polled for a short grace period
        // before best-effort work is resumed.
        if (rt_recent && rt_grace_us > 0) {
            while (rt_queue->task_queue.empty() && ns_since(last_rt_finish) < (uint64_t)rt_grace_us * 1000ull && !_shutdown.load()) {
            }
            if (!rt_queue->task_queue.empty()) continue;
            rt_recent = false;
        }
        bool interrupted = false;
        uint32_t nq = be_queue_cnt.load();
        for (uint32_t i = 0; i < nq && !interrupted; i++) {
            auto& be_queue = be_queues[i];
            while (!be_queue->task_queue.empty()) {
                if (!rt_queue->task_queue.empty()) { interrupted = true; break; }
                auto be_task = be_queue->task_queue.front();
                execute_be_task(be_task, be_queue);
                if (!rt_queue->task_queue.empty()) { interrupted = true; break; }
                if (be_task->get_state() == TaskState::Finish) {
                    be_queue->task_queue.pop();
                    n_be_tasks++;
                    finish_task(be_task);
                    continue;
                }
                break;
            }
        }
        if (!interrupted) return;
    }
}

// move completed in-flight kernels out of the window; kernel_offset = first kernel not known complete
void REEFScheduler::retire(TaskQueue& q, Task& t) {
    while (!q.inflight.empty()) {
        int pending = 1;
        if (reef_event_query(q.inflight.front().ev, &pending) != REEF_SUCC) {
            // the device reports an error (it stays set for the life of the context): nothing in flight will ever
            // complete.  The window is emptied and the task marked failed, so that it ends instead of waiting forever.
            if (!t.failed) fprintf(stderr, "[reef] best-effort task %u: the device reports an error, the task is failed\n", t.id);
            t.failed = true;
            for (auto& f : q.inflight) q.free_events.push_back(f.ev);
            q.inflight.clear();
            break;
        }
        if (pending) break;
        t.kernel_offset = std::max(t.kernel_offset, q.inflight.front().kernel + 1);
        t.block_offset = 0;
        q.free_events.push_back(q.inflight.front().ev);
        q.inflight.pop_front();
    }
}

void REEFScheduler::reset_preempt_flag_async() { write_flag(0); }

// reference: scheduler.cpp:305-346.  Step 1 raises the flag; step 2 "clears the host queue": the kernels
// not yet handed to the stream simply stay unlaunched, and the task rolls back to the first kernel not
// known to be complete (the reference rolls back conservatively too, scheduler.cpp:320-323; kernels are
// idempotent and the schedules generated here never reuse a buffer, so re-running is exact); step 3 has
// no CUDA form — running blocks leave at their next flag poll.
void REEFScheduler::preempt_reset() {
    auto t_flag = sclock::now();
    if (flag_early) {
        // timeline_padding raised the flag before it launched the real-time graph: the clock runs from there
        t_flag = t_flag_early;
        flag_early = false;
    } else {
        write_flag(1);
    }
    uint32_t nq = be_queue_cnt.load();
    struct Hit {
        std::shared_ptr<Task> task;
        TaskQueue* q;
        reef_event_t last;   // recorded behind the last kernel handed to the stream
    };
    std::vector<Hit> hit;   // tasks that had kernels on their stream
    for (uint32_t i = 0; i < nq; i++) {
        auto& q = *be_queues[i];
        if (q.task_queue.empty()) continue;
        auto task = q.task_queue.front();
        if (task->get_state() == TaskState::Executing && task->all_issued_by_padding) continue;   // nothing to abort
        if (task->get_state() == TaskState::Executing) {
            hit.push_back(Hit{task, &q, q.inflight.empty() ? nullptr : q.inflight.back().ev});
            // An event that fires after the flag went up may belong to a kernel that left early, so the
            // window is not consulted here: kernel_offset stays at what the last poll saw complete.
            q.preempted_kernels.clear();
            for (auto& f : q.inflight) {
                q.preempted_kernels.push_back(f.kernel);
                q.free_events.push_back(f.ev);
            }
            q.inflight.clear();
            task->launch_offset = task->kernel_offset;
            task->state.store(TaskState::Waiting);
            task->preempted = true;
            task->needs_recover = true;
        }
    }
    if (!wait_sync) {
        if (!mapped_flag_host) reef_stream_sync(preempt_stream);
        last_flag_ns = ns_since(t_flag);   // flag raised, queued launches dropped, tasks rolled back
        return;
    }
    last_flag_ns = ns_since(t_flag);
    // Bounded replacement of the reference's reset-until-idle loop (scheduler.cpp:336-345): every hit stream is
    // watched through the event behind its last kernel (those kernels leave at their next flag poll).  The clock
    // stops when all of them are idle; the completion counters, which give the exact restart kernel, are copied on
    // each task's own stream afterwards and read when the task is resumed, off the preemption path.
    bool drained = true;
    for (auto& h : hit) {
        if (h.last == nullptr) continue;
        int pending = 1;
        while (reef_event_query(h.last, &pending) == REEF_SUCC && pending) {
            if (ns_since(t_flag) > 200000000ull) { drained = false; break; }
        }
    }
    const uint64_t ns = ns_since(t_flag);
    if (drained && !hit.empty()) {
        drain_count++;
        drain_ns_sum += ns;
        drain_ns_max = std::max(drain_ns_max, ns);
        if (drain_samples.size() < (1u << 16)) drain_samples.push_back((uint32_t)std::min<uint64_t>(ns, 0xffffffffu));
    }
    for (auto& h : hit) {
        h.task->model->executor.copy_be_kernel_offset(h.q->stream);
        h.q->counters_pending = true;
    }
    if (device_stamps && !hit.empty()) {
        uint64_t first = 0, last = 0;
        if (reef_preempt_stamps_read(&first, &last) == REEF_SUCC && first != 0 && last >= first) {
            dev_count++;
            dev_ns_sum += last - first;
            dev_ns_max = std::max(dev_ns_max, last - first);
        }
    }
}

// reference: scheduler.cpp:348-372
void REEFScheduler::preempt_wait() {
    write_flag(1);
    if (!mapped_flag_host) reef_stream_sync(preempt_stream);
    uint32_t nq = be_queue_cnt.load();
    for (uint32_t i = 0; i < nq; i++) reef_preempt_wait(be_queues[i]->stream, 1000000);
    for (uint32_t i = 0; i < nq; i++) {
        auto& q = *be_queues[i];
        if (q.task_queue.empty()) continue;
        auto task = q.task_queue.front();
        if (task->get_state() != TaskState::Executing || task->all_issued_by_padding) continue;
        for (auto& f : q.inflight) q.free_events.push_back(f.ev);
        q.inflight.clear();
        auto& exe = task->model->executor;
        exe.copy_be_kernel_offset(preempt_stream);
        reef_stream_sync(preempt_stream);
        int k = exe.get_be_kernel_offset(task->kernel_offset);
        task->kernel_offset = std::max(task->kernel_offset, k);
        task->block_offset = 0;
        task->launch_offset = task->kernel_offset;
        task->state.store(TaskState::Waiting);
        task->preempted = true;
        task->needs_recover = true;
    }
}

void REEFScheduler::preempt_be_tasks() {
    if (preempted) return;
    preempted = true;
    auto start = sclock::now();
    switch (mode) {
        case NoPreempt: {
            reef_device_sync();
            uint32_t nq = be_queue_cnt.load();
            for (uint32_t i = 0; i < nq; i++) {
                auto& q = *be_queues[i];
                if (q.task_queue.empty()) continue;
                auto task = q.task_queue.front();
                if (task->get_state() == TaskState::Executing) retire(q, *task);
            }
            break;
        }
        case Reset:
        case REEF:
            preempt_reset();
            break;
        case WaitPreempt:
            preempt_wait();
            break;
        default:
            break;
    }
    // with wait_sync the drain is accounted on its own (drain_*): this figure stays "flag raised and rolled back"
    uint64_t ns = (mode == REEF || mode == Reset) ? last_flag_ns : ns_since(start);
    preempt_count++;
    preempt_latency_sum += ns;
    preempt_latency_max = std::max(preempt_latency_max, ns);
}

int64_t REEFScheduler::avg_preempt_latency() const {
    return preempt_count == 0 ? 0 : (int64_t)(preempt_latency_sum / preempt_count / 1000);
}
uint64_t REEFScheduler::drain_percentile(double q) const {
    if (drain_samples.empty()) return 0;
    std::vector<uint32_t> v(drain_samples);
    size_t k = std::min(v.size() - 1, (size_t)(q * (double)v.size()));
    std::nth_element(v.begin(), v.begin() + k, v.end());
    return v[k];
}
int64_t REEFScheduler::avg_kernel_sel_latency() const {
    return kernel_sel_count == 0 ? 0 : (int64_t)(kernel_sel_latency_sum / kernel_sel_count);
}
REEFScheduler::Stats REEFScheduler::stats() const {
    return Stats{preempt_count, preempt_latency_sum, preempt_latency_max, n_rt_tasks, n_be_tasks,
                 n_be_padded_finish, n_padded_kernels, n_padded_blocks,
                 drain_count, drain_ns_sum, drain_ns_max, dev_count, dev_ns_sum, dev_ns_max,
                 drain_percentile(0.50), drain_percentile(0.99)};
}

bool REEFScheduler::any_be_waiting() {
    uint32_t nq = be_queue_cnt.load();
    for (uint32_t i = 0; i < nq; i++)
        if (!be_queues[i]->task_queue.empty()) return true;
    return false;
}

// reference: scheduler.cpp:451-475
void REEFScheduler::execute_rt_task(std::shared_ptr<Task>& task) {
    task->state.store(TaskState::Executing);
    task->start = std::chrono::system_clock::now();
    auto& exe = task->model->executor;
    bool ok = true;
    if (mode == ScheduleMode::REEF && any_be_waiting() && side_padding_needed(exe)) {
        // the graph goes out first; the best-effort streams are preempted while it starts up
        ok = timeline_padding(task);
        if (reef_stream_sync(rt_queue->stream) != REEF_SUCC) ok = false;
    } else {
        preempt_be_tasks();
        if (mode == ScheduleMode::REEF && any_be_waiting()) {
            ok = dynamic_kernel_padding(task);
            if (reef_stream_sync(rt_queue->stream) != REEF_SUCC) ok = false;
        } else if (rt_graph) {
            auto t0 = sclock::now();
            if (exe.execute_graph(rt_queue->stream) != Status::Succ) {
                err_ = "real-time graph launch failed: " + exe.error();
                fprintf(stderr, "[reef] %s\n", err_.c_str());
                ok = false;
            }
            if (reef_stream_sync(rt_queue->stream) != REEF_SUCC) ok = false;
            if (ok) task->model->add_alone_sample((double)ns_since(t0));
        } else if (exe.execute(rt_queue->stream) != Status::Succ) {
            err_ = "real-time launch failed: " + exe.error();
            ok = false;
        }
    }
    if (device_error_seen("a real-time task")) ok = false;
    task->failed = !ok;
    task->end = std::chrono::system_clock::now();
    n_rt_tasks++;
    finish_task(task);
}

// Best-effort progress after `blocks` logical blocks of the task's current kernel were issued as padding
// (reference: scheduler.cpp:655-672).
void REEFScheduler::advance_padded(Task* be_task, TaskQueue* q, int blocks, bool side_launch,
                                   std::vector<std::shared_ptr<Task>>* complete) {
    auto& be_exe = be_task->model->executor;
    const HybridExecutor::KernelArg& be_args = be_exe.trans_args[be_task->kernel_offset];
    be_task->padding = true;
    be_task->needs_recover = true;   // resuming on its own stream must re-arm the counters
    be_task->block_offset += blocks;
    n_padded_kernels++;
    n_padded_blocks += blocks;
    if (be_task->block_offset < be_args.block_num) return;
    be_task->block_offset = 0;
    be_task->kernel_offset++;
    be_task->launch_offset = be_task->kernel_offset;
    const int n_be = (int)be_exe.num_kernels();
    if (be_task->kernel_offset < n_be) return;
    be_task->padding_to_finish = true;
    if (side_launch) {
        // its last blocks are on the best-effort stream: the task completes when that stream has drained,
        // which the best-effort branch of the loop sees through the window
        reef_event_t ev;
        if (!q->free_events.empty()) {
            ev = q->free_events.back();
            q->free_events.pop_back();
        } else {
            reef_event_create_untimed(&ev);
        }
        reef_event_record(ev, q->stream);
        q->inflight.push_back(InFlight{ev, n_be - 1});
        be_task->all_issued_by_padding = true;
        be_task->state.store(TaskState::Executing);
    } else {
        be_task->kernel_offset = 0;
        complete->push_back(q->task_queue.front());
        q->task_queue.pop();
    }
}

bool REEFScheduler::side_padding_needed(HybridExecutor& rt_exe) {
    if (rt_exe.has_tensor_core_kernels()) return true;
    const uint32_t nq = be_queue_cnt.load();
    for (uint32_t i = 0; i < nq; i++) {
        auto t = be_queues[i]->task_queue.front();
        if (t && t->model->executor.has_tensor_core_kernels()) return true;
    }
    return false;
}

// Dynamic kernel padding when a tensor-core (cluster) kernel is involved on either side.  Such kernels are
// not hosted by the logical-block dispatcher, so the padding is done in space and time by separate launches:
//  * the real-time task replays its CUDA graph on the high-priority stream (full speed, no per-kernel host
//    work).  Its kernels release their successor only after their own dependency wait, so at most two grids
//    of the chain are resident: the running one and the prologue of the next;
//  * while it runs, this thread issues best-effort PIECES (block ranges of a queue's head kernel, whole
//    kernels where they fit) on that queue's own low-priority stream, up to `pad_depth` per stream so that the
//    stream never idles for a launch round trip.  Pieces of one stream run one after the other;
//  * space is accounted in SM slots (two tensor-core CTAs fit one SM): the streams with pieces out may
//    together occupy what the real-time kernels of the next `pad_window` positions leave free (position =
//    elapsed time mapped onto the measured latency profile; reference policy scheduler.cpp:566-595 restated
//    for a free-running real-time stream);
//  * a queue that has issued `pad_quantum` pieces drains and yields, so every best-effort client advances.
// Pieces are launched in the plain flavour (they do not poll the preempt flag; they are short and sized to the
// free slots) and count into the task's completion slots.
static int64_t abs_ns() {
    return std::chrono::duration_cast<std::chrono::nanoseconds>(sclock::now().time_since_epoch()).count();
}
static int slots_of(const HybridExecutor::KernelArg& a, int blocks) {
    // a slot is half an SM: one tensor-core CTA, or four 256-thread logical blocks
    return a.resource.tensor_core ? blocks : (blocks + 3) / 4;
}

bool REEFScheduler::timeline_padding(std::shared_ptr<Task>& rt_task) {
    auto& rt_exe = rt_task->model->executor;
    const size_t n_rt = rt_exe.num_kernels();
    const uint32_t nq = be_queue_cnt.load();
    const int total_slots = 2 * num_sms;
    // cumulative profile time and slot footprint per real-time kernel (kernel k running + prologue of k+1)
    std::vector<double> cum(n_rt + 1, 0.0);
    std::vector<int> part(n_rt + 1, 0);
    for (size_t k = 0; k < n_rt; k++) {
        const HybridExecutor::KernelArg& a = rt_exe.trans_args[k];
        part[k] = std::min(total_slots, slots_of(a, a.block_num));
        cum[k + 1] = cum[k] + std::max(1, a.profile.total_latency);
    }
    const double unit = rt_exe.profile() ? rt_exe.profile()->latency_unit_ns : 1000;
    const double model_ns = rt_exe.profile() && rt_exe.profile()->model_latency > 0
                                ? rt_exe.profile()->model_latency * unit : cum[n_rt] * unit;
    const double scale = cum[n_rt] > 0 ? model_ns / cum[n_rt] : 1.0;   // profile units -> ns of the graph replay

    // The preempt flag goes up first (an asynchronous stream write: about two microseconds of host time), then the
    // graph: the write travels to the device and the best-effort blocks leave while the host is still busy with the
    // graph launch, instead of the write queueing up behind it.
    // With wait_sync the whole switch — flag, queued launches dropped, best-effort streams drained — completes
    // before the real-time task is launched, as in the reference (scheduler.cpp:262-303: preempt_be_tasks, then the
    // task), and its duration is what the drain statistics hold.
    if (wait_sync) {
        preempt_be_tasks();
    } else if (!preempted && (mode == REEF || mode == Reset)) {
        t_flag_early = sclock::now();
        write_flag(1);
        flag_early = true;
    }
    auto t0 = sclock::now();
    if (rt_exe.execute_graph(rt_queue->stream) != Status::Succ) {
        err_ = "real-time graph launch failed: " + rt_exe.error();
        dump_streams_once(err_.c_str());
        fprintf(stderr, "[reef] %s\n", err_.c_str());
        if (flag_early) preempt_be_tasks();   // the flag is up: bring the bookkeeping in line with it
        return false;
    }
    pad_trace.calls++;
    pad_trace.graph_launch_ns += ns_since(t0);
    preempt_be_tasks();   // flag up, tasks rolled back to what is known complete; pieces below are not preemptible
    Model& rt_model = *rt_task->model;
    // Probe windows refresh the baseline: two unpadded windows in a row (the first lets the pieces still out
    // drain, the second is measured), early on and then once per kPadProbePeriod windows.
    const uint32_t wi = rt_model.pad_windows++;
    const uint32_t phase = wi < 16 ? wi % 8 : wi % kPadProbePeriod;
    const bool drain_only = pad_target > 0 && phase == 6;
    const bool probe = pad_target > 0 && phase == 7;
    size_t pos = 0;
    int issued = 0;       // best-effort kernels issued in this window (rate limit)
    for (;;) {
        int busy = 0;
        if (reef_stream_query(rt_queue->stream, &busy) != REEF_SUCC || !busy) break;
        pad_trace.iters++;
        // retire finished pieces; slots still claimed = per stream the widest piece it has out
        int slots_out = 0, active = 0;
        for (uint32_t i = 0; i < nq; i++) {
            auto& q = *be_queues[i];
            while (!q.pad_out.empty()) {
                int pending = 1;
                if (reef_event_query(q.pad_out.front().ev, &pending) != REEF_SUCC) {
                    // device error: the pieces out will never complete; forget them (their tasks fail in retire())
                    for (auto& po : q.pad_out) q.free_events.push_back(po.ev);
                    q.pad_out.clear();
                    break;
                }
                if (pending) break;
                pad_trace.retired++;
                pad_trace.turnaround_ns += abs_ns() - q.pad_out.front().t_launch;
                q.free_events.push_back(q.pad_out.front().ev);
                q.pad_out.pop_front();
            }
            if (q.pad_out.empty()) {
                q.pad_draining = false;
                continue;
            }
            int widest = 0;
            for (auto& po : q.pad_out) widest = std::max(widest, po.slots);
            slots_out += widest;
            active++;
        }
        // estimated position of the real-time stream
        const double now_ns = (double)ns_since(t0);
        while (pos < n_rt && cum[pos + 1] * scale <= now_ns) pos++;
        if (pos >= n_rt) pos = n_rt - 1;   // the replay runs behind the profile: keep padding beside its last kernels
        int rt_slots = 0;
        for (size_t k = pos; k < std::min(n_rt, pos + (size_t)pad_window); k++) rt_slots = std::max(rt_slots, part[k] + part[k + 1]);
        const int free_slots = total_slots - std::min(total_slots, rt_slots) + pad_overcommit - slots_out;

        // rate limit: kernels allowed so far in this window (a small burst lets a whole segment through)
        const int G = HybridExecutor::kPadSegment;
        const bool limited = pad_target > 0;
        const double allowed = limited ? pad_rate * std::min(1.0, now_ns / model_ns) + G : 1e18;
        if (probe || drain_only || issued + 1 > allowed) { pad_trace.no_slot++; continue; }

        auto sel_start = sclock::now();
        bool launched = false;
        for (uint32_t n = 0; n < nq && !launched; n++) {
            const uint32_t qi = (dkp_next_queue + n) % nq;
            auto& q = *be_queues[qi];
            if (q.task_queue.empty()) { pad_trace.q_empty++; continue; }
            if (q.pad_draining) { pad_trace.q_draining++; continue; }
            if ((int)q.pad_out.size() >= pad_depth) { pad_trace.q_full++; continue; }
            auto be_task = q.task_queue.front();
            auto& be_exe = be_task->model->executor;
            if (be_task->kernel_offset >= (int)be_exe.num_kernels()) {
                // fully issued by padding: complete it here as soon as its stream has drained, so that its client
                // can submit the next request while the real-time window is still open
                if (be_task->all_issued_by_padding && be_task->get_state() == TaskState::Executing) {
                    retire(q, *be_task);
                    if (q.inflight.empty()) {
                        if (device_error_seen("a padded best-effort task")) be_task->failed = true;
                        be_task->end = std::chrono::system_clock::now();
                        n_be_padded_finish++;
                        be_task->state.store(TaskState::Finish);
                        be_task->kernel_offset = 0;
                        be_task->block_offset = 0;
                        q.task_queue.pop();
                        n_be_tasks++;
                        finish_task(be_task);
                    }
                }
                pad_trace.q_issued++;
                continue;
            }
            HybridExecutor::KernelArg& be_args = be_exe.trans_args[be_task->kernel_offset];
            int occ = 1;
            if (!be_args.resource.tensor_core) occ = std::max(1, std::min(2, be_args.resource.max_blocks_per_sm));
            const int remaining = be_args.block_num - be_task->block_offset;
            int widest = 0;
            for (auto& po : q.pad_out) widest = std::max(widest, po.slots);
            // slots this stream may use: what it already claims plus what is free
            const int avail = widest + free_slots;
            int blocks = remaining;
            // a whole segment (one graph launch, one event) when the task stands at a segment boundary
            if (be_exe.has_pad_segments() && be_task->block_offset == 0 && be_task->kernel_offset % G == 0 &&
                issued + G <= allowed + G - 1) {
                const int k0 = be_task->kernel_offset, k1 = std::min((int)be_exe.num_kernels(), k0 + G);
                int seg_slots = 0;
                for (int k = k0; k < k1; k++) {
                    seg_slots = std::max(seg_slots, slots_of(be_exe.trans_args[k], be_exe.trans_args[k].block_num));
                    if (pad_piece_bytes > 0 && be_exe.trans_args[k].resource.bytes > pad_piece_bytes) seg_slots = 1 << 30;   // goes out in ranges
                }
                if (seg_slots <= avail && (pad_piece_cap <= 0 || seg_slots <= pad_piece_cap)) {
                    if (be_task->start.time_since_epoch().count() == 0) be_task->start = std::chrono::system_clock::now();
                    if (be_exe.launch_pad_segment(k0 / G, q.stream) != Status::Succ) {
                        // the task is failed and taken off its queue: the window goes on with the other queues
                        // instead of retrying the same failing launch until the real-time stream is idle
                        fail_be_task(q, be_task, "padding segment launch failed: " + be_exe.error());
                        continue;
                    }
                    reef_event_t ev;
                    if (!q.free_events.empty()) {
                        ev = q.free_events.back();
                        q.free_events.pop_back();
                    } else {
                        reef_event_create_untimed(&ev);
                    }
                    reef_event_record(ev, q.stream);
                    if (q.pad_out.empty()) {
                        q.pad_quantum_left = pad_quantum;
                        dkp_next_queue = (qi + 1) % nq;
                    }
                    q.pad_out.push_back(PadOut{ev, seg_slots, abs_ns()});
                    q.pad_quantum_left -= k1 - k0;
                    if (q.pad_quantum_left <= 0) q.pad_draining = true;
                    launched = true;
                    issued += k1 - k0;
                    pad_trace.segments++;
                    for (int k = k0; k < k1; k++) advance_padded(be_task.get(), &q, be_exe.trans_args[k].block_num, true, nullptr);
                    continue;
                }
            }
            const double kbytes = be_args.resource.bytes;
            if (pad_piece_bytes > 0 && kbytes > pad_piece_bytes && be_args.block_num > 1) {
                // a kernel that streams hundreds of megabytes (VGG-16's first dense layer: 411 MB) would hold
                // the whole HBM bandwidth for its duration: it goes out in block ranges of bounded traffic, which
                // the rate limit then spreads over the window
                int cap_blocks = (int)(be_args.block_num * (pad_piece_bytes / kbytes));
                cap_blocks -= cap_blocks % be_args.granularity;
                cap_blocks = std::max(cap_blocks, be_args.granularity);
                blocks = std::min(remaining, cap_blocks);
                if (slots_of(be_args, blocks) > avail && (active > 0 || avail <= 0)) { pad_trace.q_nofit++; continue; }
            } else if (pad_piece_cap > 0 && slots_of(be_args, blocks) > pad_piece_cap && avail >= pad_piece_cap) {
                // a wide kernel goes out in block ranges of at most the cap: it then shares fewer SMs with the
                // real-time kernels at any one time
                blocks = be_args.resource.tensor_core ? pad_piece_cap : pad_piece_cap * 4;
                blocks -= blocks % be_args.granularity;
                if (blocks <= 0) blocks = be_args.granularity;
                blocks = std::min(blocks, remaining);
            } else if (slots_of(be_args, blocks) > avail) {
                // the kernel does not fit whole: a partial piece only when nothing else is out (progress)
                if (active > 0 || avail <= 0) { pad_trace.q_nofit++; continue; }
                blocks = be_args.resource.tensor_core ? avail : avail * 4;
                blocks -= blocks % be_args.granularity;
                if (blocks <= 0) continue;
            }
            if (be_task->start.time_since_epoch().count() == 0) be_task->start = std::chrono::system_clock::now();
            if (be_exe.launch_pad_piece(be_task->kernel_offset, be_task->block_offset, blocks, occ, q.stream) != Status::Succ) {
                fail_be_task(q, be_task, "padding piece launch failed: " + be_exe.error());
                continue;
            }
            reef_event_t ev;
            if (!q.free_events.empty()) {
                ev = q.free_events.back();
                q.free_events.pop_back();
            } else {
                reef_event_create_untimed(&ev);
            }
            reef_event_record(ev, q.stream);
            if (q.pad_out.empty()) {
                q.pad_quantum_left = pad_quantum;   // takes a place: the next free place goes to a later queue
                dkp_next_queue = (qi + 1) % nq;
            }
            q.pad_out.push_back(PadOut{ev, slots_of(be_args, blocks), abs_ns()});
            if (--q.pad_quantum_left <= 0) q.pad_draining = true;
            launched = true;
            issued++;
            pad_trace.singles++;
            advance_padded(be_task.get(), &q, blocks, true, nullptr);
        }
        kernel_sel_count++;
        kernel_sel_latency_sum += ns_since(sel_start);
        if (launched) {
            pad_trace.launched++;
            pad_trace.launch_ns += ns_since(sel_start);
        } else if (free_slots <= 0) {
            pad_trace.no_sms++;
        } else {
            pad_trace.no_queue++;
        }
    }
    const uint64_t window_ns = ns_since(t0);
    pad_trace.window_ns += window_ns;
    if (probe) {
        rt_model.add_alone_sample((double)window_ns);
    } else if (drain_only) {
    } else if (pad_target > 0 && model_ns > 0) {
        // slowdown controller: one multiplicative step per window on the kernel rate
        const double baseline = rt_model.alone_ns() > 0.0 ? rt_model.alone_ns() : 1.02 * model_ns;
        const double ratio = (double)window_ns / baseline;
        pad_ratio_ema = pad_ratio_ema == 0.0 ? ratio : 0.8 * pad_ratio_ema + 0.2 * ratio;
        if (pad_ratio_ema > 1.0 + pad_target) pad_rate *= 0.97;
        else pad_rate *= 1.015;
        pad_rate = std::max(4.0, std::min(4096.0, pad_rate));
    }
    return true;
}

// reference: scheduler.cpp:477-683.  Per real-time kernel: pick a best-effort queue whose head kernel can
// share the grid (occupancy) and whose one-wave latency fits inside the real-time kernel (profile), size its
// block count from the SMs the real-time kernel leaves free, launch ONE persistent dispatcher grid for both,
// and advance the best-effort task's (kernel_offset, block_offset).  Used when every kernel on both sides is a
// logical-block family.  Queues are tried round-robin (the reference always starts at queue 0,
// scheduler.cpp:533, which starves the later clients under a busy real-time client).
bool REEFScheduler::dynamic_kernel_padding(std::shared_ptr<Task>& rt_task) {
    auto& rt_exe = rt_task->model->executor;
    bool ok = true;
    std::vector<std::shared_ptr<Task>> complete_be_tasks;
    auto current_time_point = std::chrono::system_clock::now();
    const uint32_t nq = be_queue_cnt.load();
    const int64_t unit = rt_exe.profile() ? rt_exe.profile()->latency_unit_ns : 1000;

    for (size_t i = 0; i < rt_exe.num_kernels(); i++) {
        auto sel_start = sclock::now();
        HybridExecutor::KernelArg& rt_args = rt_exe.trans_args[i];
        const int required_occupancy = rt_args.min_occupancy;
        const int rt_latency = std::max(1, rt_args.profile.total_latency);
        const int logical_layers = std::max(1, align_up<int>(rt_args.block_num, num_sms) / num_sms);

        Task* final_be_task = nullptr;
        TaskQueue* final_queue = nullptr;
        int final_occupancy = required_occupancy, final_be_block_num = 0, sm_partition = num_sms;

        for (uint32_t n = 0; n < nq; n++) {
            const uint32_t qi = (dkp_next_queue + n) % nq;
            auto& be_queue = be_queues[qi]->task_queue;
            if (be_queue.empty()) continue;
            auto be_task = be_queue.front();
            auto& be_exe = be_task->model->executor;
            if (be_task->kernel_offset >= (int)be_exe.num_kernels()) continue;
            HybridExecutor::KernelArg& be_args = be_exe.trans_args[be_task->kernel_offset];

            // 1. occupancy both kernels can run at inside one grid
            int merged_occupancy = std::min(rt_args.resource.max_blocks_per_sm, be_args.resource.max_blocks_per_sm);
            if (merged_occupancy < required_occupancy) continue;
            // 2. latency profile decides the best-effort occupancy
            int be_occupancy = 0;
            for (int j = merged_occupancy - 1; j >= 0; j--) {
                if ((int)be_args.profile.latency.size() <= j) continue;
                if (be_args.profile.latency[j] <= rt_latency) {
                    be_occupancy = j + 1;
                    break;
                }
            }
            if (be_occupancy == 0) continue;
            // 3. partition and block budget
            int part = align_up(rt_args.block_num, logical_layers) / logical_layers;
            if (part >= num_sms) continue;   // the real-time kernel fills every SM: nothing to pad
            int be_latency_per_iter = std::max(1, be_args.profile.latency[be_occupancy - 1]);
            int be_iters = std::max(1, rt_latency / be_latency_per_iter);
            int blocks = (num_sms - part) * be_iters * be_occupancy;
            blocks = std::min(blocks, be_args.block_num - be_task->block_offset);
            if (blocks <= 0) continue;

            sm_partition = part;
            final_occupancy = std::max(required_occupancy, be_occupancy);
            final_be_block_num = blocks;
            final_be_task = be_task.get();
            final_queue = be_queues[qi].get();
            dkp_next_queue = (qi + 1) % nq;
            break;
        }
        kernel_sel_count++;
        kernel_sel_latency_sum += ns_since(sel_start);

        Status lst;
        if (final_be_task == nullptr) {
            lst = rt_exe.launch_dispatch((int)i, nullptr, 0, 0, 0, num_sms, required_occupancy, rt_queue->stream);
        } else {
            if (final_be_task->start.time_since_epoch().count() == 0) final_be_task->start = current_time_point;
            lst = rt_exe.launch_dispatch((int)i, &final_be_task->model->executor, final_be_task->kernel_offset,
                                         final_be_task->block_offset, final_be_block_num, sm_partition, final_occupancy,
                                         rt_queue->stream, nullptr);
        }
        if (lst != Status::Succ) {
            // the real-time task cannot complete: stop here, the best-effort task keeps its position
            err_ = "dispatcher launch failed: " + rt_exe.error();
            fprintf(stderr, "[reef] %s\n", err_.c_str());
            ok = false;
            break;
        }
        current_time_point += std::chrono::nanoseconds((int64_t)rt_args.profile.total_latency * unit);
        if (final_be_task != nullptr) {
            advance_padded(final_be_task, final_queue, final_be_block_num, false, &complete_be_tasks);
            if (final_be_task->padding_to_finish) final_be_task->end = current_time_point;
        }
    }
    if (!complete_be_tasks.empty()) {
        // their last blocks ran inside the dispatcher grids above: complete once the stream drained
        reef_stream_sync(rt_queue->stream);
        for (auto& t : complete_be_tasks) {
            n_be_tasks++;
            n_be_padded_finish++;
            finish_task(t);
        }
    }
    return ok;
}

// reference: scheduler.cpp:685-740
void REEFScheduler::execute_be_task(std::shared_ptr<Task>& task, std::shared_ptr<TaskQueue>& tqueue) {
    auto& exe = task->model->executor;
    const int num_kernels = (int)exe.num_kernels();
    TaskState st = task->get_state();
    if (st == TaskState::Finish) return;

    if (st == TaskState::Init || st == TaskState::Waiting) {
        if (st == TaskState::Init) task->start = std::chrono::system_clock::now();
        if (preempted) {
            reset_preempt_flag_async();
            preempted = false;
            reef_stream_sync(preempt_stream);
        }
        if (tqueue->counters_pending) {
            // a preemption with wait_sync left a copy of the completion counters on this stream: the exact restart
            // kernel is the first one whose counter is short of its block count
            tqueue->counters_pending = false;
            reef_stream_sync(tqueue->stream);
            int k = exe.get_be_kernel_offset(task->kernel_offset);
            if (k > task->kernel_offset) {
                task->kernel_offset = k;
                task->block_offset = 0;
            }
            task->launch_offset = task->kernel_offset;
        }
        if (task->needs_recover) {
            // Leftovers of preempted launches and padded pieces may still be on the stream.  Nothing waits for
            // them: the counter reset and the relaunch below are ordered behind them by the stream, and every
            // buffer from the resume point on is recomputed in order.
            for (auto& f : tqueue->inflight) tqueue->free_events.push_back(f.ev);
            tqueue->inflight.clear();
            task->needs_recover = false;
        }
        if (task->kernel_offset >= num_kernels) {
            task->kernel_offset = 0;
            task->block_offset = 0;
            task->end = std::chrono::system_clock::now();
            task->state.store(TaskState::Finish);
            return;
        }
        // completion counters restart from the resume point (a kernel half done by padding is re-run whole)
        task->block_offset = 0;
        task->launch_offset = task->kernel_offset;
        exe.reset_task_slots(tqueue->stream, task->kernel_offset);
        task->state.store(TaskState::Executing);
    } else {
        retire(*tqueue, *task);
        if (task->launch_offset >= num_kernels && tqueue->inflight.empty()) {
            if (device_error_seen("a best-effort task")) task->failed = true;
            task->end = std::chrono::system_clock::now();
            if (task->all_issued_by_padding) n_be_padded_finish++;
            task->state.store(TaskState::Finish);
            task->kernel_offset = 0;
            task->block_offset = 0;
            return;
        }
    }

    // feed the window
    while (task->launch_offset < num_kernels && (int)tqueue->inflight.size() < be_stream_device_queue_cap) {
        int k = task->launch_offset;
        if (exe.launch_preempt_kernel(k, tqueue->stream) != Status::Succ) {
            // fail the task rather than spin on it: Finish with the failed mark (wait_task returns Fail)
            err_ = "best-effort launch failed: " + exe.error();
            dump_streams_once(err_.c_str());
            fprintf(stderr, "[reef] %s\n", err_.c_str());
            for (auto& f : tqueue->inflight) tqueue->free_events.push_back(f.ev);
            tqueue->inflight.clear();
            task->failed = true;
            task->kernel_offset = 0;
            task->block_offset = 0;
            task->end = std::chrono::system_clock::now();
            task->state.store(TaskState::Finish);
            return;
        }
        reef_event_t ev;
        if (!tqueue->free_events.empty()) {
            ev = tqueue->free_events.back();
            tqueue->free_events.pop_back();
        } else {
            reef_event_create_untimed(&ev);
        }
        reef_event_record(ev, tqueue->stream);
        tqueue->inflight.push_back(InFlight{ev, k});
        task->launch_offset = k + 1;
        if (!rt_queue->task_queue.empty() && (mode == REEF || mode == Reset)) return;   // preempt during launch
    }
}

}  // namespace server
}  // namespace reef
