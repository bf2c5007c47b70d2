#include "scheduler.h"

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
    for (auto& pp : pad_pieces) reef_event_create(&pp.ev);
    if (const char* v = getenv("REEF_PAD_INFLIGHT")) set_pad_limits(atoi(v), pad_overcommit_sms);
    if (const char* v = getenv("REEF_PAD_OVERCOMMIT")) set_pad_limits(pad_inflight_max, atoi(v));
    if (const char* v = getenv("REEF_PAD_WINDOW")) set_pad_window(atoi(v));
}

REEFScheduler::~REEFScheduler() {
    if (scheduler && scheduler->joinable()) shutdown();
    reef_gpu_init(device);
    reef_device_sync();
    model_pool.clear();
    for (auto& q : be_queues)
        if (q) {
            for (auto& f : q->inflight) reef_event_destroy(f.ev);
            for (auto e : q->free_events) reef_event_destroy(e);
            if (q->stream) reef_stream_destroy(q->stream);
        }
    if (rt_queue && rt_queue->stream) reef_stream_destroy(rt_queue->stream);
    for (auto& pp : pad_pieces)
        if (pp.ev) reef_event_destroy(pp.ev);
    if (preempt_stream) reef_stream_destroy(preempt_stream);
    if (preempt_flag) reef_free(preempt_flag);
}

Status REEFScheduler::create_task_queue(std::shared_ptr<TaskQueue>& ret, bool rt) {
    executor::GPUStream_t stream;
    GPU_RETURN_STATUS(reef_gpu_init(device));
    GPU_RETURN_STATUS(reef_stream_create(&stream, rt ? 1 : 0));
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
    // spin briefly (a real-time inference is tens of microseconds), then block on the task's condvar
    auto t0 = sclock::now();
    while (task->state.load(std::memory_order_acquire) != TaskState::Finish) {
        if (ns_since(t0) > 2000000ull) break;
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
    return Status::Succ;
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
            preempt_be_tasks();
            auto rt_task = rt_queue->task_queue.front();
            rt_queue->task_queue.pop();
            execute_rt_task(rt_task);
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
        if (reef_event_query(q.inflight.front().ev, &pending) != REEF_SUCC || pending) break;
        t.kernel_offset = std::max(t.kernel_offset, q.inflight.front().kernel + 1);
        t.block_offset = 0;
        q.free_events.push_back(q.inflight.front().ev);
        q.inflight.pop_front();
    }
}

void REEFScheduler::reset_preempt_flag_async() { reef_write32_async(preempt_stream, preempt_flag, 0); }

// reference: scheduler.cpp:305-346.  Step 1 raises the flag; step 2 "clears the host queue": the kernels
// not yet handed to the stream simply stay unlaunched, and the task rolls back to the first kernel not
// known to be complete (the reference rolls back conservatively too, scheduler.cpp:320-323; kernels are
// idempotent and the schedules generated here never reuse a buffer, so re-running is exact); step 3 has
// no CUDA form — running blocks leave at their next flag poll.
void REEFScheduler::preempt_reset() {
    reef_write32_async(preempt_stream, preempt_flag, 1);
    uint32_t nq = be_queue_cnt.load();
    std::vector<std::shared_ptr<Task>> hit;   // tasks that had kernels on their stream
    for (uint32_t i = 0; i < nq; i++) {
        auto& q = *be_queues[i];
        if (q.task_queue.empty()) continue;
        auto task = q.task_queue.front();
        if (task->get_state() == TaskState::Executing && task->all_issued_by_padding) continue;   // nothing to abort
        if (task->get_state() == TaskState::Executing) {
            hit.push_back(task);
            // An event that fires after the flag went up may belong to a kernel that left early, so the
            // window is not consulted here: kernel_offset stays at what the last poll saw complete.
            for (auto& f : q.inflight) q.free_events.push_back(f.ev);
            q.inflight.clear();
            task->launch_offset = task->kernel_offset;
            task->state.store(TaskState::Waiting);
            task->preempted = true;
            task->needs_recover = true;
        }
    }
    reef_stream_sync(preempt_stream);
    if (wait_sync) {
        // bounded replacement of the reference's reset-until-idle loop (scheduler.cpp:336-345), then the
        // exact restart point from the completion counters
        for (uint32_t i = 0; i < nq; i++) reef_preempt_wait(be_queues[i]->stream, 200000);
        for (auto& task : hit) {
            auto& exe = task->model->executor;
            exe.copy_be_kernel_offset(preempt_stream);
            reef_stream_sync(preempt_stream);
            int k = exe.get_be_kernel_offset(task->kernel_offset);
            if (k > task->kernel_offset) {
                task->kernel_offset = k;
                task->block_offset = 0;
            }
            task->launch_offset = task->kernel_offset;
        }
    }
}

// reference: scheduler.cpp:348-372
void REEFScheduler::preempt_wait() {
    reef_write32_async(preempt_stream, preempt_flag, 1);
    reef_stream_sync(preempt_stream);
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
    uint64_t ns = ns_since(start);
    preempt_count++;
    preempt_latency_sum += ns;
    preempt_latency_max = std::max(preempt_latency_max, ns);
}

int64_t REEFScheduler::avg_preempt_latency() const {
    return preempt_count == 0 ? 0 : (int64_t)(preempt_latency_sum / preempt_count / 1000);
}
int64_t REEFScheduler::avg_kernel_sel_latency() const {
    return kernel_sel_count == 0 ? 0 : (int64_t)(kernel_sel_latency_sum / kernel_sel_count);
}
REEFScheduler::Stats REEFScheduler::stats() const {
    return Stats{preempt_count, preempt_latency_sum, preempt_latency_max, n_rt_tasks, n_be_tasks,
                 n_be_padded_finish, n_padded_kernels, n_padded_blocks};
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
    if (mode == ScheduleMode::REEF && any_be_waiting()) {
        if (side_padding_needed(exe)) timeline_padding(task);
        else dynamic_kernel_padding(task);
        reef_stream_sync(rt_queue->stream);
    } else if (rt_graph) {
        if (exe.execute_graph(rt_queue->stream) != Status::Succ) {
            err_ = "real-time graph launch failed: " + exe.error();
            fprintf(stderr, "[reef] %s\n", err_.c_str());
        }
        reef_stream_sync(rt_queue->stream);
    } else {
        exe.execute(rt_queue->stream);
    }
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
            reef_event_create(&ev);
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
//  * the real-time task replays its CUDA graph on the high-priority stream (full speed, no per-kernel host work);
//  * while it runs, this thread issues best-effort PIECES — block ranges of the head kernel of a best-effort
//    queue, round-robin over the queues — on that queue's own low-priority stream, one piece in flight at a time;
//  * a piece is sized from the SMs the real-time kernels of the next `pad_window` positions leave free
//    (position = elapsed time mapped onto the measured latency profile, reference policy scheduler.cpp:566-595
//    restated for a free-running real-time stream), whole clusters only.
// Pieces are launched in the plain flavour (they do not poll the preempt flag; they are short and sized to the
// idle SMs) and count into the task's completion slots.
void REEFScheduler::timeline_padding(std::shared_ptr<Task>& rt_task) {
    auto& rt_exe = rt_task->model->executor;
    const size_t n_rt = rt_exe.num_kernels();
    const uint32_t nq = be_queue_cnt.load();
    // cumulative profile time and SM footprint per real-time kernel
    std::vector<double> cum(n_rt + 1, 0.0);
    std::vector<int> part(n_rt, 0);
    for (size_t k = 0; k < n_rt; k++) {
        const HybridExecutor::KernelArg& a = rt_exe.trans_args[k];
        const int layers = std::max(1, align_up<int>(a.block_num, num_sms) / num_sms);
        part[k] = std::min(num_sms, align_up(a.block_num, layers) / layers);
        cum[k + 1] = cum[k] + std::max(1, a.profile.total_latency);
    }
    const double unit = rt_exe.profile() ? rt_exe.profile()->latency_unit_ns : 1000;
    const double model_ns = rt_exe.profile() && rt_exe.profile()->model_latency > 0
                                ? rt_exe.profile()->model_latency * unit : cum[n_rt] * unit;
    const double scale = cum[n_rt] > 0 ? model_ns / cum[n_rt] : 1.0;   // profile units -> ns of the graph replay

    auto t0 = sclock::now();
    if (rt_exe.execute_graph(rt_queue->stream) != Status::Succ) {
        err_ = "real-time graph launch failed: " + rt_exe.error();
        fprintf(stderr, "[reef] %s\n", err_.c_str());
        return;
    }
    size_t pos = 0;
    for (;;) {
        int busy = 0;
        if (reef_stream_query(rt_queue->stream, &busy) != REEF_SUCC || !busy) break;
        // retire finished pieces; count what is still out
        int inflight = 0, sms_out = 0, slot = -1;
        uint32_t busy_queues = 0;
        for (int p = 0; p < pad_inflight_max; p++) {
            PadPiece& pp = pad_pieces[p];
            if (pp.pending) {
                int pending = 1;
                if (reef_event_query(pp.ev, &pending) == REEF_SUCC && !pending) pp.pending = false;
            }
            if (pp.pending) {
                inflight++;
                sms_out += pp.sms;
                busy_queues |= 1u << pp.queue;
            } else if (slot < 0) {
                slot = p;
            }
        }
        if (slot < 0) continue;
        // estimated position of the real-time stream
        const double now_ns = (double)ns_since(t0);
        while (pos < n_rt && cum[pos + 1] * scale <= now_ns) pos++;
        if (pos >= n_rt) continue;   // in the tail: let the task finish
        int part_w = 0;
        for (size_t k = pos; k < std::min(n_rt, pos + (size_t)pad_window); k++) part_w = std::max(part_w, part[k]);
        const int free_sms = num_sms - part_w + pad_overcommit_sms - sms_out;
        if (free_sms <= 0) continue;

        auto sel_start = sclock::now();
        for (uint32_t n = 0; n < nq; n++) {
            const uint32_t qi = (dkp_next_queue + n) % nq;
            if (busy_queues & (1u << qi)) continue;   // one piece per best-effort stream: pieces of a task stay ordered
            auto& q = *be_queues[qi];
            if (q.task_queue.empty()) continue;
            auto be_task = q.task_queue.front();
            auto& be_exe = be_task->model->executor;
            if (be_task->kernel_offset >= (int)be_exe.num_kernels()) continue;   // fully issued, draining
            HybridExecutor::KernelArg& be_args = be_exe.trans_args[be_task->kernel_offset];
            int occ = 1;
            if (!be_args.resource.tensor_core) occ = std::max(1, std::min(2, be_args.resource.max_blocks_per_sm));
            int blocks = std::min(free_sms * occ, be_args.block_num - be_task->block_offset);
            blocks -= blocks % be_args.granularity;
            if (blocks <= 0) continue;
            if (be_task->start.time_since_epoch().count() == 0) be_task->start = std::chrono::system_clock::now();
            if (be_exe.launch_pad_piece(be_task->kernel_offset, be_task->block_offset, blocks, occ, q.stream) != Status::Succ) {
                err_ = be_exe.error();
                break;
            }
            PadPiece& pp = pad_pieces[slot];
            reef_event_record(pp.ev, q.stream);
            pp.pending = true;
            pp.sms = (blocks + occ - 1) / occ;
            pp.queue = qi;
            advance_padded(be_task.get(), &q, blocks, true, nullptr);
            dkp_next_queue = (qi + 1) % nq;
            break;
        }
        kernel_sel_count++;
        kernel_sel_latency_sum += ns_since(sel_start);
    }
}

// reference: scheduler.cpp:477-683.  Per real-time kernel: pick a best-effort queue whose head kernel can
// share the grid (occupancy) and whose one-wave latency fits inside the real-time kernel (profile), size its
// block count from the SMs the real-time kernel leaves free, launch ONE persistent dispatcher grid for both,
// and advance the best-effort task's (kernel_offset, block_offset).  Used when every kernel on both sides is a
// logical-block family.  Queues are tried round-robin (the reference always starts at queue 0,
// scheduler.cpp:533, which starves the later clients under a busy real-time client).
void REEFScheduler::dynamic_kernel_padding(std::shared_ptr<Task>& rt_task) {
    auto& rt_exe = rt_task->model->executor;
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

        if (final_be_task == nullptr) {
            rt_exe.launch_dispatch((int)i, nullptr, 0, 0, 0, num_sms, required_occupancy, rt_queue->stream);
        } else {
            if (final_be_task->start.time_since_epoch().count() == 0) final_be_task->start = current_time_point;
            rt_exe.launch_dispatch((int)i, &final_be_task->model->executor, final_be_task->kernel_offset,
                                   final_be_task->block_offset, final_be_block_num, sm_partition, final_occupancy,
                                   rt_queue->stream, nullptr);
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
        if (task->needs_recover) {
            // leftovers of the preempted launches have left the stream long ago; bounded wait all the same
            reef_preempt_wait(tqueue->stream, 200000);
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
            err_ = exe.error();
            task->end = std::chrono::system_clock::now();
            task->state.store(TaskState::Finish);   // fail the task rather than spin on it
            return;
        }
        reef_event_t ev;
        if (!tqueue->free_events.empty()) {
            ev = tqueue->free_events.back();
            tqueue->free_events.pop_back();
        } else {
            reef_event_create(&ev);
        }
        reef_event_record(ev, tqueue->stream);
        tqueue->inflight.push_back(InFlight{ev, k});
        task->launch_offset = k + 1;
        if (!rt_queue->task_queue.empty() && (mode == REEF || mode == Reset)) return;   // preempt during launch
    }
}

}  // namespace server
}  // namespace reef
