// REEFScheduler: model pool, one real-time queue and up to 32 best-effort queues, one scheduler
// thread per GPU, reset-style preemption and dynamic kernel padding
// (reference: src/reef/server/scheduler.{h,cpp}; public surface scheduler.h:68-126).
//
// What changes on CUDA:
//  * hipStreamCreateWithWindowSize / hipStreamClearQueue (reference: scheduler.cpp:45-50,316):
//    CUDA cannot bound or clear a stream's queue, so each best-effort queue keeps at most
//    `be_stream_device_queue_cap` kernels in flight (tracked with events) and the rest of the
//    task stays on the host, where "clearing" is free.
//  * hipResetWavefronts (reference: scheduler.cpp:332-333): running best-effort blocks cannot be
//    killed; they leave at their next preempt-flag poll (block entry and loop heads).
//  * merge_framework_N proxy kernels (reference: scheduler.cpp:613-649): one persistent dispatcher
//    kernel (reef_dispatch).
#pragma once
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "common.h"
#include "executor.h"
#include "threadsafe_queue.h"

namespace reef {
namespace server {

class REEFScheduler {
    struct Model;

public:
    typedef uint32_t ModelID;
    typedef uint32_t QueueID;
    typedef uint32_t TaskID;

    enum ScheduleMode {
        NoPreempt,    // real-time waits for running best-effort kernels
        MultiStream,  // plain concurrent streams
        WaitPreempt,  // flag + wait for the device to drain, progress from completion counters
        REEF,         // flag preemption + dynamic kernel padding
        Reset         // flag preemption without padding
    };
    enum TaskQueueType { RealTimeQueue, BestEffortQueue };
    enum TaskState { Init, Waiting, Executing, Finish };

    struct Task {
        friend class REEFScheduler;

    private:
        std::shared_ptr<Model> model;
        QueueID qid;
        TaskID id;
        std::atomic<int> state;
        int launch_offset;   // next kernel to hand to the stream
        int kernel_offset;   // first kernel not known to be complete
        int block_offset;    // logical blocks of kernel_offset already done by padding
        std::mutex mtx;
        std::condition_variable cv;
        std::chrono::system_clock::time_point submit, start, end;
        bool preempted;
        bool padding;
        bool padding_to_finish;
        bool needs_recover;
        bool all_issued_by_padding;   // every kernel went out as padding; the stream only has to drain
        bool failed;                  // a launch failed or a device-side wait expired: the output is not valid

    public:
        bool is_preempted() const { return preempted; }
        bool is_padded() const { return padding; }
        bool is_padded_to_complete() const { return padding_to_finish; }
        // The reference aborts the process on a GPU error (hip_impl.h:34-41); here the task ends in Finish with
        // this mark and wait_task returns Status::Fail, so a client never mistakes stale output for a result.
        bool is_failed() const { return failed; }
        TaskState get_state() const { return (TaskState)state.load(); }
        std::vector<std::chrono::system_clock::time_point> get_timestamp() const { return {submit, start, end}; }
    };

    explicit REEFScheduler(ScheduleMode _mode = ScheduleMode::REEF, int device = 0);
    ~REEFScheduler();

    Status load_model(const std::string& model_dir, const std::string& model_name, ModelID& mid);
    Status load_model(const std::string& rt_co_path, const std::string& be_co_path, const std::string& json_path,
                      const std::string& profile_path, const std::string& param_path, ModelID& mid);
    Status create_queue(const TaskQueueType& qtp, QueueID& qid);
    Status bind_model_queue(const QueueID& qid, const ModelID& mid);
    Status get_data_size(ModelID mid, const std::string& name, size_t& size);
    Status set_input(ModelID mid, const void* data, size_t len, const std::string& name = "data");
    Status get_output(ModelID mid, void* data, size_t len, const std::string& name = "output");
    Status new_task(const ModelID& mid, TaskID& tid);
    Status wait_task(TaskID tid);
    Status get_task(TaskID tid, std::shared_ptr<Task>& t);
    ScheduleMode sche_mode() const { return mode; }
    // wait_sync: a preemption also waits (bounded) until the best-effort streams have drained and reads the completion
    // counters for the exact restart kernel (reference: scheduler.cpp:336-345, the reset-until-idle loop)
    void set_wait_sync(bool value) { wait_sync = value; }
    // The preempt flag lives in device memory and is raised by an ordered 32-bit stream write (GPUWriteValue32Async,
    // reference: hip_impl.h:20).  With the mapped flag it lives in pinned host memory instead and is raised by a plain
    // host store; every device-side poll then crosses PCIe.  Call before the first load_model.
    Status use_mapped_flag();
    // Spatial partition (before any queue exists): best-effort streams get `be_sms` SMs of their own, the real-time
    // stream the rest; flags as reef_partition_create.  rt_sms / be_sms report what the driver provisioned.
    Status set_sm_partition(int be_sms, int flags, int* rt_sms_out, int* be_sms_out);
    // Records, on the device's own clock, when the flag was first seen by a best-effort block and when the last one
    // left (measurement; read once per preemption after the drain, so it implies wait_sync).
    Status set_device_stamps(bool on);
    // CPU placement of the threads that serve this GPU (no reference counterpart; one scheduler per GPU on a shared
    // host): the scheduler thread is pinned to `first_cpu`, a real-time closed-loop client of reef_run_clients to
    // first_cpu + 1, best-effort clients to the rest of [first_cpu, first_cpu + n_cpus).  n_cpus < 3 pins nothing.
    void set_cpu_slice(int first_cpu, int n_cpus) { cpu_first = first_cpu; cpu_count = n_cpus; }
    void cpu_slice(int* first_cpu, int* n_cpus) const { *first_cpu = cpu_first; *n_cpus = cpu_count; }
    bool is_realtime_model(ModelID mid) const { return mid < model_pool_size.load() && model_pool[mid]->qid == rt_queue_id; }
    void set_be_stream_cap(int value) { be_stream_device_queue_cap = value < 1 ? 1 : value; }
    // real-time tasks that find no best-effort work replay a CUDA graph of the model (default on)
    void set_rt_graph(bool value) { rt_graph = value; }
    // models bound to the real-time queue run their tensor-core layers as persistent chains (executor.h) of this
    // many clusters; 0 = the library's default size, -1 = off (one launch per layer)
    void set_rt_chains(int clusters) { rt_chain_clusters = clusters; }
    // Timeline padding (tensor-core models).  Unit = one SM slot: an SM holds two tensor-core CTAs.
    //  window      real-time kernels ahead of the estimated position whose footprint bounds the padding
    //  depth       padded pieces queued per best-effort stream (hides the launch-to-completion latency)
    //  overcommit  slots best-effort pieces may claim beyond what the real-time kernels leave free (default 100:
    //              the parked prologue of the next real-time kernel is counted as a full footprint, but it
    //              only needs its slots by the time the running kernel ends)
    //  quantum     pieces after which a best-effort queue drains and yields its place to the next queue
    void set_pad_window(int value) { pad_window = value < 1 ? 1 : value; }
    void set_pad_limits(int depth, int overcommit_slots, int quantum) {
        pad_depth = depth < 1 ? 1 : depth;
        pad_overcommit = overcommit_slots;
        pad_quantum = quantum < 1 ? 1 : quantum;
    }
    // Padding is throttled so that a padded real-time task takes on average (1 + value) times its latency alone
    // (the tail follows: the 99th percentile sits two to three percent above the mean slowdown).  What a best-effort
    // tensor-core kernel costs the real-time chain is close to a fixed time per kernel (0.8-1.0 us on B200: about a
    // tenth of the time the kernel is resident), whatever its launch plan, so the throttle is a rate: at most `pad_rate` best-effort kernels per real-time window, spread evenly
    // over it; after every window the rate moves a step down when the smoothed window-time / baseline ratio is
    // above the target and a smaller step up when it is below.  (Regulating a tail statistic of the last 32
    // windows instead made the rate oscillate and gave a wider tail for the same best-effort throughput.)
    // 0 switches the controller off (no rate limit).
    void set_pad_slowdown_target(double value) { pad_target = value < 0 ? 0 : value; }
    // after a real-time task, poll its queue this long before best-effort work is resumed (0: not at all)
    void set_rt_grace_us(int value) { rt_grace_us = value < 0 ? 0 : value; }
    Status run();
    Status shutdown();

    int64_t avg_preempt_latency() const;       // microseconds, as in the reference
    int64_t avg_kernel_sel_latency() const;    // nanoseconds per real-time kernel
    // finer-grained statistics (no reference counterpart)
    struct Stats {
        uint64_t preempt_count, preempt_ns_sum, preempt_ns_max;
        uint64_t rt_tasks, be_tasks, be_tasks_padded_to_finish, padded_kernels, padded_blocks;
        // preemptions that waited for the drain (wait_sync): host clock from the flag write to the best-effort streams
        // idle and the counters read; device clock from the first block that saw the flag to the last that left
        uint64_t drain_count, drain_ns_sum, drain_ns_max;
        uint64_t dev_count, dev_ns_sum, dev_ns_max;
        uint64_t drain_ns_p50, drain_ns_p99;
    };
    Stats stats() const;
    const std::string& error() const { return err_; }
    // host-side failure injection for tests: the next n kernel launches of model `mid` return an error
    Status inject_launch_failures(ModelID mid, int n);

private:
    struct Model {
        executor::HybridExecutor executor;
        QueueID qid;
        // real-time models: host-observed duration of an unpadded graph replay (ns), the baseline of the padding
        // slowdown controller = the smallest of the last four samples (anything that disturbs a sample makes it
        // longer).  Sampled by every replay that runs without best-effort work and by unpadded probe windows.
        double alone_samples[4] = {0, 0, 0, 0};
        uint32_t alone_count = 0;
        uint32_t pad_windows = 0;
        void add_alone_sample(double ns) { alone_samples[alone_count++ % 4] = ns; }
        double alone_ns() const {
            double m = 0.0;
            for (double v : alone_samples)
                if (v > 0.0 && (m == 0.0 || v < m)) m = v;
            return m;
        }
    };
    static const uint32_t kPadProbePeriod = 64;
    struct InFlight {
        reef_event_t ev;
        int kernel;
    };
    struct PadOut {
        reef_event_t ev;
        int slots;
        int64_t t_launch;
    };
    struct TaskQueue {
        ThreadSafeQueue<std::shared_ptr<Task>> task_queue;
        executor::GPUStream_t stream = nullptr;
        std::deque<InFlight> inflight;
        std::vector<reef_event_t> free_events;
        // timeline padding: pieces of this queue's head task on its stream, not yet seen complete
        std::deque<PadOut> pad_out;
        int pad_quantum_left = 0;
        bool pad_draining = false;
        bool counters_pending = false;   // a copy of the head task's completion counters is on the stream (wait_sync)
        std::vector<int> preempted_kernels;   // kernels that were in flight at the last preemption (diagnostics)
    };

    Status create_task_queue(std::shared_ptr<TaskQueue>& ret, bool rt);
    void loop_body();
    void execute_be_task(std::shared_ptr<Task>& task, std::shared_ptr<TaskQueue>& tqueue);
    void execute_rt_task(std::shared_ptr<Task>& task);
    void preempt_be_tasks();
    void reset_preempt_flag_async();
    void preempt_reset();
    void preempt_wait();
    bool dynamic_kernel_padding(std::shared_ptr<Task>& rt_task);
    bool timeline_padding(std::shared_ptr<Task>& rt_task);
    bool device_error_seen(const char* where);
    void dump_streams_once(const char* why);   // what every best-effort stream had in flight (printed once)
    bool streams_dumped = false;
    void fail_be_task(TaskQueue& q, std::shared_ptr<Task>& t, const std::string& why);
    bool side_padding_needed(executor::HybridExecutor& rt_exe);
    void advance_padded(Task* be_task, TaskQueue* q, int blocks, bool side_launch,
                        std::vector<std::shared_ptr<Task>>* complete);
    void retire(TaskQueue& q, Task& t);
    void finish_task(std::shared_ptr<Task>& t);
    bool any_be_waiting();

    ScheduleMode mode;
    int device;
    int num_sms = 0;
    static const size_t model_pool_capacity = 1024;
    std::atomic_uint32_t model_pool_size;
    std::vector<std::shared_ptr<Model>> model_pool;

    std::atomic_uint32_t task_idx_pool;
    std::unordered_map<TaskID, std::shared_ptr<Task>> task_pool;
    std::mutex task_pool_mtx;

    static const size_t max_num_be_queues = 32;
    static const QueueID rt_queue_id = 32;
    std::mutex be_queues_mtx;
    std::vector<std::shared_ptr<TaskQueue>> be_queues;
    std::atomic_uint32_t be_queue_cnt;
    std::shared_ptr<TaskQueue> rt_queue;
    std::mutex task_cnt_mtx;
    std::condition_variable task_cnt_cv;
    bool wait_sync;
    bool rt_graph;
    int rt_chain_clusters = -1;

    std::unique_ptr<std::thread> scheduler;
    executor::GPUStream_t preempt_stream = nullptr;
    executor::GPUDevicePtr_t preempt_flag = 0;
    bool preempted;
    int be_stream_device_queue_cap;
    std::atomic_bool _shutdown;
    std::atomic<uint64_t> pending_tasks;

    uint32_t dkp_next_queue = 0;
    int rt_grace_us = 30;
    bool rt_recent = false;
    std::chrono::steady_clock::time_point last_rt_finish;
    int pad_depth = 3;
    int pad_overcommit = 100;
    int pad_window = 8;
    int pad_quantum = 24;
    double pad_piece_bytes = 32e6;      // a padded piece moves at most this many algorithmic bytes (0: no limit)
    int pad_piece_cap = 0;              // > 0: best-effort pieces never claim more slots than this (wide kernels are cut)
    double pad_target = 0.065;
    double pad_ratio_ema = 0.0;
    double pad_rate = 100.0;            // best-effort kernels per real-time window (controller state)
    // loop statistics of timeline_padding, printed at destruction when REEF_PAD_TRACE is set
    struct PadTrace {
        uint64_t calls = 0, iters = 0, no_slot = 0, no_sms = 0, no_queue = 0, launched = 0;
        uint64_t launch_ns = 0, turnaround_ns = 0, retired = 0, graph_launch_ns = 0, window_ns = 0;
        uint64_t q_empty = 0, q_draining = 0, q_full = 0, q_issued = 0, q_nofit = 0, segments = 0, singles = 0;
    } pad_trace;
    uint64_t preempt_count, preempt_latency_sum, preempt_latency_max;
    uint64_t drain_count = 0, drain_ns_sum = 0, drain_ns_max = 0;
    uint64_t dev_count = 0, dev_ns_sum = 0, dev_ns_max = 0;
    bool partition_rt_whole_gpu = false;    // flags bit 2: only the best-effort side is confined, the real-time stream keeps every SM
    reef_partition_t partition = nullptr;   // non-null: queues take their streams from the two sides of an SM partition
    uint32_t* mapped_flag_host = nullptr;   // non-null: the flag is pinned host memory raised by a host store
    bool device_stamps = false;
    int cpu_first = -1, cpu_count = 0;
    uint64_t last_flag_ns = 0;
    bool flag_early = false;   // the flag was raised ahead of preempt_reset (timeline_padding, before its graph launch)
    std::chrono::steady_clock::time_point t_flag_early;
    std::vector<uint32_t> drain_samples;
    uint64_t drain_percentile(double q) const;
    void write_flag(uint32_t v);
    uint64_t kernel_sel_count, kernel_sel_latency_sum;
    uint64_t n_rt_tasks, n_be_tasks, n_be_padded_finish, n_padded_kernels, n_padded_blocks;
    std::string err_;
};

}  // namespace server
}  // namespace reef
