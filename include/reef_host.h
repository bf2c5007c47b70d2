/*
 * libreef_host — C entry points over the C++ host side (model loader, executors, scheduler) so that
 * tests, benchmarks and non-C++ front ends can drive it.  Each function wraps the C++ method of the
 * same name; the C++ classes mirror the reference's (reference: src/reef/executor/executor_base.h,
 * src/reef/executor/hybrid_executor.h, src/reef/server/scheduler.h:68-126).  Return values are the
 * reference's Status enum (reference: src/reef/util/common.h:46-52) plus 5 = Timeout.
 */
#ifndef REEF_HOST_H_
#define REEF_HOST_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define REEF_HOST_API __attribute__((visibility("default")))

typedef struct reef_executor_s* reef_executor_t;     /* HybridExecutor */
typedef struct reef_scheduler_s* reef_scheduler_t;   /* REEFScheduler  */

/* ---- resource parsers (reference tests: src/reef/test/test.cpp:59-91) ---------------------- */
/* Model::from_json: counts of storage entries, kernels and I/O args; NotFound on a bad file. */
REEF_HOST_API int reef_model_parse(const char* json_path, size_t* num_storage, size_t* num_kernels, size_t* num_args);
/* The checks the model loader makes before it touches the GPU (ExecutorBase::init_executor_base; the reference
 * resolves names only, executor_base.cpp:47-52): every kernel name resolves in the registry; launch_params,
 * argument count and shared_memory equal the registry's plan; every bound storage entry is at least as large as
 * what the kernel reads or writes through that argument (OutOfRange otherwise).  Needs no GPU.  `err` (may be
 * NULL) receives the message. */
REEF_HOST_API int reef_model_check(const char* json_path, char* err, size_t err_len);
/* ModelParamParser::parse_from_file: element count of blob `key` (0 when absent) and blob count. */
REEF_HOST_API int reef_param_parse(const char* param_path, const char* key, size_t* key_elems, size_t* num_blobs);
/* ModelProfile::from_json: kernel count, model latency, and the smallest latency entry. */
REEF_HOST_API int reef_profile_parse(const char* profile_path, size_t* num_kernels, int* model_latency, int* min_latency);

/* ---- executor (ExecutorBase / HybridExecutor) ---------------------------------------------- */
REEF_HOST_API int reef_executor_create(int device, reef_executor_t* e);
REEF_HOST_API int reef_executor_destroy(reef_executor_t e);
REEF_HOST_API const char* reef_executor_error(reef_executor_t e);
/* load_hybrid_model_from_file; profile_path may be NULL/"" (no latency tables) */
REEF_HOST_API int reef_executor_load(reef_executor_t e, const char* json_path, const char* profile_path);
REEF_HOST_API int reef_executor_load_param(reef_executor_t e, const char* param_path);
REEF_HOST_API int reef_executor_num_kernels(reef_executor_t e, size_t* n);
REEF_HOST_API int reef_executor_num_storage(reef_executor_t e, size_t* n);
REEF_HOST_API int reef_executor_get_data_size(reef_executor_t e, const char* name, size_t* bytes);
REEF_HOST_API int reef_executor_set_input(reef_executor_t e, const char* name, const void* data, size_t len);
REEF_HOST_API int reef_executor_get_output(reef_executor_t e, void* out, size_t len);
REEF_HOST_API int reef_executor_get_data(reef_executor_t e, int idx, void* out, size_t len);
REEF_HOST_API int reef_executor_execute(reef_executor_t e);                 /* raw kernels, then sync       */
REEF_HOST_API int reef_executor_execute_to(reef_executor_t e, int idx);     /* kernels [0, idx)             */
REEF_HOST_API int reef_executor_execute_kernel(reef_executor_t e, int idx);
REEF_HOST_API int reef_executor_execute_preemptable(reef_executor_t e);     /* best-effort flavour           */
REEF_HOST_API int reef_executor_execute_graph(reef_executor_t e);           /* CUDA-graph replay, then sync  */
REEF_HOST_API int reef_executor_execute_dispatch(reef_executor_t e);        /* every kernel through the dispatcher, unpadded */
/* Persistent chains (HybridExecutor::build_chains): every run of >= 2 consecutive tensor-core convolution / matmul
 * kernels becomes one persistent kernel of `clusters` 8-CTA clusters (0 = default); *num_chains (may be NULL) = runs
 * found.  execute_graph then replays the schedule with the chains; execute_chained launches it the same way without a
 * graph, then syncs.  Bit-identical to the per-kernel launches. */
REEF_HOST_API int reef_executor_build_chains(reef_executor_t e, int clusters, size_t* num_chains);
REEF_HOST_API int reef_executor_execute_chained(reef_executor_t e);
/* As reef_executor_execute_preempt_resume, with every chain launched in its best-effort form on `clusters` clusters
 * (0 = default): the flag stops a chain at a tile boundary and it is restarted at its first incomplete layer. */
REEF_HOST_API int reef_executor_execute_preempt_resume_chained(reef_executor_t e, int delay_us, int clusters, int* restarts, int* first_incomplete);
/* chain idx covers kernels [*begin, *end) of the schedule and runs on *clusters clusters of the *max_clusters the GPU holds at once */
/* the best-effort flavour of the whole schedule with its chains on `clusters` clusters, then sync */
REEF_HOST_API int reef_executor_execute_preemptable_chained(reef_executor_t e, int clusters);
/* gives the executor a stream of its own with the greatest (high != 0) or the least CUDA stream priority */
REEF_HOST_API int reef_executor_set_stream_priority(reef_executor_t e, int high);
REEF_HOST_API int reef_executor_chain_info(reef_executor_t e, size_t idx, int* begin, int* end, int* clusters, int* max_clusters);
/* Best-effort run with the preempt flag raised `delay_us` after the first launch (host timer), then
 * resumed from the first kernel whose completion counter is short until the model is done.
 * *restarts = number of resume rounds, *first_incomplete = restart kernel of the first round,
 * *first_count (may be NULL) = that kernel's completion counter when it was found short. */
REEF_HOST_API int reef_executor_execute_preempt_resume(reef_executor_t e, int delay_us, int* restarts, int* first_incomplete,
                                                       int* first_count);
/* Completion counters (task slots) and logical block counts per kernel, n entries each. */
REEF_HOST_API int reef_executor_task_slots(reef_executor_t e, int* slots, int* block_nums, size_t n);
/* Average milliseconds of `iters` executions after `warmup` (mode: 0 raw launches, 1 graph, 2 best-effort). */
REEF_HOST_API int reef_executor_time(reef_executor_t e, int mode, int warmup, int iters, float* avg_ms);
/* Average milliseconds of one replay of a CUDA graph holding only the model's tensor-core kernels, in schedule
 * order (CUDA events around `iters` replays after `warmup`); *launches = kernels in that graph.  NotFound when
 * the schedule has none.  No reference counterpart (measurement aid for the roofline of the dominant kernel). */
REEF_HOST_API int reef_executor_time_tensor_core(reef_executor_t e, int warmup, int iters, float* avg_ms, int* launches);
/* Microseconds per launch of kernel idx timed alone: a CUDA graph of `reps` back-to-back launches of that kernel,
 * replayed `iters` times between two CUDA events after `warmup` replays (its operands stay warm in L2 where they fit:
 * the figure is the kernel's own speed, not its place in the model).  No reference counterpart (roofline bookkeeping). */
REEF_HOST_API int reef_executor_time_kernel(reef_executor_t e, int idx, int reps, int warmup, int iters, float* us_per_launch);
/* Per-kernel device time in microseconds (CUDA events around each launch), n = num_kernels entries;
 * also returns algorithmic flops/bytes and the tensor-core marker per kernel when the arrays are given. */
REEF_HOST_API int reef_executor_profile_kernels(reef_executor_t e, int iters, float* us, double* flops, double* bytes,
                                                int* tensor_core, int* blocks, int* max_blocks_per_sm, size_t n);
/* One persistent wave of kernel idx at `occupancy` blocks per SM on every SM (latency[occupancy-1] of profile.json) */
REEF_HOST_API int reef_executor_profile_wave(reef_executor_t e, int idx, int occupancy, int iters, float* us);

/* Measures the latency tables of the loaded model on the current GPU and writes them as <model>.profile.json
 * (schema of the reference's ModelProfile::to_json, src/reef/executor/model.cpp:123-145, plus
 * "latency_unit_ns": 1).  Replaces the `profiler` binary the reference's resource/Makefile:32-36 calls. */
REEF_HOST_API int reef_executor_write_profile(reef_executor_t e, int iters, const char* out_path);

/* ---- scheduler (REEFScheduler) ------------------------------------------------------------ */
/* mode: 0 NoPreempt, 1 MultiStream, 2 WaitPreempt, 3 REEF, 4 Reset (reference: scheduler.h:22-28) */
REEF_HOST_API int reef_sched_create(int mode, int device, reef_scheduler_t* s);
REEF_HOST_API int reef_sched_destroy(reef_scheduler_t s);
REEF_HOST_API const char* reef_sched_error(reef_scheduler_t s);
REEF_HOST_API int reef_sched_load_model(reef_scheduler_t s, const char* model_dir, const char* model_name, uint32_t* mid);
REEF_HOST_API int reef_sched_load_model_files(reef_scheduler_t s, const char* json_path, const char* profile_path,
                                              const char* param_path, uint32_t* mid);
/* type: 0 RealTimeQueue, 1 BestEffortQueue */
REEF_HOST_API int reef_sched_create_queue(reef_scheduler_t s, int type, uint32_t* qid);
REEF_HOST_API int reef_sched_bind_model_queue(reef_scheduler_t s, uint32_t qid, uint32_t mid);
REEF_HOST_API int reef_sched_get_data_size(reef_scheduler_t s, uint32_t mid, const char* name, size_t* bytes);
REEF_HOST_API int reef_sched_set_input(reef_scheduler_t s, uint32_t mid, const void* data, size_t len, const char* name);
REEF_HOST_API int reef_sched_get_output(reef_scheduler_t s, uint32_t mid, void* data, size_t len, const char* name);
REEF_HOST_API int reef_sched_new_task(reef_scheduler_t s, uint32_t mid, uint32_t* tid);
/* Blocks until the task is finished.  Returns Fail for a task that finished as failed (a kernel launch returned an
 * error, or the device error word was set while it ran); the reference aborts the process instead
 * (src/reef/executor/hip/hip_impl.h:34-41). */
REEF_HOST_API int reef_sched_wait_task(reef_scheduler_t s, uint32_t tid);
/* Host-side failure injection for tests: the next `n` kernel launches of model `mid` return an error without
 * reaching the device. */
REEF_HOST_API int reef_sched_inject_launch_failures(reef_scheduler_t s, uint32_t mid, int n);
typedef struct {
    int state;                 /* 0 Init, 1 Waiting, 2 Executing, 3 Finish */
    int preempted, padded, padded_to_complete;
    int64_t submit_ns, start_ns, end_ns;   /* system_clock, ns since epoch */
    int failed;                /* a launch failed or a device-side wait expired while the task ran: output invalid */
} reef_task_info_t;
REEF_HOST_API int reef_sched_task_info(reef_scheduler_t s, uint32_t tid, reef_task_info_t* info);
REEF_HOST_API int reef_sched_set_wait_sync(reef_scheduler_t s, int value);
REEF_HOST_API int reef_sched_set_be_stream_cap(reef_scheduler_t s, int value);
/* Preempt flag in pinned host memory raised by a host store instead of a stream write (before the first load_model). */
REEF_HOST_API int reef_sched_use_mapped_flag(reef_scheduler_t s);
/* Spatial partition of the SMs between the real-time stream and the best-effort streams (before any queue is
 * created): see reef_partition_create in reef_cuda.h. */
REEF_HOST_API int reef_sched_set_sm_partition(reef_scheduler_t s, int be_sms, int flags, int* rt_sms, int* be_sms_out);
/* Device-clock preemption stamps on/off (implies wait_sync). */
REEF_HOST_API int reef_sched_set_device_stamps(reef_scheduler_t s, int on);
/* Dynamic-kernel-padding controller: padded real-time tasks may take (1 + value) x their latency alone; 0 = no limit. */
REEF_HOST_API int reef_sched_set_pad_slowdown_target(reef_scheduler_t s, double value);
/* CPU placement: scheduler thread on first_cpu, real-time clients of reef_run_clients on first_cpu + 1, best-effort
 * clients on the rest of [first_cpu, first_cpu + n_cpus); n_cpus < 3 pins nothing.  Call before reef_sched_run. */
REEF_HOST_API int reef_sched_set_cpu_slice(reef_scheduler_t s, int first_cpu, int n_cpus);
REEF_HOST_API int reef_sched_set_rt_graph(reef_scheduler_t s, int value);
/* Real-time models loaded AFTER this call run their tensor-core layers as persistent chains of `clusters` clusters
 * (0 = default size, -1 = off). */
REEF_HOST_API int reef_sched_set_rt_chains(reef_scheduler_t s, int clusters);
REEF_HOST_API int reef_sched_run(reef_scheduler_t s);
REEF_HOST_API int reef_sched_shutdown(reef_scheduler_t s);
REEF_HOST_API int64_t reef_sched_avg_preempt_latency(reef_scheduler_t s);
REEF_HOST_API int64_t reef_sched_avg_kernel_sel_latency(reef_scheduler_t s);
typedef struct {
    uint64_t preempt_count, preempt_ns_sum, preempt_ns_max;   /* flag raised + queued launches dropped + tasks rolled back */
    uint64_t rt_tasks, be_tasks, be_tasks_padded_to_finish, padded_kernels, padded_blocks;
    /* preemptions that also waited for the drain (set_wait_sync): host clock from the flag write to "best-effort
     * streams idle and completion counters read" — what the reference's figure covers, whose switch ends with the
     * running wavefronts killed (scheduler.cpp:332-345,406-410) */
    uint64_t drain_count, drain_ns_sum, drain_ns_max;
    /* the same on the device's clock (set_device_stamps): first best-effort block that saw the flag -> last one that left */
    uint64_t dev_count, dev_ns_sum, dev_ns_max;
    uint64_t drain_ns_p50, drain_ns_p99;
} reef_sched_stats_t;
REEF_HOST_API int reef_sched_stats(reef_scheduler_t s, reef_sched_stats_t* out);

/* ---- closed-loop clients (behaviour of the reference's reef_client_cont, src/example/rpc_client_cont.cpp:31-35):
 * every client thread repeats { set_input from its host buffer; new_task; wait_task; get_output into its host
 * buffer } and records the per-request wall-clock latency.  Clients whose max_requests is 0 run until all
 * clients with max_requests > 0 are done (background load).  All clients are measured over one window: a
 * bounded client counts from its first request after its warm-up, a background client from the first request it
 * submits once every bounded client is past its warm-up, so completed / elapsed_s of the clients can be added. */
typedef struct {
    uint32_t mid;
    uint32_t max_requests;       /* 0 = run while the bounded clients run                       */
    uint32_t warmup_requests;    /* not recorded                                                */
    const void* input;           /* host buffer for set_input (may be NULL: skip the copy)      */
    size_t input_len;
    const char* input_name;      /* NULL = "data"                                               */
    void* output;                /* host buffer for get_output (may be NULL: skip the copy)     */
    size_t output_len;
    float* latencies_ms;         /* out: max_requests entries (bounded clients only)            */
    uint64_t completed;          /* out: recorded requests                                      */
    double elapsed_s;            /* out: wall time of the recorded requests                     */
    uint32_t think_us;           /* pause between requests                                      */
    uint32_t failed;             /* out: 1 when a request of this client ended in error (the client stops) */
} reef_client_t;
REEF_HOST_API int reef_run_clients(reef_scheduler_t s, reef_client_t* clients, size_t n);

#ifdef __cplusplus
}
#endif
#endif /* REEF_HOST_H_ */
