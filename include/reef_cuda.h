/*
 * libreef_cuda — C-ABI device layer of the REEF executor kernel path on NVIDIA B200 (sm_100a).
 *
 * This header is the drop-in boundary: it replaces the reference's GPU abstraction, i.e. the
 * 19 GPU* macros over the HIP driver API (reference: src/reef/executor/hip/hip_impl.h:5-23),
 * the GPUConfig device/kernel resource model (reference: src/reef/executor/hip/hip_impl.h:58-75,
 * src/reef/executor/hip/hip_impl.cpp:9-74) and the handful of direct HIP calls that bypass the
 * macros (reference: src/reef/executor/executor_base.cpp:78, src/reef/executor/hybrid_executor.cpp:99-100,
 * src/reef/server/scheduler.cpp:45,48,353-356,458).
 *
 * Conventions: plain C types only; every function returns a reef_status (the reference's Status
 * enum, reference: src/reef/util/common.h:46-52, plus Timeout); no exceptions cross the boundary;
 * handles are opaque.  Functions are thread-compatible per handle and not internally locked — the
 * reference issues all GPU calls for a device from one scheduler thread and so does the host here.
 */
#ifndef REEF_CUDA_H_
#define REEF_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define REEF_API __attribute__((visibility("default")))

typedef int reef_status;
enum {
    REEF_SUCC = 0,        /* Status::Succ        */
    REEF_FAIL = 1,        /* Status::Fail        */
    REEF_NOT_FOUND = 2,   /* Status::NotFound    */
    REEF_OUT_OF_RANGE = 3,/* Status::OutOfRange  */
    REEF_FULL = 4,        /* Status::Full        */
    REEF_TIMEOUT = 5      /* new: a bounded wait ran out */
};

typedef struct reef_module_s* reef_module_t;   /* replaces GPUModule_t   */
typedef struct reef_kernel_s* reef_kernel_t;   /* replaces GPUFunction_t */
typedef void* reef_stream_t;                   /* replaces GPUStream_t (a cudaStream_t) */
typedef void* reef_event_t;
typedef void* reef_graph_t;
typedef uint64_t reef_dptr_t;                  /* replaces GPUDevicePtr_t */

/* Last error text of the calling thread (CUDA error string or a registry message). */
REEF_API const char* reef_last_error(void);

/* ---- device ------------------------------------------------------------------------------- */
/* GPUInit + GPUDeviceGet (reference: executor_base.cpp:19-22): selects `device` for the calling
 * thread.  One executor / scheduler thread per GPU calls this with its own ordinal. */
REEF_API reef_status reef_gpu_init(int device);
REEF_API reef_status reef_device_count(int* count);
/* GPUConfig::get_num_cus (reference: hip_impl.cpp:9-12 hard-codes 60): queried, 148 on B200. */
REEF_API reef_status reef_device_num_sms(int* num_sms);
REEF_API reef_status reef_device_sync(void);                       /* GPUDeviceSynchronize */

/* ---- memory ------------------------------------------------------------------------------- */
REEF_API reef_status reef_malloc(reef_dptr_t* ptr, size_t bytes);  /* GPUMalloc */
REEF_API reef_status reef_free(reef_dptr_t ptr);                   /* GPUFree   */
REEF_API reef_status reef_memset(reef_dptr_t ptr, int value, size_t bytes);                 /* GPUMemset */
REEF_API reef_status reef_memset_async(reef_dptr_t ptr, int value, size_t bytes, reef_stream_t s);
REEF_API reef_status reef_memcpy_h2d(reef_dptr_t dst, const void* src, size_t bytes);       /* GPUMemcpyHtoD */
REEF_API reef_status reef_memcpy_d2h(void* dst, reef_dptr_t src, size_t bytes);             /* GPUMemcpyDtoH */
REEF_API reef_status reef_memcpy_h2d_async(reef_dptr_t dst, const void* src, size_t bytes, reef_stream_t s); /* hipMemcpyHtoDAsync, scheduler.cpp:353 */
REEF_API reef_status reef_memcpy_d2h_async(void* dst, reef_dptr_t src, size_t bytes, reef_stream_t s);       /* hipMemcpyDtoHAsync, hybrid_executor.cpp:138 */
REEF_API reef_status reef_host_alloc_pinned(void** ptr, size_t bytes);                      /* hipHostMalloc, hybrid_executor.cpp:99-100 */
REEF_API reef_status reef_host_free_pinned(void* ptr);

/* ---- streams, events, graphs -------------------------------------------------------------- */
/* GPUStreamCreate / hipStreamCreateWithWindowSize (reference: scheduler.cpp:45,48).  CUDA cannot
 * bound or clear a stream's device queue, so the "window" is a host-side in-flight limiter in the
 * scheduler; `high_priority` != 0 gives the real-time stream the greatest CUDA stream priority. */
REEF_API reef_status reef_stream_create(reef_stream_t* s, int high_priority);
REEF_API reef_status reef_stream_destroy(reef_stream_t s);
REEF_API reef_status reef_stream_sync(reef_stream_t s);            /* GPUStreamSynchronize */
/* GPUStreamQuery / GPUStreamEmpty (reference: hip_impl.cpp:77-80): *busy = 0 when idle. */
REEF_API reef_status reef_stream_query(reef_stream_t s, int* busy);
/* GPUWriteValue32Async (reference: hip_impl.h:20): ordered 32-bit store to device memory. */
REEF_API reef_status reef_write32_async(reef_stream_t s, reef_dptr_t ptr, uint32_t value);
REEF_API reef_status reef_event_create(reef_event_t* e);
/* An event that only signals completion (no timestamps: reef_event_elapsed_ms must not be used on it).  The host sees
 * it complete several microseconds sooner than a timed event (measured on an idle stream: 1.6 us against 7.9 us from
 * record to a successful query), which is what the scheduler's completion tracking and the preemption drain use. */
REEF_API reef_status reef_event_create_untimed(reef_event_t* e);
REEF_API reef_status reef_event_destroy(reef_event_t e);
REEF_API reef_status reef_event_record(reef_event_t e, reef_stream_t s);
REEF_API reef_status reef_event_sync(reef_event_t e);
REEF_API reef_status reef_event_query(reef_event_t e, int* pending);
REEF_API reef_status reef_event_elapsed_ms(reef_event_t start, reef_event_t stop, float* ms);
REEF_API reef_status reef_stream_wait_event(reef_stream_t s, reef_event_t e);
/* CUDA-graph capture of a launch sequence (no reference counterpart: the reference pays one
 * hipModuleLaunchKernel per layer, executor_base.cpp:196-223). */
REEF_API reef_status reef_graph_begin(reef_stream_t s);
REEF_API reef_status reef_graph_end(reef_stream_t s, reef_graph_t* g);
REEF_API reef_status reef_graph_launch(reef_graph_t g, reef_stream_t s);
REEF_API reef_status reef_graph_destroy(reef_graph_t g);

/* ---- kernel registry ---------------------------------------------------------------------- */
/* GPUModuleLoad (reference: executor_base.cpp:24, hybrid_executor.cpp:22-23).  The reference loads
 * one code object per model; here every kernel is built into this library and a "module" is a
 * view of the built-in registry (path may be NULL and is only recorded). */
REEF_API reef_status reef_module_open(const char* path_or_null, reef_module_t* mod);
REEF_API reef_status reef_module_close(reef_module_t mod);
/* GPUModuleGetFunction (reference: executor_base.cpp:47-52): resolve a kernel by the name string
 * in <model>.json.  The name is "<family>__<key><int>_<key><int>..." ; an unknown family or an
 * unsupported shape returns REEF_NOT_FOUND. */
REEF_API reef_status reef_module_get_kernel(reef_module_t mod, const char* name, reef_kernel_t* k);
/* Launch geometry of a kernel name: dims = {grid x,y,z, block x,y,z} as stored in
 * "launch_params" (reference: model.cpp:35-37) and the dynamic shared memory in bytes as stored in
 * "shared_memory".  Needs no GPU; the resource generator calls it so json and registry agree. */
REEF_API reef_status reef_kernel_plan(const char* name, uint32_t dims[6], uint32_t* dyn_smem, int* num_args);
/* Algorithmic work of one launch of a kernel name: floating-point operations and bytes that must move
 * (weights + inputs + outputs (+ residual, + second output) + per-channel parameters), and whether the name
 * selects the tensor-core kernel.  Needs no GPU; no reference counterpart (roofline bookkeeping). */
REEF_API reef_status reef_kernel_cost(const char* name, double* flops, double* bytes, int* tensor_core);

/* Binds a kernel handle to its device pointers ahead of the first launch (no reference counterpart): builds
 * the TMA tensor maps of tensor-core kernels and does every one-time allocation or attribute call, so
 * that the first reef_launch can already be part of a CUDA-graph capture.  Optional: a launch prepares
 * lazily when the pointers it is given differ from the prepared ones. */
REEF_API reef_status reef_kernel_prepare(reef_kernel_t k, void** args);

/* Least size in bytes of the buffer behind each of the kernel's positional arguments (n >= its argument count).
 * The reference trusts <model>.json (executor_base.cpp:54-75 allocates what the storage table says and binds by
 * index); here the loader refuses a json whose storage entry is smaller than what the shape in the kernel name
 * makes the kernel touch. */
REEF_API reef_status reef_kernel_arg_bytes(reef_kernel_t k, size_t* bytes, int n);

/* GPUConfig::KernelResource + calculate_occupancy (reference: hip_impl.h:62-74, hip_impl.cpp:34-74). */
typedef struct {
    int num_blocks;        /* logical thread blocks of one launch                           */
    int threads;           /* threads per block                                             */
    int regs_per_thread;   /* replaces vgprs/sgprs                                          */
    int static_smem;       /* bytes                                                         */
    int dyn_smem;          /* bytes                                                         */
    int local_mem;         /* replaces stack_size                                           */
    int max_blocks_per_sm; /* occupancy from the CUDA occupancy API at (threads, dyn_smem)  */
    double flops;          /* algorithmic FLOPs of one launch                               */
    double bytes;          /* algorithmic HBM bytes of one launch                           */
    int tensor_core;       /* 1 when the kernel's contraction runs on tcgen05               */
    int cluster;           /* thread blocks per cluster (1 = no cluster); block ranges handed to
                              reef_dispatch for this kernel must be multiples of it           */
    int chainable;         /* 1: a tensor-core convolution / matmul that reef_chain_create accepts */
} reef_kernel_attrs_t;
REEF_API reef_status reef_kernel_attrs(reef_kernel_t k, reef_kernel_attrs_t* out);

/* GPUModuleLaunchKernel (reference: executor_base.cpp:211-223).  `args[i]` points at the i-th
 * 8-byte device pointer, positional as in the json "args" list.  dims must equal the plan. */
REEF_API reef_status reef_launch(reef_kernel_t k, const uint32_t dims[6], uint32_t dyn_smem,
                                 reef_stream_t s, void** args);
/* Best-effort flavour (reference: hybrid_executor.cpp:153-163 launches K(int* preempted,
 * int* task_slot, ...), wrapper contract script/best_effort_kernel.py:22-33).  Every block reads
 * *preempt_flag at entry and at its loop heads and leaves without side effects on the completion
 * counter when it is set; a block that ran to the end adds 1 to *task_slot.  The kernel is
 * idempotent, so a kernel whose counter is short of num_blocks is simply launched again. */
REEF_API reef_status reef_launch_be(reef_kernel_t k, const uint32_t dims[6], uint32_t dyn_smem,
                                    reef_stream_t s, reef_dptr_t preempt_flag, reef_dptr_t task_slot,
                                    void** args);
/* Dynamic kernel padding (reference: scheduler.cpp:613-649 launches merge_framework_N with
 * {rt func, rt occupancy, rt blocks, rt offset, rt args, be func, be occupancy, be blocks,
 * be offset, be args, cu_partition}; device side resource/mocked_kernel/mocked_kernel.trans.cu:112-186).
 * Runs the real-time kernel `rt` and, beside it, best-effort logical blocks
 * [be_block_offset, be_block_offset+be_block_num) of `be` (be may be NULL, rt may be NULL).
 *  - Both kernels are logical-block families and be_stream is NULL: ONE persistent grid of
 *    sms*occupancy blocks on `s`; blocks resident on SMs [0, sm_partition) take real-time blocks
 *    from a ticket counter, the others run the best-effort blocks and then help with what is left
 *    of the real-time kernel (so the result does not depend on block placement).
 *  - A tensor-core (cluster) kernel is involved, or be_stream is given: the real-time kernel is its
 *    own launch on `s` and the best-effort blocks are launched beside it on be_stream, to be placed by
 *    the hardware on the SMs the real-time kernel leaves free (`s` should have the greater priority).
 *    For a cluster kernel the block range must be a multiple of its cluster size.
 * Best-effort blocks run here do not poll the preempt flag; each one that completes adds 1 to
 * *be_task_slot.  rt_ctrl / be_ctrl: 16 bytes of zeroed device memory each, owned by the caller and
 * reused across launches (a grid re-zeroes its block when it drains); be_ctrl is only used by a
 * separate best-effort launch and must not be shared by launches that can overlap. */
REEF_API reef_status reef_dispatch(reef_kernel_t rt, void** rt_args,
                                   reef_kernel_t be, void** be_args,
                                   int be_block_offset, int be_block_num,
                                   int sm_partition, int occupancy,
                                   reef_dptr_t be_task_slot,
                                   reef_dptr_t rt_ctrl, reef_dptr_t be_ctrl,
                                   reef_stream_t s, reef_stream_t be_stream);

/* reef_dispatch for callers that must not allocate device memory.  No counterpart in the reference (its
 * proxy kernels keep no state in global memory).
 * Who needs it: the dispatcher keeps its ticket counters in 16 bytes of zeroed device memory that
 * reef_dispatch expects the caller to own (rt_ctrl).  A scheduler loop that is in the middle of serving a
 * real-time request, or code running inside a CUDA stream capture, cannot get such memory: cudaMalloc
 * synchronises the whole device (it would stall the very request being served) and is not permitted while a
 * capture is open.  This entry point keeps the counters in a file-scope static device array inside the
 * library instead, so it calls no cudaMalloc / cudaFree and no other allocating routine.
 * Limits and rules:
 *  - REEF_STATIC_DISPATCH_LANES (64) lanes of 256 bytes = 16 KB of device memory, held by every GPU that loads
 *    the library until the process exits; `lane` >= 64 is rejected with REEF_OUT_OF_RANGE and a message.
 *  - All launches that name the same lane share its counters, and a lane keeps what the last launch left in
 *    it: every call first clears the lane on `s` (stream-ordered 16-byte memset), so calls on one stream are
 *    safe back to back, but two launches that use the same lane and can overlap on the GPU race on the
 *    tickets.  Give concurrent streams different lanes.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device
 *    current); make that first call before any stream capture begins.
 *  - Logical-block kernels only (one persistent grid); a tensor-core cluster kernel on either side is
 *    refused with REEF_FAIL.  Everything else is as in reef_dispatch's single-grid form. */
#define REEF_STATIC_DISPATCH_LANES 64
REEF_API reef_status reef_dispatch_static(reef_kernel_t rt, void** rt_args,
                                          reef_kernel_t be, void** be_args,
                                          int be_block_offset, int be_block_num,
                                          int sm_partition, int occupancy,
                                          reef_dptr_t be_task_slot, int lane, reef_stream_t s);

/* A run of consecutive tensor-core layers as ONE persistent kernel (no reference counterpart: the reference launches
 * one kernel per layer, executor_base.cpp:196-223; its persistent proxies host one layer each, trans_executor.cpp:132-173).
 * reef_chain_create binds `n` kernels (all with attrs.chainable) to their argument lists (args[i] as in reef_launch)
 * and builds the layer table and the completion counters in device memory — call it at load time, never during a
 * stream capture.  reef_chain_launch sets the counters (stream-ordered) and launches a grid of `clusters` 8-CTA clusters
 * (0 = default 32, two CTAs per SM) that walks the layers in order; results are bit-identical to launching the kernels
 * one by one.  One chain object serves one stream at a time (its counters are
 * shared by its launches).  Every device-side wait is bounded; an expired wait raises the device error word. */
typedef struct reef_chain_s* reef_chain_t;
REEF_API reef_status reef_chain_create(reef_kernel_t* kernels, void*** args, int n, int clusters, reef_chain_t* chain);
REEF_API reef_status reef_chain_launch(reef_chain_t chain, reef_stream_t s);
REEF_API reef_status reef_chain_destroy(reef_chain_t chain);
/* Best-effort use of a chain (the BE wrapper contract of script/best_effort_kernel.py:22-33 for a whole run of layers):
 * the grid starts at `first_layer` (layers before it count as complete), runs on `clusters` clusters (0 = the chain's
 * default) and polls *preempt_flag whenever a cluster takes its next tile: once the flag is up every cluster leaves at
 * its next tile boundary.  The completion counters then say how far each layer got: reef_chain_copy_progress copies
 * them (stream-ordered, to pinned memory) and, after the caller has synchronised `s`, reef_chain_first_incomplete
 * returns the first layer that is not complete (the number of layers when all are): restart there, layers are
 * idempotent.  Tiles are taken by ticket and in order, so a chain makes progress with however few of its clusters the
 * hardware has made resident beside kernels of greater priority. */
REEF_API reef_status reef_chain_launch_be(reef_chain_t chain, reef_stream_t s, int first_layer, reef_dptr_t preempt_flag, int clusters);
REEF_API reef_status reef_chain_copy_progress(reef_chain_t chain, reef_stream_t s);
REEF_API reef_status reef_chain_first_incomplete(reef_chain_t chain, int* layer);
/* layers in the chain, clusters of its grid, and the most clusters the device can hold at once */
REEF_API reef_status reef_chain_info(reef_chain_t chain, int* layers, int* clusters, int* max_clusters);

/* GPUClearHostQueue / GPUResetCU (reference: hip_impl.h:21-22) have no CUDA equivalent: queued
 * launches are dropped by the host scheduler before they reach the stream and running blocks leave
 * at their next flag poll.  This call is the bounded replacement for the reference's wait loop
 * (reference: scheduler.cpp:336-345): waits until `s` is idle or `timeout_us` passed (REEF_TIMEOUT). */
REEF_API reef_status reef_preempt_wait(reef_stream_t s, uint64_t timeout_us);

/* Device-side error word: kernels with bounded waits (mbarrier waits of the tensor-core convolution) set it
 * instead of hanging or trapping.  The word lives in pinned host memory that the device writes through a mapped
 * pointer, so reading it costs no copy and no synchronisation of its own: call after the stream of interest has
 * been synchronised.  reef_device_error reads the word of the current device and clears it; *value != 0 means
 * some wait expired and the outputs are not valid.  reef_device_error_peek reads without clearing (the scheduler
 * looks at it after every task).  reef_device_error_set stores a value from the host: a supervisor that found the
 * device state invalid by other means marks it, and the tests inject a failure with it without making any device
 * wait expire.  (The reference aborts the process on any GPU error: hip_impl.h:25-41.) */
REEF_API reef_status reef_device_error(int* value);
REEF_API reef_status reef_device_error_peek(int* value);
REEF_API reef_status reef_device_error_set(int value);

/* Occupies `s` with a one-thread kernel for `ns` nanoseconds (clamped to 20 ms, bounded loop).  Used by the kernel
 * profiler (HybridExecutor::profile_kernels, which writes <model>.profile.json) to hold a stream while a whole pass
 * is queued behind it, so that the events between kernels measure no launch latency.  No reference counterpart (the
 * reference's profiler binary is not in its tree, resource/Makefile:32-36). */
REEF_API reef_status reef_stream_delay(reef_stream_t s, uint64_t ns);

/* Preemption latency on the device's own clock (no reference counterpart: the reference measures host wall clock
 * around its switch, scheduler.cpp:378,406-410).  While armed, the first best-effort block that finds the preempt
 * flag up records %globaltimer (a minimum over blocks) and every best-effort block that leaves because of the flag
 * records it again (a maximum): last_leave - first_seen is the time from the flag becoming visible on the device to
 * the last best-effort block having left.  reef_preempt_stamps_read returns both (0, 0 when no block saw the flag)
 * and re-arms; call it when the best-effort streams have drained.  Arming allocates 16 bytes of device memory. */
REEF_API reef_status reef_preempt_stamps_arm(int on);
REEF_API reef_status reef_preempt_stamps_read(uint64_t* first_seen_ns, uint64_t* last_leave_ns);

/* A preempt flag the host can raise with a plain store (the alternative to reef_write32_async on a device flag;
 * GPUWriteValue32Async, reference: hip_impl.h:20): 4 bytes of pinned host memory mapped into the device's address
 * space.  *dev_ptr is what kernels are given as their preempt flag; reef_flag_set stores through host_ptr with
 * release semantics and returns at once.  Every device-side poll is then a read across PCIe, which is why the
 * scheduler's default stays the device-resident flag. */
REEF_API reef_status reef_flag_alloc_mapped(uint32_t** host_ptr, reef_dptr_t* dev_ptr);
REEF_API reef_status reef_flag_free_mapped(uint32_t* host_ptr);
REEF_API reef_status reef_flag_set(uint32_t* host_ptr, uint32_t value);

/* Spatial partition of the current device's SMs (CUDA green contexts): `be_sms` SMs are set aside for best-effort
 * streams and the rest for real-time streams, so that best-effort blocks never share an SM with real-time blocks
 * (the reference's dynamic kernel padding partitions compute units inside one grid, `cu_partition`,
 * resource/mocked_kernel/mocked_kernel.trans.cu:112-186; here the hardware block scheduler keeps the two apart).
 * The driver rounds SM counts to its granularity (8 on this architecture): reef_partition_info reports what was
 * provisioned.  flags: bit 0 = the clean group goes to the real-time side (best-effort gets the remainder) instead
 * of the other way round; bit 1 = ask for groups that keep the largest cluster size schedulable.  (The scheduler
 * knows a third bit, 4: only the best-effort side is confined and the real-time stream keeps every SM.)
 * Streams of a partition are ordinary streams in every other respect (kernels, graphs, events, copies). */
typedef struct reef_partition_s* reef_partition_t;
REEF_API reef_status reef_partition_create(int be_sms, int flags, reef_partition_t* p);
REEF_API reef_status reef_partition_info(reef_partition_t p, int* rt_sms, int* be_sms);
REEF_API reef_status reef_partition_stream_create(reef_partition_t p, int best_effort, int high_priority, reef_stream_t* s);
REEF_API reef_status reef_partition_destroy(reef_partition_t p);

/* Measurement helper: what the host sees of the device through a stream.  `iters` times (spaced 200 us apart, after
 * iters/10 untimed rounds) it (a) issues reef_write32_async on an idle high-priority stream, (b) records an event
 * behind it and spins on reef_event_query until it completes, (c) records a bare event and spins again, (d) the same
 * with an event that also takes a timestamp.  Medians in microseconds: the cost of the write call, write + completion
 * as seen from the host, a bare completion-only event's round trip, a timed event's round trip.
 * These are the floor of any host-clocked figure that ends with "the stream is idle" (the preemption drain). */
REEF_API reef_status reef_probe_stream_latency(int iters, double* write_call_us, double* write_complete_us,
                                               double* event_round_trip_us, double* timed_event_round_trip_us);

/* Number of kernels this library launched since load (its own kernels only; graph replays count
 * the kernels inside the graph). */
REEF_API uint64_t reef_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* REEF_CUDA_H_ */
