// Executors: own a model's device storage and launch its kernels through the C-ABI device layer.
//
//   ExecutorBase   raw kernels in json order                 (reference: src/reef/executor/executor_base.{h,cpp})
//   HybridExecutor + per-kernel scheduling metadata (KernelArg: logical blocks, minimal occupancy,
//                  resources, latency profile), the best-effort flavour with preempt flag and
//                  completion counters, the dispatcher launch, and a CUDA-graph fast path
//                  (reference: src/reef/executor/trans_executor.{h,cpp}, hybrid_executor.{h,cpp})
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "../../../include/reef_cuda.h"
#include "common.h"
#include "model.h"

namespace reef {
namespace server {
class REEFScheduler;
}
namespace executor {

typedef reef_dptr_t GPUDevicePtr_t;
typedef reef_kernel_t GPUFunction_t;
typedef reef_module_t GPUModule_t;
typedef reef_stream_t GPUStream_t;

class ExecutorBase {
public:
    ExecutorBase();
    virtual ~ExecutorBase();

    // co_file_path is accepted for signature parity; kernels come from the built-in registry.
    Status load_model_from_file(const char* json_file_path, const char* co_file_path = nullptr);
    virtual Status load_model_from_GPU_module(const char* json_file_path, GPUModule_t module);
    Status load_param_from_file(const char* param_file_path);

    Status set_input(const std::string& key, const std::vector<float>& value);
    Status set_input(int idx, const void* value, size_t len);
    Status set_input(const std::string& key, const void* value, size_t len);
    Status get_data_size(const std::string& key, size_t& size);
    Status get_output(std::vector<float>& out);
    Status get_output(void* out, size_t len);
    Status get_data(int idx, void* out, size_t len);
    // asynchronous I/O on a stream from/to pinned host memory (no reference counterpart: the
    // reference copies synchronously on the default stream, executor_base.cpp:112-116)
    Status set_input_async(const std::string& key, const void* value, size_t len, GPUStream_t stream);
    Status get_output_async(void* out, size_t len, GPUStream_t stream);

    Status execute(GPUStream_t stream = nullptr);
    Status execute_to(int idx, GPUStream_t stream = nullptr);
    Status execute_kernel(int idx, GPUStream_t stream = nullptr);
    Status execute_kernel_async(int idx) { return launch_kernel(idx, s); }   // no sync
    size_t num_kernels() const;
    // name of kernel i as the schedule gives it (diagnostics)
    const char* kernel_name(size_t i) const { return model && i < model->kernels.size() ? model->kernels[i].name.c_str() : "?"; }

    void set_stream(GPUStream_t stream);
    GPUStream_t stream() const;
    const std::string& error() const { return err_; }
    // Failure injection on the host: the next `n` kernel launches of this executor return Status::Fail without
    // reaching the device (how the tests exercise the failed-task path; no GPU fault is involved).
    void inject_launch_failures(int n) { fail_launches = n; }

    std::unique_ptr<Model> model;
    static Status resolve_kernels(const Model& m, GPUModule_t mod, std::vector<GPUFunction_t>* out_kernels,
                                  std::vector<uint32_t>* out_smem, std::string* err);

protected:
    Status init_executor_base(const char* json_file_path, GPUModule_t module);
    virtual Status launch_kernel(int kernel_offset, GPUStream_t stream);
    Status find_storage_idx(const std::string& name, size_t& idx);
    size_t storage_bytes(size_t idx) const;

    std::vector<GPUDevicePtr_t> storage;            // one device pointer per storage entry (views into one arena)
    std::vector<GPUFunction_t> kernels;             // per kernel call
    std::vector<uint32_t> kernel_smem;              // per kernel call, from "shared_memory"
    std::vector<std::vector<void*>> raw_args;       // raw_args[k][j] = &storage[idx]
    GPUDevicePtr_t arena = 0;
    size_t arena_bytes = 0;
    GPUModule_t base_mod = nullptr;
    bool own_module = false;
    GPUStream_t s = nullptr;
    int fail_launches = 0;
    std::string err_;
};

class HybridExecutor : public ExecutorBase {
    friend class server::REEFScheduler;

public:
    // reference: trans_executor.h:47-63
    class KernelArg {
    public:
        int block_num = 0;        // logical thread blocks of the kernel
        int block_offset = 0;
        int threads = 0;
        int min_occupancy = 1;    // minimal blocks/SM the real-time kernel needs to finish in one wave
        int granularity = 1;      // block ranges handed to the dispatcher are multiples of this (cluster size)
        reef_kernel_attrs_t resource{};
        KernelProfile profile;
    };

    HybridExecutor();
    virtual ~HybridExecutor();

    // The three code-object paths of the reference signature are accepted and ignored.
    Status load_hybrid_model_from_file(const char* json_file_path, const char* profile_file_path,
                                       const char* trans_co_file_path = nullptr,
                                       const char* preempt_co_file_path = nullptr);

    Status execute_preemptale(GPUStream_t stream = nullptr);     // (sic) reference spelling
    Status set_preempt_flag(GPUDevicePtr_t flag);
    Status reset_task_slot_async(int kernel_offset, GPUStream_t stream);
    void reset_task_slots(GPUStream_t stream, int from_kernel = 0);
    void copy_be_kernel_offset(GPUStream_t stream);
    int get_be_kernel_offset(int begin);

    Status launch_preempt_kernel(int kernel_offset, GPUStream_t stream);
    // dispatcher launch of kernel `rt_idx`, padded with logical blocks of `be`'s kernel `be_idx`
    // `be_stream` non-null (or a tensor-core kernel on either side): the best-effort blocks are launched
    // beside the real-time kernel on be_stream instead of inside one grid
    Status launch_dispatch(int rt_idx, HybridExecutor* be, int be_idx, int be_block_offset, int be_block_num,
                           int sm_partition, int occupancy, GPUStream_t stream, GPUStream_t be_stream = nullptr);
    // best-effort logical blocks [offset, offset+num) of kernel idx alone, non-preemptible, counted into the task slot
    Status launch_pad_piece(int idx, int block_offset, int block_num, int occupancy, GPUStream_t stream);
    // Padding segments: the kernel list cut into runs of kPadSegment kernels, each run captured once as a CUDA
    // graph of whole-kernel pieces (one launch and one completion event for the run; inside it the kernels keep
    // their programmatic dependencies).  Segment g covers kernels [g*kPadSegment, (g+1)*kPadSegment).
    static const int kPadSegment = 4;
    Status build_pad_segments();
    bool has_pad_segments() const { return !pad_segments.empty(); }
    Status launch_pad_segment(int seg, GPUStream_t stream);
    bool has_tensor_core_kernels() const { return has_tc; }
    // Persistent chains: every run of two or more consecutive tensor-core convolution / matmul kernels of the
    // schedule becomes ONE persistent kernel (reef_chain_create) with `clusters` 8-CTA clusters (0 = the library's
    // default).  Built here, once; execute_graph and execute_chained then launch a run through its chain.  Results
    // are bit-identical to the per-kernel launches.  Call before the first execute_graph on a stream.
    Status build_chains(int clusters = 0);
    size_t num_chains() const { return chains.size(); }
    Status chain_info(size_t idx, int* begin, int* end, int* clusters, int* max_clusters) const {
        if (idx >= chains.size()) return Status::OutOfRange;
        int layers = 0;
        if (begin) *begin = chains[idx].begin;
        if (end) *end = chains[idx].end;
        GPU_RETURN_STATUS(reef_chain_info(chains[idx].handle, &layers, clusters, max_clusters));
        return Status::Succ;
    }
    // the whole schedule with chains where they exist and plain launches elsewhere, then sync
    Status execute_chained(GPUStream_t stream = nullptr);
    // Best-effort flavour with chains: kernel `k` must be the first kernel of a chain or inside one; the chain is
    // launched from that layer on `clusters` clusters (0 = default) with the preempt flag polled at every tile.
    // Returns the chain's end (first kernel behind it) in *next.
    Status launch_preempt_chain(int k, int clusters, GPUStream_t stream, int* next);
    // chain index whose run contains kernel k, or -1
    int chain_of(int k) const {
        for (size_t i = 0; i < chains.size(); i++)
            if (k >= chains[i].begin && k < chains[i].end) return (int)i;
        return -1;
    }
    // after a preemption: copy every chain's counters on `stream` (async); once the stream is synchronised,
    // chain_kernel_offset(from) = the first kernel at or behind `from` that is not known complete
    void copy_chain_progress(GPUStream_t stream);
    int chain_kernel_offset(int from);
    // best-effort flavour of the whole schedule, chains on `clusters` clusters, then sync (the flag is not touched)
    Status execute_preemptable_chained(int clusters, GPUStream_t stream = nullptr);
    // best-effort run of the whole schedule with chains, flag raised after delay_us, resumed until done
    Status execute_preempt_resume_chained(int delay_us, int clusters, int* restarts, int* first_incomplete);
    // CUDA graph of the whole kernel list on `stream` (captured lazily on first use)
    Status execute_graph(GPUStream_t stream);
    // every kernel through the dispatcher without a best-effort partner, then sync
    Status execute_dispatch(GPUStream_t stream = nullptr);
    // best-effort run, flag raised after delay_us, resumed from the first incomplete kernel until done
    // (*first_count: the completion counter of that kernel when it was found short — between 0 and its block count)
    Status execute_preempt_resume(int delay_us, int* restarts, int* first_incomplete, int* first_count = nullptr);
    // device time of each kernel (us, CUDA events, average of iters)
    Status profile_kernels(int iters, float* us);
    // one persistent wave of kernel idx: sms*occupancy logical blocks through the dispatcher (us)
    Status profile_wave(int idx, int occupancy, int iters, float* us);
    // Measures the latency tables the padding policy reads (the reference's profile.json, produced there by a
    // `profiler` binary that is not in its tree, resource/Makefile:32-36): per distinct kernel name the average
    // duration of back-to-back launches (total_latency) and of one persistent wave at occupancy j+1
    // (latency[j]); model_latency = one graph replay.  All in nanoseconds (latency_unit_ns = 1).
    Status measure_profile(int iters, ModelProfile* out);
    const int* host_task_slots() const { return task_slots_host; }

    std::vector<KernelArg> trans_args;
    const ModelProfile* profile() const { return model_profile.get(); }

protected:
    Status init_hybrid_executor(const char* profile_file_path);

    GPUDevicePtr_t preempt_flag = 0;
    bool own_flag = false;
    GPUDevicePtr_t task_slot_base = 0;
    GPUDevicePtr_t dispatch_ctrl = 0;
    int* task_slots_host = nullptr;
    bool has_tc = false;
    std::shared_ptr<ModelProfile> model_profile;
    reef_graph_t graph = nullptr;
    std::vector<reef_graph_t> pad_segments;
    GPUStream_t graph_stream = nullptr;
    struct Chain {
        int begin, end;          // kernels [begin, end) of the schedule
        reef_chain_t handle;
    };
    std::vector<Chain> chains;
    Status launch_schedule(GPUStream_t stream, bool use_chains);
};

}  // namespace executor
}  // namespace reef
