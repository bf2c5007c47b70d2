#include "executor.h"

#include <algorithm>
#include <chrono>
#include <cstring>

namespace reef {
namespace executor {

static const size_t kAlign = 256;

ExecutorBase::ExecutorBase() {}

ExecutorBase::~ExecutorBase() {
    if (arena) reef_free(arena);
    if (own_module && base_mod) reef_module_close(base_mod);
}

Status ExecutorBase::load_model_from_file(const char* json_file_path, const char* co_file_path) {
    GPUModule_t mod;
    GPU_RETURN_STATUS(reef_module_open(co_file_path, &mod));
    own_module = true;
    return this->load_model_from_GPU_module(json_file_path, mod);
}

Status ExecutorBase::load_model_from_GPU_module(const char* json_file_path, GPUModule_t mod) {
    return init_executor_base(json_file_path, mod);
}

size_t ExecutorBase::storage_bytes(size_t idx) const {
    const StorageInfo& si = model->storage[idx];
    return Model::get_stype_size(si.stype) * si.size;
}

// Resolves every kernel of the schedule by name and checks the json against the registry: launch_params,
// argument count, shared_memory, and that every bound storage entry is at least as large as what the shape in the
// kernel name makes the kernel read or write through that argument (a hand-edited or stale json would otherwise
// let a kernel run past its slice of the arena).  Needs no GPU.
Status ExecutorBase::resolve_kernels(const Model& m, GPUModule_t mod, std::vector<GPUFunction_t>* out_kernels,
                                     std::vector<uint32_t>* out_smem, std::string* err) {
    out_kernels->clear();
    out_smem->clear();
    for (const KernelInfo& ki : m.kernels) {
        GPUFunction_t k;
        int rc = reef_module_get_kernel(mod, ki.name.c_str(), &k);
        if (rc != REEF_SUCC) {
            *err = reef_last_error();
            return (Status)rc;
        }
        uint32_t dims[6], smem = 0;
        int nargs = 0;
        rc = reef_kernel_plan(ki.name.c_str(), dims, &smem, &nargs);
        if (rc != REEF_SUCC) {
            *err = reef_last_error();
            return (Status)rc;
        }
        if (memcmp(dims, ki.launch_params, sizeof(dims)) != 0 || (size_t)nargs != ki.args.size()) {
            *err = "launch_params or argument count of " + ki.name + " do not match the kernel registry";
            return Status::Fail;
        }
        auto it = m.shared_memory.find(ki.name);
        // "shared_memory" is descriptive in the reference (the LDS use of the code object's kernel; launches pass
        // their own value, executor_base.cpp:217-221): an entry may claim more than the kernel here uses — the
        // reference's mocked_kernel.json says 1024 bytes — but never less; launches use the registry's value
        if (it != m.shared_memory.end() && it->second < smem) {
            *err = "shared_memory of " + ki.name + " is smaller than the kernel needs";
            return Status::Fail;
        }
        size_t need[16] = {0};
        if (reef_kernel_arg_bytes(k, need, 16) != REEF_SUCC) return Status::Fail;
        for (size_t j = 0; j < ki.args.size(); j++) {
            const size_t idx = ki.args[j];
            if (idx >= m.storage.size()) {
                *err = "argument " + std::to_string(j) + " of " + ki.name + " names a storage entry that does not exist";
                return Status::OutOfRange;
            }
            const size_t have = Model::get_stype_size(m.storage[idx].stype) * m.storage[idx].size;
            if (have < need[j]) {
                *err = "storage entry " + std::to_string(idx) + " (" + std::to_string(have) + " bytes) is smaller than argument " +
                       std::to_string(j) + " of " + ki.name + " needs (" + std::to_string(need[j]) + " bytes)";
                return Status::OutOfRange;
            }
        }
        out_kernels->push_back(k);
        out_smem->push_back(smem);
    }
    return Status::Succ;
}

Status ExecutorBase::init_executor_base(const char* json_file_path, GPUModule_t mod) {
    base_mod = mod;
    // 1. json
    model.reset(Model::from_json(json_file_path, &err_));
    if (model.get() == nullptr) RETURN_STATUS(Status::NotFound);

    // 2. kernels, by name; launch geometry, shared memory and storage sizes in the json must fit the registry
    RETURN_STATUS(resolve_kernels(*model, mod, &kernels, &kernel_smem, &err_));

    // 3. device storage: one zero-filled arena, 256-byte aligned slices (the reference does one
    //    hipMalloc + zero copy per entry, executor_base.cpp:54-63)
    size_t total = 0;
    std::vector<size_t> offs;
    for (size_t i = 0; i < model->storage.size(); i++) {
        offs.push_back(total);
        total += align_up(std::max<size_t>(storage_bytes(i), 4), kAlign);
    }
    arena_bytes = total;
    GPU_RETURN_STATUS(reef_malloc(&arena, total));
    GPU_RETURN_STATUS(reef_memset(arena, 0, total));
    storage.clear();
    for (size_t i = 0; i < model->storage.size(); i++) storage.push_back(arena + offs[i]);

    // 4. positional args -> pointers to the storage slots
    raw_args.clear();
    raw_args.reserve(model->kernels.size());
    for (KernelInfo& ki : model->kernels) {
        std::vector<void*> ka;
        for (size_t idx : ki.args) ka.push_back(&storage[idx]);
        raw_args.push_back(ka);
    }
    // bind kernels to their buffers now (tensor maps, one-time device set-up), so that the first pass may
    // already be recorded into a CUDA graph
    for (size_t i = 0; i < kernels.size(); i++) {
        int rc = reef_kernel_prepare(kernels[i], raw_args[i].data());
        if (rc != REEF_SUCC) {
            err_ = reef_last_error();
            RETURN_STATUS(rc);
        }
    }
    if (s == nullptr) GPU_RETURN_STATUS(reef_stream_create(&s, 0));
    return Status::Succ;
}

Status ExecutorBase::load_param_from_file(const char* param_file_path) {
    std::unique_ptr<ModelParam> params(ModelParamParser::parse_from_file(param_file_path, &err_));
    if (!params) RETURN_STATUS(Status::NotFound);
    for (size_t i = 0; i < storage.size(); i++) {
        const ParamBlob* blob = params->find(model->storage[i].name);
        if (!blob) continue;
        size_t bytes = blob->count * sizeof(float);
        if (bytes > storage_bytes(i)) {
            err_ = "param " + model->storage[i].name + " is larger than its storage entry";
            RETURN_STATUS(Status::OutOfRange);
        }
        GPU_RETURN_STATUS(reef_memcpy_h2d(storage[i], blob->data, bytes));
    }
    return Status::Succ;
}

Status ExecutorBase::get_data_size(const std::string& key, size_t& size) {
    size_t idx;
    if (find_storage_idx(key, idx) != Status::Succ) return Status::NotFound;
    size = storage_bytes(idx);
    return Status::Succ;
}

Status ExecutorBase::set_input(const std::string& key, const std::vector<float>& value) {
    return set_input(key, (const void*)value.data(), value.size() * sizeof(float));
}

Status ExecutorBase::set_input(const std::string& key, const void* value, size_t len) {
    size_t idx;
    if (find_storage_idx(key, idx) != Status::Succ) return Status::NotFound;
    return set_input((int)idx, value, len);
}

Status ExecutorBase::set_input(int idx, const void* value, size_t len) {
    if (idx < 0 || (size_t)idx >= storage.size()) return Status::OutOfRange;
    size_t bytes = storage_bytes(idx);
    if (len < bytes) return Status::OutOfRange;
    GPU_RETURN_STATUS(reef_memcpy_h2d(storage[idx], value, bytes));
    return Status::Succ;
}

Status ExecutorBase::set_input_async(const std::string& key, const void* value, size_t len, GPUStream_t stream) {
    size_t idx;
    if (find_storage_idx(key, idx) != Status::Succ) return Status::NotFound;
    size_t bytes = storage_bytes(idx);
    if (len < bytes) return Status::OutOfRange;
    GPU_RETURN_STATUS(reef_memcpy_h2d_async(storage[idx], value, bytes, stream));
    return Status::Succ;
}

Status ExecutorBase::get_output(std::vector<float>& out) {
    size_t idx;
    if (find_storage_idx("output", idx) != Status::Succ) return Status::NotFound;
    if (Model::get_stype_size(model->storage[idx].stype) != sizeof(float)) return Status::Fail;
    out.resize(model->storage[idx].size);
    return get_data((int)idx, (void*)out.data(), out.size() * sizeof(float));
}

Status ExecutorBase::get_output(void* out, size_t len) {
    size_t idx;
    if (find_storage_idx("output", idx) != Status::Succ) return Status::NotFound;
    if (len < storage_bytes(idx)) return Status::Fail;
    return get_data((int)idx, out, len);
}

Status ExecutorBase::get_output_async(void* out, size_t len, GPUStream_t stream) {
    size_t idx;
    if (find_storage_idx("output", idx) != Status::Succ) return Status::NotFound;
    size_t bytes = storage_bytes(idx);
    if (len < bytes) return Status::Fail;
    GPU_RETURN_STATUS(reef_memcpy_d2h_async(out, storage[idx], bytes, stream));
    return Status::Succ;
}

Status ExecutorBase::get_data(int idx, void* out, size_t len) {
    if (idx < 0 || (size_t)idx >= storage.size()) return Status::OutOfRange;
    size_t bytes = storage_bytes(idx);
    if (len < bytes) return Status::Fail;
    GPU_RETURN_STATUS(reef_memcpy_d2h(out, storage[idx], bytes));
    return Status::Succ;
}

Status ExecutorBase::find_storage_idx(const std::string& name, size_t& idx) {
    for (size_t i = 0; i < storage.size(); i++)
        if (model->storage[i].name == name) {
            idx = i;
            return Status::Succ;
        }
    return Status::NotFound;
}

size_t ExecutorBase::num_kernels() const { return model ? model->kernels.size() : 0; }
void ExecutorBase::set_stream(GPUStream_t stream) { s = stream; }
GPUStream_t ExecutorBase::stream() const { return s; }

Status ExecutorBase::execute(GPUStream_t stream) { return execute_to((int)num_kernels(), stream); }

Status ExecutorBase::execute_to(int idx, GPUStream_t stream) {
    if (stream == nullptr) stream = s;
    if (idx < 0 || (size_t)idx > num_kernels()) return Status::OutOfRange;
    for (int i = 0; i < idx; i++) RETURN_STATUS(launch_kernel(i, stream));
    GPU_RETURN_STATUS(reef_stream_sync(stream));
    return Status::Succ;
}

Status ExecutorBase::execute_kernel(int idx, GPUStream_t stream) {
    if (stream == nullptr) stream = s;
    if (idx < 0 || (size_t)idx >= num_kernels()) return Status::OutOfRange;
    RETURN_STATUS(launch_kernel(idx, stream));
    GPU_RETURN_STATUS(reef_stream_sync(stream));
    return Status::Succ;
}

Status ExecutorBase::launch_kernel(int i, GPUStream_t stream) {
    if (fail_launches > 0) {   // host-side failure injection (tests): the launch call "returns an error"
        fail_launches--;
        err_ = "injected launch failure at kernel " + std::to_string(i);
        return Status::Fail;
    }
    int rc = reef_launch(kernels[i], model->kernels[i].launch_params, kernel_smem[i], stream, raw_args[i].data());
    if (rc != REEF_SUCC) err_ = reef_last_error();
    GPU_RETURN_STATUS(rc);
    return Status::Succ;
}

// ------------------------------------------------------------------------------------------------

HybridExecutor::HybridExecutor() {}

HybridExecutor::~HybridExecutor() {
    for (auto& c : chains) reef_chain_destroy(c.handle);
    if (graph) reef_graph_destroy(graph);
    for (auto g : pad_segments) reef_graph_destroy(g);
    if (own_flag && preempt_flag) reef_free(preempt_flag);
    if (task_slot_base) reef_free(task_slot_base);
    if (dispatch_ctrl) reef_free(dispatch_ctrl);
    if (task_slots_host) reef_host_free_pinned(task_slots_host);
}

Status HybridExecutor::load_hybrid_model_from_file(const char* json_file_path, const char* profile_file_path,
                                                   const char*, const char*) {
    RETURN_STATUS(load_model_from_file(json_file_path, nullptr));
    return init_hybrid_executor(profile_file_path);
}

Status HybridExecutor::init_hybrid_executor(const char* profile_file_path) {
    const size_t n = model->kernels.size();
    int num_sms = 0;
    GPU_RETURN_STATUS(reef_device_num_sms(&num_sms));

    // 1. preempt flag (replaced by the scheduler-wide flag later) and completion counters
    GPU_RETURN_STATUS(reef_malloc(&preempt_flag, 4));
    GPU_RETURN_STATUS(reef_memset(preempt_flag, 0, 4));
    own_flag = true;
    GPU_RETURN_STATUS(reef_malloc(&task_slot_base, n * 4));
    GPU_RETURN_STATUS(reef_memset(task_slot_base, 0, n * 4));
    GPU_RETURN_STATUS(reef_malloc(&dispatch_ctrl, 16));
    GPU_RETURN_STATUS(reef_memset(dispatch_ctrl, 0, 16));
    GPU_RETURN_STATUS(reef_host_alloc_pinned((void**)&task_slots_host, n * sizeof(int)));
    memset(task_slots_host, 0, n * sizeof(int));

    // 2. per-kernel scheduling metadata (reference: trans_executor.cpp:84-99)
    trans_args.assign(n, KernelArg());
    for (size_t i = 0; i < n; i++) {
        KernelArg& ka = trans_args[i];
        GPU_RETURN_STATUS(reef_kernel_attrs(kernels[i], &ka.resource));
        ka.block_num = ka.resource.num_blocks;
        ka.threads = ka.resource.threads;
        ka.granularity = std::max(1, ka.resource.cluster);
        if (ka.resource.tensor_core) has_tc = true;
        int max_layers = std::max(1, ka.resource.max_blocks_per_sm);
        int layers = align_up(ka.block_num, num_sms) / num_sms;
        ka.min_occupancy = std::max(1, std::min(layers, max_layers));
    }

    // 3. latency profile
    if (profile_file_path != nullptr && profile_file_path[0] != 0) {
        model_profile.reset(ModelProfile::from_json(profile_file_path, &err_));
        if (!model_profile) RETURN_STATUS(Status::NotFound);
        for (size_t i = 0; i < n; i++) {
            auto it = model_profile->kernel_latency.find(model->kernels[i].name);
            if (it != model_profile->kernel_latency.end()) trans_args[i].profile = it->second;
        }
    }
    return Status::Succ;
}

Status HybridExecutor::set_preempt_flag(GPUDevicePtr_t flag) {
    if (own_flag && preempt_flag) GPU_RETURN_STATUS(reef_free(preempt_flag));
    own_flag = false;
    preempt_flag = flag;
    return Status::Succ;
}

Status HybridExecutor::execute_preemptale(GPUStream_t stream) {
    if (stream == nullptr) stream = s;
    for (size_t i = 0; i < num_kernels(); i++) RETURN_STATUS(launch_preempt_kernel((int)i, stream));
    GPU_RETURN_STATUS(reef_stream_sync(stream));
    return Status::Succ;
}

Status HybridExecutor::reset_task_slot_async(int kernel_offset, GPUStream_t stream) {
    GPU_RETURN_STATUS(reef_memset_async(task_slot_base + (size_t)kernel_offset * 4, 0, 4, stream));
    return Status::Succ;
}

void HybridExecutor::reset_task_slots(GPUStream_t stream, int from_kernel) {
    size_t n = num_kernels();
    if ((size_t)from_kernel >= n) return;
    reef_memset_async(task_slot_base + (size_t)from_kernel * 4, 0, (n - from_kernel) * 4, stream);
}

void HybridExecutor::copy_be_kernel_offset(GPUStream_t stream) {
    reef_memcpy_d2h_async(task_slots_host, task_slot_base, 4 * num_kernels(), stream);
}

int HybridExecutor::get_be_kernel_offset(int begin) {
    // first kernel whose completion counter is short of its logical block count
    for (size_t i = begin; i < num_kernels(); i++)
        if (task_slots_host[i] < trans_args[i].block_num) return (int)i;
    return (int)num_kernels();
}

Status HybridExecutor::launch_preempt_kernel(int i, GPUStream_t stream) {
    if (fail_launches > 0) {
        fail_launches--;
        err_ = "injected launch failure at kernel " + std::to_string(i);
        return Status::Fail;
    }
    int rc = reef_launch_be(kernels[i], model->kernels[i].launch_params, kernel_smem[i], stream, preempt_flag,
                            task_slot_base + (size_t)i * 4, raw_args[i].data());
    if (rc != REEF_SUCC) err_ = reef_last_error();
    GPU_RETURN_STATUS(rc);
    return Status::Succ;
}

Status HybridExecutor::launch_dispatch(int rt_idx, HybridExecutor* be, int be_idx, int be_block_offset,
                                       int be_block_num, int sm_partition, int occupancy, GPUStream_t stream,
                                       GPUStream_t be_stream) {
    int rc = reef_dispatch(kernels[rt_idx], raw_args[rt_idx].data(), be ? be->kernels[be_idx] : nullptr,
                           be ? be->raw_args[be_idx].data() : nullptr, be_block_offset, be_block_num, sm_partition,
                           occupancy, be ? be->task_slot_base + (size_t)be_idx * 4 : 0, dispatch_ctrl,
                           be ? be->dispatch_ctrl : 0, stream, be_stream);
    if (rc != REEF_SUCC) err_ = reef_last_error();
    GPU_RETURN_STATUS(rc);
    return Status::Succ;
}

Status HybridExecutor::launch_pad_piece(int idx, int block_offset, int block_num, int occupancy, GPUStream_t stream) {
    int rc = reef_dispatch(nullptr, nullptr, kernels[idx], raw_args[idx].data(), block_offset, block_num, 0, occupancy,
                           task_slot_base + (size_t)idx * 4, dispatch_ctrl, dispatch_ctrl, stream, stream);
    if (rc != REEF_SUCC) err_ = reef_last_error();
    GPU_RETURN_STATUS(rc);
    return Status::Succ;
}

Status HybridExecutor::build_pad_segments() {
    if (!pad_segments.empty()) return Status::Succ;
    GPUStream_t cap = nullptr;
    GPU_RETURN_STATUS(reef_stream_create(&cap, 0));
    const int n = (int)num_kernels();
    Status st = Status::Succ;
    for (int k0 = 0; k0 < n && st == Status::Succ; k0 += kPadSegment) {
        if (reef_graph_begin(cap) != REEF_SUCC) {
            st = Status::Fail;
            break;
        }
        for (int k = k0; k < std::min(n, k0 + kPadSegment) && st == Status::Succ; k++) {
            const KernelArg& a = trans_args[k];
            const int occ = a.resource.tensor_core ? 1 : std::max(1, std::min(2, a.resource.max_blocks_per_sm));
            st = launch_pad_piece(k, 0, a.block_num, occ, cap);
        }
        reef_graph_t g = nullptr;
        int rc = reef_graph_end(cap, &g);
        if (rc != REEF_SUCC) {
            err_ = reef_last_error();
            st = Status::Fail;
        }
        if (st == Status::Succ) pad_segments.push_back(g);
        else if (g) reef_graph_destroy(g);
    }
    reef_stream_destroy(cap);
    if (st != Status::Succ) {
        for (auto g : pad_segments) reef_graph_destroy(g);
        pad_segments.clear();
    }
    return st;
}

Status HybridExecutor::launch_pad_segment(int seg, GPUStream_t stream) {
    if (seg < 0 || seg >= (int)pad_segments.size()) RETURN_STATUS(Status::OutOfRange);
    GPU_RETURN_STATUS(reef_graph_launch(pad_segments[seg], stream));
    return Status::Succ;
}

Status HybridExecutor::build_chains(int clusters) {
    if (!chains.empty()) return Status::Succ;
    const int n = (int)num_kernels();
    for (int i = 0; i < n;) {
        if (!trans_args[i].resource.chainable) {
            i++;
            continue;
        }
        int j = i;
        while (j < n && trans_args[j].resource.chainable) j++;
        if (j - i >= 2) {
            std::vector<reef_kernel_t> ks(kernels.begin() + i, kernels.begin() + j);
            std::vector<void**> as;
            for (int k = i; k < j; k++) as.push_back(raw_args[k].data());
            reef_chain_t h = nullptr;
            int rc = reef_chain_create(ks.data(), as.data(), j - i, clusters, &h);
            if (rc != REEF_SUCC) {
                err_ = reef_last_error();
                for (auto& c : chains) reef_chain_destroy(c.handle);
                chains.clear();
                RETURN_STATUS((Status)rc);
            }
            chains.push_back(Chain{i, j, h});
        }
        i = j;
    }
    // a graph captured earlier holds the per-kernel launches: it is rebuilt on next use
    if (graph) {
        reef_graph_destroy(graph);
        graph = nullptr;
        graph_stream = nullptr;
    }
    return Status::Succ;
}

// the schedule in order: a chain launch for every run that has one, a plain launch for every other kernel
Status HybridExecutor::launch_schedule(GPUStream_t stream, bool use_chains) {
    size_t ci = 0;
    for (size_t i = 0; i < num_kernels();) {
        if (use_chains && ci < chains.size() && chains[ci].begin == (int)i) {
            int rc = reef_chain_launch(chains[ci].handle, stream);
            if (rc != REEF_SUCC) {
                err_ = reef_last_error();
                return (Status)rc;
            }
            i = (size_t)chains[ci].end;
            ci++;
            continue;
        }
        Status st = ExecutorBase::launch_kernel((int)i, stream);
        if (st != Status::Succ) return st;
        i++;
    }
    return Status::Succ;
}

Status HybridExecutor::launch_preempt_chain(int k, int clusters, GPUStream_t stream, int* next) {
    const int ci = chain_of(k);
    if (ci < 0) RETURN_STATUS(Status::OutOfRange);
    int rc = reef_chain_launch_be(chains[ci].handle, stream, k - chains[ci].begin, preempt_flag, clusters);
    if (rc != REEF_SUCC) {
        err_ = reef_last_error();
        RETURN_STATUS((Status)rc);
    }
    if (next) *next = chains[ci].end;
    return Status::Succ;
}

Status HybridExecutor::execute_preemptable_chained(int clusters, GPUStream_t stream) {
    if (stream == nullptr) stream = s;
    const int n = (int)num_kernels();
    for (int i = 0; i < n;) {
        if (chain_of(i) >= 0) {
            int next = i;
            RETURN_STATUS(launch_preempt_chain(i, clusters, stream, &next));
            i = next;
        } else {
            RETURN_STATUS(launch_preempt_kernel(i, stream));
            i++;
        }
    }
    GPU_RETURN_STATUS(reef_stream_sync(stream));
    return Status::Succ;
}

void HybridExecutor::copy_chain_progress(GPUStream_t stream) {
    for (auto& c : chains) reef_chain_copy_progress(c.handle, stream);
}

int HybridExecutor::chain_kernel_offset(int from) {
    // `from` inside a chain: the chain's counters say which of its layers are complete
    const int ci = chain_of(from);
    if (ci < 0) return from;
    int layer = 0;
    if (reef_chain_first_incomplete(chains[ci].handle, &layer) != REEF_SUCC) return from;
    return std::max(from, chains[ci].begin + layer);
}

Status HybridExecutor::execute_preempt_resume_chained(int delay_us, int clusters, int* restarts, int* first_incomplete) {
    GPUStream_t flag_stream;
    GPU_RETURN_STATUS(reef_stream_create(&flag_stream, 1));
    const int n = (int)num_kernels();
    int from = 0, rounds = 0;
    if (first_incomplete) *first_incomplete = -1;
    GPU_RETURN_STATUS(reef_write32_async(flag_stream, preempt_flag, 0));
    GPU_RETURN_STATUS(reef_stream_sync(flag_stream));
    reset_task_slots(s, 0);
    Status st = Status::Succ;
    while (from < n) {
        for (int i = from; i < n && st == Status::Succ;) {
            if (chain_of(i) >= 0) {
                int next = i;
                st = launch_preempt_chain(i, clusters, s, &next);
                i = next;
            } else {
                st = launch_preempt_kernel(i, s);
                i++;
            }
        }
        if (st != Status::Succ) break;
        const bool preempt = rounds < 8;
        if (preempt) {
            auto t0 = std::chrono::steady_clock::now();
            const int us = delay_us << std::min(rounds, 6);
            while (std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count() < us) {
            }
            reef_write32_async(flag_stream, preempt_flag, 1);
            reef_stream_sync(flag_stream);
        }
        if (reef_preempt_wait(s, 5000000) != REEF_SUCC) { st = Status::Timeout; break; }
        copy_be_kernel_offset(s);
        copy_chain_progress(s);
        GPU_RETURN_STATUS(reef_stream_sync(s));
        // first kernel not complete: plain kernels by their task slots, kernels inside a chain by its counters
        int k = from;
        while (k < n) {
            const int ci = chain_of(k);
            if (ci >= 0) {
                const int kk = chain_kernel_offset(k);
                if (kk < chains[ci].end) { k = kk; break; }
                k = chains[ci].end;
            } else {
                if (task_slots_host[k] < trans_args[k].block_num) break;
                k++;
            }
        }
        if (preempt) {
            reef_write32_async(flag_stream, preempt_flag, 0);
            reef_stream_sync(flag_stream);
        }
        if (k >= n) break;
        if (rounds == 0 && first_incomplete) *first_incomplete = k;
        reset_task_slots(s, k);
        from = k;
        rounds++;
    }
    if (restarts) *restarts = rounds;
    reef_stream_destroy(flag_stream);
    return st;
}

Status HybridExecutor::execute_chained(GPUStream_t stream) {
    if (stream == nullptr) stream = s;
    RETURN_STATUS(launch_schedule(stream, true));
    GPU_RETURN_STATUS(reef_stream_sync(stream));
    return Status::Succ;
}

Status HybridExecutor::execute_graph(GPUStream_t stream) {
    if (fail_launches > 0 && graph != nullptr && graph_stream == stream) {   // injected failure of a graph replay
        fail_launches--;
        err_ = "injected graph launch failure";
        return Status::Fail;
    }
    if (graph == nullptr || graph_stream != stream) {
        if (graph) reef_graph_destroy(graph);
        graph = nullptr;
        GPU_RETURN_STATUS(reef_graph_begin(stream));
        Status st = launch_schedule(stream, true);
        int rc = reef_graph_end(stream, &graph);
        if (st != Status::Succ || rc != REEF_SUCC) {
            // a launch failed while capturing: what was captured is a partial graph and must never be replayed
            if (rc != REEF_SUCC && st == Status::Succ) err_ = reef_last_error();
            if (graph) reef_graph_destroy(graph);
            graph = nullptr;
            graph_stream = nullptr;
            return st != Status::Succ ? st : Status::Fail;
        }
        graph_stream = stream;
    }
    GPU_RETURN_STATUS(reef_graph_launch(graph, stream));
    return Status::Succ;
}

Status HybridExecutor::execute_dispatch(GPUStream_t stream) {
    if (stream == nullptr) stream = s;
    int num_sms = 0;
    GPU_RETURN_STATUS(reef_device_num_sms(&num_sms));
    for (size_t i = 0; i < num_kernels(); i++)
        RETURN_STATUS(launch_dispatch((int)i, nullptr, 0, 0, 0, num_sms, trans_args[i].min_occupancy, stream));
    GPU_RETURN_STATUS(reef_stream_sync(stream));
    return Status::Succ;
}

static void busy_wait_us(int us) {
    auto t0 = std::chrono::steady_clock::now();
    while (std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count() < us) {
    }
}

Status HybridExecutor::execute_preempt_resume(int delay_us, int* restarts, int* first_incomplete, int* first_count) {
    GPUStream_t flag_stream;
    GPU_RETURN_STATUS(reef_stream_create(&flag_stream, 1));
    const int n = (int)num_kernels();
    int from = 0, rounds = 0;
    if (first_incomplete) *first_incomplete = -1;
    if (first_count) *first_count = -1;
    GPU_RETURN_STATUS(reef_write32_async(flag_stream, preempt_flag, 0));
    GPU_RETURN_STATUS(reef_stream_sync(flag_stream));
    reset_task_slots(s, 0);
    Status st = Status::Succ;
    while (from < n) {
        for (int i = from; i < n && st == Status::Succ; i++) st = launch_preempt_kernel(i, s);
        if (st != Status::Succ) break;
        const bool preempt = rounds < 8;
        if (preempt) {
            busy_wait_us(delay_us << std::min(rounds, 6));
            reef_write32_async(flag_stream, preempt_flag, 1);
            reef_stream_sync(flag_stream);
        }
        if (reef_preempt_wait(s, 5000000) != REEF_SUCC) { st = Status::Timeout; break; }
        copy_be_kernel_offset(s);
        GPU_RETURN_STATUS(reef_stream_sync(s));
        int k = get_be_kernel_offset(from);
        if (preempt) {
            reef_write32_async(flag_stream, preempt_flag, 0);
            reef_stream_sync(flag_stream);
        }
        if (k >= n) break;
        if (rounds == 0 && first_incomplete) *first_incomplete = k;
        if (rounds == 0 && first_count) *first_count = task_slots_host[k];
        reset_task_slots(s, k);
        from = k;
        rounds++;
    }
    if (restarts) *restarts = rounds;
    reef_stream_destroy(flag_stream);
    return st;
}

Status HybridExecutor::profile_kernels(int iters, float* us) {
    // Whole-model passes with an event between consecutive kernels: every kernel is timed in context
    // (weights of the other layers have cycled through L2 since its last run).  The stream is held by
    // a short delay kernel while the host queues the pass, so event gaps hold no launch latency.
    const size_t n = num_kernels();
    std::vector<reef_event_t> ev(n + 1);
    for (auto& e : ev) GPU_RETURN_STATUS(reef_event_create(&e));
    std::vector<double> sum(n, 0.0);
    Status st = Status::Succ;
    for (int it = 0; it <= iters && st == Status::Succ; it++) {
        GPU_RETURN_STATUS(reef_stream_delay(s, 1000ull * (400 + 8 * n)));
        reef_event_record(ev[0], s);
        for (size_t i = 0; i < n && st == Status::Succ; i++) {
            st = ExecutorBase::launch_kernel((int)i, s);
            reef_event_record(ev[i + 1], s);
        }
        GPU_RETURN_STATUS(reef_stream_sync(s));
        if (it == 0) continue;   // warm-up pass
        for (size_t i = 0; i < n; i++) {
            float ms = 0;
            reef_event_elapsed_ms(ev[i], ev[i + 1], &ms);
            sum[i] += ms;
        }
    }
    for (size_t i = 0; i < n; i++) us[i] = (float)(sum[i] * 1000.0 / std::max(1, iters));
    for (auto& e : ev) reef_event_destroy(e);
    return st;
}

Status HybridExecutor::profile_wave(int idx, int occupancy, int iters, float* us) {
    if (idx < 0 || (size_t)idx >= num_kernels() || occupancy < 1) return Status::OutOfRange;
    int num_sms = 0;
    GPU_RETURN_STATUS(reef_device_num_sms(&num_sms));
    int blocks = std::min(trans_args[idx].block_num, num_sms * occupancy);
    blocks -= blocks % trans_args[idx].granularity;
    if (blocks <= 0) blocks = std::min(trans_args[idx].block_num, trans_args[idx].granularity);
    reef_event_t a, b;
    GPU_RETURN_STATUS(reef_event_create(&a));
    GPU_RETURN_STATUS(reef_event_create(&b));
    Status st = Status::Succ;
    auto once = [&]() {
        int rc = reef_dispatch(nullptr, nullptr, kernels[idx], raw_args[idx].data(), 0, blocks, 0, occupancy,
                               task_slot_base + (size_t)idx * 4, dispatch_ctrl, dispatch_ctrl, s, nullptr);
        if (rc != REEF_SUCC) { err_ = reef_last_error(); st = (Status)rc; }
    };
    once();
    reef_event_record(a, s);
    for (int r = 0; r < iters && st == Status::Succ; r++) once();
    reef_event_record(b, s);
    reef_event_sync(b);
    float ms = 0;
    reef_event_elapsed_ms(a, b, &ms);
    *us = ms * 1000.f / (float)std::max(1, iters);
    reset_task_slots(s, 0);
    reef_stream_sync(s);
    reef_event_destroy(a);
    reef_event_destroy(b);
    return st;
}

Status HybridExecutor::measure_profile(int iters, ModelProfile* out) {
    if (iters < 1) iters = 1;
    reef_event_t a, b;
    GPU_RETURN_STATUS(reef_event_create(&a));
    GPU_RETURN_STATUS(reef_event_create(&b));
    out->kernel_latency.clear();
    out->latency_unit_ns = 1;
    Status st = Status::Succ;
    auto elapsed_ns = [&](int n) {
        float ms = 0;
        reef_event_sync(b);
        reef_event_elapsed_ms(a, b, &ms);
        return (int)(ms * 1e6f / (float)n);
    };
    for (size_t i = 0; i < num_kernels() && st == Status::Succ; i++) {
        const std::string& name = model->kernels[i].name;
        if (out->kernel_latency.count(name)) continue;
        KernelProfile kp;
        for (int r = 0; r < 3 && st == Status::Succ; r++) st = ExecutorBase::launch_kernel((int)i, s);   // warm
        reef_event_record(a, s);
        for (int r = 0; r < iters && st == Status::Succ; r++) st = ExecutorBase::launch_kernel((int)i, s);
        reef_event_record(b, s);
        kp.total_latency = std::max(1, elapsed_ns(iters));
        const KernelArg& ka = trans_args[i];
        const int max_occ = std::max(1, std::min(4, ka.resource.max_blocks_per_sm));
        for (int occ = 1; occ <= max_occ && st == Status::Succ; occ++) {
            if (ka.resource.tensor_core) {
                kp.latency.push_back(kp.total_latency);   // one CTA per SM: a wave is the kernel
                continue;
            }
            float us = 0;
            st = profile_wave((int)i, occ, iters, &us);
            kp.latency.push_back(std::max(1, (int)(us * 1000.f)));
        }
        out->kernel_latency.insert({name, kp});
    }
    if (st == Status::Succ) {
        for (int r = 0; r < 3 && st == Status::Succ; r++) st = execute_graph(s);
        reef_event_record(a, s);
        for (int r = 0; r < iters && st == Status::Succ; r++) st = execute_graph(s);
        reef_event_record(b, s);
        out->model_latency = std::max(1, elapsed_ns(iters));
    }
    reef_event_destroy(a);
    reef_event_destroy(b);
    return st;
}

}  // namespace executor
}  // namespace reef
