// C entry points over the C++ host classes (see include/reef_host.h).
#include "../../../include/reef_host.h"

#include <pthread.h>
#include <sched.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <thread>
#include <vector>

#include "executor.h"
#include "scheduler.h"

using namespace reef;
using reef::executor::HybridExecutor;
using reef::server::REEFScheduler;

struct reef_executor_s {
    int device;
    HybridExecutor exe;
};
struct reef_scheduler_s {
    REEFScheduler* sched;
};

extern "C" {

int reef_model_parse(const char* json_path, size_t* ns, size_t* nk, size_t* na) {
    std::unique_ptr<executor::Model> m(executor::Model::from_json(json_path));
    if (!m) return NotFound;
    if (ns) *ns = m->storage.size();
    if (nk) *nk = m->kernels.size();
    if (na) *na = m->args.size();
    return Succ;
}

int reef_model_check(const char* json_path, char* err, size_t err_len) {
    std::string e;
    auto fail = [&](int rc) {
        if (err && err_len) snprintf(err, err_len, "%s", e.c_str());
        return rc;
    };
    std::unique_ptr<executor::Model> m(executor::Model::from_json(json_path, &e));
    if (!m) return fail(NotFound);
    reef_module_t mod = nullptr;
    if (reef_module_open(nullptr, &mod) != REEF_SUCC) return fail(Fail);
    std::vector<reef_kernel_t> ks;
    std::vector<uint32_t> smem;
    Status st = executor::ExecutorBase::resolve_kernels(*m, mod, &ks, &smem, &e);
    reef_module_close(mod);
    return st == Succ ? Succ : fail(st);
}

int reef_param_parse(const char* param_path, const char* key, size_t* key_elems, size_t* num_blobs) {
    std::unique_ptr<executor::ModelParam> p(executor::ModelParamParser::parse_from_file(param_path));
    if (!p) return NotFound;
    if (num_blobs) *num_blobs = p->size();
    if (key_elems) {
        const executor::ParamBlob* b = key ? p->find(key) : nullptr;
        *key_elems = b ? b->count : 0;
    }
    return Succ;
}

int reef_profile_parse(const char* profile_path, size_t* num_kernels, int* model_latency, int* min_latency) {
    std::unique_ptr<executor::ModelProfile> p(executor::ModelProfile::from_json(profile_path));
    if (!p) return NotFound;
    if (num_kernels) *num_kernels = p->kernel_latency.size();
    if (model_latency) *model_latency = p->model_latency;
    if (min_latency) {
        int m = 1 << 30;
        for (auto& kv : p->kernel_latency) {
            if (kv.second.latency.empty()) m = 0;
            for (int v : kv.second.latency) m = std::min(m, v);
        }
        *min_latency = m;
    }
    return Succ;
}

// ---- executor ------------------------------------------------------------------------------
int reef_executor_create(int device, reef_executor_t* e) {
    int rc = reef_gpu_init(device);
    if (rc != REEF_SUCC) return rc;
    *e = new reef_executor_s{device, {}};
    return Succ;
}
int reef_executor_destroy(reef_executor_t e) {
    if (e) {
        reef_gpu_init(e->device);
        delete e;
    }
    return Succ;
}
const char* reef_executor_error(reef_executor_t e) { return e ? e->exe.error().c_str() : ""; }
int reef_executor_load(reef_executor_t e, const char* json_path, const char* profile_path) {
    reef_gpu_init(e->device);
    return e->exe.load_hybrid_model_from_file(json_path, profile_path);
}
int reef_executor_load_param(reef_executor_t e, const char* param_path) {
    reef_gpu_init(e->device);
    return e->exe.load_param_from_file(param_path);
}
int reef_executor_num_kernels(reef_executor_t e, size_t* n) { *n = e->exe.num_kernels(); return Succ; }
int reef_executor_num_storage(reef_executor_t e, size_t* n) {
    *n = e->exe.model ? e->exe.model->storage.size() : 0;
    return Succ;
}
int reef_executor_get_data_size(reef_executor_t e, const char* name, size_t* bytes) {
    return e->exe.get_data_size(name, *bytes);
}
int reef_executor_set_input(reef_executor_t e, const char* name, const void* data, size_t len) {
    return e->exe.set_input(std::string(name), data, len);
}
int reef_executor_get_output(reef_executor_t e, void* out, size_t len) { return e->exe.get_output(out, len); }
int reef_executor_get_data(reef_executor_t e, int idx, void* out, size_t len) { return e->exe.get_data(idx, out, len); }
int reef_executor_execute(reef_executor_t e) { return e->exe.execute(); }
int reef_executor_execute_to(reef_executor_t e, int idx) { return e->exe.execute_to(idx); }
int reef_executor_execute_kernel(reef_executor_t e, int idx) { return e->exe.execute_kernel(idx); }
int reef_executor_execute_preemptable(reef_executor_t e) { return e->exe.execute_preemptale(); }
int reef_executor_execute_graph(reef_executor_t e) {
    Status st = e->exe.execute_graph(e->exe.stream());
    if (st != Succ) return st;
    return reef_stream_sync(e->exe.stream());
}
int reef_executor_execute_dispatch(reef_executor_t e) { return e->exe.execute_dispatch(); }
int reef_executor_build_chains(reef_executor_t e, int clusters, size_t* num_chains) {
    reef_gpu_init(e->device);
    Status st = e->exe.build_chains(clusters);
    if (num_chains) *num_chains = e->exe.num_chains();
    return st;
}
int reef_executor_execute_chained(reef_executor_t e) { return e->exe.execute_chained(); }
int reef_executor_execute_preempt_resume_chained(reef_executor_t e, int delay_us, int clusters, int* restarts, int* first_incomplete) {
    return e->exe.execute_preempt_resume_chained(delay_us, clusters, restarts, first_incomplete);
}
int reef_executor_execute_preemptable_chained(reef_executor_t e, int clusters) { return e->exe.execute_preemptable_chained(clusters); }
int reef_executor_set_stream_priority(reef_executor_t e, int high) {
    reef_gpu_init(e->device);
    reef_stream_t st = nullptr;
    int rc = reef_stream_create(&st, high);
    if (rc != REEF_SUCC) return rc;
    e->exe.set_stream(st);    // the executor keeps the new stream for its lifetime (the old one stays allocated)
    return Succ;
}
int reef_executor_chain_info(reef_executor_t e, size_t idx, int* begin, int* end, int* clusters, int* max_clusters) {
    return e->exe.chain_info(idx, begin, end, clusters, max_clusters);
}
int reef_executor_execute_preempt_resume(reef_executor_t e, int delay_us, int* restarts, int* first_incomplete,
                                         int* first_count) {
    return e->exe.execute_preempt_resume(delay_us, restarts, first_incomplete, first_count);
}
int reef_executor_task_slots(reef_executor_t e, int* slots, int* block_nums, size_t n) {
    if (n < e->exe.num_kernels()) return OutOfRange;
    e->exe.copy_be_kernel_offset(e->exe.stream());
    int rc = reef_stream_sync(e->exe.stream());
    if (rc != REEF_SUCC) return rc;
    for (size_t i = 0; i < e->exe.num_kernels(); i++) {
        if (slots) slots[i] = e->exe.host_task_slots()[i];
        if (block_nums) block_nums[i] = e->exe.trans_args[i].block_num;
    }
    return Succ;
}
int reef_executor_time(reef_executor_t e, int mode, int warmup, int iters, float* avg_ms) {
    reef_event_t a, b;
    if (reef_event_create(&a) != REEF_SUCC || reef_event_create(&b) != REEF_SUCC) return Fail;
    auto once = [&]() -> int {
        if (mode == 1) return e->exe.execute_graph(e->exe.stream());
        Status st = Succ;
        for (size_t i = 0; i < e->exe.num_kernels() && st == Succ; i++)
            st = mode == 2 ? e->exe.launch_preempt_kernel((int)i, e->exe.stream())
                           : (Status)e->exe.execute_kernel_async((int)i);
        return st;
    };
    int rc = Succ;
    for (int i = 0; i < warmup && rc == Succ; i++) rc = once();
    reef_stream_sync(e->exe.stream());
    reef_event_record(a, e->exe.stream());
    for (int i = 0; i < iters && rc == Succ; i++) rc = once();
    reef_event_record(b, e->exe.stream());
    reef_event_sync(b);
    float ms = 0;
    reef_event_elapsed_ms(a, b, &ms);
    *avg_ms = ms / (float)std::max(1, iters);
    reef_event_destroy(a);
    reef_event_destroy(b);
    return rc;
}
int reef_executor_time_tensor_core(reef_executor_t e, int warmup, int iters, float* avg_ms, int* launches) {
    // a CUDA graph of the tensor-core kernels alone, in schedule order (they keep their programmatic
    // dependencies on one another; the kernels between them are left out, so their inputs are stale, which
    // does not change what a launch costs)
    auto& exe = e->exe;
    int n = 0;
    for (size_t i = 0; i < exe.num_kernels(); i++) n += exe.trans_args[i].resource.tensor_core ? 1 : 0;
    if (launches) *launches = n;
    if (n == 0) return NotFound;
    reef_graph_t g = nullptr;
    if (reef_graph_begin(exe.stream()) != REEF_SUCC) return Fail;
    Status st = Succ;
    for (size_t i = 0; i < exe.num_kernels() && st == Succ; i++)
        if (exe.trans_args[i].resource.tensor_core) st = (Status)exe.execute_kernel_async((int)i);
    int rc = reef_graph_end(exe.stream(), &g);
    if (st != Succ || rc != REEF_SUCC) {
        if (g) reef_graph_destroy(g);
        return Fail;
    }
    reef_event_t a, b;
    if (reef_event_create(&a) != REEF_SUCC || reef_event_create(&b) != REEF_SUCC) return Fail;
    for (int i = 0; i < warmup && rc == REEF_SUCC; i++) rc = reef_graph_launch(g, exe.stream());
    reef_stream_sync(exe.stream());
    reef_event_record(a, exe.stream());
    for (int i = 0; i < iters && rc == REEF_SUCC; i++) rc = reef_graph_launch(g, exe.stream());
    reef_event_record(b, exe.stream());
    reef_event_sync(b);
    float ms = 0;
    reef_event_elapsed_ms(a, b, &ms);
    *avg_ms = ms / (float)std::max(1, iters);
    reef_event_destroy(a);
    reef_event_destroy(b);
    reef_graph_destroy(g);
    return rc == REEF_SUCC ? Succ : Fail;
}
int reef_executor_time_kernel(reef_executor_t e, int idx, int reps, int warmup, int iters, float* us_per_launch) {
    // a CUDA graph of `reps` back-to-back launches of kernel idx alone (its inputs are whatever the buffers hold),
    // replayed `iters` times between two events after `warmup` replays
    auto& exe = e->exe;
    if (idx < 0 || (size_t)idx >= exe.num_kernels() || reps < 1 || iters < 1) return OutOfRange;
    reef_graph_t g = nullptr;
    if (reef_graph_begin(exe.stream()) != REEF_SUCC) return Fail;
    Status st = Succ;
    for (int r = 0; r < reps && st == Succ; r++) st = (Status)exe.execute_kernel_async(idx);
    int rc = reef_graph_end(exe.stream(), &g);
    if (st != Succ || rc != REEF_SUCC) {
        if (g) reef_graph_destroy(g);
        return Fail;
    }
    reef_event_t a, b;
    if (reef_event_create(&a) != REEF_SUCC || reef_event_create(&b) != REEF_SUCC) return Fail;
    for (int i = 0; i < warmup && rc == REEF_SUCC; i++) rc = reef_graph_launch(g, exe.stream());
    reef_stream_sync(exe.stream());
    reef_event_record(a, exe.stream());
    for (int i = 0; i < iters && rc == REEF_SUCC; i++) rc = reef_graph_launch(g, exe.stream());
    reef_event_record(b, exe.stream());
    reef_event_sync(b);
    float ms = 0;
    reef_event_elapsed_ms(a, b, &ms);
    *us_per_launch = ms * 1000.f / (float)(iters * reps);
    reef_event_destroy(a);
    reef_event_destroy(b);
    reef_graph_destroy(g);
    return rc == REEF_SUCC ? Succ : Fail;
}
int reef_executor_profile_kernels(reef_executor_t e, int iters, float* us, double* flops, double* bytes,
                                  int* tensor_core, int* blocks, int* max_blocks_per_sm, size_t n) {
    if (n < e->exe.num_kernels()) return OutOfRange;
    Status st = e->exe.profile_kernels(iters, us);
    for (size_t i = 0; i < e->exe.num_kernels(); i++) {
        const reef_kernel_attrs_t& r = e->exe.trans_args[i].resource;
        if (flops) flops[i] = r.flops;
        if (bytes) bytes[i] = r.bytes;
        if (tensor_core) tensor_core[i] = r.tensor_core;
        if (blocks) blocks[i] = r.num_blocks;
        if (max_blocks_per_sm) max_blocks_per_sm[i] = r.max_blocks_per_sm;
    }
    return st;
}
int reef_executor_profile_wave(reef_executor_t e, int idx, int occupancy, int iters, float* us) {
    return e->exe.profile_wave(idx, occupancy, iters, us);
}

int reef_executor_write_profile(reef_executor_t e, int iters, const char* out_path) {
    executor::ModelProfile prof;
    Status st = e->exe.measure_profile(iters, &prof);
    if (st != Succ) return st;
    FILE* f = fopen(out_path, "w");
    if (!f) return Fail;
    std::string js = prof.to_json();
    fwrite(js.data(), 1, js.size(), f);
    fclose(f);
    return Succ;
}

// ---- scheduler -----------------------------------------------------------------------------
int reef_sched_create(int mode, int device, reef_scheduler_t* s) {
    if (mode < 0 || mode > 4) return OutOfRange;
    *s = new reef_scheduler_s{new REEFScheduler((REEFScheduler::ScheduleMode)mode, device)};
    return Succ;
}
int reef_sched_destroy(reef_scheduler_t s) {
    if (s) {
        delete s->sched;
        delete s;
    }
    return Succ;
}
const char* reef_sched_error(reef_scheduler_t s) { return s->sched->error().c_str(); }
int reef_sched_load_model(reef_scheduler_t s, const char* dir, const char* name, uint32_t* mid) {
    return s->sched->load_model(dir, name, *mid);
}
int reef_sched_load_model_files(reef_scheduler_t s, const char* json_path, const char* profile_path,
                                const char* param_path, uint32_t* mid) {
    return s->sched->load_model("", "", json_path, profile_path ? profile_path : "", param_path ? param_path : "", *mid);
}
int reef_sched_create_queue(reef_scheduler_t s, int type, uint32_t* qid) {
    return s->sched->create_queue(type == 0 ? REEFScheduler::RealTimeQueue : REEFScheduler::BestEffortQueue, *qid);
}
int reef_sched_bind_model_queue(reef_scheduler_t s, uint32_t qid, uint32_t mid) { return s->sched->bind_model_queue(qid, mid); }
int reef_sched_get_data_size(reef_scheduler_t s, uint32_t mid, const char* name, size_t* bytes) {
    return s->sched->get_data_size(mid, name, *bytes);
}
int reef_sched_set_input(reef_scheduler_t s, uint32_t mid, const void* data, size_t len, const char* name) {
    return s->sched->set_input(mid, data, len, name ? name : "data");
}
int reef_sched_get_output(reef_scheduler_t s, uint32_t mid, void* data, size_t len, const char* name) {
    return s->sched->get_output(mid, data, len, name ? name : "output");
}
int reef_sched_new_task(reef_scheduler_t s, uint32_t mid, uint32_t* tid) { return s->sched->new_task(mid, *tid); }
int reef_sched_wait_task(reef_scheduler_t s, uint32_t tid) { return s->sched->wait_task(tid); }
int reef_sched_task_info(reef_scheduler_t s, uint32_t tid, reef_task_info_t* info) {
    std::shared_ptr<REEFScheduler::Task> t;
    Status st = s->sched->get_task(tid, t);
    if (st != Succ) return st;
    info->state = (int)t->get_state();
    info->preempted = t->is_preempted();
    info->padded = t->is_padded();
    info->padded_to_complete = t->is_padded_to_complete();
    auto ts = t->get_timestamp();
    auto ns = [](std::chrono::system_clock::time_point p) {
        return (int64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(p.time_since_epoch()).count();
    };
    info->submit_ns = ns(ts[0]);
    info->start_ns = ns(ts[1]);
    info->end_ns = ns(ts[2]);
    info->failed = t->is_failed();
    return Succ;
}
int reef_sched_inject_launch_failures(reef_scheduler_t s, uint32_t mid, int n) {
    return s->sched->inject_launch_failures(mid, n);
}
int reef_sched_set_wait_sync(reef_scheduler_t s, int v) { s->sched->set_wait_sync(v != 0); return Succ; }
int reef_sched_set_be_stream_cap(reef_scheduler_t s, int v) { s->sched->set_be_stream_cap(v); return Succ; }
int reef_sched_use_mapped_flag(reef_scheduler_t s) { return s->sched->use_mapped_flag(); }
int reef_sched_set_sm_partition(reef_scheduler_t s, int be_sms, int flags, int* rt_sms, int* be_sms_out) {
    return s->sched->set_sm_partition(be_sms, flags, rt_sms, be_sms_out);
}
int reef_sched_set_device_stamps(reef_scheduler_t s, int on) { return s->sched->set_device_stamps(on != 0); }
int reef_sched_set_pad_slowdown_target(reef_scheduler_t s, double v) { s->sched->set_pad_slowdown_target(v); return Succ; }
int reef_sched_set_cpu_slice(reef_scheduler_t s, int first_cpu, int n_cpus) { s->sched->set_cpu_slice(first_cpu, n_cpus); return Succ; }
int reef_sched_set_rt_graph(reef_scheduler_t s, int v) { s->sched->set_rt_graph(v != 0); return Succ; }
int reef_sched_set_rt_chains(reef_scheduler_t s, int clusters) { s->sched->set_rt_chains(clusters); return Succ; }
int reef_sched_run(reef_scheduler_t s) { return s->sched->run(); }
int reef_sched_shutdown(reef_scheduler_t s) { return s->sched->shutdown(); }
int64_t reef_sched_avg_preempt_latency(reef_scheduler_t s) { return s->sched->avg_preempt_latency(); }
int64_t reef_sched_avg_kernel_sel_latency(reef_scheduler_t s) { return s->sched->avg_kernel_sel_latency(); }
int reef_sched_stats(reef_scheduler_t s, reef_sched_stats_t* out) {
    auto st = s->sched->stats();
    out->preempt_count = st.preempt_count;
    out->preempt_ns_sum = st.preempt_ns_sum;
    out->preempt_ns_max = st.preempt_ns_max;
    out->rt_tasks = st.rt_tasks;
    out->be_tasks = st.be_tasks;
    out->be_tasks_padded_to_finish = st.be_tasks_padded_to_finish;
    out->padded_kernels = st.padded_kernels;
    out->padded_blocks = st.padded_blocks;
    out->drain_count = st.drain_count;
    out->drain_ns_sum = st.drain_ns_sum;
    out->drain_ns_max = st.drain_ns_max;
    out->dev_count = st.dev_count;
    out->dev_ns_sum = st.dev_ns_sum;
    out->dev_ns_max = st.dev_ns_max;
    out->drain_ns_p50 = st.drain_ns_p50;
    out->drain_ns_p99 = st.drain_ns_p99;
    return Succ;
}

// ---- closed-loop clients -------------------------------------------------------------------
// All clients are measured over ONE window: a bounded client records from its first request after its warm-up,
// and a background client (max_requests == 0) starts to count with the first request it submits once every
// bounded client has finished warming up, so the throughputs of the two kinds can be added.
int reef_run_clients(reef_scheduler_t s, reef_client_t* clients, size_t n) {
    std::atomic<int> bounded_left(0), warming(0);
    std::atomic<int> failed(0);
    for (size_t i = 0; i < n; i++)
        if (clients[i].max_requests > 0) {
            bounded_left++;
            if (clients[i].warmup_requests > 0) warming++;
        }
    if (bounded_left.load() == 0) return OutOfRange;
    std::vector<std::thread> threads;
    for (size_t i = 0; i < n; i++) {
        threads.emplace_back([&, i] {
            reef_client_t& c = clients[i];
            REEFScheduler* sc = s->sched;
            const bool bounded = c.max_requests > 0;
            {
                // CPU placement inside the scheduler's slice: the real-time client gets a core of its own next to the
                // scheduler thread's, best-effort clients share the rest
                int first = -1, count = 0;
                sc->cpu_slice(&first, &count);
                if (first >= 0 && count >= 3) {
                    cpu_set_t set;
                    CPU_ZERO(&set);
                    if (sc->is_realtime_model(c.mid)) {
                        CPU_SET(first + 1, &set);
                    } else {
                        for (int k = 2; k < count; k++) CPU_SET(first + k, &set);
                    }
                    pthread_setaffinity_np(pthread_self(), sizeof(set), &set);
                }
            }
            const std::string in_name = c.input_name ? c.input_name : "data";
            uint64_t done = 0;
            c.completed = 0;
            c.failed = 0;
            c.elapsed_s = 0;
            bool recording = false;
            auto t_first = std::chrono::steady_clock::now();
            for (uint64_t r = 0;; r++) {
                if (bounded ? (r >= (uint64_t)c.warmup_requests + c.max_requests) : (bounded_left.load() == 0)) break;
                if (!recording && (bounded ? r == c.warmup_requests : warming.load() == 0)) {
                    if (bounded && c.warmup_requests > 0) warming--;
                    recording = true;
                    t_first = std::chrono::steady_clock::now();
                }
                auto t0 = std::chrono::steady_clock::now();
                uint32_t tid;
                if ((c.input && sc->set_input(c.mid, c.input, c.input_len, in_name) != Succ) ||
                    sc->new_task(c.mid, tid) != Succ || sc->wait_task(tid) != Succ ||
                    (c.output && sc->get_output(c.mid, c.output, c.output_len) != Succ)) {
                    // a task that ended in error (wait_task returns Fail) ends this client
                    c.failed = 1;
                    failed++;
                    break;
                }
                auto t1 = std::chrono::steady_clock::now();
                if (recording) {
                    if (bounded && c.latencies_ms)
                        c.latencies_ms[done] = (float)(std::chrono::duration_cast<std::chrono::nanoseconds>(t1 - t0).count() * 1e-6);
                    done++;
                    c.completed = done;
                    c.elapsed_s = std::chrono::duration_cast<std::chrono::nanoseconds>(t1 - t_first).count() * 1e-9;
                }
                if (c.think_us) std::this_thread::sleep_for(std::chrono::microseconds(c.think_us));
            }
            if (bounded) {
                if (!recording && c.warmup_requests > 0) warming--;   // left early: do not hold the others' window shut
                bounded_left--;
            }
        });
    }
    for (auto& t : threads) t.join();
    return failed.load() ? Fail : Succ;
}

}  // extern "C"
