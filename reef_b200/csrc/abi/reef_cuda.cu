// C-ABI device layer (see include/reef_cuda.h for the reference symbols each entry point replaces).
#include <cuda.h>
#include <chrono>
#include <cstring>
#include <new>
#include <string>
#include <algorithm>
#include <thread>
#include <vector>

#include "../kernels/registry.h"
#ifdef REEF_DEBUG_AIDS
#include "../../../include/reef_debug_aids.h"
#endif

using namespace reef;

struct reef_module_s {
    std::string path;
    std::vector<reef_kernel_s*> kernels;
};
struct reef_kernel_s {
    KernelSpec spec;
};
struct reef_graph_s {
    cudaGraph_t graph;
    cudaGraphExec_t exec;
    unsigned long long kernels;
};

static int g_num_sms = 0;

#define CK(call)                                                                 \
    do {                                                                         \
        cudaError_t _e = (call);                                                 \
        if (_e != cudaSuccess) {                                                 \
            set_error(std::string(#call) + ": " + cudaGetErrorString(_e));       \
            return REEF_FAIL;                                                    \
        }                                                                        \
    } while (0)

extern "C" {

const char* reef_last_error(void) { return last_error(); }

static thread_local int t_device = -1;

reef_status reef_gpu_init(int device) {
    if (t_device == device) return REEF_SUCC;   // this thread is already bound
    CK(cudaSetDevice(device));
    CK(cudaFree(0));
    cudaDeviceProp prop;
    CK(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        set_error("libreef_cuda is built for sm_100a only; device is sm_" + std::to_string(prop.major) +
                  std::to_string(prop.minor));
        return REEF_FAIL;
    }
    g_num_sms = prop.multiProcessorCount;
    t_device = device;
    return REEF_SUCC;
}

reef_status reef_device_count(int* count) {
    CK(cudaGetDeviceCount(count));
    return REEF_SUCC;
}

reef_status reef_device_num_sms(int* n) {
    if (g_num_sms == 0) {
        int dev;
        CK(cudaGetDevice(&dev));
        CK(cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev));
    }
    *n = g_num_sms;
    return REEF_SUCC;
}

reef_status reef_device_sync(void) {
    CK(cudaDeviceSynchronize());
    return REEF_SUCC;
}

reef_status reef_malloc(reef_dptr_t* ptr, size_t bytes) {
    void* p = nullptr;
    CK(cudaMalloc(&p, bytes ? bytes : 4));
    *ptr = (reef_dptr_t)p;
    return REEF_SUCC;
}
reef_status reef_free(reef_dptr_t ptr) {
    CK(cudaFree((void*)ptr));
    return REEF_SUCC;
}
// The synchronous forms return only when the bytes are in device memory.  cudaMemset and a cudaMemcpy from
// pageable host memory may return while the device-side write is still in flight on the legacy stream, and
// the executors launch on non-blocking streams, which the legacy stream does not order.
reef_status reef_memset(reef_dptr_t ptr, int value, size_t bytes) {
    CK(cudaMemset((void*)ptr, value, bytes));
    CK(cudaStreamSynchronize(cudaStreamLegacy));
    return REEF_SUCC;
}
reef_status reef_memset_async(reef_dptr_t ptr, int value, size_t bytes, reef_stream_t s) {
    CK(cudaMemsetAsync((void*)ptr, value, bytes, (cudaStream_t)s));
    return REEF_SUCC;
}
reef_status reef_memcpy_h2d(reef_dptr_t dst, const void* src, size_t bytes) {
    CK(cudaMemcpy((void*)dst, src, bytes, cudaMemcpyHostToDevice));
    CK(cudaStreamSynchronize(cudaStreamLegacy));
    return REEF_SUCC;
}
reef_status reef_memcpy_d2h(void* dst, reef_dptr_t src, size_t bytes) {
    CK(cudaMemcpy(dst, (const void*)src, bytes, cudaMemcpyDeviceToHost));
    return REEF_SUCC;
}
reef_status reef_memcpy_h2d_async(reef_dptr_t dst, const void* src, size_t bytes, reef_stream_t s) {
    CK(cudaMemcpyAsync((void*)dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)s));
    return REEF_SUCC;
}
reef_status reef_memcpy_d2h_async(void* dst, reef_dptr_t src, size_t bytes, reef_stream_t s) {
    CK(cudaMemcpyAsync(dst, (const void*)src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)s));
    return REEF_SUCC;
}
reef_status reef_host_alloc_pinned(void** ptr, size_t bytes) {
    CK(cudaHostAlloc(ptr, bytes ? bytes : 4, cudaHostAllocDefault));
    return REEF_SUCC;
}
reef_status reef_host_free_pinned(void* ptr) {
    CK(cudaFreeHost(ptr));
    return REEF_SUCC;
}

reef_status reef_stream_create(reef_stream_t* s, int high_priority) {
    int lo = 0, hi = 0;
    CK(cudaDeviceGetStreamPriorityRange(&lo, &hi));   // hi is the numerically lowest = greatest priority
    cudaStream_t st;
    CK(cudaStreamCreateWithPriority(&st, cudaStreamNonBlocking, high_priority ? hi : lo));
    *s = (reef_stream_t)st;
    return REEF_SUCC;
}
reef_status reef_stream_destroy(reef_stream_t s) {
    CK(cudaStreamDestroy((cudaStream_t)s));
    return REEF_SUCC;
}
reef_status reef_stream_sync(reef_stream_t s) {
    CK(cudaStreamSynchronize((cudaStream_t)s));
    return REEF_SUCC;
}
reef_status reef_stream_query(reef_stream_t s, int* busy) {
    cudaError_t e = cudaStreamQuery((cudaStream_t)s);
    if (e == cudaSuccess) { *busy = 0; return REEF_SUCC; }
    if (e == cudaErrorNotReady) { *busy = 1; return REEF_SUCC; }
    set_error(std::string("cudaStreamQuery: ") + cudaGetErrorString(e));
    return REEF_FAIL;
}
typedef int (*write_value32_fn)(cudaStream_t, unsigned long long, unsigned int, unsigned int);
static write_value32_fn g_write32 = nullptr;
static int g_write32_state = 0;   // 0 unknown, 1 driver entry point, 2 pinned-constant copy
static uint32_t* g_flag_consts = nullptr;

reef_status reef_write32_async(reef_stream_t s, reef_dptr_t ptr, uint32_t value) {
    if (g_write32_state == 0) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuStreamWriteValue32", &fn, cudaEnableDefault, &q);
        if (e == cudaSuccess && q == cudaDriverEntryPointSuccess && fn != nullptr) {
            g_write32 = (write_value32_fn)fn;
            g_write32_state = 1;
        } else {
            (void)cudaGetLastError();
            CK(cudaHostAlloc((void**)&g_flag_consts, 256 * sizeof(uint32_t), cudaHostAllocDefault));
            for (uint32_t i = 0; i < 256; i++) g_flag_consts[i] = i;
            g_write32_state = 2;
        }
    }
    if (g_write32_state == 1) {
        // (the no-memory-barrier form of the write is refused by this driver with CUDA_ERROR_INVALID_VALUE)
        int rc = g_write32((cudaStream_t)s, (unsigned long long)ptr, value, 0);
        if (rc != 0) {
            set_error("cuStreamWriteValue32 failed with CUresult " + std::to_string(rc));
            return REEF_FAIL;
        }
        return REEF_SUCC;
    }
    if (value > 255) {
        set_error("reef_write32_async: fallback path supports values 0..255");
        return REEF_OUT_OF_RANGE;
    }
    CK(cudaMemcpyAsync((void*)ptr, &g_flag_consts[value], 4, cudaMemcpyHostToDevice, (cudaStream_t)s));
    return REEF_SUCC;
}

// ---- SM partition (green contexts) ------------------------------------------------------------------------------
// The driver entry points are looked up at run time (the library links the runtime only).
struct reef_partition_s {
    CUgreenCtx ctx[2] = {nullptr, nullptr};   // [0] real-time side, [1] best-effort side
    int sms[2] = {0, 0};
};
namespace {
typedef CUresult (*fn_get_dev_resource)(CUdevice, CUdevResource*, CUdevResourceType);
typedef CUresult (*fn_split_by_count)(CUdevResource*, unsigned int*, const CUdevResource*, CUdevResource*, unsigned int, unsigned int);
typedef CUresult (*fn_generate_desc)(CUdevResourceDesc*, CUdevResource*, unsigned int);
typedef CUresult (*fn_green_create)(CUgreenCtx*, CUdevResourceDesc, CUdevice, unsigned int);
typedef CUresult (*fn_green_destroy)(CUgreenCtx);
typedef CUresult (*fn_green_stream)(CUstream*, CUgreenCtx, unsigned int, int);
typedef CUresult (*fn_device_get)(CUdevice*, int);
void* driver_fn(const char* name) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    return fn;
}
reef_status cu_fail(const char* what, CUresult r) {
    set_error(std::string(what) + " failed with CUresult " + std::to_string((int)r));
    return REEF_FAIL;
}
}  // namespace

reef_status reef_partition_create(int be_sms, int flags, reef_partition_t* out) {
    auto get_res = (fn_get_dev_resource)driver_fn("cuDeviceGetDevResource");
    auto split = (fn_split_by_count)driver_fn("cuDevSmResourceSplitByCount");
    auto gen = (fn_generate_desc)driver_fn("cuDevResourceGenerateDesc");
    auto create = (fn_green_create)driver_fn("cuGreenCtxCreate");
    auto dev_get = (fn_device_get)driver_fn("cuDeviceGet");
    if (!get_res || !split || !gen || !create || !dev_get) {
        set_error("reef_partition_create: this driver has no green contexts");
        return REEF_FAIL;
    }
    int ordinal = 0;
    CK(cudaGetDevice(&ordinal));
    CK(cudaFree(0));
    CUdevice dev;
    CUresult r = dev_get(&dev, ordinal);
    if (r != CUDA_SUCCESS) return cu_fail("cuDeviceGet", r);
    CUdevResource all;
    r = get_res(dev, &all, CU_DEV_RESOURCE_TYPE_SM);
    if (r != CUDA_SUCCESS) return cu_fail("cuDeviceGetDevResource", r);
    const int total = (int)all.sm.smCount;
    if (be_sms < 1 || be_sms >= total) {
        set_error("reef_partition_create: best-effort SM count outside 1.." + std::to_string(total - 1));
        return REEF_OUT_OF_RANGE;
    }
    if (flags & 8) {
        // both sides are made of whole groups of 8 SMs (the driver's granularity here): the best-effort side takes the
        // first ceil(be_sms / 8) groups, the real-time side all the others; the remainder of the split is left unused
        CUdevResource groups[32], rest8;
        unsigned int ng = 32;
        r = split(groups, &ng, &all, &rest8, (flags & 2) ? CU_DEV_SM_RESOURCE_SPLIT_MAX_POTENTIAL_CLUSTER_SIZE : 0u, 8u);
        if (r != CUDA_SUCCESS) return cu_fail("cuDevSmResourceSplitByCount(8)", r);
        const unsigned int nbe = (unsigned int)((be_sms + 7) / 8);
        if (nbe >= ng) {
            set_error("reef_partition_create: no group left for the real-time side");
            return REEF_OUT_OF_RANGE;
        }
        reef_partition_s* p8 = new (std::nothrow) reef_partition_s();
        if (!p8) return REEF_FAIL;
        CUdevResource* first[2] = {groups + nbe, groups};
        const unsigned int cnt[2] = {ng - nbe, nbe};
        for (int i = 0; i < 2; i++) {
            CUdevResourceDesc desc;
            r = gen(&desc, first[i], cnt[i]);
            if (r == CUDA_SUCCESS) r = create(&p8->ctx[i], desc, dev, CU_GREEN_CTX_DEFAULT_STREAM);
            if (r != CUDA_SUCCESS) {
                reef_partition_destroy(p8);
                return cu_fail("cuGreenCtxCreate (groups of 8)", r);
            }
            for (unsigned int g = 0; g < cnt[i]; g++) p8->sms[i] += (int)first[i][g].sm.smCount;
        }
        *out = p8;
        return REEF_SUCC;
    }
    const bool group_is_rt = (flags & 1) != 0;
    const unsigned int use = (flags & 2) ? CU_DEV_SM_RESOURCE_SPLIT_MAX_POTENTIAL_CLUSTER_SIZE : 0u;
    CUdevResource group, rest;
    unsigned int n = 1;
    r = split(&group, &n, &all, &rest, use, (unsigned int)(group_is_rt ? total - be_sms : be_sms));
    if (r != CUDA_SUCCESS || n != 1) return cu_fail("cuDevSmResourceSplitByCount", r);
    if (rest.sm.smCount == 0) {
        set_error("reef_partition_create: the split left no SMs for the other side");
        return REEF_OUT_OF_RANGE;
    }
    reef_partition_s* p = new (std::nothrow) reef_partition_s();
    if (!p) return REEF_FAIL;
    CUdevResource* side[2] = {group_is_rt ? &group : &rest, group_is_rt ? &rest : &group};
    for (int i = 0; i < 2; i++) {
        CUdevResourceDesc desc;
        r = gen(&desc, side[i], 1);
        if (r == CUDA_SUCCESS) r = create(&p->ctx[i], desc, dev, CU_GREEN_CTX_DEFAULT_STREAM);
        if (r != CUDA_SUCCESS) {
            reef_partition_destroy(p);
            return cu_fail("cuGreenCtxCreate", r);
        }
        p->sms[i] = (int)side[i]->sm.smCount;
    }
    *out = p;
    return REEF_SUCC;
}
reef_status reef_partition_info(reef_partition_t p, int* rt_sms, int* be_sms) {
    if (!p) return REEF_FAIL;
    if (rt_sms) *rt_sms = p->sms[0];
    if (be_sms) *be_sms = p->sms[1];
    return REEF_SUCC;
}
reef_status reef_partition_stream_create(reef_partition_t p, int best_effort, int high_priority, reef_stream_t* s) {
    auto mk = (fn_green_stream)driver_fn("cuGreenCtxStreamCreate");
    if (!p || !mk) return REEF_FAIL;
    int lo = 0, hi = 0;
    CK(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    CUstream st = nullptr;
    CUresult r = mk(&st, p->ctx[best_effort ? 1 : 0], CU_STREAM_NON_BLOCKING, high_priority ? hi : lo);
    if (r != CUDA_SUCCESS) return cu_fail("cuGreenCtxStreamCreate", r);
    *s = (reef_stream_t)st;
    return REEF_SUCC;
}
reef_status reef_partition_destroy(reef_partition_t p) {
    if (!p) return REEF_SUCC;
    auto destroy = (fn_green_destroy)driver_fn("cuGreenCtxDestroy");
    for (int i = 0; i < 2; i++)
        if (p->ctx[i] && destroy) destroy(p->ctx[i]);
    delete p;
    return REEF_SUCC;
}

reef_status reef_probe_stream_latency(int iters, double* write_call_us, double* write_complete_us,
                                      double* event_round_trip_us, double* timed_event_round_trip_us) {
    using clk = std::chrono::steady_clock;
    auto us = [](clk::time_point a, clk::time_point b) { return std::chrono::duration<double, std::micro>(b - a).count(); };
    if (iters < 10) iters = 10;
    cudaStream_t st;
    int lo = 0, hi = 0;
    CK(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    CK(cudaStreamCreateWithPriority(&st, cudaStreamNonBlocking, hi));
    void* flag = nullptr;
    cudaEvent_t ev;
    CK(cudaMalloc(&flag, 256));
    CK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    cudaEvent_t evt;
    CK(cudaEventCreate(&evt));
    std::vector<double> a, b, c, d;
    reef_status rc = REEF_SUCC;
    for (int i = 0; i < iters + iters / 10 && rc == REEF_SUCC; i++) {
        auto t0 = clk::now();
        rc = reef_write32_async((reef_stream_t)st, (reef_dptr_t)flag, (uint32_t)(i & 1));
        auto t1 = clk::now();
        cudaEventRecord(ev, st);
        while (cudaEventQuery(ev) == cudaErrorNotReady) {}
        auto t2 = clk::now();
        cudaEventRecord(ev, st);
        while (cudaEventQuery(ev) == cudaErrorNotReady) {}
        auto t3 = clk::now();
        cudaEventRecord(evt, st);
        while (cudaEventQuery(evt) == cudaErrorNotReady) {}
        auto t4 = clk::now();
        if (i >= iters / 10) {
            a.push_back(us(t0, t1));
            b.push_back(us(t0, t2));
            c.push_back(us(t2, t3));
            d.push_back(us(t3, t4));
        }
        while (us(t4, clk::now()) < 200.0) {}
    }
    cudaEventDestroy(ev);
    cudaEventDestroy(evt);
    cudaFree(flag);
    cudaStreamDestroy(st);
    if (rc != REEF_SUCC) return rc;
    CK(cudaGetLastError());
    auto med = [](std::vector<double>& v) { std::sort(v.begin(), v.end()); return v[v.size() / 2]; };
    if (write_call_us) *write_call_us = med(a);
    if (write_complete_us) *write_complete_us = med(b);
    if (event_round_trip_us) *event_round_trip_us = med(c);
    if (timed_event_round_trip_us) *timed_event_round_trip_us = med(d);
    return REEF_SUCC;
}

reef_status reef_event_create(reef_event_t* e) {
    cudaEvent_t ev;
    CK(cudaEventCreate(&ev));
    *e = (reef_event_t)ev;
    return REEF_SUCC;
}
reef_status reef_event_create_untimed(reef_event_t* e) {
    cudaEvent_t ev;
    CK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    *e = (reef_event_t)ev;
    return REEF_SUCC;
}
reef_status reef_event_destroy(reef_event_t e) {
    CK(cudaEventDestroy((cudaEvent_t)e));
    return REEF_SUCC;
}
reef_status reef_event_record(reef_event_t e, reef_stream_t s) {
    CK(cudaEventRecord((cudaEvent_t)e, (cudaStream_t)s));
    return REEF_SUCC;
}
reef_status reef_event_sync(reef_event_t e) {
    CK(cudaEventSynchronize((cudaEvent_t)e));
    return REEF_SUCC;
}
reef_status reef_event_query(reef_event_t e, int* pending) {
    cudaError_t r = cudaEventQuery((cudaEvent_t)e);
    if (r == cudaSuccess) { *pending = 0; return REEF_SUCC; }
    if (r == cudaErrorNotReady) { *pending = 1; return REEF_SUCC; }
    set_error(std::string("cudaEventQuery: ") + cudaGetErrorString(r));
    return REEF_FAIL;
}
reef_status reef_event_elapsed_ms(reef_event_t a, reef_event_t b, float* ms) {
    CK(cudaEventElapsedTime(ms, (cudaEvent_t)a, (cudaEvent_t)b));
    return REEF_SUCC;
}
reef_status reef_stream_wait_event(reef_stream_t s, reef_event_t e) {
    CK(cudaStreamWaitEvent((cudaStream_t)s, (cudaEvent_t)e, 0));
    return REEF_SUCC;
}

// kernels of a capture = what the capturing thread launched between begin and end (other threads may launch
// at the same time; their launches are not part of this graph)
static thread_local unsigned long long g_capture_start = 0;
reef_status reef_graph_begin(reef_stream_t s) {
    g_capture_start = thread_launch_count();
    CK(cudaStreamBeginCapture((cudaStream_t)s, cudaStreamCaptureModeThreadLocal));
    return REEF_SUCC;
}
reef_status reef_graph_end(reef_stream_t s, reef_graph_t* g) {
    *g = nullptr;
    cudaGraph_t graph = nullptr;
    CK(cudaStreamEndCapture((cudaStream_t)s, &graph));
    cudaGraphExec_t exec;
    cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(graph);
        set_error(std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e));
        return REEF_FAIL;
    }
    reef_graph_s* h = new (std::nothrow) reef_graph_s{graph, exec, thread_launch_count() - g_capture_start};
    if (!h) {
        cudaGraphExecDestroy(exec);
        cudaGraphDestroy(graph);
        return REEF_FAIL;
    }
    *g = (reef_graph_t)h;
    return REEF_SUCC;
}
reef_status reef_graph_launch(reef_graph_t g, reef_stream_t s) {
    reef_graph_s* h = (reef_graph_s*)g;
    CK(cudaGraphLaunch(h->exec, (cudaStream_t)s));
    add_launches(h->kernels);
    return REEF_SUCC;
}
reef_status reef_graph_destroy(reef_graph_t g) {
    reef_graph_s* h = (reef_graph_s*)g;
    if (!h) return REEF_SUCC;
    cudaGraphExecDestroy(h->exec);
    cudaGraphDestroy(h->graph);
    delete h;
    return REEF_SUCC;
}

reef_status reef_module_open(const char* path, reef_module_t* mod) {
    reef_module_s* m = new (std::nothrow) reef_module_s;
    if (!m) return REEF_FAIL;
    if (path) m->path = path;
    *mod = m;
    return REEF_SUCC;
}
reef_status reef_module_close(reef_module_t mod) {
    if (!mod) return REEF_SUCC;
    for (auto* k : mod->kernels) delete k;
    delete mod;
    return REEF_SUCC;
}
reef_status reef_module_get_kernel(reef_module_t mod, const char* name, reef_kernel_t* k) {
    if (!mod || !name) return REEF_FAIL;
    reef_kernel_s* h = new (std::nothrow) reef_kernel_s;
    if (!h) return REEF_FAIL;
    int rc = plan_kernel(name, &h->spec);
    if (rc != REEF_SUCC) {
        delete h;
        return rc;
    }
    mod->kernels.push_back(h);
    *k = h;
    return REEF_SUCC;
}
reef_status reef_kernel_plan(const char* name, uint32_t dims[6], uint32_t* dyn_smem, int* num_args) {
    KernelSpec s;
    int rc = plan_kernel(name, &s);
    if (rc != REEF_SUCC) return rc;
    for (int i = 0; i < 3; i++) {
        dims[i] = s.grid[i];
        dims[3 + i] = s.block[i];
    }
    if (dyn_smem) *dyn_smem = s.dyn_smem;
    if (num_args) *num_args = s.nargs;
    return REEF_SUCC;
}
reef_status reef_kernel_cost(const char* name, double* flops, double* bytes, int* tensor_core) {
    KernelSpec s;
    int rc = plan_kernel(name, &s);
    if (rc != REEF_SUCC) return (reef_status)rc;
    if (flops) *flops = s.flops;
    if (bytes) *bytes = s.bytes;
    if (tensor_core) *tensor_core = s.tensor_core;
    return REEF_SUCC;
}
reef_status reef_kernel_prepare(reef_kernel_t k, void** args) {
    if (!k || !args) return REEF_FAIL;
    return prepare_kernel(k->spec, args);
}
reef_status reef_kernel_arg_bytes(reef_kernel_t k, size_t* bytes, int n) {
    if (!k || !bytes || n < k->spec.nargs) return REEF_OUT_OF_RANGE;
    for (int i = 0; i < k->spec.nargs; i++) bytes[i] = k->spec.arg_bytes[i];
    return REEF_SUCC;
}
reef_status reef_kernel_attrs(reef_kernel_t k, reef_kernel_attrs_t* out) {
    if (!k || !out) return REEF_FAIL;
    return kernel_attrs(k->spec, out);
}

reef_status reef_launch(reef_kernel_t k, const uint32_t dims[6], uint32_t dyn_smem, reef_stream_t s, void** args) {
    if (!k) return REEF_FAIL;
    return launch_plain(k->spec, dims, dyn_smem, (cudaStream_t)s, args);
}
reef_status reef_launch_be(reef_kernel_t k, const uint32_t dims[6], uint32_t dyn_smem, reef_stream_t s,
                           reef_dptr_t flag, reef_dptr_t slot, void** args) {
    if (!k || !flag || !slot) return REEF_FAIL;
    return launch_be(k->spec, dims, dyn_smem, (cudaStream_t)s, (const int*)flag, (int*)slot, args);
}
reef_status reef_dispatch(reef_kernel_t rt, void** rt_args, reef_kernel_t be, void** be_args, int be_off,
                          int be_num, int sm_partition, int occupancy, reef_dptr_t be_slot, reef_dptr_t rt_ctrl,
                          reef_dptr_t be_ctrl, reef_stream_t s, reef_stream_t be_stream) {
    if ((!rt && !be) || !rt_ctrl) return REEF_FAIL;
    int sms = 0;
    int rc = reef_device_num_sms(&sms);
    if (rc != REEF_SUCC) return rc;
    return launch_dispatch(rt ? &rt->spec : nullptr, rt_args, be ? &be->spec : nullptr, be_args, be_off, be_num,
                           sm_partition, occupancy, sms, (int*)be_slot, (int*)rt_ctrl, (int*)be_ctrl, (cudaStream_t)s,
                           (cudaStream_t)be_stream);
}

reef_status reef_dispatch_static(reef_kernel_t rt, void** rt_args, reef_kernel_t be, void** be_args, int be_off,
                                 int be_num, int sm_partition, int occupancy, reef_dptr_t be_slot, int lane,
                                 reef_stream_t s) {
    int sms = 0;
    int rc = reef_device_num_sms(&sms);
    if (rc != REEF_SUCC) return rc;
    return launch_dispatch_static(rt ? &rt->spec : nullptr, rt_args, be ? &be->spec : nullptr, be_args, be_off, be_num,
                                  sm_partition, occupancy, sms, (int*)be_slot, lane, (cudaStream_t)s);
}

struct reef_chain_s {
    TcChain* chain;
};
reef_status reef_chain_create(reef_kernel_t* kernels, void*** args, int n, int clusters, reef_chain_t* chain) {
    if (!kernels || !args || n < 1 || !chain) return REEF_FAIL;
    std::vector<const KernelSpec*> specs;
    for (int i = 0; i < n; i++) {
        if (!kernels[i]) return REEF_FAIL;
        specs.push_back(&kernels[i]->spec);
    }
    TcChain* c = nullptr;
    int rc = make_chain(specs.data(), args, n, clusters, &c);
    if (rc != REEF_SUCC) return rc;
    *chain = new (std::nothrow) reef_chain_s{c};
    if (!*chain) {
        chain_destroy(c);
        return REEF_FAIL;
    }
    return REEF_SUCC;
}
reef_status reef_chain_launch(reef_chain_t chain, reef_stream_t s) {
    if (!chain) return REEF_FAIL;
    int rc = chain_launch(chain->chain, (cudaStream_t)s);
    if (rc == REEF_SUCC) add_launches(1);
    return rc;
}
reef_status reef_chain_launch_be(reef_chain_t chain, reef_stream_t s, int first_layer, reef_dptr_t preempt_flag, int clusters) {
    if (!chain || !preempt_flag) return REEF_FAIL;
    int rc = chain_launch(chain->chain, (cudaStream_t)s, first_layer, (const int*)preempt_flag, clusters);
    if (rc == REEF_SUCC) add_launches(1);
    return rc;
}
reef_status reef_chain_copy_progress(reef_chain_t chain, reef_stream_t s) {
    if (!chain) return REEF_FAIL;
    return chain_copy_progress(chain->chain, (cudaStream_t)s);
}
reef_status reef_chain_first_incomplete(reef_chain_t chain, int* layer) {
    if (!chain || !layer) return REEF_FAIL;
    *layer = chain_first_incomplete(chain->chain);
    return REEF_SUCC;
}
reef_status reef_chain_destroy(reef_chain_t chain) {
    if (chain) {
        chain_destroy(chain->chain);
        delete chain;
    }
    return REEF_SUCC;
}
reef_status reef_chain_info(reef_chain_t chain, int* layers, int* clusters, int* max_clusters) {
    if (!chain) return REEF_FAIL;
    if (layers) *layers = chain_num_layers(chain->chain);
    if (clusters) *clusters = chain_clusters(chain->chain);
    if (max_clusters) *max_clusters = chain_max_clusters(chain->chain);
    return REEF_SUCC;
}

reef_status reef_preempt_wait(reef_stream_t s, uint64_t timeout_us) {
    auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        int busy = 0;
        int rc = reef_stream_query(s, &busy);
        if (rc != REEF_SUCC) return rc;
        if (!busy) return REEF_SUCC;
        auto us = std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
        if ((uint64_t)us > timeout_us) return REEF_TIMEOUT;
    }
}

uint64_t reef_launch_count(void) { return launch_count(); }

reef_status reef_preempt_stamps_arm(int on) { return preempt_stamps_arm(on); }
reef_status reef_preempt_stamps_read(uint64_t* first_seen_ns, uint64_t* last_leave_ns) {
    unsigned long long v[2] = {0, 0};
    int rc = preempt_stamps_read(v);
    if (rc != REEF_SUCC) return rc;
    if (first_seen_ns) *first_seen_ns = v[0] == ~0ull ? 0 : v[0];
    if (last_leave_ns) *last_leave_ns = v[1];
    return REEF_SUCC;
}

// A preempt flag in pinned host memory that the device reads through a mapped pointer: the host raises it with a
// plain store (no stream operation, no driver call), the price being that every poll of a best-effort block is a
// read across PCIe instead of an L2 hit.
reef_status reef_flag_alloc_mapped(uint32_t** host_ptr, reef_dptr_t* dev_ptr) {
    void* h = nullptr;
    void* d = nullptr;
    CK(cudaHostAlloc(&h, 64, cudaHostAllocMapped));
    CK(cudaHostGetDevicePointer(&d, h, 0));
    *(volatile uint32_t*)h = 0;
    *host_ptr = (uint32_t*)h;
    *dev_ptr = (reef_dptr_t)d;
    return REEF_SUCC;
}
reef_status reef_flag_free_mapped(uint32_t* host_ptr) {
    CK(cudaFreeHost(host_ptr));
    return REEF_SUCC;
}
reef_status reef_flag_set(uint32_t* host_ptr, uint32_t value) {
    if (!host_ptr) return REEF_FAIL;
    __atomic_store_n(host_ptr, value, __ATOMIC_RELEASE);
    return REEF_SUCC;
}

reef_status reef_device_error(int* value) {
    volatile int* w = nullptr;
    int rc = tc_error_word_host(&w);
    if (rc != REEF_SUCC) return rc;
    *value = *w;
    if (*value != 0) *w = 0;
    return REEF_SUCC;
}
reef_status reef_device_error_peek(int* value) {
    volatile int* w = nullptr;
    int rc = tc_error_word_host(&w);
    if (rc != REEF_SUCC) return rc;
    *value = *w;
    return REEF_SUCC;
}
reef_status reef_device_error_set(int value) {
    volatile int* w = nullptr;
    int rc = tc_error_word_host(&w);
    if (rc != REEF_SUCC) return rc;
    *w = value;
    return REEF_SUCC;
}

#ifdef REEF_DEBUG_AIDS
reef_status reef_trace_enable(int on) { return tc_trace_enable(on); }
reef_status reef_trace_read(int64_t* stamps16) { return tc_trace_read((long long*)stamps16); }
#endif

reef_status reef_stream_delay(reef_stream_t s, uint64_t ns) { return launch_delay((cudaStream_t)s, ns); }

}  // extern "C"
