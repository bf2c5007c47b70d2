// Host side of the persistent chain kernel: the layer table in device memory, completion counters, cluster launch.
#include "conv_tc_chain.cuh"

#include <cstring>
#include <string>
#include <vector>

#include "registry.h"

namespace reef {

struct TcChain {
    TcParams* layers = nullptr;   // device
    int* need = nullptr;          // device
    int* done = nullptr;          // device, n + 3 words: counters, "gave up", ticket
    int* init0 = nullptr;         // pinned host image of `done` for a launch from layer 0 (constant: usable in a graph)
    int* progress = nullptr;      // pinned host copy of `done` (reef_chain_copy_progress)
    std::vector<int> need_h;      // host copies of need[] and of the group prefix
    std::vector<int> goff_h;
    int n = 0;
    int ctrl_offset = 0;
    int smem = 0;
    int clusters = 0;             // clusters of the grid
    int max_clusters = 0;
};

static bool g_chain_attr_set[16] = {false};

static int chain_prepare_device(int smem, int* max_clusters) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16 && !g_chain_attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute((const void*)reef_conv_tc_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute((const void*)reef_conv_tc_chain_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) {
            set_error(std::string("cudaFuncSetAttribute(conv_tc_chain): ") + cudaGetErrorString(e));
            return REEF_FAIL;
        }
        g_chain_attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(TC_CHAIN_CLUSTER, 64, 1);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = TC_CHAIN_CLUSTER;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&n, (const void*)reef_conv_tc_chain_kernel, &cfg);
    if (e != cudaSuccess) {
        set_error(std::string("cudaOccupancyMaxActiveClusters(conv_tc_chain): ") + cudaGetErrorString(e));
        return REEF_FAIL;
    }
    *max_clusters = n;
    return REEF_SUCC;
}

int chain_create(const std::vector<const TcParams*>& params, const std::vector<TcPlan>& plans, int clusters, TcChain** out) {
    const int n = (int)params.size();
    if (n < 1) return REEF_OUT_OF_RANGE;
    TcChain* c = new TcChain;
    c->n = n;
    std::vector<TcParams> host(n);
    std::vector<int> need(2 * n + 2, 0);
    int region = 0;
    for (int i = 0; i < n; i++) {
        host[i] = *params[i];
        host[i].preempt_flag = nullptr;
        host[i].task_slot = nullptr;
        host[i].trace = nullptr;
        host[i].stamps = nullptr;
        host[i].tile_begin = 0;
        if (plans[i].splits != 1 && plans[i].splits != 2 && plans[i].splits != 4 && plans[i].splits != 8) {
            set_error("chain: K splits of a layer must divide the cluster of 8");
            delete c;
            return REEF_FAIL;
        }
        region = plans[i].region_bytes > region ? plans[i].region_bytes : region;
        need[i + 1] = plans[i].splits * plans[i].n_tiles * plans[i].m_tiles;   // CTAs that finish layer i
        const int per = TC_CHAIN_CLUSTER / plans[i].splits;
        const int groups = (plans[i].n_tiles * plans[i].m_tiles + per - 1) / per;
        need[n + 1 + i + 1] = need[n + 1 + i] + groups;                        // tile groups before layer i + 1
    }
    need[0] = 0;
    c->ctrl_offset = region;
    // alignment slack, data region, control words, the scalar part of the layer's parameters
    c->smem = 1024 + region + 256 + (int)(sizeof(TcParams) - 5 * sizeof(CUtensorMap));
    int rc = chain_prepare_device(c->smem, &c->max_clusters);
    if (rc != REEF_SUCC) {
        delete c;
        return rc;
    }
    // every CTA of the grid must be resident at once: CTAs wait for one another through the counters
    if (c->max_clusters < 1) {
        set_error("chain: no cluster of 8 CTAs fits the device");
        delete c;
        return REEF_FAIL;
    }
    // Tile groups are taken by ticket, in order, so any number of clusters is safe: those the hardware has not made
    // resident simply take no tickets.  The default asks for two CTAs per SM.
    c->clusters = clusters > 0 ? clusters : 32;
    c->need_h.assign(need.begin(), need.begin() + n + 1);
    c->goff_h.assign(need.begin() + n + 1, need.end());
    if (cudaMalloc(&c->layers, sizeof(TcParams) * n) != cudaSuccess || cudaMalloc(&c->need, 4 * (2 * n + 2)) != cudaSuccess ||
        cudaMalloc(&c->done, 4 * (n + 3)) != cudaSuccess ||
        cudaHostAlloc((void**)&c->init0, 4 * (n + 3), cudaHostAllocDefault) != cudaSuccess ||
        cudaHostAlloc((void**)&c->progress, 4 * (n + 3), cudaHostAllocDefault) != cudaSuccess ||
        cudaMemcpy(c->layers, host.data(), sizeof(TcParams) * n, cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemcpy(c->need, need.data(), 4 * (2 * n + 2), cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemset(c->done, 0, 4 * (n + 3)) != cudaSuccess || cudaStreamSynchronize(cudaStreamLegacy) != cudaSuccess) {
        set_error("chain: cannot allocate or fill the layer table");
        chain_destroy(c);
        return REEF_FAIL;
    }
    memset(c->init0, 0, 4 * (n + 3));
    memset(c->progress, 0, 4 * (n + 3));
    *out = c;
    return REEF_SUCC;
}

void chain_destroy(TcChain* c) {
    if (!c) return;
    if (c->init0) cudaFreeHost(c->init0);
    if (c->progress) cudaFreeHost(c->progress);
    if (c->layers) cudaFree(c->layers);
    if (c->need) cudaFree(c->need);
    if (c->done) cudaFree(c->done);
    delete c;
}

int chain_num_layers(const TcChain* c) { return c->n; }
int chain_clusters(const TcChain* c) { return c->clusters; }
int chain_max_clusters(const TcChain* c) { return c->max_clusters; }

int chain_launch(TcChain* c, cudaStream_t st, int first_layer, const int* flag, int clusters) {
    if (first_layer < 0 || first_layer >= c->n) {
        set_error("chain: first layer outside the chain");
        return REEF_OUT_OF_RANGE;
    }
    ChainParams P;
    P.preempt_flag = flag;
    P.first_group = c->goff_h[first_layer];
    P.total_groups = c->goff_h[c->n];
    P.layers = c->layers;
    P.need = c->need;
    P.done = c->done;
    P.n_layers = c->n;
    P.ctrl_offset = c->ctrl_offset;
    int rc = tc_error_word(&P.error_word);
    if (rc != REEF_SUCC) return rc;
    // counters: the layers before first_layer count as complete, the ticket counter starts at its first group
    cudaError_t e;
    if (first_layer == 0) {
        e = cudaMemcpyAsync(c->done, c->init0, 4 * (c->n + 3), cudaMemcpyHostToDevice, st);   // constant pinned image
    } else {
        std::vector<int> img(c->n + 3, 0);
        for (int l = 0; l <= first_layer; l++) img[l] = c->need_h[l];
        img[c->n + 2] = c->goff_h[first_layer];
        // pageable source: the bytes are staged before the call returns (a restart is never part of a stream capture)
        e = cudaMemcpyAsync(c->done, img.data(), 4 * (c->n + 3), cudaMemcpyHostToDevice, st);
    }
    if (e != cudaSuccess) {
        set_error(std::string("chain: cannot set the completion counters: ") + cudaGetErrorString(e));
        return REEF_FAIL;
    }
    const int nc = clusters > 0 ? clusters : c->clusters;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(TC_CHAIN_CLUSTER, nc, 1);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = c->smem;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = TC_CHAIN_CLUSTER;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, reef_conv_tc_chain_kernel, P);
    if (e != cudaSuccess) {
        set_error(std::string("cudaLaunchKernelEx(conv_tc_chain): ") + cudaGetErrorString(e));
        return REEF_FAIL;
    }
    return REEF_SUCC;
}

// progress of a (possibly preempted) launch: stream-ordered copy of the counters to pinned memory, then, once the
// caller has synchronised, the first layer whose counter is short (n = every layer complete)
int chain_copy_progress(TcChain* c, cudaStream_t st) {
    if (cudaMemcpyAsync(c->progress, c->done, 4 * (c->n + 3), cudaMemcpyDeviceToHost, st) != cudaSuccess) {
        set_error("chain: cannot copy the completion counters");
        return REEF_FAIL;
    }
    return REEF_SUCC;
}
int chain_first_incomplete(const TcChain* c) {
    for (int l = 0; l < c->n; l++)
        if (c->progress[l + 1] < c->need_h[l + 1]) return l;
    return c->n;
}

}  // namespace reef
