// Host-side view of the kernel registry (internal to libreef_cuda).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <memory>
#include <string>
#include <vector>

#include "../../../include/reef_cuda.h"
#include "task.cuh"

namespace reef {

struct TcParams;

// tile / split-K plan of the tcgen05 convolution (conv_tc.cu)
struct TcPlan {
    int spatial, rows, n_valid, n_mma, tmem_cols;
    int n_tiles, m_tiles, cblocks, kb_total, kb_per_split, splits;
    int b_bytes, smem;
    int region_bytes, recv_offset_floats, cpc_max, stages;
    int xsplit, xw;
};

struct TcCache;   // tensor maps of one kernel call, rebuilt when its pointers change
struct AttParams;

struct KernelSpec {
    std::string name;
    KTask task;            // family + shape parameters; pointer slots are filled per launch
    uint32_t grid[3];
    uint32_t block[3];
    uint32_t dyn_smem;
    int nargs;
    double flops, bytes;   // algorithmic work of one launch
    size_t arg_bytes[kMaxArgs];   // least size of the buffer behind each positional argument
    int tensor_core;
    TcPlan tc;
    mutable std::shared_ptr<TcCache> tc_cache;
};

void set_error(const std::string& s);
const char* last_error();

int plan_kernel(const char* name, KernelSpec* out);
int launch_plain(const KernelSpec& s, const uint32_t dims[6], uint32_t smem, cudaStream_t st, void** args);
int launch_be(const KernelSpec& s, const uint32_t dims[6], uint32_t smem, cudaStream_t st, const int* flag,
              int* slot, void** args);
int launch_dispatch(const KernelSpec* rt, void** rt_args, const KernelSpec* be, void** be_args, int be_off,
                    int be_num, int sm_partition, int occupancy, int num_sms, int* be_slot, int* ctrl, int* be_ctrl,
                    cudaStream_t st, cudaStream_t be_st);
int launch_dispatch_static(const KernelSpec* rt, void** rt_args, const KernelSpec* be, void** be_args, int be_off,
                           int be_num, int sm_partition, int occupancy, int num_sms, int* be_slot, int lane,
                           cudaStream_t st);
int kernel_attrs(const KernelSpec& s, reef_kernel_attrs_t* out);
int prepare_kernel(const KernelSpec& s, void** args);
int dispatch_occupancy(uint32_t smem, int* occ);
int launch_delay(cudaStream_t st, unsigned long long ns);

// attention_tc.cu
int att_smem_bytes();
int att_supported(int s, int heads, int d);
int att_build_params(int s, int heads, int has_mask, void* const* args, AttParams* P);
int att_prepare_device();
int att_launch(const AttParams& P, cudaStream_t st, const int* flag, int* slot, int head_begin = 0, int head_count = -1);
int att_func_attrs(cudaFuncAttributes* fa, int* occ);

// conv_tc_chain.cu: a run of tensor-core convolution layers as one persistent kernel
struct TcChain;
int chain_create(const std::vector<const TcParams*>& params, const std::vector<TcPlan>& plans, int clusters, TcChain** out);
void chain_destroy(TcChain* c);
int chain_launch(TcChain* c, cudaStream_t st, int first_layer = 0, const int* flag = nullptr, int clusters = 0);
int chain_copy_progress(TcChain* c, cudaStream_t st);
int chain_first_incomplete(const TcChain* c);
int chain_num_layers(const TcChain* c);
int chain_clusters(const TcChain* c);
int chain_max_clusters(const TcChain* c);
// registry.cu: the chain of kernel specs [0, n) bound to their argument lists (all must be tensor-core convolutions)
int make_chain(const KernelSpec* const* specs, void*** args, int n, int clusters, TcChain** out);

// conv_tc.cu
int tc_plan(const ConvP& p, TcPlan* pl);
int tc_build_params(const ConvP& p, const TcPlan& pl, void* const* args, TcParams* P);
int tc_launch(const TcParams& P, const TcPlan& pl, cudaStream_t st, const int* flag, int* slot, int tile_begin = 0,
              int tile_count = -1);
int tc_func_attrs(const TcPlan& pl, cudaFuncAttributes* fa, int* occ);
int tc_error_word(int** out);
int tc_error_word_host(volatile int** out);
int tc_prepare_device();
#ifdef REEF_DEBUG_AIDS
int tc_trace_enable(int on);
int tc_trace_read(long long* out16);
#endif
unsigned long long* preempt_stamps_ptr();   // device words {first seen, last leave} of the current device, or null
int preempt_stamps_arm(int on);
int preempt_stamps_read(unsigned long long out[2]);
unsigned long long launch_count();          // kernels launched by this library, all threads
unsigned long long thread_launch_count();   // ... by the calling thread (a stream capture counts its own launches)
void add_launches(unsigned long long n);

}  // namespace reef
