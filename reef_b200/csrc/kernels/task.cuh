// Shared device-side vocabulary of the kernel registry.
//
// Every kernel family is written once as a __device__ body that executes ONE logical thread
// block ("vblock") of 256 threads.  Three __global__ flavours wrap the same body, mirroring the
// three code objects the reference builds per model (reference: resource/Makefile:22-66):
//   plain      one CUDA block per vblock                       (<m>.raw.co)
//   best-effort  plain + preempt-flag poll + completion counter (<m>.be.co,
//              reference: script/best_effort_kernel.py:22-33)
//   dispatcher a persistent grid that pulls vblocks of a real-time and a best-effort
//              kernel (<m>.trans.co, reference: resource/mocked_kernel/mocked_kernel.trans.cu:112-186)
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace reef {

constexpr int kThreads = 256;   // every family runs 256-thread blocks so the dispatcher can host any of them
constexpr int kMaxArgs = 8;

enum Family : int {
    F_MOCK_ADD = 0,
    F_MOCK_MUL,
    F_FUSED_ADD_NCHW,
    F_BIAS_RELU,
    F_CONV_SIMT,
    F_MAX_POOL,
    F_AVG_POOL,
    F_GLOBAL_AVG_POOL,
    F_COPY,
    F_DENSE,
    F_SOFTMAX,
    F_EMBEDDING,
    F_LAYERNORM,
    F_ATTENTION,
    F_NCHW_TO_NHWC4,
    F_IM2COL_NCHW,
    F_COUNT,
    // families with their own __global__ kernel (not hosted by the 256-thread logical-block wrappers)
    F_CONV_TC = 100,
    F_ATTENTION_TC = 101
};

// epilogue / option bits
enum : int { EP_RES = 1, EP_BIAS = 2, EP_GB = 4, EP_RELU = 8, EP_GELU = 16, EP_DUAL = 32 };

struct ConvP {
    int ci, hi, wi, co, kh, kw, sh, sw, ph, pw, ho, wo;
    int ics, ioff, ocs, ooff, nchw;
    int ktot, ptot;          // K = kh*kw*ci, P = ho*wo
    int tiles_p, tiles_c;    // tile grid: pixels x out-channels
    int ep;                  // EP_* bits
    int i_res, i_bias, i_gamma, i_beta;   // positions in the arg list, -1 when absent
    int round_tf32;          // tensor-core variant: store activations rounded to the nearest TF32 value
    int i_bias2, i_out2;     // EP_DUAL: second output out2 = relu(out + bias2) (the next unit's pre-activation)
    int plan_cap, plan_splits;   // tensor-core variant: tile cap / K splits fixed by the name (tp, ts), 0 = planner's choice
};

struct PoolP {
    int c, hi, wi, k, s, p, ho, wo, ics, ioff, ocs, ooff, cip, has_bias;
};

struct EltP {
    int c, n, ics, ioff;     // channels, rows (pixels) ; NCHW fused_add: c planes of n elements
};

struct DenseP {
    int k, n, relu;
};

struct SoftmaxP {
    int rows, n;
};

struct KTask {
    int family;
    int nblocks;             // logical blocks of one launch
    union {
        ConvP conv;
        PoolP pool;
        EltP elt;
        DenseP dense;
        SoftmaxP softmax;
        int raw[32];
    } p;
    void* a[kMaxArgs];       // device pointers, positional like the json "args"
    int* err;                // device error word (set when a bounded wait expired), may be null
};

__device__ __forceinline__ int ld_flag(const int* flag) {
    return *reinterpret_cast<const volatile int*>(flag);
}

}  // namespace reef
