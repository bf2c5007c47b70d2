/*
 * Stand-in for <hip/hip_runtime.h> so that the reference's generated kernel sources (resource/<model>/<model>.cu of
 * SJTU-IPADS/reef, written by TVM for AMD gfx906) compile with g++ as plain C++ and run on the CPU, one fiber per GPU
 * thread (emu.cpp).  TEST INFRASTRUCTURE ONLY: it builds oracle/_ref, the checker of the checker — the reference's
 * own kernel arithmetic against which the C oracle is pinned.  Nothing here is part of the product.
 *
 * What the sources use and what it becomes here:
 *   __global__ / __restrict__          nothing / g++'s own keyword
 *   __shared__                         static storage (blocks run one after the other, fibers share the process)
 *   threadIdx, blockIdx                globals the fiber scheduler sets before it resumes a fiber
 *   __syncthreads()                    yield to the scheduler; every fiber of the block runs up to the same barrier
 *   __ocml_fma_f32 / exp / sqrt / erf  fmaf / expf / sqrtf / erff (fmaf is a true fused multiply-add, as on the GPU)
 *   (volatile float*) shared memory    lock-step stores (struct reef_emu_vf below)
 *   __mbcnt_lo / __mbcnt_hi            lane index inside a 64-wide wavefront, in the two halves the hardware counts
 *   __hip_ds_bpermute                  a 64-lane permute through a per-call-site log of what every lane passed
 */
#ifndef REEF_ORACLE_HIP_SHIM_H_
#define REEF_ORACLE_HIP_SHIM_H_
#include <math.h>
#include <stdint.h>

struct reef_emu_dim3 {
    unsigned x, y, z;
};
extern reef_emu_dim3 threadIdx, blockIdx, blockDim, gridDim;

#define __global__
#define __shared__ static
#define __launch_bounds__(...)

extern "C" void reef_emu_barrier(void);
extern "C" int reef_emu_lane(void);
extern "C" float reef_emu_bpermute_site(int site, int byte_addr, float v);

extern "C" void reef_emu_yield(void);
static inline void __syncthreads(void) { reef_emu_barrier(); }
/* The generated tree reductions of bert.cu are "warp-synchronous": the lanes of a wavefront add through VOLATILE
 * shared memory with no barrier between the steps and rely on running in lock step (bert.cu:185-191).  The build
 * recipe reads `(volatile float*)` as `(reef_emu_vf*)` (a stream edit on the way into the compiler, the source file
 * is not touched): a store through this type yields before and after it takes effect, so every lane has read the
 * operands of a step before any lane stores, and every lane has stored before any lane reads the next step. */
struct reef_emu_vf {
    float v;
    reef_emu_vf& operator=(float x) {
        reef_emu_yield();
        v = x;
        reef_emu_yield();
        return *this;
    }
    operator float() const { return v; }
};
static inline float __ocml_fma_f32(float a, float b, float c) { return fmaf(a, b, c); }
static inline float __ocml_exp_f32(float a) { return expf(a); }
static inline float __ocml_sqrt_f32(float a) { return sqrtf(a); }
static inline float __ocml_erf_f32(float a) { return erff(a); }
static inline float __int_as_float(int v) {
    union { int i; float f; } u;
    u.i = v;
    return u.f;
}
static inline float max(float a, float b) { return a > b ? a : b; }
static inline float min(float a, float b) { return a < b ? a : b; }
static inline int max(int a, int b) { return a > b ? a : b; }
static inline int min(int a, int b) { return a < b ? a : b; }
static inline long max(long a, long b) { return a > b ? a : b; }
static inline long min(long a, long b) { return a < b ? a : b; }
/* v_mbcnt_lo/hi_u32_b32 with an all-ones mask: lanes below this one in the low / high 32 lanes of the wavefront */
static inline int __mbcnt_lo(int, int base) {
    int l = reef_emu_lane();
    return base + (l < 32 ? l : 32);
}
static inline int __mbcnt_hi(int, int base) {
    int l = reef_emu_lane();
    return base + (l > 32 ? l - 32 : 0);
}
/* one id per call site in the source (see reef_emu_bpermute_site) */
#define __hip_ds_bpermute(byte_addr, v) reef_emu_bpermute_site(__COUNTER__, (byte_addr), (v))
#define __hip_ds_bpermutef(byte_addr, v) reef_emu_bpermute_site(__COUNTER__, (byte_addr), (v))
#endif
