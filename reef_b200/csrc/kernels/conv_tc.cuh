// conv2d / matmul on the 5th-generation tensor cores (tcgen05, TF32 inputs, fp32 accumulate in TMEM).
//
// GEMM view (implicit, no im2col buffer):  D[co][pixel] = sum_k W[co][k] * X[pixel][k]
//   A = weights  OHWI = [Cout][kh*kw*Cin]  : K-major, M = Cout  -> TMEM lanes (128 per tile)
//   B = activations NHWC                    : K-major per filter tap, N = pixels -> TMEM columns
// Both operands are staged by TMA (cp.async.bulk.tensor, 128-byte swizzle) into a 4-stage shared-memory
// ring; a K block is 32 channels of one filter tap = one 128-byte row per pixel / per output channel.
// Zero padding, ragged tiles and strides are folded into the tensor maps (out-of-bounds boxes read
// zeros; a stride-s conv uses up to s*s maps over the s-strided sub-lattices of the input).
//
// Batch-1 convolutions are tiny GEMMs (N = 49..3136 pixels), far too few tiles for 148 SMs and too
// many weight bytes per tile for one SM's load bandwidth, so K is split across a thread-block
// CLUSTER (1..8 CTAs).  Each CTA accumulates its K range in TMEM, parks the partial tile in its own
// shared memory, and after a cluster barrier every CTA sums a slice of the tile over all ranks through
// distributed shared memory in rank order 0..S-1 — a fixed order, so results are bit-reproducible (no
// float atomics, no global scratch, no counters to reset when a best-effort run is preempted and re-run).
//
// One thread issues TMA, one thread issues tcgen05.mma, all eight warps run the epilogue
// (tcgen05.ld -> +residual -> +bias | *gamma+beta -> ReLU -> coalesced 128-byte stores, one output
// channel per lane).  Every mbarrier wait is bounded: on expiry the kernel records an error word,
// skips further waits, still joins every cluster barrier, frees its TMEM and returns.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "conv_tc_params.h"

namespace reef {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: returns false when the phase did not complete within the iteration limit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    unsigned long long t0 = 0;
    for (int i = 0; i < (1 << 26); i++) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
        if ((i & 255) == 255) {   // give up after one second of wall time
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (t0 == 0) t0 = t;
            else if (t - t0 > 1000000000ull) return false;
        }
    }
    return false;
}
// The same wait for the best-effort flavour's MMA thread: it also gives up when `abort_word` (shared memory, written
// by the TMA producer of the same CTA when it saw the preempt flag) becomes non-zero.  0 = phase complete,
// 1 = wait expired, 2 = abort requested.
__device__ __forceinline__ int mbar_wait_abortable(uint32_t bar, uint32_t parity, const volatile uint32_t* abort_word) {
    unsigned long long t0 = 0;
    for (int i = 0; i < (1 << 26); i++) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return 0;
        if (*abort_word) return 2;
        if ((i & 255) == 255) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (t0 == 0) t0 = t;
            else if (t - t0 > 1000000000ull) return 1;
        }
    }
    return 1;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(tm), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(tm), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// split form: arrive early, wait where the guarantee is needed, so the barrier latency hides behind other work
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
// control-only arrive: what the barrier orders was already observed complete through an mbarrier
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// volatile keeps the load behind the cluster barrier (also a volatile asm); no "memory" clobber, so the
// loads of one reduction batch are issued back to back and overlap
__device__ __forceinline__ float ld_dsmem_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float4 ld_dsmem_v4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void st_dsmem_u32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);         // start address >> 4, bits [0,14)
    d |= (uint64_t)1 << 16;                          // leading byte offset (unused with swizzle), bits [16,30)
    d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset between 8-row groups, bits [32,46)
    d |= (uint64_t)1 << 46;                          // descriptor version for sm_100
    d |= (uint64_t)2 << 61;                          // SWIZZLE_128B
    return d;
}
// Instruction descriptor: D fp32, A/B tf32, both K-major, M=128, N=n.
__device__ __forceinline__ uint32_t umma_idesc_tf32(int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 32 columns of one TMEM lane per thread; the wait is separate so that several loads can be in flight
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

enum : int { TC_EP_RES = 1, TC_EP_BIAS = 2, TC_EP_GB = 4, TC_EP_RELU = 8, TC_EP_ROUND = 16, TC_EP_GELU = 32 };

// Branch-free form of (+residual) (+bias | *gamma+beta) (ReLU): r = 0, sc = 1, sh = 0, lo = -inf stand in for
// the absent terms (v + 0 and fma(v, 1, b) are exact, so this equals the conditional form bit for bit).
// exact-erf GELU (reference: resource/bert/bert.cu:167-173).  Not inlined on purpose: inlined, the compiler turned
// the uniform `if (gelu)` of the epilogue into straight-line code and every layer paid for erff on each element
// (0.5 us per launch on the row-finishing loop).
__device__ __noinline__ float tc_gelu(float v) { return v * (0.5f * erff(v * 0.70710678118654752440f) + 0.5f); }

__device__ __forceinline__ float tc_epilogue(float v, float r, float sc, float sh, float lo, bool rnd, bool gelu = false) {
    if (gelu) {
        // matmul + bias -> GELU -> (+residual)
        v = tc_gelu(v + sh) + r;
    } else {
        v = fmaxf(fmaf(v + r, sc, sh), lo);
    }
    if (rnd) {
        // The tensor core reads only the upper 19 bits of an fp32 operand (truncation, a bias toward zero).
        // Rounding the stored activation to the nearest TF32 value makes the consumer's truncation exact.
        uint32_t u;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v));
        v = __uint_as_float(u);
    }
    return v;
}

// the same on the 4 channels of a lane at once: one uniform branch per pixel row instead of one per element
__device__ __forceinline__ float4 tc_epilogue4(float4 v, float4 r, float4 sc, float4 sh, float lo, bool rnd, bool gelu) {
    float4 o;
    if (gelu) {
        o.x = tc_gelu(v.x + sh.x) + r.x; o.y = tc_gelu(v.y + sh.y) + r.y;
        o.z = tc_gelu(v.z + sh.z) + r.z; o.w = tc_gelu(v.w + sh.w) + r.w;
    } else {
        o.x = fmaxf(fmaf(v.x + r.x, sc.x, sh.x), lo); o.y = fmaxf(fmaf(v.y + r.y, sc.y, sh.y), lo);
        o.z = fmaxf(fmaf(v.z + r.z, sc.z, sh.z), lo); o.w = fmaxf(fmaf(v.w + r.w, sc.w, sh.w), lo);
    }
    if (rnd) {
        uint32_t u;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(o.x)); o.x = __uint_as_float(u);
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(o.y)); o.y = __uint_as_float(u);
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(o.z)); o.z = __uint_as_float(u);
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(o.w)); o.w = __uint_as_float(u);
    }
    return o;
}

// second output of the dual epilogue: relu(o + b2), rounded like the first when the layer rounds
__device__ __forceinline__ float4 tc_preact(float4 o, float4 b2, bool rnd) {
    float4 r;
    r.x = fmaxf(o.x + b2.x, 0.f); r.y = fmaxf(o.y + b2.y, 0.f); r.z = fmaxf(o.z + b2.z, 0.f); r.w = fmaxf(o.w + b2.w, 0.f);
    if (rnd) {
        uint32_t u;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(r.x)); r.x = __uint_as_float(u);
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(r.y)); r.y = __uint_as_float(u);
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(r.z)); r.z = __uint_as_float(u);
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(r.w)); r.w = __uint_as_float(u);
    }
    return r;
}

// by the warp that allocated, after a CTA barrier behind every tcgen05 operation that used the columns
__device__ __forceinline__ void tmem_free(uint32_t tmem, uint32_t cols) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(cols) : "memory");
}

// Phase trace: compiled in only with -DREEF_DEBUG_AIDS (a development aid; the default build carries no stamps)
#ifdef REEF_DEBUG_AIDS
__device__ __forceinline__ void tc_stamp(const TcParams& P, int slot) {
    if (P.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0) P.trace[slot] = clock64();
}
#else
__device__ __forceinline__ void tc_stamp(const TcParams&, int) {}
#endif

// Finishes the pixel rows [jb, je) a cluster rank owns after a K split: sums the partials of ranks 0..S-1 in
// rank order (a fixed order: bit-reproducible), applies the epilogue and stores 512-byte rows.  RB rows per warp
// are in flight at a time, RB * SMAX 128-bit loads per lane (16: the kernel is built for two CTAs per SM, so
// a thread has 128 registers).
template <int RB, int SMAX>
__device__ __forceinline__ void tc_finish_split(const TcParams& P, const float* stage, const float* recv, int S, int split,
                                                int jb, int je, int warp, int cbase, int co, int pix0, float4 sc, float4 sh,
                                                float lo, bool rnd, bool gelu, bool has_res, float4 b2, const float4* rpre) {
    const float* src[SMAX];
#pragma unroll
    for (int q = 0; q < SMAX; q++)
        src[q] = (q == split) ? stage + (size_t)jb * TC_BM + cbase
                              : recv + (size_t)(q < S ? (q < split ? q : q - 1) : 0) * P.cpc_max * TC_BM + cbase;
    for (int jbase = warp; jbase < je - jb; jbase += 8 * RB) {
        float4 part[RB][SMAX], rv[RB];
#pragma unroll
        for (int u = 0; u < RB; u++) {
            const int jr = jbase + 8 * u;   // row within this rank's slice
            rv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (jr < je - jb) {
#pragma unroll
                for (int q = 0; q < SMAX; q++)
                    if (q < S) part[u][q] = *reinterpret_cast<const float4*>(src[q] + (size_t)jr * TC_BM);
                if (has_res) rv[u] = (u < 2 && jbase == warp) ? rpre[u & 1] : __ldg(reinterpret_cast<const float4*>(P.res + (size_t)(pix0 + jb + jr) * P.co + co));
            }
        }
#pragma unroll
        for (int u = 0; u < RB; u++) {
            const int jr = jbase + 8 * u;
            if (jr < je - jb) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int q = 0; q < SMAX; q++)   // fixed rank order: deterministic sum
                    if (q < S) { v.x += part[u][q].x; v.y += part[u][q].y; v.z += part[u][q].z; v.w += part[u][q].w; }
                const float4 o = tc_epilogue4(v, rv[u], sc, sh, lo, rnd, gelu);
                *reinterpret_cast<float4*>(P.out + (size_t)(pix0 + jb + jr) * P.ocs + P.ooff + co) = o;
                if (P.out2 != nullptr) *reinterpret_cast<float4*>(P.out2 + (size_t)(pix0 + jb + jr) * P.co + co) = tc_preact(o, b2, rnd);
            }
        }
    }
}

// BE = best-effort flavour (reference wrapper contract: script/best_effort_kernel.py:22-33, with the polls the
// reference gets for free from killing wavefronts): the preempt flag is read at block entry and, by the TMA producer,
// at the head of its refill loop (every 4th K block).  A CTA that saw the flag stops loading, lets the tensor core
// finish what has landed, and takes part in every cluster barrier; at the first barrier the ranks of a cluster
// exchange what they saw, and if any rank stopped, ALL ranks skip the exchange, the stores and the completion counter —
// the kernel is idempotent, so it is simply launched again later.  The real-time flavour carries none of this.
template <bool BE>
__global__ void __launch_bounds__(TC_THREADS, 2) reef_conv_tc_kernel(const __grid_constant__ TcParams P) {
    extern __shared__ __align__(16) unsigned char tc_smem_raw[];
    // stage buffers need 1024-byte alignment (swizzle atom); carve barriers behind them
    const uint32_t raw = smem_u32(tc_smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* smem = tc_smem_raw + (base - raw);
    const uint32_t stage_bytes = TC_A_BYTES + (uint32_t)P.n_mma * 128u;
    // the control words sit behind the data region (stage ring, reused by the epilogue's staging + exchange area)
    const uint32_t ctrl = base + (uint32_t)P.region_bytes;
    const int NS = P.stages;   // ring depth of this launch (<= TC_MAX_STAGES)
    const uint32_t bar_full = ctrl, bar_empty = ctrl + 8 * TC_MAX_STAGES, bar_acc = ctrl + 16 * TC_MAX_STAGES;
    const uint32_t bar_red = bar_acc + 8;
    volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem + P.region_bytes + 16 * TC_MAX_STAGES + 16);
    volatile uint32_t* s_flags = s_tmem + 1;    // [0] abort (preempt flag seen by this CTA), [1] wait expired,
                                                //  [2] K blocks whose loads were issued when the producer stopped

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) tc_stamp(P, 0);
    // grid = (K splits = cluster, tiles of this launch); a launch may cover a sub-range of the tiles
    const int split = blockIdx.x;
    const int tile = P.tile_begin + (int)blockIdx.y;
    const int tile_n = tile % P.n_tiles, tile_m = tile / P.n_tiles;
    const int S = P.splits;
    const int kb_begin = split * P.kb_per_split;
    const int kb_end = min(kb_begin + P.kb_per_split, P.kb_total);
    const int nkb = kb_end - kb_begin;

    if (tid == 0) {
        for (int s = 0; s < NS; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc, 1);
        mbar_init(bar_red, 1);
        s_flags[0] = BE ? (uint32_t)(*reinterpret_cast<const volatile int*>(P.preempt_flag) != 0) : 0u;   // poll at block entry
        s_flags[1] = 0;
        s_flags[2] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&P.tm_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&P.tm_x[0]) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)s_tmem)),
                     "r"((uint32_t)P.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *s_tmem;
    if (tid == 0) tc_stamp(P, 1);   // set-up done (barriers, TMEM)

    // K-split exchange barrier: armed now, so that peers may send as soon as their own tile is staged.  The
    // cluster barrier below (cheap here: all CTAs of a cluster start together, and it overlaps the first loads'
    // latency) guarantees every peer's barrier is initialised and armed before any remote completion.
    // spatial tiles: tile_n -> (row group ty, row piece tx); tx > 0 only where a row is wider than a tile
    const int tile_y = P.xsplit > 1 ? tile_n / P.xsplit : tile_n, tile_x = P.xsplit > 1 ? tile_n - tile_y * P.xsplit : 0;
    const int pix0 = P.spatial ? tile_y * P.rows * P.wo + tile_x * P.xw : tile_n * P.n_valid;
    const int n_lim = min(P.n_valid, P.ptot - pix0);   // columns of this tile that are real pixels
    const int cpc = (n_lim + S - 1) / S;               // pixel rows one rank finishes
    const int jb = min(split * cpc, n_lim), je = min(jb + cpc, n_lim);
    if (S > 1 && tid == 0) mbar_expect_tx(bar_red, (uint32_t)((S - 1) * (je - jb) * TC_BM * 4));
    // best-effort flavour: what this CTA saw at entry.  Nothing is loaded then; the cluster agrees at its first barrier.
    const bool abort0 = BE && s_flags[0] != 0;

    {
        const int m0 = tile_m * TC_BM;
        // ---------------- TMA producer, part 1: fill the ring (no waits) ----------------
        const uint32_t tx = TC_A_BYTES + (uint32_t)P.b_bytes;
        const int first = nkb < NS ? nkb : NS;
        // tap and channel block of a K block (2^32/1 does not fit the magic: one channel block per tap is a copy)
        auto tap_of = [&](int kb) { return P.cblocks == 1 ? kb : (int)__umulhi((unsigned)kb, P.cb_magic); };
        auto load_a = [&](int i, int s) {   // weights: 32 channels of one tap for this tile's 128 output channels
            const int kb = kb_begin + i, tap = tap_of(kb), cb = kb - tap * P.cblocks;
            tma_load_3d(base + s * stage_bytes, &P.tm_w, bar_full + 8 * s, cb * TC_BK, tap, m0);
        };
        auto load_b = [&](int i, int s) {
            const uint32_t st = base + s * stage_bytes;
            const int kb = kb_begin + i;
            // the per-tap sub-lattice and offsets come from a host table
            const int tap = tap_of(kb), cb = kb - tap * P.cblocks;
            if (P.spatial) {
                tma_load_3d(st + TC_A_BYTES, &P.tm_x[P.tap_map[tap]], bar_full + 8 * s, cb * TC_BK,
                            tile_x * P.xw + P.tap_qx[tap], tile_y * P.rows + P.tap_qy[tap]);
            } else {
                tma_load_2d(st + TC_A_BYTES, &P.tm_x[0], bar_full + 8 * s, cb * TC_BK, tile_n * P.n_valid);
            }
        };
        if (warp == 0) {
            // one lane per stage: issuing a load costs a few hundred cycles of address arithmetic and
            // descriptor traffic, so the ring is filled by up to eight lanes at once.  Weights do not depend
            // on the previous kernel: they are requested before the dependency wait, activations after it.
            // coordinates of this lane's activation load: worked out before the dependency wait, so that after it
            // only the copy instruction itself is left on the critical path
            const CUtensorMap* bmap = &P.tm_x[0];
            int bc0 = 0, bc1 = tile_n * P.n_valid, bc2 = 0;
            if (lane < first && !abort0) {
                mbar_expect_tx(bar_full + 8 * lane, tx);
                load_a(lane, lane);
                const int kb = kb_begin + lane, tap = tap_of(kb);
                bc0 = (kb - tap * P.cblocks) * TC_BK;
                if (P.spatial) {
                    bmap = &P.tm_x[P.tap_map[tap]];
                    bc1 = tile_x * P.xw + P.tap_qx[tap];
                    bc2 = tile_y * P.rows + P.tap_qy[tap];
                }
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            // Only now may the next kernel of the stream begin its prologue (set-up, weight loads).  Released
            // any earlier, a chain of these kernels runs ahead without bound and parks its blocks on every SM;
            // in this order at most two grids of a chain are resident and the other SM slots stay free for
            // best-effort kernels.  One thread per CTA executing the instruction counts for the CTA.
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            if (lane < first && !abort0) {
                const uint32_t bdst = base + lane * stage_bytes + TC_A_BYTES;
                if (P.spatial) tma_load_3d(bdst, bmap, bar_full + 8 * lane, bc0, bc1, bc2);
                else tma_load_2d(bdst, bmap, bar_full + 8 * lane, bc0, bc1);
            }
            if (lane == 0) tc_stamp(P, 2);   // ring filled (loads issued)
        }
        __syncwarp();

        // epilogue parameters of this lane's 4 output channels: model constants, requested right after the first loads so
        // that their latency is long gone when the accumulator is ready
        const int cbase = lane * 4;
        const int co = m0 + cbase;
        const bool cvalid = co < P.co;
        float4 sc = make_float4(1.f, 1.f, 1.f, 1.f), sh = make_float4(0.f, 0.f, 0.f, 0.f);
        float4 b2 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (cvalid) {
            if (P.ep & TC_EP_GB) {
                sc = __ldg(reinterpret_cast<const float4*>(P.gamma + co));
                sh = __ldg(reinterpret_cast<const float4*>(P.beta + co));
            } else if (P.ep & TC_EP_BIAS) {
                sh = __ldg(reinterpret_cast<const float4*>(P.bias + co));
            }
            if (P.bias2 != nullptr) b2 = __ldg(reinterpret_cast<const float4*>(P.bias2 + co));
        }
        const float lo = (P.ep & TC_EP_RELU) ? 0.f : -__int_as_float(0x7f800000);
        const bool has_res = (P.ep & TC_EP_RES) != 0;
        const bool rnd = (P.ep & TC_EP_ROUND) != 0;
        const bool gelu = (P.ep & TC_EP_GELU) != 0;

        if (warp == 0 && lane == 0) {
            // ---------------- TMA producer, part 2: refill stages as the MMAs release them ----------------
            // (stage index and phase parity are carried along: a division by the runtime ring depth per K block
            // is dozens of cycles on this single thread's critical path)
            bool ok = true;
            int s = first == NS ? 0 : first;      // first < NS only when nkb < NS, and then this loop does not run
            uint32_t par = 0;                      // parity of the "empty" phase awaited: ((i / NS) - 1) & 1
            int issued = abort0 ? 0 : first;       // K blocks whose loads are out
            bool stop = abort0;
            for (int i = first; i < nkb && ok && !stop; i++) {
                // loop-head poll of the preempt flag (every 4th K block): the load is issued before the wait for a
                // free stage and looked at after it, so its latency hides behind the wait
                int f = 0;
                if (BE && (i & 3) == 0) f = *reinterpret_cast<const volatile int*>(P.preempt_flag);
                ok = mbar_wait(bar_empty + 8 * s, par);
                if (!ok) break;
                if (BE && f != 0) { stop = true; break; }
                mbar_expect_tx(bar_full + 8 * s, tx);
                load_a(i, s);
                load_b(i, s);
                issued++;
                if (++s == NS) { s = 0; par ^= 1u; }
            }
            if (BE && stop) {
                s_flags[2] = (uint32_t)issued;     // first how far the loads got, then the request to stop
                __threadfence_block();
                s_flags[0] = 1;
            }
            if (!ok) s_flags[1] = 1;
        } else if (warp == 1 && lane == 0) {
            // ---------------- MMA issuer ----------------
            bool ok = true;
            const uint32_t idesc = umma_idesc_tf32(P.n_mma);
#ifdef REEF_DEBUG_AIDS
            const bool tr = P.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0;
#endif
            int s = 0;
            uint32_t par = 0;
            for (int i = 0; i < nkb && ok; i++) {
                const uint32_t st = base + s * stage_bytes;
                if (BE) {
                    const int w = mbar_wait_abortable(bar_full + 8 * s, par, &s_flags[0]);
                    if (w == 2) {
                        // The producer stopped.  Loads it had issued may still be in flight: they must have landed
                        // before this CTA leaves or reuses its shared memory, so their barriers are awaited (bounded)
                        // without multiplying.
                        __threadfence_block();
                        const int issued = (int)s_flags[2];
                        for (; i < issued && ok; i++) {
                            ok = mbar_wait(bar_full + 8 * s, par);
                            if (++s == NS) { s = 0; par ^= 1u; }
                        }
                        break;
                    }
                    ok = w == 0;
                } else {
                    ok = mbar_wait(bar_full + 8 * s, par);
                }
                if (!ok) break;
#ifdef REEF_DEBUG_AIDS
                if (tr && i == 0) P.trace[4] = clock64();          // first K block landed
                if (tr && i == nkb - 1) P.trace[5] = clock64();    // last K block landed
#endif
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = umma_desc_sw128(st), db = umma_desc_sw128(st + TC_A_BYTES);
                // one tcgen05.mma covers K = 8 tf32 = 32 bytes.  (Skipping the steps of a ragged last channel block
                // that hold only zero fill was tried: the extra branch in this loop cost every launch 1.3 %.)
#pragma unroll
                for (int k = 0; k < TC_BK / 8; k++)
                    umma_tf32(tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(bar_empty + 8 * s);   // frees the stage once these MMAs have read it
                if (++s == NS) { s = 0; par ^= 1u; }
            }
            if (ok) umma_commit(bar_acc);
            else s_flags[1] = 1;
        }
        __syncwarp();   // lanes 1..31 of the two role warps park here instead of spinning beside their lane 0
        if (warp != 0) asm volatile("griddepcontrol.wait;" ::: "memory");
        // the first two residual rows of this warp's pass over its pixel rows (rows jb + warp + 8u): requested now, used
        // after the exchange
        float4 rpre[2];
#pragma unroll
        for (int u = 0; u < 2; u++) {
            rpre[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            const int jr = warp + 8 * u;
            if (has_res && cvalid && jr < je - jb)
                rpre[u] = __ldg(reinterpret_cast<const float4*>(P.res + (size_t)(pix0 + jb + jr) * P.co + co));
        }

        // ---------------- epilogue: all eight warps ----------------
        bool ok = mbar_wait(bar_acc, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0) tc_stamp(P, 6);   // accumulator complete
        // cluster barrier #1 (arrive here, wait after staging): every rank has finished its main loop, so its
        // stage ring is free to receive exchange data
        // (best-effort flavour: with release semantics, the peers read this CTA's abort word behind the barrier)
        if (S > 1) {
            if (BE) cluster_arrive();
            else cluster_arrive_relaxed();
        }
        const bool my_abort = BE && s_flags[0] != 0;   // final: producer and MMA thread are past their loops
        if (!ok || s_flags[1]) {
            ok = false;
            if (tid == 0 && P.error_word) *reinterpret_cast<volatile int*>(P.error_word) = 1;
        }
        // Phase A — eight warps move the accumulator tile TMEM -> registers -> shared memory as
        // stage[pixel][channel] (warp w reads TMEM lanes 32*(w%4).., its hardware quadrant, and the column
        // chunks of parity w/4).  The stage ring is free by now and is reused for this.
        // Phase B — the tile is finished pixel row by pixel row with 128-bit accesses: one warp per pixel,
        // a lane owns 4 consecutive output channels; it sums the K-split partials of all cluster ranks in
        // rank order 0..S-1 through distributed shared memory (S = 1: its own tile), adds the residual,
        // applies bias | gamma,beta and ReLU, and stores one coalesced 512-byte row per warp.
        const int quad = warp & 3, half = warp >> 2;
        const int row = quad * 32 + lane;              // TMEM lane == output channel within the tile
        const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16);
        float* stage = reinterpret_cast<float*>(smem);
        if (ok && !my_abort) {
            for (int j0 = half * 32; j0 < n_lim; j0 += 64) {
                uint32_t r[32];
                tmem_ld32_nowait(taddr + j0, r);
                tmem_ld_wait();
                float* dst = stage + j0 * TC_BM + row;
                if (j0 + 32 <= n_lim) {   // a full chunk: no per-column test
#pragma unroll
                    for (int j = 0; j < 32; j++) dst[j * TC_BM] = __uint_as_float(r[j]);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (j0 + j < n_lim) dst[j * TC_BM] = __uint_as_float(r[j]);
                }
            }
        }
        if (tid == 0) tc_stamp(P, 7);   // accumulator tile staged in shared memory
        // K-split exchange: rank q finishes pixel rows [q*cpc, (q+1)*cpc).  Every rank sends the rows owned
        // by each peer with ONE bulk shared-memory-to-shared-memory copy per peer (the copy engine moves the
        // bytes and completes the owner's mbarrier); remote loads from distributed shared memory proved an
        // order of magnitude slower here.  Owners then read only their own shared memory.
        float* recv = stage + P.recv_offset_floats;    // recv[slot][cpc_max][128]; sender q uses slot q - (q > owner)
        // The accumulator is out of tensor memory once every warp has passed the barrier below, so the allocating
        // warp frees it there and not at the very end: nothing is then left to do between a CTA's last store and
        // its exit, which is what the next kernel of the stream waits for.
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        bool abort_all = my_abort;
        if (S > 1) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // staged tile -> visible to the copy engine
            __syncthreads();      // the whole tile is staged
            if (warp == 1) tmem_free(tmem, (uint32_t)P.tmem_cols);
            cluster_wait();       // barrier #1: all peers are past their main loops (and their barriers are armed)
            if (tid == 0) tc_stamp(P, 3);
            if (BE) {
                // every rank learns whether ANY rank of the cluster stopped for the preempt flag: one thread per rank
                // reads that rank's abort word through distributed shared memory; all ranks compute the same OR
                uint32_t f = 0;
                if (tid < S)
                    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(f) : "r"(mapa_shared(smem_u32((const void*)&s_flags[0]), (uint32_t)tid)) : "memory");
                abort_all = __syncthreads_or((int)f) != 0;
            }
            if (!abort_all) {
                if (tid < S && tid != split) {   // one thread per peer: the copies are issued side by side
                    const int q = tid;
                    const int qb = min(q * cpc, n_lim), qe = min(qb + cpc, n_lim);
                    const uint32_t bytes = (uint32_t)((qe - qb) * TC_BM * 4);
                    if (bytes != 0) {
                        const int slot = split < q ? split : split - 1;   // the owner keeps no slot for itself
                        const uint32_t dst = mapa_shared(smem_u32(recv + (size_t)slot * P.cpc_max * TC_BM), (uint32_t)q);
                        const uint32_t rbar = mapa_shared(bar_red, (uint32_t)q);
                        asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                     ::"r"(dst), "r"(smem_u32(stage + (size_t)qb * TC_BM)), "r"(bytes), "r"(rbar)
                                     : "memory");
                    }
                }
                if (!mbar_wait(bar_red, 0)) {
                    ok = false;
                    if (tid == 0 && P.error_word) *reinterpret_cast<volatile int*>(P.error_word) = 1;
                }
            }
            // cluster barrier #2 (arrive here, wait before leaving): once all ranks have received what they are
            // owed (and, best-effort flavour, have read each other's abort words), nobody reads a peer's shared
            // memory any more and every CTA may exit
            cluster_arrive();
        } else {
            __syncthreads();
            if (warp == 1) tmem_free(tmem, (uint32_t)P.tmem_cols);
        }

        if (tid == 0) tc_stamp(P, 8);   // exchange complete
        // Four pixel rows per warp are in flight at a time (all partial and residual loads issued before the
        // first use): with one or two warps per scheduler the loop is latency-bound, not bandwidth-bound.
        if (ok && cvalid && !abort_all) {
            constexpr int RB = 4;
            if (S == 1) {
                for (int jbase = jb + warp; jbase < je; jbase += 8 * RB) {
                    float4 v[RB], rv[RB];
#pragma unroll
                    for (int u = 0; u < RB; u++) {
                        const int j = jbase + 8 * u;
                        rv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (j < je) {
                            v[u] = *reinterpret_cast<const float4*>(stage + j * TC_BM + cbase);
                            if (has_res) rv[u] = (u < 2 && jbase == jb + warp) ? rpre[u & 1] : __ldg(reinterpret_cast<const float4*>(P.res + (size_t)(pix0 + j) * P.co + co));
                        }
                    }
#pragma unroll
                    for (int u = 0; u < RB; u++) {
                        const int j = jbase + 8 * u;
                        if (j < je) {
                            const float4 o = tc_epilogue4(v[u], rv[u], sc, sh, lo, rnd, gelu);
                            *reinterpret_cast<float4*>(P.out + (size_t)(pix0 + j) * P.ocs + P.ooff + co) = o;
                            if (P.out2 != nullptr) *reinterpret_cast<float4*>(P.out2 + (size_t)(pix0 + j) * P.co + co) = tc_preact(o, b2, rnd);
                        }
                    }
                }
            } else {
                // partial of rank q for row j: own rows come from the staged tile, the others from recv[q]
                if (S <= 4)
                    tc_finish_split<4, 4>(P, stage, recv, S, split, jb, je, warp, cbase, co, pix0, sc, sh, lo, rnd, gelu, has_res, b2, rpre);
                else
                    tc_finish_split<2, TC_MAX_SPLITS>(P, stage, recv, S, split, jb, je, warp, cbase, co, pix0, sc, sh, lo, rnd,
                                                      gelu, has_res, b2, rpre);
            }
        }
        if (S > 1) cluster_wait();      // barrier #2
        if (tid == 0) tc_stamp(P, 9);   // rows finished
        if (BE && abort_all && tid == 0 && P.stamps != nullptr) {
            // measurement only: when this block saw the preempt flag and left (device clock)
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            atomicMin(&P.stamps[0], t);
            atomicMax(&P.stamps[1], t);
        }
        if (P.task_slot != nullptr && ok && !abort_all) {
            __syncthreads();
            if (tid == 0) {
                __threadfence();
                atomicAdd(P.task_slot, 1);
            }
        }
    }

    if (tid == 32) tc_stamp(P, 10);   // leaving
}

}  // namespace reef
