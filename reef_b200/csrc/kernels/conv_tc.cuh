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
#include "tc_common.cuh"

namespace reef {


enum : int { TC_EP_RES = 1, TC_EP_BIAS = 2, TC_EP_GB = 4, TC_EP_RELU = 8, TC_EP_ROUND = 16, TC_EP_GELU = 32 };

// Branch-free form of (+residual) (+bias | *gamma+beta) (ReLU): r = 0, sc = 1, sh = 0, lo = -inf stand in for
// the absent terms (v + 0 and fma(v, 1, b) are exact, so this equals the conditional form bit for bit).
// exact-erf GELU (reference: resource/bert/bert.cu:167-173).  Not inlined on purpose: inlined, the compiler turned
// the uniform `if (gelu)` of the epilogue into straight-line code and every layer paid for erff on each element
// (0.5 us per launch on the row-finishing loop).
static __device__ __noinline__ float tc_gelu(float v) { return v * (0.5f * erff(v * 0.70710678118654752440f) + 0.5f); }

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
// CG: the residual was written earlier in the SAME launch (persistent chain kernel): it is read at L2 (ld.global.cg),
// never through the non-coherent path, and there is no early prefetch.
template <int RB, int SMAX, bool CG = false>
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
                if (has_res) {
                    const float4* rp = reinterpret_cast<const float4*>(P.res + (size_t)(pix0 + jb + jr) * P.co + co);
                    if (CG) rv[u] = __ldcg(rp);
                    else rv[u] = (u < 2 && jbase == warp) ? rpre[u & 1] : __ldg(rp);
                }
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
    // best-effort flavour: the poll at block entry is issued first, so that its latency hides behind the set-up
    int flag0 = 0;
    if (BE && tid == 0) flag0 = *reinterpret_cast<const volatile int*>(P.preempt_flag);
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
        s_flags[0] = (uint32_t)(flag0 != 0);
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
            // A second look at the preempt flag, behind the dependency wait: a best-effort kernel queued behind a
            // running one is resident early (programmatic dependent launch) and made its entry poll long before its
            // predecessor finished, possibly before the flag went up.  Its first loads are out (their barriers were
            // armed for both operands, so the activation loads had to follow the weight loads); it issues no more, and
            // the MMA thread only waits for those to land.
            if (BE && !stop && *reinterpret_cast<const volatile int*>(P.preempt_flag) != 0) stop = true;
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
        const bool my_abort = BE && s_flags[0] != 0;   // final: producer and MMA thread are past their loops
        if (S > 1) {
            // (best-effort flavour: with release semantics, the peers read this CTA's abort word behind the barrier.
            // Nothing may be written into a peer's shared memory before this barrier: only behind it is every CTA
            // of the cluster known to have started.)
            if (BE) cluster_arrive();
            else cluster_arrive_relaxed();
        }
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
            if (tid == 0) red_release_gpu_add(P.task_slot, 1);
        }
    }

    if (tid == 32) tc_stamp(P, 10);   // leaving
}

}  // namespace reef
