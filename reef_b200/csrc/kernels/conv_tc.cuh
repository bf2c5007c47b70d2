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
// One thread issues TMA, one thread issues tcgen05.mma, all four warps run the epilogue
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
__device__ __forceinline__ float ld_dsmem_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
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

enum : int { TC_EP_RES = 1, TC_EP_BIAS = 2, TC_EP_GB = 4, TC_EP_RELU = 8, TC_EP_ROUND = 16 };

__device__ __forceinline__ float tc_epilogue(float v, float r, float sc, float sh, int ep) {
    if (ep & TC_EP_RES) v += r;
    if (ep & TC_EP_GB) v = fmaf(v, sc, sh);
    else v += sh;
    if (ep & TC_EP_RELU) v = fmaxf(v, 0.f);
    if (ep & TC_EP_ROUND) {
        // The tensor core reads only the upper 19 bits of an fp32 operand (truncation, a bias toward zero).
        // Rounding the stored activation to the nearest TF32 value makes the consumer's truncation exact.
        uint32_t u;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v));
        v = __uint_as_float(u);
    }
    return v;
}

__global__ void __launch_bounds__(TC_THREADS, 1) reef_conv_tc_kernel(const __grid_constant__ TcParams P) {
    extern __shared__ __align__(16) unsigned char tc_smem_raw[];
    // stage buffers need 1024-byte alignment (swizzle atom); carve barriers behind them
    const uint32_t raw = smem_u32(tc_smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* smem = tc_smem_raw + (base - raw);
    const uint32_t stage_bytes = TC_A_BYTES + (uint32_t)P.n_mma * 128u;
    const uint32_t ctrl = base + TC_STAGES * stage_bytes;
    const uint32_t bar_full = ctrl, bar_empty = ctrl + 8 * TC_STAGES, bar_acc = ctrl + 16 * TC_STAGES;
    volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem + TC_STAGES * stage_bytes + 16 * TC_STAGES + 8);
    volatile uint32_t* s_flags = s_tmem + 1;    // [0] abort (preempt flag seen), [1] wait expired

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // grid = (K splits = cluster, tiles of this launch); a launch may cover a sub-range of the tiles
    const int split = blockIdx.x;
    const int tile = P.tile_begin + (int)blockIdx.y;
    const int tile_n = tile % P.n_tiles, tile_m = tile / P.n_tiles;
    const int S = P.splits;
    const int kb_begin = split * P.kb_per_split;
    const int kb_end = min(kb_begin + P.kb_per_split, P.kb_total);
    const int nkb = kb_end - kb_begin;

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the next kernel may begin its prologue
    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc, 1);
        s_flags[0] = 0;
        s_flags[1] = 0;
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

    // best-effort flavour: one flag read per cluster (rank 0), published to every CTA, so that all CTAs of
    // a cluster take the same decision and none is left alone at a cluster barrier
    bool abort = false;
    if (P.preempt_flag != nullptr) {
        if (tid == 0) s_flags[0] = (uint32_t)(*reinterpret_cast<const volatile int*>(P.preempt_flag) != 0);
        __syncthreads();
        if (S > 1) {
            cluster_sync_all();   // rank 0's observation is written and every CTA of the cluster is running
            uint32_t f;
            asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(f) : "r"(mapa_shared(smem_u32((const void*)&s_flags[0]), 0)) : "memory");
            abort = f != 0;
            cluster_sync_all();   // rank 0 may leave only after everyone has read it
        } else {
            abort = s_flags[0] != 0;
        }
    }

    if (!abort) {
        const int m0 = tile_m * TC_BM;
        if (warp == 0 && lane == 0) {
            // ---------------- TMA producer ----------------
            bool ok = true;
            const uint32_t tx = TC_A_BYTES + (uint32_t)P.b_bytes;
            int issued_a = 0;
            if (P.pdl) {
                // weights do not depend on the previous kernel: start fetching them before the dependency wait
                for (; issued_a < nkb && issued_a < TC_STAGES; issued_a++) {
                    const uint32_t st = base + issued_a * stage_bytes;
                    mbar_expect_tx(bar_full + 8 * issued_a, tx);
                    tma_load_2d(st, &P.tm_w, bar_full + 8 * issued_a, (kb_begin + issued_a) * TC_BK, m0);
                }
                asm volatile("griddepcontrol.wait;" ::: "memory");
            }
            for (int i = 0; i < nkb && ok; i++) {
                const int s = i % TC_STAGES;
                const uint32_t st = base + s * stage_bytes;
                const int kb = kb_begin + i;
                if (i >= TC_STAGES) {
                    ok = mbar_wait(bar_empty + 8 * s, ((i / TC_STAGES) - 1) & 1);
                    if (!ok) break;
                }
                if (i >= issued_a) {
                    mbar_expect_tx(bar_full + 8 * s, tx);
                    tma_load_2d(st, &P.tm_w, bar_full + 8 * s, kb * TC_BK, m0);
                }
                const int tap = kb / P.cblocks, cb = kb - tap * P.cblocks;
                if (P.spatial) {
                    const int ky = tap / P.kw, kx = tap - ky * P.kw;
                    const int dy = ky - P.ph, dx = kx - P.pw;
                    const int sdiv = P.stride;
                    const int ry = ((dy % sdiv) + sdiv) % sdiv, rx = ((dx % sdiv) + sdiv) % sdiv;
                    const int qy = (dy - ry) / sdiv, qx = (dx - rx) / sdiv;
                    tma_load_3d(st + TC_A_BYTES, &P.tm_x[ry * sdiv + rx], bar_full + 8 * s, cb * TC_BK, qx,
                                tile_n * P.rows + qy);
                } else {
                    tma_load_2d(st + TC_A_BYTES, &P.tm_x[0], bar_full + 8 * s, cb * TC_BK, tile_n * P.n_valid);
                }
            }
            if (!ok) s_flags[1] = 1;
        } else if (warp == 1 && lane == 0) {
            // ---------------- MMA issuer ----------------
            bool ok = true;
            const uint32_t idesc = umma_idesc_tf32(P.n_mma);
            for (int i = 0; i < nkb && ok; i++) {
                const int s = i % TC_STAGES;
                const uint32_t st = base + s * stage_bytes;
                ok = mbar_wait(bar_full + 8 * s, (i / TC_STAGES) & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = umma_desc_sw128(st), db = umma_desc_sw128(st + TC_A_BYTES);
#pragma unroll
                for (int k = 0; k < TC_BK / 8; k++)   // one tcgen05.mma covers K = 8 tf32 = 32 bytes
                    umma_tf32(tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(bar_empty + 8 * s);   // frees the stage once these MMAs have read it
            }
            if (ok) umma_commit(bar_acc);
            else s_flags[1] = 1;
        }
        __syncwarp();   // lanes 1..31 of the two role warps park here instead of spinning beside their lane 0
        if (P.pdl && tid != 0) asm volatile("griddepcontrol.wait;" ::: "memory");

        // ---------------- epilogue: all four warps ----------------
        bool ok = mbar_wait(bar_acc, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        __syncthreads();
        if (!ok || s_flags[1]) {
            ok = false;
            if (tid == 0 && P.error_word) atomicExch(P.error_word, 1);
        }
        const int co = m0 + tid;                       // TMEM lane == output channel of the tile
        const bool cvalid = co < P.co;
        const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16);
        const int pix0 = P.spatial ? tile_n * P.rows * P.wo : tile_n * P.n_valid;
        float sc = 1.f, sh = 0.f;
        if (cvalid) {
            if (P.ep & TC_EP_GB) { sc = P.gamma[co]; sh = P.beta[co]; }
            else if (P.ep & TC_EP_BIAS) sh = P.bias[co];
        }
        if (S == 1) {
            if (ok) {
                for (int j0 = 0; j0 < P.n_valid; j0 += 16) {
                    uint32_t r[16];
                    tmem_ld16(taddr + j0, r);
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int pix = pix0 + j0 + j;
                        if (cvalid && j0 + j < P.n_valid && pix < P.ptot) {
                            const float rv = (P.ep & TC_EP_RES) ? P.res[(size_t)pix * P.co + co] : 0.f;
                            P.out[(size_t)pix * P.ocs + P.ooff + co] = tc_epilogue(__uint_as_float(r[j]), rv, sc, sh, P.ep);
                        }
                    }
                }
            }
        } else {
            // park the partial tile in shared memory as red[column][lane]; the stage ring is free now
            float* red = reinterpret_cast<float*>(smem);
            if (ok) {
                for (int j0 = 0; j0 < P.n_mma; j0 += 16) {
                    uint32_t r[16];
                    tmem_ld16(taddr + j0, r);
#pragma unroll
                    for (int j = 0; j < 16; j++) red[(j0 + j) * TC_BM + tid] = __uint_as_float(r[j]);
                }
            }
            cluster_sync_all();
            const int cpc = (P.n_valid + S - 1) / S;   // columns this CTA finishes
            const int jb = split * cpc, je = min(jb + cpc, P.n_valid);
            const uint32_t red_u32 = smem_u32(red);
            if (ok) {
                for (int j = jb; j < je; j++) {
                    float v = 0.f;
                    for (int q = 0; q < S; q++)   // fixed rank order: deterministic sum
                        v += ld_dsmem_f32(mapa_shared(red_u32 + (uint32_t)(j * TC_BM + tid) * 4u, (uint32_t)q));
                    const int pix = pix0 + j;
                    if (cvalid && pix < P.ptot) {
                        const float rv = (P.ep & TC_EP_RES) ? P.res[(size_t)pix * P.co + co] : 0.f;
                        P.out[(size_t)pix * P.ocs + P.ooff + co] = tc_epilogue(v, rv, sc, sh, P.ep);
                    }
                }
            }
            cluster_sync_all();   // nobody leaves while a peer still reads its shared memory
        }
        if (P.task_slot != nullptr && ok) {
            __syncthreads();
            if (tid == 0) {
                __threadfence();
                atomicAdd(P.task_slot, 1);
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)P.tmem_cols) : "memory");
    }
}

}  // namespace reef
