// A run of consecutive tensor-core layers of a schedule as ONE persistent kernel.
//
// The per-layer kernel (conv_tc.cuh) is launched once per layer: every launch sets up barriers and tensor memory
// again and the hand-over from one grid to the next goes through the hardware work distributor — which is also where
// best-effort grids that launch and retire beside a real-time chain cost it time.  Here a resident grid of
// 8-CTA clusters walks the layer list itself:
//   * tensor memory is allocated and the mbarriers are initialised once; their phases are carried from tile to tile;
//   * the tile groups of all layers form one ordered list; a cluster takes the next group with a ticket (one atomic
//     by rank 0, handed to the other ranks through distributed shared memory).  Groups are taken in order, so the
//     layers a group depends on are always held by clusters that are running: the walk cannot deadlock however few
//     clusters the hardware has made resident (a best-effort chain shares the GPU with real-time kernels of greater
//     priority).  Which cluster computes a tile does not matter for the result: the arithmetic of a tile is fixed;
//   * a cluster of 8 serves every K split of the per-layer plans: with S splits it works on 8/S tiles at once, the
//     K-split exchange staying inside each group of S ranks;
//   * layers are ordered by completion counters in global memory: every CTA that has stored its rows adds one
//     (release) to the counter of its layer, and the TMA producer of a tile of layer l+1 first requests its weights
//     (they depend on nothing), then waits (acquire, bounded by %globaltimer -> error word) until the counter of
//     layer l is complete before it requests activations.  By induction a tile of layer l+1 that runs implies every
//     layer before l+1 is complete, so residual inputs need no counter of their own.
// The tile body is the per-layer kernel's: TMA ring -> tcgen05.mma (TF32, fp32 accumulate in TMEM) -> staging ->
// K-split exchange over distributed shared memory in fixed rank order -> fused epilogue; results are bit-identical
// to the per-layer launches.
// Best-effort use (preempt_flag != nullptr): rank 0 reads the flag whenever it takes a ticket and hands out "stop"
// instead: every cluster leaves at its next tile boundary (a tile is a few microseconds).  The completion counters
// say how far each layer got; the host restarts the chain at the first incomplete layer (layers are idempotent).
#pragma once
#include <cstddef>

#include "conv_tc.cuh"

namespace reef {

constexpr int TC_CHAIN_CLUSTER = 8;

struct ChainParams {
    const int* preempt_flag;  // best-effort use: polled at every ticket; nullptr for a real-time chain
    int first_group;          // (informative) the ticket counter starts here: a restart skips the complete layers
    int total_groups;
    const TcParams* layers;   // device array, one entry per layer (tensor maps included: 64-byte aligned entries)
    const int* need;          // need[l] = CTAs of layer l-1 that must have finished before layer l may read (need[0] = 0);
                              // need[n_layers + 1 + l] = tile groups of all layers before l (deals the groups out in turn)
    int* done;                // done[l] = CTAs of layer l-1 that have finished; done[n_layers + 1] = "a CTA gave up";
                              // done[n_layers + 2] = the ticket counter.  Initialised by the host before every launch
    int* error_word;
    int n_layers;
    int ctrl_offset;          // offset of the control words in dynamic shared memory = largest data region of any layer
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(TC_THREADS, 2) reef_conv_tc_chain_kernel(const __grid_constant__ ChainParams C) {
    extern __shared__ __align__(16) unsigned char tc_smem_raw[];
    const uint32_t raw = smem_u32(tc_smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* smem = tc_smem_raw + (base - raw);
    const uint32_t ctrl = base + (uint32_t)C.ctrl_offset;
    const uint32_t bar_full = ctrl, bar_empty = ctrl + 8 * TC_MAX_STAGES, bar_acc = ctrl + 16 * TC_MAX_STAGES;
    const uint32_t bar_red = bar_acc + 8;
    volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem + C.ctrl_offset + 16 * TC_MAX_STAGES + 16);
    volatile uint32_t* s_flags = s_tmem + 1;    // [0] some CTA of the grid gave up (read once per tile), [1] a wait of
                                                //  this CTA expired; both sticky for the rest of the launch.  [4],[5]: tickets

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rank = (int)cluster_ctarank();      // 0..7
    constexpr uint32_t TMEM_COLS = 256;

    if (tid == 0) {
        for (int s = 0; s < TC_MAX_STAGES; s++) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc, 1);
        mbar_init(bar_red, 1);
        s_flags[0] = 0;
        s_flags[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)s_tmem)), "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *s_tmem;
    // every CTA of the cluster has initialised its barriers before any peer may complete one remotely
    cluster_sync_all();
    // the layers before this chain belong to earlier kernels of the stream
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // mbarrier phases carried across tiles: bit s = parity the next wait on slot s uses
    uint32_t full_bits = 0;          // MMA thread
    uint32_t empty_bits = 0xffu;     // producer (lane 0 of warp 0): a fresh barrier passes a wait on parity 1 at once
    uint32_t acc_par = 0, red_par = 0;
    bool ok = true;

    // The scalar fields of the current layer's parameters live in shared memory (a per-layer cooperative copy: read
    // from global memory on every use they put dependent L1/L2 latencies into the producer's and the MMA thread's
    // loops); the tensor maps are used where they are, in global memory, as TMA requires.
    // (the copy skips the five tensor maps at the head of the struct: the pointer below is only ever used for the
    // fields behind them)
    constexpr int kMapBytes = 5 * (int)sizeof(CUtensorMap);
    static_assert(offsetof(TcParams, out) == kMapBytes, "the tensor maps lead the struct");
    static_assert((sizeof(TcParams) - kMapBytes) % 8 == 0, "copied in 8-byte words");
    TcParams* Ps = reinterpret_cast<TcParams*>(smem + C.ctrl_offset + 256 - kMapBytes);

    const int* goff = C.need + C.n_layers + 1;          // goff[l] = tile groups of all layers before l
    volatile int* s_ticket = reinterpret_cast<volatile int*>(s_flags + 4);   // [2]: alternating, a rank lags at most one turn
    int L = 0, cur_L = -1, turn = 0;

#pragma unroll 1
    for (;; turn ^= 1) {
        // ---- the next tile group: rank 0 takes a ticket and hands it to every rank of the cluster ----
        if (rank == 0 && tid == 0) {
            int G = -1;
            const bool stop = (C.preempt_flag != nullptr && *reinterpret_cast<const volatile int*>(C.preempt_flag) != 0) || s_flags[0] != 0 || s_flags[1] != 0;
            if (!stop) {
                G = atomicAdd(&C.done[C.n_layers + 2], 1);
                if (G >= C.total_groups) G = -1;
            }
            for (uint32_t q = 0; q < (uint32_t)TC_CHAIN_CLUSTER; q++)
                st_dsmem_u32(mapa_shared(smem_u32((const void*)&s_ticket[turn]), q), (uint32_t)G);
        }
        cluster_sync_all();      // the ticket is in every rank's shared memory
        const int G = s_ticket[turn];
        if (G < 0) break;
        while (G >= goff[L + 1]) L++;
        const TcParams& Pg = C.layers[L];
        if (L != cur_L) {
            __syncthreads();     // every thread is done with the previous layer's parameters
            const unsigned long long* src = reinterpret_cast<const unsigned long long*>(reinterpret_cast<const unsigned char*>(&Pg) + kMapBytes);
            unsigned long long* dst = reinterpret_cast<unsigned long long*>(smem + C.ctrl_offset + 256);
            for (int i = tid; i < (int)((sizeof(TcParams) - kMapBytes) / 8); i += TC_THREADS) dst[i] = __ldg(src + i);
            __syncthreads();
            cur_L = L;
        }
        const TcParams& P = *Ps;
        const int S = P.splits;
        const int per = TC_CHAIN_CLUSTER / S;                       // tiles a cluster works on at once
        const int tiles = P.n_tiles * ((P.co + TC_BM - 1) / TC_BM);
        const int NS = P.stages;
        const uint32_t stage_bytes = TC_A_BYTES + (uint32_t)P.n_mma * 128u;
        const int split = rank % S, sub = rank / S;                 // K-split rank and tile slot inside the cluster
        const uint32_t grp_base = (uint32_t)(sub * S);              // cluster rank of this group's split 0
        const int g = G - goff[L];
        {
            const int tile = g * per + sub;
            // after a failure anywhere in the grid the CTAs only keep their cluster barriers going (every wait is
            // bounded, and nothing new is started, so the launch ends within a few seconds at worst)
            const bool valid = tile < tiles && s_flags[0] == 0 && s_flags[1] == 0;
            const int tile_n = tile % P.n_tiles, tile_m = tile / P.n_tiles;
            const int kb_begin = split * P.kb_per_split;
            const int kb_end = min(kb_begin + P.kb_per_split, P.kb_total);
            const int nkb = valid ? kb_end - kb_begin : 0;
            const int tile_y = P.xsplit > 1 ? tile_n / P.xsplit : tile_n, tile_x = P.xsplit > 1 ? tile_n - tile_y * P.xsplit : 0;
            const int pix0 = P.spatial ? tile_y * P.rows * P.wo + tile_x * P.xw : tile_n * P.n_valid;
            const int n_lim = valid ? min(P.n_valid, P.ptot - pix0) : 0;
            const int cpc = (n_lim + S - 1) / S;
            const int jb = min(split * cpc, n_lim), je = min(jb + cpc, n_lim);
            if (S > 1 && valid && tid == 0) mbar_expect_tx(bar_red, (uint32_t)((S - 1) * (je - jb) * TC_BM * 4));

            const int m0 = tile_m * TC_BM;
            const uint32_t tx = TC_A_BYTES + (uint32_t)P.b_bytes;
            const int first = nkb < NS ? nkb : NS;
            auto tap_of = [&](int kb) { return P.cblocks == 1 ? kb : (int)__umulhi((unsigned)kb, P.cb_magic); };
            auto load_a = [&](int i, int s) {
                const int kb = kb_begin + i, tap = tap_of(kb), cb = kb - tap * P.cblocks;
                tma_load_3d(base + s * stage_bytes, &Pg.tm_w, bar_full + 8 * s, cb * TC_BK, tap, m0);
            };
            auto load_b = [&](int i, int s) {
                const uint32_t st = base + s * stage_bytes;
                const int kb = kb_begin + i;
                const int tap = tap_of(kb), cb = kb - tap * P.cblocks;
                if (P.spatial) {
                    tma_load_3d(st + TC_A_BYTES, &Pg.tm_x[P.tap_map[tap]], bar_full + 8 * s, cb * TC_BK,
                                tile_x * P.xw + P.tap_qx[tap], tile_y * P.rows + P.tap_qy[tap]);
                } else {
                    tma_load_2d(st + TC_A_BYTES, &Pg.tm_x[0], bar_full + 8 * s, cb * TC_BK, tile_n * P.n_valid);
                }
            };
            if (warp == 0 && nkb > 0) {
                // ---- producer, part 1: one lane per stage; weights first, then the dependency, then activations ----
                const uint32_t ebits = __shfl_sync(0xffffffffu, empty_bits, 0);
                bool lane_ok = true;
                if (lane < first) {
                    lane_ok = mbar_wait(bar_empty + 8 * lane, (ebits >> lane) & 1u);   // free since the previous tile's commits
                    if (lane_ok) {
                        mbar_expect_tx(bar_full + 8 * lane, tx);
                        load_a(lane, lane);
                    }
                }
                // the previous layer is complete: bounded acquire spin by lane 0, one confirming acquire by the others
                const int need = C.need[L];
                if (need > 0) {
                    int have = 0;
                    if (lane == 0) {
                        unsigned long long t0 = 0;
                        for (int it = 0;; it++) {
                            have = ld_acquire_gpu(&C.done[L]);
                            if (have >= need) break;
                            if ((it & 63) == 63) {
                                if (ld_acquire_gpu(&C.done[C.n_layers + 1]) != 0) break;   // some CTA gave up
                                unsigned long long t;
                                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                                if (t0 == 0) t0 = t;
                                else if (t - t0 > 1000000000ull) break;
                            }
                        }
                    }
                    have = __shfl_sync(0xffffffffu, have, 0);
                    if (have < need) lane_ok = false;
                    asm volatile("fence.proxy.async.global;" ::: "memory");   // generic stores of other CTAs -> the TMA reads below
                }
                if (lane < first && lane_ok) load_b(lane, lane);
                const unsigned bad = __ballot_sync(0xffffffffu, !lane_ok);
                if (lane == 0) {
                    for (int s = 0; s < first; s++) empty_bits ^= 1u << s;
                    // ---- producer, part 2: refill stages as the MMAs release them ----
                    bool pok = bad == 0;
                    int s = first == NS ? 0 : first;
                    for (int i = first; i < nkb && pok; i++) {
                        pok = mbar_wait(bar_empty + 8 * s, (empty_bits >> s) & 1u);
                        if (!pok) break;
                        empty_bits ^= 1u << s;
                        mbar_expect_tx(bar_full + 8 * s, tx);
                        load_a(i, s);
                        load_b(i, s);
                        if (++s == NS) s = 0;
                    }
                    if (!pok) s_flags[1] = 1;
                }
            } else if (warp == 1 && lane == 0 && nkb > 0) {
                // ---- MMA issuer ----
                bool mok = true;
                const uint32_t idesc = umma_idesc_tf32(P.n_mma);
                int s = 0;
                for (int i = 0; i < nkb && mok; i++) {
                    const uint32_t st = base + s * stage_bytes;
                    mok = mbar_wait(bar_full + 8 * s, (full_bits >> s) & 1u);
                    if (!mok) break;
                    full_bits ^= 1u << s;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t da = umma_desc_sw128(st), db = umma_desc_sw128(st + TC_A_BYTES);
#pragma unroll
                    for (int k = 0; k < TC_BK / 8; k++)
                        umma_tf32(tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
                    umma_commit(bar_empty + 8 * s);
                    if (++s == NS) s = 0;
                }
                if (mok) umma_commit(bar_acc);
                else s_flags[1] = 1;
            }
            __syncwarp();

            // epilogue parameters of this lane's 4 output channels
            const int cbase = lane * 4;
            const int co = m0 + cbase;
            const bool cvalid = valid && co < P.co;
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

            // ---- epilogue: all eight warps ----
            if (nkb > 0) {
                if (!mbar_wait(bar_acc, acc_par)) ok = false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            __syncthreads();
            if (nkb > 0) acc_par ^= 1u;
            if (S > 1) cluster_arrive_relaxed();     // barrier #1: this rank's ring is free to receive exchange data
            if (s_flags[1]) ok = false;
            const int quad = warp & 3, half = warp >> 2;
            const int row = quad * 32 + lane;
            const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16);
            float* stage = reinterpret_cast<float*>(smem);
            if (ok && nkb > 0) {
                for (int j0 = half * 32; j0 < n_lim; j0 += 64) {
                    uint32_t r[32];
                    tmem_ld32_nowait(taddr + j0, r);
                    tmem_ld_wait();
                    float* dst = stage + j0 * TC_BM + row;
                    if (j0 + 32 <= n_lim) {
#pragma unroll
                        for (int j = 0; j < 32; j++) dst[j * TC_BM] = __uint_as_float(r[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (j0 + j < n_lim) dst[j * TC_BM] = __uint_as_float(r[j]);
                    }
                }
            }
            float* recv = stage + P.recv_offset_floats;
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            if (S > 1) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncthreads();
                cluster_wait();                   // barrier #1
                if (valid && ok) {
                    if (tid < S && tid != split) {
                        const int q = tid;
                        const int qb = min(q * cpc, n_lim), qe = min(qb + cpc, n_lim);
                        const uint32_t bytes = (uint32_t)((qe - qb) * TC_BM * 4);
                        if (bytes != 0) {
                            const int slot = split < q ? split : split - 1;
                            const uint32_t dst = mapa_shared(smem_u32(recv + (size_t)slot * P.cpc_max * TC_BM), grp_base + (uint32_t)q);
                            const uint32_t rbar = mapa_shared(bar_red, grp_base + (uint32_t)q);
                            asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                         ::"r"(dst), "r"(smem_u32(stage + (size_t)qb * TC_BM)), "r"(bytes), "r"(rbar)
                                         : "memory");
                        }
                    }
                }
                if (valid) {
                    // (a rank whose peers gave up never receives: the wait is bounded and the launch is marked failed)
                    if (!mbar_wait(bar_red, red_par)) ok = false;
                    red_par ^= 1u;
                }
                cluster_arrive();                 // barrier #2: nobody reads this rank's shared memory after it
            } else {
                __syncthreads();
            }

            if (ok && cvalid) {
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
                                if (has_res) rv[u] = __ldcg(reinterpret_cast<const float4*>(P.res + (size_t)(pix0 + j) * P.co + co));
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
                } else if (S <= 4) {
                    tc_finish_split<4, 4, true>(P, stage, recv, S, split, jb, je, warp, cbase, co, pix0, sc, sh, lo, rnd, gelu, has_res, b2, nullptr);
                } else {
                    tc_finish_split<2, TC_MAX_SPLITS, true>(P, stage, recv, S, split, jb, je, warp, cbase, co, pix0, sc, sh, lo, rnd, gelu,
                                                            has_res, b2, nullptr);
                }
            }
            // this CTA's rows of layer L are in global memory: publish (every thread orders its own stores first)
            __threadfence();
            if (S > 1) cluster_wait();            // barrier #2
            __syncthreads();
            if (tid == 0) {
                if (valid && ok && !s_flags[1]) red_release_gpu_add(&C.done[L + 1], 1);
                else if (!ok || s_flags[1]) red_release_gpu_add(&C.done[C.n_layers + 1], 1);   // tell the grid
                // (looked at behind the increment: the read is off the path the next layer waits on; it takes
                // effect from the tile after next, which the second barrier below makes uniform for the CTA)
                if (ld_acquire_gpu(&C.done[C.n_layers + 1]) != 0) s_flags[0] = 1;
            }
            __syncthreads();
        }
    }
    if (!ok && tid == 0 && C.error_word) *reinterpret_cast<volatile int*>(C.error_word) = 1;
    // the kernels behind the chain may start their prologues
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();     // no CTA leaves while a peer could still address its shared memory
    if (warp == 1) tmem_free(tmem, TMEM_COLS);
}

}  // namespace reef
