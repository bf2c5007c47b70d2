// Multi-head self-attention on the 5th-generation tensor cores (tcgen05, TF32 inputs, fp32 accumulate in TMEM).
//
// One CTA per head, up to 128 tokens, head dimension 64.  On the fused [token][Q | K | V] buffer the QKV projection
// wrote (reference: the same math spread over resource/bert/bert.cu:22-157 batch_matmul_4/5, :289-311 the Q / sqrt(d)
// divide and the head transposes, :381-387 the masked fill, and the four softmax launches :3-12,159-165,327-336,389-395):
//
//   1. TMA brings Q and K of the head into shared memory as K-major 128-byte-swizzled UMMA operands (two blocks of
//      32 dimensions each); rows beyond the sequence come back as zeros.
//   2. scores[query][key] = Q K^T: 8 tcgen05.mma (M = 128 queries on the TMEM lanes, N = 128 keys on its columns).
//      Meanwhile all threads transpose V through registers into a K-major operand Vt[d][key].
//   3. Every thread owns one query row and half of its keys (tcgen05.ld, 64 columns): scale, mask, row maximum and
//      sum (exchanged between the two threads of a row through shared memory), exp; the probabilities go back to
//      shared memory, rounded to TF32, as the A operand of the second product — over the dead Q and K tiles.
//   4. ctx = P Vt^T: 16 tcgen05.mma (N = 64) into another 64 TMEM columns; the epilogue divides by the row sum and
//      stores 128 contiguous bytes per thread.
//
// Every mbarrier wait is bounded (error word, as in the convolution).  Best-effort flavour: the preempt flag is read
// at block entry and again at the head of the second product; a CTA that sees it frees its TMEM and leaves without
// counting itself complete.
#pragma once
#include "tc_common.cuh"

namespace reef {

constexpr int ATT_THREADS = 256;
constexpr int ATT_D = 64;
constexpr int ATT_MAX_S = 128;
constexpr int ATT_KBLOCK_BYTES = 128 * 128;            // 128 rows x 32 floats: one K block of a 128-row operand
constexpr int ATT_QK_BYTES = 4 * ATT_KBLOCK_BYTES;     // Q (2 blocks) + K (2 blocks) = 64 KB, later P (4 blocks)
constexpr int ATT_VT_BYTES = 4 * 64 * 128;             // Vt: 4 key blocks of [64 d rows][32 keys] = 32 KB
constexpr int ATT_SMEM = 1024 + ATT_QK_BYTES + ATT_VT_BYTES + 2 * 2 * 128 * 4 + 128 * 4 + 64;

struct AttParams {
    CUtensorMap tm_qkv;      // 2-d map over [token][3H]: dims (3H, S), box (32, 128)
    const float* qkv;
    const float* mask;       // [S], 0 = masked key, or nullptr
    float* out;              // [S][H]
    const int* preempt_flag; // best-effort flavour, else nullptr
    int* task_slot;
    int* error_word;
    unsigned long long* stamps;
    int S, heads;
    int head_begin;          // first head of this launch (dynamic kernel padding launches sub-ranges)
    float scale;             // 1 / sqrt(d)
};

template <bool BE>
__global__ void __launch_bounds__(ATT_THREADS, 2) reef_attention_tc_kernel(const __grid_constant__ AttParams P) {
    extern __shared__ __align__(16) unsigned char att_smem_raw[];
    const uint32_t raw = smem_u32(att_smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* smem = att_smem_raw + (base - raw);
    const uint32_t qk = base;                             // Q blocks 0,1 | K blocks 0,1 ; later P blocks 0..3
    const uint32_t vt = base + ATT_QK_BYTES;
    float* red_max = reinterpret_cast<float*>(smem + ATT_QK_BYTES + ATT_VT_BYTES);   // [2][128]
    float* red_sum = red_max + 2 * 128;                                               // [2][128]
    float* s_bias = red_sum + 2 * 128;                                                // [128]: 0 or -inf per key
    const uint32_t ctrl = base + ATT_QK_BYTES + ATT_VT_BYTES + 5 * 128 * 4;
    const uint32_t bar_qk = ctrl, bar_mma1 = ctrl + 8, bar_mma2 = ctrl + 16;
    volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem + ATT_QK_BYTES + ATT_VT_BYTES + 5 * 128 * 4 + 24);
    volatile uint32_t* s_flags = s_tmem + 1;   // [0] preempt flag seen, [1] wait expired

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int head = P.head_begin + (int)blockIdx.x;
    const int S = P.S, H = P.heads * ATT_D;
    constexpr uint32_t TMEM_COLS = 256;   // 128 score columns + 64 context columns, rounded up to a power of two

    if (tid == 0) {
        mbar_init(bar_qk, 1);
        mbar_init(bar_mma1, 1);
        mbar_init(bar_mma2, 1);
        s_flags[0] = BE ? (uint32_t)(*reinterpret_cast<const volatile int*>(P.preempt_flag) != 0) : 0u;   // poll at block entry
        s_flags[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&P.tm_qkv) : "memory");
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

    // the QKV projection is the previous kernel of the stream: nothing of it may be read before this wait
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // best-effort flavour: the flag is looked at again behind the wait (a kernel queued behind a running one is
    // resident early and made its entry poll before its predecessor finished, possibly before the flag went up)
    bool stop = false;
    if (BE) {
        if (tid == 0 && *reinterpret_cast<const volatile int*>(P.preempt_flag) != 0) s_flags[0] = 1;
        __syncthreads();
        stop = s_flags[0] != 0;
    }

    bool ok = true;
    if (!stop) {
        if (tid == 0) {
            // Q and K of this head: four boxes of [128 tokens][32 dims]
            mbar_expect_tx(bar_qk, (uint32_t)ATT_QK_BYTES);
            const int cq = head * ATT_D, ck = H + head * ATT_D;
            tma_load_2d(qk + 0 * ATT_KBLOCK_BYTES, &P.tm_qkv, bar_qk, cq, 0);
            tma_load_2d(qk + 1 * ATT_KBLOCK_BYTES, &P.tm_qkv, bar_qk, cq + 32, 0);
            tma_load_2d(qk + 2 * ATT_KBLOCK_BYTES, &P.tm_qkv, bar_qk, ck, 0);
            tma_load_2d(qk + 3 * ATT_KBLOCK_BYTES, &P.tm_qkv, bar_qk, ck + 32, 0);
        }
        // additive key bias: -inf for keys beyond the sequence and for masked keys
        if (tid < 128) {
            const bool dead = tid >= S || (P.mask != nullptr && P.mask[tid] == 0.f);
            s_bias[tid] = dead ? -__int_as_float(0x7f800000) : 0.f;
        }
        // V -> Vt[d][key], K-major with the 128-byte swizzle: element (d, key) lives in key block key / 32, row d,
        // 16-byte chunk ((key % 32) / 4) ^ (d % 8), word key % 4.  A lane stands for a key, a warp for two groups of
        // four dimensions: all eight 128-bit loads of a thread are in flight at once, and for a fixed d the 32
        // lanes store to 32 different banks.
        {
            float* vts = reinterpret_cast<float*>(smem + ATT_QK_BYTES);
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int key = (u >> 1) * 32 + lane, d0 = (warp * 2 + (u & 1)) * 4;
                v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (key < S) v[u] = *reinterpret_cast<const float4*>(P.qkv + (size_t)key * 3 * H + 2 * H + head * ATT_D + d0);
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int kb = u >> 1, d0 = (warp * 2 + (u & 1)) * 4;
                const float e[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int d = d0 + j;
                    vts[kb * (64 * 32) + d * 32 + (((lane >> 2) ^ (d & 7)) << 2) + (lane & 3)] = e[j];
                }
            }
        }
        // ---- scores = Q K^T ----
        if (warp == 1 && lane == 0) {
            ok = mbar_wait(bar_qk, 0);
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t idesc = umma_idesc_tf32(128);
#pragma unroll
                for (int kb = 0; kb < 2; kb++) {
                    const uint64_t da = umma_desc_sw128(qk + kb * ATT_KBLOCK_BYTES);
                    const uint64_t db = umma_desc_sw128(qk + (2 + kb) * ATT_KBLOCK_BYTES);
#pragma unroll
                    for (int k = 0; k < 4; k++) umma_tf32(tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(bar_mma1);
            } else {
                s_flags[1] = 1;
            }
        }
        __syncwarp();
        __syncthreads();                       // s_bias and Vt written; the MMA thread is past its wait (or gave up)
        if (s_flags[1]) ok = false;
        if (ok) ok = mbar_wait(bar_mma1, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

        // ---- softmax over the 128 keys of a row: thread = (row, half of the keys) ----
        const int quad = warp & 3, half = warp >> 2;
        const int row = quad * 32 + lane;
        const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16);
        // pass 1: the row maximum of this thread's 64 keys (32 columns at a time: the scores stay in tensor memory
        // and are read again in pass 2, which keeps this kernel at two CTAs per SM like its neighbours)
        float m = -__int_as_float(0x7f800000);
        if (ok) {
#pragma unroll
            for (int c = 0; c < 2; c++) {
                uint32_t r[32];
                tmem_ld32_nowait(taddr + half * 64 + c * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; j++) m = fmaxf(m, fmaf(__uint_as_float(r[j]), P.scale, s_bias[half * 64 + c * 32 + j]));
            }
        }
        red_max[half * 128 + row] = m;
        __syncthreads();                       // both halves of every row have their maximum
        m = fmaxf(red_max[row], red_max[128 + row]);
        float sum = 0.f;
        if (ok) {
            // pass 2: exp, rounded to TF32 (what the tensor core will multiply; the row sum adds the same rounded
            // values), written as the A operand of the second product.  Q and K are dead (the first product is
            // complete): P takes their place, one 128-byte row per key block.
            float* ps = reinterpret_cast<float*>(smem);
#pragma unroll
            for (int c = 0; c < 2; c++) {
                uint32_t r[32];
                tmem_ld32_nowait(taddr + half * 64 + c * 32, r);
                tmem_ld_wait();
                float* blk = ps + (half * 2 + c) * (128 * 32) + row * 32;
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    float e[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float v = __expf(fmaf(__uint_as_float(r[q * 4 + j]), P.scale, s_bias[half * 64 + c * 32 + q * 4 + j]) - m);
                        uint32_t u;
                        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v));
                        e[j] = __uint_as_float(u);
                        sum += e[j];
                    }
                    *reinterpret_cast<float4*>(blk + ((q ^ (row & 7)) << 2)) = make_float4(e[0], e[1], e[2], e[3]);
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        red_sum[half * 128 + row] = sum;
        // loop-head poll of the preempt flag before the second product
        if (BE && tid == 0 && *reinterpret_cast<const volatile int*>(P.preempt_flag) != 0) s_flags[0] = 1;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P and Vt (generic stores) -> visible to the tensor core
        __syncthreads();
        stop = BE && s_flags[0] != 0;

        // ---- ctx = P Vt^T ----
        if (!stop) {
            if (warp == 1 && lane == 0 && ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t idesc = umma_idesc_tf32(ATT_D);
#pragma unroll
                for (int kb = 0; kb < 4; kb++) {
                    const uint64_t da = umma_desc_sw128(qk + kb * ATT_KBLOCK_BYTES);
                    const uint64_t db = umma_desc_sw128(vt + kb * (64 * 128));
#pragma unroll
                    for (int k = 0; k < 4; k++) umma_tf32(tmem + 128, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(bar_mma2);
            }
            __syncwarp();
            if (ok) ok = mbar_wait(bar_mma2, 0);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (ok) {
                uint32_t r[32];
                tmem_ld32_nowait(taddr + 128 + half * 32, r);   // warp-collective: every lane loads, valid rows store
                tmem_ld_wait();
                if (row < S) {
                const float inv = 1.0f / (red_sum[row] + red_sum[128 + row]);
                float* dst = P.out + (size_t)row * H + head * ATT_D + half * 32;
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    float4 o;
                    o.x = __uint_as_float(r[c * 4]) * inv; o.y = __uint_as_float(r[c * 4 + 1]) * inv;
                    o.z = __uint_as_float(r[c * 4 + 2]) * inv; o.w = __uint_as_float(r[c * 4 + 3]) * inv;
                    *reinterpret_cast<float4*>(dst + c * 4) = o;
                }
                }
            }
        }
    }
    if (!ok && tid == 0 && P.error_word) *reinterpret_cast<volatile int*>(P.error_word) = 1;
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) tmem_free(tmem, TMEM_COLS);
    if (tid == 0) {
        if (BE && stop && P.stamps != nullptr) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            atomicMin(&P.stamps[0], t);
            atomicMax(&P.stamps[1], t);
        }
        if (P.task_slot != nullptr && ok && !stop) red_release_gpu_add(P.task_slot, 1);
    }
}

}  // namespace reef
