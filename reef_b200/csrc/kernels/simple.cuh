// HBM-bound kernel families: elementwise, pooling, dense (GEMV), softmax, copies and the
// reference's mocked add/multiply.  All are written as 256-thread logical-block bodies
// (see task.cuh) with 128-bit coalesced accesses and warp-shuffle reductions; none of them
// touches a tensor core — their roofline is HBM bandwidth.
#pragma once
#include "task.cuh"
#include <float.h>

namespace reef {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---- mocked_kernel (reference: resource/mocked_kernel/mocked_kernel.cu:9-29) -------------------
// launch [64,1,1, 4,8,4]: 128 threads; out[blk*128+t] = a[t] (op) b[blk*128+t].
constexpr int kMockThreads = 128;
template <bool MUL>
__device__ __forceinline__ bool body_mock(const KTask& t, int vb, unsigned char*, const int*) {
    const float* a = (const float*)t.a[0];
    const float* b = (const float*)t.a[1];
    float* out = (float*)t.a[2];
    int tid = threadIdx.x + threadIdx.y * blockDim.x + threadIdx.z * blockDim.x * blockDim.y;
    if (tid < kMockThreads) {
        int i = vb * kMockThreads + tid;
        out[i] = MUL ? a[tid] * b[i] : a[tid] + b[i];
    }
    return true;
}

// ---- fused_add on the NCHW model input (reference: resource/resnet152/resnet152.cu:771-773) ----
// args: out, in, bias.  One vblock = 4096 consecutive elements of one plane-major tensor.
constexpr int kEltPerBlock = 1024;   // one 128-bit access per thread: batch-1 tensors are small, parallelism beats reuse
__device__ __forceinline__ bool body_fused_add_nchw(const KTask& t, int vb, unsigned char*, const int*) {
    const EltP& p = t.p.elt;
    float* out = (float*)t.a[0];
    const float* in = (const float*)t.a[1];
    const float* bias = (const float*)t.a[2];
    const int total = p.c * p.n;
    int base = vb * kEltPerBlock + threadIdx.x * 4;
#pragma unroll
    for (int it = 0; it < kEltPerBlock / (kThreads * 4); it++) {
        int i = base + it * kThreads * 4;
        if (i + 3 < total && (p.n & 3) == 0) {
            float4 v = *reinterpret_cast<const float4*>(in + i);
            float b = bias[i / p.n];
            v.x += b; v.y += b; v.z += b; v.w += b;
            *reinterpret_cast<float4*>(out + i) = v;
        } else {
            for (int j = 0; j < 4; j++)
                if (i + j < total) out[i + j] = in[i + j] + bias[(i + j) / p.n];
        }
    }
    return true;
}

// ---- model input for the tensor-core stem: planar NCHW (c <= 4) + per-channel bias -> channels-last with 4
// channels per pixel (the missing ones zero), rounded to the nearest TF32 value.  The reference adds the bias
// with its fused_add kernel on the planar tensor (resource/resnet152/resnet152.cu:771-773); the layout change
// lets the first convolution run on the tensor cores (a 16-byte pixel is the smallest TMA element).
// args: out [hw][4], in [c][hw], bias [c].  One thread = one pixel.
__device__ __forceinline__ bool body_nchw_to_nhwc4(const KTask& t, int vb, unsigned char*, const int*) {
    const EltP& p = t.p.elt;
    float* out = (float*)t.a[0];
    const float* in = (const float*)t.a[1];
    const float* bias = (const float*)t.a[2];
    const int i = vb * kThreads + threadIdx.x;
    if (i < p.n) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        for (int c = 0; c < p.c; c++) {
            uint32_t u;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(in[(size_t)c * p.n + i] + bias[c]));
            v[c] = __uint_as_float(u);
        }
        *reinterpret_cast<float4*>(out + (size_t)i * 4) = make_float4(v[0], v[1], v[2], v[3]);
    }
    return true;
}

// ---- model input for the first convolution on the tensor cores: planar NCHW (+ per-channel bias) -> the im2col
// matrix out[pixel][kp], k = (ky * kw + kx) * c + channel for k < kh*kw*c, zero beyond (kp = K rounded up to whole
// 32-channel K blocks) and zero where the tap falls into the padding (the bias is added to real input values only:
// the reference adds it with fused_add on the planar tensor, resource/resnet152/resnet152.cu:771-773, and the
// convolution pads the sum with zeros).  Values are rounded to the nearest TF32.  The first convolution is then a
// 1x1 convolution (X W^T) over kp "channels" with the weights flattened in the same k order: 7x7x3 = 147 of 160
// operand columns carry data, where a 4-channel channels-last input left 7/8 of every K block empty.
// args: out [ho*wo][kp], in [c][hi][wi], bias [c].  A thread writes four consecutive k of a pixel per step.
constexpr int kIm2colPerBlock = 1024;   // 128-bit items per logical block
constexpr int kIm2colMaxKp = 512;       // columns of the matrix (the lookup table lives in shared memory)
__device__ __forceinline__ bool body_im2col_nchw(const KTask& t, int vb, unsigned char* smem_raw, const int*) {
    const ConvP& p = t.p.conv;
    float* out = (float*)t.a[0];
    const float* in = (const float*)t.a[1];
    const float* bias = (const float*)t.a[2];
    const int kp = p.ocs, kp4 = kp >> 2;
    const int total = p.ptot * kp4;
    // per column k: offset of its tap inside the input plane stack, the tap's (dy, dx), the channel's bias — the
    // divisions that take k apart are done once per block here, not once per element
    int* s_off = reinterpret_cast<int*>(smem_raw);            // (ch * hi + ky) * wi + kx, or -1 beyond K
    int* s_dyx = s_off + kp;                                   // ky << 16 | kx
    float* s_bias = reinterpret_cast<float*>(s_dyx + kp);
    __syncthreads();   // a persistent caller may still be reading the previous logical block's table
    for (int k = threadIdx.x; k < kp; k += kThreads) {
        int off = -1, dyx = 0;
        float b = 0.f;
        if (k < p.ktot) {
            const int tap = k / p.ci, ch = k - tap * p.ci;
            const int ky = tap / p.kw, kx = tap - ky * p.kw;
            off = (ch * p.hi + ky) * p.wi + kx;
            dyx = (ky << 16) | kx;
            b = bias[ch];
        }
        s_off[k] = off;
        s_dyx[k] = dyx;
        s_bias[k] = b;
    }
    __syncthreads();
#pragma unroll 1
    for (int it = 0; it < kIm2colPerBlock / kThreads; it++) {
        const int item = vb * kIm2colPerBlock + it * kThreads + (int)threadIdx.x;
        if (item >= total) break;
        const int pix = item / kp4, q = item - pix * kp4;
        const int oy = pix / p.wo, ox = pix - oy * p.wo;
        const int y0 = oy * p.sh - p.ph, x0 = ox * p.sw - p.pw;
        const int base = y0 * p.wi + x0;
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int k = q * 4 + e;
            const int off = s_off[k], dyx = s_dyx[k];
            const int iy = y0 + (dyx >> 16), ix = x0 + (dyx & 0xffff);
            float x = 0.f;
            if (off >= 0 && iy >= 0 && iy < p.hi && ix >= 0 && ix < p.wi) x = __ldg(in + base + off) + s_bias[k];
            uint32_t u;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
            v[e] = __uint_as_float(u);
        }
        *reinterpret_cast<float4*>(out + (size_t)item * 4) = make_float4(v[0], v[1], v[2], v[3]);
    }
    return true;
}

// ---- fused_add_nn_relu, channels-last (reference: resource/resnet152/resnet152.cu:4056-4066) ---
// args: out, in, bias.  out[p][c] = max(in[p*ics+ioff+c] + bias[c], 0); c, ics, ioff multiples of 4.
__device__ __forceinline__ bool body_bias_relu(const KTask& t, int vb, unsigned char*, const int*) {
    const EltP& p = t.p.elt;
    float* out = (float*)t.a[0];
    const float* in = (const float*)t.a[1];
    const float* bias = (const float*)t.a[2];
    const int c4 = p.c >> 2;
    const int total4 = p.n * c4;
    int base = vb * (kEltPerBlock / 4) + threadIdx.x;
#pragma unroll
    for (int it = 0; it < kEltPerBlock / (kThreads * 4); it++) {
        int i = base + it * kThreads;
        if (i < total4) {
            int pix = i / c4, cc = (i - pix * c4) << 2;
            float4 v = *reinterpret_cast<const float4*>(in + (size_t)pix * p.ics + p.ioff + cc);
            float4 b = *reinterpret_cast<const float4*>(bias + cc);
            v.x = fmaxf(v.x + b.x, 0.f); v.y = fmaxf(v.y + b.y, 0.f);
            v.z = fmaxf(v.z + b.z, 0.f); v.w = fmaxf(v.w + b.w, 0.f);
            *reinterpret_cast<float4*>(out + (size_t)pix * p.c + cc) = v;
        }
    }
    return true;
}

// ---- batch_flatten: copy (reference: resource/resnet152/resnet152.cu:4472-4474) ----------------
// args: out, in.
__device__ __forceinline__ bool body_copy(const KTask& t, int vb, unsigned char*, const int*) {
    const int n = t.p.elt.n;
    float* out = (float*)t.a[0];
    const float* in = (const float*)t.a[1];
    int base = vb * kEltPerBlock + threadIdx.x * 4;
#pragma unroll
    for (int it = 0; it < kEltPerBlock / (kThreads * 4); it++) {
        int i = base + it * kThreads * 4;
        if (i + 3 < n) {
            *reinterpret_cast<float4*>(out + i) = *reinterpret_cast<const float4*>(in + i);
        } else {
            for (int j = 0; j < 4; j++)
                if (i + j < n) out[i + j] = in[i + j];
        }
    }
    return true;
}

// ---- pooling, channels-last ---------------------------------------------------------------------
// max: pad value -3.402823e38, optional +bias, ReLU (reference: resource/resnet152/resnet152.cu:365-374)
// avg: count-include-pad multiplies by 1/k^2 (reference: resource/inception/inception.cu:578-587)
// args: in, out[, bias].  One thread = 4 channels of one output pixel; vblock = 256 such items.
constexpr int kPoolItemsPerBlock = kThreads;
template <bool MAX>
__device__ __forceinline__ bool body_pool(const KTask& t, int vb, unsigned char*, const int*) {
    const PoolP& p = t.p.pool;
    const float* in = (const float*)t.a[0];
    float* out = (float*)t.a[1];
    const float* bias = p.has_bias ? (const float*)t.a[2] : nullptr;
    const int c4 = p.c >> 2;
    const int total = p.ho * p.wo * c4;
#pragma unroll 1
    for (int it = 0; it < kPoolItemsPerBlock / kThreads; it++) {
        int i = vb * kPoolItemsPerBlock + it * kThreads + threadIdx.x;
        if (i >= total) break;
        int pix = i / c4, cc = (i - pix * c4) << 2;
        int oy = pix / p.wo, ox = pix - oy * p.wo;
        float4 acc = MAX ? make_float4(-3.402823e38f, -3.402823e38f, -3.402823e38f, -3.402823e38f)
                         : make_float4(0.f, 0.f, 0.f, 0.f);
        int cnt = 0;
        for (int ky = 0; ky < p.k; ky++) {
            int iy = oy * p.s + ky - p.p;
            if (iy < 0 || iy >= p.hi) continue;
            for (int kx = 0; kx < p.k; kx++) {
                int ix = ox * p.s + kx - p.p;
                if (ix < 0 || ix >= p.wi) continue;
                float4 v = *reinterpret_cast<const float4*>(in + ((size_t)iy * p.wi + ix) * p.ics + p.ioff + cc);
                if (MAX) {
                    acc.x = fmaxf(acc.x, v.x); acc.y = fmaxf(acc.y, v.y);
                    acc.z = fmaxf(acc.z, v.z); acc.w = fmaxf(acc.w, v.w);
                } else {
                    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                }
                cnt++;
            }
        }
        if (MAX) {
            if (bias) {
                float4 b = *reinterpret_cast<const float4*>(bias + cc);
                acc.x = fmaxf(acc.x + b.x, 0.f); acc.y = fmaxf(acc.y + b.y, 0.f);
                acc.z = fmaxf(acc.z + b.z, 0.f); acc.w = fmaxf(acc.w + b.w, 0.f);
            }
        } else {
            float sc = p.cip ? 1.0f / (float)(p.k * p.k) : 1.0f / (float)(cnt > 0 ? cnt : 1);
            acc.x *= sc; acc.y *= sc; acc.z *= sc; acc.w *= sc;
        }
        *reinterpret_cast<float4*>(out + (size_t)pix * p.ocs + p.ooff + cc) = acc;
    }
    return true;
}

// ---- global average pool (reference: resource/resnet152/resnet152.cu:4390-4403) ----------------
// args: in [hw][c], out [c].  vblock = 32 channels; 8 warps split the hw range, lanes = channels.
__device__ __forceinline__ bool body_gap(const KTask& t, int vb, unsigned char* smem, const int*) {
    const int c = t.p.elt.c, hw = t.p.elt.n;
    const float* in = (const float*)t.a[0];
    float* out = (float*)t.a[1];
    float* red = reinterpret_cast<float*>(smem);   // [8][32]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ch = vb * 32 + lane;
    float s = 0.f;
    if (ch < c)
        for (int p = warp; p < hw; p += 8) s += in[(size_t)p * c + ch];
    red[warp * 32 + lane] = s;
    __syncthreads();
    if (warp == 0 && ch < c) {
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) tot += red[w * 32 + lane];   // fixed order: deterministic
        out[ch] = tot * (1.0f / (float)hw);
    }
    __syncthreads();
    return true;
}

// ---- dense_add[_nn_relu] : GEMV at batch 1 (reference: resource/resnet152/resnet152.cu:2-33) ---
// args: x[k], W[n][k], out[n], bias[n].  HBM-bound: every weight byte is read exactly once, and what decides the
// speed is how the reads look to the DRAM: thousands of short interleaved row streams (a warp or a block hopping
// between many weight rows) reach 0.55-0.6 of the HBM rate whether they are issued as plain loads or by the copy
// engine; a few hundred long sequential streams reach it.  So:
//  * the rows are dealt out in equal shares to 296 logical blocks (two per SM on B200): block b owns the contiguous
//    rows [b*n/B, (b+1)*n/B), at most 16, and walks them four at a time from end to end, i.e. each block reads four
//    sequential streams in 8 KB pieces;
//  * the pieces are fetched by the copy engine (cp.async.bulk, no tensor map: a row is contiguous) into a ring of
//    three 32 KB shared-memory stages, completion on mbarriers, so that ~96 KB per block are in flight without
//    tying up registers;
//  * thread t owns eight K positions of every stage: two 128-bit loads of x, two 128-bit shared-memory reads per
//    row, 32 FMAs.  The partial sums of the 8 warps meet in shared memory in a fixed order.
// Best-effort flavour: thread 0 polls the preempt flag before it refills a stage (once per 32 KB of weights); it
// then stops issuing copies and publishes how far it got; every thread waits out what is in flight (its barriers
// must have completed before the block may leave) and the block exits uncounted.  Waits are bounded.
constexpr int kDenseBlocks = 296;
constexpr int kDenseMaxRows = 16;
// Measured on VGG-16's 411 MB layer (rows together, bytes per piece, stages -> fraction of the measured HBM copy rate):
// 4 x 4 KB x 6: 0.68 | 2 x 8 KB x 6: 0.92 | 4 x 8 KB x 3: 0.91 | 2 x 4 KB x 12: 0.56 | 1 x 16 KB x 6: 0.86.
// The piece size decides; 4 rows x 8 KB x 3 stages is also the fastest on the small layers.
#ifndef REEF_DENSE_RG
#define REEF_DENSE_RG 4
#define REEF_DENSE_KC 2048
#define REEF_DENSE_NS 3
#endif
constexpr int kDenseRG = REEF_DENSE_RG;         // rows walked together
constexpr int kDenseKC = REEF_DENSE_KC;         // K positions per stage and row (8 KB pieces)
constexpr int kDenseStages = REEF_DENSE_NS;
constexpr int kDenseVec = kDenseKC / 1024;      // 128-bit slices of a stage row per thread
constexpr int kDenseStageFloats = kDenseRG * kDenseKC;
// ring + partial sums [4 groups][8 warps][4 rows] + alignment slack, barriers, control words
constexpr int kDenseSmem = kDenseStages * kDenseStageFloats * 4 + (kDenseMaxRows / kDenseRG) * 8 * kDenseRG * 4 + 512;
__host__ __device__ inline int dense_num_blocks(int n) {
    int b = n < kDenseBlocks ? n : kDenseBlocks;
    while ((n + b - 1) / b > kDenseMaxRows) b++;     // never more than kDenseMaxRows rows in a block
    return b;
}
__device__ __forceinline__ bool dense_mbar_wait(uint32_t bar, uint32_t parity) {
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
// The consumers' wait in the best-effort flavour: 0 = the stage landed, 1 = the wait expired, 2 = the producer stopped
// before it issued this stage (ctl[0] set and st >= ctl[1]).  A warp that runs ahead of the producer can already be
// waiting for a stage when the producer sees the preempt flag and decides never to issue it: the stop has to be looked
// at inside the wait, or that warp sits out the whole time limit.
__device__ __forceinline__ int dense_mbar_wait_abortable(uint32_t bar, uint32_t parity, const volatile int* ctl, int st) {
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
        if (ctl[0] && st >= ctl[1]) return 2;
        if ((i & 255) == 255) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (t0 == 0) t0 = t;
            else if (t - t0 > 1000000000ull) return 1;
        }
    }
    return 1;
}
__device__ __forceinline__ bool body_dense(const KTask& t, int vb, unsigned char* smem_raw, const int* flag) {
    const DenseP& p = t.p.dense;
    const float* x = (const float*)t.a[0];
    const float* w = (const float*)t.a[1];
    float* out = (float*)t.a[2];
    const float* bias = (const float*)t.a[3];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int B = t.nblocks;
    const int r0 = (int)(((long long)vb * p.n) / B), r1 = (int)(((long long)(vb + 1) * p.n) / B);
    const int nr = r1 - r0;
    const int ngroups = (nr + kDenseRG - 1) / kDenseRG;
    // dynamic shared memory: ring | partial sums | barriers (8-byte aligned) | control words
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t ring_off = ((sbase + 127u) & ~127u) - sbase;
    float* ring = reinterpret_cast<float*>(smem_raw + ring_off);
    constexpr int kPartFloats = (kDenseMaxRows / kDenseRG) * 8 * kDenseRG;
    float* part = ring + kDenseStages * kDenseStageFloats;                 // [group][warp][row in group]
    const uint32_t bars = sbase + ring_off + (kDenseStages * kDenseStageFloats + kPartFloats) * 4;
    volatile int* ctl = reinterpret_cast<volatile int*>(smem_raw + ring_off + (kDenseStages * kDenseStageFloats + kPartFloats) * 4 + 16 * kDenseStages);
    // ctl[0] = stop requested, ctl[1] = stages issued when the producer stopped, ctl[2] = a wait expired
    int stopped = 0;
    if ((p.k & 3) == 0) {
        const int spg = (p.k + kDenseKC - 1) / kDenseKC;     // stages per row group
        const int nst = ngroups * spg;                        // stages to stream
        const uint32_t bar_full = bars, bar_empty = bars + 8 * kDenseStages;
        if (tid == 0) {
            for (int s = 0; s < kDenseStages; s++) {
                asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_full + 8 * s), "r"(1));
                asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_empty + 8 * s), "r"(8));   // one arrive per warp
            }
            ctl[0] = 0; ctl[1] = 0; ctl[2] = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncthreads();
        // one stage = the next 4 KB of each row of a group: lanes 0..3 of warp 0 copy a row's piece each, lane 0
        // arms the barrier with the byte count
        auto issue = [&](int st) {
            const int s = st % kDenseStages;
            const int g = st / spg, k0 = (st - g * spg) * kDenseKC;
            const int kc = min(kDenseKC, p.k - k0);
            const int rows = min(kDenseRG, nr - g * kDenseRG);
            if (lane == 0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_full + 8 * s), "r"((uint32_t)(rows * kc * 4)) : "memory");
            __syncwarp();
            if (lane < rows) {
                const uint32_t dst = sbase + ring_off + (uint32_t)((s * kDenseStageFloats + lane * kDenseKC) * 4);
                const float* src = w + (size_t)(r0 + g * kDenseRG + lane) * p.k + k0;
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(dst), "l"(src), "r"((uint32_t)(kc * 4)), "r"(bar_full + 8 * s)
                             : "memory");
            }
        };
        const int first = nst < kDenseStages ? nst : kDenseStages;
        if (warp == 0)
            for (int st = 0; st < first; st++) issue(st);
        int issued = first;        // meaningful in warp 0 only
        bool ok = true;
        float acc[kDenseRG];
        int st = 0;
        for (int g = 0; g < ngroups && ok && !stopped; g++) {
            const int rows = min(kDenseRG, nr - g * kDenseRG);
#pragma unroll
            for (int r = 0; r < kDenseRG; r++) acc[r] = 0.f;
            for (int kq = 0; kq < spg; kq++, st++) {
                const int s = st % kDenseStages;
                const uint32_t par = (uint32_t)((st / kDenseStages) & 1);
                const int k0 = kq * kDenseKC;
                const int kc = min(kDenseKC, p.k - k0);
                float4 xv[kDenseVec];
#pragma unroll
                for (int j = 0; j < kDenseVec; j++) {       // requested before the wait
                    xv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if ((tid + j * kThreads) * 4 < kc) xv[j] = __ldg(reinterpret_cast<const float4*>(x + k0) + tid + j * kThreads);
                }
                if (flag != nullptr) {
                    const int w = dense_mbar_wait_abortable(bar_full + 8 * s, par, ctl, st);
                    if (w == 2) {          // the producer stopped before this stage: nothing of it is in flight
                        stopped = 1;
                        break;
                    }
                    if (w == 1) {
                        ok = false;
                        break;
                    }
                } else if (!dense_mbar_wait(bar_full + 8 * s, par)) {
                    ok = false;
                    break;
                }
                if (!(flag != nullptr && ctl[0])) {
                    const float4* sw = reinterpret_cast<const float4*>(ring + (size_t)s * kDenseStageFloats) + tid;
#pragma unroll
                    for (int j = 0; j < kDenseVec; j++) {
                        if ((tid + j * kThreads) * 4 < kc) {
#pragma unroll
                            for (int r = 0; r < kDenseRG; r++) {
                                if (r < rows) {
                                    const float4 wv = sw[r * (kDenseKC / 4) + j * kThreads];
                                    acc[r] = fmaf(wv.x, xv[j].x, acc[r]); acc[r] = fmaf(wv.y, xv[j].y, acc[r]);
                                    acc[r] = fmaf(wv.z, xv[j].z, acc[r]); acc[r] = fmaf(wv.w, xv[j].w, acc[r]);
                                }
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_empty + 8 * s) : "memory");
                // refill this stage with the piece kDenseStages ahead, once every warp has released it
                if (warp == 0 && st + kDenseStages < nst && !(flag != nullptr && ctl[0])) {
                    int go = 1;
                    if (lane == 0) {
                        if (flag != nullptr && ld_flag(flag)) {              // loop-head poll of the preempt flag
                            ctl[1] = issued;                                 // first how far the copies got, then the request
                            __threadfence_block();
                            ctl[0] = 1;
                            go = 0;
                        } else if (!dense_mbar_wait(bar_empty + 8 * s, par)) {
                            ctl[2] = 1;
                            go = 0;
                        }
                    }
                    go = __shfl_sync(0xffffffffu, go, 0);
                    if (go) {
                        issue(st + kDenseStages);
                        issued = st + kDenseStages + 1;
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < kDenseRG; r++) {
                const float v = warp_sum(acc[r]);
                if (lane == 0) part[(g * 8 + warp) * kDenseRG + r] = v;
            }
        }
        if (!ok || ctl[2]) {   // a wait expired: nothing is stored, the block is counted incomplete, the error word is raised
            stopped = 1;
            if (t.err != nullptr && tid == 0) *reinterpret_cast<volatile int*>(t.err) = 1;
        }
        if (flag != nullptr && ctl[0]) stopped = 1;
    } else {
        // K not a multiple of 4 (no 16-byte alignment for the copy engine): plain loads
        for (int g = 0; g < ngroups; g++) {
            float acc[kDenseRG];
#pragma unroll
            for (int r = 0; r < kDenseRG; r++) acc[r] = 0.f;
            const int rows = min(kDenseRG, nr - g * kDenseRG);
            for (int i = tid; i < p.k; i += kThreads) {
                const float xv = x[i];
#pragma unroll
                for (int r = 0; r < kDenseRG; r++)
                    if (r < rows) acc[r] = fmaf(w[(size_t)(r0 + g * kDenseRG + r) * p.k + i], xv, acc[r]);
            }
#pragma unroll
            for (int r = 0; r < kDenseRG; r++) {
                const float v = warp_sum(acc[r]);
                if (lane == 0) part[(g * 8 + warp) * kDenseRG + r] = v;
            }
        }
    }
    if (__syncthreads_or(stopped)) return false;     // every thread of the block takes the same exit
    if (tid < nr) {
        const int g = tid / kDenseRG, j = tid - g * kDenseRG;
        float v = 0.f;
#pragma unroll
        for (int q = 0; q < 8; q++) v += part[(g * 8 + q) * kDenseRG + j];   // fixed order: deterministic
        v += bias[r0 + tid];
        if (p.relu) v = fmaxf(v, 0.f);
        out[r0 + tid] = v;
    }
    __syncthreads();   // shared memory may be reused by the next logical block of a persistent caller
    return true;
}

// ---- softmax over n values (reference: resource/resnet152/resnet152.cu:775-841) ----------------
// args: in, out.  One vblock per row; max-subtract, expf, sum, divide.
__device__ __forceinline__ bool body_softmax(const KTask& t, int vb, unsigned char* smem, const int*) {
    const int n = t.p.softmax.n;
    const float* in = (const float*)t.a[0] + (size_t)vb * n;
    float* out = (float*)t.a[1] + (size_t)vb * n;
    float* red = reinterpret_cast<float*>(smem);   // [8] + [8]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float m = -3.402823e38f;
    for (int i = threadIdx.x; i < n; i += kThreads) m = fmaxf(m, in[i]);
    m = warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < 8; w++) m = fmaxf(m, red[w]);
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += kThreads) s += expf(in[i] - m);
    s = warp_sum(s);
    if (lane == 0) red[8 + warp] = s;
    __syncthreads();
    s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) s += red[8 + w];
    for (int i = threadIdx.x; i < n; i += kThreads) out[i] = expf(in[i] - m) / s;
    __syncthreads();
    return true;
}

}  // namespace reef
