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
// args: x[k], W[n][k], out[n], bias[n].  HBM-bound: every weight byte is read exactly once (streaming loads).
// A warp owns TWO output rows (x is fetched once for both) and keeps 8 independent 128-bit weight loads in flight
// per lane: with VGG-16's 4096 rows only 1.7 blocks are resident per SM, so the bytes in flight per block, not the
// number of blocks, are what covers the HBM latency.  16 rows per logical block.
// Best-effort flavour: every warp polls the preempt flag at the head of every second pass of its main loop (a pass
// is 16 KB of weights per warp) and leaves; the wrapper counts the block complete only if no warp left.
constexpr int kDenseRowsPerBlock = 16;
__device__ __forceinline__ float dense_dot4(float4 a, float4 b, float acc) {
    acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc);
    acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
    return acc;
}
__device__ __forceinline__ bool body_dense(const KTask& t, int vb, unsigned char*, const int* flag) {
    const DenseP& p = t.p.dense;
    const float* x = (const float*)t.a[0];
    const float* w = (const float*)t.a[1];
    float* out = (float*)t.a[2];
    const float* bias = (const float*)t.a[3];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row0 = vb * kDenseRowsPerBlock + warp * 2;
    if (row0 >= p.n) return true;
    const bool two = row0 + 1 < p.n;
    const float* wr0 = w + (size_t)row0 * p.k;
    const float* wr1 = two ? wr0 + p.k : wr0;   // a last odd row is computed twice, stored once
    float acc0 = 0.f, acc1 = 0.f;
    if ((p.k & 3) == 0) {
        const float4* a4 = reinterpret_cast<const float4*>(wr0);
        const float4* b4 = reinterpret_cast<const float4*>(wr1);
        const float4* x4 = reinterpret_cast<const float4*>(x);
        const int k4 = p.k >> 2;
        int i = lane, pass = 0;
        for (; i + 96 < k4; i += 128, pass++) {
            if (flag != nullptr && (pass & 1) == 1 && ld_flag(flag)) return false;   // loop-head poll
            float4 wa[4], wb[4], xv[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                wa[u] = __ldcs(a4 + i + 32 * u);
                wb[u] = __ldcs(b4 + i + 32 * u);
            }
#pragma unroll
            for (int u = 0; u < 4; u++) xv[u] = __ldg(x4 + i + 32 * u);
#pragma unroll
            for (int u = 0; u < 4; u++) {
                acc0 = dense_dot4(wa[u], xv[u], acc0);
                acc1 = dense_dot4(wb[u], xv[u], acc1);
            }
        }
        for (; i < k4; i += 32) {
            const float4 xv = __ldg(x4 + i);
            acc0 = dense_dot4(__ldcs(a4 + i), xv, acc0);
            acc1 = dense_dot4(__ldcs(b4 + i), xv, acc1);
        }
    } else {
        for (int i = lane; i < p.k; i += 32) {
            acc0 = fmaf(wr0[i], x[i], acc0);
            acc1 = fmaf(wr1[i], x[i], acc1);
        }
    }
    acc0 = warp_sum(acc0);
    acc1 = warp_sum(acc1);
    if (lane == 0) {
        float v = acc0 + bias[row0];
        if (p.relu) v = fmaxf(v, 0.f);
        out[row0] = v;
        if (two) {
            v = acc1 + bias[row0 + 1];
            if (p.relu) v = fmaxf(v, 0.f);
            out[row0 + 1] = v;
        }
    }
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
