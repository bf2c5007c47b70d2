// BERT families: embedding gather, LayerNorm (with optional residual add) and multi-head attention.
// The reference's TVM build spreads these over dozens of small kernels per layer — four softmax passes
// through an HBM scratch buffer, five LayerNorm launches, head split/merge transposes, a Q/sqrt(d) divide
// (reference: resource/bert/bert.cu:3-12,159-204,273-395).  Here each is one kernel; the dense projections
// run on the tensor-core GEMM with bias / GELU / residual fused in its epilogue (conv_tc.cuh).
#pragma once
#include "simple.cuh"

namespace reef {

// ---- embedding: out[s][h] = word[clamp(ids[s], 0, vocab-1)][h] + pos[s][h]  (reference: bert.cu:313-325) -----
// args: out, word_emb, ids (int64), pos_emb.  One thread = 4 channels of one token.
__device__ __forceinline__ bool body_embedding(const KTask& t, int vb, unsigned char*, const int*) {
    const int s = t.p.raw[0], h = t.p.raw[1], vocab = t.p.raw[2];
    float* out = (float*)t.a[0];
    const float* word = (const float*)t.a[1];
    const long long* ids = (const long long*)t.a[2];
    const float* pos = (const float*)t.a[3];
    const int h4 = h >> 2, total = s * h4;
#pragma unroll
    for (int it = 0; it < 4; it++) {
        const int i = vb * (kThreads * 4) + it * kThreads + threadIdx.x;
        if (i >= total) break;
        const int tok = i / h4, c = (i - tok * h4) << 2;
        long long id = ids[tok];
        id = id < 0 ? 0 : (id > vocab - 1 ? vocab - 1 : id);
        const float4 w = *reinterpret_cast<const float4*>(word + (size_t)id * h + c);
        const float4 p = *reinterpret_cast<const float4*>(pos + (size_t)tok * h + c);
        *reinterpret_cast<float4*>(out + (size_t)tok * h + c) = make_float4(w.x + p.x, w.y + p.y, w.z + p.z, w.w + p.w);
    }
    return true;
}

// ---- LayerNorm of x (+ residual): mean, two-pass variance, (x-mu)/sqrt(var+1e-12)*gamma+beta ------------------
// (reference: bert.cu:175-204,338-342,352-379; eps at :201).  args: out, x, [residual], gamma, beta.
// One warp per row, the row lives in registers (h <= 1024, h % 128 == 0), warp-shuffle reductions.
constexpr int kLnRowsPerBlock = 8;
__device__ __forceinline__ bool body_layernorm(const KTask& t, int vb, unsigned char*, const int*) {
    const int rows = t.p.raw[0], h = t.p.raw[1], has_res = t.p.raw[2];
    float* out = (float*)t.a[0];
    const float* x = (const float*)t.a[1];
    const float* res = has_res ? (const float*)t.a[2] : nullptr;
    const float* gamma = (const float*)t.a[has_res ? 3 : 2];
    const float* beta = (const float*)t.a[has_res ? 4 : 3];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = vb * kLnRowsPerBlock + warp;
    if (row >= rows) return true;
    const int n4 = h >> 7;   // float4 per lane
    float4 v[8];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        if (i < n4) {
            const int c = (i * 32 + lane) * 4;
            v[i] = *reinterpret_cast<const float4*>(x + (size_t)row * h + c);
            if (res) {
                const float4 r = *reinterpret_cast<const float4*>(res + (size_t)row * h + c);
                v[i].x += r.x; v[i].y += r.y; v[i].z += r.z; v[i].w += r.w;
            }
            sum += v[i].x + v[i].y + v[i].z + v[i].w;
        }
    }
    const float mu = warp_sum(sum) / (float)h;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        if (i < n4) {
            const float a = v[i].x - mu, b = v[i].y - mu, c = v[i].z - mu, d = v[i].w - mu;
            sq += a * a + b * b + c * c + d * d;
        }
    }
    const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)h + 1e-12f);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        if (i < n4) {
            const int c = (i * 32 + lane) * 4;
            const float4 g = *reinterpret_cast<const float4*>(gamma + c);
            const float4 b = *reinterpret_cast<const float4*>(beta + c);
            float4 o;
            o.x = (v[i].x - mu) * rstd * g.x + b.x;
            o.y = (v[i].y - mu) * rstd * g.y + b.y;
            o.z = (v[i].z - mu) * rstd * g.z + b.z;
            o.w = (v[i].w - mu) * rstd * g.w + b.w;
            *reinterpret_cast<float4*>(out + (size_t)row * h + c) = o;
        }
    }
    return true;
}

// ---- multi-head self-attention on a fused [S][3H] buffer (Q | K | V, head-major inside each H) ----------------
// scores = Q K^T / sqrt(d); mask[j] == 0 -> -inf; row softmax (max-subtracted, online over key chunks);
// ctx = P V   (reference: bert.cu:22-157 batch_matmul_4/5, :289-311 divide + transposes, :381-387 where,
// softmax :3-12,159-165,327-336,389-395).  args: qkv, [mask], out.  d == 64.
// One logical block = one head x 32 query rows; a warp owns 4 rows; keys/values are staged through shared
// memory 64 at a time; for the scores a lane owns a key, for P*V a lane owns two output dimensions.
constexpr int kAttRows = 32;
constexpr int kAttChunk = 64;
constexpr int kAttD = 64;
constexpr int kAttSmem = (2 * kAttChunk * (kAttD + 1) + 8 * 4 * kAttD + 8 * kAttChunk) * 4;   // 43.5 KB: under the 48 KB default limit
__device__ __forceinline__ bool body_attention(const KTask& t, int vb, unsigned char* smem_raw, const int*) {
    const int S = t.p.raw[0], heads = t.p.raw[1], has_mask = t.p.raw[3];
    const int H = heads * kAttD;
    const float* qkv = (const float*)t.a[0];
    const float* mask = has_mask ? (const float*)t.a[1] : nullptr;
    float* out = (float*)t.a[has_mask ? 2 : 1];
    float* Ks = reinterpret_cast<float*>(smem_raw);            // [64][65]
    float* Vs = Ks + kAttChunk * (kAttD + 1);                  // [64][65]
    float* Qs = Vs + kAttChunk * (kAttD + 1);                  // [8 warps][4 rows][64]
    float* Ps = Qs + 8 * 4 * kAttD;                            // [8 warps][64]: probabilities of the row in work
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rblocks = (S + kAttRows - 1) / kAttRows;
    const int head = vb / rblocks, r0 = (vb - head * rblocks) * kAttRows + warp * 4;
    const float scale = rsqrtf((float)kAttD);
    // this warp's 4 query rows -> shared (read back as broadcasts)
    for (int r = 0; r < 4; r++) {
        const int row = r0 + r;
        for (int c = lane; c < kAttD; c += 32)
            Qs[(warp * 4 + r) * kAttD + c] = row < S ? qkv[(size_t)row * 3 * H + head * kAttD + c] : 0.f;
    }
    float m[4], l[4], acc[4][2];
#pragma unroll
    for (int r = 0; r < 4; r++) { m[r] = -__int_as_float(0x7f800000); l[r] = 0.f; acc[r][0] = acc[r][1] = 0.f; }

    for (int k0 = 0; k0 < S; k0 += kAttChunk) {
        __syncthreads();   // previous chunk fully consumed
        for (int i = threadIdx.x; i < kAttChunk * kAttD; i += kThreads) {
            const int j = i / kAttD, c = i - j * kAttD, key = k0 + j;
            Ks[j * (kAttD + 1) + c] = key < S ? qkv[(size_t)key * 3 * H + H + head * kAttD + c] : 0.f;
            Vs[j * (kAttD + 1) + c] = key < S ? qkv[(size_t)key * 3 * H + 2 * H + head * kAttD + c] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const float* q = Qs + (warp * 4 + r) * kAttD;
            float sc[2];
#pragma unroll
            for (int g = 0; g < 2; g++) {
                const int j = g * 32 + lane, key = k0 + j;
                float a = 0.f;
#pragma unroll 16
                for (int c = 0; c < kAttD; c++) a = fmaf(q[c], Ks[j * (kAttD + 1) + c], a);
                a *= scale;
                if (key >= S || (mask && mask[key] == 0.f)) a = -__int_as_float(0x7f800000);
                sc[g] = a;
            }
            const float cmax = warp_max(fmaxf(sc[0], sc[1]));
            const float mnew = fmaxf(m[r], cmax);
            const float corr = (mnew == -__int_as_float(0x7f800000)) ? 1.f : expf(m[r] - mnew);
            const float p0 = (sc[0] == -__int_as_float(0x7f800000)) ? 0.f : expf(sc[0] - mnew);
            const float p1 = (sc[1] == -__int_as_float(0x7f800000)) ? 0.f : expf(sc[1] - mnew);
            l[r] = l[r] * corr + warp_sum(p0 + p1);
            m[r] = mnew;
            float* pr = Ps + warp * kAttChunk;
            pr[lane] = p0;
            pr[32 + lane] = p1;
            __syncwarp();
            float a0 = acc[r][0] * corr, a1 = acc[r][1] * corr;
#pragma unroll 16
            for (int j = 0; j < kAttChunk; j++) {
                const float p = pr[j];
                a0 = fmaf(p, Vs[j * (kAttD + 1) + lane], a0);
                a1 = fmaf(p, Vs[j * (kAttD + 1) + 32 + lane], a1);
            }
            acc[r][0] = a0;
            acc[r][1] = a1;
            __syncwarp();
        }
    }
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const int row = r0 + r;
        if (row < S) {
            const float inv = 1.0f / l[r];
            out[(size_t)row * H + head * kAttD + lane] = acc[r][0] * inv;
            out[(size_t)row * H + head * kAttD + 32 + lane] = acc[r][1] * inv;
        }
    }
    __syncthreads();
    return true;
}

}  // namespace reef
