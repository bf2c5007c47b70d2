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
// One logical block = one head x 16 query rows (S = 128: 96 blocks); a warp owns 2 rows and works on both at
// once, so every shared-memory operand feeds two multiply-adds.  Keys/values are staged through shared memory
// 64 at a time (128-bit global loads); for the scores a lane owns two keys, for P*V two output dimensions.
constexpr int kAttRows = 16;
constexpr int kAttChunk = 64;
constexpr int kAttD = 64;
constexpr int kAttSmem = (2 * kAttChunk * (kAttD + 1) + 8 * 2 * kAttD + 8 * 2 * kAttChunk) * 4;   // 41.3 KB
__device__ __forceinline__ bool body_attention(const KTask& t, int vb, unsigned char* smem_raw, const int* flag) {
    const int S = t.p.raw[0], heads = t.p.raw[1], has_mask = t.p.raw[3];
    const int H = heads * kAttD;
    const float* qkv = (const float*)t.a[0];
    const float* mask = has_mask ? (const float*)t.a[1] : nullptr;
    float* out = (float*)t.a[has_mask ? 2 : 1];
    float* Ks = reinterpret_cast<float*>(smem_raw);            // [64][65]
    float* Vs = Ks + kAttChunk * (kAttD + 1);                  // [64][65]
    float* Qs = Vs + kAttChunk * (kAttD + 1);                  // [8 warps][2 rows][64]
    float* Ps = Qs + 8 * 2 * kAttD;                            // [8 warps][2 rows][64]: probabilities of the rows in work
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rblocks = (S + kAttRows - 1) / kAttRows;
    const int head = vb / rblocks, r0 = (vb - head * rblocks) * kAttRows + warp * 2;
    const float scale = rsqrtf((float)kAttD);
    const float ninf = -__int_as_float(0x7f800000);
    // this warp's 2 query rows -> shared (read back as 128-bit broadcasts)
    for (int r = 0; r < 2; r++) {
        const int row = r0 + r;
        for (int c = lane; c < kAttD; c += 32)
            Qs[(warp * 2 + r) * kAttD + c] = row < S ? qkv[(size_t)row * 3 * H + head * kAttD + c] : 0.f;
    }
    float m[2], l[2], acc[2][2];
#pragma unroll
    for (int r = 0; r < 2; r++) { m[r] = ninf; l[r] = 0.f; acc[r][0] = acc[r][1] = 0.f; }

    for (int k0 = 0; k0 < S; k0 += kAttChunk) {
        // the barrier says the previous chunk is fully consumed; in the best-effort flavour it also carries the
        // loop-head poll of the preempt flag (an OR over the block, so that all threads take the same exit)
        if (flag != nullptr) {
            if (__syncthreads_or(ld_flag(flag))) return false;
        } else {
            __syncthreads();
        }
        for (int i = threadIdx.x; i < kAttChunk * (kAttD / 4); i += kThreads) {
            const int j = i / (kAttD / 4), c = (i - j * (kAttD / 4)) * 4, key = k0 + j;
            float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
            if (key < S) {
                kv = *reinterpret_cast<const float4*>(qkv + (size_t)key * 3 * H + H + head * kAttD + c);
                vv = *reinterpret_cast<const float4*>(qkv + (size_t)key * 3 * H + 2 * H + head * kAttD + c);
            }
            float* kd = Ks + j * (kAttD + 1) + c;
            float* vd = Vs + j * (kAttD + 1) + c;
            kd[0] = kv.x; kd[1] = kv.y; kd[2] = kv.z; kd[3] = kv.w;
            vd[0] = vv.x; vd[1] = vv.y; vd[2] = vv.z; vd[3] = vv.w;
        }
        __syncthreads();
        // scores of both rows against keys lane and 32 + lane
        const float4* qa = reinterpret_cast<const float4*>(Qs + (warp * 2 + 0) * kAttD);
        const float4* qb = reinterpret_cast<const float4*>(Qs + (warp * 2 + 1) * kAttD);
        const float* ka = Ks + lane * (kAttD + 1);
        const float* kb = Ks + (32 + lane) * (kAttD + 1);
        float s00 = 0.f, s01 = 0.f, s10 = 0.f, s11 = 0.f;    // s[row][key group]
#pragma unroll 4
        for (int c4 = 0; c4 < kAttD / 4; c4++) {
            const float4 a = qa[c4], b = qb[c4];
            const float x0 = ka[4 * c4], x1 = ka[4 * c4 + 1], x2 = ka[4 * c4 + 2], x3 = ka[4 * c4 + 3];
            const float y0 = kb[4 * c4], y1 = kb[4 * c4 + 1], y2 = kb[4 * c4 + 2], y3 = kb[4 * c4 + 3];
            s00 = fmaf(a.x, x0, s00); s00 = fmaf(a.y, x1, s00); s00 = fmaf(a.z, x2, s00); s00 = fmaf(a.w, x3, s00);
            s01 = fmaf(a.x, y0, s01); s01 = fmaf(a.y, y1, s01); s01 = fmaf(a.z, y2, s01); s01 = fmaf(a.w, y3, s01);
            s10 = fmaf(b.x, x0, s10); s10 = fmaf(b.y, x1, s10); s10 = fmaf(b.z, x2, s10); s10 = fmaf(b.w, x3, s10);
            s11 = fmaf(b.x, y0, s11); s11 = fmaf(b.y, y1, s11); s11 = fmaf(b.z, y2, s11); s11 = fmaf(b.w, y3, s11);
        }
        const bool dead0 = (k0 + lane >= S) || (mask && mask[min(k0 + lane, S - 1)] == 0.f);
        const bool dead1 = (k0 + 32 + lane >= S) || (mask && mask[min(k0 + 32 + lane, S - 1)] == 0.f);
        float sc[2][2] = {{dead0 ? ninf : s00 * scale, dead1 ? ninf : s01 * scale},
                          {dead0 ? ninf : s10 * scale, dead1 ? ninf : s11 * scale}};
        float corr[2];
        float* pr = Ps + warp * 2 * kAttChunk;
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const float cmax = warp_max(fmaxf(sc[r][0], sc[r][1]));
            const float mnew = fmaxf(m[r], cmax);
            corr[r] = (mnew == ninf) ? 1.f : expf(m[r] - mnew);
            const float p0 = (sc[r][0] == ninf) ? 0.f : expf(sc[r][0] - mnew);
            const float p1 = (sc[r][1] == ninf) ? 0.f : expf(sc[r][1] - mnew);
            l[r] = l[r] * corr[r] + warp_sum(p0 + p1);
            m[r] = mnew;
            pr[r * kAttChunk + lane] = p0;
            pr[r * kAttChunk + 32 + lane] = p1;
        }
        __syncwarp();
        float a00 = acc[0][0] * corr[0], a01 = acc[0][1] * corr[0], a10 = acc[1][0] * corr[1], a11 = acc[1][1] * corr[1];
        const float4* pa = reinterpret_cast<const float4*>(pr);
        const float4* pb = reinterpret_cast<const float4*>(pr + kAttChunk);
#pragma unroll 4
        for (int j4 = 0; j4 < kAttChunk / 4; j4++) {
            const float4 u = pa[j4], w = pb[j4];
            const float* v = Vs + (4 * j4) * (kAttD + 1) + lane;
            const float v00 = v[0], v01 = v[32], v10 = v[kAttD + 1], v11 = v[kAttD + 1 + 32];
            const float v20 = v[2 * (kAttD + 1)], v21 = v[2 * (kAttD + 1) + 32], v30 = v[3 * (kAttD + 1)], v31 = v[3 * (kAttD + 1) + 32];
            a00 = fmaf(u.x, v00, a00); a00 = fmaf(u.y, v10, a00); a00 = fmaf(u.z, v20, a00); a00 = fmaf(u.w, v30, a00);
            a01 = fmaf(u.x, v01, a01); a01 = fmaf(u.y, v11, a01); a01 = fmaf(u.z, v21, a01); a01 = fmaf(u.w, v31, a01);
            a10 = fmaf(w.x, v00, a10); a10 = fmaf(w.y, v10, a10); a10 = fmaf(w.z, v20, a10); a10 = fmaf(w.w, v30, a10);
            a11 = fmaf(w.x, v01, a11); a11 = fmaf(w.y, v11, a11); a11 = fmaf(w.z, v21, a11); a11 = fmaf(w.w, v31, a11);
        }
        acc[0][0] = a00; acc[0][1] = a01; acc[1][0] = a10; acc[1][1] = a11;
        __syncwarp();
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
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
