// conv2d family on CUDA cores: fp32 implicit GEMM, channels-last activations, OHWI weights.
//
//   out[y][x][co] = sum_{ky,kx,ci} in[y*sh+ky-ph][x*sw+kx-pw][ci] * W[co][ky][kx][ci]   (zero pad)
//   then (+residual[y][x][co]) (+bias[co] | *gamma[co]+beta[co]) (ReLU)
// (reference: resource/resnet152/resnet152.cu:315-363,3393-3418; args in, W, out, [residual], [bias | gamma, beta]).
//
// GEMM view: M = pixels (ho*wo), N = co, K = kh*kw*ci with ci fastest, so a 16-wide K slice is
// one contiguous 64-byte run of both the activation pixel and the weight row.  A logical block
// computes a 64x64 tile with 4x4 register micro-tiles; tiles are staged through double-buffered
// shared memory (17 KB).  The exact-fp32 path of the library: used for the 3-channel NCHW stem,
// odd shapes, and wherever the schedule asks for fp32 instead of TF32 tensor cores.
#pragma once
#include "task.cuh"

namespace reef {

constexpr int CBM = 64;   // pixels per tile
constexpr int CBN = 64;   // out-channels per tile
constexpr int CBK = 16;   // K slice
constexpr int CPAD = 4;
constexpr int kConvSimtSmem = 2 * CBK * (CBM + CPAD) * 4 + 2 * CBK * (CBN + CPAD) * 4 + 16;

__device__ __forceinline__ bool body_conv_simt(const KTask& t, int vb, unsigned char* smem_raw, const int* flag) {
    const ConvP& p = t.p.conv;
    const float* __restrict__ in = (const float*)t.a[0];
    const float* __restrict__ wgt = (const float*)t.a[1];
    float* __restrict__ out = (float*)t.a[2];

    typedef float (*TileA)[CBK][CBM + CPAD];
    typedef float (*TileB)[CBK][CBN + CPAD];
    TileA As = reinterpret_cast<TileA>(smem_raw);
    TileB Bs = reinterpret_cast<TileB>(smem_raw + 2 * CBK * (CBM + CPAD) * 4);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem_raw + kConvSimtSmem - 16);

    const int tid = threadIdx.x;
    const int tile_c = vb % p.tiles_c, tile_p = vb / p.tiles_c;
    const int p0 = tile_p * CBM, c0 = tile_c * CBN;

    // loader mapping: one float4 of A and one of B per thread and K slice
    const int lrow = tid >> 2, lk = (tid & 3) * 4;
    const int pix = p0 + lrow;
    const bool pvalid = pix < p.ptot;
    const int oy = pvalid ? pix / p.wo : 0, ox = pvalid ? pix - (pix / p.wo) * p.wo : 0;
    const int lco = c0 + lrow;
    const bool cvalid = lco < p.co;
    const float* wrow = wgt + (size_t)(cvalid ? lco : 0) * p.ktot;
    const bool fast = (p.ci % CBK) == 0 && !p.nchw;

    const int ty = tid >> 4, tx = tid & 15;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    const int ktiles = (p.ktot + CBK - 1) / CBK;
    if (tid == 0) *s_abort = 0;

    auto load_a = [&](int kt) -> float4 {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        const int k0 = kt * CBK;
        if (fast) {
            const int tap = k0 / p.ci, cb = k0 - tap * p.ci;
            const int ky = tap / p.kw, kx = tap - ky * p.kw;
            const int iy = oy * p.sh + ky - p.ph, ix = ox * p.sw + kx - p.pw;
            if (pvalid && iy >= 0 && iy < p.hi && ix >= 0 && ix < p.wi)
                v = *reinterpret_cast<const float4*>(in + ((size_t)iy * p.wi + ix) * p.ics + p.ioff + cb + lk);
        } else {
            float e[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                e[j] = 0.f;
                const int k = k0 + lk + j;
                if (pvalid && k < p.ktot) {
                    const int tap = k / p.ci, c = k - tap * p.ci;
                    const int ky = tap / p.kw, kx = tap - ky * p.kw;
                    const int iy = oy * p.sh + ky - p.ph, ix = ox * p.sw + kx - p.pw;
                    if (iy >= 0 && iy < p.hi && ix >= 0 && ix < p.wi)
                        e[j] = p.nchw ? in[((size_t)c * p.hi + iy) * p.wi + ix]
                                      : in[((size_t)iy * p.wi + ix) * p.ics + p.ioff + c];
                }
            }
            v = make_float4(e[0], e[1], e[2], e[3]);
        }
        return v;
    };
    auto load_b = [&](int kt) -> float4 {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        const int k = kt * CBK + lk;
        if (cvalid) {
            if (fast) {
                v = __ldg(reinterpret_cast<const float4*>(wrow + k));
            } else {
                float e[4];
#pragma unroll
                for (int j = 0; j < 4; j++) e[j] = (k + j < p.ktot) ? wrow[k + j] : 0.f;
                v = make_float4(e[0], e[1], e[2], e[3]);
            }
        }
        return v;
    };
    auto store_tiles = [&](int buf, const float4& a, const float4& b) {
        As[buf][lk + 0][lrow] = a.x; As[buf][lk + 1][lrow] = a.y;
        As[buf][lk + 2][lrow] = a.z; As[buf][lk + 3][lrow] = a.w;
        Bs[buf][lk + 0][lrow] = b.x; Bs[buf][lk + 1][lrow] = b.y;
        Bs[buf][lk + 2][lrow] = b.z; Bs[buf][lk + 3][lrow] = b.w;
    };

    {
        float4 a = load_a(0), b = load_b(0);
        store_tiles(0, a, b);
    }
    __syncthreads();

    for (int kt = 0; kt < ktiles; kt++) {
        const int buf = kt & 1;
        float4 na, nb;
        const bool more = kt + 1 < ktiles;
        if (more) {
            na = load_a(kt + 1);
            nb = load_b(kt + 1);
        }
        // best-effort flavour: one thread polls the preempt flag every 4th K slice; the value is
        // published through the barrier that already ends the slice
        if (flag != nullptr && (kt & 3) == 3 && tid == 0) *s_abort = ld_flag(flag);
#pragma unroll
        for (int k = 0; k < CBK; k++) {
            const float4 a = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w};
            const float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        if (more) store_tiles(buf ^ 1, na, nb);
        __syncthreads();
        if (flag != nullptr && *s_abort) return false;
    }

    // epilogue
    const int cb = c0 + tx * 4;
    if (cb < p.co) {
        const float* res = (p.ep & EP_RES) ? (const float*)t.a[p.i_res] : nullptr;
        float4 sc = make_float4(1.f, 1.f, 1.f, 1.f), sh = make_float4(0.f, 0.f, 0.f, 0.f);
        if (p.ep & EP_GB) {
            sc = *reinterpret_cast<const float4*>((const float*)t.a[p.i_gamma] + cb);
            sh = *reinterpret_cast<const float4*>((const float*)t.a[p.i_beta] + cb);
        } else if (p.ep & EP_BIAS) {
            sh = *reinterpret_cast<const float4*>((const float*)t.a[p.i_bias] + cb);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int op = p0 + ty * 4 + i;
            if (op >= p.ptot) continue;
            float4 v = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
            if (res) {
                const float4 r = *reinterpret_cast<const float4*>(res + (size_t)op * p.co + cb);
                v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
            }
            if (p.ep & EP_GB) {
                // explicit fused multiply-add: the three flavours of this body are compiled in different
                // kernels and must round identically
                v.x = fmaf(v.x, sc.x, sh.x); v.y = fmaf(v.y, sc.y, sh.y);
                v.z = fmaf(v.z, sc.z, sh.z); v.w = fmaf(v.w, sc.w, sh.w);
            } else {
                v.x += sh.x; v.y += sh.y; v.z += sh.z; v.w += sh.w;
            }
            if (p.ep & EP_GELU) {
                // exact-erf GELU (reference: resource/bert/bert.cu:167-173)
                v.x = v.x * (0.5f * erff(v.x * 0.70710678118654752440f) + 0.5f);
                v.y = v.y * (0.5f * erff(v.y * 0.70710678118654752440f) + 0.5f);
                v.z = v.z * (0.5f * erff(v.z * 0.70710678118654752440f) + 0.5f);
                v.w = v.w * (0.5f * erff(v.w * 0.70710678118654752440f) + 0.5f);
            }
            if (p.ep & EP_RELU) {
                v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f);
                v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
            }
            *reinterpret_cast<float4*>(out + (size_t)op * p.ocs + p.ooff + cb) = v;
        }
    }
    __syncthreads();   // tiles may be reused by the next logical block of a persistent caller
    return true;
}

}  // namespace reef
