// Host side of the tcgen05 convolution: tile/split planning, TMA tensor maps, cluster launch.
#include "conv_tc.cuh"

#include <cstdlib>
#include <cstring>
#include <string>

#include "registry.h"

namespace reef {

static int ceil_div_i(int a, int b) { return (a + b - 1) / b; }

// ---- planning (needs no GPU) --------------------------------------------------------------------
// One candidate plan: pixel tiles of at most `cap` pixels.
static int tc_plan_cap(const ConvP& p, int cap, TcPlan* pl) {
    memset(pl, 0, sizeof(*pl));
    pl->spatial = (p.kh * p.kw > 1 || p.sh > 1 || p.ph || p.pw) ? 1 : 0;
    pl->xsplit = 1;
    pl->xw = p.wo;
    if (pl->spatial && p.wo > cap) {
        // rows wider than a tile: cut every row into xsplit equal pieces
        int xs = ceil_div_i(p.wo, cap);
        while (xs <= p.wo && p.wo % xs != 0) xs++;
        if (xs > p.wo || p.wo / xs < 8) return REEF_NOT_FOUND;
        pl->xsplit = xs;
        pl->xw = p.wo / xs;
        pl->rows = 1;
        pl->n_valid = pl->xw;
        pl->n_tiles = p.ho * xs;
    } else if (pl->spatial) {
        int best = 1;
        const int rmax = cap / p.wo;
        const int lim = rmax < p.ho ? rmax : p.ho;
        for (int r = 1; r <= lim; r++)
            if (p.ho % r == 0) best = r;               // largest divisor of Ho that fits the tile
        if (best * 2 <= lim) best = lim;               // no useful divisor: ragged last tile
        pl->rows = best;
        pl->n_valid = best * p.wo;
        pl->n_tiles = ceil_div_i(p.ho, best);
    } else {
        int t = ceil_div_i(p.ptot, cap);
        pl->n_valid = ceil_div_i(p.ptot, t);
        pl->rows = 0;
        pl->n_tiles = ceil_div_i(p.ptot, pl->n_valid);
    }
    pl->n_mma = ceil_div_i(pl->n_valid, 16) * 16;
    if (pl->n_mma < 16) pl->n_mma = 16;
    pl->tmem_cols = 32;
    while (pl->tmem_cols < pl->n_mma) pl->tmem_cols *= 2;
    pl->m_tiles = ceil_div_i(p.co, TC_BM);
    pl->cblocks = ceil_div_i(p.ci, TC_BK);   // a ragged last channel block reads zeros beyond Cin (TMA out-of-bounds fill)
    pl->kb_total = p.kh * p.kw * pl->cblocks;
    // split K over a cluster until about 128 CTAs are in flight, keeping >= 2 K blocks per CTA
    const int base = pl->m_tiles * pl->n_tiles;
    int s = 1;
    if (p.plan_splits > 0) {
        while (s < p.plan_splits && s < TC_MAX_SPLITS && pl->kb_total >= s * 2) s *= 2;
    } else {
        while (s < TC_MAX_SPLITS && base * s * 2 <= 128 && pl->kb_total >= 2 * (s * 2)) s *= 2;
    }
    // every rank must own at least one K block and the cluster size stays a power of two
    for (;; s /= 2) {
        pl->kb_per_split = ceil_div_i(pl->kb_total, s);
        pl->splits = ceil_div_i(pl->kb_total, pl->kb_per_split);
        if (pl->splits == s || s == 1) break;
    }
    pl->b_bytes = pl->n_valid * 128;
    // Shared memory: at most TC_SMEM_CAP per CTA, so that two CTAs fit one SM (a real-time kernel beside the
    // early-launched prologue of its successor, or beside a best-effort kernel).  The stage ring is reused by
    // the epilogue for the staged accumulator tile (one 512-byte row per pixel) and, with a K split, the
    // exchange area recv[S-1][cpc_max][128].
    const int budget = TC_SMEM_CAP - 1024 - 256;   // alignment slack and control words
    const int stage_bytes = TC_A_BYTES + pl->n_mma * 128;
    pl->stages = pl->kb_per_split < TC_MAX_STAGES ? pl->kb_per_split : TC_MAX_STAGES;
    while (pl->stages > 1 && pl->stages * stage_bytes > budget) pl->stages--;
    if (pl->stages * stage_bytes > budget || (pl->stages < 2 && pl->kb_per_split > 1)) return REEF_NOT_FOUND;
    const int ring = pl->stages * stage_bytes;
    pl->cpc_max = ceil_div_i(pl->n_valid, pl->splits);
    pl->recv_offset_floats = pl->n_valid * TC_BM;
    const int epi = pl->n_valid * 512 + (pl->splits > 1 ? (pl->splits - 1) * pl->cpc_max * 512 : 0);
    if (epi > budget) return REEF_NOT_FOUND;
    pl->region_bytes = ring > epi ? ring : epi;
    pl->region_bytes = ((pl->region_bytes + 127) / 128) * 128;
    pl->smem = 1024 + pl->region_bytes + 256;   // alignment slack + data region + control words
    return REEF_SUCC;
}

// ---- planning (needs no GPU) --------------------------------------------------------------------
// Default plan (names without a tuned plan): tile caps are tried from large to small; the first plan that fits
// shared memory and puts at least 48 CTAs in flight wins, else the feasible plan with the most CTAs.  A batch-1
// layer is bound by what one SM can pull from L2 (about 85 GB/s per CTA measured): more CTAs shorten every
// CTA's load stream, at the price of re-reading weights from L2; where the balance lies depends on the shape
// (ResNet's 14x14 layers are fastest at 112-128 CTAs, BERT's 128-token matmuls at 48-96), so the resource
// generator writes measured plans into the kernel names (tp = tile cap, ts = K splits; reef_b200/tune.py).
int tc_plan(const ConvP& p, TcPlan* pl) {
    if (p.nchw || (p.ci & 3) || p.ci < 4 || p.sh != p.sw || (p.sh != 1 && p.sh != 2)) return REEF_NOT_FOUND;
    if ((p.ics & 3) || (p.ioff & 3) || (p.ocs & 3) || (p.ooff & 3) || (p.co & 3)) return REEF_NOT_FOUND;
    if (p.kh * p.kw > 64) return REEF_NOT_FOUND;
    if (p.plan_cap > 0) {
        // tile cap fixed by the kernel name (a tuned plan): that candidate or nothing
        if (p.plan_cap < 8 || p.plan_cap > 208) return REEF_NOT_FOUND;
        return tc_plan_cap(p, p.plan_cap, pl);
    }
    static const int caps[] = {208, 160, 112, 96, 64, 48, 32};
    TcPlan best;
    int best_ctas = 0;
    for (int cap : caps) {
        TcPlan c;
        if (tc_plan_cap(p, cap, &c) != REEF_SUCC) continue;
        const int ctas = c.splits * c.n_tiles * c.m_tiles;
        if (ctas > best_ctas && ctas <= 148) {
            best = c;
            best_ctas = ctas;
        } else if (best_ctas == 0) {
            best = c;
            best_ctas = ctas;
        }
        if (best_ctas >= 48) break;
    }
    if (best_ctas == 0) return REEF_NOT_FOUND;
    *pl = best;
    return REEF_SUCC;
}

// ---- tensor maps ---------------------------------------------------------------------------------
typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static encode_tiled_fn g_encode = nullptr;

static int get_encode() {
    if (g_encode) return REEF_SUCC;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
        set_error("cuTensorMapEncodeTiled is not available from the driver");
        return REEF_FAIL;
    }
    g_encode = (encode_tiled_fn)fn;
    return REEF_SUCC;
}

static int encode(CUtensorMap* tm, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes,
                  const cuuint32_t* box) {
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = g_encode(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<void*>(base), dims,
                          strides_bytes, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r));
        return REEF_FAIL;
    }
    return REEF_SUCC;
}

// The error word is pinned host memory mapped into the device's address space: a kernel whose bounded wait
// expired stores 1 through the device pointer, the host reads the word directly once the stream is synchronised.
static int* g_error_word[16] = {nullptr};        // device view
static int* g_error_word_host[16] = {nullptr};   // host view of the same word

int tc_error_word(int** out) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 16) return REEF_FAIL;
    if (!g_error_word[dev]) {
        int* h = nullptr;
        int* d = nullptr;
        if (cudaHostAlloc((void**)&h, 64, cudaHostAllocMapped) != cudaSuccess ||
            cudaHostGetDevicePointer((void**)&d, h, 0) != cudaSuccess) {
            set_error("cannot allocate the device error word");
            return REEF_FAIL;
        }
        *h = 0;
        g_error_word_host[dev] = h;
        g_error_word[dev] = d;
    }
    *out = g_error_word[dev];
    return REEF_SUCC;
}

int tc_error_word_host(volatile int** out) {
    int* d = nullptr;
    int rc = tc_error_word(&d);
    if (rc != REEF_SUCC) return rc;
    int dev = 0;
    cudaGetDevice(&dev);
    *out = g_error_word_host[dev];
    return REEF_SUCC;
}

int tc_build_params(const ConvP& p, const TcPlan& pl, void* const* a, TcParams* P) {
    int rc = get_encode();
    if (rc != REEF_SUCC) return rc;
    memset(P, 0, sizeof(*P));
    const float* in = (const float*)a[0];
    const float* wgt = (const float*)a[1];
    {
        // weights [Cout][tap][Cin] as a 3-d map (Cin, taps, Cout): a box is 32 channels of one tap for 128 output
        // channels, and channels beyond Cin (Cin not a multiple of 32) come back as zeros
        cuuint64_t dims[3] = {(cuuint64_t)p.ci, (cuuint64_t)(p.kh * p.kw), (cuuint64_t)p.co};
        cuuint64_t strides[2] = {(cuuint64_t)p.ci * 4, (cuuint64_t)p.ktot * 4};
        cuuint32_t box[3] = {TC_BK, 1, TC_BM};
        rc = encode(&P->tm_w, wgt, 3, dims, strides, box);
        if (rc != REEF_SUCC) return rc;
    }
    if (pl.spatial) {
        const int s = p.sh;
        for (int ry = 0; ry < s; ry++)
            for (int rx = 0; rx < s; rx++) {
                const int nx = (p.wi - rx + s - 1) / s, ny = (p.hi - ry + s - 1) / s;
                if (nx <= 0 || ny <= 0) continue;
                const float* base = in + p.ioff + ((size_t)ry * p.wi + rx) * p.ics;
                cuuint64_t dims[3] = {(cuuint64_t)p.ci, (cuuint64_t)nx, (cuuint64_t)ny};
                cuuint64_t strides[2] = {(cuuint64_t)s * p.ics * 4, (cuuint64_t)s * p.wi * p.ics * 4};
                cuuint32_t box[3] = {TC_BK, (cuuint32_t)pl.xw, (cuuint32_t)pl.rows};
                rc = encode(&P->tm_x[ry * s + rx], base, 3, dims, strides, box);
                if (rc != REEF_SUCC) return rc;
            }
    } else {
        cuuint64_t dims[2] = {(cuuint64_t)p.ci, (cuuint64_t)p.ptot};
        cuuint64_t strides[1] = {(cuuint64_t)p.ics * 4};
        cuuint32_t box[2] = {TC_BK, (cuuint32_t)pl.n_valid};
        rc = encode(&P->tm_x[0], in + p.ioff, 2, dims, strides, box);
        if (rc != REEF_SUCC) return rc;
    }
    P->out = (float*)a[2];
    P->res = (p.ep & EP_RES) ? (const float*)a[p.i_res] : nullptr;
    P->bias = (p.ep & EP_BIAS) ? (const float*)a[p.i_bias] : nullptr;
    P->gamma = (p.ep & EP_GB) ? (const float*)a[p.i_gamma] : nullptr;
    P->beta = (p.ep & EP_GB) ? (const float*)a[p.i_beta] : nullptr;
    P->out2 = (p.ep & EP_DUAL) ? (float*)a[p.i_out2] : nullptr;
    P->bias2 = (p.ep & EP_DUAL) ? (const float*)a[p.i_bias2] : nullptr;
    rc = tc_error_word(&P->error_word);
    if (rc != REEF_SUCC) return rc;
    P->co = p.co; P->ci = p.ci; P->ptot = p.ptot; P->ocs = p.ocs; P->ooff = p.ooff;
    P->spatial = pl.spatial; P->wo = p.wo; P->rows = pl.rows; P->xsplit = pl.xsplit; P->xw = pl.xw;
    P->n_valid = pl.n_valid; P->n_mma = pl.n_mma; P->tmem_cols = pl.tmem_cols;
    P->kh = p.kh; P->kw = p.kw; P->stride = p.sh; P->ph = p.ph; P->pw = p.pw;
    P->cblocks = pl.cblocks; P->kb_total = pl.kb_total; P->kb_per_split = pl.kb_per_split; P->splits = pl.splits;
    P->ep = 0;
    if (p.ep & EP_RES) P->ep |= TC_EP_RES;
    if (p.ep & EP_BIAS) P->ep |= TC_EP_BIAS;
    if (p.ep & EP_GB) P->ep |= TC_EP_GB;
    if (p.ep & EP_RELU) P->ep |= TC_EP_RELU;
    if (p.ep & EP_GELU) P->ep |= TC_EP_GELU;
    if (p.round_tf32) P->ep |= TC_EP_ROUND;
    P->b_bytes = pl.b_bytes;
    P->cb_magic = (unsigned)((0x100000000ull + (unsigned long long)pl.cblocks - 1) / (unsigned long long)pl.cblocks);
    for (int ky = 0; ky < p.kh; ky++)
        for (int kx = 0; kx < p.kw; kx++) {
            const int s = p.sh, dy = ky - p.ph, dx = kx - p.pw;
            const int ry = ((dy % s) + s) % s, rx = ((dx % s) + s) % s;
            const int tap = ky * p.kw + kx;
            P->tap_map[tap] = (signed char)(ry * s + rx);
            P->tap_qx[tap] = (signed char)((dx - rx) / s);
            P->tap_qy[tap] = (signed char)((dy - ry) / s);
        }
    P->stages = pl.stages;
    P->region_bytes = pl.region_bytes;
    P->recv_offset_floats = pl.recv_offset_floats;
    P->cpc_max = pl.cpc_max;
    P->n_tiles = pl.n_tiles;
    P->tile_begin = 0;
    P->pdl = 1;
    return REEF_SUCC;
}

static bool g_attr_set[16] = {false};

#ifdef REEF_DEBUG_AIDS
static long long* g_trace[16] = {nullptr};
// Phase trace of the tensor-core convolution (development builds only): when enabled, block (0,0) of every launch
// stamps the SM clock at 11 points (entry, set-up done, ring filled, peers up, first K block landed, last K block
// landed, accumulator complete, tile staged, exchange complete, rows finished, TMEM freed) into one 16-word device
// record that the host reads back.
int tc_trace_enable(int on) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 16) return REEF_FAIL;
    if (on && !g_trace[dev]) {
        if (cudaMalloc(&g_trace[dev], 128) != cudaSuccess || cudaMemset(g_trace[dev], 0, 128) != cudaSuccess) {
            set_error("cannot allocate the trace record");
            return REEF_FAIL;
        }
    } else if (!on && g_trace[dev]) {
        cudaFree(g_trace[dev]);
        g_trace[dev] = nullptr;
    }
    return REEF_SUCC;
}
int tc_trace_read(long long* out16) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 16 || !g_trace[dev]) return REEF_NOT_FOUND;
    if (cudaMemcpy(out16, g_trace[dev], 128, cudaMemcpyDeviceToHost) != cudaSuccess) return REEF_FAIL;
    return REEF_SUCC;
}
#endif

// Programmatic dependent launch is on (development builds can switch it off with REEF_PDL=0, and for padded
// best-effort pieces alone with REEF_PAD_PDL=0).
static bool env_flag_on(const char* name) {
#ifdef REEF_DEBUG_AIDS
    const char* v = getenv(name);
    return !(v && v[0] == '0');
#else
    (void)name;
    return true;
#endif
}

// one-time, per device: shared-memory opt-in of both flavours of the kernel and the error word (never during a capture)
int tc_prepare_device() {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16 && !g_attr_set[dev]) {
        const void* fns[2] = {(const void*)reef_conv_tc_kernel<false>, (const void*)reef_conv_tc_kernel<true>};
        for (const void* fn : fns) {
            cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
            if (e == cudaSuccess)   // the whole unified L1/shared array as shared memory, so that two CTAs are resident
                e = cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            if (e != cudaSuccess) {
                set_error(std::string("cudaFuncSetAttribute(conv_tc): ") + cudaGetErrorString(e));
                return REEF_FAIL;
            }
        }
        int* w = nullptr;
        int rc = tc_error_word(&w);
        if (rc != REEF_SUCC) return rc;
        g_attr_set[dev] = true;
    }
    return REEF_SUCC;
}

int tc_launch(const TcParams& P0, const TcPlan& pl, cudaStream_t st, const int* flag, int* slot, int tile_begin,
              int tile_count) {
    static const bool use_pdl = env_flag_on("REEF_PDL"), pad_pdl = env_flag_on("REEF_PAD_PDL");
    TcParams P = P0;
    P.preempt_flag = flag;
    P.task_slot = slot;
    const int tiles = pl.n_tiles * pl.m_tiles;
    if (tile_count < 0) tile_count = tiles - tile_begin;
    if (tile_begin < 0 || tile_count <= 0 || tile_begin + tile_count > tiles) {
        set_error("tensor-core convolution: tile range outside the kernel");
        return REEF_OUT_OF_RANGE;
    }
    P.tile_begin = tile_begin;
    P.stamps = flag != nullptr ? preempt_stamps_ptr() : nullptr;
    P.trace = nullptr;
#ifdef REEF_DEBUG_AIDS
    {
        int dev = 0;
        cudaGetDevice(&dev);
        P.trace = (dev >= 0 && dev < 16) ? g_trace[dev] : nullptr;
    }
#endif
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(pl.splits, tile_count, 1);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = st;
    cudaLaunchAttribute attrs[2];
    int na = 0;
    if (pl.splits > 1) {
        attrs[na].id = cudaLaunchAttributeClusterDimension;
        attrs[na].val.clusterDim.x = pl.splits;
        attrs[na].val.clusterDim.y = 1;
        attrs[na].val.clusterDim.z = 1;
        na++;
    }
    const bool piece = flag == nullptr && slot != nullptr;   // a padded best-effort piece
    if (use_pdl && (!piece || pad_pdl)) {
        attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = na;
    // the best-effort flavour (flag polls at block entry and at the producer's loop head) is its own instantiation:
    // the real-time flavour carries no poll
    cudaError_t e = flag != nullptr ? cudaLaunchKernelEx(&cfg, reef_conv_tc_kernel<true>, P)
                                    : cudaLaunchKernelEx(&cfg, reef_conv_tc_kernel<false>, P);
    if (e != cudaSuccess) {
        set_error(std::string("cudaLaunchKernelEx(conv_tc): ") + cudaGetErrorString(e));
        return REEF_FAIL;
    }
    return REEF_SUCC;
}

int tc_func_attrs(const TcPlan& pl, cudaFuncAttributes* fa, int* occ) {
    cudaError_t e = cudaFuncGetAttributes(fa, (const void*)reef_conv_tc_kernel<false>);
    if (e != cudaSuccess) {
        set_error(std::string("cudaFuncGetAttributes(conv_tc): ") + cudaGetErrorString(e));
        return REEF_FAIL;
    }
    // shared memory (plus the 1 KB the hardware reserves per CTA) and 124 registers x 256 threads: two at most
    const int by_smem = (228 * 1024) / (pl.smem + 1024);
    *occ = by_smem < 1 ? 1 : (by_smem > 2 ? 2 : by_smem);
    return REEF_SUCC;
}

}  // namespace reef
