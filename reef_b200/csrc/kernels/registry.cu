// Kernel registry: resolves "<family>__<key><int>_..." names from <model>.json to hand-written
// sm_100a kernels, plans their launch geometry, and launches them in the three flavours
// (plain, best-effort, dispatcher).  Replaces GPUModuleGetFunction / GPUModuleLaunchKernel on a
// per-model code object (reference: src/reef/executor/executor_base.cpp:47-52,211-223,
// src/reef/executor/hybrid_executor.cpp:153-163, src/reef/server/scheduler.cpp:613-649).
#include "registry.h"

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>

#include "attention_tc.cuh"
#include "bert.cuh"
#include "conv_simt.cuh"
#include "conv_tc_params.h"
#include "simple.cuh"

namespace reef {

// launches are counted from the scheduler thread and from request threads (a best-effort model captures its
// padding segments when it is bound to a queue)
static std::atomic<unsigned long long> g_launches{0};
static thread_local unsigned long long t_launches = 0;
static inline void count_launch() {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    t_launches++;
}

struct TcCache {
    TcParams params;
    AttParams att;
    void* ptrs[kMaxArgs];
    bool valid = false;
};

static inline bool is_tc_family(int f) { return f == F_CONV_TC || f == F_ATTENTION_TC; }

static thread_local std::string g_err;
void set_error(const std::string& s) { g_err = s; }
const char* last_error() { return g_err.c_str(); }

// ------------------------------------------------------------------------------------------
// name grammar
// ------------------------------------------------------------------------------------------
struct Attrs {
    std::map<std::string, long long> kv;
    bool has(const char* k) const { return kv.count(k) != 0; }
    long long get(const char* k, long long dflt) const {
        auto it = kv.find(k);
        return it == kv.end() ? dflt : it->second;
    }
    bool need(const char* k, int* out) const {
        auto it = kv.find(k);
        if (it == kv.end()) return false;
        *out = (int)it->second;
        return true;
    }
};

static bool parse_name(const std::string& name, std::string* op, Attrs* attrs) {
    size_t pos = name.find("__");
    if (pos == std::string::npos) {
        *op = name;
        return true;
    }
    *op = name.substr(0, pos);
    std::string tail = name.substr(pos + 2);
    size_t i = 0;
    while (i < tail.size()) {
        size_t j = tail.find('_', i);
        if (j == std::string::npos) j = tail.size();
        std::string tok = tail.substr(i, j - i);
        size_t d = 0;
        while (d < tok.size() && !(tok[d] >= '0' && tok[d] <= '9')) d++;
        if (d == 0 || d == tok.size()) return false;
        attrs->kv[tok.substr(0, d)] = atoll(tok.c_str() + d);
        i = j + 1;
    }
    return true;
}

static int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Build the device task + launch plan for a name.  Returns REEF_SUCC / REEF_NOT_FOUND.
static int build_spec(const std::string& name, KernelSpec* s) {
    std::string op;
    Attrs a;
    if (!parse_name(name, &op, &a)) {
        set_error("malformed kernel name: " + name);
        return REEF_NOT_FOUND;
    }
    memset(&s->task, 0, sizeof(KTask));
    s->name = name;
    s->block[0] = kThreads; s->block[1] = 1; s->block[2] = 1;
    s->dyn_smem = 0;
    s->flops = 0;
    s->bytes = 0;
    s->tensor_core = 0;
    KTask& t = s->task;

    if (op == "add" || op == "multiply") {
        // reference: resource/mocked_kernel/mocked_kernel.json launch_params [64,1,1,4,8,4]
        t.family = op == "add" ? F_MOCK_ADD : F_MOCK_MUL;
        t.nblocks = 64;
        s->block[0] = 4; s->block[1] = 8; s->block[2] = 4;
        s->nargs = 3;
        s->bytes = 4.0 * (128 + 2 * 8192);
        return REEF_SUCC;
    }
    if (op == "fused_add") {
        EltP& p = t.p.elt;
        if (!a.need("c", &p.c) || !a.need("hw", &p.n)) goto bad;
        t.family = F_FUSED_ADD_NCHW;
        t.nblocks = ceil_div(p.c * p.n, kEltPerBlock);
        s->nargs = 3;
        s->bytes = 4.0 * (2.0 * p.c * p.n + p.c);
        return REEF_SUCC;
    }
    if (op == "reef_nchw_to_nhwc4") {
        EltP& p = t.p.elt;
        if (!a.need("c", &p.c) || !a.need("hw", &p.n) || p.c < 1 || p.c > 4) goto bad;
        t.family = F_NCHW_TO_NHWC4;
        t.nblocks = ceil_div(p.n, kThreads);
        s->nargs = 3;
        s->bytes = 4.0 * ((double)p.c * p.n + 4.0 * p.n + p.c);
        return REEF_SUCC;
    }
    if (op == "reef_im2col_nchw") {
        ConvP& p = t.p.conv;
        if (!a.need("c", &p.ci) || !a.need("hi", &p.hi) || !a.need("wi", &p.wi) || !a.need("kh", &p.kh) ||
            !a.need("kw", &p.kw) || !a.need("sh", &p.sh) || !a.need("sw", &p.sw) || !a.need("ph", &p.ph) ||
            !a.need("pw", &p.pw) || !a.need("kp", &p.ocs))
            goto bad;
        if (p.ci < 1 || p.kh < 1 || p.kw < 1 || p.sh < 1 || p.sw < 1 || p.ph < 0 || p.pw < 0) goto bad;
        p.ho = (p.hi + 2 * p.ph - p.kh) / p.sh + 1;
        p.wo = (p.wi + 2 * p.pw - p.kw) / p.sw + 1;
        p.ktot = p.kh * p.kw * p.ci;
        p.ptot = p.ho * p.wo;
        if (p.ho < 1 || p.wo < 1 || (p.ocs & 3) || p.ocs < p.ktot || p.ocs > kIm2colMaxKp || (double)p.ptot * p.ocs > 5e8) goto bad;
        p.nchw = 1;
        t.family = F_IM2COL_NCHW;
        s->dyn_smem = (uint32_t)(p.ocs * 12);
        t.nblocks = ceil_div(p.ptot * (p.ocs / 4), kIm2colPerBlock);
        s->nargs = 3;
        s->bytes = 4.0 * ((double)p.ci * p.hi * p.wi + (double)p.ptot * p.ocs + p.ci);
        return REEF_SUCC;
    }
    if (op == "fused_add_nn_relu") {
        EltP& p = t.p.elt;
        if (!a.need("c", &p.c) || !a.need("n", &p.n)) goto bad;
        p.ics = (int)a.get("ics", p.c);
        p.ioff = (int)a.get("ioff", 0);
        if ((p.c | p.ics | p.ioff) & 3) goto bad;
        t.family = F_BIAS_RELU;
        t.nblocks = ceil_div(p.c * p.n, kEltPerBlock);
        s->nargs = 3;
        s->bytes = 4.0 * (2.0 * p.c * p.n + p.c);
        return REEF_SUCC;
    }
    if (op == "fused_nn_batch_flatten") {
        EltP& p = t.p.elt;
        if (!a.need("n", &p.n)) goto bad;
        t.family = F_COPY;
        t.nblocks = ceil_div(p.n, kEltPerBlock);
        s->nargs = 2;
        s->bytes = 8.0 * p.n;
        return REEF_SUCC;
    }
    if (op == "fused_nn_global_avg_pool2d") {
        EltP& p = t.p.elt;
        if (!a.need("c", &p.c) || !a.need("hw", &p.n)) goto bad;
        t.family = F_GLOBAL_AVG_POOL;
        t.nblocks = ceil_div(p.c, 32);
        s->dyn_smem = 8 * 32 * 4;
        s->nargs = 2;
        s->bytes = 4.0 * ((double)p.c * p.n + p.c);
        return REEF_SUCC;
    }
    if (op == "fused_nn_max_pool2d" || op == "fused_nn_max_pool2d_add_nn_relu" || op == "fused_nn_avg_pool2d") {
        PoolP& p = t.p.pool;
        if (!a.need("c", &p.c) || !a.need("hi", &p.hi) || !a.need("wi", &p.wi) || !a.need("k", &p.k) ||
            !a.need("s", &p.s) || !a.need("p", &p.p) || !a.need("ho", &p.ho) || !a.need("wo", &p.wo))
            goto bad;
        p.ics = (int)a.get("ics", p.c); p.ioff = (int)a.get("ioff", 0);
        p.ocs = (int)a.get("ocs", p.c); p.ooff = (int)a.get("ooff", 0);
        p.cip = (int)a.get("cip", 1);
        p.has_bias = op == "fused_nn_max_pool2d_add_nn_relu";
        if ((p.c | p.ics | p.ioff | p.ocs | p.ooff) & 3) goto bad;
        t.family = op == "fused_nn_avg_pool2d" ? F_AVG_POOL : F_MAX_POOL;
        t.nblocks = ceil_div(p.ho * p.wo * (p.c / 4), kPoolItemsPerBlock);
        s->nargs = p.has_bias ? 3 : 2;
        s->bytes = 4.0 * ((double)p.c * p.hi * p.wi + (double)p.c * p.ho * p.wo + (p.has_bias ? p.c : 0));
        return REEF_SUCC;
    }
    if (op == "fused_nn_dense_add" || op == "fused_nn_dense_add_nn_relu") {
        DenseP& p = t.p.dense;
        if (!a.need("k", &p.k) || !a.need("n", &p.n)) goto bad;
        p.relu = op == "fused_nn_dense_add_nn_relu";
        t.family = F_DENSE;
        t.nblocks = dense_num_blocks(p.n);
        s->dyn_smem = kDenseSmem;
        s->nargs = 4;
        s->flops = 2.0 * p.k * p.n;
        s->bytes = 4.0 * ((double)p.k * p.n + p.k + 2.0 * p.n);
        return REEF_SUCC;
    }
    if (op == "fused_nn_softmax") {
        SoftmaxP& p = t.p.softmax;
        if (!a.need("n", &p.n)) goto bad;
        p.rows = (int)a.get("rows", 1);
        t.family = F_SOFTMAX;
        t.nblocks = p.rows;
        s->dyn_smem = 16 * 4;
        s->nargs = 2;
        s->bytes = 8.0 * p.rows * p.n;
        return REEF_SUCC;
    }
    if (op == "reef_embedding") {
        int sN, h, vocab;
        if (!a.need("s", &sN) || !a.need("h", &h) || !a.need("vocab", &vocab) || (h & 3)) goto bad;
        t.p.raw[0] = sN; t.p.raw[1] = h; t.p.raw[2] = vocab;
        t.family = F_EMBEDDING;
        t.nblocks = ceil_div(sN * (h / 4), kThreads * 4);
        s->nargs = 4;
        s->bytes = 4.0 * 3.0 * sN * h + 8.0 * sN;
        return REEF_SUCC;
    }
    if (op == "reef_layernorm" || op == "reef_add_layernorm") {
        int rows, h;
        if (!a.need("rows", &rows) || !a.need("h", &h) || (h % 128) != 0 || h > 1024) goto bad;
        t.p.raw[0] = rows; t.p.raw[1] = h; t.p.raw[2] = op == "reef_add_layernorm";
        t.family = F_LAYERNORM;
        t.nblocks = ceil_div(rows, kLnRowsPerBlock);
        s->nargs = t.p.raw[2] ? 5 : 4;
        s->bytes = 4.0 * ((2.0 + t.p.raw[2]) * rows * h + 2.0 * h);
        return REEF_SUCC;
    }
    if (op == "reef_attention") {
        int sN, heads, d;
        if (!a.need("s", &sN) || !a.need("heads", &heads) || !a.need("d", &d) || d != kAttD) goto bad;
        t.p.raw[0] = sN; t.p.raw[1] = heads; t.p.raw[2] = d; t.p.raw[3] = (int)a.get("mask", 0);
        s->nargs = t.p.raw[3] ? 3 : 2;
        s->flops = 4.0 * heads * (double)sN * sN * d;
        s->bytes = 4.0 * 4.0 * sN * heads * d;
        if ((int)a.get("v", 0) == 1) {
            // tensor-core variant: one CTA per head, both products on tcgen05 (attention_tc.cuh)
            if (!att_supported(sN, heads, d)) {
                set_error("shape not supported by the tensor-core attention (at most 128 tokens, d = 64): " + name);
                return REEF_NOT_FOUND;
            }
            t.family = F_ATTENTION_TC;
            t.nblocks = heads;
            s->dyn_smem = (uint32_t)att_smem_bytes();
            s->block[0] = ATT_THREADS;
            s->tensor_core = 1;
            return REEF_SUCC;
        }
        t.family = F_ATTENTION;
        t.nblocks = heads * ceil_div(sN, kAttRows);
        s->dyn_smem = kAttSmem;
        return REEF_SUCC;
    }
    if (op.rfind("reef_matmul_nt", 0) == 0) {
        // C[m][n] = sum_k A[m][k] * B[n][k] (+bias[n]) (GELU) (+residual[m][n])  (reference: bert.cu:206-271):
        // a 1x1 convolution over m "pixels": A = channels-last activations, B = weights [n][k]
        ConvP& p = t.p.conv;
        std::string tail = op.substr(strlen("reef_matmul_nt"));
        int m, n, k;
        if (!a.need("m", &m) || !a.need("n", &n) || !a.need("k", &k)) goto bad;
        p.ep = 0;
        p.i_res = p.i_bias = p.i_gamma = p.i_beta = p.i_bias2 = p.i_out2 = -1;
        int nargs = 3;
        if (tail.find("_bias") != std::string::npos) { p.ep |= EP_BIAS; p.i_bias = nargs++; }
        if (tail.find("_gelu") != std::string::npos) p.ep |= EP_GELU;
        if (tail.find("_residual") != std::string::npos) { p.ep |= EP_RES; p.i_res = nargs++; }
        p.ci = k; p.hi = 1; p.wi = m; p.co = n; p.kh = p.kw = 1; p.sh = p.sw = 1; p.ph = p.pw = 0;
        p.ho = 1; p.wo = m; p.nchw = 0; p.ics = k; p.ioff = 0; p.ocs = n; p.ooff = 0;
        p.ktot = k; p.ptot = m;
        if ((n & 3) || (k & 3)) goto bad;
        s->nargs = nargs;
        s->flops = 2.0 * m * (double)n * k;
        s->bytes = 4.0 * ((double)m * k + (double)n * k + (double)m * n * ((p.ep & EP_RES) ? 2.0 : 1.0) + n);
        if ((int)a.get("v", 0) == 1) {
            p.round_tf32 = (int)a.get("rt", 0);   // outputs feed LayerNorm / attention in fp32: no TF32 rounding
            p.plan_cap = (int)a.get("tp", 0);
            p.plan_splits = (int)a.get("ts", 0);
            if (tc_plan(p, &s->tc) != REEF_SUCC) goto bad;
            t.family = F_CONV_TC;
            t.nblocks = s->tc.splits * s->tc.n_tiles * s->tc.m_tiles;
            s->dyn_smem = (uint32_t)s->tc.smem;
            s->block[0] = TC_THREADS;
            s->tensor_core = 1;
            return REEF_SUCC;
        }
        t.family = F_CONV_SIMT;
        p.tiles_p = ceil_div(p.ptot, CBM);
        p.tiles_c = ceil_div(p.co, CBN);
        t.nblocks = p.tiles_p * p.tiles_c;
        s->dyn_smem = kConvSimtSmem;
        return REEF_SUCC;
    }
    // reef_conv2d_add_preact: conv + residual written to `out`, and relu(out + bias2) written to `out2` by the
    // same epilogue: the reference's fused_nn_conv2d_add followed by the next unit's fused_add_nn_relu
    // (resource/resnet152/resnet152.cu:340-363 and :2-12) in one launch.  args: in, weight, out, residual, bias2, out2.
    if (op == "reef_conv2d_add_preact" || op.rfind("fused_nn_conv2d", 0) == 0) {
        const bool preact = op == "reef_conv2d_add_preact";
        ConvP& p = t.p.conv;
        std::string tail = preact ? std::string("_add") : op.substr(strlen("fused_nn_conv2d"));
        p.ep = 0;
        p.i_res = p.i_bias = p.i_gamma = p.i_beta = p.i_bias2 = p.i_out2 = -1;
        bool relu = false;
        const std::string r = "_nn_relu";
        if (tail.size() >= r.size() && tail.compare(tail.size() - r.size(), r.size(), r) == 0) {
            relu = true;
            tail = tail.substr(0, tail.size() - r.size());
        }
        int nargs = 3;
        if (tail == "") {
        } else if (tail == "_add") {
            if (relu) { p.ep |= EP_BIAS; p.i_bias = 3; } else { p.ep |= EP_RES; p.i_res = 3; }
            nargs = 4;
        } else if (tail == "_add_add") {
            p.ep |= EP_RES | EP_BIAS; p.i_res = 3; p.i_bias = 4;
            nargs = 5;
        } else if (tail == "_add_multiply_add") {
            p.ep |= EP_RES | EP_GB; p.i_res = 3; p.i_gamma = 4; p.i_beta = 5;
            nargs = 6;
        } else {
            set_error("unknown conv2d family: " + op);
            return REEF_NOT_FOUND;
        }
        if (relu) p.ep |= EP_RELU;
        if (preact) {
            p.ep |= EP_DUAL;
            p.i_bias2 = 4;
            p.i_out2 = 5;
            nargs = 6;
        }
        if (!a.need("ci", &p.ci) || !a.need("hi", &p.hi) || !a.need("wi", &p.wi) || !a.need("co", &p.co) ||
            !a.need("kh", &p.kh) || !a.need("kw", &p.kw) || !a.need("sh", &p.sh) || !a.need("sw", &p.sw) ||
            !a.need("ph", &p.ph) || !a.need("pw", &p.pw))
            goto bad;
        p.nchw = (int)a.get("nchw", 0);
        p.ics = (int)a.get("ics", p.ci); p.ioff = (int)a.get("ioff", 0);
        p.ocs = (int)a.get("ocs", p.co); p.ooff = (int)a.get("ooff", 0);
        p.ho = (p.hi + 2 * p.ph - p.kh) / p.sh + 1;
        p.wo = (p.wi + 2 * p.pw - p.kw) / p.sw + 1;
        p.ktot = p.kh * p.kw * p.ci;
        p.ptot = p.ho * p.wo;
        if (p.ho <= 0 || p.wo <= 0) goto bad;
        if ((p.co | p.ocs | p.ooff) & 3) goto bad;
        if (!p.nchw && (p.ci % CBK) == 0 && ((p.ics | p.ioff) & 3)) goto bad;
        s->nargs = nargs;
        // algorithmic work counts the real input channels (cr: the 3-channel model input is padded to 4)
        const double cr = (double)a.get("cr", p.ci);
        s->flops = 2.0 * p.co * (double)(p.kh * p.kw) * cr * p.ptot;
        s->bytes = 4.0 * (cr * p.hi * p.wi + (double)p.co * p.kh * p.kw * cr + (double)p.co * p.ptot *
                          ((p.ep & EP_RES) ? 2.0 : 1.0) + p.co * ((p.ep & EP_GB) ? 2.0 : ((p.ep & EP_BIAS) ? 1.0 : 0.0)));
        if (preact) s->bytes += 4.0 * ((double)p.co * p.ptot + p.co);
        int impl = (int)a.get("v", 0);
        if (preact && (impl != 1 || p.ocs != p.co || p.ooff != 0)) {
            set_error("reef_conv2d_add_preact exists as the tensor-core variant (_v1) with a dense output only: " + name);
            return REEF_NOT_FOUND;
        }
        if (impl == 0) {
            t.family = F_CONV_SIMT;
            p.tiles_p = ceil_div(p.ptot, CBM);
            p.tiles_c = ceil_div(p.co, CBN);
            t.nblocks = p.tiles_p * p.tiles_c;
            s->dyn_smem = kConvSimtSmem;
            return REEF_SUCC;
        }
        if (impl == 1) {
            // tcgen05 TF32 implicit GEMM; "rt0" in the name keeps full fp32 bits in the stored activations
            p.round_tf32 = (int)a.get("rt", 1);
            p.plan_cap = (int)a.get("tp", 0);       // tuned plan carried by the name: tile cap and K splits
            p.plan_splits = (int)a.get("ts", 0);
            if (tc_plan(p, &s->tc) != REEF_SUCC) {
                set_error("shape not supported by the tensor-core convolution: " + name);
                return REEF_NOT_FOUND;
            }
            t.family = F_CONV_TC;
            t.nblocks = s->tc.splits * s->tc.n_tiles * s->tc.m_tiles;
            s->dyn_smem = (uint32_t)s->tc.smem;
            s->block[0] = TC_THREADS;
            s->tensor_core = 1;
            return REEF_SUCC;
        }
        set_error("unknown conv2d variant in: " + name);
        return REEF_NOT_FOUND;
    }
    set_error("unknown kernel family: " + op);
    return REEF_NOT_FOUND;
bad:
    set_error("unsupported shape or missing attribute in kernel name: " + name);
    return REEF_NOT_FOUND;
}

// Least size in bytes of the buffer behind each positional argument: what one launch reads or writes through it.
// The model loader compares these with the storage table of <model>.json, so that a json whose storage entry is too
// small for the shape in the kernel name is refused instead of letting the kernel run past its slice of the arena.
static void fill_arg_bytes(KernelSpec* s) {
    for (int i = 0; i < kMaxArgs; i++) s->arg_bytes[i] = 0;
    const KTask& t = s->task;
    size_t* b = s->arg_bytes;
    auto f4 = [](double n) { return (size_t)(n > 0 ? n : 0) * 4; };
    switch (t.family) {
        case F_MOCK_ADD:
        case F_MOCK_MUL:
            b[0] = f4(kMockThreads); b[1] = f4(64.0 * kMockThreads); b[2] = b[1];
            break;
        case F_FUSED_ADD_NCHW:
            b[0] = b[1] = f4((double)t.p.elt.c * t.p.elt.n); b[2] = f4(t.p.elt.c);
            break;
        case F_NCHW_TO_NHWC4:
            b[0] = f4(4.0 * t.p.elt.n); b[1] = f4((double)t.p.elt.c * t.p.elt.n); b[2] = f4(t.p.elt.c);
            break;
        case F_IM2COL_NCHW:
            b[0] = f4((double)t.p.conv.ptot * t.p.conv.ocs);
            b[1] = f4((double)t.p.conv.ci * t.p.conv.hi * t.p.conv.wi);
            b[2] = f4(t.p.conv.ci);
            break;
        case F_BIAS_RELU:
            b[0] = f4((double)t.p.elt.c * t.p.elt.n);
            b[1] = f4((double)(t.p.elt.n - 1) * t.p.elt.ics + t.p.elt.ioff + t.p.elt.c);
            b[2] = f4(t.p.elt.c);
            break;
        case F_COPY:
            b[0] = b[1] = f4(t.p.elt.n);
            break;
        case F_GLOBAL_AVG_POOL:
            b[0] = f4((double)t.p.elt.c * t.p.elt.n); b[1] = f4(t.p.elt.c);
            break;
        case F_MAX_POOL:
        case F_AVG_POOL: {
            const PoolP& p = t.p.pool;
            b[0] = f4((double)(p.hi * p.wi - 1) * p.ics + p.ioff + p.c);
            b[1] = f4((double)(p.ho * p.wo - 1) * p.ocs + p.ooff + p.c);
            if (p.has_bias) b[2] = f4(p.c);
            break;
        }
        case F_DENSE:
            b[0] = f4(t.p.dense.k); b[1] = f4((double)t.p.dense.k * t.p.dense.n); b[2] = b[3] = f4(t.p.dense.n);
            break;
        case F_SOFTMAX:
            b[0] = b[1] = f4((double)t.p.softmax.rows * t.p.softmax.n);
            break;
        case F_EMBEDDING: {
            const double sN = t.p.raw[0], h = t.p.raw[1], vocab = t.p.raw[2];
            b[0] = f4(sN * h); b[1] = f4(vocab * h); b[2] = (size_t)sN * 8; b[3] = f4(sN * h);
            break;
        }
        case F_LAYERNORM: {
            const double rows = t.p.raw[0], h = t.p.raw[1];
            int i = 0;
            b[i++] = f4(rows * h); b[i++] = f4(rows * h);
            if (t.p.raw[2]) b[i++] = f4(rows * h);
            b[i++] = f4(h); b[i++] = f4(h);
            break;
        }
        case F_ATTENTION:
        case F_ATTENTION_TC: {
            const double sN = t.p.raw[0], H = (double)t.p.raw[1] * t.p.raw[2];
            int i = 0;
            b[i++] = f4(sN * 3 * H);
            if (t.p.raw[3]) b[i++] = f4(sN);
            b[i++] = f4(sN * H);
            break;
        }
        case F_CONV_SIMT:
        case F_CONV_TC: {
            const ConvP& p = t.p.conv;
            b[0] = p.nchw ? f4((double)p.ci * p.hi * p.wi) : f4((double)(p.hi * p.wi - 1) * p.ics + p.ioff + p.ci);
            b[1] = f4((double)p.co * p.ktot);
            b[2] = f4((double)(p.ptot - 1) * p.ocs + p.ooff + p.co);
            if (p.i_res >= 0) b[p.i_res] = f4((double)p.ptot * p.co);
            if (p.i_bias >= 0) b[p.i_bias] = f4(p.co);
            if (p.i_gamma >= 0) b[p.i_gamma] = f4(p.co);
            if (p.i_beta >= 0) b[p.i_beta] = f4(p.co);
            if (p.i_bias2 >= 0) b[p.i_bias2] = f4(p.co);
            if (p.i_out2 >= 0) b[p.i_out2] = f4((double)p.ptot * p.co);
            break;
        }
        default:
            break;
    }
}

int plan_kernel(const char* name, KernelSpec* s) {
    int rc = build_spec(name, s);
    if (rc != REEF_SUCC) return rc;
    fill_arg_bytes(s);
    if (s->task.family == F_CONV_TC) {
        s->grid[0] = (uint32_t)s->tc.splits;
        s->grid[1] = (uint32_t)(s->tc.n_tiles * s->tc.m_tiles);
        s->grid[2] = 1;
        return REEF_SUCC;
    }
    s->grid[0] = (uint32_t)s->task.nblocks;
    s->grid[1] = 1;
    s->grid[2] = 1;
    return REEF_SUCC;
}

// ------------------------------------------------------------------------------------------
// device flavours
// ------------------------------------------------------------------------------------------
template <int F>
__device__ __forceinline__ bool run_body(const KTask& t, int vb, unsigned char* smem, const int* flag) {
    if (F == F_MOCK_ADD) return body_mock<false>(t, vb, smem, flag);
    if (F == F_MOCK_MUL) return body_mock<true>(t, vb, smem, flag);
    if (F == F_FUSED_ADD_NCHW) return body_fused_add_nchw(t, vb, smem, flag);
    if (F == F_NCHW_TO_NHWC4) return body_nchw_to_nhwc4(t, vb, smem, flag);
    if (F == F_IM2COL_NCHW) return body_im2col_nchw(t, vb, smem, flag);
    if (F == F_BIAS_RELU) return body_bias_relu(t, vb, smem, flag);
    if (F == F_CONV_SIMT) return body_conv_simt(t, vb, smem, flag);
    if (F == F_MAX_POOL) return body_pool<true>(t, vb, smem, flag);
    if (F == F_AVG_POOL) return body_pool<false>(t, vb, smem, flag);
    if (F == F_GLOBAL_AVG_POOL) return body_gap(t, vb, smem, flag);
    if (F == F_COPY) return body_copy(t, vb, smem, flag);
    if (F == F_DENSE) return body_dense(t, vb, smem, flag);
    if (F == F_SOFTMAX) return body_softmax(t, vb, smem, flag);
    if (F == F_EMBEDDING) return body_embedding(t, vb, smem, flag);
    if (F == F_LAYERNORM) return body_layernorm(t, vb, smem, flag);
    if (F == F_ATTENTION) return body_attention(t, vb, smem, flag);
    return true;
}

__device__ __forceinline__ bool run_any(const KTask& t, int vb, unsigned char* smem, const int* flag) {
    switch (t.family) {
        case F_MOCK_ADD: return run_body<F_MOCK_ADD>(t, vb, smem, flag);
        case F_MOCK_MUL: return run_body<F_MOCK_MUL>(t, vb, smem, flag);
        case F_FUSED_ADD_NCHW: return run_body<F_FUSED_ADD_NCHW>(t, vb, smem, flag);
        case F_NCHW_TO_NHWC4: return run_body<F_NCHW_TO_NHWC4>(t, vb, smem, flag);
        case F_IM2COL_NCHW: return run_body<F_IM2COL_NCHW>(t, vb, smem, flag);
        case F_BIAS_RELU: return run_body<F_BIAS_RELU>(t, vb, smem, flag);
        case F_CONV_SIMT: return run_body<F_CONV_SIMT>(t, vb, smem, flag);
        case F_MAX_POOL: return run_body<F_MAX_POOL>(t, vb, smem, flag);
        case F_AVG_POOL: return run_body<F_AVG_POOL>(t, vb, smem, flag);
        case F_GLOBAL_AVG_POOL: return run_body<F_GLOBAL_AVG_POOL>(t, vb, smem, flag);
        case F_COPY: return run_body<F_COPY>(t, vb, smem, flag);
        case F_DENSE: return run_body<F_DENSE>(t, vb, smem, flag);
        case F_SOFTMAX: return run_body<F_SOFTMAX>(t, vb, smem, flag);
        case F_EMBEDDING: return run_body<F_EMBEDDING>(t, vb, smem, flag);
        case F_LAYERNORM: return run_body<F_LAYERNORM>(t, vb, smem, flag);
        case F_ATTENTION: return run_body<F_ATTENTION>(t, vb, smem, flag);
        default: return true;
    }
}

extern __shared__ __align__(16) unsigned char reef_dyn_smem[];

// Programmatic dependent launch: this kernel waits for its predecessor's results before touching memory (a
// no-op for an ordinary launch) and only then lets its successor start its prologue.  Releasing the successor
// before the wait would let a chain of kernels run ahead without bound: every grid's blocks would become
// resident, release the next grid and park at their wait, until the SMs are full of parked blocks and a
// best-effort kernel on another stream finds no room.  In this order at most two grids of a chain are resident.
__device__ __forceinline__ void pdl_prologue() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Device-side preemption stamps (optional, measurement only): when the host has armed the two words with
// reef_preempt_stamps_arm, the first best-effort block that sees the preempt flag up records %globaltimer into word
// 0 (minimum) and every block that leaves because of the flag records it into word 1 (maximum), so that
// word1 - word0 is the time, on the device's own clock, from the flag becoming visible to the last best-effort
// block leaving.
__device__ unsigned long long* g_preempt_stamps = nullptr;
__device__ __forceinline__ void preempt_stamp_leave() {
    unsigned long long* w = g_preempt_stamps;
    if (w == nullptr) return;
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    atomicMin(&w[0], t);
    atomicMax(&w[1], t);
}

template <int F>
__global__ void __launch_bounds__(kThreads) k_plain(const __grid_constant__ KTask t) {
    pdl_prologue();
    run_body<F>(t, blockIdx.x, reef_dyn_smem, nullptr);
}

// Best-effort flavour (reference wrapper: script/best_effort_kernel.py:22-33): leave at once when
// the preempt flag is up; bodies poll it again at their loop heads; a block that ran to the end
// (all of its stores issued, fenced) adds one to the kernel's completion counter.
template <int F>
__global__ void __launch_bounds__(kThreads) k_be(const __grid_constant__ KTask t, const int* __restrict__ flag,
                                                 int* __restrict__ task_slot) {
    pdl_prologue();
    // ONE thread reads the flag and the block takes one decision: were every thread to read it for itself, a flag
    // that goes up between the reads of two warps would let part of a block leave and the rest run the body with
    // threads missing (wrong partial sums counted as a complete block, barriers short of arrivals).
    if (__syncthreads_or(threadIdx.x == 0 ? ld_flag(flag) : 0)) {
        if (threadIdx.x == 0) preempt_stamp_leave();
        return;
    }
    const bool done = run_body<F>(t, blockIdx.x, reef_dyn_smem, flag);
    // a body may stop at a loop head in some of its warps only (the GEMV polls per warp): the block counts as
    // complete only when every thread ran to the end
    const int stopped = __syncthreads_or(done ? 0 : 1);
    if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) {
        if (!stopped) {
            red_release_gpu_add(task_slot, 1);
        } else {
            preempt_stamp_leave();
        }
    }
}

// Persistent dispatcher (dynamic kernel padding).  ctrl[0] = real-time ticket, ctrl[1] =
// best-effort ticket, ctrl[2] = drained blocks.  The role of a block comes from the SM it is
// resident on, not from its index: the reference assumes round-robin block placement over CUs
// (reference: resource/mocked_kernel/mocked_kernel.trans.cu:112-186, blockIdx.x % 60), which
// CUDA does not promise; tickets make the result independent of placement.
__device__ __forceinline__ int next_ticket(int* counter, int* s_slot) {
    __syncthreads();
    if (threadIdx.x == 0) *s_slot = atomicAdd(counter, 1);
    __syncthreads();
    return *s_slot;
}

__global__ void __launch_bounds__(kThreads) k_dispatch(const __grid_constant__ KTask rt, const __grid_constant__ KTask be,
                                                       int be_off, int be_num, int sm_partition,
                                                       int* __restrict__ be_slot, int* __restrict__ ctrl) {
    __shared__ int s_ticket;
    unsigned smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    const bool rt_first = (int)smid < sm_partition;

#pragma unroll 1
    for (int phase = 0; phase < 2; phase++) {
        const bool do_rt = (phase == 0) == rt_first;
        if (do_rt) {
            for (;;) {
                int v = next_ticket(&ctrl[0], &s_ticket);
                if (v >= rt.nblocks) break;
                run_any(rt, v, reef_dyn_smem, nullptr);
            }
        } else {
            for (;;) {
                int v = next_ticket(&ctrl[1], &s_ticket);
                if (v >= be_num) break;
                run_any(be, be_off + v, reef_dyn_smem, nullptr);
                __syncthreads();
                if (threadIdx.x == 0) red_release_gpu_add(be_slot, 1);
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        int d = atomicAdd(&ctrl[2], 1);
        if (d == (int)gridDim.x - 1) {
            ctrl[0] = 0;
            ctrl[1] = 0;
            __threadfence();
            ctrl[2] = 0;
        }
    }
}

// Bounded busy-wait of one thread (profiling aid: holds a stream while the host queues launches behind it).
__global__ void k_delay(unsigned long long ns) {
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    if (ns > 20000000ull) ns = 20000000ull;   // never more than 20 ms
    for (int i = 0; i < (1 << 24); i++) {
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 >= ns) break;
        __nanosleep(200);
    }
}

// ---- preemption stamps: host side ---------------------------------------------------------------------------
static unsigned long long* g_stamps_dev[16] = {nullptr};

unsigned long long* preempt_stamps_ptr() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
    return g_stamps_dev[dev];
}

static int stamps_reset(unsigned long long* d) {
    const unsigned long long init[2] = {~0ull, 0ull};
    if (cudaMemcpy(d, init, sizeof(init), cudaMemcpyHostToDevice) != cudaSuccess) {
        set_error("preemption stamps: cannot reset the device words");
        return REEF_FAIL;
    }
    return REEF_SUCC;
}

int preempt_stamps_arm(int on) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return REEF_FAIL;
    unsigned long long* d = g_stamps_dev[dev];
    if (on && d == nullptr) {
        if (cudaMalloc(&d, 16) != cudaSuccess) {
            set_error("preemption stamps: cannot allocate the device words");
            return REEF_FAIL;
        }
        if (stamps_reset(d) != REEF_SUCC) return REEF_FAIL;
        g_stamps_dev[dev] = d;
    } else if (!on && d != nullptr) {
        g_stamps_dev[dev] = nullptr;
        unsigned long long* null = nullptr;
        cudaMemcpyToSymbol(g_preempt_stamps, &null, sizeof(null));
        cudaDeviceSynchronize();
        cudaFree(d);
        return REEF_SUCC;
    }
    unsigned long long* sym = on ? g_stamps_dev[dev] : nullptr;
    if (cudaMemcpyToSymbol(g_preempt_stamps, &sym, sizeof(sym)) != cudaSuccess) {
        set_error("preemption stamps: cannot set the device pointer");
        return REEF_FAIL;
    }
    return REEF_SUCC;
}

int preempt_stamps_read(unsigned long long out[2]) {
    unsigned long long* d = preempt_stamps_ptr();
    if (d == nullptr) return REEF_NOT_FOUND;
    if (cudaMemcpy(out, d, 16, cudaMemcpyDeviceToHost) != cudaSuccess) {
        set_error("preemption stamps: cannot read the device words");
        return REEF_FAIL;
    }
    return stamps_reset(d);
}

int launch_delay(cudaStream_t st, unsigned long long ns) {
    k_delay<<<1, 1, 0, st>>>(ns);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error(std::string("k_delay: ") + cudaGetErrorString(e));
        return REEF_FAIL;
    }
    return REEF_SUCC;
}

// ------------------------------------------------------------------------------------------
// host launchers
// ------------------------------------------------------------------------------------------
unsigned long long launch_count() { return g_launches.load(std::memory_order_relaxed); }
unsigned long long thread_launch_count() { return t_launches; }
void add_launches(unsigned long long n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

#define FOR_EACH_FAMILY(X)                                                                      \
    X(F_MOCK_ADD) X(F_MOCK_MUL) X(F_FUSED_ADD_NCHW) X(F_BIAS_RELU) X(F_CONV_SIMT) X(F_MAX_POOL) \
    X(F_AVG_POOL) X(F_GLOBAL_AVG_POOL) X(F_COPY) X(F_DENSE) X(F_SOFTMAX) X(F_EMBEDDING) X(F_LAYERNORM) X(F_ATTENTION) \
    X(F_NCHW_TO_NHWC4) X(F_IM2COL_NCHW)

static const void* plain_fn(int family) {
    switch (family) {
#define X(F) case F: return (const void*)k_plain<F>;
        FOR_EACH_FAMILY(X)
#undef X
        default: return nullptr;
    }
}
static const void* be_fn(int family) {
    switch (family) {
#define X(F) case F: return (const void*)k_be<F>;
        FOR_EACH_FAMILY(X)
#undef X
        default: return nullptr;
    }
}

// One-time, per device: every kernel asks for the same split of the SM's unified L1/shared array as the
// tensor-core kernel (all of it as shared memory).  CTAs of kernels with different carve-outs cannot share an
// SM: behind a tensor-core kernel that fills every SM, a kernel with another preference had to wait for whole
// SMs to drain and be reconfigured (BERT-base replay 0.92 -> 1.13 ms with 216-CTA matmul plans).
static bool g_carveout_set[16] = {false};
static void prepare_carveout() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16 || g_carveout_set[dev]) return;
    for (int f = 0; f < F_COUNT; f++) {
        cudaFuncSetAttribute(plain_fn(f), cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(be_fn(f), cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    }
    cudaFuncSetAttribute((const void*)k_dispatch, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    // the GEMV's copy ring takes more than the 48 KB a kernel gets without asking (also when the dispatcher hosts it)
    cudaFuncSetAttribute(plain_fn(F_DENSE), cudaFuncAttributeMaxDynamicSharedMemorySize, kDenseSmem);
    cudaFuncSetAttribute(be_fn(F_DENSE), cudaFuncAttributeMaxDynamicSharedMemorySize, kDenseSmem);
    cudaFuncSetAttribute((const void*)k_dispatch, cudaFuncAttributeMaxDynamicSharedMemorySize, kDenseSmem);
    int* w = nullptr;
    tc_error_word(&w);   // the device error word exists before any launch can be part of a stream capture
    cudaGetLastError();
    g_carveout_set[dev] = true;
}

// Launch with the programmatic-stream-serialization attribute: the kernel may be scheduled while its predecessor
// in the stream still runs; all kernels here wait in their prologue.  (Development builds, -DREEF_DEBUG_AIDS, can
// switch it off with REEF_PDL=0.)
static cudaError_t launch_pdl(const void* fn, dim3 grid, dim3 block, void** kargs, uint32_t smem, cudaStream_t st) {
    static int use_pdl = -1;
    if (use_pdl < 0) {
        use_pdl = 1;
#ifdef REEF_DEBUG_AIDS
        const char* v = getenv("REEF_PDL");
        if (v && v[0] == '0') use_pdl = 0;
#endif
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    return cudaLaunchKernelExC(&cfg, fn, kargs);
}

static int check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return REEF_SUCC;
    set_error(std::string(what) + ": " + cudaGetErrorString(e));
    return REEF_FAIL;
}

static void fill_args(const KernelSpec& s, void** args, KTask* t) {
    *t = s.task;
    for (int i = 0; i < s.nargs; i++) t->a[i] = *reinterpret_cast<void**>(args[i]);
    t->err = nullptr;
    if (s.task.family == F_DENSE) tc_error_word(&t->err);   // created by prepare_kernel, looked up here
}

static bool dims_match(const KernelSpec& s, const uint32_t dims[6], uint32_t smem) {
    return dims[0] == s.grid[0] && dims[1] == s.grid[1] && dims[2] == s.grid[2] && dims[3] == s.block[0] &&
           dims[4] == s.block[1] && dims[5] == s.block[2] && smem == s.dyn_smem;
}

static int bind_tc(const KernelSpec& s, void** args) {
    if (!s.tc_cache) s.tc_cache = std::make_shared<TcCache>();
    TcCache& c = *s.tc_cache;
    bool same = c.valid;
    for (int i = 0; i < s.nargs && same; i++) same = c.ptrs[i] == *reinterpret_cast<void**>(args[i]);
    if (!same) {
        void* ptrs[kMaxArgs] = {nullptr};
        for (int i = 0; i < s.nargs; i++) ptrs[i] = *reinterpret_cast<void**>(args[i]);
        int rc;
        if (s.task.family == F_ATTENTION_TC) {
            rc = att_prepare_device();
            if (rc != REEF_SUCC) return rc;
            rc = att_build_params(s.task.p.raw[0], s.task.p.raw[1], s.task.p.raw[3], ptrs, &c.att);
        } else {
            rc = tc_prepare_device();
            if (rc != REEF_SUCC) return rc;
            rc = tc_build_params(s.task.p.conv, s.tc, ptrs, &c.params);
        }
        if (rc != REEF_SUCC) return rc;
        for (int i = 0; i < s.nargs; i++) c.ptrs[i] = ptrs[i];
        c.valid = true;
    }
    return REEF_SUCC;
}

int make_chain(const KernelSpec* const* specs, void*** args, int n, int clusters, TcChain** out) {
    std::vector<const TcParams*> params;
    std::vector<TcPlan> plans;
    for (int i = 0; i < n; i++) {
        if (specs[i]->task.family != F_CONV_TC) {
            set_error("a chain holds tensor-core convolution / matmul kernels only: " + specs[i]->name);
            return REEF_FAIL;
        }
        int rc = bind_tc(*specs[i], args[i]);
        if (rc != REEF_SUCC) return rc;
        params.push_back(&specs[i]->tc_cache->params);
        plans.push_back(specs[i]->tc);
    }
    return chain_create(params, plans, clusters, out);
}

int prepare_kernel(const KernelSpec& s, void** args) {
    prepare_carveout();
    if (is_tc_family(s.task.family)) return bind_tc(s, args);
    return REEF_SUCC;
}

static int launch_tc(const KernelSpec& s, cudaStream_t st, void** args, const int* flag, int* slot, int tile_begin = 0,
                     int tile_count = -1) {
    int rc = bind_tc(s, args);
    if (rc != REEF_SUCC) return rc;
    TcCache& c = *s.tc_cache;
    count_launch();
    if (s.task.family == F_ATTENTION_TC) return att_launch(c.att, st, flag, slot, tile_begin, tile_count);
    return tc_launch(c.params, s.tc, st, flag, slot, tile_begin, tile_count);
}

int launch_plain(const KernelSpec& s, const uint32_t dims[6], uint32_t smem, cudaStream_t st, void** args) {
    if (!dims_match(s, dims, smem)) {
        set_error("launch_params / shared_memory do not match the kernel plan of " + s.name);
        return REEF_OUT_OF_RANGE;
    }
    if (is_tc_family(s.task.family)) return launch_tc(s, st, args, nullptr, nullptr);
    KTask t;
    fill_args(s, args, &t);
    void* kargs[] = {&t};
    cudaError_t e = launch_pdl(plain_fn(t.family), dim3(dims[0], dims[1], dims[2]), dim3(dims[3], dims[4], dims[5]), kargs,
                               smem, st);
    count_launch();
    return check_cuda(e, "cudaLaunchKernel");
}

int launch_be(const KernelSpec& s, const uint32_t dims[6], uint32_t smem, cudaStream_t st, const int* flag,
              int* slot, void** args) {
    if (!dims_match(s, dims, smem)) {
        set_error("launch_params / shared_memory do not match the kernel plan of " + s.name);
        return REEF_OUT_OF_RANGE;
    }
    if (is_tc_family(s.task.family)) return launch_tc(s, st, args, flag, slot);
    KTask t;
    fill_args(s, args, &t);
    void* kargs[] = {&t, (void*)&flag, (void*)&slot};
    cudaError_t e = launch_pdl(be_fn(t.family), dim3(dims[0], dims[1], dims[2]), dim3(dims[3], dims[4], dims[5]), kargs, smem,
                               st);
    count_launch();
    return check_cuda(e, "cudaLaunchKernel(be)");
}

// One padded step.  Two shapes:
//  * both kernels are logical-block families and no separate best-effort stream is given: ONE persistent
//    dispatcher grid on `st` runs the real-time blocks and the best-effort blocks (SM-partitioned);
//  * otherwise (a tensor-core cluster kernel is involved, or `be_st` is given): the real-time kernel runs
//    as its own launch on `st` and the best-effort block range runs beside it on `be_st` — the hardware
//    block scheduler places the best-effort blocks on the SMs the real-time kernel leaves free, the
//    real-time stream having the greater priority.  Best-effort blocks launched here do not read the
//    preempt flag (they were sized to fit beside the real-time kernel) but do count into the task slot.
int launch_dispatch(const KernelSpec* rt, void** rt_args, const KernelSpec* be, void** be_args, int be_off,
                    int be_num, int sm_partition, int occupancy, int num_sms, int* be_slot, int* ctrl, int* be_ctrl,
                    cudaStream_t st, cudaStream_t be_st) {
    if (be == nullptr) be_num = 0;
    const bool rt_tc = rt != nullptr && is_tc_family(rt->task.family);
    const bool be_tc = be_num > 0 && is_tc_family(be->task.family);
    if (occupancy < 1) occupancy = 1;
    if (be_num > 0 && (be_off < 0 || be_off + be_num > be->task.nblocks)) {
        set_error("best-effort block range outside the kernel");
        return REEF_OUT_OF_RANGE;
    }
    const bool split_launch = rt_tc || be_tc || (be_st != nullptr && be_num > 0);

    if (!split_launch) {
        KTask trt, tbe;
        uint32_t smem = 0;
        if (rt != nullptr) {
            fill_args(*rt, rt_args, &trt);
            smem = rt->dyn_smem;
        } else {
            memset(&trt, 0, sizeof(trt));   // nblocks = 0: the real-time phase ends at once
        }
        if (be_num > 0) {
            fill_args(*be, be_args, &tbe);
            if (be->dyn_smem > smem) smem = be->dyn_smem;
        } else {
            memset(&tbe, 0, sizeof(tbe));
        }
        int grid = num_sms * occupancy;
        void* kargs[] = {&trt, &tbe, &be_off, &be_num, &sm_partition, (void*)&be_slot, (void*)&ctrl};
        cudaError_t e = cudaLaunchKernel((const void*)k_dispatch, dim3(grid), dim3(kThreads), kargs, smem, st);
        count_launch();
        return check_cuda(e, "cudaLaunchKernel(dispatch)");
    }

    // real-time part
    if (rt != nullptr) {
        int rc;
        if (rt_tc) {
            rc = launch_tc(*rt, st, rt_args, nullptr, nullptr);
        } else {
            KTask trt, tbe;
            fill_args(*rt, rt_args, &trt);
            memset(&tbe, 0, sizeof(tbe));
            int zero = 0, part = num_sms;
            int* null_slot = nullptr;
            int grid = num_sms * occupancy;
            if (grid > trt.nblocks) grid = trt.nblocks;
            void* kargs[] = {&trt, &tbe, &zero, &zero, &part, (void*)&null_slot, (void*)&ctrl};
            cudaError_t e = cudaLaunchKernel((const void*)k_dispatch, dim3(grid), dim3(kThreads), kargs, rt->dyn_smem, st);
            count_launch();
            rc = check_cuda(e, "cudaLaunchKernel(dispatch rt)");
        }
        if (rc != REEF_SUCC) return rc;
    }
    // best-effort part
    if (be_num > 0) {
        cudaStream_t bs = be_st != nullptr ? be_st : st;
        if (be_tc) {
            const int sp = be->task.family == F_CONV_TC ? be->tc.splits : 1;
            if (be_off % sp != 0 || be_num % sp != 0) {
                set_error("best-effort block range of a cluster kernel must be a multiple of its cluster size");
                return REEF_OUT_OF_RANGE;
            }
            return launch_tc(*be, bs, be_args, nullptr, be_slot, be_off / sp, be_num / sp);
        }
        KTask trt, tbe;
        memset(&trt, 0, sizeof(trt));
        fill_args(*be, be_args, &tbe);
        int part = 0;
        int grid = be_num < num_sms * occupancy ? be_num : num_sms * occupancy;
        // its own control block keeps this grid's tickets apart from the real-time grid's
        int* ctrl2 = be_ctrl != nullptr ? be_ctrl : ctrl;
        if (be_ctrl == nullptr && rt != nullptr) {
            set_error("a separate best-effort launch needs its own control block");
            return REEF_FAIL;
        }
        void* kargs[] = {&trt, &tbe, &be_off, &be_num, &part, (void*)&be_slot, (void*)&ctrl2};
        cudaError_t e = cudaLaunchKernel((const void*)k_dispatch, dim3(grid), dim3(kThreads), kargs, be->dyn_smem, bs);
        count_launch();
        return check_cuda(e, "cudaLaunchKernel(dispatch be)");
    }
    return REEF_SUCC;
}

// ---- dispatcher without any allocation -------------------------------------------------------------
// Ticket blocks for callers that must not allocate: one 256-byte lane per concurrent dispatcher launch, held
// by every GPU that loads this library until the process exits (16 KB).  In host code the array's name is
// only a stand-in for the device object; its device address comes from cudaGetSymbolAddress, once per device.
constexpr int kStaticLanes = REEF_STATIC_DISPATCH_LANES;
constexpr int kLaneInts = 64;   // 256 bytes apart: lanes never share a cache line
static __device__ __align__(256) int g_static_dispatch_ctrl[kStaticLanes * kLaneInts];
static int* g_static_ctrl_ptr[16] = {nullptr};

int launch_dispatch_static(const KernelSpec* rt, void** rt_args, const KernelSpec* be, void** be_args, int be_off,
                           int be_num, int sm_partition, int occupancy, int num_sms, int* be_slot, int lane,
                           cudaStream_t st) {
    if (lane < 0 || lane >= kStaticLanes) {
        set_error("reef_dispatch_static: lane " + std::to_string(lane) + " is beyond the " +
                  std::to_string(kStaticLanes) + " statically reserved lanes (REEF_STATIC_DISPATCH_LANES)");
        return REEF_OUT_OF_RANGE;
    }
    if (rt == nullptr && be == nullptr) return REEF_FAIL;
    if (be == nullptr) be_num = 0;
    if ((rt != nullptr && is_tc_family(rt->task.family)) || (be_num > 0 && is_tc_family(be->task.family))) {
        set_error("reef_dispatch_static hosts logical-block kernels only (a tensor-core cluster kernel was given)");
        return REEF_FAIL;
    }
    if (be_num > 0 && (be_off < 0 || be_off + be_num > be->task.nblocks)) {
        set_error("best-effort block range outside the kernel");
        return REEF_OUT_OF_RANGE;
    }
    int dev = 0;
    if (check_cuda(cudaGetDevice(&dev), "cudaGetDevice") != REEF_SUCC) return REEF_FAIL;
    if (dev < 0 || dev >= 16) {
        set_error("reef_dispatch_static: device ordinal out of range");
        return REEF_OUT_OF_RANGE;
    }
    if (g_static_ctrl_ptr[dev] == nullptr) {
        // set-up, once per device, with that device current.  The cache is filled without a lock: two threads that
        // both find it empty ask the runtime for the same symbol of the same device and store the same address, so
        // whichever store lands last changes nothing (a pointer-sized aligned store is not torn on the host).
        void* p = nullptr;
        int rc = check_cuda(cudaGetSymbolAddress(&p, g_static_dispatch_ctrl), "cudaGetSymbolAddress(static dispatch lanes)");
        if (rc != REEF_SUCC) return rc;
        g_static_ctrl_ptr[dev] = static_cast<int*>(p);
    }
    int* ctrl = g_static_ctrl_ptr[dev] + lane * kLaneInts;
    // the lane keeps whatever the previous launch left (zero after a launch that drained): start from zero
    int rc = check_cuda(cudaMemsetAsync(ctrl, 0, 16, st), "cudaMemsetAsync(static dispatch lane)");
    if (rc != REEF_SUCC) return rc;
    KTask trt, tbe;
    uint32_t smem = 0;
    if (rt != nullptr) {
        fill_args(*rt, rt_args, &trt);
        smem = rt->dyn_smem;
    } else {
        memset(&trt, 0, sizeof(trt));
    }
    if (be_num > 0) {
        fill_args(*be, be_args, &tbe);
        if (be->dyn_smem > smem) smem = be->dyn_smem;
    } else {
        memset(&tbe, 0, sizeof(tbe));
    }
    if (occupancy < 1) occupancy = 1;
    int grid = num_sms * occupancy;
    void* kargs[] = {&trt, &tbe, &be_off, &be_num, &sm_partition, (void*)&be_slot, (void*)&ctrl};
    cudaError_t e = cudaLaunchKernel((const void*)k_dispatch, dim3(grid), dim3(kThreads), kargs, smem, st);
    count_launch();
    return check_cuda(e, "cudaLaunchKernel(dispatch, static lane)");
}

int kernel_attrs(const KernelSpec& s, reef_kernel_attrs_t* out) {
    cudaFuncAttributes fa;
    int threads = s.block[0] * s.block[1] * s.block[2];
    int occ = 0;
    int rc;
    if (s.task.family == F_CONV_TC) {
        rc = tc_func_attrs(s.tc, &fa, &occ);
        if (rc != REEF_SUCC) return rc;
    } else if (s.task.family == F_ATTENTION_TC) {
        rc = att_func_attrs(&fa, &occ);
        if (rc != REEF_SUCC) return rc;
    } else {
        const void* fn = plain_fn(s.task.family);
        rc = check_cuda(cudaFuncGetAttributes(&fa, fn), "cudaFuncGetAttributes");
        if (rc != REEF_SUCC) return rc;
        rc = check_cuda(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, fn, threads, s.dyn_smem),
                        "cudaOccupancyMaxActiveBlocksPerMultiprocessor");
        if (rc != REEF_SUCC) return rc;
    }
    out->num_blocks = s.task.nblocks;
    out->threads = threads;
    out->regs_per_thread = fa.numRegs;
    out->static_smem = (int)fa.sharedSizeBytes;
    out->dyn_smem = (int)s.dyn_smem;
    out->local_mem = (int)fa.localSizeBytes;
    out->max_blocks_per_sm = occ;
    out->flops = s.flops;
    out->bytes = s.bytes;
    out->tensor_core = s.tensor_core;
    out->cluster = s.task.family == F_CONV_TC ? s.tc.splits : 1;
    out->chainable = s.task.family == F_CONV_TC ? 1 : 0;
    return REEF_SUCC;
}

int dispatch_occupancy(uint32_t smem, int* occ) {
    return check_cuda(cudaOccupancyMaxActiveBlocksPerMultiprocessor(occ, (const void*)k_dispatch, kThreads, smem),
                      "cudaOccupancyMaxActiveBlocksPerMultiprocessor(dispatch)");
}

}  // namespace reef
