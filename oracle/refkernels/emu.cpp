// Runs a GPU kernel of the reference's generated sources on the CPU: one ucontext fiber per GPU thread, blocks one
// after the other, __syncthreads() as a yield that lets every fiber of the block reach the same barrier.
// TEST INFRASTRUCTURE ONLY (see hip/hip_runtime.h in this directory).  Built into oracle/_ref/libref_<model>.so
// together with the reference source it serves; exported entry point: reef_ref_launch().
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <ucontext.h>

#include <vector>

#include "hip/hip_runtime.h"

reef_emu_dim3 threadIdx, blockIdx, blockDim, gridDim;

namespace {

const size_t kStack = 256 * 1024;

struct Fiber {
    ucontext_t ctx;
    char* stack;
    bool done;
    reef_emu_dim3 tid;
    int linear;
};

ucontext_t g_main;
std::vector<Fiber> g_fibers;
int g_cur = -1;
void* g_fn = nullptr;
void** g_args = nullptr;
int g_nargs = 0;

typedef void (*fn1)(void*);
typedef void (*fn2)(void*, void*);
typedef void (*fn3)(void*, void*, void*);
typedef void (*fn4)(void*, void*, void*, void*);
typedef void (*fn5)(void*, void*, void*, void*, void*);
typedef void (*fn6)(void*, void*, void*, void*, void*, void*);
typedef void (*fn7)(void*, void*, void*, void*, void*, void*, void*);
typedef void (*fn8)(void*, void*, void*, void*, void*, void*, void*, void*);

void trampoline() {
    void** a = g_args;
    switch (g_nargs) {
        case 1: ((fn1)g_fn)(a[0]); break;
        case 2: ((fn2)g_fn)(a[0], a[1]); break;
        case 3: ((fn3)g_fn)(a[0], a[1], a[2]); break;
        case 4: ((fn4)g_fn)(a[0], a[1], a[2], a[3]); break;
        case 5: ((fn5)g_fn)(a[0], a[1], a[2], a[3], a[4]); break;
        case 6: ((fn6)g_fn)(a[0], a[1], a[2], a[3], a[4], a[5]); break;
        case 7: ((fn7)g_fn)(a[0], a[1], a[2], a[3], a[4], a[5], a[6]); break;
        case 8: ((fn8)g_fn)(a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7]); break;
        default: break;
    }
    g_fibers[g_cur].done = true;
    // returning resumes uc_link = the scheduler
}

}  // namespace

// yield to the scheduler; it resumes the other live fibers of the block and comes back
static void yield_fiber() {
    Fiber& f = g_fibers[g_cur];
    swapcontext(&f.ctx, &g_main);
}

extern "C" void reef_emu_yield(void) { yield_fiber(); }

// __syncthreads(): a counting barrier over the fibers of the block that have not finished
static int g_live = 0, g_arrived = 0;
static unsigned g_generation = 0;
static int g_error = 0;
extern "C" void reef_emu_barrier(void) {
    const unsigned gen = g_generation;
    if (++g_arrived >= g_live) {
        g_arrived = 0;
        g_generation++;
        return;
    }
    while (g_generation == gen) yield_fiber();
}

extern "C" int reef_emu_lane(void) { return g_fibers[g_cur].linear & 63; }

// ds_bpermute: lane L receives the value that lane (byte_addr / 4) % 64 of its wavefront passed to the SAME
// instruction.  The hardware runs the 64 lanes in lock step; here every lane logs what it passed per call site and
// per invocation of that site, and a reader yields until its source lane has logged the same invocation.  Keyed by
// call site, lanes that skip a conditional call (the generated softmax permutes under a per-lane bound check,
// resnet152.cu:805-809) do not shift the bookkeeping of the unconditional reductions around it.
static const int kSites = 96, kInv = 64, kLanes = 256;
static float* g_log = nullptr;          // [site][invocation][thread]
static unsigned short* g_count = nullptr;   // [site][thread]
extern "C" float reef_emu_bpermute_site(int site, int byte_addr, float v) {
    const int lin = g_fibers[g_cur].linear, wave = lin >> 6;
    const int src = wave * 64 + ((byte_addr >> 2) & 63);
    if (site < 0 || site >= kSites || lin >= kLanes || src >= kLanes) {
        g_error = 1;
        return v;
    }
    const int n = g_count[site * kLanes + lin];
    if (n >= kInv) {
        g_error = 1;
        return v;
    }
    g_log[((size_t)site * kInv + n) * kLanes + lin] = v;
    g_count[site * kLanes + lin] = (unsigned short)(n + 1);
    if (src == lin) return v;
    for (int spin = 0; g_count[site * kLanes + src] <= n; spin++) {
        if (spin > 100000) {   // the source lane never executes this instruction: not lock-step code
            g_error = 1;
            return v;
        }
        yield_fiber();
    }
    return g_log[((size_t)site * kInv + n) * kLanes + src];
}

// Launches kernel `name` (resolved in this shared object) over grid x block; args = nargs device-style pointers.
// Returns 0, or -1 when the kernel is unknown, -2 for an unsupported shape.
extern "C" __attribute__((visibility("default"))) int reef_ref_launch(const char* name, const int dims[6], void** args, int nargs) {
    void* self = dlopen(nullptr, RTLD_NOW);
    Dl_info info;
    void* fn = nullptr;
    if (dladdr((void*)&reef_ref_launch, &info) && info.dli_fname) {
        void* h = dlopen(info.dli_fname, RTLD_NOW | RTLD_NOLOAD);
        if (h) fn = dlsym(h, name);
    }
    if (!fn && self) fn = dlsym(self, name);
    if (!fn) return -1;
    const int nthreads = dims[3] * dims[4] * dims[5];
    if (nthreads <= 0 || nthreads > 4096 || nargs < 1 || nargs > 8) return -2;
    if (!g_log) {
        g_log = (float*)malloc(sizeof(float) * (size_t)kSites * kInv * kLanes);
        g_count = (unsigned short*)malloc(sizeof(unsigned short) * kSites * kLanes);
    }
    g_error = 0;
    g_fn = fn;
    g_args = args;
    g_nargs = nargs;
    gridDim = {(unsigned)dims[0], (unsigned)dims[1], (unsigned)dims[2]};
    blockDim = {(unsigned)dims[3], (unsigned)dims[4], (unsigned)dims[5]};
    if ((int)g_fibers.size() < nthreads) {
        size_t old = g_fibers.size();
        g_fibers.resize(nthreads);
        for (size_t i = old; i < g_fibers.size(); i++) g_fibers[i].stack = (char*)malloc(kStack);
    }
    for (int bz = 0; bz < dims[2]; bz++)
        for (int by = 0; by < dims[1]; by++)
            for (int bx = 0; bx < dims[0]; bx++) {
                int t = 0;
                for (int tz = 0; tz < dims[5]; tz++)
                    for (int ty = 0; ty < dims[4]; ty++)
                        for (int tx = 0; tx < dims[3]; tx++, t++) {
                            Fiber& f = g_fibers[t];
                            getcontext(&f.ctx);
                            f.ctx.uc_stack.ss_sp = f.stack;
                            f.ctx.uc_stack.ss_size = kStack;
                            f.ctx.uc_link = &g_main;
                            f.done = false;
                            f.tid = {(unsigned)tx, (unsigned)ty, (unsigned)tz};
                            f.linear = t;
                            makecontext(&f.ctx, trampoline, 0);
                        }
                g_live = nthreads;
                g_arrived = 0;
                if (g_count) memset(g_count, 0, sizeof(unsigned short) * kSites * kLanes);
                while (g_live > 0) {   // one pass = every live fiber runs until it yields (or to its end)
                    for (int i = 0; i < nthreads; i++) {
                        Fiber& f = g_fibers[i];
                        if (f.done) continue;
                        g_cur = i;
                        threadIdx = f.tid;
                        blockIdx = {(unsigned)bx, (unsigned)by, (unsigned)bz};
                        swapcontext(&g_main, &f.ctx);
                        if (f.done) {
                            g_live--;
                            if (g_live > 0 && g_arrived >= g_live) {   // the others all wait at a barrier: release it
                                g_arrived = 0;
                                g_generation++;
                            }
                        }
                    }
                }
            }
    return g_error ? -3 : 0;
}
