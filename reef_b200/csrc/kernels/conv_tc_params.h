// Parameters of the tcgen05 convolution kernel shared by its host planner and the registry
// (the kernel itself lives in conv_tc.cuh and is compiled once, in conv_tc.cu).
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace reef {

constexpr int TC_MAX_STAGES = 8;      // shared-memory ring depth is chosen per launch, up to this
constexpr int TC_BM = 128;            // output channels per tile (TMEM lanes)
constexpr int TC_BK = 32;             // fp32 elements per K block = 128 bytes
constexpr int TC_A_BYTES = TC_BM * TC_BK * 4;
constexpr int TC_THREADS = 256;
constexpr int TC_MAX_SPLITS = 8;
// Dynamic shared memory of one CTA at most: two CTAs (each + 1 KB the hardware reserves) fit the 228 KB of an SM
constexpr int TC_SMEM_CAP = 112 * 1024;

struct TcParams {
    CUtensorMap tm_w;        // weights  dims (Cin, taps, Cout), box (32, 1, 128)
    CUtensorMap tm_x[4];     // activations, one per stride sub-lattice (ry*s + rx)
    float* out;
    const float* res;
    const float* bias;
    const float* gamma;
    const float* beta;
    float* out2;             // second output [P][Cout] = relu(out + bias2), else nullptr
    const float* bias2;
    const int* preempt_flag; // best-effort flavour, else nullptr
    int* task_slot;
    int* error_word;         // device word set non-zero when a bounded wait expired
    long long* trace;        // optional: 16 SM-clock stamps of block (0,0) (phase trace), else nullptr
    unsigned long long* stamps;   // optional: {first flag observation, last leave} in %globaltimer ns, else nullptr
    int co, ci, ptot;
    int ocs, ooff;
    int spatial;             // 0: flat [P][C] view, tile = n_valid consecutive pixels; 1: tile = rows x Wo
    int wo, rows;            // spatial: output width, rows per tile
    int xsplit, xw;          // spatial: a row is cut into xsplit tiles of xw pixels (rows == 1), else xsplit == 1
    int n_valid;             // pixels per tile
    int n_mma;               // UMMA N (multiple of 16, >= n_valid)
    int tmem_cols;           // power of two >= n_mma
    int kh, kw, stride, ph, pw;
    int cblocks;             // Cin / 32
    int kb_total, kb_per_split, splits;
    int ep;                  // EP_* bits
    int b_bytes;             // bytes TMA delivers per B stage (box size)
    int stages;              // ring depth of this launch
    int region_bytes;        // data region of shared memory: max(stage ring, staging tile + exchange area)
    int recv_offset_floats;  // exchange area offset inside the region, in floats
    int cpc_max;             // pixel rows a rank finishes at most = ceil(n_valid / splits)
    int n_tiles;             // pixel tiles; linear tile index = tile_m * n_tiles + tile_n
    int tile_begin;          // first tile of this launch (dynamic kernel padding launches sub-ranges)
    unsigned cb_magic;       // ceil(2^32 / cblocks): tap = umulhi(kb, cb_magic) without an integer division
    signed char tap_map[64]; // per filter tap (ky*kw + kx): index of the sub-lattice tensor map ...
    signed char tap_qx[64];  // ... and the tap's offset on that sub-lattice, so that the input coordinate
    signed char tap_qy[64];  //     stride*x + kx - pw becomes (x + qx) on map (ry*stride + rx)
    int pdl;                 // programmatic dependent launch: weights are fetched before the grid dependency wait
};

}  // namespace reef
