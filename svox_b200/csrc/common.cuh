// Shared device code of the B200 svox kernels: coordinate transform, octree
// descent, device status word, launch helpers.
//
// Arithmetic rule: every float operation that decides WHERE a ray or a
// point is (positions, t, cell sizes) is written with explicit-rounding
// intrinsics (__fmul_rn, __fadd_rn, __fmaf_rn, ...), which the compiler never
// re-associates or contracts.  The fused/unfused choice per site is fixed in
// arith.cuh to the one that reproduces the compiled reference bit for bit.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/svox_b200.h"
#include "arith.cuh"

namespace svoxb {

// Per-device anomaly word (see svoxb_device_status).
__device__ int g_status = 0;  // the library is a single translation unit

__device__ __forceinline__ void report(int code) { atomicMax(&g_status, code); }

// 16-byte vector reduction into global memory (addr 16-byte aligned).
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b),
                 "f"(c), "f"(d)
                 : "memory");
}

constexpr int kMaxDescent = 40;  // levels; far beyond any float-resolvable depth

// clamp_coord of the reference (svox/csrc/include/common.cuh:36-41): the bound
// float(1) - 1e-6 is a double there and the clamped value is rounded back to
// float.  For a float q that is exactly min(q, float(1.0 - 1e-6)).
__device__ __forceinline__ float clamp01(float q) {
    const float hi = (float)(1.0 - 1e-6);
    return fmaxf(0.0f, fminf(hi, q));
}

// transform_coord (svox/csrc/include/common.cuh:43-50)
__device__ __forceinline__ float to_tree(float q, float offset, float scaling) {
    return mad_site<FC_TRANSFORM>(scaling, q, offset);
}

struct LeafHit {
    int64_t slot;   // node * N^3 + u*N^2 + v*N + w  (the reference's packed id)
    float cube_sz;  // cells of the leaf's size per unit side (N^(depth+1))
    float fx, fy, fz;  // fractional position inside the leaf
};

// Top-of-tree jump table for N = 2: entry (ix,iy,iz) of the 2^L cube holds the
// id of the node whose children are the level-(L+1) cells at that place, or
// -1 if the tree ends above level L there.
struct TopTable {
    const int32_t* cells;  // shared or global memory
    int level;             // L (0 = no table)
    const int32_t* bricks = nullptr;  // queue kernels only: see render_queue.cuh
};

// Descent of query_single_from_root (svox/csrc/include/common.cuh:52-90) for
// N = 2.  Multiplying by 2, taking the floor and subtracting are exact in
// float, so the fractional position and the cell size do not depend on how
// the leaf is found; only the node id chain has to be followed.
__device__ __forceinline__ bool descend2(const int32_t* __restrict__ child, int64_t M,
                                         const TopTable& top, float px, float py, float pz,
                                         LeafHit& hit) {
    float x = clamp01(px), y = clamp01(py), z = clamp01(pz);
    int64_t node = 0;
    float cube = 1.0f;
    if (top.level > 0) {
        const float s = (float)(1 << top.level);
        const float xs = x * s, ys = y * s, zs = z * s;  // exact (power of two)
        const int ix = (int)xs, iy = (int)ys, iz = (int)zs;
        const int32_t e = top.cells[((((ix << top.level) + iy) << top.level) + iz)];
        if (e >= 0) {
            node = e;
            cube = s;
            x = xs - (float)ix; y = ys - (float)iy; z = zs - (float)iz;
        }
    }
#pragma unroll 1
    for (int lvl = 0; lvl < kMaxDescent; ++lvl) {
        x *= 2.0f; y *= 2.0f; z *= 2.0f;
        const int u = (int)x, v = (int)y, w = (int)z;  // x >= 0: truncation == floor
        x -= (float)u; y -= (float)v; z -= (float)w;
        cube *= 2.0f;
        const int64_t slot = node * 8 + (u * 4 + v * 2 + w);
        const int32_t skip = __ldg(child + slot);
        if (skip == 0) {
            hit.slot = slot; hit.cube_sz = cube; hit.fx = x; hit.fy = y; hit.fz = z;
            return true;
        }
        node += skip;
        if (node < 0 || node >= M) break;
    }
    report(SVOXB_ERR_TREE);
    return false;
}

// Same descent for any branching factor N (no table; N is small).
__device__ __forceinline__ bool descendN(const int32_t* __restrict__ child, int64_t M, int N,
                                         float px, float py, float pz, LeafHit& hit) {
    float x = clamp01(px), y = clamp01(py), z = clamp01(pz);
    const float Nf = (float)N;
    const int n3 = N * N * N;
    int64_t node = 0;
    float cube = 1.0f;
#pragma unroll 1
    for (int lvl = 0; lvl < kMaxDescent; ++lvl) {
        x = __fmul_rn(x, Nf); y = __fmul_rn(y, Nf); z = __fmul_rn(z, Nf);
        const float fu = floorf(x), fv = floorf(y), fw = floorf(z);
        x = __fsub_rn(x, fu); y = __fsub_rn(y, fv); z = __fsub_rn(z, fw);
        cube = __fmul_rn(cube, Nf);
        const int64_t slot = node * n3 + ((int)fu * N * N + (int)fv * N + (int)fw);
        const int32_t skip = __ldg(child + slot);
        if (skip == 0) {
            hit.slot = slot; hit.cube_sz = cube; hit.fx = x; hit.fy = y; hit.fz = z;
            return true;
        }
        node += skip;
        if (node < 0 || node >= M) break;
    }
    report(SVOXB_ERR_TREE);
    return false;
}

// ---------------------------------------------------------------------------
// Host helpers
int set_cuda_error(cudaError_t e);  // records the text, returns SVOXB_ERR_CUDA
int sm_count();                     // multiprocessors of the current device

#define SVOXB_CUDA(call)                                              \
    do {                                                              \
        cudaError_t e__ = (call);                                     \
        if (e__ != cudaSuccess) return svoxb::set_cuda_error(e__);    \
    } while (0)

int validate_tree(const svoxb_tree* t);
int keep_pool_cached();  // stream-ordered pool keeps freed scratch for the next call

// Scratch jump table of one call: chosen level, device buffer from the
// stream-ordered pool (released by the destructor on the same stream).
struct TopScratch {
    int32_t* cells = nullptr;
    int level = 0;
    cudaStream_t stream = nullptr;
    int build(const svoxb_tree* t, int max_level, cudaStream_t s);
    ~TopScratch() { if (cells) cudaFreeAsync(cells, stream); }
};

// Queue kernels: lanes that must be idle before rays are loaded.  Measured on the training
// step's logged forward: 1 to 3 are level, 4 costs 1 %, 8 3 %, 16 11 %.
constexpr int kRefillBatch = 2;
// Replay scatter: 1 = packets evict-first, 2 = gradient evict-last.  Measured (backward of the
// training step): 3 -> 2.83 ms, 2 -> 2.78, 0 -> 2.79, 1 -> 2.89.
constexpr int kReplayHints = 2;

// The two switches the tests flip to show that an index or a bin size changes no result
// (svoxb_test_knob).
struct Tuning {
    int replay_bin_mb = 32;  // gradient MB one replay bin spans (measured: 16 -> 3.05 ms of
                             // backward per training step, 32 and 64 -> 2.94, 128 -> 3.86)
    int render_bricks = 1;   // queue kernels: bricks below the leaf table
};
extern Tuning g_tuning;
extern int g_reserved_sms;

}  // namespace svoxb
