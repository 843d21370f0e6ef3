// Point query kernels: query_vertical and its backward.
//
// Replaces query_single_kernel / query_single_kernel_backward of the
// reference (svox/csrc/svox_kernel.cu:56-78).  The reference copies each
// point's K-float record with a per-thread scalar loop, so every warp
// instruction touches 32 different cache lines on both sides.  Here a thread
// still descends for its own point, but the records of a warp's 32 points
// are then moved by the whole warp: lane l handles elements l, l+32, ... of
// the warp's contiguous (32, K) output block, so stores are fully coalesced
// and loads walk each record contiguously.
//
// HBM roofline per point: 12 B in + K*4 B gathered + K*4 B written + 8 B id
// (+ one 4-B child entry per level below the jump table, L2 resident).
#pragma once

#include "common.cuh"

namespace svoxb {

constexpr int kQueryBlock = 256;

struct TreeArgs {
    const float* __restrict__ data;
    const int32_t* __restrict__ child;
    const float* __restrict__ offset;
    const float* __restrict__ scaling;
    int64_t M;
    int32_t N;
    int32_t K;
    float* weight_accum;      // forward render only (null: off)
    int32_t weight_accum_max;
    int32_t extra_cols;       // row length of `extra`
    const float* __restrict__ extra;   // lobe parameters of the SG / ASG colour bases
};

static inline TreeArgs tree_args(const svoxb_tree* t) {
    return TreeArgs{t->data, t->child, t->offset, t->scaling, t->M, t->N, t->K,
                    t->weight_accum, t->weight_accum_max, t->extra_cols, t->extra_data};
}

// One sample's weight into the accumulator of its leaf (svox/csrc/rt_kernel.cu:298-304).
// Weights are >= 0 unless the density is negative; for those the maximum goes through a
// compare-and-swap like the reference's (svox/csrc/include/common.cuh:152-161).
__device__ __forceinline__ void accumulate_weight(const TreeArgs& tr, int64_t slot, float w) {
    float* p = tr.weight_accum + slot;
    if (!tr.weight_accum_max) {
        atomicAdd(p, w);
    } else if (w >= 0.f) {
        // non-negative floats order like their bit patterns; the buffer starts at +0
        if (__float_as_int(*reinterpret_cast<volatile float*>(p)) < __float_as_int(w))
            atomicMax(reinterpret_cast<int*>(p), __float_as_int(w));
    } else {
        unsigned* u = reinterpret_cast<unsigned*>(p);
        unsigned old = *u, assumed;
        int guard = 0;
        do {
            assumed = old;
            old = atomicCAS(u, assumed, __float_as_uint(fmaxf(w, __uint_as_float(assumed))));
        } while (old != assumed && ++guard < 1024);
    }
}

__device__ __forceinline__ int64_t locate_point(const TreeArgs& tr, const TopTable& top,
                                                const float* __restrict__ pts, int64_t i) {
    const float px = to_tree(__ldg(pts + 3 * i + 0), __ldg(tr.offset + 0), __ldg(tr.scaling + 0));
    const float py = to_tree(__ldg(pts + 3 * i + 1), __ldg(tr.offset + 1), __ldg(tr.scaling + 1));
    const float pz = to_tree(__ldg(pts + 3 * i + 2), __ldg(tr.offset + 2), __ldg(tr.scaling + 2));
    LeafHit hit;
    const bool ok = (tr.N == 2) ? descend2(tr.child, tr.M, top, px, py, pz, hit)
                                : descendN(tr.child, tr.M, tr.N, px, py, pz, hit);
    return ok ? hit.slot : -1;
}

// MODE 0: copy records out (forward).  MODE 1: scatter-add rows in (backward).
// MODE 2: overwrite the first Kg floats of each point's record with its row of `grad_out`
// (assign_single_kernel, svox/csrc/svox_kernel.cu:80-89; points that share a leaf race, as in
// the reference).
template <int MODE>
__global__ void __launch_bounds__(kQueryBlock)
query_kernel(TreeArgs tr, TopTable top, const float* __restrict__ pts, int64_t Q,
             float* __restrict__ values_out, int64_t* __restrict__ ids_out,
             const float* __restrict__ grad_out, float* __restrict__ grad_data, int Kg) {
    const int64_t i = (int64_t)blockIdx.x * kQueryBlock + threadIdx.x;
    const int lane = threadIdx.x & 31;
    int64_t slot = -1;
    if (i < Q) {
        slot = locate_point(tr, top, pts, i);
        if (MODE == 0 && ids_out != nullptr && slot >= 0) ids_out[i] = slot;
    }
    if (MODE == 0 && values_out == nullptr) return;

    // Warp-cooperative record move.  `wb` is the first point of this warp.
    const int64_t wb = i - lane;
    if (wb >= Q) return;
    const int K = (MODE == 0) ? tr.K : Kg;
    const int nvalid = (int)((Q - wb) < 32 ? (Q - wb) : 32);
    if (MODE == 2) {
        // lanes walk the warp's (nvalid, Kg) block of rows in order: coalesced reads, and
        // writes that are contiguous within each record
        const int total = nvalid * K;
        int p = 0, e = lane;
        while (e >= K) { e -= K; ++p; }
        for (int base = 0; base < total; base += 32) {        // warp-uniform trip count
            const int j = base + lane;
            const int64_t s = __shfl_sync(0xffffffffu, slot, p < nvalid ? p : nvalid - 1);
            if (j < total && s >= 0) grad_data[s * tr.K + e] = __ldg(grad_out + wb * K + j);
            e += 32;
            while (e >= K) { e -= K; ++p; }
        }
        return;
    }
    if (MODE == 1) {
        // Backward: add row p of the upstream gradient into the record of point p's leaf.  A
        // record is K floats at 4-byte alignment, so each is cut into at most 3 single floats
        // up to the next 16-byte boundary, whole 16-byte words (one vector reduction each,
        // a quarter of the requests of scalar atomics) and at most 3 single floats behind
        // them.  Lanes take these pieces of the warp's 32 records round robin.
        const int per_point = 6 + (K >> 2);        // 3 head + K/4 word + 3 tail places
        const bool vec_ok = (reinterpret_cast<uintptr_t>(grad_data) & 15) == 0;
        const int n_units = nvalid * per_point;
        for (int base = 0; base < n_units; base += 32) {       // warp-uniform trip count
            const int u = base + lane;
            const int p = u < n_units ? u / per_point : 0, j = u - p * per_point;
            const int64_t s = __shfl_sync(0xffffffffu, slot, p);
            if (u >= n_units || s < 0) continue;
            const int64_t first = s * K;                       // destination, in floats
            int head = vec_ok ? (int)((4 - (first & 3)) & 3) : 0;
            if (head > K) head = K;
            const int words = vec_ok ? (K - head) >> 2 : 0;
            const float* __restrict__ src = grad_out + (wb + p) * K;
            if (j < 3) {
                if (j < head && j < K) atomicAdd(grad_data + first + j, __ldg(src + j));
            } else if (j < 3 + (K >> 2)) {
                const int w = j - 3;
                if (w < words) {
                    const int e = head + 4 * w;
                    red_add_v4(grad_data + first + e, __ldg(src + e), __ldg(src + e + 1),
                               __ldg(src + e + 2), __ldg(src + e + 3));
                } else if (!vec_ok) {                           // unaligned buffer: scalars
                    for (int e = 4 * w; e < 4 * w + 4 && e < K; ++e)
                        atomicAdd(grad_data + first + e, __ldg(src + e));
                }
            } else {
                const int e = (vec_ok ? head + 4 * words : 4 * (K >> 2)) + (j - 3 - (K >> 2));
                if (e < K) atomicAdd(grad_data + first + e, __ldg(src + e));
            }
        }
        return;
    }
    const int total = nvalid * K;
    int p = 0, e = lane;  // element j = p*K + e of the warp's (nvalid, K) block
    while (e >= K) { e -= K; ++p; }
    // Batches of kBatch steps: all loads of a batch are issued before the first store, so that
    // a warp keeps kBatch 128-byte requests in flight (the path is bound by memory latency).
    constexpr int kBatch = 8;
    for (int base = 0; base < total; base += 32 * kBatch) {
        float v[kBatch];
        int64_t dst[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int j = base + 32 * u + lane;
            const int src_lane = p < nvalid ? p : nvalid - 1;
            const int64_t s = __shfl_sync(0xffffffffu, slot, src_lane);
            dst[u] = -1;
            v[u] = 0.f;
            if (j < total && s >= 0) {
                v[u] = __ldg(tr.data + s * K + e);
                dst[u] = wb * K + j;
            }
            e += 32;
            while (e >= K) { e -= K; ++p; }
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u)
            if (dst[u] >= 0) values_out[dst[u]] = v[u];
    }
}

// calc_corner_kernel (svox/csrc/svox_kernel.cu:91-115): the lower corner of cell (node, i, j, k)
// in tree-local coordinates, by walking parent_depth up to the root with the reference's
// add-then-divide per level (for N = 3 the roundings of that order are part of the result).
// parent_depth is (M, 2): packed index of the parent cell, depth.
__global__ void calc_corners_kernel(const int32_t* __restrict__ parent_depth, int64_t M, int N,
                                    const int64_t* __restrict__ indexer, int64_t Q,
                                    float* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= Q) return;
    int64_t node = indexer[4 * i];
    int c[3] = {(int)indexer[4 * i + 1], (int)indexer[4 * i + 2], (int)indexer[4 * i + 3]};
    float r[3] = {0.f, 0.f, 0.f};
    const float fn = (float)N;
    for (int level = 0;; ++level) {
        if (node < 0 || node >= M || level > 64) {   // not a tree: reported, never followed
            report(SVOXB_ERR_TREE);
            break;
        }
#pragma unroll
        for (int a = 0; a < 3; ++a) r[a] = __fdiv_rn(__fadd_rn(r[a], (float)c[a]), fn);
        if (node == 0) break;
        int32_t packed = __ldg(parent_depth + 2 * node);
        for (int a = 2; a >= 0; --a) {
            c[a] = packed % N;
            packed /= N;
        }
        node = packed;
    }
    out[3 * i + 0] = r[0];
    out[3 * i + 1] = r[1];
    out[3 * i + 2] = r[2];
}

static int launch_query(int mode, const svoxb_tree* tree, const float* indices, int64_t Q,
                        float* values_out, int64_t* ids_out, const float* grad_out,
                        float* grad_data, int Kg, cudaStream_t stream) {
    if (Q == 0) return SVOXB_OK;
    if (!indices) return SVOXB_ERR_NULL;
    if ((Q + kQueryBlock - 1) / kQueryBlock > 0x7fffffffLL) return SVOXB_ERR_TOO_LARGE;
    TopScratch top;
    int st = top.build(tree, 7, stream);
    if (st) return st;
    const TopTable tt{top.cells, top.level};
    const unsigned grid = (unsigned)((Q + kQueryBlock - 1) / kQueryBlock);
    if (mode == 0)
        query_kernel<0><<<grid, kQueryBlock, 0, stream>>>(tree_args(tree), tt, indices, Q,
                                                          values_out, ids_out, nullptr,
                                                          nullptr, 0);
    else if (mode == 2)
        query_kernel<2><<<grid, kQueryBlock, 0, stream>>>(tree_args(tree), tt, indices, Q,
                                                          nullptr, nullptr, grad_out,
                                                          grad_data, Kg);
    else
        query_kernel<1><<<grid, kQueryBlock, 0, stream>>>(tree_args(tree), tt, indices, Q,
                                                          nullptr, nullptr, grad_out,
                                                          grad_data, Kg);
    SVOXB_CUDA(cudaGetLastError());
    return SVOXB_OK;
}

}  // namespace svoxb
