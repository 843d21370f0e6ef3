// Host-side helpers shared by the entry points: error text, validation, the
// per-call top-of-tree jump table.
#pragma once

#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace svoxb {

Tuning g_tuning;
int g_reserved_sms = 0;  // multiprocessors the persistent grids leave without a block

static thread_local char t_cuda_error[256] = "";

int set_cuda_error(cudaError_t e) {
    snprintf(t_cuda_error, sizeof t_cuda_error, "%s: %s", cudaGetErrorName(e),
             cudaGetErrorString(e));
    return SVOXB_ERR_CUDA;
}

int sm_count() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 148;
    return n > 0 ? n : 148;
}

int validate_tree(const svoxb_tree* t) {
    if (!t || !t->data || !t->child || !t->offset || !t->scaling) return SVOXB_ERR_NULL;
    if (t->M < 1 || t->N < 2 || t->N > 16 || t->K < 1) return SVOXB_ERR_SHAPE;
    return SVOXB_OK;
}

__global__ void build_top_kernel(const int32_t* __restrict__ child, int64_t M, int L,
                                 int32_t* __restrict__ cells) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (1 << (3 * L))) return;
    const int S = (1 << L) - 1;
    const int iz = idx & S, iy = (idx >> L) & S, ix = idx >> (2 * L);
    int64_t node = 0;
    for (int l = L - 1; l >= 0; --l) {
        const int u = (ix >> l) & 1, v = (iy >> l) & 1, w = (iz >> l) & 1;
        const int32_t skip = child[node * 8 + (u * 4 + v * 2 + w)];
        if (skip == 0) { node = -1; break; }
        node += skip;
        if (node < 0 || node >= M) { node = -1; break; }
    }
    cells[idx] = (int32_t)node;
}

// Level L needs the complete top of the tree: 1 + 8 + ... + 8^L nodes.
static int auto_top_level(int64_t M, int max_level) {
    int L = 0;
    int64_t need = 1, pw = 1;
    while (L < max_level) {
        pw *= 8;
        if (need + pw > M) break;
        need += pw;
        ++L;
    }
    return L;
}

// Scratch buffers come from the device's stream-ordered pool.  By default that
// pool hands its memory back to the driver at every synchronisation, which
// makes the next call pay for a fresh allocation; keep it cached instead.
int keep_pool_cached() {
    static bool done[64] = {false};
    int dev = 0;
    SVOXB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || done[dev]) return SVOXB_OK;
    cudaMemPool_t pool;
    SVOXB_CUDA(cudaDeviceGetDefaultMemPool(&pool, dev));
    unsigned long long keep = ~0ull;
    SVOXB_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
    done[dev] = true;
    return SVOXB_OK;
}

int TopScratch::build(const svoxb_tree* t, int max_level, cudaStream_t s) {
    stream = s;
    level = (t->N == 2) ? auto_top_level(t->M, max_level) : 0;
    if (level == 0) return SVOXB_OK;
    int st = keep_pool_cached();
    if (st) return st;
    const size_t n = (size_t)1 << (3 * level);
    SVOXB_CUDA(cudaMallocAsync((void**)&cells, n * sizeof(int32_t), s));
    build_top_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(t->child, t->M, level, cells);
    SVOXB_CUDA(cudaGetLastError());
    return SVOXB_OK;
}

}  // namespace svoxb
