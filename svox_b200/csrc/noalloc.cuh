// svoxb_volume_render_noalloc: the forward ray render for callers that must
// not allocate device memory.
//
// The regular entry points take their per-call scratch (the annotated copy of
// the child array and the jump table over the top of the tree) from the CUDA
// memory pool.  Some hosts cannot do that: a renderer embedded in an
// application that owns the whole device heap, a plug-in that runs inside
// someone else's allocator-free real-time loop, or a process whose memory
// budget is fixed at start-up.  For them this variant keeps the scratch in a
// file-scope __device__ array of fixed size, so a call touches no allocator
// at all -- at the price of a cap on the tree size and of the array being
// resident on every GPU that loads the library.
#pragma once

#include "render_queue.cuh"

namespace svoxb {

constexpr int64_t kNoAllocMaxNodes = 1 << 19;  // 524288 nodes -> 16 MiB of annotated entries
constexpr int kNoAllocTopLevel = 6;            // leaf table: 64^3 entries (1 MiB)
constexpr int64_t kNoAllocTopCells = 1 << (3 * kNoAllocTopLevel);

// [0, 8 * kNoAllocMaxNodes): annotated child entries; then the leaf table.
static __device__ __align__(256) int32_t g_noalloc_scratch[kNoAllocMaxNodes * 8 + kNoAllocTopCells];

// Device address of the array, per device.  In host code the symbol's name is
// only a stand-in: the address a kernel can use has to be asked for, once per
// device, with that device current.
static int noalloc_scratch_address(int32_t** out) {
    static int32_t* address[64] = {nullptr};
    int dev = 0;
    SVOXB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SVOXB_ERR_CUDA;
    if (address[dev] == nullptr) {
        int32_t* p = nullptr;
        SVOXB_CUDA(cudaGetSymbolAddress((void**)&p, g_noalloc_scratch));
        address[dev] = p;
    }
    *out = address[dev];
    return SVOXB_OK;
}

template <int BD>
static int launch_noalloc(const RenderCall& c, const RayBatch& src, int32_t* scratch) {
    const svoxb_tree* t = c.tree;
    int32_t* annotated = scratch;
    int32_t* table = scratch + kNoAllocMaxNodes * 8;
    const int64_t n = t->M * 8;
    // Both scratch regions are fully overwritten before they are read, so nothing
    // left over from an earlier call matters.
    annotate_sigma_kernel<<<index_grid(n, 256, sm_count()), 256, 0, c.stream>>>(
        t->child, t->data, t->K, n, c.opt.sigma_thresh, c.opt.density_softplus, annotated,
        LogGate{});
    SVOXB_CUDA(cudaGetLastError());
    const int level = auto_top_level(t->M, kNoAllocTopLevel);
    if (level > 0) {
        const int cells = 1 << (3 * level);
        build_leaf_table_kernel<<<index_grid(cells, 256, sm_count()), 256, 0, c.stream>>>(annotated, t->M, level,
                                                                          table, LogGate{});
        SVOXB_CUDA(cudaGetLastError());
    }
    const TopTable top{table, level};
    TreeArgs tr = tree_args(t);
    tr.child = annotated;
    return launch_queue_fitted<BD>(c, src, tr, top);
}

}  // namespace svoxb

extern "C" int svoxb_volume_render_noalloc(const svoxb_tree* tree, const svoxb_rays* rays,
                                           const svoxb_render_options* opt, float* out,
                                           void* stream) {
    using namespace svoxb;
    if (!tree || !rays || !opt) return SVOXB_ERR_NULL;
    if (rays->Q > 0 && (!rays->origins || !rays->dirs || !rays->vdirs)) return SVOXB_ERR_NULL;
    int st = validate_tree(tree);
    if (st) return st;
    if ((st = validate_options(tree, *opt))) return st;
    if (rays->Q < 0) return SVOXB_ERR_SHAPE;
    if (tree->M > kNoAllocMaxNodes) return SVOXB_ERR_TOO_LARGE;
    // only the layouts of the queue kernels: octree, SH colour in three channels
    if (tree->N != 2 || opt->format != SVOXB_FORMAT_SH || tree->K != 3 * opt->basis_dim + 1)
        return SVOXB_ERR_FORMAT;
    if (tree->K % 4 == 0 && (uintptr_t)tree->data % 16 != 0) return SVOXB_ERR_FORMAT;
    if (rays->Q == 0) return SVOXB_OK;
    if (!out) return SVOXB_ERR_NULL;
    int32_t* scratch = nullptr;
    if ((st = noalloc_scratch_address(&scratch))) return st;
    RenderCall c{tree, *opt, rays->Q};
    c.out = out;
    c.stream = (cudaStream_t)stream;
    const RayBatch src{rays->origins, rays->dirs, rays->vdirs};
    switch (opt->basis_dim) {
        case 1: return launch_noalloc<1>(c, src, scratch);
        case 4: return launch_noalloc<4>(c, src, scratch);
        case 9: return launch_noalloc<9>(c, src, scratch);
        case 16: return launch_noalloc<16>(c, src, scratch);
        case 25: return launch_noalloc<25>(c, src, scratch);
    }
    return SVOXB_ERR_FORMAT;
}
