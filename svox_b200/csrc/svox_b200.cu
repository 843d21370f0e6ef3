// C-ABI entry points of libsvox_b200 (see include/svox_b200.h) and the
// dispatch from run-time record layouts to the templated sm_100a kernels.
// The library is this single translation unit.
#include "common.cuh"
#include "host.cuh"
#include "query.cuh"
#include "render.cuh"
#include "render_queue.cuh"
#include "render_replay.cuh"
#include "collective.cuh"
#include <new>

namespace svoxb {

struct RenderCall {
    const svoxb_tree* tree;
    svoxb_render_options opt;
    int64_t Q;
    // forward
    float* out = nullptr;
    // backward
    bool backward = false;
    const float* grad_out = nullptr;
    const float* fwd_out = nullptr;
    float* grad_data = nullptr;
    cudaStream_t stream = nullptr;
    // item log (logged forward / replay backward)
    int32_t* log = nullptr;
    int64_t log_capacity = 0;
    // forward with a scratch built earlier by svoxb_render_scratch_build (else per call)
    int32_t* prepared = nullptr;
    // marching backward as the fallback of a replay: does its work only if this log overflowed
    LogGate gate{};
};

static int out_dim_of(const svoxb_tree* t, const svoxb_render_options& o) {
    // get_out_data_dim, svox/csrc/rt_kernel.cu:1009-1015
    return o.format != SVOXB_FORMAT_RGBA ? (t->K - 1) / o.basis_dim : t->K - 1;
}

// The records hold three colour channels of basis_dim coefficients each and a density, and
// basis_dim is one of the sizes the specialised kernels are compiled for.
static bool basis3(const svoxb_tree* t, const svoxb_render_options& o) {
    const int b = o.basis_dim;
    return o.format != SVOXB_FORMAT_RGBA && t->K == 3 * b + 1 &&
           (b == 1 || b == 4 || b == 9 || b == 16 || b == 25);
}

static int validate_options(const svoxb_tree* t, const svoxb_render_options& o) {
    if (!(o.step_size >= 0.f)) return SVOXB_ERR_OPTION;
    if (o.format < SVOXB_FORMAT_RGBA || o.format > SVOXB_FORMAT_ASG) return SVOXB_ERR_FORMAT;
    if (o.format != SVOXB_FORMAT_RGBA) {
        const int b = o.basis_dim;
        if (o.format == SVOXB_FORMAT_SH) {
            if (b != 1 && b != 4 && b != 9 && b != 16 && b != 25) return SVOXB_ERR_FORMAT;
        } else {
            // the reference keeps the basis in an array of 25 (svox/csrc/rt_kernel.cu:253)
            if (b < 1 || b > 25) return SVOXB_ERR_FORMAT;
            if (!t->extra_data) return SVOXB_ERR_NULL;
            if (t->extra_rows < b || t->extra_cols < (o.format == SVOXB_FORMAT_SG ? 4 : 11))
                return SVOXB_ERR_SHAPE;
        }
        if (o.min_comp < 0 || o.max_comp >= b) return SVOXB_ERR_OPTION;
        if (t->K - 1 < b) return SVOXB_ERR_SHAPE;
    } else if (t->K < 2) {
        return SVOXB_ERR_SHAPE;
    }
    const int od = out_dim_of(t, o);
    if (od < 1) return SVOXB_ERR_SHAPE;
    if (o.ndc_width >= 0 && (o.ndc_width == 0 || o.ndc_height <= 0)) return SVOXB_ERR_OPTION;
    return SVOXB_OK;
}

template <class Kernel>
static int persistent_grid(Kernel kernel, int block, size_t smem, int64_t n_gran, unsigned* grid) {
    // the 48 KB a kernel gets without asking cover its static shared memory too (up to 4 KB here)
    if (smem > 40 * 1024)
        SVOXB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
    int per_sm = 0;
    SVOXB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, block, smem));
    if (per_sm < 1) per_sm = 1;
    int sms = sm_count() - g_reserved_sms;     // see svoxb_reserve_sms
    if (sms < 1) sms = 1;
    int64_t g = (int64_t)sms * per_sm;
    const int64_t need = (n_gran * 32 + block - 1) / block;  // blocks that can get a granule each
    if (g > need) g = need;
    if (g < 1) g = 1;
    *grid = (unsigned)g;
    return SVOXB_OK;
}

template <int BD, bool VEC, int BLOCK, class Source>
static int launch_sh(const RenderCall& c, const Source& src, const TopTable& top, bool in_smem,
                     size_t smem) {
    const TreeArgs tr = tree_args(c.tree);
    const int64_t n_gran = (c.Q + 31) / 32;
    unsigned grid = 1;
    int st;
    if (!c.backward) {
        auto k = render_fwd_sh<BD, VEC, BLOCK, Source>;
        if ((st = persistent_grid(k, BLOCK, smem, n_gran, &grid))) return st;
        k<<<grid, BLOCK, smem, c.stream>>>(tr, src, c.opt, top, in_smem, c.out, c.Q);
    } else if (c.fwd_out != nullptr && c.opt.sigma_thresh == 0.f && c.opt.stop_thresh == 0.f) {
        auto k = render_bwd_sh<BD, VEC, BLOCK, true, Source>;
        if ((st = persistent_grid(k, BLOCK, smem, n_gran, &grid))) return st;
        k<<<grid, BLOCK, smem, c.stream>>>(tr, src, c.opt, top, in_smem, c.grad_out, c.fwd_out,
                                          c.grad_data, c.Q);
    } else {
        auto k = render_bwd_sh<BD, VEC, BLOCK, false, Source>;
        if ((st = persistent_grid(k, BLOCK, smem, n_gran, &grid))) return st;
        k<<<grid, BLOCK, smem, c.stream>>>(tr, src, c.opt, top, in_smem, c.grad_out, nullptr,
                                          c.grad_data, c.Q);
    }
    SVOXB_CUDA(cudaGetLastError());
    return SVOXB_OK;
}

// Queue kernels (render_queue.cuh).  The block size is the largest whose
// per-warp queues fit in shared memory next to the jump table.
constexpr size_t kMaxSmem = 227 * 1024;

// Replay bins: a bin is a range of 2^shift leaf slots whose gradient spans
// about g_tuning.replay_bin_mb MB, at most kMaxBins of them.
static int replay_bin_shift(int64_t M, int K) {
    const int64_t per_bin = ((int64_t)g_tuning.replay_bin_mb << 20) / (K * 4);
    int shift = 0;
    while ((2LL << shift) <= per_bin) ++shift;
    while (((M * 8 - 1) >> shift) + 1 > kMaxBins) ++shift;
    return shift;
}

template <int BD, int BLOCK, class Source>
static int launch_queue_block(const RenderCall& c, const Source& src, const TreeArgs& tr,
                              const TopTable& top, size_t top_bytes) {
    constexpr int K = 3 * BD + 1;
    const int64_t n_gran = (c.Q + 31) / 32;
    unsigned grid = 1;
    int st;
    if (!c.backward && c.log != nullptr) {
        const size_t smem = top_bytes + (size_t)(BLOCK / 32) * sizeof(WarpQueue<K, kModeForwardLogged>);
        auto k = render_queue_kernel<BD, BLOCK, kModeForwardLogged, Source>;
        if ((st = persistent_grid(k, BLOCK, smem, n_gran, &grid))) return st;
        k<<<grid, BLOCK, smem, c.stream>>>(tr, src, c.opt, top, (int)top_bytes, c.Q, c.out,
                                          nullptr, nullptr, nullptr, c.log, c.log_capacity,
                                          replay_bin_shift(c.tree->M, K), kRefillBatch);
    } else if (!c.backward) {
        const size_t smem = top_bytes + (size_t)(BLOCK / 32) * sizeof(WarpQueue<K, kModeForward>);
        auto k = render_queue_kernel<BD, BLOCK, kModeForward, Source>;
        if ((st = persistent_grid(k, BLOCK, smem, n_gran, &grid))) return st;
        k<<<grid, BLOCK, smem, c.stream>>>(tr, src, c.opt, top, (int)top_bytes, c.Q, c.out,
                                          nullptr, nullptr, nullptr, nullptr, 0, 0, kRefillBatch);
    } else {
        const size_t smem = top_bytes + (size_t)(BLOCK / 32) * sizeof(WarpQueue<K, kModeBackward>);
        const bool single = c.fwd_out != nullptr && c.opt.sigma_thresh == 0.f &&
                            c.opt.stop_thresh == 0.f;
        auto k = render_queue_kernel<BD, BLOCK, kModeBackward, Source>;
        if ((st = persistent_grid(k, BLOCK, smem, n_gran, &grid))) return st;
        k<<<grid, BLOCK, smem, c.stream>>>(tr, src, c.opt, top, (int)top_bytes, c.Q, nullptr,
                                          c.grad_out, single ? c.fwd_out : nullptr, c.grad_data,
                                          const_cast<int32_t*>(c.gate.log), c.gate.capacity, 0,
                                          kRefillBatch);
    }
    SVOXB_CUDA(cudaGetLastError());
    return SVOXB_OK;
}

// Picks the block size: 640 threads where the record allows it (the kernel needs ~90
// registers; at 768 threads it spilled inside the loop), fewer while the per-warp queues
// do not fit in shared memory.
template <int BD, class Source>
static int launch_queue_fitted(const RenderCall& c, const Source& src, const TreeArgs& tr,
                               const TopTable& top) {
    constexpr int K = 3 * BD + 1;
    const size_t top_bytes = 0;  // the leaf table stays in global memory
    const size_t per_warp = c.backward ? sizeof(WarpQueue<K, kModeBackward>)
                            : c.log    ? sizeof(WarpQueue<K, kModeForwardLogged>)
                                       : sizeof(WarpQueue<K, kModeForward>);
    // the lobe bases are compiled for the smallest block only
    if constexpr (Source::kLobes) return launch_queue_block<BD, 256>(c, src, tr, top, top_bytes);
    int want = 640;
    // static shared memory: the ticket counter, and the bin histogram of the logged forward
    const size_t fixed = 64 + (c.log ? (size_t)kMaxBins * sizeof(int) : 0);
    while (want > 256 && top_bytes + (size_t)(want / 32) * per_warp + fixed > kMaxSmem) want -= 128;
    if constexpr (BD <= 9) {
        if (want >= 640) return launch_queue_block<BD, 640>(c, src, tr, top, top_bytes);
    }
    if constexpr (BD <= 16) {
        if (want >= 512) return launch_queue_block<BD, 512>(c, src, tr, top, top_bytes);
    }
    return launch_queue_block<BD, 256>(c, src, tr, top, top_bytes);
}

// Replay backward (render_replay.cuh): prefix, pack, bin, then the scatter in one
// or several parts (bin ranges).  A ReplayJob holds the scratch between the calls.
struct ReplayJob {
    ReplayBins bins{};
    int32_t* base = nullptr;     // pool allocation
    const int32_t* log = nullptr;
    svoxb_render_options opt{};
    TreeArgs lobes{};            // for the lobe parameters of an SG / ASG basis
    int64_t n_slots = 0, n_rays = 0, chunks = 0;
    int K = 0, basis_dim = 0, n_parts = 1, shift = 0, n_bins = 1;
    bool hess = false;   // Gauss-Newton diagonal instead of the gradient
};

// Prefix + pack + bin.  SVOXB_ERR_TOO_LARGE when the packet buffer cannot be had
// (the caller then marches instead).
template <class Source>
static int replay_begin(const RenderCall& c, const Source& src, int64_t chunks, int n_parts,
                        ReplayJob* job, bool hess = false) {
    if (chunks > c.log_capacity) chunks = c.log_capacity;
    if (n_parts < 1 || n_parts > kMaxParts) return SVOXB_ERR_OPTION;
    const int64_t packets = (chunks > 0 ? chunks : 1) * 32;
    if (packets >= (1LL << 30)) return SVOXB_ERR_TOO_LARGE;

    int st = keep_pool_cached();
    if (st) return st;
    // cursors | offsets | work counters | packed rays | packets
    const size_t head_words =
        (size_t)kMaxBins * kCursorStride + kMaxBins + 8 + 2 * kMaxParts;  // 32-byte multiple
    const size_t ray_words = (size_t)c.Q * 12;
    const size_t pad = (8 - (head_words + ray_words) % 8) % 8;
    int32_t* base = nullptr;
    if (cudaMallocAsync((void**)&base,
                        (head_words + ray_words + pad + 8 * (size_t)packets) * sizeof(int32_t),
                        c.stream) != cudaSuccess) {
        (void)cudaGetLastError();
        return SVOXB_ERR_TOO_LARGE;
    }
    ReplayBins& b = job->bins;
    b.cursor = base;
    b.offset = base + (size_t)kMaxBins * kCursorStride;
    b.work = reinterpret_cast<int64_t*>(b.offset + kMaxBins + 2);  // 8-byte aligned
    float4* rays = reinterpret_cast<float4*>(base + head_words);
    b.rays = rays;
    b.capacity = packets;
    b.packet = reinterpret_cast<int4*>(base + head_words + ray_words + pad);
    job->base = base;
    job->log = c.log;
    job->opt = c.opt;
    job->lobes = tree_args(c.tree);
    job->n_slots = c.tree->M * 8;
    job->n_rays = c.Q;
    job->chunks = chunks;
    job->K = c.tree->K;
    job->basis_dim = c.opt.basis_dim;
    job->n_parts = n_parts;
    job->hess = hess;
    job->shift = replay_bin_shift(c.tree->M, c.tree->K);
    job->n_bins = (int)(((job->n_slots - 1) >> job->shift) + 1);

    replay_prefix_kernel<<<1, 256, 0, c.stream>>>(c.log, b, n_parts, c.log_capacity);
    if (chunks > 0) {
        replay_pack_rays_kernel<<<(unsigned)((c.Q + 255) / 256), 256, 0, c.stream>>>(
            tree_args(c.tree), src, c.opt, c.grad_out, c.fwd_out, c.Q, rays);
        unsigned grid = 1;
        auto run_bin = [&](auto k, int block) {
            int s2 = persistent_grid(k, block, 0, chunks, &grid);
            if (s2 == SVOXB_OK)
                k<<<grid, block, 0, c.stream>>>(c.opt, c.log, chunks, c.log_capacity, c.Q, b,
                                                c.tree->data, c.tree->K);
            return s2;
        };
        st = hess ? run_bin(replay_bin_kernel<128, 2, 12, true>, 128)
                  : run_bin(replay_bin_kernel<128, 2, 12, false>, 128);
    }
    const cudaError_t e = cudaGetLastError();
    if (st == SVOXB_OK && e != cudaSuccess) st = set_cuda_error(e);
    if (st != SVOXB_OK) {
        cudaFreeAsync(base, c.stream);
        job->base = nullptr;
    }
    return st;
}

// Scatter of one part.  With `reserve_sms` > 0 that many SMs are left without a block
// (for a collective that runs beside the scatter); small records then use one 1024-thread
// block per SM, so that the SMs left out are really empty.
template <int BD, int BLOCK, bool HESS, bool LOBES = false>
static int replay_scatter_block(const ReplayJob& job, int part, float* grad, int reserve_sms,
                                cudaStream_t stream) {
    constexpr int K = 3 * BD + 1;
    const size_t smem = (size_t)(BLOCK / 32) * sizeof(ScatterSmem<K>);
    auto k = replay_scatter_kernel<BD, BLOCK, HESS, LOBES>;
    unsigned grid = 1;
    int st = persistent_grid(k, BLOCK, smem, job.chunks, &grid);
    if (st) return st;
    if (reserve_sms > 0) {
        const int sms = sm_count();
        const int64_t per_sm = ((int64_t)grid + sms - 1) / sms;
        const int64_t most = ((int64_t)sms - reserve_sms) * per_sm;
        if ((int64_t)grid > most) grid = (unsigned)(most > 1 ? most : 1);
    }
    k<<<grid, BLOCK, smem, stream>>>(job.n_slots, job.opt, job.lobes, grad, job.log, job.bins,
                                    kReplayHints, part, job.n_parts);
    const cudaError_t e = cudaGetLastError();
    return e != cudaSuccess ? set_cuda_error(e) : SVOXB_OK;
}

template <int BD>
static int replay_scatter_bd(const ReplayJob& job, int part, float* grad, int reserve_sms,
                             cudaStream_t stream) {
    if (job.opt.format != SVOXB_FORMAT_SH)
        return job.hess ? replay_scatter_block<BD, 512, true, true>(job, part, grad, 0, stream)
                        : replay_scatter_block<BD, 512, false, true>(job, part, grad, reserve_sms,
                                                                     stream);
    if (job.hess) return replay_scatter_block<BD, 512, true>(job, part, grad, 0, stream);
    if constexpr (BD <= 9) {
        if (reserve_sms > 0)
            return replay_scatter_block<BD, 1024, false>(job, part, grad, reserve_sms, stream);
    }
    // 256-thread blocks: measured 2.83 ms of backward per training step against 2.94 with 512
    // (more, smaller blocks keep the window of packets in flight narrower)
    return replay_scatter_block<BD, 256, false>(job, part, grad, reserve_sms, stream);
}

static int replay_scatter(const ReplayJob& job, int part, float* grad, int reserve_sms,
                          cudaStream_t stream) {
    if (part < 0 || part >= job.n_parts) return SVOXB_ERR_OPTION;
    if (job.chunks < 1) return SVOXB_OK;
    switch (job.basis_dim) {
        case 1: return replay_scatter_bd<1>(job, part, grad, reserve_sms, stream);
        case 4: return replay_scatter_bd<4>(job, part, grad, reserve_sms, stream);
        case 9: return replay_scatter_bd<9>(job, part, grad, reserve_sms, stream);
        case 16: return replay_scatter_bd<16>(job, part, grad, reserve_sms, stream);
        case 25: return replay_scatter_bd<25>(job, part, grad, reserve_sms, stream);
    }
    return SVOXB_ERR_FORMAT;
}

static void replay_end(ReplayJob* job, cudaStream_t stream) {
    if (job->base) cudaFreeAsync(job->base, stream);
    job->base = nullptr;
}

// Per-call scratch of the queue kernels: the annotated child array followed by
// the leaf table (render_queue.cuh); one pool allocation, freed on the stream.
struct QueueScratch {
    int32_t* annotated = nullptr;
    int32_t* table = nullptr;
    int32_t* bricks = nullptr;
    int level = 0;
    bool owned = false;
    cudaStream_t stream = nullptr;

    // annotated | table | brick counter (8 words) | brick roots | bricks
    struct Layout {
        int64_t n, cells, cap;
        int level;
        size_t head, words;
    };
    static Layout layout(const svoxb_tree* t, int max_level) {
        Layout l{};
        l.n = t->M * 8;
        l.level = auto_top_level(t->M, max_level);
        l.cells = l.level > 0 ? ((int64_t)1 << (3 * l.level)) : 0;
        // bricks: one per table cell that holds a node, while the budget lasts
        l.cap = 0;
        if (l.level > 0 && g_tuning.render_bricks && t->M < kBrickMaxNodes &&
            l.level + kBrickLevels < kCoordBits) {
            l.cap = l.cells < t->M ? l.cells : t->M;
            if (l.cap > kMaxBricks) l.cap = kMaxBricks;
        }
        l.head = (size_t)(l.n + l.cells) + 8 + (size_t)((l.cap + 7) & ~(int64_t)7);
        l.words = l.head + (size_t)l.cap * kBrickWords;
        return l;
    }
    // Level of the leaf table: 6 (64^3 cells, 1 MB); 7 (128^3, 8 MB) for trees of several
    // million nodes, whose leaves lie up to ten levels deep: the bricks below the table then
    // still reach them in one step.
    static int default_level(const svoxb_tree* t) {
        return t->M >= (4LL << 20) ? 7 : 6;
    }
    void adopt(const Layout& l, int32_t* mem) {
        annotated = mem;
        table = mem + l.n;
        bricks = l.cap > 0 ? mem + l.head : nullptr;
        level = l.level;
    }

    // Fills `external` (layout(t, max_level).words int32) or a pool allocation of its own.
    int build(const svoxb_tree* t, float thresh, int softplus, int max_level, cudaStream_t s,
              int32_t* external = nullptr, LogGate gate = LogGate{}) {
        stream = s;
        const Layout l = layout(t, max_level);
        int32_t* mem = external;
        if (!mem) {
            int st = keep_pool_cached();
            if (st) return st;
            SVOXB_CUDA(cudaMallocAsync((void**)&mem, l.words * sizeof(int32_t), s));
            owned = true;
        }
        adopt(l, mem);
        const int sms = sm_count();
        annotate_sigma_kernel<<<index_grid(l.n, 256, sms), 256, 0, s>>>(
            t->child, t->data, t->K, l.n, thresh, softplus, annotated, gate);
        SVOXB_CUDA(cudaGetLastError());
        if (level > 0) {
            build_leaf_table_kernel<<<index_grid(l.cells, 256, sms), 256, 0, s>>>(
                annotated, t->M, level, table, gate);
            SVOXB_CUDA(cudaGetLastError());
        }
        if (l.cap > 0) {
            int32_t* counter = table + l.cells;
            int32_t* roots = counter + 8;
            SVOXB_CUDA(cudaMemsetAsync(counter, 0, sizeof(int32_t), s));
            assign_bricks_kernel<<<index_grid(l.cells, 256, sms), 256, 0, s>>>(
                table, (int)l.cells, (int)l.cap, counter, roots, gate);
            fill_bricks_kernel<<<index_grid(l.cap * kBrickCells, kBrickCells, sms), kBrickCells, 0, s>>>(
                annotated, t->M, level, (int)l.cap, counter, roots, bricks, gate);
            SVOXB_CUDA(cudaGetLastError());
        }
        return SVOXB_OK;
    }
    ~QueueScratch() { if (owned && annotated) cudaFreeAsync(annotated, stream); }
};

template <int BD, class Source>
static int launch_queue(const RenderCall& c, const Source& src) {
    QueueScratch scratch;
    if (c.prepared != nullptr && !c.backward) {
        scratch.adopt(QueueScratch::layout(c.tree, QueueScratch::default_level(c.tree)), c.prepared);
    } else {
        const int st = scratch.build(c.tree, c.backward ? 0.f : c.opt.sigma_thresh,
                                     c.opt.density_softplus, QueueScratch::default_level(c.tree),
                                     c.stream, nullptr, c.gate);
        if (st) return st;
    }
    TreeArgs tr = tree_args(c.tree);
    tr.child = scratch.annotated;
    const TopTable top{scratch.table, scratch.level, scratch.bricks};
    if (c.opt.format != SVOXB_FORMAT_SH)
        return launch_queue_fitted<BD>(c, WithLobes<Source>{src}, tr, top);
    return launch_queue_fitted<BD>(c, src, tr, top);
}

template <int BLOCK, class Source>
static int launch_generic(const RenderCall& c, const Source& src, const TopTable& top,
                          bool in_smem, size_t smem) {
    const TreeArgs tr = tree_args(c.tree);
    const int64_t n_gran = (c.Q + 31) / 32;
    const int od = out_dim_of(c.tree, c.opt);
    if (od > kMaxGenericOut) return SVOXB_ERR_FORMAT;
    unsigned grid = 1;
    int st;
    if (!c.backward) {
        auto k = render_fwd_generic<BLOCK, Source>;
        if ((st = persistent_grid(k, BLOCK, smem, n_gran, &grid))) return st;
        k<<<grid, BLOCK, smem, c.stream>>>(tr, src, c.opt, top, in_smem, c.out, c.Q, od);
    } else {
        auto k = render_bwd_generic<BLOCK, Source>;
        if ((st = persistent_grid(k, BLOCK, smem, n_gran, &grid))) return st;
        k<<<grid, BLOCK, smem, c.stream>>>(tr, src, c.opt, top, in_smem, c.grad_out, c.grad_data,
                                          c.Q, od);
    }
    SVOXB_CUDA(cudaGetLastError());
    return SVOXB_OK;
}

template <int BLOCK, class Source>
static int dispatch_layout(const RenderCall& c, const Source& src, const TopTable& top,
                           bool in_smem, size_t smem) {
    const svoxb_tree* t = c.tree;
    const bool sh3 = basis3(t, c.opt) && c.opt.format == SVOXB_FORMAT_SH;
    if (!sh3) return launch_generic<BLOCK>(c, src, top, in_smem, smem);
    const bool aligned = ((uintptr_t)t->data % 16 == 0) &&
                         (!c.backward || (uintptr_t)c.grad_data % 16 == 0);
    const bool vec = aligned && (t->K % 4 == 0);
    switch (c.opt.basis_dim) {
        case 1:
            return vec ? launch_sh<1, true, BLOCK>(c, src, top, in_smem, smem)
                       : launch_sh<1, false, BLOCK>(c, src, top, in_smem, smem);
        case 4: return launch_sh<4, false, BLOCK>(c, src, top, in_smem, smem);
        case 9:
            return vec ? launch_sh<9, true, BLOCK>(c, src, top, in_smem, smem)
                       : launch_sh<9, false, BLOCK>(c, src, top, in_smem, smem);
        case 16: return launch_sh<16, false, BLOCK>(c, src, top, in_smem, smem);
        case 25:
            return vec ? launch_sh<25, true, BLOCK>(c, src, top, in_smem, smem)
                       : launch_sh<25, false, BLOCK>(c, src, top, in_smem, smem);
    }
    return SVOXB_ERR_FORMAT;
}

template <class Source>
static int render_dispatch(const RenderCall& c, const Source& src) {
    int st = validate_tree(c.tree);
    if (st) return st;
    if ((st = validate_options(c.tree, c.opt))) return st;
    if (c.Q < 0) return SVOXB_ERR_SHAPE;
    if (c.backward) {
        if (!c.grad_data) return SVOXB_ERR_NULL;
    }
    if (c.Q == 0) return SVOXB_OK;
    if (c.backward ? !c.grad_out : !c.out) return SVOXB_ERR_NULL;

    // Default path: the queue kernels, for octrees with three colour channels of 1, 4, 9, 16
    // or 25 basis functions whose buffers allow the record's word size.
    {
        const svoxb_tree* t = c.tree;
        const bool sh3 = basis3(t, c.opt);
        const bool aligned = ((uintptr_t)t->data % 16 == 0) &&
                             (!c.backward || (uintptr_t)c.grad_data % 16 == 0);
        if (sh3 && t->N == 2 && (aligned || t->K % 4 != 0) &&
            t->M < (1LL << 28)) {
            switch (c.opt.basis_dim) {
                case 1: return launch_queue<1>(c, src);
                case 4: return launch_queue<4>(c, src);
                case 9: return launch_queue<9>(c, src);
                case 16: return launch_queue<16>(c, src);
                case 25: return launch_queue<25>(c, src);
            }
        }
    }

    TopScratch scratch;
    if ((st = scratch.build(c.tree, 5, c.stream))) return st;
    const TopTable top{scratch.cells, scratch.level};
    // The table is staged in shared memory up to level 5 (128 KB).
    const bool in_smem = scratch.level > 0 && scratch.level <= 5;
    const size_t smem = in_smem ? ((size_t)4 << (3 * scratch.level)) : 0;
    if (smem > 64 * 1024) return dispatch_layout<1024>(c, src, top, in_smem, smem);
    return dispatch_layout<256>(c, src, top, in_smem, smem);
}

static int zero_grad(const svoxb_tree* t, float* grad, int K, cudaStream_t s) {
    const size_t n = (size_t)t->M * t->N * t->N * t->N * (size_t)K;
    SVOXB_CUDA(cudaMemsetAsync(grad, 0, n * sizeof(float), s));
    return SVOXB_OK;
}

}  // namespace svoxb

using namespace svoxb;

extern "C" {

int svoxb_query_vertical(const svoxb_tree* tree, const float* indices, int64_t Q,
                         float* values_out, int64_t* node_ids_out, void* stream) {
    int st = validate_tree(tree);
    if (st) return st;
    if (Q < 0) return SVOXB_ERR_SHAPE;
    return launch_query(0, tree, indices, Q, values_out, node_ids_out, nullptr, nullptr, 0,
                        (cudaStream_t)stream);
}

int svoxb_query_vertical_backward(const svoxb_tree* tree, const float* indices, int64_t Q,
                                  const float* grad_output, int32_t Kg, float* grad_data_out,
                                  int zero_first, void* stream) {
    int st = validate_tree(tree);
    if (st) return st;
    if (Q < 0 || Kg < 1) return SVOXB_ERR_SHAPE;
    if (!grad_data_out || (Q > 0 && !grad_output)) return SVOXB_ERR_NULL;
    if (zero_first && (st = zero_grad(tree, grad_data_out, Kg, (cudaStream_t)stream))) return st;
    return launch_query(1, tree, indices, Q, nullptr, nullptr, grad_output, grad_data_out, Kg,
                        (cudaStream_t)stream);
}

int svoxb_assign_vertical(const svoxb_tree* tree, const float* indices, int64_t Q,
                          const float* values, int32_t Kv, float* data_out, void* stream) {
    int st = validate_tree(tree);
    if (st) return st;
    if (Q < 0 || Kv < 1 || Kv > tree->K) return SVOXB_ERR_SHAPE;
    if (!data_out || (Q > 0 && !values)) return SVOXB_ERR_NULL;
    return launch_query(2, tree, indices, Q, nullptr, nullptr, values, data_out, Kv,
                        (cudaStream_t)stream);
}

int svoxb_calc_corners(const svoxb_tree* tree, const int32_t* parent_depth,
                       const int64_t* indexer, int64_t Q, float* out, void* stream) {
    int st = validate_tree(tree);
    if (st) return st;
    if (Q < 0) return SVOXB_ERR_SHAPE;
    if (Q == 0) return SVOXB_OK;
    if (!parent_depth || !indexer || !out) return SVOXB_ERR_NULL;
    if ((Q + 255) / 256 > 0x7fffffffLL) return SVOXB_ERR_TOO_LARGE;
    calc_corners_kernel<<<(unsigned)((Q + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        parent_depth, tree->M, tree->N, indexer, Q, out);
    SVOXB_CUDA(cudaGetLastError());
    return SVOXB_OK;
}

int svoxb_volume_render(const svoxb_tree* tree, const svoxb_rays* rays,
                        const svoxb_render_options* opt, float* out, void* stream) {
    if (!tree || !rays || !opt) return SVOXB_ERR_NULL;
    if (rays->Q > 0 && (!rays->origins || !rays->dirs || !rays->vdirs)) return SVOXB_ERR_NULL;
    RenderCall c{tree, *opt, rays->Q};
    c.out = out;
    c.stream = (cudaStream_t)stream;
    return render_dispatch(c, RayBatch{rays->origins, rays->dirs, rays->vdirs});
}

int svoxb_volume_render_image(const svoxb_tree* tree, const svoxb_camera* cam,
                              const svoxb_render_options* opt, float* out, void* stream) {
    if (!tree || !cam || !opt || !cam->c2w) return SVOXB_ERR_NULL;
    if (cam->width < 0 || cam->height < 0) return SVOXB_ERR_SHAPE;
    RenderCall c{tree, *opt, (int64_t)cam->width * cam->height};
    c.out = out;
    c.stream = (cudaStream_t)stream;
    return render_dispatch(c, PixelRays{cam->c2w, cam->fx, cam->fy, cam->width, cam->height});
}

// Whether the queue kernels take this tree and these options (the prepared scratch is theirs).
static int queue_eligible(const svoxb_tree* t, const svoxb_render_options* o) {
    int st = validate_tree(t);
    if (st) return st;
    if ((st = validate_options(t, *o))) return st;
    if (!basis3(t, *o) || t->N != 2)
        return SVOXB_ERR_FORMAT;
    if (t->K % 4 == 0 && (uintptr_t)t->data % 16 != 0) return SVOXB_ERR_FORMAT;
    if (t->M >= (1LL << 28)) return SVOXB_ERR_TOO_LARGE;
    return SVOXB_OK;
}

int64_t svoxb_render_scratch_words(const svoxb_tree* tree) {
    if (!tree || tree->M < 1 || tree->N != 2) return 0;
    return (int64_t)QueueScratch::layout(tree, QueueScratch::default_level(tree)).words;
}

int svoxb_render_scratch_build(const svoxb_tree* tree, const svoxb_render_options* opt,
                               int32_t* scratch, void* stream) {
    if (!tree || !opt || !scratch) return SVOXB_ERR_NULL;
    int st = queue_eligible(tree, opt);
    if (st) return st;
    QueueScratch q;
    return q.build(tree, opt->sigma_thresh, opt->density_softplus, QueueScratch::default_level(tree),
                   (cudaStream_t)stream, scratch);
}

int svoxb_volume_render_prepared(const svoxb_tree* tree, const svoxb_rays* rays,
                                 const svoxb_render_options* opt, const int32_t* scratch,
                                 float* out, void* stream) {
    if (!tree || !rays || !opt || !scratch) return SVOXB_ERR_NULL;
    if (rays->Q > 0 && (!rays->origins || !rays->dirs || !rays->vdirs)) return SVOXB_ERR_NULL;
    int st = queue_eligible(tree, opt);
    if (st) return st;
    RenderCall c{tree, *opt, rays->Q};
    c.out = out;
    c.stream = (cudaStream_t)stream;
    c.prepared = const_cast<int32_t*>(scratch);
    return render_dispatch(c, RayBatch{rays->origins, rays->dirs, rays->vdirs});
}

int svoxb_volume_render_image_prepared(const svoxb_tree* tree, const svoxb_camera* cam,
                                       const svoxb_render_options* opt, const int32_t* scratch,
                                       float* out, void* stream) {
    if (!tree || !cam || !opt || !cam->c2w || !scratch) return SVOXB_ERR_NULL;
    if (cam->width < 0 || cam->height < 0) return SVOXB_ERR_SHAPE;
    int st = queue_eligible(tree, opt);
    if (st) return st;
    RenderCall c{tree, *opt, (int64_t)cam->width * cam->height};
    c.out = out;
    c.stream = (cudaStream_t)stream;
    c.prepared = const_cast<int32_t*>(scratch);
    return render_dispatch(c, PixelRays{cam->c2w, cam->fx, cam->fy, cam->width, cam->height});
}

int svoxb_volume_render_backward(const svoxb_tree* tree, const svoxb_rays* rays,
                                 const svoxb_render_options* opt, const float* grad_output,
                                 const float* fwd_out, float* grad_data_out, int zero_first,
                                 void* stream) {
    if (!tree || !rays || !opt) return SVOXB_ERR_NULL;
    if (rays->Q > 0 && (!rays->origins || !rays->dirs || !rays->vdirs)) return SVOXB_ERR_NULL;
    int st = validate_tree(tree);
    if (st) return st;
    if (!grad_data_out) return SVOXB_ERR_NULL;
    if (zero_first && (st = zero_grad(tree, grad_data_out, tree->K, (cudaStream_t)stream)))
        return st;
    RenderCall c{tree, *opt, rays->Q};
    c.backward = true;
    c.grad_out = grad_output;
    c.fwd_out = fwd_out;
    c.grad_data = grad_data_out;
    c.stream = (cudaStream_t)stream;
    return render_dispatch(c, RayBatch{rays->origins, rays->dirs, rays->vdirs});
}

int svoxb_volume_render_image_backward(const svoxb_tree* tree, const svoxb_camera* cam,
                                       const svoxb_render_options* opt,
                                       const float* grad_output, const float* fwd_out,
                                       float* grad_data_out, int zero_first, void* stream) {
    if (!tree || !cam || !opt || !cam->c2w) return SVOXB_ERR_NULL;
    if (cam->width < 0 || cam->height < 0) return SVOXB_ERR_SHAPE;
    int st = validate_tree(tree);
    if (st) return st;
    if (!grad_data_out) return SVOXB_ERR_NULL;
    if (zero_first && (st = zero_grad(tree, grad_data_out, tree->K, (cudaStream_t)stream)))
        return st;
    RenderCall c{tree, *opt, (int64_t)cam->width * cam->height};
    c.backward = true;
    c.grad_out = grad_output;
    c.fwd_out = fwd_out;
    c.grad_data = grad_data_out;
    c.stream = (cudaStream_t)stream;
    return render_dispatch(c, PixelRays{cam->c2w, cam->fx, cam->fy, cam->width, cam->height});
}

}  // extern "C"

// Whether a call can take the logged forward / replay backward pair.
static int log_eligible(const svoxb_tree* t, const svoxb_render_options* o, const float* grad) {
    if (!basis3(t, *o) || t->N != 2)
        return SVOXB_ERR_FORMAT;
    if (o->sigma_thresh != 0.f || o->stop_thresh != 0.f) return SVOXB_ERR_OPTION;
    if (t->M >= (1LL << 28)) return SVOXB_ERR_TOO_LARGE;
    if (t->K % 4 == 0 && ((uintptr_t)t->data % 16 != 0 || (uintptr_t)grad % 16 != 0))
        return SVOXB_ERR_FORMAT;
    return SVOXB_OK;
}

template <class Source>
static int logged_forward(const svoxb_tree* tree, const Source& src, int64_t Q,
                          const svoxb_render_options* opt, float* out, int32_t* log,
                          int64_t capacity_chunks, void* stream) {
    int st = validate_tree(tree);
    if (st) return st;
    if ((st = validate_options(tree, *opt))) return st;
    if ((st = log_eligible(tree, opt, nullptr))) return st;
    if (!log || capacity_chunks < 1 || Q < 0) return SVOXB_ERR_SHAPE;
    if (Q > 0 && !out) return SVOXB_ERR_NULL;
    SVOXB_CUDA(cudaMemsetAsync(log, 0, kLogChunks * sizeof(int32_t), (cudaStream_t)stream));
    if (Q == 0) return SVOXB_OK;
    RenderCall c{tree, *opt, Q};
    c.out = out;
    c.stream = (cudaStream_t)stream;
    c.log = log;
    c.log_capacity = capacity_chunks;
    switch (opt->basis_dim) {
        case 1: return launch_queue<1>(c, src);
        case 4: return launch_queue<4>(c, src);
        case 9: return launch_queue<9>(c, src);
        case 16: return launch_queue<16>(c, src);
        case 25: return launch_queue<25>(c, src);
    }
    return SVOXB_ERR_FORMAT;
}

template <class Source>
static int replay_backward(const svoxb_tree* tree, const Source& src, int64_t Q,
                           const svoxb_render_options* opt, const float* grad_output,
                           const float* fwd_out, int32_t* log, int64_t capacity_chunks,
                           int64_t chunks_used, float* grad_data_out, int zero_first,
                           void* stream, bool hess = false) {
    int st = validate_tree(tree);
    if (st) return st;
    if ((st = validate_options(tree, *opt))) return st;
    if (!grad_data_out || !log) return SVOXB_ERR_NULL;
    if ((st = log_eligible(tree, opt, grad_data_out))) return st;
    if (zero_first && (st = zero_grad(tree, grad_data_out, tree->K, (cudaStream_t)stream)))
        return st;
    if (Q == 0) return SVOXB_OK;
    if ((!hess && !grad_output) || !fwd_out) return SVOXB_ERR_NULL;
    RenderCall c{tree, *opt, Q};
    c.backward = true;
    c.grad_out = grad_output;
    c.fwd_out = fwd_out;
    c.grad_data = grad_data_out;
    c.stream = (cudaStream_t)stream;
    c.log = log;
    c.log_capacity = capacity_chunks;
    // chunks_used > 0: the caller has read the count (svoxb_item_log_used) and vouches that
    // the log did not overflow.  Otherwise the count stays on the device: the scratch is sized
    // for the whole log, the kernels read the count themselves, and a marching backward is
    // enqueued behind them that does its work only if the log overflowed.
    const bool known = chunks_used > 0 && chunks_used <= capacity_chunks;
    if (hess && !known) return SVOXB_ERR_OPTION;
    ReplayJob job;
    st = replay_begin(c, src, known ? chunks_used : capacity_chunks, 1, &job, hess);
    if (st == SVOXB_OK) {
        st = replay_scatter(job, 0, grad_data_out, 0, c.stream);
        replay_end(&job, c.stream);
    }
    if (hess) return st;
    RenderCall march = c;
    march.log = nullptr;
    march.log_capacity = 0;
    if (st == SVOXB_ERR_TOO_LARGE) return render_dispatch(march, src);  // no room for packets
    if (st == SVOXB_OK && !known) {
        march.gate = LogGate{log, capacity_chunks};
        st = render_dispatch(march, src);
    }
    return st;
}

extern "C" {

int64_t svoxb_item_log_words(int64_t capacity_chunks) {
    return (int64_t)kLogChunks + capacity_chunks * kLogChunkWords;
}

int svoxb_volume_render_logged(const svoxb_tree* tree, const svoxb_rays* rays,
                               const svoxb_render_options* opt, float* out, int32_t* log,
                               int64_t capacity_chunks, void* stream) {
    if (!tree || !rays || !opt) return SVOXB_ERR_NULL;
    if (rays->Q > 0 && (!rays->origins || !rays->dirs || !rays->vdirs)) return SVOXB_ERR_NULL;
    return logged_forward(tree, RayBatch{rays->origins, rays->dirs, rays->vdirs}, rays->Q, opt,
                          out, log, capacity_chunks, stream);
}

int svoxb_volume_render_image_logged(const svoxb_tree* tree, const svoxb_camera* cam,
                                     const svoxb_render_options* opt, float* out, int32_t* log,
                                     int64_t capacity_chunks, void* stream) {
    if (!tree || !cam || !opt || !cam->c2w) return SVOXB_ERR_NULL;
    if (cam->width < 0 || cam->height < 0) return SVOXB_ERR_SHAPE;
    return logged_forward(tree, PixelRays{cam->c2w, cam->fx, cam->fy, cam->width, cam->height},
                          (int64_t)cam->width * cam->height, opt, out, log, capacity_chunks,
                          stream);
}

int svoxb_volume_render_backward_replay(const svoxb_tree* tree, const svoxb_rays* rays,
                                        const svoxb_render_options* opt,
                                        const float* grad_output, const float* fwd_out,
                                        int32_t* log, int64_t capacity_chunks,
                                        int64_t chunks_used, float* grad_data_out,
                                        int zero_first, void* stream) {
    if (!tree || !rays || !opt) return SVOXB_ERR_NULL;
    if (rays->Q > 0 && (!rays->origins || !rays->dirs || !rays->vdirs)) return SVOXB_ERR_NULL;
    return replay_backward(tree, RayBatch{rays->origins, rays->dirs, rays->vdirs}, rays->Q, opt,
                           grad_output, fwd_out, log, capacity_chunks, chunks_used, grad_data_out,
                           zero_first, stream);
}

int svoxb_volume_render_image_backward_replay(const svoxb_tree* tree, const svoxb_camera* cam,
                                              const svoxb_render_options* opt,
                                              const float* grad_output, const float* fwd_out,
                                              int32_t* log, int64_t capacity_chunks,
                                              int64_t chunks_used, float* grad_data_out,
                                              int zero_first, void* stream) {
    if (!tree || !cam || !opt || !cam->c2w) return SVOXB_ERR_NULL;
    if (cam->width < 0 || cam->height < 0) return SVOXB_ERR_SHAPE;
    return replay_backward(tree, PixelRays{cam->c2w, cam->fx, cam->fy, cam->width, cam->height},
                           (int64_t)cam->width * cam->height, opt, grad_output, fwd_out, log,
                           capacity_chunks, chunks_used, grad_data_out, zero_first, stream);
}

/* Gauss-Newton diagonal of the squared error from the item log (the third result of the
 * reference's se_grad, svox/csrc/rt_kernel.cu:479-715, 1111-1173). */
int svoxb_volume_render_hessdiag_replay(const svoxb_tree* tree, const svoxb_rays* rays,
                                        const svoxb_render_options* opt, const float* fwd_out,
                                        int32_t* log, int64_t capacity_chunks,
                                        int64_t chunks_used, float* hessdiag_out,
                                        int zero_first, void* stream) {
    if (!tree || !rays || !opt) return SVOXB_ERR_NULL;
    if (rays->Q > 0 && (!rays->origins || !rays->dirs || !rays->vdirs)) return SVOXB_ERR_NULL;
    return replay_backward(tree, RayBatch{rays->origins, rays->dirs, rays->vdirs}, rays->Q, opt,
                           nullptr, fwd_out, log, capacity_chunks, chunks_used, hessdiag_out,
                           zero_first, stream, true);
}

int svoxb_volume_render_image_hessdiag_replay(const svoxb_tree* tree, const svoxb_camera* cam,
                                              const svoxb_render_options* opt,
                                              const float* fwd_out, int32_t* log,
                                              int64_t capacity_chunks, int64_t chunks_used,
                                              float* hessdiag_out, int zero_first,
                                              void* stream) {
    if (!tree || !cam || !opt || !cam->c2w) return SVOXB_ERR_NULL;
    if (cam->width < 0 || cam->height < 0) return SVOXB_ERR_SHAPE;
    return replay_backward(tree, PixelRays{cam->c2w, cam->fx, cam->fy, cam->width, cam->height},
                           (int64_t)cam->width * cam->height, opt, nullptr, fwd_out, log,
                           capacity_chunks, chunks_used, hessdiag_out, zero_first, stream, true);
}

}  // extern "C"

// se_grad by marching (any record layout the generic kernels take): gradient and
// Gauss-Newton diagonal of the squared error from the forward's output.
template <class Source>
static int se_grad_march(const svoxb_tree* tree, const Source& src, int64_t Q,
                         const svoxb_render_options* opt, const float* fwd_out,
                         const float* color_ref, float* grad, float* hess, int zero_first,
                         cudaStream_t stream) {
    int st = validate_tree(tree);
    if (st) return st;
    if ((st = validate_options(tree, *opt))) return st;
    if (Q < 0) return SVOXB_ERR_SHAPE;
    if (!grad || !hess || (Q > 0 && (!fwd_out || !color_ref))) return SVOXB_ERR_NULL;
    const int od = out_dim_of(tree, *opt);
    if (od > kMaxSeGradOut) return SVOXB_ERR_FORMAT;
    if (zero_first) {
        if ((st = zero_grad(tree, grad, tree->K, stream))) return st;
        if ((st = zero_grad(tree, hess, tree->K, stream))) return st;
    }
    if (Q == 0) return SVOXB_OK;
    TopScratch scratch;
    if ((st = scratch.build(tree, 5, stream))) return st;
    const TopTable top{scratch.cells, scratch.level};
    const bool in_smem = scratch.level > 0 && scratch.level <= 5;
    const size_t smem = in_smem ? ((size_t)4 << (3 * scratch.level)) : 0;
    const TreeArgs tr = tree_args(tree);
    const int64_t n_gran = (Q + 31) / 32;
    unsigned grid = 1;
    auto run = [&](auto k, int block) {
        int s2 = persistent_grid(k, block, smem, n_gran, &grid);
        if (s2) return s2;
        k<<<grid, block, smem, stream>>>(tr, src, *opt, top, in_smem, fwd_out, color_ref, grad,
                                        hess, Q, od);
        const cudaError_t e = cudaGetLastError();
        return e != cudaSuccess ? set_cuda_error(e) : (int)SVOXB_OK;
    };
    return smem > 64 * 1024 ? run(render_se_grad_generic<1024, Source>, 1024)
                            : run(render_se_grad_generic<256, Source>, 256);
}

extern "C" {

int svoxb_se_grad_march(const svoxb_tree* tree, const svoxb_rays* rays,
                        const svoxb_render_options* opt, const float* fwd_out,
                        const float* color_ref, float* grad_data_out, float* hessdiag_out,
                        int zero_first, void* stream) {
    if (!tree || !rays || !opt) return SVOXB_ERR_NULL;
    if (rays->Q > 0 && (!rays->origins || !rays->dirs || !rays->vdirs)) return SVOXB_ERR_NULL;
    return se_grad_march(tree, RayBatch{rays->origins, rays->dirs, rays->vdirs}, rays->Q, opt,
                         fwd_out, color_ref, grad_data_out, hessdiag_out, zero_first,
                         (cudaStream_t)stream);
}

int svoxb_se_grad_image_march(const svoxb_tree* tree, const svoxb_camera* cam,
                              const svoxb_render_options* opt, const float* fwd_out,
                              const float* color_ref, float* grad_data_out, float* hessdiag_out,
                              int zero_first, void* stream) {
    if (!tree || !cam || !opt || !cam->c2w) return SVOXB_ERR_NULL;
    if (cam->width < 0 || cam->height < 0) return SVOXB_ERR_SHAPE;
    return se_grad_march(tree, PixelRays{cam->c2w, cam->fx, cam->fy, cam->width, cam->height},
                         (int64_t)cam->width * cam->height, opt, fwd_out, color_ref,
                         grad_data_out, hessdiag_out, zero_first, (cudaStream_t)stream);
}

}  // extern "C"

template <class Source>
static int replay_begin_checked(const svoxb_tree* tree, const Source& src, int64_t Q,
                                const svoxb_render_options* opt, const float* grad_output,
                                const float* fwd_out, int32_t* log, int64_t capacity_chunks,
                                int64_t chunks_used, int n_parts, float* grad_data_out,
                                void* stream, void** job_out) {
    if (!job_out) return SVOXB_ERR_NULL;
    *job_out = nullptr;
    int st = validate_tree(tree);
    if (st) return st;
    if ((st = validate_options(tree, *opt))) return st;
    if (!log || !grad_data_out || (Q > 0 && (!grad_output || !fwd_out))) return SVOXB_ERR_NULL;
    if ((st = log_eligible(tree, opt, grad_data_out))) return st;
    RenderCall c{tree, *opt, Q};
    c.backward = true;
    c.grad_out = grad_output;
    c.fwd_out = fwd_out;
    c.stream = (cudaStream_t)stream;
    c.log = log;
    c.log_capacity = capacity_chunks;
    const bool known = chunks_used > 0 && chunks_used <= capacity_chunks;
    if (!known) chunks_used = capacity_chunks;
    if (Q == 0) chunks_used = 0;
    ReplayJob* job = new (std::nothrow) ReplayJob;
    if (!job) return SVOXB_ERR_TOO_LARGE;
    st = replay_begin(c, src, chunks_used, n_parts, job);
    if (st == SVOXB_OK && !known && Q > 0) {
        // the fallback for an overflowed log goes BEFORE the parts: if it runs, it produces the
        // whole gradient and the parts add nothing, so every part's rows are final when the
        // caller hands them on, whichever of the two happened
        RenderCall march = c;
        march.grad_data = grad_data_out;
        march.log = nullptr;
        march.log_capacity = 0;
        march.gate = LogGate{log, capacity_chunks};
        st = render_dispatch(march, src);
        if (st != SVOXB_OK) replay_end(job, c.stream);
    }
    if (st != SVOXB_OK) {
        delete job;
        return st;
    }
    *job_out = job;
    return SVOXB_OK;
}

extern "C" {

int svoxb_replay_begin(const svoxb_tree* tree, const svoxb_rays* rays,
                       const svoxb_render_options* opt, const float* grad_output,
                       const float* fwd_out, int32_t* log, int64_t capacity_chunks,
                       int64_t chunks_used, int n_parts, float* grad_data_out, void* stream,
                       void** job) {
    if (!tree || !rays || !opt) return SVOXB_ERR_NULL;
    if (rays->Q > 0 && (!rays->origins || !rays->dirs || !rays->vdirs)) return SVOXB_ERR_NULL;
    return replay_begin_checked(tree, RayBatch{rays->origins, rays->dirs, rays->vdirs}, rays->Q,
                                opt, grad_output, fwd_out, log, capacity_chunks, chunks_used,
                                n_parts, grad_data_out, stream, job);
}

int svoxb_replay_image_begin(const svoxb_tree* tree, const svoxb_camera* cam,
                             const svoxb_render_options* opt, const float* grad_output,
                             const float* fwd_out, int32_t* log, int64_t capacity_chunks,
                             int64_t chunks_used, int n_parts, float* grad_data_out,
                             void* stream, void** job) {
    if (!tree || !cam || !opt || !cam->c2w) return SVOXB_ERR_NULL;
    if (cam->width < 0 || cam->height < 0) return SVOXB_ERR_SHAPE;
    return replay_begin_checked(tree,
                                PixelRays{cam->c2w, cam->fx, cam->fy, cam->width, cam->height},
                                (int64_t)cam->width * cam->height, opt, grad_output, fwd_out, log,
                                capacity_chunks, chunks_used, n_parts, grad_data_out, stream, job);
}

int svoxb_replay_bin_shift(int64_t M, int32_t K) {
    if (M < 1 || K < 1) return 0;
    return replay_bin_shift(M, K);
}

int svoxb_replay_part_range(const void* job, int part, int64_t* slot_begin, int64_t* slot_end) {
    if (!job || !slot_begin || !slot_end) return SVOXB_ERR_NULL;
    const ReplayJob* j = static_cast<const ReplayJob*>(job);
    if (part < 0 || part >= j->n_parts) return SVOXB_ERR_OPTION;
    const int64_t lo = (int64_t)replay_part_first_bin(part, j->n_parts, j->n_bins) << j->shift;
    int64_t hi = (int64_t)replay_part_first_bin(part + 1, j->n_parts, j->n_bins) << j->shift;
    if (hi > j->n_slots) hi = j->n_slots;
    *slot_begin = lo < j->n_slots ? lo : j->n_slots;
    *slot_end = hi;
    return SVOXB_OK;
}

int svoxb_replay_scatter(const void* job, int part, float* grad_data_out, int reserve_sms,
                         void* stream) {
    if (!job || !grad_data_out) return SVOXB_ERR_NULL;
    const ReplayJob* j = static_cast<const ReplayJob*>(job);
    if (j->K % 4 == 0 && (uintptr_t)grad_data_out % 16 != 0) return SVOXB_ERR_FORMAT;
    return replay_scatter(*j, part, grad_data_out, reserve_sms, (cudaStream_t)stream);
}

int svoxb_replay_end(void* job, void* stream) {
    if (!job) return SVOXB_ERR_NULL;
    ReplayJob* j = static_cast<ReplayJob*>(job);
    replay_end(j, (cudaStream_t)stream);
    delete j;
    return SVOXB_OK;
}

int svoxb_item_log_used(const int32_t* log, int64_t* chunks_used, void* stream) {
    if (!log || !chunks_used) return SVOXB_ERR_NULL;
    int32_t used = 0;
    SVOXB_CUDA(cudaMemcpyAsync(&used, log, sizeof(int32_t), cudaMemcpyDeviceToHost,
                               (cudaStream_t)stream));
    SVOXB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    *chunks_used = used;
    return SVOXB_OK;
}

int svoxb_march_stats(const svoxb_tree* tree, const svoxb_rays* rays,
                      const svoxb_render_options* opt, int32_t* visits, int32_t* contrib_fwd,
                      int32_t* contrib_bwd, void* stream) {
    if (!tree || !rays || !opt) return SVOXB_ERR_NULL;
    if (rays->Q > 0 && (!rays->origins || !rays->dirs || !rays->vdirs)) return SVOXB_ERR_NULL;
    int st = validate_tree(tree);
    if (st) return st;
    if (!(opt->step_size >= 0.f)) return SVOXB_ERR_OPTION;
    if (rays->Q < 0) return SVOXB_ERR_SHAPE;
    if (rays->Q == 0) return SVOXB_OK;
    cudaStream_t s = (cudaStream_t)stream;
    TopScratch scratch;
    if ((st = scratch.build(tree, 4, s))) return st;
    const TopTable top{scratch.cells, scratch.level};
    const bool in_smem = scratch.level > 0;
    const size_t smem = in_smem ? ((size_t)4 << (3 * scratch.level)) : 0;
    auto k = march_stats_kernel<256, RayBatch>;
    unsigned grid = 1;
    if ((st = persistent_grid(k, 256, smem, (rays->Q + 31) / 32, &grid))) return st;
    k<<<grid, 256, smem, s>>>(tree_args(tree), RayBatch{rays->origins, rays->dirs, rays->vdirs},
                             *opt, top, in_smem, visits, contrib_fwd, contrib_bwd, rays->Q);
    SVOXB_CUDA(cudaGetLastError());
    return SVOXB_OK;
}

int svoxb_device_status(int clear, void* stream) {
    int word = 0;
    SVOXB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    SVOXB_CUDA(cudaMemcpyFromSymbol(&word, g_status, sizeof(int)));
    if (clear && word != 0) {
        const int zero = 0;
        SVOXB_CUDA(cudaMemcpyToSymbol(g_status, &zero, sizeof(int)));
    }
    return word;
}

const char* svoxb_strerror(int status) {
    switch (status) {
        case SVOXB_OK: return "ok";
        case SVOXB_ERR_NULL: return "a required pointer is null";
        case SVOXB_ERR_SHAPE: return "inconsistent or negative size";
        case SVOXB_ERR_FORMAT: return "data format / record layout not supported";
        case SVOXB_ERR_OPTION: return "invalid render option";
        case SVOXB_ERR_CUDA: return "CUDA runtime error";
        case SVOXB_ERR_TREE: return "corrupt tree: a descent left the node array";
        case SVOXB_ERR_MARCH: return "a ray exceeded the marching step cap";
        case SVOXB_ERR_TOO_LARGE: return "size beyond the supported maximum";
    }
    return "unknown status";
}

const char* svoxb_last_cuda_error(void) { return t_cuda_error; }

int svoxb_reserve_sms(int n) {
    const int before = g_reserved_sms;
    if (n >= 0) g_reserved_sms = n;
    return before;
}

int svoxb_allreduce_multimem(float* multicast, int64_t n_floats, int rank, int world,
                             void* stream) {
    if (!multicast) return SVOXB_ERR_NULL;
    if (world < 1 || rank < 0 || rank >= world || n_floats < 0) return SVOXB_ERR_OPTION;
    if ((uintptr_t)multicast % 16 != 0 || n_floats % 4 != 0) return SVOXB_ERR_SHAPE;
    const int64_t words = n_floats / 4;
    const int64_t first = words * rank / world, last = words * (rank + 1) / world;
    if (last <= first) return SVOXB_OK;
    int sms = sm_count() - g_reserved_sms;
    if (sms < 1) sms = 1;
    int64_t grid = (last - first + kReduceBlock - 1) / kReduceBlock;
    if (grid > 2 * sms) grid = 2 * sms;
    multimem_allreduce_kernel<<<(unsigned)grid, kReduceBlock, 0, (cudaStream_t)stream>>>(
        multicast, first, last);
    SVOXB_CUDA(cudaGetLastError());
    return SVOXB_OK;
}

const char* svoxb_version(void) { return "0.3.0"; }

// Test hook (include/svox_b200_testing.h): key 5 = MB of gradient one replay bin spans,
// key 7 = bricks below the render leaf table on / off.
int svoxb_test_knob(int key, int value) {
    switch (key) {
        case 7: g_tuning.render_bricks = value != 0; return SVOXB_OK;
        case 5:
            if (value < 1 || value > 1024) return SVOXB_ERR_OPTION;
            g_tuning.replay_bin_mb = value;
            return SVOXB_OK;
    }
    return SVOXB_ERR_OPTION;
}

}  // extern "C"

#include "noalloc.cuh"
