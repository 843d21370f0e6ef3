// Queue-based warp-cooperative volume rendering for octrees (N = 2) with SH
// colour in three channels (record K = 3 * basis_dim + 1): forward, and
// backward in one or two marches.
//
// The path is bound by memory LATENCY (dependent loads of the descent, then
// the record fetch), not by arithmetic, so the kernel is organised to expose
// at most one L2 round trip per loop iteration and no HBM round trip at all:
//
//   G step  one lane = one ray.  Every iteration consumes ONE child entry that
//           was requested during the previous iteration (software-pipelined):
//           an inner node moves the lane's cursor one level down; a leaf is
//           sampled (step length, density, transmittance, weight), the ray
//           advances, and the cursor of the next sample restarts at the leaf
//           table, or, while the ray stays inside the same table cell, at the
//           cell's BRICK, which resolves three more levels with one load (see
//           below).  Lanes never wait for another lane's longer descent.  The descent reads an ANNOTATED copy of the child
//           array whose leaf entries carry the density of leaves that pass
//           the density test (annotate_sigma_kernel, built per call), so the
//           march itself runs out of L2-resident data and empty leaves never
//           touch HBM.  A contributing sample is pushed as an ITEM (leaf slot,
//           weight, ...) into the warp's queue in shared memory.
//   S step  one lane = one item.  When 32 items are queued their records are
//           requested with cp.async (coalesced 16-byte pieces, global ->
//           shared staging rows) and the warp goes on marching; the batch is
//           evaluated when the next one is full, by which time the data has
//           arrived.  Lane i evaluates item i (SH dot products, sigmoids) with
//           the owner ray's basis; then every owner folds the results of its
//           own items into its ray state in march order, which keeps the
//           reference's order of accumulation (svox/csrc/rt_kernel.cu:282-295,
//           379-411, 442-471).  In the backward pass lane i forms the gradient
//           of record i in its staging row and groups of lanes flush the rows
//           with red.global.add.v4.f32, 16 bytes per lane.
//
// Lanes whose ray has ended refill from a block-wide ticket counter.  All
// control flow around warp-level primitives is driven by votes.
#pragma once

#include "render.cuh"

namespace svoxb {

constexpr int kModeForward = 0;
constexpr int kModeBackward = 1;
constexpr int kModeForwardLogged = 2;  // forward that also records its items for the backward

// Mark in the annotated child array: a leaf that passes the density test but
// whose density cannot ride in the entry itself.
constexpr int32_t kOccupied = INT32_MIN;

// How the lanes of a warp move K-float records between global memory and the
// per-item staging rows in shared memory.
template <int K>
struct RecordShape {
    static constexpr bool VEC = (K % 4 == 0);            // 16-byte words possible
    static constexpr int WORDS = VEC ? K / 4 : K;         // words per record
    static constexpr int GROUP = WORDS <= 1 ? 1 : WORDS <= 2 ? 2 : WORDS <= 4 ? 4
                                 : WORDS <= 8 ? 8 : WORDS <= 16 ? 16 : 32;  // lanes per item
    static constexpr int IPP = 32 / GROUP;                // items per pass
    static constexpr int WPL = (WORDS + GROUP - 1) / GROUP;  // words per lane per item
    // staging row stride in floats: 16-byte rows for vector access, odd
    // otherwise (both conflict-free for the owner's reads)
    static constexpr int STRIDE = VEC ? K : (K | 1);
};

// Item log: what a logged forward leaves behind so that the backward pass can
// replay the contributing samples without marching again and without reading
// the leaf records a second time.  int32 words:
//   [0] chunks allocated   [2] bin shift   [3] number of bins
//   [kLogHeads + b]        items whose leaf slot falls into bin b (= slot >> shift)
//   chunk c at kLogChunks + c * kLogChunkWords: 12 rows of 32 words,
//     row 0: word 0 = items in the chunk
//     rows 1-11, one word per item: slot, ray, weight, T after, delta_t*delta_scale
//     (times the derivative of the density's softplus, if that is on), sigmoid of the
//     three channels, colour sums of the ray up to and including the item (three channels)
// With the partial colour sums every item is self-contained: the reference's
// running `accum` after item k (svox/csrc/rt_kernel.cu:462-471) equals
// <grad_out, out> - <grad_out, partial sums>, so the backward can take the
// items in any order.
constexpr int kLogHeads = 32;
constexpr int kMaxBins = 1024;
constexpr int kLogChunks = kLogHeads + kMaxBins;
constexpr int kLogRows = 12;
constexpr int kLogChunkWords = kLogRows * 32;
constexpr int kLogGrab = 8;  // chunks a warp takes per bump of the allocation counter

// A launch that is a FALLBACK for an overflowed item log: its kernels do their work only if
// the logged forward needed more chunks than the log holds (word 0 of the log counts the
// chunks it asked for), so the host can enqueue replay and fallback without knowing which of
// the two applies.  `log` null: unconditional.
struct LogGate {
    const int32_t* log = nullptr;
    int64_t capacity = 0;
    __device__ __forceinline__ bool closed() const {
        return log != nullptr && (int64_t)__ldg(log) <= capacity;
    }
};

constexpr int kCoordBits = 24;  // integer coordinates: floor(x * 2^24), exact for float x < 1

// Bricks: every inner cell of the leaf table gets the 8x8x8 grid of the three
// levels below it: 512 CELL words followed by 64 GROUP words (one per 2x2x2
// group of fine cells), 2304 bytes per brick.
//   cell   the annotated child entry of the leaf that covers the fine cell (<= 0), or, if
//          the tree goes deeper there, the link (> 0) from the group's node to the child
//   group  bits 28-29 = k, bits 0-27 = payload: k = 2: the group's fine cells are the
//          children of node `payload`; k = 1 / k = 0: the whole group lies in a leaf one /
//          two levels up, whose slot is `payload`
// A table cell with a brick holds kBrickFlag + brick id instead of the node id.
// Samples in refined regions then cost one round trip (two independent loads),
// like samples in empty space; trees deeper than table level + 3 continue from
// the brick entry through the annotated child array.  Table cells beyond the
// brick budget keep their node id and are walked level by level.
constexpr int kBrickLevels = 3;
constexpr int kBrickCells = 512;
constexpr int kBrickWords = kBrickCells + 64;
constexpr int32_t kBrickFlag = 1 << 30;
constexpr int64_t kBrickMaxNodes = 1 << 25;  // slots must fit 28 bits
constexpr int kMaxBricks = 1 << 17;

// Annotated child entry: > 0 link; 0 leaf failing the density test; < 0 leaf
// passing it, with the density's float bits in the low 31 bits when the
// density is a non-negative float that needs no softplus, else kOccupied
// (the reader then fetches the density from the record).
__global__ void annotate_sigma_kernel(const int32_t* __restrict__ child,
                                      const float* __restrict__ data, int K, int64_t n_slots,
                                      float thresh, int softplus, int32_t* __restrict__ out,
                                      LogGate gate) {
    if (gate.closed()) return;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_slots;
         i += (int64_t)gridDim.x * blockDim.x) {
        int32_t c = child[i];
        if (c == 0) {
            const float raw = __ldg(data + i * K + (K - 1));
            const float sigma = softplus ? softplus_m1(raw) : raw;
            if (sigma > thresh)
                c = (!softplus && raw >= 0.f) ? (int32_t)(0x80000000u | __float_as_uint(raw))
                                              : kOccupied;
        }
        out[i] = c;
    }
}

// Grid of an index-building kernel over n items: enough blocks to fill the device, not one
// per 256 items (a launch that finds its gate closed should cost next to nothing).
inline unsigned index_grid(int64_t n, int block, int sms) {
    const int64_t need = (n + block - 1) / block, most = (int64_t)sms * (2048 / block) * 2;
    return (unsigned)(need < most ? (need > 0 ? need : 1) : most);
}

// L2 residency hints.  The annotated child array (tens of MB, re-read hundreds
// of times per launch) must stay in L2 while the leaf records and gradients
// (GBs, touched a few times each) stream through it; without hints the stream
// evicts a third of the child entries and every descent step waits on HBM.
__device__ __forceinline__ uint64_t l2_policy_keep() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_stream() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ int32_t ld_keep(const int32_t* a, uint64_t pol) {
    int32_t v;
    asm volatile("ld.global.nc.L2::cache_hint.s32 %0, [%1], %2;" : "=r"(v) : "l"(a), "l"(pol));
    return v;
}
__device__ __forceinline__ void st_stream(int32_t* a, int32_t v, uint64_t pol) {
    asm volatile("st.global.L2::cache_hint.s32 [%0], %1, %2;" ::"l"(a), "r"(v), "l"(pol) : "memory");
}
// The 64-byte L2 fetch granularity is a measured choice: records are 112-196 bytes at arbitrary
// 16-byte offsets, and the logged forward of the training step runs 1 % faster with it than with the
// default granularity and 6 % faster than with 256 bytes.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, uint64_t pol) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global.L2::cache_hint.L2::64B [%0], [%1], 16, %2;" ::"r"(s),
                 "l"(gmem), "l"(pol)
                 : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem, uint64_t pol) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global.L2::cache_hint [%0], [%1], 4, %2;" ::"r"(s),
                 "l"(gmem), "l"(pol)
                 : "memory");
}
__device__ __forceinline__ void red_add_v4_hint(float* addr, float a, float b, float c, float d,
                                                uint64_t pol) {
    asm volatile("red.global.add.L2::cache_hint.v4.f32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(addr),
                 "f"(a), "f"(b), "f"(c), "f"(d), "l"(pol)
                 : "memory");
}
// Leaf table over the top `level` levels of the annotated tree, one int32 per
// cell of the 2^level cube, in global memory (1 MB at level 6, kept in L2):
//   > 0          id of the node at that level (its children are the next level's cells)
//   -d (d >= 1)  the cell lies in a leaf of depth d that fails the density test:
//                a sample there needs no further look-up at all
//   kTabDescend  anything else (a shallow leaf that passes the test): walk from the root
// Most samples of a sparse scene fall into empty space; with this table each of
// them costs exactly one dependent load.
constexpr int32_t kTabDescend = INT32_MIN;

__global__ void build_leaf_table_kernel(const int32_t* __restrict__ annotated, int64_t M, int L,
                                        int32_t* __restrict__ cells, LogGate gate) {
    if (gate.closed()) return;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < (1 << (3 * L));
         idx += gridDim.x * blockDim.x) {
        const int S = (1 << L) - 1;
        const int iz = idx & S, iy = (idx >> L) & S, ix = idx >> (2 * L);
        int64_t node = 0;
        int32_t entry = 0;
        for (int l = L - 1; l >= 0; --l) {
            const int u = (ix >> l) & 1, v = (iy >> l) & 1, w = (iz >> l) & 1;
            const int32_t e = annotated[node * 8 + (u * 4 + v * 2 + w)];
            if (e <= 0) {
                entry = (e == 0) ? -(L - l) : kTabDescend;
                node = -1;
                break;
            }
            node += e;
            if (node >= M) { entry = kTabDescend; node = -1; break; }
        }
        cells[idx] = node >= 0 ? (int32_t)node : entry;
    }
}

// Gives every table cell that holds a node a brick while the budget lasts.
__global__ void assign_bricks_kernel(int32_t* __restrict__ cells, int n_cells, int cap,
                                     int32_t* __restrict__ counter, int32_t* __restrict__ roots,
                                     LogGate gate) {
    if (gate.closed()) return;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < n_cells;
         idx += gridDim.x * blockDim.x) {
        const int32_t e = cells[idx];
        if (e <= 0) continue;
        const int id = atomicAdd(counter, 1);
        if (id >= cap) continue;
        roots[id] = e;
        cells[idx] = kBrickFlag + id;
    }
}

// One block per brick, one thread per fine cell.
__global__ void __launch_bounds__(kBrickCells)
fill_bricks_kernel(const int32_t* __restrict__ annotated, int64_t M, int L, int cap,
                   const int32_t* __restrict__ counter, const int32_t* __restrict__ roots,
                   int32_t* __restrict__ bricks, LogGate gate) {
    if (gate.closed()) return;
    int n = *counter;
    if (n > cap) n = cap;
    const int c = threadIdx.x;
    const int x = c >> 6, y = (c >> 3) & 7, z = c & 7;
    for (int b = blockIdx.x; b < n; b += gridDim.x) {
        int64_t node = roots[b];
        int32_t cell_word = 0;
        uint32_t group_word = 0;
        bool done = false;
        for (int l = 0; l < kBrickLevels && !done; ++l) {
            const int sh = kBrickLevels - 1 - l;
            const int cell = (((x >> sh) & 1) << 2) | (((y >> sh) & 1) << 1) | ((z >> sh) & 1);
            const int32_t e = annotated[node * 8 + cell];
            if (l == kBrickLevels - 1) {
                // fine cell: leaf code or link, both relative to the group's node
                cell_word = e;
                if (e > 0 && node + e >= M) cell_word = (int32_t)(M - node);  // reported by the march
                group_word = (2u << 28) | (uint32_t)node;
                done = true;
            } else if (e <= 0) {
                cell_word = e;
                group_word = ((uint32_t)l << 28) | (uint32_t)(node * 8 + cell);
                done = true;
            } else {
                node += e;
                if (node >= M) {  // corrupt link: reported by the march via an out-of-range link
                    cell_word = 1;
                    group_word = (2u << 28) | (uint32_t)(M - 1);
                    done = true;
                }
            }
        }
        int32_t* brick = bricks + (size_t)b * kBrickWords;
        brick[c] = cell_word;
        if (((x | y | z) & 1) == 0)
            brick[kBrickCells + ((x >> 1) << 4 | (y >> 1) << 2 | (z >> 1))] = (int32_t)group_word;
    }
}

// Shared memory of one warp.
template <int K, int MODE>
struct alignas(16) WarpQueue {
    static constexpr bool BWD = MODE == kModeBackward;
    static constexpr bool LOG = MODE == kModeForwardLogged;
    using Shape = RecordShape<K>;
    static constexpr int CAP = 96;  // a batch in flight (32) + items being collected (< 64)
    static constexpr int BD = (K - 1) / 3;
    static constexpr int RAYW = (BD + (BWD ? 3 : 0)) | 1;  // odd stride: no bank conflicts
    uint32_t slot[CAP];
    float w[CAP];                   // weight T * (1 - att)
    float T[(BWD || LOG) ? CAP : 4];   // transmittance after the sample
    float dd[(BWD || LOG) ? CAP : 4];  // delta_t * delta_scale
    int rayid[LOG ? CAP : 4];          // ray of the item (logged forward)
    unsigned char owner[CAP];       // bits 0-4 owner lane, bit 5 ray parity, bit 7 accumulation march
    float rayv[2][32][RAYW];        // per lane and ray parity: SH basis [0,BD), upstream gradient
    float oldv[BWD ? 1 : 32][4];    // forward: colour sums and transmittance of the previous ray
    long long oldray[BWD ? 1 : 32];
    unsigned char oldstop[BWD ? 4 : 32];
    // Staging rows (cp.async targets).  After lane i has read row i it reuses the
    // row's first words for the item's results.
    alignas(16) float rows[32 * Shape::STRIDE + 4];
};

enum { kNeedRay = 0, kMarching = 1, kDraining = 2, kExhausted = 3 };
enum { kFromChild = 0, kFromTable = 1, kFromBrick = 2 };

template <int BD, int BLOCK, int MODE, class Source>
__global__ void __launch_bounds__(BLOCK)
render_queue_kernel(TreeArgs tr, Source src, svoxb_render_options opt, TopTable topg,
                    int top_bytes, int64_t Q, float* __restrict__ out,
                    const float* __restrict__ grad_out, const float* __restrict__ fwd_out,
                    float* __restrict__ grad_data, int32_t* __restrict__ log,
                    int64_t log_capacity, int log_shift, int refill_batch) {
    constexpr int K = 3 * BD + 1;
    constexpr bool BWD = MODE == kModeBackward;
    constexpr bool LOG = MODE == kModeForwardLogged;
    using WQ = WarpQueue<K, MODE>;
    using Shape = RecordShape<K>;
    static_assert(Shape::STRIDE >= 3, "result words live in the staging row");
    extern __shared__ __align__(16) unsigned char s_raw[];
    __shared__ unsigned s_next;
    __shared__ int s_hist[LOG ? kMaxBins : 1];  // logged forward: items per bin
    // backward with a log: the marching fallback of a replay, needed only if the log overflowed
    if (BWD && LogGate{log, log_capacity}.closed()) return;
    if (threadIdx.x == 0) s_next = 0;
    if (LOG) {
        for (int i = threadIdx.x; i < kMaxBins; i += BLOCK) s_hist[i] = 0;
        if (blockIdx.x == 0 && threadIdx.x == 0) {
            log[2] = log_shift;
            log[3] = (int)(((tr.M * 8 - 1) >> log_shift) + 1);
        }
    }
    const TopTable top = topg;  // leaf table in global memory (top_bytes is 0)
    const int lane = threadIdx.x & 31;
    WQ& q = *reinterpret_cast<WQ*>(s_raw + top_bytes + (size_t)(threadIdx.x >> 5) * sizeof(WQ));
    __syncthreads();
    const float d_rgb_pad = 1 + 2 * opt.rgb_padding;
    const bool single = BWD && fwd_out != nullptr;
    const float bg = opt.background_brightness;
    const int sub = lane / Shape::GROUP, wj = lane % Shape::GROUP;
    const int32_t* __restrict__ child = tr.child;
    const int M = (int)tr.M;
    const int base = top.level;  // level of the jump table (0: none)
    const float big = (float)(1 << kCoordBits);
    const uint64_t pol_keep = l2_policy_keep(), pol_stream = l2_policy_stream();
    // records stream through L2 (evict-first): measured 0.2 ms faster per launch than the
    // default policy and than evict-last, which push the tree's index out of L2
    const uint64_t pol_rec = pol_stream;

    // ---- per-lane state -------------------------------------------------------
    // A lane marches one ray (the CURRENT one) and may still have items queued for
    // the ray it marched before (the OLD one): a finished ray hands its partial
    // result over and the lane refills at once instead of waiting for the queue.
    Ray r;
    r.hit = false;
    int64_t ray = 0;
    int state = kNeedRay;
    float t = 0.f, light = 1.f;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f;  // forward: colour sums of the current ray
    float accum = 0.f, accum_old = 0.f;   // backward
    bool stopped = false;
    int par = 0;                 // parity tag of the current ray's items
    int cnt_cur = 0, cnt_old = 0;  // queued items of the current / old ray
    bool old_valid = false;
    int phase = 1;  // backward: 0 = accumulation march (reference PASS 1), 1 = scatter march
    int it = 0;
    // cursor of the descent in progress
    int node = 0, lvl = 0, ix = 0, iy = 0, iz = 0;
    float px = 0.f, py = 0.f, pz = 0.f;
    int32_t e_pre = 0, e_aux = 0;  // entry at the cursor, requested one iteration ahead ...
    int kind = kFromChild;         // ... from the annotated child array, the leaf table or a brick
    int tab_idx = 0;
    int cur_cell = -1, cur_brick = -1;  // table cell of the last brick used, and that brick
    unsigned mine_lo = 0u;              // my items among queue positions [0, 32)
    unsigned long long mine_hi = 0ull;  // ... among [32, 96)
    int qn = 0;                         // queued items (warp-uniform)
    bool inflight = false;              // records of items [0, 32) have been requested
    // logged forward: the warp takes kLogGrab chunks at a time from the log
    int64_t log_chunk = 0;
    int log_left = 0;

    // Places the cursor for the sample at parameter t: at the brick of the table cell
    // the ray is in if that is the brick used last, else at the leaf table.
    auto place_cursor = [&]() {
        px = clamp01(mad_site<FC_POS>(t, r.dx, r.ox));
        py = clamp01(mad_site<FC_POS>(t, r.dy, r.oy));
        pz = clamp01(mad_site<FC_POS>(t, r.dz, r.oz));
        ix = (int)(px * big); iy = (int)(py * big); iz = (int)(pz * big);
        node = 0;
        lvl = 0;
        kind = kFromChild;
        if (base > 0) {
            const int sh = kCoordBits - base;
            tab_idx = ((((ix >> sh) << base) + (iy >> sh)) << base) + (iz >> sh);
            kind = (tab_idx == cur_cell && cur_brick >= 0) ? kFromBrick : kFromTable;
        }
    };

    // Requests the entry at the cursor.
    auto request_entry = [&]() {
        if (kind == kFromBrick) {
            const int sh = kCoordBits - base - kBrickLevels;
            const int x = (ix >> sh) & 7, y = (iy >> sh) & 7, z = (iz >> sh) & 7;
            const int32_t* brick = top.bricks + (size_t)cur_brick * kBrickWords;
            e_pre = ld_keep(brick + ((x << 6) | (y << 3) | z), pol_keep);
            e_aux = ld_keep(brick + kBrickCells + (((x >> 1) << 4) | ((y >> 1) << 2) | (z >> 1)),
                            pol_keep);
        } else if (kind == kFromTable) {
            e_pre = ld_keep(top.cells + tab_idx, pol_keep);
        } else {
            const int b = kCoordBits - 1 - lvl;
            const int cell = (((ix >> b) & 1) << 2) | (((iy >> b) & 1) << 1) | ((iz >> b) & 1);
            e_pre = ld_keep(child + ((uint32_t)node * 8u + (uint32_t)cell), pol_keep);
        }
    };

    // Writes the result of a finished forward ray.
    auto write_out = [&](int64_t ry, float c0, float c1, float c2, float lt, bool stp) {
        if (stp) {
            const float scale = 1.0 / (1.0 - lt);
            out[3 * ry + 0] = c0 * scale; out[3 * ry + 1] = c1 * scale; out[3 * ry + 2] = c2 * scale;
        } else {
            out[3 * ry + 0] = c0 + lt * bg; out[3 * ry + 1] = c1 + lt * bg; out[3 * ry + 2] = c2 + lt * bg;
        }
    };

    // Evaluates the first nb queued items, whose records are in the staging rows.
    auto evaluate = [&](int nb) {
        float sg[3] = {0.f, 0.f, 0.f};
        float raw_sigma = 0.f;
        int own = lane, opar = 0;
        bool acc_item = false;
        if (lane < nb) {
            const int ob = q.owner[lane];
            own = ob & 31;
            opar = (ob >> 5) & 1;
            acc_item = (ob & 0x80) != 0;
            float* row = q.rows + lane * Shape::STRIDE;
            float bs[BD];
#pragma unroll
            for (int i = 0; i < BD; ++i) bs[i] = q.rayv[opar][own][i];
            float v[K];
            if (Shape::VEC) {
#pragma unroll
                for (int w = 0; w < K / 4; ++w) {
                    const float4 x = reinterpret_cast<const float4*>(row)[w];
                    v[4 * w] = x.x; v[4 * w + 1] = x.y; v[4 * w + 2] = x.z; v[4 * w + 3] = x.w;
                }
            } else {
#pragma unroll
                for (int w = 0; w < K; ++w) v[w] = row[w];
            }
            raw_sigma = v[K - 1];
            float col[3];
#pragma unroll
            for (int ch = 0; ch < 3; ++ch) {
                float tmp = 0.0f;
#pragma unroll
                for (int i = 0; i < BD; ++i) tmp += bs[i] * v[ch * BD + i];
                sg[ch] = sigmoid_ref(tmp);
                col[ch] = sg[ch] * d_rgb_pad - opt.rgb_padding;
            }
            if (!BWD) {
                row[0] = col[0]; row[1] = col[1]; row[2] = col[2];
                if (tr.weight_accum != nullptr) accumulate_weight(tr, q.slot[lane], q.w[lane]);
            } else {
                float total_color = 0.f;
#pragma unroll
                for (int ch = 0; ch < 3; ++ch) total_color += col[ch] * q.rayv[opar][own][BD + ch];
                row[0] = total_color;
            }
        }
        __syncwarp();
        // every owner folds in its items, in march order
        {
            unsigned m = mine_lo;
            while (m != 0u) {
                const int k = __ffs(m) - 1;
                m &= m - 1u;
                const float wk = q.w[k];
                const int ob = q.owner[k];
                const bool is_cur = ((ob >> 5) & 1) == par;
                float* res = q.rows + k * Shape::STRIDE;
                if (!BWD) {
                    if (is_cur) {
                        a0 += wk * res[0]; a1 += wk * res[1]; a2 += wk * res[2];
                        if (LOG) { res[0] = a0; res[1] = a1; res[2] = a2; }
                        --cnt_cur;
                    } else {
                        float o0 = q.oldv[lane][0], o1 = q.oldv[lane][1], o2 = q.oldv[lane][2];
                        o0 += wk * res[0]; o1 += wk * res[1]; o2 += wk * res[2];
                        q.oldv[lane][0] = o0; q.oldv[lane][1] = o1; q.oldv[lane][2] = o2;
                        if (LOG) { res[0] = o0; res[1] = o1; res[2] = o2; }
                        --cnt_old;
                    }
                } else {
                    const float tc = res[0];
                    if (ob & 0x80) {
                        accum += wk * tc;
                        --cnt_cur;
                    } else if (is_cur) {
                        accum -= wk * tc;
                        res[1] = q.dd[k] * (tc * q.T[k] - accum);
                        --cnt_cur;
                    } else {
                        accum_old -= wk * tc;
                        res[1] = q.dd[k] * (tc * q.T[k] - accum_old);
                        --cnt_old;
                    }
                }
            }
            if (old_valid && cnt_old == 0) {
                if (!BWD)
                    write_out(q.oldray[lane], q.oldv[lane][0], q.oldv[lane][1], q.oldv[lane][2],
                              q.oldv[lane][3], q.oldstop[lane] != 0);
                old_valid = false;
            }
        }
        if (LOG) {
            __syncwarp();
            // lane i writes item i, now with its ray's colour sums, into the log
            if (log_left == 0) {
                int c = 0;
                if (lane == 0) c = atomicAdd(log, kLogGrab);
                log_chunk = __shfl_sync(0xffffffffu, c, 0);
                log_left = kLogGrab;
            }
            if (log_chunk < log_capacity) {
                int32_t* ch = log + kLogChunks + log_chunk * kLogChunkWords;
                if (lane == 0) ch[0] = nb;
                if (lane < nb) {
                    const float* res = q.rows + lane * Shape::STRIDE;
                    const uint32_t sl = q.slot[lane];
                    st_stream(ch + 32 * 1 + lane, (int32_t)sl, pol_stream);
                    st_stream(ch + 32 * 2 + lane, q.rayid[lane], pol_stream);
                    st_stream(ch + 32 * 3 + lane, __float_as_int(q.w[lane]), pol_stream);
                    st_stream(ch + 32 * 4 + lane, __float_as_int(q.T[lane]), pol_stream);
                    st_stream(ch + 32 * 5 + lane, __float_as_int(q.dd[lane]), pol_stream);
                    st_stream(ch + 32 * 6 + lane, __float_as_int(sg[0]), pol_stream);
                    st_stream(ch + 32 * 7 + lane, __float_as_int(sg[1]), pol_stream);
                    st_stream(ch + 32 * 8 + lane, __float_as_int(sg[2]), pol_stream);
                    st_stream(ch + 32 * 9 + lane, __float_as_int(res[0]), pol_stream);
                    st_stream(ch + 32 * 10 + lane, __float_as_int(res[1]), pol_stream);
                    st_stream(ch + 32 * 11 + lane, __float_as_int(res[2]), pol_stream);
                }
                if (lane < nb) {
                    const uint32_t bin = q.slot[lane] >> log_shift;
                    atomicAdd(&s_hist[bin < (uint32_t)kMaxBins ? bin : kMaxBins - 1], 1);
                }
            }
            ++log_chunk;
            --log_left;
        }
        if (BWD) {
            __syncwarp();
            // lane i forms the gradient of record i in its staging row
            if (lane < nb && !acc_item) {
                float* row = q.rows + lane * Shape::STRIDE;
                const float wk = q.w[lane];
                const float gs = row[1];
                float v[K];
#pragma unroll
                for (int ch = 0; ch < 3; ++ch) {
                    const float tmp2 =
                        wk * sg[ch] * (1.0 - sg[ch]) * q.rayv[opar][own][BD + ch] * d_rgb_pad;
#pragma unroll
                    for (int i = 0; i < BD; ++i) v[ch * BD + i] = q.rayv[opar][own][i] * tmp2;
                }
                v[K - 1] = gs * (opt.density_softplus ? sigmoid_ref(raw_sigma - 1) : 1);
                if (Shape::VEC) {
#pragma unroll
                    for (int w = 0; w < K / 4; ++w)
                        reinterpret_cast<float4*>(row)[w] =
                            make_float4(v[4 * w], v[4 * w + 1], v[4 * w + 2], v[4 * w + 3]);
                } else {
#pragma unroll
                    for (int w = 0; w < K; ++w) row[w] = v[w];
                }
            }
            __syncwarp();
            // groups of lanes flush the gradient rows
#pragma unroll
            for (int p = 0; p < 32 / Shape::IPP; ++p) {
                const int k = p * Shape::IPP + sub;
                if (k < nb && !(q.owner[k] & 0x80)) {
                    float* __restrict__ g = grad_data + (size_t)q.slot[k] * K;
                    const float* row = q.rows + k * Shape::STRIDE;
#pragma unroll
                    for (int w = 0; w < Shape::WPL; ++w) {
                        const int word = wj + w * Shape::GROUP;
                        if (word < Shape::WORDS) {
                            if (Shape::VEC) {
                                const float4 x = reinterpret_cast<const float4*>(row)[word];
                                red_add_v4_hint(g + 4 * word, x.x, x.y, x.z, x.w, pol_stream);
                            } else {
                                atomicAdd(g + word, row[word]);
                            }
                        }
                    }
                }
            }
        }
        __syncwarp();
        // drop the first 32 positions: entries 32.. move to the front
        const int rem = qn > 32 ? qn - 32 : 0;
        for (int b0 = 0; b0 < rem; b0 += 32) {
            const int i = b0 + lane;
            uint32_t s_ = 0; float w_ = 0.f, T_ = 0.f, d_ = 0.f; unsigned char o_ = 0; int r_ = 0;
            if (i < rem) {
                s_ = q.slot[32 + i]; w_ = q.w[32 + i]; o_ = q.owner[32 + i];
                if (BWD || LOG) { T_ = q.T[32 + i]; d_ = q.dd[32 + i]; }
                if (LOG) r_ = q.rayid[32 + i];
            }
            __syncwarp();
            if (i < rem) {
                q.slot[i] = s_; q.w[i] = w_; q.owner[i] = o_;
                if (BWD || LOG) { q.T[i] = T_; q.dd[i] = d_; }
                if (LOG) q.rayid[i] = r_;
            }
            __syncwarp();
        }
        qn = rem;
        mine_lo = (unsigned)(mine_hi & 0xffffffffull);
        mine_hi >>= 32;
    };

    // Requests the records of the first nb queued items into the staging rows: groups of
    // lanes copy a record each, 16 (or 4) bytes per lane, asynchronously.  (One bulk copy
    // per record through the copy engine was measured instead: 13 % slower, the engine's
    // rate of small requests then bounds the kernel.)
    auto request = [&](int nb) {
#pragma unroll
        for (int p = 0; p < 32 / Shape::IPP; ++p) {
            const int k = p * Shape::IPP + sub;
            if (k < nb) {
                const float* __restrict__ rec = tr.data + (size_t)q.slot[k] * K;
                float* row = q.rows + k * Shape::STRIDE;
#pragma unroll
                for (int w = 0; w < Shape::WPL; ++w) {
                    const int word = wj + w * Shape::GROUP;
                    if (word < Shape::WORDS) {
                        if (Shape::VEC) cp_async16(row + 4 * word, rec + 4 * word, pol_rec);
                        else cp_async4(row + word, rec + word, pol_rec);
                    }
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // Waits until the records requested last have arrived.
    auto wait_records = [&]() {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
    };

    for (;;) {
        bool force = false;
        // ---- lanes that are not marching: finish, refill, termination ---------------------
        if (__ballot_sync(0xffffffffu, state != kMarching) != 0u) {
            if (state == kDraining && cnt_cur == 0) {
                if (BWD && phase == 0) {
                    // tail of the reference's PASS 1 (rt_kernel.cu:415-418), then march again
                    const float* g = &q.rayv[par][lane][BD];
                    const float total_grad = g[0] + g[1] + g[2];
                    accum += light * bg * total_grad;
                    phase = 1;
                    t = r.tmin; light = 1.f; it = 0;
                    state = kMarching;
                    place_cursor();
                    request_entry();
                } else {
                    if (!BWD) write_out(ray, a0, a1, a2, light, stopped);
                    state = kNeedRay;
                }
            }
            // Refills are taken a few lanes at a time: the set-up of a ray is some hundred
            // instructions, which a single active lane would make the whole warp pay for.
            const unsigned need = __ballot_sync(0xffffffffu, state == kNeedRay);
            const bool refill_now = __popc(need) >= refill_batch ||
                                    __ballot_sync(0xffffffffu, state == kMarching) == 0u;
            if (state == kNeedRay && refill_now) {
                const unsigned ticket = atomicAdd(&s_next, 1u);
                const int64_t gran = (int64_t)blockIdx.x + (int64_t)gridDim.x * (ticket >> 5);
                ray = gran * 32 + (ticket & 31);
                if (ray >= Q) {
                    if (gran * 32 >= Q) state = kExhausted;
                } else {
                    src.load(ray, tr, opt, r);
                    ray_setup(r, tr.scaling);
                    if (!r.hit || !(r.tmin < r.tmax)) {
                        if (!BWD) { out[3 * ray + 0] = bg; out[3 * ray + 1] = bg; out[3 * ray + 2] = bg; }
                    } else {
                        state = kMarching;
                        t = r.tmin; light = 1.f; it = 0; stopped = false;
                        float basis[BD];
                        colour_basis<BD, Source::kLobes>(tr, opt, r.vdir, basis);
#pragma unroll
                        for (int i = 0; i < BD; ++i)
                            q.rayv[par][lane][i] =
                                (i < opt.min_comp || i > opt.max_comp) ? 0.f : basis[i];
                        if (!BWD) {
                            a0 = a1 = a2 = 0.f;
                        } else {
                            const float g0 = __ldg(grad_out + 3 * ray), g1 = __ldg(grad_out + 3 * ray + 1),
                                        g2 = __ldg(grad_out + 3 * ray + 2);
                            float* g = &q.rayv[par][lane][BD];
                            g[0] = g0; g[1] = g1; g[2] = g2;
                            if (single) {
                                accum = __ldg(fwd_out + 3 * ray) * g0;
                                accum += __ldg(fwd_out + 3 * ray + 1) * g1;
                                accum += __ldg(fwd_out + 3 * ray + 2) * g2;
                                phase = 1;
                            } else {
                                accum = 0.f;
                                phase = 0;
                            }
                        }
                        place_cursor();
                        request_entry();
                    }
                }
            }
            __syncwarp();
            if (__ballot_sync(0xffffffffu, state == kMarching) == 0u) {
                // nobody marches: flush what is queued, then stop when every lane is done
                if (qn == 0) {
                    if (__all_sync(0xffffffffu, state == kExhausted)) break;
                    continue;
                }
                force = true;
            } else if (__any_sync(0xffffffffu, state == kDraining)) {
                force = true;
            }
        }

        // ---- G step: every lane consumes the entry it requested one iteration ago -----------
        // An inner node moves the cursor one level down; a leaf is sampled and the cursor
        // moves to the next sample.  Either way the next entry is requested at the end,
        // so its latency overlaps the queue work below and the loop overhead.
        bool item = false;
        uint32_t slot = 0;
        float weight = 0.f, dd = 0.f;
        if (state == kMarching) {
            int32_t e = e_pre;
            bool go = true, is_leaf = false, have_slot = false;
            int depth = 0;
            if (kind == kFromBrick) {
                const int gk = (int)((uint32_t)e_aux >> 28);
                const uint32_t payload = (uint32_t)e_aux & 0x0fffffffu;
                if (e > 0) {                    // deeper than the brick: go on from that node
                    node = (int)payload + e;
                    lvl = base + kBrickLevels;
                    kind = kFromChild;
                    if (node >= M || lvl >= kCoordBits) {
                        report(SVOXB_ERR_TREE);
                        state = kDraining;
                        go = false;
                    }
                } else {
                    is_leaf = true;
                    have_slot = true;
                    depth = base + 1 + gk;
                    if (gk == 2) {
                        const int b = kCoordBits - depth;
                        slot = payload * 8u + (uint32_t)((((ix >> b) & 1) << 2) |
                                                         (((iy >> b) & 1) << 1) | ((iz >> b) & 1));
                    } else {
                        slot = payload;
                    }
                }
            } else if (kind == kFromTable) {
                if (e >= kBrickFlag) {          // the cell has a brick: look the sample up there
                    cur_cell = tab_idx;
                    cur_brick = e - kBrickFlag;
                    kind = kFromBrick;
                } else if (e > 0) {             // node at the table level, no brick
                    node = e;
                    lvl = base;
                    kind = kFromChild;
                } else if (e == kTabDescend) {  // resolve from the root
                    kind = kFromChild;
                } else {                        // empty leaf of depth -e: nothing else to read
                    is_leaf = true;
                    depth = -e;
                    e = 0;
                }
            } else if (e > 0) {
                node += e;                      // inner node: one level down
                ++lvl;
                if (node >= M || lvl >= kCoordBits) {
                    report(SVOXB_ERR_TREE);
                    state = kDraining;
                    go = false;
                }
            } else {
                is_leaf = true;
                depth = lvl + 1;
            }
            if (is_leaf) {
                bool done = false;
                const int b = kCoordBits - depth;
                const float cube = __int_as_float((127 + depth) << 23);      // 2^depth
                const float inv_cube = __int_as_float((127 - depth) << 23);  // 2^-depth
                const float fx = __fmaf_rn(px, cube, -(float)(ix >> b));  // exact
                const float fy = __fmaf_rn(py, cube, -(float)(iy >> b));
                const float fz = __fmaf_rn(pz, cube, -(float)(iz >> b));
                float smin, smax;
                dda_unit<FC_DDA_LEAF>(fx, fy, fz, r.ix, r.iy, r.iz, smin, smax);
                // dividing by 2^depth == multiplying by 2^-depth, exactly
                const float delta_t =
                    __fadd_rn(__fmul_rn(__fsub_rn(smax, smin), inv_cube), opt.step_size);
                if (e < 0) {
                    if (!have_slot)
                        slot = (uint32_t)node * 8u + (uint32_t)((((ix >> b) & 1) << 2) |
                                                                (((iy >> b) & 1) << 1) |
                                                                ((iz >> b) & 1));
                    float sigma = (e == kOccupied) ? __ldg(tr.data + (size_t)slot * K + (K - 1))
                                                   : __uint_as_float((uint32_t)e & 0x7fffffffu);
                    dd = delta_t * r.delta_scale;
                    if (opt.density_softplus) {
                        // the log's step length carries d softplus / d raw density, the one
                        // factor the replayed density gradient needs from the raw value
                        // (svox/csrc/rt_kernel.cu:469-470)
                        if (LOG) dd *= sigmoid_ref(sigma - 1);
                        sigma = softplus_m1(sigma);
                    }
                    const float att = BWD ? expf(-delta_t * sigma * r.delta_scale)
                                          : expf(-delta_t * r.delta_scale * sigma);
                    weight = light * (1.f - att);
                    light *= att;
                    item = true;
                    if (!BWD && light <= opt.stop_thresh) {
                        stopped = true;
                        done = true;
                    }
                }
                t = __fadd_rn(t, delta_t);
                if (!(t < r.tmax)) done = true;
                if (++it > kMaxSteps) {
                    report(SVOXB_ERR_MARCH);
                    done = true;
                }
                if (!done) {
                    place_cursor();
                } else {
                    go = false;
                    const int pending = cnt_cur + (item ? 1 : 0);
                    if (BWD && phase == 0) {
                        state = kDraining;     // accum must be complete before the second march
                    } else if (pending == 0) {
                        if (!BWD) write_out(ray, a0, a1, a2, light, stopped);
                        state = kNeedRay;
                    } else if (!old_valid) {
                        // hand the ray over to the "old" context and refill at once
                        if (!BWD) {
                            q.oldv[lane][0] = a0; q.oldv[lane][1] = a1; q.oldv[lane][2] = a2;
                            q.oldv[lane][3] = light;
                            q.oldray[lane] = ray;
                            q.oldstop[lane] = stopped ? 1 : 0;
                        } else {
                            accum_old = accum;
                        }
                        cnt_old = pending;
                        cnt_cur = item ? -1 : 0;  // the push below counts the last item ...
                        if (!item) par ^= 1;      // ... and then switches the parity tag
                        old_valid = true;
                        state = kNeedRay;
                    } else {
                        state = kDraining;     // both contexts busy: wait for the queue
                    }
                }
            }
            if (go) request_entry();
        }

        // ---- push items --------------------------------------------------------------
        const unsigned pushed = __ballot_sync(0xffffffffu, item);
        if (item) {
            const int pos = qn + __popc(pushed & ((1u << lane) - 1u));
            q.slot[pos] = slot;
            q.w[pos] = weight;
            if (BWD || LOG) { q.T[pos] = light; q.dd[pos] = dd; }
            if (LOG) q.rayid[pos] = (int)ray;
            q.owner[pos] = (unsigned char)(lane | (par << 5) | ((BWD && phase == 0) ? 0x80 : 0));
            if (pos < 32) mine_lo |= 1u << pos;
            else mine_hi |= 1ull << (pos - 32);
            ++cnt_cur;
            // a ray that ended with this item has just been handed over: its items carry
            // the parity they were pushed with, the next ray uses the other one
            if (cnt_cur == 0) par ^= 1;
        }
        qn += __popc(pushed);
        const int collected = qn - (inflight ? 32 : 0);
        if (collected < 32 && !(force && qn > 0)) continue;
        __syncwarp();

        // ---- S step -------------------------------------------------------------------
        if (inflight) {
            wait_records();
            evaluate(32);
            inflight = false;
        }
        if (force) {
            // a lane waits for its items (or nobody marches any more): flush everything now
            while (qn > 0) {
                const int nb = qn < 32 ? qn : 32;
                request(nb);
                wait_records();
                evaluate(nb);
            }
        } else if (qn >= 32) {
            request(32);
            inflight = true;
        }
    }
    if (LOG) {
        // chunks taken but not used hold no items
        if (lane < log_left && log_chunk + lane < log_capacity)
            log[kLogChunks + (log_chunk + lane) * kLogChunkWords] = 0;
        __syncthreads();
        for (int i = threadIdx.x; i < kMaxBins; i += BLOCK)
            if (s_hist[i] != 0) atomicAdd(log + kLogHeads + i, s_hist[i]);
    }
}

}  // namespace svoxb
