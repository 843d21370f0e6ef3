// Backward pass by replay of the forward's item log (see render_queue.cuh for
// the log layout).
//
// The logged forward has already found every contributing sample, evaluated
// its colour sigmoids and recorded the ray's colour sums up to the sample, so
// the backward neither marches nor reads a leaf record, and every item can be
// handled on its own: with g = grad_out[ray],
//   total_color = <g, colour of the sample>
//   accum       = <g, out[ray]> - <g, colour sums up to and including the sample>
//   d/d sigma   = delta * (total_color * T - accum)          (rt_kernel.cu:462-471)
//   d/d coef    = basis[i] * weight * sg (1 - sg) * g[ch] * (1 + 2 pad)   (:386-392)
// What is left is adding one K-float record per item into `grad_data`.  Done in
// ray order that is the whole cost: every leaf is touched ~8 times per launch
// by rays far apart in time, each touch misses L2 and becomes a 32-byte
// read-modify-write in HBM (20 GB for the benchmark scene).  So the replay
// sorts first:
//
//   prefix   turns the forward's histogram of items per BIN (a bin = a range of
//            leaf slots whose gradient spans a few MB) into bin offsets;
//   bin      streams the log; lane i turns item i into a 32-byte packet (slot,
//            the three colour factors, the density gradient, the ray's view
//            direction) and appends it to its bin.  A block reserves room for the packets of 8 chunks at a
//            time, so the bin cursors see one atomic per bin and block step;
//   scatter  walks the packets bin after bin: all SMs work on the same few bins
//            at a time, so the gradient lines they reduce into stay in L2 and
//            reach HBM once.  Lane i expands packet i to its K-float record in a
//            shared-memory row; groups of lanes flush the rows with
//            red.global.add.v4.f32.
#pragma once

#include "render_queue.cuh"

namespace svoxb {

constexpr int kCursorStride = 32;
constexpr int kMaxParts = 16;        // the scatter can run in up to 16 parts (bin ranges)
constexpr int kScatterUnit = 2048;  // packets a block of the scatter kernel takes at a time

struct ReplayBins {
    int32_t* cursor;      // [kMaxBins * kCursorStride] append cursors (one per 128-byte line)
    int32_t* offset;      // [kMaxBins + 1] exclusive prefix of the histogram
    // packets: 32 bytes each {slot, f0, f1, f2 | gs, view direction}; a packet nobody wrote
    // is told by its position (see the scatter kernel)
    int64_t capacity;
    int4* packet;   // [capacity * 2]
    int64_t* work;  // [kMaxParts] scatter work counters, one per part of the bin range
    const float4* rays;  // [3 per ray] {g0,g1,g2,out0} {out1,out2,v0,v1} {v2,-,-,-}
};

// First bin of part p when n_bins bins are cut into n_parts ranges.
__host__ __device__ inline int replay_part_first_bin(int p, int n_parts, int n_bins) {
    return (int)(((int64_t)p * n_bins) / n_parts);
}

// One block: exclusive prefix of the forward's histogram.  A log that overflowed (the forward
// asked for more chunks than it holds) must not be replayed: all bins are then left empty, so
// the bin pass and the scatter find nothing to do.
__global__ void replay_prefix_kernel(const int32_t* __restrict__ log, ReplayBins b, int n_parts,
                                     int64_t capacity_chunks) {
    __shared__ int s[kMaxBins];
    int n_bins = log[3];
    if ((int64_t)log[0] > capacity_chunks) n_bins = 0;
    if (n_bins < 0) n_bins = 0;
    if (n_bins > kMaxBins) n_bins = kMaxBins;
    for (int i = threadIdx.x; i < kMaxBins; i += blockDim.x) {
        s[i] = i < n_bins ? log[kLogHeads + i] : 0;
        b.cursor[i * kCursorStride] = 0;
    }

    __syncthreads();
    if (threadIdx.x == 0) {
        int64_t run = 0;
        for (int i = 0; i < kMaxBins; ++i) {
            b.offset[i] = (int)(run < b.capacity ? run : b.capacity);
            run += s[i] > 0 ? s[i] : 0;
        }
        b.offset[kMaxBins] = (int)(run < b.capacity ? run : b.capacity);
        // part p of the scatter covers bins [first_bin(p), first_bin(p + 1)): its work
        // counter starts at the first packet of its first bin
        for (int p = 0; p < n_parts && p < kMaxParts; ++p)
            b.work[p] = b.offset[replay_part_first_bin(p, n_parts, n_bins)];
    }
}

// Per-ray inputs of the bin pass, packed so that one item needs three 16-byte
// loads instead of nine 4-byte ones.
template <class Source>
__global__ void replay_pack_rays_kernel(TreeArgs tr, Source src, svoxb_render_options opt,
                                        const float* __restrict__ grad_out,
                                        const float* __restrict__ fwd_out, int64_t n_rays,
                                        float4* __restrict__ rays) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rays) return;
    float v[3];
    src.load_vdir(i, tr, opt, v);
    float g[3] = {0.f, 0.f, 0.f};
    if (grad_out != nullptr) {
        g[0] = grad_out[3 * i]; g[1] = grad_out[3 * i + 1]; g[2] = grad_out[3 * i + 2];
    }
    rays[3 * i] = make_float4(g[0], g[1], g[2], fwd_out[3 * i]);
    rays[3 * i + 1] = make_float4(fwd_out[3 * i + 1], fwd_out[3 * i + 2], v[0], v[1]);
    rays[3 * i + 2] = make_float4(v[2], 0.f, 0.f, 0.f);
}

// HESS: instead of the gradient for an upstream grad_out, the packets carry what the
// diagonal of the Gauss-Newton matrix of the squared error needs, i.e. the square of each
// output's derivative summed over the three outputs (svox/csrc/rt_kernel.cu:596-605, 683-698):
// the colour factor without grad_out, and sum_j (d out_j / d sigma)^2.
template <int BLOCK, int CPW, int MINB, bool HESS>   // CPW: chunks per warp and block step
__global__ void __launch_bounds__(BLOCK, MINB)
replay_bin_kernel(svoxb_render_options opt, const int32_t* __restrict__ log, int64_t n_chunks,
                  int64_t capacity_chunks, int64_t n_rays, ReplayBins b,
                  const float* __restrict__ data, int K) {
    constexpr int WARPS = BLOCK / 32;
    {
        // the chunks the forward really wrote (n_chunks is the host's upper bound); none of
        // them counts if the log overflowed
        const int64_t used = log[0];
        if (used > capacity_chunks) return;
        if (used < n_chunks) n_chunks = used;
    }
    __shared__ int s_cnt[kMaxBins];   // packets of this block step per bin, then their base
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float d_rgb_pad = 1 + 2 * opt.rgb_padding;
    const int shift = log[2];
    int n_bins = log[3];
    if (n_bins > kMaxBins) n_bins = kMaxBins;
    const int64_t n_steps = (n_chunks + WARPS * CPW - 1) / (WARPS * CPW);

    for (int64_t step = blockIdx.x; step < n_steps; step += gridDim.x) {
        for (int i = threadIdx.x; i < n_bins; i += BLOCK) s_cnt[i] = 0;
        __syncthreads();
        int bin[CPW], rank[CPW];
        int32_t slot[CPW], ray[CPW];
        float f[CPW][3], gs[CPW], vd[CPW][3];
#pragma unroll
        for (int j = 0; j < CPW; ++j) {
            bin[j] = -1;
            const int64_t c = (step * WARPS + warp) * CPW + j;
            int n = 0;
            const int32_t* __restrict__ ch = log + kLogChunks + c * kLogChunkWords;
            if (c < n_chunks) n = ch[0];
            if (lane < n && n <= 32) {
                slot[j] = ch[32 * 1 + lane];
                ray[j] = ch[32 * 2 + lane];
                const uint32_t bb = (uint32_t)slot[j] >> shift;
                if (bb < (uint32_t)n_bins && ray[j] >= 0 && ray[j] < n_rays) bin[j] = (int)bb;
            }
        }
#pragma unroll
        for (int j = 0; j < CPW; ++j) {
            if (bin[j] >= 0) {
                const int64_t c = (step * WARPS + warp) * CPW + j;
                const int32_t* __restrict__ ch = log + kLogChunks + c * kLogChunkWords;
                const float wk = __int_as_float(ch[32 * 3 + lane]);
                const float T = __int_as_float(ch[32 * 4 + lane]);
                const float dd = __int_as_float(ch[32 * 5 + lane]);
                const float4 ra = __ldg(b.rays + 3 * (int64_t)ray[j]),
                             rb = __ldg(b.rays + 3 * (int64_t)ray[j] + 1),
                             rc = __ldg(b.rays + 3 * (int64_t)ray[j] + 2);
                const float gg[3] = {ra.x, ra.y, ra.z}, oo[3] = {ra.w, rb.x, rb.y};
                vd[j][0] = rb.z; vd[j][1] = rb.w; vd[j][2] = rc.x;
                float total_color = 0.f, accum = 0.f;
                // Gauss-Newton diagonal with a softplus density: the reference adds, per
                // channel, (d out / d raw)^2 + (d out / d density) * softplus'' with its own
                // formula for the second term (svox/csrc/rt_kernel.cu:683-693); the logged
                // step length already holds the factor softplus' = s
                float one_minus_s = 0.f;
                if (HESS && opt.density_softplus)
                    one_minus_s = 1.f - sigmoid_ref(__ldg(data + (int64_t)(uint32_t)slot[j] * K +
                                                         (K - 1)) - 1);
#pragma unroll
                for (int chn = 0; chn < 3; ++chn) {
                    const float sg = __int_as_float(ch[32 * (6 + chn) + lane]);
                    const float part = __int_as_float(ch[32 * (9 + chn) + lane]);
                    const float g = gg[chn];
                    if (!HESS) {
                        total_color += (sg * d_rgb_pad - opt.rgb_padding) * g;
                        accum += (oo[chn] - part) * g;
                        // colour-coefficient factor (rt_kernel.cu:390)
                        f[j][chn] = wk * sg * (1.0 - sg) * g * d_rgb_pad;
                    } else {
                        f[j][chn] = wk * sg * (1.0 - sg) * d_rgb_pad;
                        const float ds = dd * ((sg * d_rgb_pad - opt.rgb_padding) * T -
                                               (oo[chn] - part));
                        total_color += ds * ds + ds * one_minus_s;
                    }
                }
                gs[j] = HESS ? total_color : dd * (total_color * T - accum);
                rank[j] = atomicAdd(&s_cnt[bin[j]], 1);
            }
        }
        __syncthreads();
        // one reservation per bin for the whole block step
        for (int i = threadIdx.x; i < n_bins; i += BLOCK) {
            const int cnt = s_cnt[i];
            if (cnt > 0) s_cnt[i] = atomicAdd(&b.cursor[i * kCursorStride], cnt);
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < CPW; ++j) {
            if (bin[j] >= 0) {
                const int64_t pos = (int64_t)b.offset[bin[j]] + s_cnt[bin[j]] + rank[j];
                if (pos < b.offset[bin[j] + 1]) {
                    b.packet[2 * pos] = make_int4(slot[j], __float_as_int(f[j][0]),
                                                  __float_as_int(f[j][1]), __float_as_int(f[j][2]));
                    b.packet[2 * pos + 1] =
                        make_int4(__float_as_int(gs[j]), __float_as_int(vd[j][0]),
                                  __float_as_int(vd[j][1]), __float_as_int(vd[j][2]));
                }
            }
        }
        __syncthreads();
    }
}

__device__ __forceinline__ int4 ld_stream16(const int4* a, uint64_t pol) {
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.s32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(a), "l"(pol));
    return v;
}

template <int K>
struct alignas(16) ScatterSmem {
    using Shape = RecordShape<K>;
    uint32_t slot[32];
    alignas(16) float rows[32 * Shape::STRIDE + 4];
};

template <int BD, int BLOCK, bool HESS, bool LOBES>
__global__ void __launch_bounds__(BLOCK)
replay_scatter_kernel(int64_t n_slots, svoxb_render_options opt, TreeArgs lobes,
                      float* __restrict__ grad_data, const int32_t* __restrict__ log,
                      ReplayBins b, int flags, int part, int n_parts) {
    constexpr int K = 3 * BD + 1;
    using Shape = RecordShape<K>;
    using SM = ScatterSmem<K>;
    extern __shared__ __align__(16) unsigned char s_raw[];
    const int lane = threadIdx.x & 31;
    SM& sm = *reinterpret_cast<SM*>(s_raw + (size_t)(threadIdx.x >> 5) * sizeof(SM));
    const int sub = lane / Shape::GROUP, wj = lane % Shape::GROUP;
    // packets of this part: those of its bin range
    int n_bins = log[3];
    if (n_bins > kMaxBins) n_bins = kMaxBins;
    const int64_t total = b.offset[replay_part_first_bin(part + 1, n_parts, n_bins)];
    const int shift = log[2];
    const uint64_t pol_keep = l2_policy_keep(), pol_stream = l2_policy_stream();
    // Blocks take units of kScatterUnit packets in bin order from one counter, so the
    // whole grid works within a window much smaller than a bin.
    __shared__ int64_t s_unit;
    const int warp = threadIdx.x >> 5;
    constexpr int PER_WARP = kScatterUnit / (BLOCK / 32);

    for (;;) {
    __syncthreads();
    if (threadIdx.x == 0)
        s_unit = (int64_t)atomicAdd(reinterpret_cast<unsigned long long*>(b.work + part),
                                    (unsigned long long)kScatterUnit);
    __syncthreads();
    const int64_t unit = s_unit;
    if (unit >= total) break;
    for (int64_t first = unit + warp * PER_WARP; first < unit + (warp + 1) * PER_WARP && first < total;
         first += 32) {
        const int n = (int)((total - first) < 32 ? (total - first) : 32);
        uint32_t slot = 0xffffffffu;
        int4 pa = make_int4(-1, 0, 0, 0), pb = make_int4(0, 0, 0, 0);
        if (lane < n) {
            if (flags & 1) {
                pa = ld_stream16(b.packet + 2 * (first + lane), pol_stream);
                pb = ld_stream16(b.packet + 2 * (first + lane) + 1, pol_stream);
            } else {
                pa = __ldg(b.packet + 2 * (first + lane));
                pb = __ldg(b.packet + 2 * (first + lane) + 1);
            }
            slot = (uint32_t)pa.x;
        }
        // a position the bin pass left unwritten holds stale bytes: a packet counts only
        // if it lies in the written part of the bin its slot names
        {
            const uint32_t bin = slot >> shift;
            bool ok = (int64_t)slot < n_slots && bin < (uint32_t)kMaxBins;
            if (ok) {
                const int64_t rel = first + lane - b.offset[bin];
                ok = rel >= 0 && rel < b.cursor[bin * kCursorStride];
            }
            if (!ok) slot = 0xffffffffu;
        }
        sm.slot[lane] = slot;
        if (slot != 0xffffffffu) {
            const float f[3] = {__int_as_float(pa.y), __int_as_float(pa.z), __int_as_float(pa.w)};
            const float vdir[3] = {__int_as_float(pb.y), __int_as_float(pb.z), __int_as_float(pb.w)};
            float basis[BD];
            colour_basis<BD, LOBES>(lobes, opt, vdir, basis);
#pragma unroll
            for (int k = 0; k < BD; ++k)
                if (k < opt.min_comp || k > opt.max_comp) basis[k] = 0.f;
            float v[K];
#pragma unroll
            for (int chn = 0; chn < 3; ++chn)
#pragma unroll
                for (int k = 0; k < BD; ++k) {
                    const float gw = basis[k] * f[chn];
                    v[chn * BD + k] = HESS ? gw * gw : gw;
                }
            v[K - 1] = __int_as_float(pb.x);
            float* row = sm.rows + lane * Shape::STRIDE;
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
#pragma unroll
        for (int p = 0; p < 32 / Shape::IPP; ++p) {
            const int k = p * Shape::IPP + sub;
            if (k < n) {
                const uint32_t sl = sm.slot[k];
                if ((int64_t)sl < n_slots) {
                    float* __restrict__ gp = grad_data + (size_t)sl * K;
                    const float* row = sm.rows + k * Shape::STRIDE;
#pragma unroll
                    for (int w = 0; w < Shape::WPL; ++w) {
                        const int word = wj + w * Shape::GROUP;
                        if (word < Shape::WORDS) {
                            if (Shape::VEC) {
                                const float4 x = reinterpret_cast<const float4*>(row)[word];
                                if (flags & 2)
                                    red_add_v4_hint(gp + 4 * word, x.x, x.y, x.z, x.w, pol_keep);
                                else
                                    red_add_v4(gp + 4 * word, x.x, x.y, x.z, x.w);
                            } else {
                                atomicAdd(gp + word, row[word]);
                            }
                        }
                    }
                }
            }
        }
        __syncwarp();
    }
    }
}

}  // namespace svoxb
