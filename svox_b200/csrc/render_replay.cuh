// Backward pass by replay of the forward's item log (see render_queue.cuh for
// the log layout).
//
// The logged forward has already found every contributing sample and
// evaluated its colour sigmoids.  The backward therefore neither marches nor
// reads a leaf record: it streams the log (coalesced 128-byte rows), redoes
// the reference's per-ray bookkeeping in log order
// (svox/csrc/rt_kernel.cu:386-411, 462-471 with `accum` started from
// <grad_out, fwd_out>), and scatters one gradient record per item with
// red.global.add.v4.f32.  What remains is the HBM traffic of the gradient
// itself.
//
// One warp replays one chunk list (= the items one forward warp produced, in
// order).  Lane i handles item i of a chunk; the lane recorded as the item's
// owner keeps the running `accum` of that item's ray (two rays per owner can
// interleave, told apart by the parity bit).
#pragma once

#include "render_queue.cuh"

namespace svoxb {

template <int K>
struct alignas(16) ReplaySmem {
    using Shape = CoopShape<K>;
    float w[32], T[32], dd[32], tc[32], gs[32];
    int ray[32];
    unsigned mask[64];  // items per owner lane and parity
    alignas(16) float rows[32 * Shape::STRIDE + 4];
};

template <int BD, int BLOCK, class Source>
__global__ void __launch_bounds__(BLOCK)
render_replay_kernel(TreeArgs tr, Source src, svoxb_render_options opt, int32_t* __restrict__ log,
                     const float* __restrict__ grad_out, const float* __restrict__ fwd_out,
                     float* __restrict__ grad_data, int64_t log_capacity) {
    constexpr int K = 3 * BD + 1;
    using Shape = CoopShape<K>;
    using SM = ReplaySmem<K>;
    extern __shared__ __align__(16) unsigned char s_raw[];
    const int lane = threadIdx.x & 31;
    SM& sm = *reinterpret_cast<SM*>(s_raw + (size_t)(threadIdx.x >> 5) * sizeof(SM));
    const float d_rgb_pad = 1 + 2 * opt.rgb_padding;
    const int sub = lane / Shape::GROUP, wj = lane % Shape::GROUP;
    const uint64_t pol_stream = l2_policy_stream();
    const int n_lists = log[2];

    for (;;) {
        int list = 0;
        if (lane == 0) list = atomicAdd(log + 1, 1);
        list = __shfl_sync(0xffffffffu, list, 0);
        if (list >= n_lists) break;
        int64_t c = log[kLogHeads + list];
        // per owner lane: the ray of each parity and its running accum
        int cur_ray[2] = {-1, -1};
        float accum[2] = {0.f, 0.f};
        int guard = 0;
        while (c >= 0 && c < log_capacity && ++guard < (1 << 28)) {
            const int32_t* __restrict__ ch = log + kLogChunks + c * kLogChunkWords;
            const int n = ch[0];
            const int64_t nxt = ch[1];
            if (n <= 0 || n > 32) break;
            sm.mask[lane] = 0u;
            sm.mask[32 + lane] = 0u;
            __syncwarp();
            // lane i: item i
            float wk = 0.f, sg[3] = {0.f, 0.f, 0.f}, g[3] = {0.f, 0.f, 0.f};
            float basis[BD];
#pragma unroll
            for (int i = 0; i < BD; ++i) basis[i] = 0.f;
            if (lane < n) {
                wk = __int_as_float(ch[32 * 2 + lane]);
                const float T = __int_as_float(ch[32 * 3 + lane]);
                const float dd = __int_as_float(ch[32 * 4 + lane]);
                sg[0] = __int_as_float(ch[32 * 5 + lane]);
                sg[1] = __int_as_float(ch[32 * 6 + lane]);
                sg[2] = __int_as_float(ch[32 * 7 + lane]);
                const int ray = ch[32 * 8 + lane];
                const int meta = ch[32 * 9 + lane];
                g[0] = __ldg(grad_out + 3 * (int64_t)ray);
                g[1] = __ldg(grad_out + 3 * (int64_t)ray + 1);
                g[2] = __ldg(grad_out + 3 * (int64_t)ray + 2);
                Ray r;
                src.load(ray, tr, opt, r);  // only the view direction is used
                sh_basis<BD>(r.vdir, basis);
#pragma unroll
                for (int i = 0; i < BD; ++i)
                    if (i < opt.min_comp || i > opt.max_comp) basis[i] = 0.f;
                float total_color = 0.f;
#pragma unroll
                for (int chn = 0; chn < 3; ++chn)
                    total_color += (sg[chn] * d_rgb_pad - opt.rgb_padding) * g[chn];
                sm.w[lane] = wk; sm.T[lane] = T; sm.dd[lane] = dd; sm.tc[lane] = total_color;
                sm.ray[lane] = ray;
                atomicOr(&sm.mask[(meta & 31) + 32 * ((meta >> 5) & 1)], 1u << lane);
            }
            __syncwarp();
            // owner lanes: sequential accum per ray, in log order
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                unsigned m = sm.mask[lane + 32 * p];
                while (m != 0u) {
                    const int k = __ffs(m) - 1;
                    m &= m - 1u;
                    const int ray = sm.ray[k];
                    if (ray != cur_ray[p]) {
                        cur_ray[p] = ray;
                        float a = __ldg(fwd_out + 3 * (int64_t)ray) * __ldg(grad_out + 3 * (int64_t)ray);
                        a += __ldg(fwd_out + 3 * (int64_t)ray + 1) * __ldg(grad_out + 3 * (int64_t)ray + 1);
                        a += __ldg(fwd_out + 3 * (int64_t)ray + 2) * __ldg(grad_out + 3 * (int64_t)ray + 2);
                        accum[p] = a;
                    }
                    const float tc = sm.tc[k];
                    accum[p] -= sm.w[k] * tc;
                    sm.gs[k] = sm.dd[k] * (tc * sm.T[k] - accum[p]);
                }
            }
            __syncwarp();
            // lane i forms the gradient of record i
            if (lane < n) {
                float* row = sm.rows + lane * Shape::STRIDE;
                float v[K];
#pragma unroll
                for (int chn = 0; chn < 3; ++chn) {
                    const float tmp2 = wk * sg[chn] * (1.0 - sg[chn]) * g[chn] * d_rgb_pad;
#pragma unroll
                    for (int i = 0; i < BD; ++i) v[chn * BD + i] = basis[i] * tmp2;
                }
                v[K - 1] = sm.gs[lane];
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
            // groups of lanes flush the rows
#pragma unroll
            for (int p = 0; p < 32 / Shape::IPP; ++p) {
                const int k = p * Shape::IPP + sub;
                if (k < n) {
                    const uint32_t sl = (uint32_t)ch[32 * 1 + k];
                    if ((int64_t)sl < tr.M * 8) {
                        float* __restrict__ gp = grad_data + (size_t)sl * K;
                        const float* row = sm.rows + k * Shape::STRIDE;
#pragma unroll
                        for (int w = 0; w < Shape::WPL; ++w) {
                            const int word = wj + w * Shape::GROUP;
                            if (word < Shape::WORDS) {
                                if (Shape::VEC) {
                                    const float4 x = reinterpret_cast<const float4*>(row)[word];
                                    red_add_v4_hint(gp + 4 * word, x.x, x.y, x.z, x.w, pol_stream);
                                } else {
                                    atomicAdd(gp + word, row[word]);
                                }
                            }
                        }
                    }
                }
            }
            __syncwarp();
            c = nxt;
        }
    }
}

}  // namespace svoxb
