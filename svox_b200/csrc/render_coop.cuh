// Warp-cooperative volume rendering kernels for SH colour with three channels
// (record K = 3 * basis_dim + 1): forward, and backward in one or two marches.
//
// Organisation of one warp (32 lanes = 32 rays in flight):
//
//   refill   a lane whose ray has ended writes its result and takes the next
//            ray of the block (ticket from a shared counter), so all lanes stay
//            busy whatever the spread of ray lengths;
//   G step   every lane advances its own ray by one leaf: sample position,
//            descent, step length.  The descent reads an ANNOTATED copy of the
//            child array in which a leaf entry also says whether the leaf's
//            density passes the test (built per call by annotate_kernel), so
//            empty leaves cost no HBM access at all;
//   S step   the lanes that hit a contributing leaf ("items") are compacted;
//            groups of lanes fetch the items' records with coalesced 128-bit
//            (or 32-bit) loads into a shared-memory staging row per item; each
//            owner lane then reads its row (conflict-free) and does the colour
//            and compositing arithmetic exactly as the reference orders it;
//   scatter  (backward) the owner writes the record's gradient to its staging
//            row and the groups flush the rows with vector reductions
//            (red.global.add.v4.f32), one coalesced 16-byte lane each.
//
// The loop is warp-uniform (driven by votes), which keeps the warp converged.
// Sample positions, step lengths and the per-ray order of accumulation are
// those of the reference (svox/csrc/rt_kernel.cu:222-477); see arith.cuh.
#pragma once

#include "render.cuh"

namespace svoxb {

// Marks in the annotated child array: > 0 link to a child node, 0 leaf that
// fails the density test, kOccupied leaf that passes it.
constexpr int32_t kOccupied = INT32_MIN;

// One thread per slot.  thresh is sigma_thresh (forward) or 0 (backward); the
// test is the expression the reference evaluates per sample
// (svox/csrc/rt_kernel.cu:276-278, 375-377).
__global__ void annotate_kernel(const int32_t* __restrict__ child,
                                const float* __restrict__ data, int K, int64_t n_slots,
                                float thresh, int softplus, int32_t* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_slots) return;
    int32_t c = child[i];
    if (c == 0) {
        float sigma = __ldg(data + i * K + (K - 1));
        if (softplus) sigma = softplus_m1(sigma);
        if (sigma > thresh) c = kOccupied;
    }
    out[i] = c;
}

// Descent over the annotated array (N = 2).  Same arithmetic as descend2.
__device__ __forceinline__ bool descend2_annot(const int32_t* __restrict__ child, int64_t M,
                                               const TopTable& top, float px, float py,
                                               float pz, uint32_t& slot_out, bool& occupied,
                                               float& cube_out, float& fx, float& fy,
                                               float& fz) {
    float x = clamp01(px), y = clamp01(py), z = clamp01(pz);
    int64_t node = 0;
    float cube = 1.0f;
    if (top.level > 0) {
        const float s = (float)(1 << top.level);
        const float xs = x * s, ys = y * s, zs = z * s;
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
        const int u = (int)x, v = (int)y, w = (int)z;
        x -= (float)u; y -= (float)v; z -= (float)w;
        cube *= 2.0f;
        const int64_t slot = node * 8 + (u * 4 + v * 2 + w);
        const int32_t skip = __ldg(child + slot);
        if (skip <= 0) {
            slot_out = (uint32_t)slot; occupied = skip < 0; cube_out = cube;
            fx = x; fy = y; fz = z;
            return true;
        }
        node += skip;
        if (node >= M) break;
    }
    report(SVOXB_ERR_TREE);
    return false;
}

// Shapes of the cooperative record transfer for a K-float record.
template <int K>
struct CoopShape {
    static constexpr bool VEC = (K % 4 == 0);            // 16-byte words possible
    static constexpr int WORDS = VEC ? K / 4 : K;         // words per record
    static constexpr int GROUP = WORDS <= 1 ? 1 : WORDS <= 2 ? 2 : WORDS <= 4 ? 4
                                 : WORDS <= 8 ? 8 : WORDS <= 16 ? 16 : 32;  // lanes per item
    static constexpr int IPP = 32 / GROUP;                // items per pass
    static constexpr int WPL = (WORDS + GROUP - 1) / GROUP;  // words per lane per item
    // staging row stride in floats: 16-byte rows for vector access, odd
    // otherwise (both conflict-free for the owner's reads)
    static constexpr int STRIDE = VEC ? K : (K | 1);
    static constexpr int ROWS_RAW = 1792 / (STRIDE * 4);
    static constexpr int ROWS0 = ROWS_RAW >= 32 ? 32 : ROWS_RAW >= 16 ? 16 : ROWS_RAW >= 8 ? 8 : 4;
    static constexpr int ROWS = ROWS0 < IPP ? IPP : ROWS0;  // items per chunk
    static constexpr int STAGE_FLOATS = ROWS * STRIDE + 4;
    static constexpr int PASSES = ROWS / IPP;
};

constexpr int kModeForward = 0;
constexpr int kModeBackward = 1;

template <int BD, int BLOCK, int MODE, class Source>
__global__ void __launch_bounds__(BLOCK)
render_coop_kernel(TreeArgs tr, Source src, svoxb_render_options opt, TopTable topg,
                   bool top_in_smem, int top_bytes, int64_t Q,
                   float* __restrict__ out,             // forward result
                   const float* __restrict__ grad_out,  // backward inputs
                   const float* __restrict__ fwd_out, float* __restrict__ grad_data) {
    constexpr int K = 3 * BD + 1;
    using Shape = CoopShape<K>;
    constexpr int WARPS = BLOCK / 32;
    extern __shared__ __align__(16) unsigned char s_raw[];
    int32_t* s_top = reinterpret_cast<int32_t*>(s_raw);
    float* s_stage_all = reinterpret_cast<float*>(s_raw + top_bytes);
    unsigned char* s_list_all =
        reinterpret_cast<unsigned char*>(s_stage_all + WARPS * Shape::STAGE_FLOATS);
    __shared__ unsigned s_next;
    if (threadIdx.x == 0) s_next = 0;
    const TopTable top = stage_top(topg, s_top, top_in_smem);
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    float* stage = s_stage_all + warp * Shape::STAGE_FLOATS;
    unsigned char* list = s_list_all + warp * 32;
    const float d_rgb_pad = 1 + 2 * opt.rgb_padding;
    const bool single = (MODE == kModeBackward) && fwd_out != nullptr;
    const float bg = opt.background_brightness;

    // ---- per-lane ray state -------------------------------------------------
    Ray r;
    r.hit = false;
    int64_t ray = 0;
    bool have = false, exhausted = false;
    float t = 0.f, light = 1.f;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f;  // forward: colour sums; backward: upstream gradient
    float accum = 0.f;
    float basis[BD];
    int phase = 1;  // backward: 0 = form accum (reference PASS 1), 1 = scatter march
    int it = 0;
#pragma unroll
    for (int i = 0; i < BD; ++i) basis[i] = 0.f;

    for (;;) {
        // ---- refill ------------------------------------------------------------
        if (__any_sync(0xffffffffu, !have && !exhausted)) {
            if (!have && !exhausted) {
                const unsigned ticket = atomicAdd(&s_next, 1u);
                ray = ((int64_t)blockIdx.x + (int64_t)gridDim.x * (ticket >> 5)) * 32 +
                      (ticket & 31);
                if (ray >= Q) {
                    // tickets grow with ray index: nothing is left for this lane
                    exhausted = ((int64_t)blockIdx.x + (int64_t)gridDim.x * (ticket >> 5)) * 32 >= Q;
                } else {
                    src.load(ray, tr, opt, r);
                    ray_setup(r, tr.scaling);
                    if (!r.hit || !(r.tmin < r.tmax)) {
                        if (MODE == kModeForward) {
                            const float v = r.hit ? (0.f + 1.f * bg) : bg;
                            out[3 * ray + 0] = v; out[3 * ray + 1] = v; out[3 * ray + 2] = v;
                        }
                    } else {
                        have = true;
                        t = r.tmin; light = 1.f; it = 0;
                        sh_basis<BD>(r.vdir, basis);
#pragma unroll
                        for (int i = 0; i < BD; ++i)
                            if (i < opt.min_comp || i > opt.max_comp) basis[i] = 0.f;
                        if (MODE == kModeForward) {
                            a0 = a1 = a2 = 0.f;
                        } else {
                            a0 = __ldg(grad_out + 3 * ray);
                            a1 = __ldg(grad_out + 3 * ray + 1);
                            a2 = __ldg(grad_out + 3 * ray + 2);
                            if (single) {
                                accum = __ldg(fwd_out + 3 * ray) * a0;
                                accum += __ldg(fwd_out + 3 * ray + 1) * a1;
                                accum += __ldg(fwd_out + 3 * ray + 2) * a2;
                                phase = 1;
                            } else {
                                accum = 0.f;
                                phase = 0;
                            }
                        }
                    }
                }
            }
        }
        if (!__any_sync(0xffffffffu, have)) {
            if (__all_sync(0xffffffffu, exhausted)) break;
            continue;
        }

        // ---- G step: one leaf per lane --------------------------------------------
        bool item = false, done = false;
        uint32_t slot = 0;
        float delta_t = 0.f;
        if (have) {
            if (++it > kMaxSteps) {
                report(SVOXB_ERR_MARCH);
                done = true;
            } else {
                const float px = mad_site<FC_POS>(t, r.dx, r.ox);
                const float py = mad_site<FC_POS>(t, r.dy, r.oy);
                const float pz = mad_site<FC_POS>(t, r.dz, r.oz);
                float cube, fx, fy, fz;
                bool occ = false;
                if (!descend2_annot(tr.child, tr.M, top, px, py, pz, slot, occ, cube, fx, fy, fz)) {
                    done = true;
                } else {
                    float smin, smax;
                    dda_unit<FC_DDA_LEAF>(fx, fy, fz, r.ix, r.iy, r.iz, smin, smax);
                    delta_t = __fadd_rn(__fdiv_rn(__fsub_rn(smax, smin), cube), opt.step_size);
                    item = occ;
                    if (!occ) {
                        t = __fadd_rn(t, delta_t);
                        if (!(t < r.tmax)) done = true;
                    }
                }
            }
        }

        // ---- S step: cooperative record fetch, owner arithmetic, scatter -------------
        const unsigned items = __ballot_sync(0xffffffffu, item);
        if (items != 0u) {
            const int n = __popc(items);
            const int rank = __popc(items & ((1u << lane) - 1u));
            if (item) list[rank] = (unsigned char)lane;
            __syncwarp();
            const int sub = lane / Shape::GROUP;   // item within a pass
            const int j = lane % Shape::GROUP;     // word lane within the item
            for (int c0 = 0; c0 < n; c0 += Shape::ROWS) {
                const int c1 = (c0 + Shape::ROWS < n) ? c0 + Shape::ROWS : n;
                // fetch
#pragma unroll
                for (int p = 0; p < Shape::PASSES; ++p) {
                    const int k = c0 + p * Shape::IPP + sub;
                    const bool valid = k < c1;
                    const int srcl = valid ? list[k] : 0;
                    const uint32_t sl = __shfl_sync(0xffffffffu, slot, srcl);
                    if (valid) {
                        const float* __restrict__ rec = tr.data + (size_t)sl * K;
                        float* row = stage + (k - c0) * Shape::STRIDE;
#pragma unroll
                        for (int w = 0; w < Shape::WPL; ++w) {
                            const int word = j + w * Shape::GROUP;
                            if (word < Shape::WORDS) {
                                if (Shape::VEC)
                                    reinterpret_cast<float4*>(row)[word] =
                                        __ldg(reinterpret_cast<const float4*>(rec) + word);
                                else
                                    row[word] = __ldg(rec + word);
                            }
                        }
                    }
                }
                __syncwarp();
                // owner arithmetic
                bool scatter = false;
                if (item && rank >= c0 && rank < c1) {
                    float* row = stage + (rank - c0) * Shape::STRIDE;
                    float v[K];
                    if (Shape::VEC) {
#pragma unroll
                        for (int w = 0; w < K / 4; ++w) {
                            const float4 q = reinterpret_cast<const float4*>(row)[w];
                            v[4 * w] = q.x; v[4 * w + 1] = q.y; v[4 * w + 2] = q.z; v[4 * w + 3] = q.w;
                        }
                    } else {
#pragma unroll
                        for (int w = 0; w < K; ++w) v[w] = row[w];
                    }
                    float sigma = v[K - 1];
                    const float raw_sigma = sigma;
                    if (opt.density_softplus) sigma = softplus_m1(sigma);
                    if (MODE == kModeForward) {
                        const float att = expf(-delta_t * r.delta_scale * sigma);
                        const float weight = light * (1.f - att);
                        float c[3];
#pragma unroll
                        for (int ch = 0; ch < 3; ++ch) {
                            float tmp = 0.0f;
#pragma unroll
                            for (int i = 0; i < BD; ++i) tmp += basis[i] * v[ch * BD + i];
                            c[ch] = sigmoid_ref(tmp) * d_rgb_pad - opt.rgb_padding;
                        }
                        a0 += weight * c[0];
                        a1 += weight * c[1];
                        a2 += weight * c[2];
                        light *= att;
                        if (light <= opt.stop_thresh) {
                            const float scale = 1.0 / (1.0 - light);
                            out[3 * ray + 0] = a0 * scale;
                            out[3 * ray + 1] = a1 * scale;
                            out[3 * ray + 2] = a2 * scale;
                            have = false;   // stopped: no background term
                        }
                    } else {
                        const float att = expf(-delta_t * sigma * r.delta_scale);
                        const float weight = light * (1.f - att);
                        float total_color = 0.f;
                        const float gch[3] = {a0, a1, a2};
#pragma unroll
                        for (int ch = 0; ch < 3; ++ch) {
                            float tmp = 0.0f;
#pragma unroll
                            for (int i = 0; i < BD; ++i) tmp += basis[i] * v[ch * BD + i];
                            const float sg = sigmoid_ref(tmp);
                            const float tmp2 = weight * sg * (1.0 - sg) * gch[ch] * d_rgb_pad;
#pragma unroll
                            for (int i = 0; i < BD; ++i) v[ch * BD + i] = basis[i] * tmp2;
                            total_color += (sg * d_rgb_pad - opt.rgb_padding) * gch[ch];
                        }
                        light *= att;
                        if (phase == 0) {
                            accum += weight * total_color;
                        } else {
                            accum -= weight * total_color;
                            v[K - 1] = delta_t * r.delta_scale * (total_color * light - accum) *
                                       (opt.density_softplus ? sigmoid_ref(raw_sigma - 1) : 1);
                            scatter = true;
                            if (Shape::VEC) {
#pragma unroll
                                for (int w = 0; w < K / 4; ++w)
                                    reinterpret_cast<float4*>(row)[w] = make_float4(
                                        v[4 * w], v[4 * w + 1], v[4 * w + 2], v[4 * w + 3]);
                            } else {
#pragma unroll
                                for (int w = 0; w < K; ++w) row[w] = v[w];
                            }
                        }
                    }
                    if (have) {
                        t = __fadd_rn(t, delta_t);
                        if (!(t < r.tmax)) done = true;
                    }
                }
                if (MODE == kModeBackward) {
                    __syncwarp();  // owners' gradient rows are visible to the groups
                    const unsigned scat = __ballot_sync(0xffffffffu, scatter);
                    if (scat != 0u) {
#pragma unroll
                        for (int p = 0; p < Shape::PASSES; ++p) {
                            const int k = c0 + p * Shape::IPP + sub;
                            const bool valid = k < c1;
                            const int srcl = valid ? list[k] : 0;
                            const uint32_t sl = __shfl_sync(0xffffffffu, slot, srcl);
                            if (valid && ((scat >> srcl) & 1u)) {
                                float* __restrict__ g = grad_data + (size_t)sl * K;
                                const float* row = stage + (k - c0) * Shape::STRIDE;
#pragma unroll
                                for (int w = 0; w < Shape::WPL; ++w) {
                                    const int word = j + w * Shape::GROUP;
                                    if (word < Shape::WORDS) {
                                        if (Shape::VEC) {
                                            const float4 q = reinterpret_cast<const float4*>(row)[word];
                                            red_add_v4(g + 4 * word, q.x, q.y, q.z, q.w);
                                        } else {
                                            atomicAdd(g + word, row[word]);
                                        }
                                    }
                                }
                            }
                        }
                    }
                }
                __syncwarp();
            }
        }

        // ---- end of ray ----------------------------------------------------------
        if (have && done) {
            if (MODE == kModeForward) {
                out[3 * ray + 0] = a0 + light * bg;
                out[3 * ray + 1] = a1 + light * bg;
                out[3 * ray + 2] = a2 + light * bg;
                have = false;
            } else if (phase == 0) {
                // end of the reference's PASS 1 (rt_kernel.cu:415-418): restart for the scatter
                const float total_grad = a0 + a1 + a2;
                accum += light * bg * total_grad;
                phase = 1;
                t = r.tmin; light = 1.f; it = 0;
            } else {
                have = false;
            }
        }
    }
}

}  // namespace svoxb
