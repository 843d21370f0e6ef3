// Volume rendering kernels: forward and backward, for ray batches and for
// perspective images.
//
// Replaces render_ray_kernel / render_image_kernel and their backward
// kernels (svox/csrc/rt_kernel.cu:717-756, 799-844) together with
// trace_ray / trace_ray_backward (rt_kernel.cu:222-477).
//
// What is different from the reference, by design:
//  * the top levels of the octree are resolved by one shared-memory lookup
//    (a jump table built per call), the reference walks from the root at
//    every sample;
//  * the output colour lives in registers and is written once (the reference
//    read-modify-writes the global output row at every sample);
//  * a leaf record is fetched with 128-bit loads when its size allows, and
//    only after the density test passed;
//  * basis_dim is a template parameter, so the SH basis and the record stay in
//    registers (the reference indexes local-memory arrays dynamically);
//  * the backward pass scatters a whole record's gradient with vector
//    reductions (red.global.add.v4.f32) in ONE march when the caller supplies
//    the forward output, instead of scalar atomics in two marches;
//  * warps pull 32-ray granules from a block-local counter, so a block's
//    warps stay busy whatever the spread of ray lengths;
//  * every loop is bounded and reports through the device status word.
//
// Sample positions follow the reference operation for operation (see
// arith.cuh): leaf sequences and step lengths are bit-identical.
#pragma once

#include "common.cuh"
#include "query.cuh"

namespace svoxb {

constexpr int kMaxSteps = 1 << 16;   // samples per ray before SVOXB_ERR_MARCH
constexpr int kMaxGenericOut = 32;   // colour channels in the generic kernel
constexpr int kMaxSeGradOut = 4;     // ... in se_grad, the reference's bound (rt_kernel.cu:1123)

// SH constants (the published real SH normalisation factors, as float).
__device__ constexpr float kC0 = 0.28209479177387814;
__device__ constexpr float kC1 = 0.4886025119029199;
__device__ constexpr float kC2[5] = {1.0925484305920792, -1.0925484305920792,
                                      0.31539156525252005, -1.0925484305920792,
                                      0.5462742152960396};
__device__ constexpr float kC3[7] = {-0.5900435899266435, 2.890611442640554,
                                      -0.4570457994644658, 0.3731763325901154,
                                      -0.4570457994644658, 1.445305721320277,
                                      -0.5900435899266435};
__device__ constexpr float kC4[9] = {2.5033429417967046,  -1.7701307697799304,
                                      0.9461746957575601,  -0.6690465435572892,
                                      0.10578554691520431, -0.6690465435572892,
                                      0.47308734787878004, -1.7701307697799304,
                                      0.6258357354491761};

// SH basis for a view direction, basis_dim in {1,4,9,16,25}
// (svox/csrc/rt_kernel.cu:141-181, same expression shapes).
template <int BD>
__device__ __forceinline__ void sh_basis(const float* __restrict__ dir, float* __restrict__ out) {
    out[0] = kC0;
    const float x = dir[0], y = dir[1], z = dir[2];
    const float xx = x * x, yy = y * y, zz = z * z;
    const float xy = x * y, yz = y * z, xz = x * z;
    if (BD >= 25) {
        out[16] = kC4[0] * xy * (xx - yy);
        out[17] = kC4[1] * yz * (3 * xx - yy);
        out[18] = kC4[2] * xy * (7 * zz - 1.f);
        out[19] = kC4[3] * yz * (7 * zz - 3.f);
        out[20] = kC4[4] * (zz * (35 * zz - 30) + 3);
        out[21] = kC4[5] * xz * (7 * zz - 3);
        out[22] = kC4[6] * (xx - yy) * (7 * zz - 1.f);
        out[23] = kC4[7] * xz * (xx - 3 * yy);
        out[24] = kC4[8] * (xx * (xx - 3 * yy) - yy * (3 * xx - yy));
    }
    if (BD >= 16) {
        out[9] = kC3[0] * y * (3 * xx - yy);
        out[10] = kC3[1] * xy * z;
        out[11] = kC3[2] * y * (4 * zz - xx - yy);
        out[12] = kC3[3] * z * (2 * zz - 3 * xx - 3 * yy);
        out[13] = kC3[4] * x * (4 * zz - xx - yy);
        out[14] = kC3[5] * z * (xx - yy);
        out[15] = kC3[6] * x * (xx - 3 * yy);
    }
    if (BD >= 9) {
        out[4] = kC2[0] * xy;
        out[5] = kC2[1] * yz;
        out[6] = kC2[2] * (2.0 * zz - xx - yy);  // double expression, as in the reference
        out[7] = kC2[3] * xz;
        out[8] = kC2[4] * (xx - yy);
    }
    if (BD >= 4) {
        out[1] = -kC1 * y;
        out[2] = kC1 * z;
        out[3] = -kC1 * x;
    }
}

// Spherical-Gaussian and anisotropic-spherical-Gaussian bases
// (svox/csrc/rt_kernel.cu:120-140): lobe i takes its parameters from row i of the tree's
// extra data.
__device__ __forceinline__ void lobe_basis(int format, int basis_dim, const float* __restrict__ extra,
                                        int cols, const float* __restrict__ dir,
                                        float* __restrict__ out) {
    const float x = dir[0], y = dir[1], z = dir[2];
#pragma unroll
    for (int i = 0; i < basis_dim; ++i) {
        const float* __restrict__ p = extra + (int64_t)i * cols;
        if (format == SVOXB_FORMAT_ASG) {
            const float S = x * __ldg(p + 8) + y * __ldg(p + 9) + z * __ldg(p + 10);
            const float dot_x = x * __ldg(p + 2) + y * __ldg(p + 3) + z * __ldg(p + 4);
            const float dot_y = x * __ldg(p + 5) + y * __ldg(p + 6) + z * __ldg(p + 7);
            out[i] = S * expf(-__ldg(p) * dot_x * dot_x - __ldg(p + 1) * dot_y * dot_y) / basis_dim;
        } else {
            const float d = x * __ldg(p + 1) + y * __ldg(p + 2) + z * __ldg(p + 3);
            out[i] = expf(__ldg(p) * (d - 1.f)) / basis_dim;
        }
    }
}

// The colour basis of a render for one view direction: SH, or (LOBES) one of the lobe bases.
// A compile-time choice: the SH kernels carry no trace of the other bases (with a run-time
// branch the training step's forward ran 2 % slower, with an out-of-line call 27 %).
template <int BD, bool LOBES>
__device__ __forceinline__ void colour_basis(const TreeArgs& tr, const svoxb_render_options& opt,
                                             const float* __restrict__ dir,
                                             float* __restrict__ out) {
    if constexpr (LOBES) {
        lobe_basis(opt.format, BD, tr.extra, tr.extra_cols, dir, out);
    } else {
        sh_basis<BD>(dir, out);
    }
}

// The same with the basis size known only at run time (at most 25 functions).
__device__ __forceinline__ void colour_basis_any(const TreeArgs& tr,
                                                 const svoxb_render_options& opt,
                                                 const float* __restrict__ dir,
                                                 float* __restrict__ out) {
    if (opt.format != SVOXB_FORMAT_SH) {
        lobe_basis(opt.format, opt.basis_dim, tr.extra, tr.extra_cols, dir, out);
        return;
    }
    switch (opt.basis_dim) {
        case 25: sh_basis<25>(dir, out); break;
        case 16: sh_basis<16>(dir, out); break;
        case 9: sh_basis<9>(dir, out); break;
        case 4: sh_basis<4>(dir, out); break;
        default: sh_basis<1>(dir, out); break;
    }
}

__device__ __forceinline__ float sigmoid_ref(float x) { return 1 / (1 + expf(-x)); }
__device__ __forceinline__ float softplus_m1(float x) { return logf(1 + expf(x - 1)); }

// _dda_unit (svox/csrc/rt_kernel.cu:203-220): slab test against the unit cube.
template <int FUSED>
__device__ __forceinline__ void dda_unit(float cx, float cy, float cz, float ix, float iy,
                                         float iz, float& tmin, float& tmax) {
    tmin = 0.0f;
    tmax = 1e9f;
    float t1, t2;
    t1 = __fmul_rn(-cx, ix);
    t2 = FUSED ? __fmaf_rn(-cx, ix, ix) : __fadd_rn(t1, ix);
    tmin = fmaxf(tmin, fminf(t1, t2)); tmax = fminf(tmax, fmaxf(t1, t2));
    t1 = __fmul_rn(-cy, iy);
    t2 = FUSED ? __fmaf_rn(-cy, iy, iy) : __fadd_rn(t1, iy);
    tmin = fmaxf(tmin, fminf(t1, t2)); tmax = fminf(tmax, fmaxf(t1, t2));
    t1 = __fmul_rn(-cz, iz);
    t2 = FUSED ? __fmaf_rn(-cz, iz, iz) : __fadd_rn(t1, iz);
    tmin = fmaxf(tmin, fminf(t1, t2)); tmax = fminf(tmax, fmaxf(t1, t2));
}

struct Ray {
    float ox, oy, oz;  // origin, tree space
    float dx, dy, dz;  // unit direction, tree space
    float ix, iy, iz;  // reciprocal direction
    float vdir[3];     // view direction for the colour basis
    float delta_scale;
    float tmin, tmax;
    bool hit;
};

// Per-ray set-up common to forward and backward: _get_delta_scale, the
// double-precision reciprocal and the cube slab test
// (svox/csrc/rt_kernel.cu:189-201, 236-240).  (ox,oy,oz) already in tree space.
__device__ __forceinline__ void ray_setup(Ray& r, const float* __restrict__ scaling) {
    float dx = __fmul_rn(r.dx, __ldg(scaling + 0));
    float dy = __fmul_rn(r.dy, __ldg(scaling + 1));
    float dz = __fmul_rn(r.dz, __ldg(scaling + 2));
    const float nrm = __fsqrt_rn(sumsq3<FC_NORM>(dx, dy, dz));
    r.delta_scale = __fdiv_rn(1.f, nrm);
    r.dx = dx = __fmul_rn(dx, r.delta_scale);
    r.dy = dy = __fmul_rn(dy, r.delta_scale);
    r.dz = dz = __fmul_rn(dz, r.delta_scale);
    r.ix = (float)(1.0 / ((double)dx + 1e-9));
    r.iy = (float)(1.0 / ((double)dy + 1e-9));
    r.iz = (float)(1.0 / ((double)dz + 1e-9));
    dda_unit<FC_DDA_ROOT>(r.ox, r.oy, r.oz, r.ix, r.iy, r.iz, r.tmin, r.tmax);
    r.hit = !(r.tmax < 0 || r.tmin > r.tmax);
}

// Ray sources ---------------------------------------------------------------
struct RayBatch {  // render_ray_kernel's inputs (svox/csrc/rt_kernel.cu:717-733)
    static constexpr bool kLobes = false;
    const float* __restrict__ origins;
    const float* __restrict__ dirs;
    const float* __restrict__ vdirs;

    __device__ __forceinline__ void load(int64_t i, const TreeArgs& tr,
                                         const svoxb_render_options&, Ray& r) const {
        r.ox = to_tree(__ldg(origins + 3 * i + 0), __ldg(tr.offset + 0), __ldg(tr.scaling + 0));
        r.oy = to_tree(__ldg(origins + 3 * i + 1), __ldg(tr.offset + 1), __ldg(tr.scaling + 1));
        r.oz = to_tree(__ldg(origins + 3 * i + 2), __ldg(tr.offset + 2), __ldg(tr.scaling + 2));
        r.dx = __ldg(dirs + 3 * i + 0);
        r.dy = __ldg(dirs + 3 * i + 1);
        r.dz = __ldg(dirs + 3 * i + 2);
        r.vdir[0] = __ldg(vdirs + 3 * i + 0);
        r.vdir[1] = __ldg(vdirs + 3 * i + 1);
        r.vdir[2] = __ldg(vdirs + 3 * i + 2);
    }
    // The view direction alone (colour basis of the backward's gradient records).
    __device__ __forceinline__ void load_vdir(int64_t i, const TreeArgs&,
                                              const svoxb_render_options&, float v[3]) const {
        v[0] = __ldg(vdirs + 3 * i + 0);
        v[1] = __ldg(vdirs + 3 * i + 1);
        v[2] = __ldg(vdirs + 3 * i + 2);
    }
};

struct PixelRays {  // render_image_kernel's inputs (svox/csrc/rt_kernel.cu:758-819)
    static constexpr bool kLobes = false;
    const float* __restrict__ c2w;  // row-major, row stride 4
    float fx, fy;
    int width, height;

    __device__ __forceinline__ void load(int64_t tid, const TreeArgs& tr,
                                         const svoxb_render_options& opt, Ray& r) const {
        const int iy = (int)(tid / width), ix = (int)(tid % width);
        // cam2world_ray: pixel centre offsets are formed in double
        float x = (float)((ix - 0.5 * width) / (double)fx);
        float y = (float)(-(iy - 0.5 * height) / (double)fy);
        float s;
        if (FC_CAM_XY == 1) s = __fmaf_rn(y, y, __fmul_rn(x, x));
        else if (FC_CAM_XY == 2) s = __fmaf_rn(x, x, __fmul_rn(y, y));
        else s = __fadd_rn(__fmul_rn(x, x), __fmul_rn(y, y));
        float z = __fsqrt_rn((float)((double)s + 1.0));
        x = __fdiv_rn(x, z); y = __fdiv_rn(y, z); z = __fdiv_rn(-1.0f, z);
        float d[3], o[3];
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            const float c0 = __ldg(c2w + 4 * k), c1 = __ldg(c2w + 4 * k + 1),
                        c2 = __ldg(c2w + 4 * k + 2);
            if (fc_cam_rot(k) == 1) d[k] = __fmaf_rn(c2, z, __fmaf_rn(c1, y, __fmul_rn(c0, x)));
            else if (fc_cam_rot(k) == 2) d[k] = __fmaf_rn(c2, z, __fmaf_rn(c0, x, __fmul_rn(c1, y)));
            else d[k] = __fadd_rn(__fadd_rn(__fmul_rn(c0, x), __fmul_rn(c1, y)), __fmul_rn(c2, z));
            o[k] = __ldg(c2w + 4 * k + 3);
            r.vdir[k] = d[k];
        }
        if (opt.ndc_width >= 0) {
            // maybe_world2ndc (svox/csrc/rt_kernel.cu:775-796), near = 1
            const float near = 1.f;
            const float t = __fdiv_rn(-__fadd_rn(near, o[2]), d[2]);
#pragma unroll
            for (int k = 0; k < 3; ++k) o[k] = mad_site<FC_NDC_SHIFT>(t, d[k], o[k]);
            const float ax = -__fdiv_rn(__fmul_rn(2.f, opt.ndc_focal), (float)opt.ndc_width);
            const float ay = -__fdiv_rn(__fmul_rn(2.f, opt.ndc_focal), (float)opt.ndc_height);
            const float d0 = __fmul_rn(ax, __fsub_rn(__fdiv_rn(d[0], d[2]), __fdiv_rn(o[0], o[2])));
            const float d1 = __fmul_rn(ay, __fsub_rn(__fdiv_rn(d[1], d[2]), __fdiv_rn(o[1], o[2])));
            const float d2 = __fdiv_rn(__fmul_rn(-2.f, near), o[2]);
            const float o0 = __fmul_rn(ax, __fdiv_rn(o[0], o[2]));
            const float o1 = __fmul_rn(ay, __fdiv_rn(o[1], o[2]));
            const float o2 = __fadd_rn(1.f, __fdiv_rn(__fmul_rn(2.f, near), o[2]));
            const float nrm = __fsqrt_rn(sumsq3<FC_NORM>(d0, d1, d2));
            d[0] = __fdiv_rn(d0, nrm); d[1] = __fdiv_rn(d1, nrm); d[2] = __fdiv_rn(d2, nrm);
            o[0] = o0; o[1] = o1; o[2] = o2;
        }
        r.ox = to_tree(o[0], __ldg(tr.offset + 0), __ldg(tr.scaling + 0));
        r.oy = to_tree(o[1], __ldg(tr.offset + 1), __ldg(tr.scaling + 1));
        r.oz = to_tree(o[2], __ldg(tr.offset + 2), __ldg(tr.scaling + 2));
        r.dx = d[0]; r.dy = d[1]; r.dz = d[2];
    }
    __device__ __forceinline__ void load_vdir(int64_t i, const TreeArgs& tr,
                                              const svoxb_render_options& opt, float v[3]) const {
        Ray r;
        load(i, tr, opt, r);
        v[0] = r.vdir[0]; v[1] = r.vdir[1]; v[2] = r.vdir[2];
    }
};

// A ray source whose colour basis is one of the lobe bases (SG / ASG) instead of SH.
template <class Source>
struct WithLobes : Source {
    static constexpr bool kLobes = true;
};

// One marching step: sample position, leaf, step length.
struct Step {
    LeafHit leaf;
    float delta_t;
};

__device__ __forceinline__ bool march_step(const TreeArgs& tr, const TopTable& top, const Ray& r,
                                           float t, float step_size, Step& s) {
    const float px = mad_site<FC_POS>(t, r.dx, r.ox);
    const float py = mad_site<FC_POS>(t, r.dy, r.oy);
    const float pz = mad_site<FC_POS>(t, r.dz, r.oz);
    const bool ok = (tr.N == 2) ? descend2(tr.child, tr.M, top, px, py, pz, s.leaf)
                                : descendN(tr.child, tr.M, tr.N, px, py, pz, s.leaf);
    if (!ok) return false;
    float smin, smax;
    dda_unit<FC_DDA_LEAF>(s.leaf.fx, s.leaf.fy, s.leaf.fz, r.ix, r.iy, r.iz, smin, smax);
    const float t_sub = __fdiv_rn(__fsub_rn(smax, smin), s.leaf.cube_sz);
    s.delta_t = __fadd_rn(t_sub, step_size);
    return true;
}

// Record access -------------------------------------------------------------
// VEC: the record is a whole number of 16-byte words and 16-byte aligned.
template <int K, bool VEC>
__device__ __forceinline__ void load_record(const float* __restrict__ rec, float* __restrict__ v) {
    if (VEC) {
        const float4* __restrict__ p = reinterpret_cast<const float4*>(rec);
#pragma unroll
        for (int i = 0; i < K / 4; ++i) {
            const float4 q = __ldg(p + i);
            v[4 * i] = q.x; v[4 * i + 1] = q.y; v[4 * i + 2] = q.z; v[4 * i + 3] = q.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < K; ++i) v[i] = __ldg(rec + i);
    }
}

template <int K, bool VEC>
__device__ __forceinline__ void scatter_record(float* __restrict__ g, const float* __restrict__ v) {
    if (VEC) {
#pragma unroll
        for (int i = 0; i < K / 4; ++i)
            red_add_v4(g + 4 * i, v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < K; ++i) atomicAdd(g + i, v[i]);
    }
}

// Granule scheduler: the block's warps pull 32-ray granules
// blockIdx.x + gridDim.x * k from a shared counter.
__device__ __forceinline__ int64_t next_granule(unsigned* counter, int lane) {
    unsigned k = 0;
    if (lane == 0) k = atomicAdd(counter, 1u);
    k = __shfl_sync(0xffffffffu, k, 0);
    return (int64_t)blockIdx.x + (int64_t)gridDim.x * k;
}

__device__ __forceinline__ TopTable stage_top(const TopTable& g, int32_t* smem, bool in_smem) {
    if (g.level == 0 || !in_smem) return g;
    const int n = 1 << (3 * g.level);
    for (int i = threadIdx.x; i < n; i += blockDim.x) smem[i] = g.cells[i];
    return TopTable{smem, g.level};
}

// ---------------------------------------------------------------------------
// Forward, SH colour with 3 channels, basis_dim BD (record K = 3*BD + 1)
template <int BD, bool VEC, int BLOCK, class Source>
__global__ void __launch_bounds__(BLOCK)
render_fwd_sh(TreeArgs tr, Source src, svoxb_render_options opt, TopTable topg, bool top_in_smem,
              float* __restrict__ out, int64_t Q) {
    constexpr int K = 3 * BD + 1;
    extern __shared__ int32_t s_top[];
    __shared__ unsigned s_next;
    if (threadIdx.x == 0) s_next = 0;
    const TopTable top = stage_top(topg, s_top, top_in_smem);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int64_t n_gran = (Q + 31) >> 5;
    const float d_rgb_pad = 1 + 2 * opt.rgb_padding;

    for (;;) {
        const int64_t gran = next_granule(&s_next, lane);
        if (gran >= n_gran) break;
        const int64_t ray = gran * 32 + lane;
        const bool valid = ray < Q;
        Ray r;
        r.hit = false;
        if (valid) {
            src.load(ray, tr, opt, r);
            ray_setup(r, tr.scaling);
        }
        float o0, o1, o2;
        o0 = o1 = o2 = r.hit ? 0.f : opt.background_brightness;
        float basis[BD];
        if (r.hit) {
            sh_basis<BD>(r.vdir, basis);
#pragma unroll
            for (int i = 0; i < BD; ++i)
                if (i < opt.min_comp || i > opt.max_comp) basis[i] = 0.f;
        }
        float light = 1.f, t = r.tmin;
        bool stopped = false;
        int it = 0;
        // Warp-uniform loop: the vote makes the warp reconverge every step.
        bool go = r.hit && t < r.tmax;
        while (__any_sync(0xffffffffu, go)) {
            if (go) {
                Step s;
                if (++it > kMaxSteps) {
                    report(SVOXB_ERR_MARCH);
                    go = false;
                } else if (!march_step(tr, top, r, t, opt.step_size, s)) {
                    go = false;
                } else {
                    const float* __restrict__ rec = tr.data + s.leaf.slot * K;
                    float sigma = __ldg(rec + (K - 1));
                    if (opt.density_softplus) sigma = softplus_m1(sigma);
                    if (sigma > opt.sigma_thresh) {
                        const float att = expf(-s.delta_t * r.delta_scale * sigma);
                        const float weight = light * (1.f - att);
                        if (tr.weight_accum != nullptr) accumulate_weight(tr, s.leaf.slot, weight);
                        float v[K];
                        load_record<K, VEC>(rec, v);
                        float c[3];
#pragma unroll
                        for (int ch = 0; ch < 3; ++ch) {
                            float tmp = 0.0f;
#pragma unroll
                            for (int i = 0; i < BD; ++i) tmp += basis[i] * v[ch * BD + i];
                            c[ch] = sigmoid_ref(tmp) * d_rgb_pad - opt.rgb_padding;
                        }
                        o0 += weight * c[0];
                        o1 += weight * c[1];
                        o2 += weight * c[2];
                        light *= att;
                        if (light <= opt.stop_thresh) {
                            const float scale = 1.0 / (1.0 - light);
                            o0 *= scale; o1 *= scale; o2 *= scale;
                            stopped = true;
                            go = false;
                        }
                    }
                    t = __fadd_rn(t, s.delta_t);
                    if (!(t < r.tmax)) go = false;
                }
            }
        }
        if (r.hit && !stopped) {
            o0 += light * opt.background_brightness;
            o1 += light * opt.background_brightness;
            o2 += light * opt.background_brightness;
        }
        if (valid) {
            out[3 * ray + 0] = o0;
            out[3 * ray + 1] = o1;
            out[3 * ray + 2] = o2;
        }
    }
}

// Backward, SH colour with 3 channels.  SINGLE: the forward output is given
// and both thresholds are off, so accum = <grad_out, fwd_out> and one march
// suffices; otherwise a first march forms accum as the reference's PASS 1.
template <int BD, bool VEC, int BLOCK, bool SINGLE, class Source>
__global__ void __launch_bounds__(BLOCK)
render_bwd_sh(TreeArgs tr, Source src, svoxb_render_options opt, TopTable topg, bool top_in_smem,
              const float* __restrict__ grad_out, const float* __restrict__ fwd_out,
              float* __restrict__ grad_data, int64_t Q) {
    constexpr int K = 3 * BD + 1;
    extern __shared__ int32_t s_top[];
    __shared__ unsigned s_next;
    if (threadIdx.x == 0) s_next = 0;
    const TopTable top = stage_top(topg, s_top, top_in_smem);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int64_t n_gran = (Q + 31) >> 5;
    const float d_rgb_pad = 1 + 2 * opt.rgb_padding;

    for (;;) {
        const int64_t gran = next_granule(&s_next, lane);
        if (gran >= n_gran) break;
        const int64_t ray = gran * 32 + lane;
        Ray r;
        r.hit = false;
        if (ray < Q) {
            src.load(ray, tr, opt, r);
            ray_setup(r, tr.scaling);
        }
        float basis[BD];
        float gch[3] = {0.f, 0.f, 0.f};
        float accum = 0.f;
        if (r.hit) {
            sh_basis<BD>(r.vdir, basis);
#pragma unroll
            for (int i = 0; i < BD; ++i)
                if (i < opt.min_comp || i > opt.max_comp) basis[i] = 0.f;
            gch[0] = __ldg(grad_out + 3 * ray);
            gch[1] = __ldg(grad_out + 3 * ray + 1);
            gch[2] = __ldg(grad_out + 3 * ray + 2);
            if (SINGLE) {
                accum = __ldg(fwd_out + 3 * ray) * gch[0];
                accum += __ldg(fwd_out + 3 * ray + 1) * gch[1];
                accum += __ldg(fwd_out + 3 * ray + 2) * gch[2];
            }
        }
        if (!SINGLE) {
            // PASS 1 of the reference (rt_kernel.cu:357-419) without the scatter
            float light = 1.f, t = r.tmin;
            int it = 0;
            bool go = r.hit && t < r.tmax;
            while (__any_sync(0xffffffffu, go)) {
                if (go) {
                    Step s;
                    if (++it > kMaxSteps) {
                        report(SVOXB_ERR_MARCH);
                        go = false;
                    } else if (!march_step(tr, top, r, t, opt.step_size, s)) {
                        go = false;
                    } else {
                        const float* __restrict__ rec = tr.data + s.leaf.slot * K;
                        float sigma = __ldg(rec + (K - 1));
                        if (opt.density_softplus) sigma = softplus_m1(sigma);
                        if (sigma > 0.0f) {
                            const float att = expf(-s.delta_t * sigma * r.delta_scale);
                            const float weight = light * (1.f - att);
                            float v[K];
                            load_record<K, VEC>(rec, v);
                            float total_color = 0.f;
#pragma unroll
                            for (int ch = 0; ch < 3; ++ch) {
                                float tmp = 0.0f;
#pragma unroll
                                for (int i = 0; i < BD; ++i) tmp += basis[i] * v[ch * BD + i];
                                total_color +=
                                    (sigmoid_ref(tmp) * d_rgb_pad - opt.rgb_padding) * gch[ch];
                            }
                            light *= att;
                            accum += weight * total_color;
                        }
                        t = __fadd_rn(t, s.delta_t);
                        if (!(t < r.tmax)) go = false;
                    }
                }
            }
            const float total_grad = gch[0] + gch[1] + gch[2];
            accum += light * opt.background_brightness * total_grad;
        }
        // Scatter march: colour-coefficient gradients (reference PASS 1) and
        // the density gradient (reference PASS 2, rt_kernel.cu:420-475).
        {
            float light = 1.f, t = r.tmin;
            int it = 0;
            bool go = r.hit && t < r.tmax;
            while (__any_sync(0xffffffffu, go)) {
                if (go) {
                    Step s;
                    if (++it > kMaxSteps) {
                        report(SVOXB_ERR_MARCH);
                        go = false;
                    } else if (!march_step(tr, top, r, t, opt.step_size, s)) {
                        go = false;
                    } else {
                        const int64_t off = s.leaf.slot * K;
                        const float* __restrict__ rec = tr.data + off;
                        float sigma = __ldg(rec + (K - 1));
                        const float raw_sigma = sigma;
                        if (opt.density_softplus) sigma = softplus_m1(sigma);
                        if (sigma > 0.0f) {
                            const float att = expf(-s.delta_t * sigma * r.delta_scale);
                            const float weight = light * (1.f - att);
                            float v[K];
                            load_record<K, VEC>(rec, v);
                            float total_color = 0.f;
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
                            accum -= weight * total_color;
                            v[K - 1] = s.delta_t * r.delta_scale * (total_color * light - accum) *
                                       (opt.density_softplus ? sigmoid_ref(raw_sigma - 1) : 1);
                            scatter_record<K, VEC>(grad_data + off, v);
                        }
                        t = __fadd_rn(t, s.delta_t);
                        if (!(t < r.tmax)) go = false;
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Per-ray march statistics (no counterpart in the reference): the number of
// leaves a ray samples, how many of them pass the forward density test
// (sigma > sigma_thresh, until the early stop) and how many the backward one
// (sigma > 0).  These are the V / C_f / C_b of the byte model.
template <int BLOCK, class Source>
__global__ void __launch_bounds__(BLOCK)
march_stats_kernel(TreeArgs tr, Source src, svoxb_render_options opt, TopTable topg,
                   bool top_in_smem, int32_t* __restrict__ visits,
                   int32_t* __restrict__ contrib_fwd, int32_t* __restrict__ contrib_bwd,
                   int64_t Q) {
    extern __shared__ int32_t s_top[];
    __shared__ unsigned s_next;
    if (threadIdx.x == 0) s_next = 0;
    const TopTable top = stage_top(topg, s_top, top_in_smem);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int64_t n_gran = (Q + 31) >> 5;
    const int K = tr.K;
    for (;;) {
        const int64_t gran = next_granule(&s_next, lane);
        if (gran >= n_gran) break;
        const int64_t ray = gran * 32 + lane;
        if (ray >= Q) continue;
        Ray r;
        src.load(ray, tr, opt, r);
        ray_setup(r, tr.scaling);
        int nv = 0, nf = 0, nb = 0;
        if (r.hit) {
            float light = 1.f, t = r.tmin;
            bool stopped = false;
            while (t < r.tmax && nv < kMaxSteps) {
                Step s;
                if (!march_step(tr, top, r, t, opt.step_size, s)) break;
                float sigma = __ldg(tr.data + s.leaf.slot * K + (K - 1));
                if (opt.density_softplus) sigma = softplus_m1(sigma);
                ++nv;
                if (sigma > 0.0f) ++nb;
                if (!stopped && sigma > opt.sigma_thresh) {
                    ++nf;
                    light *= expf(-s.delta_t * r.delta_scale * sigma);
                    if (light <= opt.stop_thresh) stopped = true;
                }
                t = __fadd_rn(t, s.delta_t);
            }
        }
        if (visits) visits[ray] = nv;
        if (contrib_fwd) contrib_fwd[ray] = nf;
        if (contrib_bwd) contrib_bwd[ray] = nb;
    }
}

// ---------------------------------------------------------------------------
// Generic kernels: any record size, RGBA or SH with run-time dimensions.
// Slower (local-memory arrays); used for layouts without a specialisation.
template <int BLOCK, class Source>
__global__ void __launch_bounds__(BLOCK)
render_fwd_generic(TreeArgs tr, Source src, svoxb_render_options opt, TopTable topg,
                   bool top_in_smem, float* __restrict__ out, int64_t Q, int out_dim) {
    extern __shared__ int32_t s_top[];
    __shared__ unsigned s_next;
    if (threadIdx.x == 0) s_next = 0;
    const TopTable top = stage_top(topg, s_top, top_in_smem);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int64_t n_gran = (Q + 31) >> 5;
    const int K = tr.K;
    const float d_rgb_pad = 1 + 2 * opt.rgb_padding;
    const bool sh = opt.format != SVOXB_FORMAT_RGBA;

    for (;;) {
        const int64_t gran = next_granule(&s_next, lane);
        if (gran >= n_gran) break;
        const int64_t ray = gran * 32 + lane;
        const bool valid = ray < Q;
        Ray r;
        r.hit = false;
        if (valid) {
            src.load(ray, tr, opt, r);
            ray_setup(r, tr.scaling);
        }
        float o[kMaxGenericOut];
        for (int j = 0; j < out_dim; ++j) o[j] = r.hit ? 0.f : opt.background_brightness;
        float basis[25];
        if (r.hit && sh) {
            colour_basis_any(tr, opt, r.vdir, basis);
        }
        float light = 1.f, t = r.tmin;
        bool stopped = false;
        int it = 0;
        // Warp-uniform loop: the vote makes the warp reconverge every step.
        bool go = r.hit && t < r.tmax;
        while (__any_sync(0xffffffffu, go)) {
            if (go) {
                Step s;
                if (++it > kMaxSteps) {
                    report(SVOXB_ERR_MARCH);
                    go = false;
                } else if (!march_step(tr, top, r, t, opt.step_size, s)) {
                    go = false;
                } else {
                    const float* __restrict__ rec = tr.data + s.leaf.slot * K;
                    float sigma = __ldg(rec + (K - 1));
                    if (opt.density_softplus) sigma = softplus_m1(sigma);
                    if (sigma > opt.sigma_thresh) {
                        const float att = expf(-s.delta_t * r.delta_scale * sigma);
                        const float weight = light * (1.f - att);
                        if (tr.weight_accum != nullptr)
                            accumulate_weight(tr, s.leaf.slot, weight);
                        for (int ch = 0; ch < out_dim; ++ch) {
                            float tmp;
                            if (sh) {
                                tmp = 0.0f;
                                const int off = ch * opt.basis_dim;
                                for (int i = opt.min_comp; i <= opt.max_comp; ++i)
                                    tmp += basis[i] * __ldg(rec + off + i);
                            } else {
                                tmp = __ldg(rec + ch);
                            }
                            o[ch] += weight * (sigmoid_ref(tmp) * d_rgb_pad - opt.rgb_padding);
                        }
                        light *= att;
                        if (light <= opt.stop_thresh) {
                            const float scale = 1.0 / (1.0 - light);
                            for (int j = 0; j < out_dim; ++j) o[j] *= scale;
                            stopped = true;
                            go = false;
                        }
                    }
                    t = __fadd_rn(t, s.delta_t);
                    if (!(t < r.tmax)) go = false;
                }
            }
        }
        if (r.hit && !stopped)
            for (int j = 0; j < out_dim; ++j) o[j] += light * opt.background_brightness;
        if (valid)
            for (int j = 0; j < out_dim; ++j) out[ray * out_dim + j] = o[j];
    }
}

// Generic backward: the reference's two marches with scalar atomics.
template <int BLOCK, class Source>
__global__ void __launch_bounds__(BLOCK)
render_bwd_generic(TreeArgs tr, Source src, svoxb_render_options opt, TopTable topg,
                   bool top_in_smem, const float* __restrict__ grad_out,
                   float* __restrict__ grad_data, int64_t Q, int out_dim) {
    extern __shared__ int32_t s_top[];
    __shared__ unsigned s_next;
    if (threadIdx.x == 0) s_next = 0;
    const TopTable top = stage_top(topg, s_top, top_in_smem);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int64_t n_gran = (Q + 31) >> 5;
    const int K = tr.K;
    const float d_rgb_pad = 1 + 2 * opt.rgb_padding;
    const bool sh = opt.format != SVOXB_FORMAT_RGBA;

    for (;;) {
        const int64_t gran = next_granule(&s_next, lane);
        if (gran >= n_gran) break;
        const int64_t ray = gran * 32 + lane;
        Ray r;
        r.hit = false;
        if (ray < Q) {
            src.load(ray, tr, opt, r);
            ray_setup(r, tr.scaling);
        }
        float basis[25];
        if (r.hit && sh) {
            colour_basis_any(tr, opt, r.vdir, basis);
        }
        const float* __restrict__ g = grad_out + (r.hit ? ray : 0) * out_dim;
        float accum = 0.f;
        for (int pass = 0; pass < 2; ++pass) {
            float light = 1.f, t = r.tmin;
            int it = 0;
            // Warp-uniform loop: the vote makes the warp reconverge every step.
            bool go = r.hit && t < r.tmax;
            while (__any_sync(0xffffffffu, go)) {
                if (go) {
                    Step s;
                    if (++it > kMaxSteps) {
                        report(SVOXB_ERR_MARCH);
                        go = false;
                    } else if (!march_step(tr, top, r, t, opt.step_size, s)) {
                        go = false;
                    } else {
                        const int64_t off = s.leaf.slot * K;
                        const float* __restrict__ rec = tr.data + off;
                        float sigma = __ldg(rec + (K - 1));
                        const float raw_sigma = sigma;
                        if (opt.density_softplus) sigma = softplus_m1(sigma);
                        if (sigma > 0.0f) {
                            const float att = expf(-s.delta_t * sigma * r.delta_scale);
                            const float weight = light * (1.f - att);
                            float total_color = 0.f;
                            for (int ch = 0; ch < out_dim; ++ch) {
                                float tmp;
                                const int coff = sh ? ch * opt.basis_dim : ch;
                                if (sh) {
                                    tmp = 0.0f;
                                    for (int i = opt.min_comp; i <= opt.max_comp; ++i)
                                        tmp += basis[i] * __ldg(rec + coff + i);
                                } else {
                                    tmp = __ldg(rec + ch);
                                }
                                const float sg = sigmoid_ref(tmp);
                                const float gc = __ldg(g + ch);
                                if (pass == 0) {
                                    if (sh) {
                                        const float tmp2 =
                                            weight * sg * (1.0 - sg) * gc * d_rgb_pad;
                                        for (int i = opt.min_comp; i <= opt.max_comp; ++i)
                                            atomicAdd(grad_data + off + coff + i, basis[i] * tmp2);
                                    } else {
                                        atomicAdd(grad_data + off + ch,
                                                  weight * sg * (1.f - sg) * gc * d_rgb_pad);
                                    }
                                }
                                total_color += (sg * d_rgb_pad - opt.rgb_padding) * gc;
                            }
                            light *= att;
                            if (pass == 0) {
                                accum += weight * total_color;
                            } else {
                                accum -= weight * total_color;
                                atomicAdd(grad_data + off + (K - 1),
                                          s.delta_t * r.delta_scale *
                                              (total_color * light - accum) *
                                              (opt.density_softplus ? sigmoid_ref(raw_sigma - 1)
                                                                    : 1));
                            }
                        }
                        t = __fadd_rn(t, s.delta_t);
                        if (!(t < r.tmax)) go = false;
                    }
                }
            }
            if (pass == 0 && r.hit) {
                float total_grad = 0.f;
                for (int j = 0; j < out_dim; ++j) total_grad += __ldg(g + j);
                accum += light * opt.background_brightness * total_grad;
            }
        }
    }
}

// Gradient and Gauss-Newton diagonal of the squared error 1/2 (render - colour)^2 for any
// record layout: what the reference's se_grad kernel adds up in its second and third march
// (svox/csrc/rt_kernel.cu:566-709), with its per-channel running sums.  One march is enough
// here because the colour the reference re-accumulates in its second march is the forward's
// output (`fwd_out`, rendered without thresholds), which the caller already has.
template <int BLOCK, class Source>
__global__ void __launch_bounds__(BLOCK)
render_se_grad_generic(TreeArgs tr, Source src, svoxb_render_options opt, TopTable topg,
                       bool top_in_smem, const float* __restrict__ fwd_out,
                       const float* __restrict__ color_ref, float* __restrict__ grad,
                       float* __restrict__ hess, int64_t Q, int out_dim) {
    extern __shared__ int32_t s_top[];
    __shared__ unsigned s_next;
    if (threadIdx.x == 0) s_next = 0;
    const TopTable top = stage_top(topg, s_top, top_in_smem);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int64_t n_gran = (Q + 31) >> 5;
    const int K = tr.K;
    const float d_rgb_pad = 1 + 2 * opt.rgb_padding;
    const bool sh = opt.format != SVOXB_FORMAT_RGBA;

    for (;;) {
        const int64_t gran = next_granule(&s_next, lane);
        if (gran >= n_gran) break;
        const int64_t ray = gran * 32 + lane;
        Ray r;
        r.hit = false;
        if (ray < Q) {
            src.load(ray, tr, opt, r);
            ray_setup(r, tr.scaling);
        }
        float basis[25];
        if (r.hit && sh) colour_basis_any(tr, opt, r.vdir, basis);
        float accum[kMaxSeGradOut], curr[kMaxSeGradOut], resid[kMaxSeGradOut];
        for (int j = 0; j < out_dim; ++j) {
            accum[j] = r.hit ? __ldg(fwd_out + ray * out_dim + j) : 0.f;
            resid[j] = r.hit ? accum[j] - __ldg(color_ref + ray * out_dim + j) : 0.f;
        }
        float light = 1.f, t = r.tmin;
        int it = 0;
        // Warp-uniform loop: the vote makes the warp reconverge every step.
        bool go = r.hit && t < r.tmax;
        while (__any_sync(0xffffffffu, go)) {
            if (go) {
                Step s;
                if (++it > kMaxSteps) {
                    report(SVOXB_ERR_MARCH);
                    go = false;
                } else if (!march_step(tr, top, r, t, opt.step_size, s)) {
                    go = false;
                } else {
                    const int64_t off = s.leaf.slot * K;
                    const float* __restrict__ rec = tr.data + off;
                    float sigma = __ldg(rec + (K - 1));
                    const float raw_sigma = sigma;
                    if (opt.density_softplus) sigma = softplus_m1(sigma);
                    if (sigma > 0.0f) {
                        const float att = expf(-s.delta_t * sigma * r.delta_scale);
                        const float weight = light * (1.f - att);
                        for (int ch = 0; ch < out_dim; ++ch) {
                            float tmp;
                            const int coff = sh ? ch * opt.basis_dim : ch;
                            if (sh) {
                                tmp = 0.0f;
                                for (int i = opt.min_comp; i <= opt.max_comp; ++i)
                                    tmp += basis[i] * __ldg(rec + coff + i);
                            } else {
                                tmp = __ldg(rec + ch);
                            }
                            const float sg = sigmoid_ref(tmp);
                            const float grad_ci = weight * sg * (1.0 - sg) * d_rgb_pad;
                            if (sh) {
                                for (int i = opt.min_comp; i <= opt.max_comp; ++i) {
                                    const float grad_wi = basis[i] * grad_ci;
                                    atomicAdd(grad + off + coff + i, grad_wi * resid[ch]);
                                    atomicAdd(hess + off + coff + i, grad_wi * grad_wi);
                                }
                            } else {
                                atomicAdd(grad + off + ch, grad_ci * resid[ch]);
                                atomicAdd(hess + off + ch, grad_ci * grad_ci);
                            }
                            curr[ch] = sg * d_rgb_pad - opt.rgb_padding;
                            accum[ch] -= weight * curr[ch];
                        }
                        light *= att;
                        float g = 0.f, h = 0.f;
                        for (int j = 0; j < out_dim; ++j) {
                            const float grad_sigma =
                                s.delta_t * r.delta_scale * (curr[j] * light - accum[j]);
                            if (opt.density_softplus) {
                                const float sgm = sigmoid_ref(raw_sigma - 1);
                                g += grad_sigma * resid[j] * sgm;
                                h += grad_sigma * grad_sigma * sgm * sgm +
                                     grad_sigma * (sgm * (1.f - sgm));
                            } else {
                                g += grad_sigma * resid[j];
                                h += grad_sigma * grad_sigma;
                            }
                        }
                        atomicAdd(grad + off + (K - 1), g);
                        atomicAdd(hess + off + (K - 1), h);
                    }
                    t = __fadd_rn(t, s.delta_t);
                    if (!(t < r.tmax)) go = false;
                }
            }
        }
    }
}

}  // namespace svoxb
