/*
 * CPU oracle for the svox octree-query and volume-rendering path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the
 * reference's algorithm (sxyu/svox v0.2.32).  It exists to check the CUDA
 * kernels and to be timed as the CPU baseline; the shipped library never
 * links, loads or calls it.
 *
 * Every function cites the reference source it follows (paths are relative
 * to the reference project root).  Mixed-precision sites of the reference
 * are reproduced as written there: the clamp bound, the reciprocal
 * direction and the pixel-ray set-up are evaluated in double and rounded to
 * float; everything else is float.
 *
 * nvcc contracts some float `a*b+c` expressions of the reference into a
 * fused multiply-add.  Which ones is a property of the compiled reference,
 * not of its source, so every such site is switchable here (OrcContract)
 * and this file must be compiled with -ffp-contract=off: a site is fused if
 * and only if its switch says so.  The defaults are the pattern that
 * reproduces the outputs of the reference extension compiled with nvcc 12.9
 * for sm_100 (see tests/golden).
 *
 * Parity status: pinned against (1) the reference's only known-answer
 * (docs/source/ex_opt_toy.rst:21), (2) outputs of the reference's Python
 * CPU path and (3) outputs of the reference's CUDA extension, both stored
 * as fixtures under tests/golden together with their generating scripts.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_FORMAT_RGBA 0
#define ORC_FORMAT_SH 1
#define ORC_FORMAT_SG 2
#define ORC_FORMAT_ASG 3

typedef struct {
    const float* data;     /* (M, N, N, N, K) */
    const int32_t* child;  /* (M, N, N, N): 0 = leaf, else relative node offset */
    int64_t M;
    int32_t N;
    int32_t K;
    float offset[3];
    float scaling[3];
    const float* extra;    /* (basis_dim, extra_cols): lobe parameters of SG / ASG, else NULL */
    int32_t extra_cols;
} OrcTree;

/* Field for field svox/csrc/include/data_spec.hpp:107-126. */
typedef struct {
    float step_size;
    float background_brightness;
    int32_t format;
    int32_t basis_dim;
    int32_t ndc_width;
    int32_t ndc_height;
    float ndc_focal;
    int32_t min_comp;
    int32_t max_comp;
    float sigma_thresh;
    float stop_thresh;
    int32_t density_softplus;
    float rgb_padding;
} OrcOptions;

typedef struct {
    int32_t transform; /* offset + scaling*q            (common.cuh:48)      */
    int32_t norm;      /* 0 none, 1 fma(z,z,fma(y,y,x*x)), 2 fma(z,z,fma(x,x,y*y)) (rt_kernel.cu:92) */
    int32_t pos;       /* origin + t*dir                 (rt_kernel.cu:263)   */
    int32_t dda_root;  /* t2 = t1 + invdir, t1 = -cen*invdir, root box  (rt_kernel.cu:215-216,240) */
    int32_t dda_leaf;  /* same expression inside a leaf  (rt_kernel.cu:271)   */
    int32_t sh_dot;    /* tmp += basis*coef              (rt_kernel.cu:287)   */
    int32_t color_pad; /* sigmoid*d_rgb_pad - padding    (rt_kernel.cu:289)   */
    int32_t out_acc;   /* out += weight*colour           (rt_kernel.cu:289)   */
    int32_t bg_acc;    /* out += T*background            (rt_kernel.cu:318)   */
    int32_t cam_xy;    /* 0 none, 1 fma(y,y,x*x), 2 fma(x,x,y*y) (rt_kernel.cu:766) */
    int32_t cam_rot;   /* per output row r (base-3 digit r): 0 none, 1 fma(c2,z,fma(c1,y,c0*x)),
                          2 fma(c2,z,fma(c0,x,c1*y))       (rt_kernel.cu:768-770) */
    int32_t ndc_shift; /* cen + t*dir                    (rt_kernel.cu:784)   */
    int32_t sh_basis;  /* a*b-c forms inside the SH basis (rt_kernel.cu:147-180) */
    int32_t ndc_norm;  /* sum of squares in the NDC re-normalisation, as `norm` (rt_kernel.cu:795) */
    int32_t descend;   /* x*N - floor(x*N) as fma(x, N, -floor) (common.cuh:68-76; exact, so moot, for N = 2) */
} OrcContract;

/* The forward and the backward kernels of the reference are separate
 * compilations of the same source, so each has its own pattern. */
#define ORC_DEFAULT_CONTRACT {1, 2, 1, 0, 0, 1, 1, 1, 1, 1, 1 + 3 * 2 + 9 * 2, 1, 1, 2, 0}
static OrcContract g_fw = ORC_DEFAULT_CONTRACT;
static OrcContract g_bw = ORC_DEFAULT_CONTRACT;
static const OrcContract* g_cur = &g_fw;
#define g_fc (*g_cur)

/* which: 0 = forward kernels and point query, 1 = backward render kernels */
void orc_set_contract(int which, const OrcContract* c) { *(which ? &g_bw : &g_fw) = *c; }
void orc_get_contract(int which, OrcContract* c) { *c = which ? g_bw : g_fw; }

static inline float madd(int fused, float a, float b, float c) {
    return fused ? fmaf(a, b, c) : a * b + c;
}

/* ------------------------------------------------------------------ */
/* svox/csrc/include/common.cuh:36-41.  The bound `float(1) - 1e-6` is a
 * double; min/max promote q to double; the result is rounded to float. */
static inline void clamp_coord(float* q) {
    for (int i = 0; i < 3; ++i) {
        double hi = (double)1.0f - 1e-6;
        double v = (double)q[i];
        v = hi < v ? hi : v;
        v = 0.0 > v ? 0.0 : v;
        q[i] = (float)v;
    }
}

/* svox/csrc/include/common.cuh:43-50 */
static inline void transform_coord(float* q, const float* offset, const float* scaling) {
    for (int i = 0; i < 3; ++i) q[i] = madd(g_fc.transform, scaling[i], q[i], offset[i]);
}

/* svox/csrc/include/common.cuh:52-90.  Returns the flat slot index
 * node*N^3 + u*N^2 + v*N + w of the leaf (the packed id of :81-82); the
 * leaf's record starts at slot*K floats.  xyz becomes the fractional
 * position inside the leaf, cube_sz the number of leaf-sized cells per side.
 * A bounded loop replaces while(true): a corrupt child array gives -1. */
static inline int64_t descend(const OrcTree* tr, float* xyz, float* cube_sz) {
    const float N = (float)tr->N;
    const int32_t Ni = tr->N;
    clamp_coord(xyz);
    int64_t node = 0;
    *cube_sz = N;
    for (int lvl = 0; lvl < 64; ++lvl) {
        const float x0 = xyz[0], x1 = xyz[1], x2 = xyz[2];
        xyz[0] *= N; xyz[1] *= N; xyz[2] *= N;
        int32_t u = (int32_t)floorf(xyz[0]);
        int32_t v = (int32_t)floorf(xyz[1]);
        int32_t w = (int32_t)floorf(xyz[2]);
        if (g_fc.descend) {
            xyz[0] = fmaf(x0, N, -(float)u); xyz[1] = fmaf(x1, N, -(float)v);
            xyz[2] = fmaf(x2, N, -(float)w);
        } else {
            xyz[0] -= (float)u; xyz[1] -= (float)v; xyz[2] -= (float)w;
        }
        int64_t slot = node * (int64_t)(Ni * Ni * Ni) + u * (Ni * Ni) + v * Ni + w;
        int32_t skip = tr->child[slot];
        if (skip == 0) return slot;
        *cube_sz *= N;
        node += skip;
        if (node < 0 || node >= tr->M) return -1;
    }
    return -1;
}

/* ------------------------------------------------------------------ */
/* Point query: svox/csrc/svox_kernel.cu:42-66,120-143 */
int orc_query_vertical(const OrcTree* tr, const float* points, int64_t Q,
                       float* values_out, int64_t* ids_out) {
    int bad = 0;
#pragma omp parallel for schedule(static) reduction(| : bad)
    for (int64_t i = 0; i < Q; ++i) {
        float xyz[3] = {points[3 * i], points[3 * i + 1], points[3 * i + 2]};
        float cs;
        transform_coord(xyz, tr->offset, tr->scaling);
        int64_t slot = descend(tr, xyz, &cs);
        if (slot < 0) { bad = 1; continue; }
        if (ids_out) ids_out[i] = slot;
        if (values_out)
            memcpy(values_out + i * tr->K, tr->data + slot * tr->K, sizeof(float) * tr->K);
    }
    return bad;
}

/* Point-query backward: svox/csrc/svox_kernel.cu:68-78,160-182.  The sum per
 * leaf is formed in double so that it does not depend on the order. */
int orc_query_vertical_backward(const OrcTree* tr, const float* points, int64_t Q,
                                const float* grad_out, int32_t Kg, double* grad_data) {
    int bad = 0;
#pragma omp parallel for schedule(static) reduction(| : bad)
    for (int64_t i = 0; i < Q; ++i) {
        float xyz[3] = {points[3 * i], points[3 * i + 1], points[3 * i + 2]};
        float cs;
        transform_coord(xyz, tr->offset, tr->scaling);
        int64_t slot = descend(tr, xyz, &cs);
        if (slot < 0) { bad = 1; continue; }
        for (int k = 0; k < Kg; ++k) {
#pragma omp atomic
            grad_data[slot * Kg + k] += (double)grad_out[i * Kg + k];
        }
    }
    return bad;
}

/* ------------------------------------------------------------------ */
/* SH constants: svox/csrc/rt_kernel.cu:53-83 (double literals rounded to float). */
static const float C0 = 0.28209479177387814;
static const float C1 = 0.4886025119029199;
static const float C2[] = {1.0925484305920792, -1.0925484305920792, 0.31539156525252005,
                           -1.0925484305920792, 0.5462742152960396};
static const float C3[] = {-0.5900435899266435, 2.890611442640554, -0.4570457994644658,
                           0.3731763325901154, -0.4570457994644658, 1.445305721320277,
                           -0.5900435899266435};
static const float C4[] = {2.5033429417967046, -1.7701307697799304, 0.9461746957575601,
                           -0.6690465435572892, 0.10578554691520431, -0.6690465435572892,
                           0.47308734787878004, -1.7701307697799304, 0.6258357354491761};

/* a*b - c with the switchable contraction of the SH basis expressions */
static inline float msub(float a, float b, float c) {
    return g_fc.sh_basis ? fmaf(a, b, -c) : a * b - c;
}

/* svox/csrc/rt_kernel.cu:141-181 (SH branch of maybe_precalc_basis). */
static void sh_basis(int basis_dim, const float* dir, float* out) {
    out[0] = C0;
    const float x = dir[0], y = dir[1], z = dir[2];
    const float xx = x * x, yy = y * y, zz = z * z;
    const float xy = x * y, yz = y * z, xz = x * z;
    switch (basis_dim) {
        case 25:
            out[16] = C4[0] * xy * (xx - yy);
            out[17] = C4[1] * yz * msub(3, xx, yy);
            out[18] = C4[2] * xy * msub(7, zz, 1.f);
            out[19] = C4[3] * yz * msub(7, zz, 3.f);
            out[20] = C4[4] * madd(g_fc.sh_basis, zz, msub(35, zz, 30), 3);
            out[21] = C4[5] * xz * msub(7, zz, 3);
            out[22] = C4[6] * (xx - yy) * msub(7, zz, 1.f);
            out[23] = C4[7] * xz * (g_fc.sh_basis ? fmaf(-3.f, yy, xx) : xx - 3 * yy);
            {
                float a = g_fc.sh_basis ? fmaf(-3.f, yy, xx) : xx - 3 * yy;
                float b = msub(3, xx, yy);
                float t = yy * b;
                out[24] = C4[8] * (g_fc.sh_basis ? fmaf(xx, a, -t) : xx * a - t);
            }
            /* fall through */
        case 16:
            out[9] = C3[0] * y * msub(3, xx, yy);
            out[10] = C3[1] * xy * z;
            out[11] = C3[2] * y * (msub(4, zz, xx) - yy);
            out[12] = C3[3] * z *
                      (g_fc.sh_basis ? fmaf(-3.f, yy, fmaf(-3.f, xx, 2 * zz))
                                     : 2 * zz - 3 * xx - 3 * yy);
            out[13] = C3[4] * x * (msub(4, zz, xx) - yy);
            out[14] = C3[5] * z * (xx - yy);
            out[15] = C3[6] * x * (g_fc.sh_basis ? fmaf(-3.f, yy, xx) : xx - 3 * yy);
            /* fall through */
        case 9:
            out[4] = C2[0] * xy;
            out[5] = C2[1] * yz;
            /* `2.0 * zz` is a double expression in the reference (:171) */
            out[6] = (float)((double)C2[2] * (2.0 * (double)zz - (double)xx - (double)yy));
            out[7] = C2[3] * xz;
            out[8] = C2[4] * (xx - yy);
            /* fall through */
        case 4:
            out[1] = -C1 * y;
            out[2] = C1 * z;
            out[3] = -C1 * x;
    }
}

void orc_sh_basis(int basis_dim, const float* dir, float* out) { sh_basis(basis_dim, dir, out); }

/* u.v as nvcc contracts u0*v0 + u1*v1 + u2*v2 (svox/csrc/rt_kernel.cu:103-107) */
static inline float dot3(const float* u, const float* v) {
    return g_fc.sh_basis ? fmaf(u[2], v[2], fmaf(u[1], v[1], u[0] * v[0]))
                         : u[0] * v[0] + u[1] * v[1] + u[2] * v[2];
}

/* svox/csrc/rt_kernel.cu:110-184 (maybe_precalc_basis): SH, or the spherical-Gaussian (SG) and
 * anisotropic spherical-Gaussian (ASG) lobes whose parameters are the rows of extra. */
static void colour_basis(const OrcTree* tr, const OrcOptions* opt, const float* dir, float* out) {
    const int n = opt->basis_dim;
    if (opt->format == ORC_FORMAT_SH) {
        sh_basis(n, dir, out);
    } else if (opt->format == ORC_FORMAT_SG) {
        for (int i = 0; i < n; ++i) {
            const float* p = tr->extra + (int64_t)i * tr->extra_cols;
            out[i] = expf(p[0] * (dot3(dir, p + 1) - 1.f)) / n;
        }
    } else if (opt->format == ORC_FORMAT_ASG) {
        for (int i = 0; i < n; ++i) {
            const float* p = tr->extra + (int64_t)i * tr->extra_cols;
            const float S = dot3(dir, p + 8), dx = dot3(dir, p + 2), dy = dot3(dir, p + 5);
            const float a = -p[0] * dx * dx, b = p[1] * dy;
            const float e = g_fc.sh_basis ? fmaf(-b, dy, a) : a - b * dy;
            out[i] = S * expf(e) / n;
        }
    }
}

/* svox/csrc/rt_kernel.cu:89-93 */
static inline float norm3(const float* d) {
    float a = d[0] * d[0], b = d[1] * d[1];
    float s;
    if (g_fc.norm == 1) s = fmaf(d[2], d[2], fmaf(d[1], d[1], a));
    else if (g_fc.norm == 2) s = fmaf(d[2], d[2], fmaf(d[0], d[0], b));
    else s = a + b + d[2] * d[2];
    return sqrtf(s);
}

/* svox/csrc/rt_kernel.cu:189-201 */
static inline float get_delta_scale(const float* scaling, float* dir) {
    dir[0] *= scaling[0]; dir[1] *= scaling[1]; dir[2] *= scaling[2];
    float delta_scale = 1.f / norm3(dir);
    dir[0] *= delta_scale; dir[1] *= delta_scale; dir[2] *= delta_scale;
    return delta_scale;
}

/* svox/csrc/rt_kernel.cu:203-220 */
static inline void dda_unit(int fused, const float* cen, const float* invdir, float* tmin,
                            float* tmax) {
    float t1, t2;
    *tmin = 0.0f;
    *tmax = 1e9f;
    for (int i = 0; i < 3; ++i) {
        t1 = -cen[i] * invdir[i];
        t2 = fused ? fmaf(-cen[i], invdir[i], invdir[i]) : t1 + invdir[i];
        *tmin = fmaxf(*tmin, fminf(t1, t2));
        *tmax = fminf(*tmax, fmaxf(t1, t2));
    }
}

static inline float softplus_m1(float x) { return logf(1 + expf(x - 1)); }
static inline float sigmoidf(float x) { return 1 / (1 + expf(-x)); }

static inline int out_dim_of(const OrcTree* tr, const OrcOptions* opt) {
    /* svox/csrc/rt_kernel.cu:1009-1015 */
    return opt->format != ORC_FORMAT_RGBA ? (tr->K - 1) / opt->basis_dim : tr->K - 1;
}

typedef struct {
    int64_t visits;   /* loop iterations */
    int64_t contrib;  /* iterations that passed the sigma test */
    int32_t hit;      /* ray entered the cube */
    /* optional per-visit log */
    int32_t log_cap;
    int64_t* log_slot;
    float* log_dt;
    float* log_t;
} OrcRayStats;

/* Per-ray set-up shared by forward and backward:
 * svox/csrc/rt_kernel.cu:228-248 / :329-348.  origin is in tree space. */
static inline int ray_setup(const OrcTree* tr, const float* origin, float* dir, float* invdir,
                            float* delta_scale, float* tmin, float* tmax) {
    *delta_scale = get_delta_scale(tr->scaling, dir);
    for (int i = 0; i < 3; ++i) invdir[i] = (float)(1.0 / ((double)dir[i] + 1e-9));
    dda_unit(g_fc.dda_root, origin, invdir, tmin, tmax);
    return !(*tmax < 0 || *tmin > *tmax);
}

/* svox/csrc/rt_kernel.cu:222-321 (trace_ray).  origin in tree space, dir is
 * modified in place as in the reference. */
/* Weight accumulation of the forward render (svox/csrc/rt_kernel.cu:298-304,
 * TreeSpec::_weight_accum): when set, every contributing sample adds its
 * weight to (or, with `max`, raises) the entry of its leaf.  The sum is kept
 * in double so that it does not depend on the order of the rays. */
static double* g_weight_accum = NULL;
static int g_weight_accum_max = 0;

void orc_set_weight_accum(double* buf, int use_max) {
    g_weight_accum = buf;
    g_weight_accum_max = use_max;
}

static inline void accumulate_weight(int64_t slot, float weight) {
    if (!g_weight_accum) return;
    if (g_weight_accum_max) {
#pragma omp critical(orc_weight_max)
        if ((double)weight > g_weight_accum[slot]) g_weight_accum[slot] = (double)weight;
    } else {
#pragma omp atomic
        g_weight_accum[slot] += (double)weight;
    }
}

static int trace_ray(const OrcTree* tr, const float* origin, float* dir, const float* vdir,
                     const OrcOptions* opt, float* out, OrcRayStats* st) {
    const int out_dim = out_dim_of(tr, opt);
    const int K = tr->K;
    float invdir[3], delta_scale, tmin, tmax;
    if (st) { st->visits = st->contrib = 0; st->hit = 0; }
    if (!ray_setup(tr, origin, dir, invdir, &delta_scale, &tmin, &tmax)) {
        for (int j = 0; j < out_dim; ++j) out[j] = opt->background_brightness;
        return 0;
    }
    if (st) st->hit = 1;
    for (int j = 0; j < out_dim; ++j) out[j] = 0.f;
    float pos[3], basis_fn[25];
    colour_basis(tr, opt, vdir, basis_fn);
    float light = 1.f, t = tmin, cube_sz;
    const float d_rgb_pad = 1 + 2 * opt->rgb_padding;
    while (t < tmax) {
        for (int j = 0; j < 3; ++j) pos[j] = madd(g_fc.pos, t, dir[j], origin[j]);
        int64_t slot = descend(tr, pos, &cube_sz);
        if (slot < 0) return 1;
        const float* val = tr->data + slot * K;
        float smin, smax;
        dda_unit(g_fc.dda_leaf, pos, invdir, &smin, &smax);
        const float t_sub = (smax - smin) / cube_sz;
        const float delta_t = t_sub + opt->step_size;
        float sigma = val[K - 1];
        if (opt->density_softplus) sigma = softplus_m1(sigma);
        if (st) {
            if (st->log_slot && st->visits < st->log_cap) {
                st->log_slot[st->visits] = slot;
                st->log_dt[st->visits] = delta_t;
                st->log_t[st->visits] = t;
            }
            st->visits++;
        }
        if (sigma > opt->sigma_thresh) {
            if (st) st->contrib++;
            const float att = expf(-delta_t * delta_scale * sigma);
            const float weight = light * (1.f - att);
            if (opt->format != ORC_FORMAT_RGBA) {
                for (int c = 0; c < out_dim; ++c) {
                    const int off = c * opt->basis_dim;
                    float tmp = 0.0f;
                    for (int i = opt->min_comp; i <= opt->max_comp; ++i)
                        tmp = madd(g_fc.sh_dot, basis_fn[i], val[off + i], tmp);
                    float col = g_fc.color_pad ? fmaf(sigmoidf(tmp), d_rgb_pad, -opt->rgb_padding)
                                               : sigmoidf(tmp) * d_rgb_pad - opt->rgb_padding;
                    out[c] = madd(g_fc.out_acc, weight, col, out[c]);
                }
            } else {
                for (int c = 0; c < out_dim; ++c) {
                    float col = g_fc.color_pad
                                    ? fmaf(sigmoidf(val[c]), d_rgb_pad, -opt->rgb_padding)
                                    : sigmoidf(val[c]) * d_rgb_pad - opt->rgb_padding;
                    out[c] = madd(g_fc.out_acc, weight, col, out[c]);
                }
            }
            light *= att;
            accumulate_weight(slot, weight);
            if (light <= opt->stop_thresh) {
                const float scale = (float)(1.0 / (1.0 - (double)light));
                for (int j = 0; j < out_dim; ++j) out[j] *= scale;
                return 0;
            }
        }
        t += delta_t;
    }
    for (int j = 0; j < out_dim; ++j)
        out[j] = madd(g_fc.bg_acc, light, opt->background_brightness, out[j]);
    return 0;
}

/* Optional second accumulator: the sum of |contribution| per element, the
 * scale against which a float-atomics sum may legitimately differ. */
static double* g_grad_abs = NULL;
static int64_t g_grad_abs_delta = 0; /* element offset from grad to grad_abs */

static inline void scatter_scaled(double* g, float v, double scale) {
#pragma omp atomic
    *g += (double)v;
    if (g_grad_abs) {
#pragma omp atomic
        g[g_grad_abs_delta] += scale;
    }
}

static inline void scatter(double* g, float v) { scatter_scaled(g, v, fabs((double)v)); }

/* svox/csrc/rt_kernel.cu:323-477 (trace_ray_backward).  Per-ray arithmetic
 * is float as in the reference; the scatter into grad is a double sum so
 * the result is independent of the order in which rays are processed. */
static int trace_ray_backward(const OrcTree* tr, const float* grad_output, const float* origin,
                              float* dir, const float* vdir, const OrcOptions* opt,
                              double* grad, OrcRayStats* st) {
    const int out_dim = out_dim_of(tr, opt);
    const int K = tr->K;
    float invdir[3], delta_scale, tmin, tmax;
    if (st) { st->visits = st->contrib = 0; st->hit = 0; }
    if (!ray_setup(tr, origin, dir, invdir, &delta_scale, &tmin, &tmax)) return 0;
    if (st) st->hit = 1;
    float pos[3], basis_fn[25];
    colour_basis(tr, opt, vdir, basis_fn);
    float accum = 0.0f;
    double accum_abs = 0.0; /* sum of |terms| of accum: the scale of its rounding error */
    const float d_rgb_pad = 1 + 2 * opt->rgb_padding;
    /* PASS 1 (:357-419) */
    {
        float light = 1.f, t = tmin, cube_sz;
        while (t < tmax) {
            for (int j = 0; j < 3; ++j) pos[j] = madd(g_fc.pos, t, dir[j], origin[j]);
            int64_t slot = descend(tr, pos, &cube_sz);
            if (slot < 0) return 1;
            const float* val = tr->data + slot * K;
            double* gval = grad + slot * K;
            float smin, smax;
            dda_unit(g_fc.dda_leaf, pos, invdir, &smin, &smax);
            const float t_sub = (smax - smin) / cube_sz;
            const float delta_t = t_sub + opt->step_size;
            float sigma = val[K - 1];
            if (opt->density_softplus) sigma = softplus_m1(sigma);
            if (st) st->visits++;
            if (sigma > 0.0f) {
                if (st) st->contrib++;
                const float att = expf(-delta_t * sigma * delta_scale);
                const float weight = light * (1.f - att);
                float total_color = 0.f;
                if (opt->format != ORC_FORMAT_RGBA) {
                    for (int c = 0; c < out_dim; ++c) {
                        const int off = c * opt->basis_dim;
                        float tmp = 0.0f;
                        for (int i = opt->min_comp; i <= opt->max_comp; ++i)
                            tmp = madd(g_fc.sh_dot, basis_fn[i], val[off + i], tmp);
                        const float sg = sigmoidf(tmp);
                        /* (1.0 - sigmoid) promotes the whole product to double (:390) */
                        const float tmp2 = (float)((double)(weight * sg) * (1.0 - (double)sg) *
                                                   (double)grad_output[c] * (double)d_rgb_pad);
                        for (int i = opt->min_comp; i <= opt->max_comp; ++i) {
                            const float toadd = basis_fn[i] * tmp2;
                            scatter(&gval[off + i], toadd);
                        }
                        float col = g_fc.color_pad ? fmaf(sg, d_rgb_pad, -opt->rgb_padding)
                                                   : sg * d_rgb_pad - opt->rgb_padding;
                        total_color = madd(g_fc.out_acc, col, grad_output[c], total_color);
                    }
                } else {
                    for (int c = 0; c < out_dim; ++c) {
                        const float sg = sigmoidf(val[c]);
                        const float toadd = weight * sg * (1.f - sg) * grad_output[c] * d_rgb_pad;
                        scatter(&gval[c], toadd);
                        float col = g_fc.color_pad ? fmaf(sg, d_rgb_pad, -opt->rgb_padding)
                                                   : sg * d_rgb_pad - opt->rgb_padding;
                        total_color = madd(g_fc.out_acc, col, grad_output[c], total_color);
                    }
                }
                light *= att;
                accum = madd(g_fc.out_acc, weight, total_color, accum);
                accum_abs += fabs((double)weight * total_color);
            }
            t += delta_t;
        }
        float total_grad = 0.f;
        for (int j = 0; j < out_dim; ++j) total_grad += grad_output[j];
        accum = madd(g_fc.bg_acc, light * opt->background_brightness, total_grad, accum);
        for (int j = 0; j < out_dim; ++j)
            accum_abs += fabs((double)light * opt->background_brightness * grad_output[j]);
    }
    /* PASS 2 (:420-475) */
    {
        float light = 1.f, t = tmin, cube_sz;
        while (t < tmax) {
            for (int j = 0; j < 3; ++j) pos[j] = madd(g_fc.pos, t, dir[j], origin[j]);
            int64_t slot = descend(tr, pos, &cube_sz);
            if (slot < 0) return 1;
            const float* val = tr->data + slot * K;
            double* gval = grad + slot * K;
            float smin, smax;
            dda_unit(g_fc.dda_leaf, pos, invdir, &smin, &smax);
            const float t_sub = (smax - smin) / cube_sz;
            const float delta_t = t_sub + opt->step_size;
            float sigma = val[K - 1];
            const float raw_sigma = sigma;
            if (opt->density_softplus) sigma = softplus_m1(sigma);
            if (sigma > 0.0f) {
                const float att = expf(-delta_t * sigma * delta_scale);
                const float weight = light * (1.f - att);
                float total_color = 0.f;
                if (opt->format != ORC_FORMAT_RGBA) {
                    for (int c = 0; c < out_dim; ++c) {
                        const int off = c * opt->basis_dim;
                        float tmp = 0.0f;
                        for (int i = opt->min_comp; i <= opt->max_comp; ++i)
                            tmp = madd(g_fc.sh_dot, basis_fn[i], val[off + i], tmp);
                        float col = g_fc.color_pad
                                        ? fmaf(sigmoidf(tmp), d_rgb_pad, -opt->rgb_padding)
                                        : sigmoidf(tmp) * d_rgb_pad - opt->rgb_padding;
                        total_color = madd(g_fc.out_acc, col, grad_output[c], total_color);
                    }
                } else {
                    for (int c = 0; c < out_dim; ++c) {
                        float col = g_fc.color_pad
                                        ? fmaf(sigmoidf(val[c]), d_rgb_pad, -opt->rgb_padding)
                                        : sigmoidf(val[c]) * d_rgb_pad - opt->rgb_padding;
                        total_color = madd(g_fc.out_acc, col, grad_output[c], total_color);
                    }
                }
                light *= att;
                accum = g_fc.out_acc ? fmaf(-weight, total_color, accum)
                                     : accum - weight * total_color;
                float inner = g_fc.out_acc ? fmaf(total_color, light, -accum)
                                           : total_color * light - accum;
                float gs = delta_t * delta_scale * inner *
                           (opt->density_softplus ? sigmoidf(raw_sigma - 1) : 1);
                /* the density gradient is a difference of two quantities of the
                 * size of accum's terms: that is its error scale */
                scatter_scaled(&gval[K - 1], gs,
                               fabs((double)delta_t * delta_scale) *
                                   (fabs((double)total_color * light) + accum_abs));
            }
            t += delta_t;
        }
    }
    return 0;
}

/* svox/csrc/rt_kernel.cu:758-772 (cam2world_ray); c2w is 3x4 row-major. */
static inline void cam2world_ray(int ix, int iy, float* dir, float* origin, const float* c2w,
                                 float fx, float fy, int width, int height) {
    float x = (float)(((double)ix - 0.5 * (double)width) / (double)fx);
    float y = (float)(-((double)iy - 0.5 * (double)height) / (double)fy);
    float s;
    if (g_fc.cam_xy == 1) s = fmaf(y, y, x * x);
    else if (g_fc.cam_xy == 2) s = fmaf(x, x, y * y);
    else s = x * x + y * y;
    float z = sqrtf((float)((double)s + 1.0));
    x /= z; y /= z; z = -1.0f / z;
    int code = g_fc.cam_rot; /* base-3 digits: pattern of row 0, 1, 2 */
    for (int r = 0; r < 3; ++r) {
        const float* c = c2w + 4 * r;
        const int pat = code % 3;
        code /= 3;
        if (pat == 1) dir[r] = fmaf(c[2], z, fmaf(c[1], y, c[0] * x));
        else if (pat == 2) dir[r] = fmaf(c[2], z, fmaf(c[0], x, c[1] * y));
        else dir[r] = c[0] * x + c[1] * y + c[2] * z;
        origin[r] = c[3];
    }
}

/* svox/csrc/rt_kernel.cu:775-796 (maybe_world2ndc), near = 1 */
static inline void maybe_world2ndc(const OrcOptions* opt, float* dir, float* cen) {
    if (opt->ndc_width < 0) return;
    const float near = 1.f;
    float t = -(near + cen[2]) / dir[2];
    for (int i = 0; i < 3; ++i) cen[i] = madd(g_fc.ndc_shift, t, dir[i], cen[i]);
    dir[0] = -((2 * opt->ndc_focal) / opt->ndc_width) * (dir[0] / dir[2] - cen[0] / cen[2]);
    dir[1] = -((2 * opt->ndc_focal) / opt->ndc_height) * (dir[1] / dir[2] - cen[1] / cen[2]);
    dir[2] = -2 * near / cen[2];
    cen[0] = -((2 * opt->ndc_focal) / opt->ndc_width) * (cen[0] / cen[2]);
    cen[1] = -((2 * opt->ndc_focal) / opt->ndc_height) * (cen[1] / cen[2]);
    cen[2] = 1 + 2 * near / cen[2];
    float a = dir[0] * dir[0], b = dir[1] * dir[1], s;
    if (g_fc.ndc_norm == 1) s = fmaf(dir[2], dir[2], fmaf(dir[1], dir[1], a));
    else if (g_fc.ndc_norm == 2) s = fmaf(dir[2], dir[2], fmaf(dir[0], dir[0], b));
    else s = a + b + dir[2] * dir[2];
    float n = sqrtf(s);
    dir[0] /= n; dir[1] /= n; dir[2] /= n;
}

/* ------------------------------------------------------------------ */
/* svox/csrc/rt_kernel.cu:717-733 + 1019-1036.  visits/contrib may be NULL. */
int orc_volume_render(const OrcTree* tr, const float* origins, const float* dirs,
                      const float* vdirs, int64_t Q, const OrcOptions* opt, float* out,
                      int32_t* visits, int32_t* contrib) {
    const int od = out_dim_of(tr, opt);
    int bad = 0;
#pragma omp parallel for schedule(dynamic, 64) reduction(| : bad)
    for (int64_t i = 0; i < Q; ++i) {
        float o[3] = {origins[3 * i], origins[3 * i + 1], origins[3 * i + 2]};
        float d[3] = {dirs[3 * i], dirs[3 * i + 1], dirs[3 * i + 2]};
        transform_coord(o, tr->offset, tr->scaling);
        OrcRayStats st;
        memset(&st, 0, sizeof st);
        bad |= trace_ray(tr, o, d, vdirs + 3 * i, opt, out + i * od, &st);
        if (visits) visits[i] = (int32_t)st.visits;
        if (contrib) contrib[i] = (int32_t)st.contrib;
    }
    return bad;
}

/* svox/csrc/rt_kernel.cu:479-715 (trace_ray_se_grad_hess): rendered colour,
 * gradient and Gauss-Newton diagonal of 1/2 (render - color_ref)^2 for one
 * ray, in three marches like the reference.  Per-ray arithmetic is float;
 * grad and hess are double sums.  Colour formats with at most 4 outputs. */
static int trace_ray_se_grad(const OrcTree* tr, const float* origin, float* dir,
                             const float* vdir, const OrcOptions* opt, const float* color_ref,
                             float* color_out, double* grad, double* hess) {
    const int out_dim = out_dim_of(tr, opt);
    const int K = tr->K;
    float invdir[3], delta_scale, tmin, tmax;
    if (!ray_setup(tr, origin, dir, invdir, &delta_scale, &tmin, &tmax)) {
        for (int j = 0; j < out_dim; ++j) color_out[j] = opt->background_brightness;
        return 0;
    }
    float pos[3], basis_fn[25];
    colour_basis(tr, opt, vdir, basis_fn);
    const float d_rgb_pad = 1 + 2 * opt->rgb_padding;
    const int sh = opt->format != ORC_FORMAT_RGBA;
    for (int j = 0; j < out_dim; ++j) color_out[j] = 0.f;
    /* PASS 1 (:517-563): residual */
    {
        float light = 1.f, t = tmin, cube_sz;
        while (t < tmax) {
            for (int j = 0; j < 3; ++j) pos[j] = madd(g_fc.pos, t, dir[j], origin[j]);
            int64_t slot = descend(tr, pos, &cube_sz);
            if (slot < 0) return 1;
            const float* val = tr->data + slot * K;
            float smin, smax;
            dda_unit(g_fc.dda_leaf, pos, invdir, &smin, &smax);
            const float delta_t = (smax - smin) / cube_sz + opt->step_size;
            float sigma = val[K - 1];
            if (opt->density_softplus) sigma = softplus_m1(sigma);
            if (sigma > 0.0f) {
                const float att = expf(-delta_t * delta_scale * sigma);
                const float weight = light * (1.f - att);
                for (int c = 0; c < out_dim; ++c) {
                    float tmp = 0.0f;
                    if (sh) {
                        const int off = c * opt->basis_dim;
                        for (int i = opt->min_comp; i <= opt->max_comp; ++i)
                            tmp = madd(g_fc.sh_dot, basis_fn[i], val[off + i], tmp);
                    } else {
                        tmp = val[c];
                    }
                    color_out[c] += weight * (sigmoidf(tmp) * d_rgb_pad - opt->rgb_padding);
                }
                light *= att;
            }
            t += delta_t;
        }
        for (int j = 0; j < out_dim; ++j)
            color_out[j] += light * opt->background_brightness - color_ref[j];
    }
    /* PASS 2 (:566-633): colour gradient and the full colour sum */
    float color_accum[4] = {0, 0, 0, 0};
    {
        float light = 1.f, t = tmin, cube_sz;
        while (t < tmax) {
            for (int j = 0; j < 3; ++j) pos[j] = madd(g_fc.pos, t, dir[j], origin[j]);
            int64_t slot = descend(tr, pos, &cube_sz);
            if (slot < 0) return 1;
            const float* val = tr->data + slot * K;
            double* gval = grad + slot * K;
            double* hval = hess + slot * K;
            float smin, smax;
            dda_unit(g_fc.dda_leaf, pos, invdir, &smin, &smax);
            const float delta_t = (smax - smin) / cube_sz + opt->step_size;
            float sigma = val[K - 1];
            if (opt->density_softplus) sigma = softplus_m1(sigma);
            if (sigma > 0.0f) {
                const float att = expf(-delta_t * sigma * delta_scale);
                const float weight = light * (1.f - att);
                for (int c = 0; c < out_dim; ++c) {
                    const int off = sh ? c * opt->basis_dim : c;
                    float tmp = 0.0f;
                    if (sh) {
                        for (int i = opt->min_comp; i <= opt->max_comp; ++i)
                            tmp = madd(g_fc.sh_dot, basis_fn[i], val[off + i], tmp);
                    } else {
                        tmp = val[c];
                    }
                    const float sg = sigmoidf(tmp);
                    const float grad_ci = (float)((double)(weight * sg) * (1.0 - (double)sg) *
                                                  (double)d_rgb_pad);
                    if (sh) {
                        for (int i = opt->min_comp; i <= opt->max_comp; ++i) {
                            const float grad_wi = basis_fn[i] * grad_ci;
                            scatter(&gval[off + i], grad_wi * color_out[c]);
#pragma omp atomic
                            hval[off + i] += (double)(grad_wi * grad_wi);
                        }
                    } else {
                        scatter(&gval[c], grad_ci * color_out[c]);
#pragma omp atomic
                        hval[c] += (double)(grad_ci * grad_ci);
                    }
                    color_accum[c] += weight * (sg * d_rgb_pad - opt->rgb_padding);
                }
                light *= att;
            }
            t += delta_t;
        }
        for (int j = 0; j < out_dim; ++j) color_accum[j] += light * opt->background_brightness;
    }
    /* PASS 3 (:636-709): density gradient */
    {
        float light = 1.f, t = tmin, cube_sz, color_curr[4];
        while (t < tmax) {
            for (int j = 0; j < 3; ++j) pos[j] = madd(g_fc.pos, t, dir[j], origin[j]);
            int64_t slot = descend(tr, pos, &cube_sz);
            if (slot < 0) return 1;
            const float* val = tr->data + slot * K;
            double* gval = grad + slot * K;
            double* hval = hess + slot * K;
            float smin, smax;
            dda_unit(g_fc.dda_leaf, pos, invdir, &smin, &smax);
            const float delta_t = (smax - smin) / cube_sz + opt->step_size;
            float sigma = val[K - 1];
            const float raw_sigma = sigma;
            if (opt->density_softplus) sigma = softplus_m1(sigma);
            if (sigma > 0.0f) {
                const float att = expf(-delta_t * sigma * delta_scale);
                const float weight = light * (1.f - att);
                for (int c = 0; c < out_dim; ++c) {
                    float tmp = 0.0f;
                    if (sh) {
                        const int off = c * opt->basis_dim;
                        for (int i = opt->min_comp; i <= opt->max_comp; ++i)
                            tmp = madd(g_fc.sh_dot, basis_fn[i], val[off + i], tmp);
                    } else {
                        tmp = val[c];
                    }
                    color_curr[c] = sigmoidf(tmp) * d_rgb_pad - opt->rgb_padding;
                    color_accum[c] -= weight * color_curr[c];
                }
                light *= att;
                for (int j = 0; j < out_dim; ++j) {
                    const float grad_sigma =
                        delta_t * delta_scale * (color_curr[j] * light - color_accum[j]);
                    const float grad2_sigma = grad_sigma * grad_sigma;
                    if (opt->density_softplus) {
                        const float sgm = sigmoidf(raw_sigma - 1);
                        const float d_sgm = sgm * (1.f - sgm);
                        scatter(&gval[K - 1], grad_sigma * color_out[j] * sgm);
#pragma omp atomic
                        hval[K - 1] += (double)(grad2_sigma * sgm * sgm + grad_sigma * d_sgm);
                    } else {
                        scatter(&gval[K - 1], grad_sigma * color_out[j]);
#pragma omp atomic
                        hval[K - 1] += (double)grad2_sigma;
                    }
                }
            }
            t += delta_t;
        }
    }
    for (int j = 0; j < out_dim; ++j) color_out[j] += color_ref[j];
    return 0;
}

/* svox/csrc/rt_kernel.cu:846-870 + 1111-1141 (se_grad). */
int orc_se_grad(const OrcTree* tr, const float* origins, const float* dirs, const float* vdirs,
                int64_t Q, const OrcOptions* opt, const float* colors, float* out, double* grad,
                double* hess) {
    const int od = out_dim_of(tr, opt);
    if (od > 4) return 2;
    int bad = 0;
#pragma omp parallel for schedule(dynamic, 64) reduction(| : bad)
    for (int64_t i = 0; i < Q; ++i) {
        float o[3] = {origins[3 * i], origins[3 * i + 1], origins[3 * i + 2]};
        float d[3] = {dirs[3 * i], dirs[3 * i + 1], dirs[3 * i + 2]};
        transform_coord(o, tr->offset, tr->scaling);
        bad |= trace_ray_se_grad(tr, o, d, vdirs + 3 * i, opt, colors + i * od, out + i * od,
                                 grad, hess);
    }
    return bad;
}

/* Per-visit log of one ray (leaf slot, delta_t, t at entry): returns the
 * number of visits; at most cap are stored. */
int64_t orc_trace_log(const OrcTree* tr, const float* origin, const float* dir,
                      const float* vdir, const OrcOptions* opt, int32_t cap, int64_t* slots,
                      float* dts, float* ts, float* out) {
    float o[3] = {origin[0], origin[1], origin[2]};
    float d[3] = {dir[0], dir[1], dir[2]};
    transform_coord(o, tr->offset, tr->scaling);
    OrcRayStats st;
    memset(&st, 0, sizeof st);
    st.log_cap = cap; st.log_slot = slots; st.log_dt = dts; st.log_t = ts;
    float tmp[64];
    trace_ray(tr, o, d, vdir, opt, out ? out : tmp, &st);
    return st.visits;
}

/* svox/csrc/rt_kernel.cu:736-756 + 1059-1083.  grad is (M*N^3*K) doubles,
 * zeroed by the caller. */
int orc_volume_render_backward(const OrcTree* tr, const float* origins, const float* dirs,
                               const float* vdirs, int64_t Q, const OrcOptions* opt,
                               const float* grad_out, double* grad, int32_t* visits,
                               int32_t* contrib) {
    const int od = out_dim_of(tr, opt);
    int bad = 0;
    g_cur = &g_bw;
#pragma omp parallel for schedule(dynamic, 64) reduction(| : bad)
    for (int64_t i = 0; i < Q; ++i) {
        float o[3] = {origins[3 * i], origins[3 * i + 1], origins[3 * i + 2]};
        float d[3] = {dirs[3 * i], dirs[3 * i + 1], dirs[3 * i + 2]};
        transform_coord(o, tr->offset, tr->scaling);
        OrcRayStats st;
        memset(&st, 0, sizeof st);
        bad |= trace_ray_backward(tr, grad_out + i * od, o, d, vdirs + 3 * i, opt, grad, &st);
        if (visits) visits[i] = (int32_t)st.visits;
        if (contrib) contrib[i] = (int32_t)st.contrib;
    }
    g_cur = &g_fw;
    return bad;
}

static inline void pixel_ray(const OrcTree* tr, const float* c2w, float fx, float fy, int W,
                             int H, const OrcOptions* opt, int64_t tid, float* o, float* d,
                             float* vd) {
    int iy = (int)(tid / W), ix = (int)(tid % W);
    cam2world_ray(ix, iy, d, o, c2w, fx, fy, W, H);
    vd[0] = d[0]; vd[1] = d[1]; vd[2] = d[2];
    maybe_world2ndc(opt, d, o);
    transform_coord(o, tr->offset, tr->scaling);
}

/* svox/csrc/rt_kernel.cu:799-819 + 1038-1057 */
int orc_volume_render_image(const OrcTree* tr, const float* c2w, float fx, float fy, int32_t W,
                            int32_t H, const OrcOptions* opt, float* out, int32_t* visits,
                            int32_t* contrib) {
    const int od = out_dim_of(tr, opt);
    const int64_t Q = (int64_t)W * H;
    int bad = 0;
#pragma omp parallel for schedule(dynamic, 64) reduction(| : bad)
    for (int64_t i = 0; i < Q; ++i) {
        float o[3], d[3], vd[3];
        pixel_ray(tr, c2w, fx, fy, W, H, opt, i, o, d, vd);
        OrcRayStats st;
        memset(&st, 0, sizeof st);
        bad |= trace_ray(tr, o, d, vd, opt, out + i * od, &st);
        if (visits) visits[i] = (int32_t)st.visits;
        if (contrib) contrib[i] = (int32_t)st.contrib;
    }
    return bad;
}

/* svox/csrc/rt_kernel.cu:821-844 + 1085-1109 */
int orc_volume_render_image_backward(const OrcTree* tr, const float* c2w, float fx, float fy,
                                     int32_t W, int32_t H, const OrcOptions* opt,
                                     const float* grad_out, double* grad) {
    const int od = out_dim_of(tr, opt);
    const int64_t Q = (int64_t)W * H;
    int bad = 0;
    g_cur = &g_bw;
#pragma omp parallel for schedule(dynamic, 64) reduction(| : bad)
    for (int64_t i = 0; i < Q; ++i) {
        float o[3], d[3], vd[3];
        pixel_ray(tr, c2w, fx, fy, W, H, opt, i, o, d, vd);
        bad |= trace_ray_backward(tr, grad_out + i * od, o, d, vd, opt, grad, NULL);
    }
    g_cur = &g_fw;
    return bad;
}

/* Pixel rays as the image kernels build them (world-space origin and
 * direction before the tree transform, and the view direction). */
void orc_pixel_rays(const float* c2w, float fx, float fy, int32_t W, int32_t H, float* origins,
                    float* dirs) {
    const int64_t Q = (int64_t)W * H;
    for (int64_t i = 0; i < Q; ++i)
        cam2world_ray((int)(i % W), (int)(i / W), dirs + 3 * i, origins + 3 * i, c2w, fx, fy, W, H);
}

/* Direct the next backward calls to also accumulate sum(|contribution|) into
 * grad_abs (same shape as grad; NULL switches it off).  grad_abs and grad
 * must be the two halves of ONE allocation: grad_abs = grad + n_elements. */
void orc_set_grad_abs(double* grad, double* grad_abs) {
    g_grad_abs = grad_abs;
    g_grad_abs_delta = grad_abs ? (int64_t)(grad_abs - grad) : 0;
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void orc_set_num_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
