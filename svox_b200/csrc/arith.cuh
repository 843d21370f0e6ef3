// Fused-multiply-add pattern of the position arithmetic.
//
// The reference (svox/csrc/rt_kernel.cu, include/common.cuh) writes plain
// `a * b + c`; whether nvcc fuses each of them is a property of the compiled
// reference.  Rendered colours are extremely sensitive to the last bit of a
// sample position (a different bit can put a sample in the neighbouring leaf),
// so each such site is pinned here, 1 = fused (one rounding), 0 = separate
// multiply and add (two roundings), to the choice that reproduces the
// reference extension built with nvcc 12.9 for sm_100 on the seeded fixtures
// (tests/golden/ref_cuda_*.npz).  The forward and the backward kernels of the
// reference turned out to use the same pattern.
#pragma once

namespace svoxb {

constexpr int FC_TRANSFORM = 1;  // offset + scaling * q            (common.cuh:48)
constexpr int FC_NORM = 2;       // 1: fma(z,z,fma(y,y,x*x)); 2: fma(z,z,fma(x,x,y*y)); 0: none (rt_kernel.cu:92)
constexpr int FC_POS = 1;        // origin + t * dir                (rt_kernel.cu:263)
constexpr int FC_DDA_ROOT = 0;   // t2 = (-cen*invdir) + invdir, cube entry (rt_kernel.cu:215-216,240)
constexpr int FC_DDA_LEAF = 0;   // same expression inside a leaf   (rt_kernel.cu:271)
constexpr int FC_CAM_XY = 1;     // x*x + y*y: 1 fma(y,y,x*x), 2 fma(x,x,y*y), 0 none (rt_kernel.cu:766)
// c0*x + c1*y + c2*z per output row: 1 fma(c2,z,fma(c1,y,c0*x)), 2 fma(c2,z,fma(c0,x,c1*y)), 0 none
// (rt_kernel.cu:768-770; the three rows of the compiled reference differ)
__host__ __device__ constexpr int fc_cam_rot(int row) { return row == 0 ? 1 : 2; }
constexpr int FC_NDC_SHIFT = 1;  // cen + t * dir                   (rt_kernel.cu:784)

template <int FUSED>
__device__ __forceinline__ float mad_site(float a, float b, float c) {
    if (FUSED) return __fmaf_rn(a, b, c);
    return __fadd_rn(__fmul_rn(a, b), c);
}

// x*x + y*y + z*z with the pinned pattern
template <int MODE>
__device__ __forceinline__ float sumsq3(float x, float y, float z) {
    if (MODE == 1) return __fmaf_rn(z, z, __fmaf_rn(y, y, __fmul_rn(x, x)));
    if (MODE == 2) return __fmaf_rn(z, z, __fmaf_rn(x, x, __fmul_rn(y, y)));
    return __fadd_rn(__fadd_rn(__fmul_rn(x, x), __fmul_rn(y, y)), __fmul_rn(z, z));
}

}  // namespace svoxb
