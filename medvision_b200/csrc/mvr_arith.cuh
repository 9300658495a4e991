// Element-type arithmetic of the resampling path.
//
// The reference computes EVERYTHING in the tensor's element type (scalar_t of
// medvision/csrc/cuda/roi_align_rotated_3d_cuda_kernel.cuh:15-120): for half tensors the
// roi decode, the sample coordinates, the rotation, the interpolation weights and the tap
// sum are all rounded to half after every single operation (c10::Half operators widen to
// float, do one float operation and round back).  Results only match to the stated
// tolerance if that rounding sequence is reproduced, so every operation below is an
// explicitly rounded, never-contracted intrinsic:
//   * half: native `__h*_rn` instructions.  A correctly rounded half operation equals the
//     float operation followed by a rounding to half (float carries 24 >= 2*11+2 bits, so the
//     double rounding is innocuous for + - * /), which is what c10::Half does.
//   * float / double: `__f*_rn` / `__d*_rn`; products that nvcc fuses into the following add
//     in the reference build are selected by the contraction bits of `mvr_contraction`.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace mvr {

template <typename T> struct Ar;

template <> struct Ar<float> {
  typedef float T;
  static constexpr bool kCanFuse = true;
  __device__ __forceinline__ static T add(T a, T b) { return __fadd_rn(a, b); }
  __device__ __forceinline__ static T sub(T a, T b) { return __fsub_rn(a, b); }
  __device__ __forceinline__ static T mul(T a, T b) { return __fmul_rn(a, b); }
  __device__ __forceinline__ static T div(T a, T b) { return __fdiv_rn(a, b); }
  // a / 2^k written as a * 2^-k (r = 2^-k): the product is exact before its one rounding, so it equals the division
  __device__ __forceinline__ static T scale_pow2(T a, float r) { return __fmul_rn(a, r); }
  __device__ __forceinline__ static T fma_(T a, T b, T c) { return __fmaf_rn(a, b, c); }
  __device__ __forceinline__ static T neg(T a) { return -a; }
  __device__ __forceinline__ static T fi(int i) { return __int2float_rn(i); }
  __device__ __forceinline__ static T ff(float f) { return f; }
  __device__ __forceinline__ static T cosT(T a) { return cosf(a); }
  __device__ __forceinline__ static T sinT(T a) { return sinf(a); }
  __device__ __forceinline__ static float tof(T a) { return a; }
  __device__ __forceinline__ static int toi(T a) { return __float2int_rz(a); }
  __device__ __forceinline__ static T ceilT(T a) { return ceilf(a); }
  __device__ __forceinline__ static T halve_neg(T a) { return -a * 0.5f; }  // exact
  __device__ __forceinline__ static bool finite(T a) { return isfinite(a); }
  __device__ __forceinline__ static bool le_zero(T a) { return a <= 0.0f; }
  __device__ __forceinline__ static bool ge_half(T a) { return a >= 0.5f; }
  __device__ __forceinline__ static bool ge_one(T a) { return a >= 1.0f; }
};

template <> struct Ar<double> {
  typedef double T;
  static constexpr bool kCanFuse = true;
  __device__ __forceinline__ static T add(T a, T b) { return __dadd_rn(a, b); }
  __device__ __forceinline__ static T sub(T a, T b) { return __dsub_rn(a, b); }
  __device__ __forceinline__ static T mul(T a, T b) { return __dmul_rn(a, b); }
  __device__ __forceinline__ static T div(T a, T b) { return __ddiv_rn(a, b); }
  __device__ __forceinline__ static T scale_pow2(T a, float r) { return __dmul_rn(a, (double)r); }
  __device__ __forceinline__ static T fma_(T a, T b, T c) { return __fma_rn(a, b, c); }
  __device__ __forceinline__ static T neg(T a) { return -a; }
  __device__ __forceinline__ static T fi(int i) { return (double)i; }
  __device__ __forceinline__ static T ff(float f) { return (double)f; }
  __device__ __forceinline__ static T cosT(T a) { return cos(a); }
  __device__ __forceinline__ static T sinT(T a) { return sin(a); }
  __device__ __forceinline__ static float tof(T a) { return (float)a; }
  __device__ __forceinline__ static int toi(T a) { return __double2int_rz(a); }
  __device__ __forceinline__ static T ceilT(T a) { return ceil(a); }
  __device__ __forceinline__ static T halve_neg(T a) { return -a * 0.5; }
  __device__ __forceinline__ static bool finite(T a) { return isfinite(a); }
  __device__ __forceinline__ static bool le_zero(T a) { return a <= 0.0; }
  __device__ __forceinline__ static bool ge_half(T a) { return a >= 0.5; }
  __device__ __forceinline__ static bool ge_one(T a) { return a >= 1.0; }
};

template <> struct Ar<__half> {
  typedef __half T;
  static constexpr bool kCanFuse = false;
  __device__ __forceinline__ static T add(T a, T b) { return __hadd_rn(a, b); }
  __device__ __forceinline__ static T sub(T a, T b) { return __hsub_rn(a, b); }
  __device__ __forceinline__ static T mul(T a, T b) { return __hmul_rn(a, b); }
  __device__ __forceinline__ static T div(T a, T b) {
    return __float2half_rn(__fdiv_rn(__half2float(a), __half2float(b)));
  }
  // the float quotient by 2^k is exact, so the reference's float division + rounding is one rounded half product
  __device__ __forceinline__ static T scale_pow2(T a, float r) { return __hmul_rn(a, __float2half_rn(r)); }
  __device__ __forceinline__ static T fma_(T a, T b, T c) { return __hadd_rn(__hmul_rn(a, b), c); }  // never fused
  __device__ __forceinline__ static T neg(T a) { return __hneg(a); }
  __device__ __forceinline__ static T fi(int i) { return __float2half_rn(__int2float_rn(i)); }
  __device__ __forceinline__ static T ff(float f) { return __float2half_rn(f); }
  __device__ __forceinline__ static T cosT(T a) { return __float2half_rn(cosf(__half2float(a))); }
  __device__ __forceinline__ static T sinT(T a) { return __float2half_rn(sinf(__half2float(a))); }
  __device__ __forceinline__ static float tof(T a) { return __half2float(a); }
  __device__ __forceinline__ static int toi(T a) { return __float2int_rz(__half2float(a)); }
  __device__ __forceinline__ static T ceilT(T a) { return __float2half_rn(ceilf(__half2float(a))); }
  __device__ __forceinline__ static T halve_neg(T a) {
    return __float2half_rn(-__half2float(a) * 0.5f);  // rounds only for subnormal results, as the reference
  }
  __device__ __forceinline__ static bool finite(T a) { return isfinite(__half2float(a)); }
  __device__ __forceinline__ static bool le_zero(T a) { return __half2float(a) <= 0.0f; }
  __device__ __forceinline__ static bool ge_half(T a) { return __half2float(a) >= 0.5f; }
  __device__ __forceinline__ static bool ge_one(T a) { return __half2float(a) >= 1.0f; }
};

// Float contraction pattern: which products the reference build (nvcc -fmad=true) fused into
// the following addition.  Bit fields of one word; half never fuses.
//   bit  0      sample lattice  start + p*bin          0 plain | 1 fma(p, bin, start)
//   bit  1      roi centre      roi*scale - offset     0 plain | 1 fma(roi, scale, -offset)
//   bit  2      box size        end*scale - start      0 plain | 1 fma(end, scale, -start)
//   bits 3-4    tap sum         w1*v1 + w2*v2 + ...    0 plain | 1 fma(w1,v1,w2*v2) then fma chain
//                                                      | 2 fma(w2,v2,w1*v1) then fma chain
//   bits 5-6    2D rotation     x*a -/+ y*b            0 plain | 1 fma(x,a,-/+(y*b)) | 2 fma(-/+y,b,x*a)
//   bits 7-9, 10-12, 13-15   3D rotation rows 1..3   (a1*x + a2*y) + a3*z
//                               0 plain | 1 fma(a1,x,a2*y) + a3*z | 2 fma(a3,z,fma(a1,x,a2*y))
//                               | 3 fma(a2,y,a1*x) + a3*z | 4 fma(a3,z,fma(a2,y,a1*x)) | 5 fma(a3,z,a1*x + a2*y)
//   bits 16-17, 18-19, 20-21, 22-23   rotation entries R12, R13, R22, R23   a*b*c -/+ d*e
//                               0 plain | 1 fma(a*b,c,-/+(d*e)) | 2 fma(-/+d,e,(a*b)*c)
struct Fm {
  __host__ __device__ static constexpr int lattice(int fm) { return fm & 1; }
  __host__ __device__ static constexpr int centre(int fm) { return (fm >> 1) & 1; }
  __host__ __device__ static constexpr int boxsize(int fm) { return (fm >> 2) & 1; }
  __host__ __device__ static constexpr int tap(int fm) { return (fm >> 3) & 3; }
  __host__ __device__ static constexpr int rot2(int fm) { return (fm >> 5) & 3; }
  __host__ __device__ static constexpr int row(int fm, int r) { return (fm >> (7 + 3 * r)) & 7; }
  __host__ __device__ static constexpr int entry(int fm, int e) { return (fm >> (16 + 2 * e)) & 3; }
  __host__ __device__ static constexpr int make(int lattice, int centre, int boxsize, int tap, int rot2, int row1,
                                                int row2, int row3, int e12, int e13, int e22, int e23) {
    return lattice | (centre << 1) | (boxsize << 2) | (tap << 3) | (rot2 << 5) | (row1 << 7) | (row2 << 10) |
           (row3 << 13) | (e12 << 16) | (e13 << 18) | (e22 << 20) | (e23 << 22);
  }
};

// The pattern of the reference build (nvcc 12.9, default -fmad=true, sm_100a).
constexpr int kReferenceContraction = Fm::make(1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 2, 1);

}  // namespace mvr
