// Roi decode, sample lattice and interpolation taps of the resampling path, written once
// for every element type (see mvr_arith.cuh for why each step is a separately rounded
// operation).  Follows
//   roi decode + lattice   medvision/csrc/cuda/roi_align_{2d,3d}_cuda_kernel.cuh:26-69,
//                          medvision/csrc/cuda/roi_align_rotated_{2d,3d}_cuda_kernel.cuh:30-103
//   taps                   medvision/csrc/cuda/interpolation_helpers_{2d,3d}.h
#pragma once
#include "mvr_arith.cuh"

namespace mvr {

enum { KIND_BOX = 0, KIND_ROTATED = 1 };

// Geometry of one roi, decoded once per CTA.  Axis index 0 = x (w), 1 = y (h), 2 = z (d).
template <typename T>
struct RoiGeom {
  int batch;
  int grid[3];
  T start[3];   // box: roi start in the volume; rotated: -size/2 in the roi frame
  T bin[3];
  T centre[3];  // rotated only
  T rot[9];     // rotated 3D: R11..R33 (row major); rotated 2D: rot[0] = cos, rot[1] = sin
  T count_fwd, count_bwd;
};

template <typename T>
__device__ __forceinline__ T rot_entry(T a, T b, T c, T d, T e, bool minus, int mode_) {
  typedef Ar<T> A;
  const T ab = A::mul(a, b);
  const T de = A::mul(d, e);
  const int mode = A::kCanFuse ? mode_ : 0;
  if (mode == 1) return A::fma_(ab, c, minus ? A::neg(de) : de);
  const T abc = A::mul(ab, c);
  if (mode == 2) return A::fma_(minus ? A::neg(d) : d, e, abc);
  return minus ? A::sub(abc, de) : A::add(abc, de);
}

// osz = {ow, oh, od}
template <typename T>
__device__ void decode_roi(const T* __restrict__ rois, long long n, int ndim, int kind, const int* osz,
                           float spatial_scale, int sampling_ratio, int aligned, int fm, RoiGeom<T>& g) {
  typedef Ar<T> A;
  const int width = (kind == KIND_BOX) ? (ndim == 2 ? 5 : 7) : (ndim == 2 ? 6 : 10);
  const T scale = A::ff(spatial_scale);
  const T one = A::fi(1);
  T r[10];
  for (int k = 0; k < width; ++k) r[k] = rois[n * width + k];
  g.batch = A::toi(r[0]);
  T size[3];
  if (kind == KIND_BOX) {
    for (int a = 0; a < ndim; ++a) {
      const T s = A::mul(r[1 + a], scale);
      const T e = A::mul(r[1 + ndim + a], scale);
      T sz = (A::kCanFuse && Fm::boxsize(fm)) ? A::fma_(r[1 + ndim + a], scale, A::neg(s)) : A::sub(e, s);
      if (!A::ge_one(sz)) sz = one;  // max(size, 1); a NaN size becomes 1 (fmax)
      g.start[a] = s;
      size[a] = sz;
      g.centre[a] = A::fi(0);
    }
  } else {
    const T off = aligned ? A::ff(0.5f) : A::fi(0);
    for (int a = 0; a < ndim; ++a) {
      if (A::kCanFuse && Fm::centre(fm)) g.centre[a] = A::fma_(r[1 + a], scale, A::neg(off));
      else g.centre[a] = A::sub(A::mul(r[1 + a], scale), off);
      T sz = A::mul(r[1 + ndim + a], scale);
      if (!aligned && !A::ge_one(sz)) sz = one;
      size[a] = sz;
    }
    if (ndim == 2) {
      g.rot[0] = A::cosT(r[5]);
      g.rot[1] = A::sinT(r[5]);
    } else {
      const T cg = A::cosT(r[7]), sg = A::sinT(r[7]);
      const T cb = A::cosT(r[8]), sb = A::sinT(r[8]);
      const T ca = A::cosT(r[9]), sa = A::sinT(r[9]);
      g.rot[0] = A::mul(ca, cb);
      g.rot[1] = rot_entry<T>(ca, sb, sg, sa, cg, true, Fm::entry(fm, 0));
      g.rot[2] = rot_entry<T>(ca, sb, cg, sa, sg, false, Fm::entry(fm, 1));
      g.rot[3] = A::mul(sa, cb);
      g.rot[4] = rot_entry<T>(sa, sb, sg, ca, cg, false, Fm::entry(fm, 2));
      g.rot[5] = rot_entry<T>(sa, sb, cg, ca, sg, true, Fm::entry(fm, 3));
      g.rot[6] = A::neg(sb);
      g.rot[7] = A::mul(cb, sg);
      g.rot[8] = A::mul(cb, cg);
    }
  }
  int prod = 1;
  for (int a = 0; a < ndim; ++a) {
    const T o = A::fi(osz[a]);
    g.bin[a] = A::div(size[a], o);
    if (sampling_ratio > 0) {
      g.grid[a] = sampling_ratio;
    } else {
      const float cq = A::tof(A::ceilT(A::div(size[a], o)));
      g.grid[a] = (cq == cq && fabsf(cq) < 2e9f) ? (int)cq : 0;
    }
    if (kind == KIND_ROTATED) g.start[a] = A::halve_neg(size[a]);
    prod *= g.grid[a];
  }
  for (int a = ndim; a < 3; ++a) {
    g.grid[a] = 1;
    g.start[a] = g.bin[a] = g.centre[a] = A::fi(0);
  }
  g.count_fwd = A::fi(max(prod, 1));
  // the 2D backward kernels divide by the plain product, the 3D ones by max(product, 1)
  g.count_bwd = (ndim == 2) ? A::fi(prod) : A::fi(max(prod, 1));
}

// in-bin offset of sub-sample i:  ((i + .5) * bin) / g
template <typename T>
__device__ __forceinline__ T lattice_sub(T bin, int i, int g) {
  typedef Ar<T> A;
  return A::div(A::mul(A::ff((float)i + .5f), bin), A::fi(g));
}

// start + p*bin
template <typename T>
__device__ __forceinline__ T lattice_base(T start, int p, T bin, int fm) {
  typedef Ar<T> A;
  if (A::kCanFuse && Fm::lattice(fm)) return A::fma_(A::fi(p), bin, start);
  return A::add(start, A::mul(A::fi(p), bin));
}

// ((a1*x + a2*y) + a3*z) + c
template <typename T>
__device__ __forceinline__ T rot_row3(T a1, T x, T a2, T y, T a3, T z, T c, int mode_) {
  typedef Ar<T> A;
  const int mode = A::kCanFuse ? mode_ : 0;
  T t;
  switch (mode) {
    case 1: t = A::add(A::fma_(a1, x, A::mul(a2, y)), A::mul(a3, z)); break;
    case 2: t = A::fma_(a3, z, A::fma_(a1, x, A::mul(a2, y))); break;
    case 3: t = A::add(A::fma_(a2, y, A::mul(a1, x)), A::mul(a3, z)); break;
    case 4: t = A::fma_(a3, z, A::fma_(a2, y, A::mul(a1, x))); break;
    case 5: t = A::fma_(a3, z, A::add(A::mul(a1, x), A::mul(a2, y))); break;
    default: t = A::add(A::add(A::mul(a1, x), A::mul(a2, y)), A::mul(a3, z)); break;
  }
  return A::add(t, c);
}

// (x*a -/+ y*b) + c
template <typename T>
__device__ __forceinline__ T rot_row2(T x, T a, T y, T b, bool minus, T c, int fm) {
  typedef Ar<T> A;
  const int mode = A::kCanFuse ? Fm::rot2(fm) : 0;
  T t;
  if (mode == 1) {
    const T yb = A::mul(y, b);
    t = A::fma_(x, a, minus ? A::neg(yb) : yb);
  } else if (mode == 2) {
    t = A::fma_(minus ? A::neg(y) : y, b, A::mul(x, a));
  } else {
    t = minus ? A::sub(A::mul(x, a), A::mul(y, b)) : A::add(A::mul(x, a), A::mul(y, b));
  }
  return A::add(t, c);
}

// One axis of the interpolation helpers: clamp to >= 0, truncate, neighbour, low/high weight.
template <typename T>
struct AxisTap {
  int i0, i1;
  T l, h;
};

template <typename T>
__device__ __forceinline__ bool axis_outside(T c, int size) {
  const float f = Ar<T>::tof(c);  // exact for half; float compare equals the reference's for float
  return (f < -1.0f) || (f > (float)size);
}
template <>
__device__ __forceinline__ bool axis_outside<double>(double c, int size) {
  return (c < -1.0) || (c > (double)size);
}

template <typename T>
__device__ __forceinline__ void axis_tap(T c, int size, AxisTap<T>& t) {
  typedef Ar<T> A;
  if (A::le_zero(c)) c = A::fi(0);
  int i0 = A::toi(c);
  int i1;
  if (i0 >= size - 1) {
    i1 = i0 = size - 1;
    c = A::fi(i0);
  } else {
    i1 = i0 + 1;
  }
  t.i0 = i0;
  t.i1 = i1;
  t.l = A::sub(c, A::fi(i0));
  t.h = A::sub(A::fi(1), t.l);  // equals the reference's double-precision 1. - l rounded once
}

// in-bin offset of sub-sample I of a grid of G per axis, G a power of two known at compile time
template <typename T, int G>
__device__ __forceinline__ T lattice_sub_pow2(T bin, int i) {
  typedef Ar<T> A;
  static_assert(G == 1 || G == 2 || G == 4, "power of two");
  const T prod = A::mul(A::ff((float)i + .5f), bin);
  return (G == 1) ? prod : A::scale_pow2(prod, 1.0f / (float)G);
}

// order 0: weight 1 for the first tap, in the reference's order, whose per-axis weights are all >= 0.5
// (tap k uses the high weight of axis a when bit a of k is clear; x is the lowest bit, then y, then z)
template <typename T, int NDIM>
__device__ __forceinline__ void nearest_pick(const AxisTap<T>* t, T* w) {
  typedef Ar<T> A;
  bool lo[NDIM], hi[NDIM];
#pragma unroll
  for (int a = 0; a < NDIM; ++a) {
    lo[a] = A::ge_half(t[a].l);
    hi[a] = A::ge_half(t[a].h);
  }
  bool found = false;
#pragma unroll
  for (int k = 0; k < (1 << NDIM); ++k) {
    bool ok = !found;
#pragma unroll
    for (int a = 0; a < NDIM; ++a) ok = ok && (((k >> a) & 1) ? lo[a] : hi[a]);
    w[k] = ok ? A::fi(1) : A::fi(0);
    found = found || ok;
  }
}

// Weights and flat element offsets of the 2^ndim taps of a sample at (z, y, x).
// Returns false when the sample lies outside the [-1, size] band: value 0, no gradient.
// Tap order: k bit0 = x1, bit1 = y1, bit2 = z1 (the reference's w1..w8 / v1..v8 order).
// OFF = long long, or int when D*H*W < 2^31.
template <typename T, int NDIM, typename OFF = long long>
__device__ __forceinline__ bool make_taps(int D, int H, int W, T z, T y, T x, int order, T* w, OFF* off) {
  typedef Ar<T> A;
  AxisTap<T> t[3];
  if (axis_outside<T>(y, H) || axis_outside<T>(x, W)) return false;
  if (NDIM == 3 && axis_outside<T>(z, D)) return false;
  axis_tap<T>(x, W, t[0]);
  axis_tap<T>(y, H, t[1]);
  if (NDIM == 3) axis_tap<T>(z, D, t[2]);
  if (NDIM == 2) {
    const OFF y0 = (OFF)t[1].i0 * W, y1 = (OFF)t[1].i1 * W;
    off[0] = y0 + t[0].i0;
    off[1] = y0 + t[0].i1;
    off[2] = y1 + t[0].i0;
    off[3] = y1 + t[0].i1;
    if (order == 0) {
      nearest_pick<T, 2>(t, w);
    } else {
      w[0] = A::mul(t[1].h, t[0].h);
      w[1] = A::mul(t[1].h, t[0].l);
      w[2] = A::mul(t[1].l, t[0].h);
      w[3] = A::mul(t[1].l, t[0].l);
    }
  } else {
    const OFF HW = (OFF)H * W;
    const OFF z0 = t[2].i0 * HW, z1 = t[2].i1 * HW;
    const OFF y0 = (OFF)t[1].i0 * W, y1 = (OFF)t[1].i1 * W;
    off[0] = z0 + y0 + t[0].i0;
    off[1] = z0 + y0 + t[0].i1;
    off[2] = z0 + y1 + t[0].i0;
    off[3] = z0 + y1 + t[0].i1;
    off[4] = z1 + y0 + t[0].i0;
    off[5] = z1 + y0 + t[0].i1;
    off[6] = z1 + y1 + t[0].i0;
    off[7] = z1 + y1 + t[0].i1;
    if (order == 0) {
      nearest_pick<T, 3>(t, w);
    } else {
      const T hzhy = A::mul(t[2].h, t[1].h), hzly = A::mul(t[2].h, t[1].l);
      const T lzhy = A::mul(t[2].l, t[1].h), lzly = A::mul(t[2].l, t[1].l);
      w[0] = A::mul(hzhy, t[0].h);
      w[1] = A::mul(hzhy, t[0].l);
      w[2] = A::mul(hzly, t[0].h);
      w[3] = A::mul(hzly, t[0].l);
      w[4] = A::mul(lzhy, t[0].h);
      w[5] = A::mul(lzhy, t[0].l);
      w[6] = A::mul(lzly, t[0].h);
      w[7] = A::mul(lzly, t[0].l);
    }
  }
  return true;
}

// w1*v1 + w2*v2 + ... summed left to right.
template <typename T, int NT>
__device__ __forceinline__ T tap_sum(const T* w, const T* v, int fm) {
  typedef Ar<T> A;
  T acc;
  const int mode = A::kCanFuse ? Fm::tap(fm) : 0;
  if (mode) {
    acc = (mode == 1) ? A::fma_(w[0], v[0], A::mul(w[1], v[1])) : A::fma_(w[1], v[1], A::mul(w[0], v[0]));
#pragma unroll
    for (int k = 2; k < NT; ++k) acc = A::fma_(w[k], v[k], acc);
    return acc;
  }
  acc = A::mul(w[0], v[0]);
#pragma unroll
  for (int k = 1; k < NT; ++k) acc = A::add(acc, A::mul(w[k], v[k]));
  return acc;
}

// ---- Catmull-Rom (order 3) of the affine_* entry points --------------------------------------
// medvision/csrc/cuda_aug/interpolation_helpers_2d.h:335-424, interpolation_helpers_3d.h:572-792.
// Per axis: i1 = (int)c after the c <= 0 clamp, u = c - i1 (element type, then float), taps
// i1-1 .. i1+2 clamped into the image.  The reference writes every one of the 16 / 64 weights as a
// polynomial in DOUBLE over u, u^2, u^3 (u^2, u^3 rounded to float in 2D and to the element type
// in 3D) and rounds the result to the element type; those polynomials are the products of the
// per-axis cubics below, so the weights here are the products of three doubles -- equal to the
// reference's up to ~1e-16 before the rounding to the element type.
template <typename T>
__device__ __forceinline__ T from_double(double d);
template <> __device__ __forceinline__ float from_double<float>(double d) { return __double2float_rn(d); }
template <> __device__ __forceinline__ double from_double<double>(double d) { return d; }
template <> __device__ __forceinline__ __half from_double<__half>(double d) {
  return __float2half_rn(__double2float_rn(d));  // c10::Half(double) goes through float
}

template <typename T, bool POWERS_IN_T>
__device__ __forceinline__ void hermite_axis(T c, int size, int* idx, double* w) {
  typedef Ar<T> A;
  if (A::le_zero(c)) c = A::fi(0);
  const int i1 = A::toi(c);
  const float u = A::tof(A::sub(c, A::fi(i1)));
  double u2, u3;
  if (POWERS_IN_T) {  // 3D: `T ux2 = ux * ux; T ux3 = ux * ux * ux;` with float ux
    u2 = (double)A::tof(A::ff(__fmul_rn(u, u)));
    u3 = (double)A::tof(A::ff(__fmul_rn(__fmul_rn(u, u), u)));
  } else {            // 2D: float ux2, ux3
    u2 = (double)__fmul_rn(u, u);
    u3 = (double)__fmul_rn(__fmul_rn(u, u), u);
  }
  const double ud = (double)u;
  w[0] = -0.5 * u3 + u2 - 0.5 * ud;
  w[1] = 1.5 * u3 - 2.5 * u2 + 1.0;
  w[2] = -1.5 * u3 + 2.0 * u2 + 0.5 * ud;
  w[3] = 0.5 * u3 - 0.5 * u2;
#pragma unroll
  for (int k = 0; k < 4; ++k) idx[k] = min(max(i1 - 1 + k, 0), size - 1);
}

// running sum of w*v in the reference's order; float fuses as in the linear tap sum
template <typename T>
__device__ __forceinline__ T hermite_group4(const T* w, const T* v, int fm) {
  typedef Ar<T> A;
  if (A::kCanFuse && Fm::tap(fm)) {
    T t = A::fma_(w[0], v[0], A::mul(w[1], v[1]));
    t = A::fma_(w[2], v[2], t);
    return A::fma_(w[3], v[3], t);
  }
  T t = A::add(A::mul(w[0], v[0]), A::mul(w[1], v[1]));
  t = A::add(t, A::mul(w[2], v[2]));
  return A::add(t, A::mul(w[3], v[3]));
}

template <typename T>
__device__ T hermite_2d(const T* __restrict__ img, int H, int W, T y, T x, int fm) {
  typedef Ar<T> A;
  if (axis_outside<T>(y, H) || axis_outside<T>(x, W)) return A::fi(0);
  int ix[4], iy[4];
  double wx[4], wy[4];
  hermite_axis<T, false>(x, W, ix, wx);
  hermite_axis<T, false>(y, H, iy, wy);
  // one 16-term expression, summed left to right: w00*v00 + w10*v10 + ... (x fastest)
  T acc = A::fi(0);
  bool first = true;
  T pw = A::fi(0), pv = A::fi(0);
  for (int j = 0; j < 4; ++j)
    for (int i = 0; i < 4; ++i) {
      const T w = from_double<T>(wx[i] * wy[j]);
      const T v = __ldg(img + (long long)iy[j] * W + ix[i]);
      if (j == 0 && i == 0) { pw = w; pv = v; continue; }
      if (first) {
        acc = (A::kCanFuse && Fm::tap(fm)) ? A::fma_(pw, pv, A::mul(w, v)) : A::add(A::mul(pw, pv), A::mul(w, v));
        first = false;
      } else {
        acc = (A::kCanFuse && Fm::tap(fm)) ? A::fma_(w, v, acc) : A::add(acc, A::mul(w, v));
      }
    }
  return acc;
}

template <typename T>
__device__ T hermite_3d(const T* __restrict__ vol, int D, int H, int W, T z, T y, T x, int fm) {
  typedef Ar<T> A;
  if (axis_outside<T>(y, H) || axis_outside<T>(x, W) || axis_outside<T>(z, D)) return A::fi(0);
  int ix[4], iy[4], iz[4];
  double wx[4], wy[4], wz[4];
  hermite_axis<T, true>(x, W, ix, wx);
  hermite_axis<T, true>(y, H, iy, wy);
  hermite_axis<T, true>(z, D, iz, wz);
  // val = 0; val += (four terms along x) for every (y, z), z outermost
  T val = A::fi(0);
  for (int k = 0; k < 4; ++k)
    for (int j = 0; j < 4; ++j) {
      T w[4], v[4];
      const T* row = vol + ((long long)iz[k] * H + iy[j]) * W;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        w[i] = from_double<T>(wx[i] * wy[j] * wz[k]);
        v[i] = __ldg(row + ix[i]);
      }
      val = A::add(val, hermite_group4<T>(w, v, fm));
    }
  return val;
}

}  // namespace mvr
