// TEST INFRASTRUCTURE -- NOT PRODUCT CODE.
//
// CPU restatement of the MedVision RoI Align / RoI Align Rotated / affine_{2d,3d}
// resampling kernels, used only as the checker in tests, in the smoke test and as the
// timed "what the reference computes, on host cores" baseline.  The shipped library
// never links or calls this file.
//
// Pinning: the reference's own tests for this path hold no golden vectors or
// assertions (test/ops_test_RoIAlign.py, test/ops_test_interpolation.py only print and
// save images).  This restatement is pinned instead against (a) outputs of the
// reference's own CUDA kernels, compiled unmodified and run on a B200
// (tests/golden/*.npz with the script that made them) and (b) torchvision's CPU
// roi_align(aligned=False) for the 2D axis-aligned forward.
//
// Every arithmetic step is written out as one rounded operation in the reference's
// element type (float, double, or half with c10::Half semantics: operands widened to
// float, one float operation, result rounded to nearest-even half), in the
// reference's order:
//   roi decode / sample lattice / loops
//     axis-aligned 2D   medvision/csrc/cuda/roi_align_2d_cuda_kernel.cuh:19-73 (fwd) 85-165 (bwd)
//     axis-aligned 3D   medvision/csrc/cuda/roi_align_3d_cuda_kernel.cuh:19-85, 97-201
//     rotated 2D        medvision/csrc/cuda/roi_align_rotated_2d_cuda_kernel.cuh:23-89, 101-195
//     rotated 3D        medvision/csrc/cuda/roi_align_rotated_3d_cuda_kernel.cuh:23-119, 130-264
//     affine_2d/3d      medvision/csrc/cuda_aug/affine_{2d,3d}_cuda_kernel.cuh (same as rotated fwd
//                       for order 0/1; order 3 adds the Catmull-Rom taps below)
//   interpolation       medvision/csrc/cuda/interpolation_helpers_2d.h:6-198,
//                       medvision/csrc/cuda/interpolation_helpers_3d.h:6-265
//   Catmull-Rom         medvision/csrc/cuda_aug/interpolation_helpers_2d.h:335-424,
//                       medvision/csrc/cuda_aug/interpolation_helpers_3d.h:572-792
//
// Float contraction: the reference is built with nvcc's default -fmad=true, so for
// float/double the device code may fuse a*b+c.  `fma_mode` selects which products
// are fused here (0 = none; see Arith<float>::mad* below), so tests can state which
// contraction pattern reproduces the device result.  Half arithmetic cannot fuse
// (a rounding to half separates every product from the following sum).

#include <cmath>
#include <cstdint>
#include <cstring>
#include <algorithm>
#include <vector>
#include <atomic>
#include <thread>
#include <immintrin.h>

namespace {

enum { DT_F32 = 0, DT_F16 = 1, DT_F64 = 2 };
enum { KIND_BOX = 0, KIND_ROTATED = 1 };

// ------------------------------------------------------------------ host threading
// Dynamic self-scheduling over [0, n) on plain std::thread workers (no OpenMP runtime needed).
template <class F>
void parallel_for(int64_t n, int nthreads, F body) {
  if (nthreads <= 0) nthreads = (int)std::max(1u, std::thread::hardware_concurrency());
  nthreads = (int)std::min<int64_t>(nthreads, std::max<int64_t>(n, 1));
  if (nthreads == 1) {
    for (int64_t i = 0; i < n; ++i) body(i);
    return;
  }
  std::atomic<int64_t> next(0);
  std::vector<std::thread> pool;
  for (int t = 0; t < nthreads; ++t)
    pool.emplace_back([&]() {
      for (;;) {
        const int64_t i = next.fetch_add(1);
        if (i >= n) break;
        body(i);
      }
    });
  for (auto& th : pool) th.join();
}

// ------------------------------------------------------------------ half helpers
inline float h2f(uint16_t h) { return _cvtsh_ss(h); }
inline uint16_t f2h(float f) { return _cvtss_sh(f, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC); }
inline float rh(float f) { return h2f(f2h(f)); }  // round a float to the nearest half, kept as float

// ------------------------------------------------------------------ arithmetic policies
// T is the carrier type of a value of the reference's scalar_t.
template <int DT> struct Arith;

template <> struct Arith<DT_F32> {
  typedef float T;
  typedef float S;  // storage
  static T ld(const void* p, int64_t i) { return ((const float*)p)[i]; }
  static void st(void* p, int64_t i, T v) { ((float*)p)[i] = v; }
  static T add(T a, T b) { return a + b; }
  static T sub(T a, T b) { return a - b; }
  static T mul(T a, T b) { return a * b; }
  static T div(T a, T b) { return a / b; }
  static T neg(T a) { return -a; }
  static T fi(int i) { return (float)i; }
  static T ff(float f) { return f; }
  static T fd(double d) { return (float)d; }
  static T cosT(T a) { return cosf(a); }
  static T sinT(T a) { return sinf(a); }
  static T fma_(T a, T b, T c) { return fmaf(a, b, c); }
  static const bool can_fuse = true;
};

template <> struct Arith<DT_F64> {
  typedef double T;
  typedef double S;
  static T ld(const void* p, int64_t i) { return ((const double*)p)[i]; }
  static void st(void* p, int64_t i, T v) { ((double*)p)[i] = v; }
  static T add(T a, T b) { return a + b; }
  static T sub(T a, T b) { return a - b; }
  static T mul(T a, T b) { return a * b; }
  static T div(T a, T b) { return a / b; }
  static T neg(T a) { return -a; }
  static T fi(int i) { return (double)i; }
  static T ff(float f) { return (double)f; }
  static T fd(double d) { return d; }
  static T cosT(T a) { return cos(a); }
  static T sinT(T a) { return sin(a); }
  static T fma_(T a, T b, T c) { return fma(a, b, c); }
  static const bool can_fuse = true;
};

// c10::Half semantics (torch/headeronly/util/Half.h): Half op Half = Half(float(a) op float(b));
// Half op int converts the int to Half first; construction from float/double rounds to
// nearest even (double goes through float).  The carrier is a float that always holds a
// half-representable value.
template <> struct Arith<DT_F16> {
  typedef float T;
  typedef uint16_t S;
  static T ld(const void* p, int64_t i) { return h2f(((const uint16_t*)p)[i]); }
  static void st(void* p, int64_t i, T v) { ((uint16_t*)p)[i] = f2h(v); }
  static T add(T a, T b) { return rh(a + b); }
  static T sub(T a, T b) { return rh(a - b); }
  static T mul(T a, T b) { return rh(a * b); }
  static T div(T a, T b) { return rh(a / b); }
  static T neg(T a) { return -a; }
  static T fi(int i) { return rh((float)i); }
  static T ff(float f) { return rh(f); }
  static T fd(double d) { return rh((float)d); }
  static T cosT(T a) { return rh(cosf(a)); }
  static T sinT(T a) { return rh(sinf(a)); }
  static T fma_(T a, T b, T c) { return rh(rh(a * b) + c); }  // never fused
  static const bool can_fuse = false;
};

// Which float products the device compiler fused into the following add (half never fuses).
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
  static int lattice(int fm) { return fm & 1; }
  static int centre(int fm) { return (fm >> 1) & 1; }
  static int boxsize(int fm) { return (fm >> 2) & 1; }
  static int tap(int fm) { return (fm >> 3) & 3; }
  static int rot2(int fm) { return (fm >> 5) & 3; }
  static int row(int fm, int r) { return (fm >> (7 + 3 * r)) & 7; }
  static int entry(int fm, int e) { return (fm >> (16 + 2 * e)) & 3; }
};

// ------------------------------------------------------------------ interpolation
// One axis of interpolation_helpers_*: clamp, floor, neighbour and the low/high weights.
template <class A>
struct AxisTap {
  int i0, i1;
  typename A::T l, h;
};

template <class A>
inline void axis_tap(typename A::T c, int size, AxisTap<A>& t) {
  typedef typename A::T T;
  if (c <= (T)0) c = (T)0;
  int i0 = (c == c) ? (int)c : 0;  // device float->int conversion maps NaN to 0
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
  t.h = A::fd(1.0 - (double)t.l);
}

// `c < -1.0 || c > size` of the reference (double / float comparisons of an exact value).
template <class A>
inline bool outside(typename A::T c, int size) {
  return ((double)c < -1.0) || ((double)c > (double)size);
}

// Left-to-right sum of w_k * v_k in the reference's order, with the optional float contraction.
template <class A>
inline typename A::T tap_sum(const typename A::T* w, const typename A::T* v, int n, int fma_mode) {
  typedef typename A::T T;
  const int mode = A::can_fuse ? Fm::tap(fma_mode) : 0;
  if (mode) {
    T acc;
    if (mode == 1) acc = A::fma_(w[0], v[0], A::mul(w[1], v[1]));
    else acc = A::fma_(w[1], v[1], A::mul(w[0], v[0]));
    for (int k = 2; k < n; ++k) acc = A::fma_(w[k], v[k], acc);
    return acc;
  }
  T acc = A::mul(w[0], v[0]);
  for (int k = 1; k < n; ++k) acc = A::add(acc, A::mul(w[k], v[k]));
  return acc;
}

// weights and flat offsets of the 4 (2D) or 8 (3D) taps; returns false if the sample is
// outside the [-1, size] band (value 0, gradient skipped).
template <class A>
inline bool taps_2d(int H, int W, typename A::T y, typename A::T x, int order,
                    typename A::T* w, int64_t* off) {
  typedef typename A::T T;
  if (outside<A>(y, H) || outside<A>(x, W)) return false;
  AxisTap<A> ty, tx;
  axis_tap<A>(y, H, ty);
  axis_tap<A>(x, W, tx);
  off[0] = (int64_t)ty.i0 * W + tx.i0;
  off[1] = (int64_t)ty.i0 * W + tx.i1;
  off[2] = (int64_t)ty.i1 * W + tx.i0;
  off[3] = (int64_t)ty.i1 * W + tx.i1;
  if (order == 0) {
    const T half = (T)0.5;
    for (int k = 0; k < 4; ++k) w[k] = (T)0;
    if (ty.h >= half && tx.h >= half) w[0] = (T)1;
    else if (ty.h >= half && tx.l >= half) w[1] = (T)1;
    else if (ty.l >= half && tx.h >= half) w[2] = (T)1;
    else if (ty.l >= half && tx.l >= half) w[3] = (T)1;
  } else {
    w[0] = A::mul(ty.h, tx.h);
    w[1] = A::mul(ty.h, tx.l);
    w[2] = A::mul(ty.l, tx.h);
    w[3] = A::mul(ty.l, tx.l);
  }
  return true;
}

template <class A>
inline bool taps_3d(int D, int H, int W, typename A::T z, typename A::T y, typename A::T x, int order,
                    typename A::T* w, int64_t* off) {
  typedef typename A::T T;
  if (outside<A>(y, H) || outside<A>(x, W) || outside<A>(z, D)) return false;
  AxisTap<A> tz, ty, tx;
  axis_tap<A>(z, D, tz);
  axis_tap<A>(y, H, ty);
  axis_tap<A>(x, W, tx);
  const int64_t HW = (int64_t)H * W;
  off[0] = tz.i0 * HW + (int64_t)ty.i0 * W + tx.i0;
  off[1] = tz.i0 * HW + (int64_t)ty.i0 * W + tx.i1;
  off[2] = tz.i0 * HW + (int64_t)ty.i1 * W + tx.i0;
  off[3] = tz.i0 * HW + (int64_t)ty.i1 * W + tx.i1;
  off[4] = tz.i1 * HW + (int64_t)ty.i0 * W + tx.i0;
  off[5] = tz.i1 * HW + (int64_t)ty.i0 * W + tx.i1;
  off[6] = tz.i1 * HW + (int64_t)ty.i1 * W + tx.i0;
  off[7] = tz.i1 * HW + (int64_t)ty.i1 * W + tx.i1;
  if (order == 0) {
    const T half = (T)0.5;
    for (int k = 0; k < 8; ++k) w[k] = (T)0;
    if (tz.h >= half && ty.h >= half && tx.h >= half) w[0] = (T)1;
    else if (tz.h >= half && ty.h >= half && tx.l >= half) w[1] = (T)1;
    else if (tz.h >= half && ty.l >= half && tx.h >= half) w[2] = (T)1;
    else if (tz.h >= half && ty.l >= half && tx.l >= half) w[3] = (T)1;
    else if (tz.l >= half && ty.h >= half && tx.h >= half) w[4] = (T)1;
    else if (tz.l >= half && ty.h >= half && tx.l >= half) w[5] = (T)1;
    else if (tz.l >= half && ty.l >= half && tx.h >= half) w[6] = (T)1;
    else if (tz.l >= half && ty.l >= half && tx.l >= half) w[7] = (T)1;
  } else {
    const T hzhy = A::mul(tz.h, ty.h), hzly = A::mul(tz.h, ty.l);
    const T lzhy = A::mul(tz.l, ty.h), lzly = A::mul(tz.l, ty.l);
    w[0] = A::mul(hzhy, tx.h);
    w[1] = A::mul(hzhy, tx.l);
    w[2] = A::mul(hzly, tx.h);
    w[3] = A::mul(hzly, tx.l);
    w[4] = A::mul(lzhy, tx.h);
    w[5] = A::mul(lzhy, tx.l);
    w[6] = A::mul(lzly, tx.h);
    w[7] = A::mul(lzly, tx.l);
  }
  return true;
}

// ------------------------------------------------------------------ per-roi geometry
template <class A>
struct RoiGeom {
  typedef typename A::T T;
  int batch;
  // per axis, index 0 = w (x), 1 = h (y), 2 = d (z)
  T start[3];   // box: roi start in the volume; rotated: -size/2 in the roi frame
  T bin[3];
  int grid[3];
  T centre[3];  // rotated only
  T rot[9];     // rotated 3D: R11..R33 ; rotated 2D: rot[0]=cos, rot[1]=sin
  T count_fwd, count_bwd;
};

template <class A>
inline typename A::T mad_centre(typename A::T r, typename A::T s, typename A::T off, int fma_mode) {
  if (A::can_fuse && Fm::centre(fma_mode)) return A::fma_(r, s, A::neg(off));
  return A::sub(A::mul(r, s), off);
}

// a*b*c -/+ d*e of the rotation-matrix entries
template <class A>
inline typename A::T rot_entry(typename A::T a, typename A::T b, typename A::T c, typename A::T d,
                               typename A::T e, bool minus, int mode_) {
  typedef typename A::T T;
  const T ab = A::mul(a, b);
  const T de = A::mul(d, e);
  const int mode = A::can_fuse ? mode_ : 0;
  if (mode == 1) return A::fma_(ab, c, minus ? A::neg(de) : de);
  const T abc = A::mul(ab, c);
  if (mode == 2) return A::fma_(minus ? A::neg(d) : d, e, abc);
  return minus ? A::sub(abc, de) : A::add(abc, de);
}

template <class A>
void decode_roi(const void* rois, int64_t n, int ndim, int kind, const int* osz /*w,h,d*/,
                float spatial_scale_f, int sampling_ratio, int aligned, int fma_mode, const void* trig,
                RoiGeom<A>& g) {
  typedef typename A::T T;
  const int nax = ndim;
  const int width = (kind == KIND_BOX) ? (ndim == 2 ? 5 : 7) : (ndim == 2 ? 6 : 10);
  const T scale = A::ff(spatial_scale_f);
  T r[10];
  for (int k = 0; k < width; ++k) r[k] = A::ld(rois, n * width + k);
  g.batch = (int)r[0];
  T size[3];
  if (kind == KIND_BOX) {
    for (int a = 0; a < nax; ++a) {
      const T s = A::mul(r[1 + a], scale);
      const T e = A::mul(r[1 + nax + a], scale);
      T sz = (A::can_fuse && Fm::boxsize(fma_mode)) ? A::fma_(r[1 + nax + a], scale, A::neg(s)) : A::sub(e, s);
      if (!(sz >= (T)1)) sz = (T)1;  // max(sz, 1) as fmaxf: a NaN size becomes 1
      g.start[a] = s;
      size[a] = sz;
    }
  } else {
    const T off = aligned ? (T)0.5 : (T)0.0;
    for (int a = 0; a < nax; ++a) {
      g.centre[a] = mad_centre<A>(r[1 + a], scale, off, fma_mode);
      T sz = A::mul(r[1 + nax + a], scale);
      if (!aligned && !(sz >= (T)1)) sz = (T)1;
      size[a] = sz;
    }
    // `trig` (optional): per roi, cos and sin of each angle as evaluated elsewhere (the device's
    // sinf/cosf differ from the host's by an ulp for some arguments)
    if (ndim == 2) {
      const T th = r[5];
      g.rot[0] = trig ? A::ld(trig, n * 2 + 0) : A::cosT(th);
      g.rot[1] = trig ? A::ld(trig, n * 2 + 1) : A::sinT(th);
    } else {
      const T cg = trig ? A::ld(trig, n * 6 + 0) : A::cosT(r[7]), sg = trig ? A::ld(trig, n * 6 + 1) : A::sinT(r[7]);
      const T cb = trig ? A::ld(trig, n * 6 + 2) : A::cosT(r[8]), sb = trig ? A::ld(trig, n * 6 + 3) : A::sinT(r[8]);
      const T ca = trig ? A::ld(trig, n * 6 + 4) : A::cosT(r[9]), sa = trig ? A::ld(trig, n * 6 + 5) : A::sinT(r[9]);
      g.rot[0] = A::mul(ca, cb);
      g.rot[1] = rot_entry<A>(ca, sb, sg, sa, cg, true, Fm::entry(fma_mode, 0));
      g.rot[2] = rot_entry<A>(ca, sb, cg, sa, sg, false, Fm::entry(fma_mode, 1));
      g.rot[3] = A::mul(sa, cb);
      g.rot[4] = rot_entry<A>(sa, sb, sg, ca, cg, false, Fm::entry(fma_mode, 2));
      g.rot[5] = rot_entry<A>(sa, sb, cg, ca, sg, true, Fm::entry(fma_mode, 3));
      g.rot[6] = A::neg(sb);
      g.rot[7] = A::mul(cb, sg);
      g.rot[8] = A::mul(cb, cg);
    }
  }
  int prod = 1;
  for (int a = 0; a < nax; ++a) {
    const T o = A::fi(osz[a]);
    g.bin[a] = A::div(size[a], o);
    if (sampling_ratio > 0) {
      g.grid[a] = sampling_ratio;
    } else {
      const T q = A::div(size[a], o);
      const double cq = std::ceil((double)q);
      g.grid[a] = (cq == cq && std::fabs(cq) < 2e9) ? (int)cq : 0;
    }
    if (kind == KIND_ROTATED) g.start[a] = A::fd((double)A::neg(size[a]) / 2.0);
    prod *= g.grid[a];
  }
  for (int a = nax; a < 3; ++a) { g.grid[a] = 1; }
  g.count_fwd = A::fi(std::max(prod, 1));
  // 2D backward kernels divide by the plain product (no max); 3D ones use max(.,1)
  g.count_bwd = (ndim == 2) ? A::fi(prod) : A::fi(std::max(prod, 1));
}

// local sample coordinate along one axis:  (start + p*bin) + ((i+.5)*bin)/g
template <class A>
inline typename A::T lattice(typename A::T start, int p, typename A::T bin, int i, int g, int fma_mode) {
  typedef typename A::T T;
  const T t = A::div(A::mul(A::ff((float)i + .5f), bin), A::fi(g));
  T base;
  if (A::can_fuse && Fm::lattice(fma_mode)) base = A::fma_(A::fi(p), bin, start);
  else base = A::add(start, A::mul(A::fi(p), bin));
  return A::add(base, t);
}

// r = ((a1*x + a2*y) + a3*z) + c   with optional contraction
template <class A>
inline typename A::T rot_row3(typename A::T a1, typename A::T x, typename A::T a2, typename A::T y,
                              typename A::T a3, typename A::T z, typename A::T c, int mode_) {
  typedef typename A::T T;
  const int mode = A::can_fuse ? mode_ : 0;
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

// 2D: rx = (x*cos - y*sin) + cw ; ry = (x*sin + y*cos) + ch
template <class A>
inline typename A::T rot_row2(typename A::T x, typename A::T a, typename A::T y, typename A::T b, bool minus,
                              typename A::T c, int fma_mode) {
  typedef typename A::T T;
  const int mode = A::can_fuse ? Fm::rot2(fma_mode) : 0;
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

// ------------------------------------------------------------------ Catmull-Rom (affine_* order 3)
// medvision/csrc/cuda_aug/interpolation_helpers_{2d,3d}.h hermite_*_interpolate.  Filled in by
// hermite.inc-style code below (kept in this file).
template <class A>
typename A::T hermite_2d(const void* vol, int64_t base, int H, int W, typename A::T y, typename A::T x, int fma_mode);
template <class A>
typename A::T hermite_3d(const void* vol, int64_t base, int D, int H, int W, typename A::T z, typename A::T y,
                         typename A::T x, int fma_mode);

// ------------------------------------------------------------------ drivers
struct Args {
  const void* in;     // fwd: features ; bwd: grad_out
  const void* rois;
  void* out;          // fwd: output   ; bwd: grad_in (accumulated into)
  int ndim, kind;
  int64_t N, C, D, H, W, R;
  int od, oh, ow;
  float spatial_scale;
  int sampling_ratio, aligned, order;
  int fma_mode;
  int wide_acc;       // bwd only: accumulate in double and round once (not what the reference does)
  int nthreads;       // <= 0: all hardware threads
  const void* trig;   // optional (R, 2|6) table of cos/sin per roi angle, element type; may be null
};

template <class A>
int run_fwd(const Args& a) {
  typedef typename A::T T;
  const int osz[3] = {a.ow, a.oh, a.od};
  const int64_t vol = a.D * a.H * a.W;
  const int64_t ovol = (int64_t)a.od * a.oh * a.ow;
  std::atomic<int> err(0);
  // one work item = one (roi, channel, output z-slab)
  parallel_for(a.R * a.C * a.od, a.nthreads, [&](int64_t item) {
    const int64_t n = item / (a.C * a.od);
    const int64_t c = (item / a.od) % a.C;
    const int pd = (int)(item % a.od);
    {
      RoiGeom<A> g;
      decode_roi<A>(a.rois, n, a.ndim, a.kind, osz, a.spatial_scale, a.sampling_ratio, a.aligned, a.fma_mode, a.trig, g);
      if (g.batch < 0 || g.batch >= a.N) {
        err.store(1);
        for (int64_t i = 0; i < (int64_t)a.oh * a.ow; ++i)
          A::st(a.out, (n * a.C + c) * ovol + (int64_t)pd * a.oh * a.ow + i, (T)0);
        return;
      }
      const int64_t base = ((int64_t)g.batch * a.C + c) * vol;
      const int gd = (a.ndim == 3) ? g.grid[2] : 1;
        for (int ph = 0; ph < a.oh; ++ph)
          for (int pw = 0; pw < a.ow; ++pw) {
            T acc = (T)0;
            for (int iz = 0; iz < gd; ++iz) {
              const T z = (a.ndim == 3) ? lattice<A>(g.start[2], pd, g.bin[2], iz, g.grid[2], a.fma_mode) : (T)0;
              for (int iy = 0; iy < g.grid[1]; ++iy) {
                const T y = lattice<A>(g.start[1], ph, g.bin[1], iy, g.grid[1], a.fma_mode);
                for (int ix = 0; ix < g.grid[0]; ++ix) {
                  const T x = lattice<A>(g.start[0], pw, g.bin[0], ix, g.grid[0], a.fma_mode);
                  T sx = x, sy = y, sz = z;
                  if (a.kind == KIND_ROTATED) {
                    if (a.ndim == 2) {
                      sx = rot_row2<A>(x, g.rot[0], y, g.rot[1], true, g.centre[0], a.fma_mode);
                      sy = rot_row2<A>(x, g.rot[1], y, g.rot[0], false, g.centre[1], a.fma_mode);
                    } else {
                      sx = rot_row3<A>(g.rot[0], x, g.rot[1], y, g.rot[2], z, g.centre[0], Fm::row(a.fma_mode, 0));
                      sy = rot_row3<A>(g.rot[3], x, g.rot[4], y, g.rot[5], z, g.centre[1], Fm::row(a.fma_mode, 1));
                      sz = rot_row3<A>(g.rot[6], x, g.rot[7], y, g.rot[8], z, g.centre[2], Fm::row(a.fma_mode, 2));
                    }
                  }
                  T val = (T)0;
                  if (a.order == 3) {
                    val = (a.ndim == 2) ? hermite_2d<A>(a.in, base, (int)a.H, (int)a.W, sy, sx, a.fma_mode)
                                        : hermite_3d<A>(a.in, base, (int)a.D, (int)a.H, (int)a.W, sz, sy, sx, a.fma_mode);
                  } else {
                    T w[8], v[8];
                    int64_t off[8];
                    bool in;
                    int nt;
                    if (a.ndim == 2) { in = taps_2d<A>((int)a.H, (int)a.W, sy, sx, a.order, w, off); nt = 4; }
                    else { in = taps_3d<A>((int)a.D, (int)a.H, (int)a.W, sz, sy, sx, a.order, w, off); nt = 8; }
                    if (in) {
                      for (int k = 0; k < nt; ++k) v[k] = A::ld(a.in, base + off[k]);
                      val = tap_sum<A>(w, v, nt, a.fma_mode);
                    }
                  }
                  acc = A::add(acc, val);
                }
              }
            }
            acc = A::div(acc, g.count_fwd);
            A::st(a.out, (n * a.C + c) * ovol + ((int64_t)pd * a.oh + ph) * a.ow + pw, acc);
          }
    }
  });
  return err.load();
}

template <class A>
int run_bwd(const Args& a) {
  typedef typename A::T T;
  const int osz[3] = {a.ow, a.oh, a.od};
  const int64_t vol = a.D * a.H * a.W;
  const int64_t ovol = (int64_t)a.od * a.oh * a.ow;
  std::atomic<int> err(0);
  // The device scatters with atomics in no fixed order; here rois are visited in index order
  // for every channel, and channels run in parallel (they never share an address).
  parallel_for(a.C, a.nthreads, [&](int64_t c) {
    std::vector<double> wide;
    if (a.wide_acc) wide.assign((size_t)(a.N * vol), 0.0);
    for (int64_t n = 0; n < a.R; ++n) {
      RoiGeom<A> g;
      decode_roi<A>(a.rois, n, a.ndim, a.kind, osz, a.spatial_scale, a.sampling_ratio, a.aligned, a.fma_mode, a.trig, g);
      if (g.batch < 0 || g.batch >= a.N) {
        err.store(1);
        continue;
      }
      const int64_t base = ((int64_t)g.batch * a.C + c) * vol;
      const int gd = (a.ndim == 3) ? g.grid[2] : 1;
      for (int pd = 0; pd < a.od; ++pd)
        for (int ph = 0; ph < a.oh; ++ph)
          for (int pw = 0; pw < a.ow; ++pw) {
            const T go = A::ld(a.in, (n * a.C + c) * ovol + ((int64_t)pd * a.oh + ph) * a.ow + pw);
            for (int iz = 0; iz < gd; ++iz) {
              const T z = (a.ndim == 3) ? lattice<A>(g.start[2], pd, g.bin[2], iz, g.grid[2], a.fma_mode) : (T)0;
              for (int iy = 0; iy < g.grid[1]; ++iy) {
                const T y = lattice<A>(g.start[1], ph, g.bin[1], iy, g.grid[1], a.fma_mode);
                for (int ix = 0; ix < g.grid[0]; ++ix) {
                  const T x = lattice<A>(g.start[0], pw, g.bin[0], ix, g.grid[0], a.fma_mode);
                  T sx = x, sy = y, sz = z;
                  if (a.kind == KIND_ROTATED) {
                    if (a.ndim == 2) {
                      sx = rot_row2<A>(x, g.rot[0], y, g.rot[1], true, g.centre[0], a.fma_mode);
                      sy = rot_row2<A>(x, g.rot[1], y, g.rot[0], false, g.centre[1], a.fma_mode);
                    } else {
                      sx = rot_row3<A>(g.rot[0], x, g.rot[1], y, g.rot[2], z, g.centre[0], Fm::row(a.fma_mode, 0));
                      sy = rot_row3<A>(g.rot[3], x, g.rot[4], y, g.rot[5], z, g.centre[1], Fm::row(a.fma_mode, 1));
                      sz = rot_row3<A>(g.rot[6], x, g.rot[7], y, g.rot[8], z, g.centre[2], Fm::row(a.fma_mode, 2));
                    }
                  }
                  T w[8];
                  int64_t off[8];
                  bool in;
                  int nt;
                  if (a.ndim == 2) { in = taps_2d<A>((int)a.H, (int)a.W, sy, sx, a.order, w, off); nt = 4; }
                  else { in = taps_3d<A>((int)a.D, (int)a.H, (int)a.W, sz, sy, sx, a.order, w, off); nt = 8; }
                  if (!in) continue;
                  for (int k = 0; k < nt; ++k) {
                    const T gk = A::div(A::mul(go, w[k]), g.count_bwd);
                    if (a.wide_acc) {
                      wide[(size_t)((int64_t)g.batch * vol + off[k])] += (double)gk;
                    } else {
                      const int64_t idx = base + off[k];
                      A::st(a.out, idx, A::add(A::ld(a.out, idx), gk));
                    }
                  }
                }
              }
            }
          }
    }
    if (a.wide_acc) {
      for (int64_t b = 0; b < a.N; ++b)
        for (int64_t i = 0; i < vol; ++i) {
          const int64_t idx = (b * a.C + c) * vol + i;
          A::st(a.out, idx, A::fd((double)A::ld(a.out, idx) + wide[(size_t)(b * vol + i)]));
        }
    }
  });
  return err.load();
}

// ------------------------------------------------------------------ Catmull-Rom bodies
// medvision/csrc/cuda_aug/interpolation_helpers_2d.h:335-424, interpolation_helpers_3d.h:572-792.
// Per axis: i1 = (int)c after the c <= 0 clamp; u = c - i1 in the element type, held as float;
// u^2 and u^3 are float products (2D: kept as float; 3D: rounded to the element type); the
// reference then evaluates each of the 16 / 64 weights as an expanded polynomial in DOUBLE and
// rounds it to the element type.  Those polynomials factor exactly into the per-axis cubics
// below, so the weights are formed here as products of doubles: the same real numbers, equal in
// double up to ~1e-16 before the final rounding.
template <class A>
inline typename A::T from_double(double d) { return A::fd(d); }

template <class A, bool POWERS_IN_T>
inline void hermite_axis(typename A::T c, int size, int* idx, double* w) {
  typedef typename A::T T;
  if (c <= (T)0) c = (T)0;
  const int i1 = (c == c) ? (int)c : 0;
  const float u = (float)A::sub(c, A::fi(i1));
  double u2, u3;
  if (POWERS_IN_T) {
    u2 = (double)A::ff(u * u);
    u3 = (double)A::ff((u * u) * u);
  } else {
    u2 = (double)(float)(u * u);
    u3 = (double)(float)((float)(u * u) * u);
  }
  const double ud = (double)u;
  w[0] = -0.5 * u3 + u2 - 0.5 * ud;
  w[1] = 1.5 * u3 - 2.5 * u2 + 1.0;
  w[2] = -1.5 * u3 + 2.0 * u2 + 0.5 * ud;
  w[3] = 0.5 * u3 - 0.5 * u2;
  for (int k = 0; k < 4; ++k) idx[k] = std::min(std::max(i1 - 1 + k, 0), size - 1);
}

template <class A>
typename A::T hermite_2d(const void* vol, int64_t base, int H, int W, typename A::T y, typename A::T x, int fma_mode) {
  typedef typename A::T T;
  if (outside<A>(y, H) || outside<A>(x, W)) return (T)0;
  int ix[4], iy[4];
  double wx[4], wy[4];
  hermite_axis<A, false>(x, W, ix, wx);
  hermite_axis<A, false>(y, H, iy, wy);
  T w[16], v[16];
  for (int j = 0; j < 4; ++j)
    for (int i = 0; i < 4; ++i) {
      w[j * 4 + i] = from_double<A>(wx[i] * wy[j]);
      v[j * 4 + i] = A::ld(vol, base + (int64_t)iy[j] * W + ix[i]);
    }
  return tap_sum<A>(w, v, 16, fma_mode);  // one left-to-right sum, x fastest
}

template <class A>
typename A::T hermite_3d(const void* vol, int64_t base, int D, int H, int W, typename A::T z, typename A::T y,
                         typename A::T x, int fma_mode) {
  typedef typename A::T T;
  if (outside<A>(y, H) || outside<A>(x, W) || outside<A>(z, D)) return (T)0;
  int ix[4], iy[4], iz[4];
  double wx[4], wy[4], wz[4];
  hermite_axis<A, true>(x, W, ix, wx);
  hermite_axis<A, true>(y, H, iy, wy);
  hermite_axis<A, true>(z, D, iz, wz);
  T val = (T)0;  // val = 0; val += (four terms along x), for every (y, z), z outermost
  for (int k = 0; k < 4; ++k)
    for (int j = 0; j < 4; ++j) {
      T w[4], v[4];
      for (int i = 0; i < 4; ++i) {
        w[i] = from_double<A>(wx[i] * wy[j] * wz[k]);
        v[i] = A::ld(vol, base + ((int64_t)iz[k] * H + iy[j]) * W + ix[i]);
      }
      val = A::add(val, tap_sum<A>(w, v, 4, fma_mode));
    }
  return val;
}

// ------------------------------------------------------------------ displacement-field warp
// medvision/ops/cuda_fun_tools.py:94-167 apply_offset_2d/3d -> deform_2d/deform_3d with a 1x1(x1)
// kernel, stride 1, no padding, one deformable group, identity weight and zero bias.  The
// deformable im2col (medvision/csrc/cuda_aug/deform_3d_cuda_kernel.cuh:44-90, the 2D file alike)
// writes, for voxel p of channel c, interp(img[b, c], (T)p + offset[b, :, p]) when every
// coordinate lies strictly inside (-1, size) and 0 otherwise; offset channels are (d, h, w) /
// (h, w).  The addmm with the identity weight and the zero bias (deform_3d_cuda.cu:118-146)
// returns a finite column value unchanged, so it is not restated.
struct OffsetArgs {
  const void* img;
  const void* off;
  void* out;
  int ndim;
  int64_t B, C, D, H, W;
  int order, fma_mode, nthreads;
};

template <class A>
int run_offset(const OffsetArgs& a) {
  typedef typename A::T T;
  const int64_t vol = a.D * a.H * a.W;
  parallel_for(a.B * a.D * a.H, a.nthreads, [&](int64_t row) {
    const int64_t b = row / (a.D * a.H);
    const int d = (int)((row / a.H) % a.D), h = (int)(row % a.H);
    for (int w = 0; w < (int)a.W; ++w) {
      const int64_t s = ((int64_t)d * a.H + h) * a.W + w;
      const int64_t ob = b * a.ndim * vol + s;
      T z = (T)0, y, x;
      if (a.ndim == 3) {
        z = A::add(A::fi(d), A::ld(a.off, ob));
        y = A::add(A::fi(h), A::ld(a.off, ob + vol));
        x = A::add(A::fi(w), A::ld(a.off, ob + 2 * vol));
      } else {
        y = A::add(A::fi(h), A::ld(a.off, ob));
        x = A::add(A::fi(w), A::ld(a.off, ob + vol));
      }
      const bool in = (double)y > -1.0 && (double)x > -1.0 && (double)y < (double)a.H && (double)x < (double)a.W &&
                      (a.ndim == 2 || ((double)z > -1.0 && (double)z < (double)a.D));
      T wt[8];
      int64_t off[8];
      const int n = a.ndim == 3 ? 8 : 4;
      if (in && a.order != 3) {
        if (a.ndim == 3) taps_3d<A>((int)a.D, (int)a.H, (int)a.W, z, y, x, a.order, wt, off);
        else taps_2d<A>((int)a.H, (int)a.W, y, x, a.order, wt, off);
      }
      for (int64_t c = 0; c < a.C; ++c) {
        const int64_t base = (b * a.C + c) * vol;
        T val = (T)0;
        if (in) {
          if (a.order == 3) {
            val = a.ndim == 3 ? hermite_3d<A>(a.img, base, (int)a.D, (int)a.H, (int)a.W, z, y, x, a.fma_mode)
                              : hermite_2d<A>(a.img, base, (int)a.H, (int)a.W, y, x, a.fma_mode);
          } else {
            T v[8];
            for (int k = 0; k < n; ++k) v[k] = A::ld(a.img, base + off[k]);
            val = tap_sum<A>(wt, v, n, a.fma_mode);
          }
        }
        A::st(a.out, base + s, val);
      }
    }
  });
  return 0;
}

int check(const Args& a, int dtype, bool fwd) {
  if (dtype != DT_F32 && dtype != DT_F16 && dtype != DT_F64) return -1;
  if (a.ndim != 2 && a.ndim != 3) return -2;
  if (a.kind != KIND_BOX && a.kind != KIND_ROTATED) return -3;
  if (a.order != 0 && a.order != 1 && !(fwd && a.order == 3 && a.kind == KIND_ROTATED)) return -4;
  if (a.ndim == 2 && (a.D != 1 || a.od != 1)) return -5;
  if (a.N < 0 || a.C < 0 || a.D < 1 || a.H < 1 || a.W < 1 || a.R < 0 || a.od < 1 || a.oh < 1 || a.ow < 1) return -6;
  return 0;
}

}  // namespace

extern "C" {

// All sizes are element counts; buffers are host memory, contiguous NC(D)HW / (R, roi_width).
// Returns 0, 1 when some roi's batch index was outside [0, N) (its outputs are zero /
// its gradient is skipped), or a negative argument error.
int mvr_oracle_fwd(const void* features, const void* rois, void* output, int dtype, int ndim, int roi_kind,
                   int64_t N, int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int od, int oh, int ow,
                   float spatial_scale, int sampling_ratio, int aligned, int order, int fma_mode, int nthreads,
                   const void* trig) {
  Args a = {features, rois, output, ndim, roi_kind, N, C, D, H, W, R, od, oh, ow,
            spatial_scale, sampling_ratio, aligned, order, fma_mode, 0, nthreads, trig};
  int e = check(a, dtype, true);
  if (e) return e;
  switch (dtype) {
    case DT_F32: return run_fwd<Arith<DT_F32> >(a);
    case DT_F16: return run_fwd<Arith<DT_F16> >(a);
    default: return run_fwd<Arith<DT_F64> >(a);
  }
}

// grad_in must be zero-filled by the caller (the reference's Python does that); it is
// accumulated into, in the element type, exactly as the reference's atomicAdd does
// (wide_acc = 0), or through a double accumulator rounded once at the end (wide_acc = 1).
int mvr_oracle_bwd(const void* grad_out, const void* rois, void* grad_in, int dtype, int ndim, int roi_kind,
                   int64_t N, int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int od, int oh, int ow,
                   float spatial_scale, int sampling_ratio, int aligned, int order, int fma_mode, int wide_acc,
                   int nthreads, const void* trig) {
  Args a = {grad_out, rois, grad_in, ndim, roi_kind, N, C, D, H, W, R, od, oh, ow,
            spatial_scale, sampling_ratio, aligned, order, fma_mode, wide_acc, nthreads, trig};
  int e = check(a, dtype, false);
  if (e) return e;
  switch (dtype) {
    case DT_F32: return run_bwd<Arith<DT_F32> >(a);
    case DT_F16: return run_bwd<Arith<DT_F16> >(a);
    default: return run_bwd<Arith<DT_F64> >(a);
  }
}

// img / out (B, C, [D,] H, W), offset (B, ndim, [D,] H, W); D = 1 for ndim 2.
int mvr_oracle_offset(const void* img, const void* offset, void* out, int dtype, int ndim, int64_t B, int64_t C,
                      int64_t D, int64_t H, int64_t W, int order, int fma_mode, int nthreads) {
  if (dtype != DT_F32 && dtype != DT_F16 && dtype != DT_F64) return -1;
  if (ndim != 2 && ndim != 3) return -2;
  if (order != 0 && order != 1 && order != 3) return -4;
  if ((ndim == 2 && D != 1) || B < 0 || C < 0 || D < 1 || H < 1 || W < 1) return -6;
  OffsetArgs a = {img, offset, out, ndim, B, C, D, H, W, order, fma_mode, nthreads};
  switch (dtype) {
    case DT_F32: return run_offset<Arith<DT_F32> >(a);
    case DT_F16: return run_offset<Arith<DT_F16> >(a);
    default: return run_offset<Arith<DT_F64> >(a);
  }
}

int mvr_oracle_max_threads(void) { return (int)std::max(1u, std::thread::hardware_concurrency()); }

}  // extern "C"
