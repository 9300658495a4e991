// Streaming forward kernel for dense 3D resampling: one sample per output voxel
// (sampling_ratio == 1), half or float, rotated rois (RoIAlignRotated 3D / affine_3d) and
// axis-aligned boxes (RoIAlign 3D).  This is the shape of every batched augmentation call
// (Resize, RandomAffine/Scale/Shift/Rotate, CropRandomWithAffine:
// medvision/aug_cuda_batch/aug_spatial.py:118-155,404-446,674-715), where the output has
// millions of voxels per roi and the work is a stream over the volume.
//
// Layout of the work
//   * CTA = 256 threads = a 32 (w) x 16 (h) tile of output positions x a chunk of output depth
//     of ONE (roi, channel).  A thread owns two w-adjacent voxels and walks the depth chunk,
//     so output stores are 2-element vectors, contiguous along w within a warp row.
//   * The roi is decoded (incl. its six sin/cos) once per CTA; per-depth quantities are
//     tabulated once per CTA in shared memory.
//   * Every arithmetic step keeps the reference's rounding sequence (mvr_arith.cuh); what is
//     removed is only work whose result is provably identical:
//       - z-separable rois (no rotation, or rotation about z only -- the only rotation the
//         augmentations use): R13 = R23 = R31 = R32 = 0 and R33 = 1 exactly, so the in-plane
//         sample position, its four in-plane tap offsets and weights depend on (h, w) only and
//         are computed once per thread; the z tap (planes, weights) depends on depth only and
//         is tabulated per CTA.  Adding a*0 or multiplying by 1 never changes a finite value.
//       - consecutive output depths usually share a source plane (z1 of one = z0 of the next):
//         its four tap values stay in registers instead of being reloaded.
//       - general rotations: the products R_i2*y, R_i1*x (per thread) and R_i3*z (per depth)
//         are formed once; they are separately rounded values in the reference as well
//         (half: every product is rounded; float: see the contraction pattern).
//   * Half math runs on both lanes of half2 instructions (the two voxels of a thread).
//
// Gathers go through L1/L2 (__ldg): neighbouring threads and consecutive depths hit the same
// lines, and the per-thread register reuse above removes about half of the loads outright.
#pragma once
#include "mvr_generic.cuh"

namespace mvr {

constexpr int MVR_STREAM3D_NOT_APPLICABLE = 1;

constexpr int kS3Threads = 256;
constexpr int kS3TileW = 32;   // output voxels along w per CTA (2 per thread)
constexpr int kS3TileH = 16;
constexpr int kS3MaxChunk = 128;  // output depths per CTA

// The float contraction pattern this kernel hard-codes (the reference build's).
constexpr int kS3FloatPattern = kReferenceContraction;

// ---- two-lane arithmetic: lane a = voxel at w, lane b = voxel at w+1 -----------------------
template <typename T> struct P2;

template <> struct P2<__half> {
  typedef __half2 V;
  __device__ __forceinline__ static V make(__half a, __half b) { return __halves2half2(a, b); }
  __device__ __forceinline__ static V dup(__half a) { return __half2half2(a); }
  __device__ __forceinline__ static V add(V a, V b) { return __hadd2_rn(a, b); }
  __device__ __forceinline__ static V mul(V a, V b) { return __hmul2_rn(a, b); }
  // a1*x + py : both roundings kept
  __device__ __forceinline__ static V row_xy(V a1, V x, V py) { return __hadd2_rn(__hmul2_rn(a1, x), py); }
  __device__ __forceinline__ static V tap_first(V w0, V v0, V w1, V v1) {
    return __hadd2_rn(__hmul2_rn(w0, v0), __hmul2_rn(w1, v1));
  }
  __device__ __forceinline__ static V tap_next(V acc, V w, V v) { return __hadd2_rn(acc, __hmul2_rn(w, v)); }
  __device__ __forceinline__ static __half lo(V v) { return __low2half(v); }
  __device__ __forceinline__ static __half hi(V v) { return __high2half(v); }
  __device__ __forceinline__ static V select(V v, bool keep_a, bool keep_b) {
    unsigned u = *reinterpret_cast<unsigned*>(&v);
    u &= (keep_a ? 0x0000ffffu : 0u) | (keep_b ? 0xffff0000u : 0u);
    return *reinterpret_cast<V*>(&u);
  }
  __device__ __forceinline__ static void store2(__half* p, V v) { *reinterpret_cast<__half2*>(p) = v; }
  typedef unsigned M;  // lane mask, built once per thread
  __device__ __forceinline__ static M make_mask(bool keep_a, bool keep_b) {
    return (keep_a ? 0x0000ffffu : 0u) | (keep_b ? 0xffff0000u : 0u);
  }
  __device__ __forceinline__ static V apply(V v, M m) {
    unsigned u = *reinterpret_cast<unsigned*>(&v) & m;
    return *reinterpret_cast<V*>(&u);
  }
};

struct Float2Lanes { float a, b; };
template <> struct P2<float> {
  typedef Float2Lanes V;
  __device__ __forceinline__ static V make(float a, float b) { V v; v.a = a; v.b = b; return v; }
  __device__ __forceinline__ static V dup(float a) { return make(a, a); }
  __device__ __forceinline__ static V add(V a, V b) { return make(__fadd_rn(a.a, b.a), __fadd_rn(a.b, b.b)); }
  __device__ __forceinline__ static V mul(V a, V b) { return make(__fmul_rn(a.a, b.a), __fmul_rn(a.b, b.b)); }
  // fma(a1, x, py): the x product is the fused one in the reference build
  __device__ __forceinline__ static V row_xy(V a1, V x, V py) {
    return make(__fmaf_rn(a1.a, x.a, py.a), __fmaf_rn(a1.b, x.b, py.b));
  }
  __device__ __forceinline__ static V tap_first(V w0, V v0, V w1, V v1) {
    return make(__fmaf_rn(w0.a, v0.a, __fmul_rn(w1.a, v1.a)), __fmaf_rn(w0.b, v0.b, __fmul_rn(w1.b, v1.b)));
  }
  __device__ __forceinline__ static V tap_next(V acc, V w, V v) {
    return make(__fmaf_rn(w.a, v.a, acc.a), __fmaf_rn(w.b, v.b, acc.b));
  }
  __device__ __forceinline__ static float lo(V v) { return v.a; }
  __device__ __forceinline__ static float hi(V v) { return v.b; }
  __device__ __forceinline__ static V select(V v, bool keep_a, bool keep_b) {
    return make(keep_a ? v.a : 0.0f, keep_b ? v.b : 0.0f);
  }
  __device__ __forceinline__ static void store2(float* p, V v) { *reinterpret_cast<float2*>(p) = make_float2(v.a, v.b); }
  typedef unsigned M;
  __device__ __forceinline__ static M make_mask(bool keep_a, bool keep_b) { return (keep_a ? 1u : 0u) | (keep_b ? 2u : 0u); }
  __device__ __forceinline__ static V apply(V v, M m) { return make((m & 1u) ? v.a : 0.0f, (m & 2u) ? v.b : 0.0f); }
};

// per-axis (l, h) of one sample; order 0 replaces them by the one-hot choice that the
// reference's first-match rule makes on this axis (prefer the low index when h >= .5)
template <typename T>
__device__ __forceinline__ void nearest_axis(T& l, T& h) {
  typedef Ar<T> A;
  const bool hh = A::ge_half(h), ll = A::ge_half(l);
  h = hh ? A::fi(1) : A::fi(0);
  l = (!hh && ll) ? A::fi(1) : A::fi(0);
}

// One interpolation axis for the two voxels of a pair at once (same results as axis_tap /
// axis_outside / nearest_axis applied to each lane; `size` must be at most 2048 for half so that
// it is a half value).
template <typename T>
struct AxisTap2 {
  int i0a, i0b;        // lower tap index per lane
  int da, db;          // 1 when the upper tap is i0 + 1, 0 when it is clamped onto i0
  typename P2<T>::V l, h;
  bool outa, outb;     // coordinate outside [-1, size]: the sample contributes nothing
};

template <typename T>
__device__ __forceinline__ void axis_tap2(typename P2<T>::V c, int size, int order, AxisTap2<T>& t);

template <>
__device__ __forceinline__ void axis_tap2<__half>(__half2 c, int size, int order, AxisTap2<__half>& t) {
  const __half2 zero = __float2half2_rn(0.0f), one = __float2half2_rn(1.0f);
  const unsigned out = __hlt2_mask(c, __float2half2_rn(-1.0f)) | __hgt2_mask(c, __float2half2_rn((float)size));
  t.outa = (out & 0xffffu) != 0;
  t.outb = (out >> 16) != 0;
  // `if (c <= 0) c = 0`: a NaN stays a NaN
  c = __hmax2_nan(c, zero);
  int ia = __half2int_rz(__low2half(c)), ib = __half2int_rz(__high2half(c));
  const bool ca = ia >= size - 1, cb = ib >= size - 1;  // upper neighbour clamped onto the last index
  ia = ca ? size - 1 : ia;
  ib = cb ? size - 1 : ib;
  t.i0a = ia; t.i0b = ib;
  t.da = ca ? 0 : 1; t.db = cb ? 0 : 1;
  // l = c - (T)i0: i0 = floor(c) for c >= 0; a clamped lane has c := (T)i0, hence l = +0
  __half2 l = __hsub2_rn(c, h2floor(c));
  const unsigned keep = (ca ? 0u : 0x0000ffffu) | (cb ? 0u : 0xffff0000u);
  unsigned lu = *reinterpret_cast<unsigned*>(&l) & keep;
  l = *reinterpret_cast<__half2*>(&lu);
  __half2 h = __hsub2_rn(one, l);
  if (order == 0) {  // one-hot choice per axis: prefer the lower index when h >= .5
    const __half2 half_ = __float2half2_rn(0.5f);
    const unsigned hh = __hge2_mask(h, half_);
    const unsigned ll = __hge2_mask(l, half_) & ~hh;
    unsigned ou = *reinterpret_cast<const unsigned*>(&one);
    unsigned hu = ou & hh, l2 = ou & ll;
    h = *reinterpret_cast<__half2*>(&hu);
    l = *reinterpret_cast<__half2*>(&l2);
  }
  t.l = l;
  t.h = h;
}

template <>
__device__ __forceinline__ void axis_tap2<float>(Float2Lanes c, int size, int order, AxisTap2<float>& t) {
  AxisTap<float> a, b;
  t.outa = axis_outside<float>(c.a, size);
  t.outb = axis_outside<float>(c.b, size);
  axis_tap<float>(c.a, size, a);
  axis_tap<float>(c.b, size, b);
  if (order == 0) { nearest_axis<float>(a.l, a.h); nearest_axis<float>(b.l, b.h); }
  t.i0a = a.i0; t.i0b = b.i0;
  t.da = a.i1 - a.i0; t.db = b.i1 - b.i0;
  t.l = P2<float>::make(a.l, b.l);
  t.h = P2<float>::make(a.h, b.h);
}

template <typename T>
struct S3ZTap {        // z-separable: per output depth
  long long o0, o1;    // element offsets of the two source planes inside the volume
  T l, h;
  int inside;
  int z0, z1;          // the two source planes' indices
};
template <typename T>
struct S3ZProd {       // general rotation: per output depth, the rounded products R_i3 * z
  T p[3];
};

template <typename T>
struct S3Shared {
  RoiGeom<T> g;
  int zsep;            // 1: z-separable path
  union {
    S3ZTap<T> zt[kS3MaxChunk];
    S3ZProd<T> zp[kS3MaxChunk];
  };
};

struct S3Launch {
  int tiles_w, tiles_h, chunks, chunk;  // chunk = output depths per CTA
  int vec_store;                        // 1: two-element vector stores are aligned
  int filter;                           // 0: every roi; 1: only rois that turn about z at most; 2: only the others
  // plane-streaming kernel only: limits of its bounded waits, and the self-test's left-out plane (-1: none)
  int skip_plane = -1;
  unsigned wait_tries = 1u << 20;       // tries of a bounded wait on a ring slot's barrier (each may be suspended by the hardware)
};

// General-rotation depth loop for NP voxel pairs of one thread (pair q sits q*row_step output
// rows below pair 0): positions change with depth, so all three axis taps are formed per voxel;
// the x- and y-products of the rotation are formed once per thread, the z-products once per
// depth and CTA (S3ZProd table).  Both lanes of a pair go through the same instructions.
template <typename T, int NP>
__device__ __forceinline__ void s3_full_depth_loop(const Params& p, const S3Shared<T>& sh, int npd, int c,
                                                   int pw0, int ph0, int row_step, bool vec_store, T* out0) {
  typedef Ar<T> A;
  typedef P2<T> Q;
  typedef typename Q::V V;
  const RoiGeom<T>& g = sh.g;
  const int fm = kS3FloatPattern;
  const bool has_b = (pw0 + 1 < p.ow);
  const T* vol = (const T*)p.in + ((long long)g.batch * p.C + c) * p.vol;
  const V zero2 = Q::dup(A::fi(0));
  const T sub_x = lattice_sub<T>(g.bin[0], 0, 1), sub_y = lattice_sub<T>(g.bin[1], 0, 1);
  const T xa = A::add(lattice_base<T>(g.start[0], pw0, g.bin[0], fm), sub_x);
  const T xb = A::add(lattice_base<T>(g.start[0], has_b ? pw0 + 1 : pw0, g.bin[0], fm), sub_x);
  const V x2 = Q::make(xa, xb);
  V sxy[NP][3];
  bool act[NP];
#pragma unroll
  for (int q = 0; q < NP; ++q) {
    const int ph = ph0 + q * row_step;
    act[q] = ph < p.oh;
    const T y = A::add(lattice_base<T>(g.start[1], act[q] ? ph : 0, g.bin[1], fm), sub_y);
#pragma unroll
    for (int r = 0; r < 3; ++r)
      sxy[q][r] = Q::row_xy(Q::dup(g.rot[3 * r]), x2, Q::dup(A::mul(g.rot[3 * r + 1], y)));
  }
  const V c2[3] = {Q::dup(g.centre[0]), Q::dup(g.centre[1]), Q::dup(g.centre[2])};
  const int W = p.W, HW = p.H * p.W;
  const long long plane_o = (long long)p.oh * p.ow;
  const long long sub_o = (long long)row_step * p.ow;
  T* o = out0;
  for (int i = 0; i < npd; ++i, o += plane_o) {
    const S3ZProd<T> e = sh.zp[i];
#pragma unroll
    for (int q = 0; q < NP; ++q) {
      if (!act[q]) continue;
      const V rx2 = Q::add(Q::add(sxy[q][0], Q::dup(e.p[0])), c2[0]);
      const V ry2 = Q::add(Q::add(sxy[q][1], Q::dup(e.p[1])), c2[1]);
      const V rz2 = Q::add(Q::add(sxy[q][2], Q::dup(e.p[2])), c2[2]);
      AxisTap2<T> tx, ty, tz;
      axis_tap2<T>(rx2, p.W, p.order, tx);
      axis_tap2<T>(ry2, p.H, p.order, ty);
      axis_tap2<T>(rz2, p.D, p.order, tz);
      const bool ina = !(tx.outa || ty.outa || tz.outa);
      const bool inb = has_b && !(tx.outb || ty.outb || tz.outb);
      // element offsets of the eight taps inside the volume, per lane
      const int ba = (tz.i0a * p.H + ty.i0a) * W + tx.i0a;
      const int bb = (tz.i0b * p.H + ty.i0b) * W + tx.i0b;
      const int dya = ty.da ? W : 0, dyb = ty.db ? W : 0, dza = tz.da ? HW : 0, dzb = tz.db ? HW : 0;
      const T* pa = vol + (ina ? ba : 0);
      const T* pb = vol + (inb ? bb : 0);
      const int xa1 = ina ? tx.da : 0, xb1 = inb ? tx.db : 0;
      const int ya1 = ina ? dya : 0, yb1 = inb ? dyb : 0, za1 = ina ? dza : 0, zb1 = inb ? dzb : 0;
      V v[8];
      v[0] = Q::make(__ldg(pa), __ldg(pb));
      v[1] = Q::make(__ldg(pa + xa1), __ldg(pb + xb1));
      v[2] = Q::make(__ldg(pa + ya1), __ldg(pb + yb1));
      v[3] = Q::make(__ldg(pa + ya1 + xa1), __ldg(pb + yb1 + xb1));
      v[4] = Q::make(__ldg(pa + za1), __ldg(pb + zb1));
      v[5] = Q::make(__ldg(pa + za1 + xa1), __ldg(pb + zb1 + xb1));
      v[6] = Q::make(__ldg(pa + za1 + ya1), __ldg(pb + zb1 + yb1));
      v[7] = Q::make(__ldg(pa + za1 + ya1 + xa1), __ldg(pb + zb1 + yb1 + xb1));
      const V hzhy = Q::mul(tz.h, ty.h), hzly = Q::mul(tz.h, ty.l);
      const V lzhy = Q::mul(tz.l, ty.h), lzly = Q::mul(tz.l, ty.l);
      V acc = Q::tap_first(Q::mul(hzhy, tx.h), v[0], Q::mul(hzhy, tx.l), v[1]);
      acc = Q::tap_next(acc, Q::mul(hzly, tx.h), v[2]);
      acc = Q::tap_next(acc, Q::mul(hzly, tx.l), v[3]);
      acc = Q::tap_next(acc, Q::mul(lzhy, tx.h), v[4]);
      acc = Q::tap_next(acc, Q::mul(lzhy, tx.l), v[5]);
      acc = Q::tap_next(acc, Q::mul(lzly, tx.h), v[6]);
      acc = Q::tap_next(acc, Q::mul(lzly, tx.l), v[7]);
      const V val = Q::apply(Q::add(zero2, acc), Q::make_mask(ina, inb));
      T* oq = o + q * sub_o;
      if (vec_store && has_b) {
        Q::store2(oq, val);
      } else {
        oq[0] = Q::lo(val);
        if (has_b) oq[1] = Q::hi(val);
      }
    }
  }
}

// CTA coordinates of the streaming kernels: tile_w fastest, then tile_h, depth chunk, (roi, channel)
struct S3Cta {
  int tw, th, ck, c, pd0, npd;
  long long nc, n;
};
__device__ __forceinline__ S3Cta s3_cta(const Params& p, const S3Launch& L, long long cta) {
  S3Cta k;
  k.tw = (int)(cta % L.tiles_w); cta /= L.tiles_w;
  k.th = (int)(cta % L.tiles_h); cta /= L.tiles_h;
  k.ck = (int)(cta % L.chunks);  cta /= L.chunks;
  k.nc = cta;
  k.n = k.nc / p.C;
  k.c = (int)(k.nc % p.C);
  k.pd0 = k.ck * L.chunk;
  k.npd = min(L.chunk, p.od - k.pd0);
  return k;
}
__device__ __forceinline__ S3Cta s3_cta(const Params& p, const S3Launch& L) { return s3_cta(p, L, blockIdx.x); }

// The forward runs as two launches when the rois may be rotated: rois that turn about z at most
// stream whole source planes through shared memory and want few, long CTAs (their set-up costs
// as much as five depths); rois under a general rotation gather through L1, are bound by load
// latency and want many short work items.  The test reads the two angles themselves (exact
// zeros give sin = 0 and cos = 1 exactly), so it needs no decoding and both launches agree.
template <typename T>
__device__ __forceinline__ bool s3_roi_is_planar(const Params& p, long long n) {
  if (p.kind != KIND_ROTATED) return true;
  const T* r = (const T*)p.rois + n * 10;
  return (Ar<T>::tof(__ldg(r + 7)) == 0.0f) && (Ar<T>::tof(__ldg(r + 8)) == 0.0f);
}
template <typename T>
__device__ __forceinline__ bool s3_filtered_out(const Params& p, const S3Launch& L, const S3Cta& k) {
  if (L.filter == 0) return false;
  return s3_roi_is_planar<T>(p, k.n) != (L.filter == 1);
}

// Decode the roi, classify it, and fill the per-depth table.  Ends with a __syncthreads().
template <typename T>
__device__ __forceinline__ void s3_prologue(const Params& p, const S3Cta& k, S3Shared<T>& sh) {
  typedef Ar<T> A;
  const long long n = k.n;
  const int pd0 = k.pd0, npd = k.npd;
  const int fm = kS3FloatPattern;
  if (threadIdx.x == 0) {
    const int osz[3] = {p.ow, p.oh, p.od};
    decode_roi<T>((const T*)p.rois, n, 3, p.kind, osz, p.spatial_scale, 1, p.aligned, fm, sh.g);
    const RoiGeom<T>& g = sh.g;
    int zsep = 1;
    if (p.kind == KIND_ROTATED) {
      const float one = 1.0f;
      zsep = (A::tof(g.rot[2]) == 0.0f) && (A::tof(g.rot[5]) == 0.0f) && (A::tof(g.rot[6]) == 0.0f) &&
             (A::tof(g.rot[7]) == 0.0f) && (A::tof(g.rot[8]) == one);
    }
    // the shortcut drops terms of the form 0*coordinate: every lattice coordinate must be finite
    const int last[3] = {p.ow - 1, p.oh - 1, p.od - 1};
    for (int a = 0; a < 3; ++a) {
      const T sub = lattice_sub<T>(g.bin[a], 0, 1);
      const T c0 = A::add(lattice_base<T>(g.start[a], 0, g.bin[a], fm), sub);
      const T c1 = A::add(lattice_base<T>(g.start[a], last[a], g.bin[a], fm), sub);
      zsep = zsep && A::finite(c0) && A::finite(c1) && A::finite(g.centre[a]);
    }
    sh.zsep = zsep;
  }
  __syncthreads();
  const RoiGeom<T>& g = sh.g;
  const bool zsep = sh.zsep != 0;
  const bool rotated = (p.kind == KIND_ROTATED);
  const bool bad_batch = (g.batch < 0 || g.batch >= p.N);
  const long long HW = (long long)p.H * p.W;

  // ---- per-depth table
  if (!bad_batch && (int)threadIdx.x < npd) {
    const int i = threadIdx.x;
    const T z = A::add(lattice_base<T>(g.start[2], pd0 + i, g.bin[2], fm), lattice_sub<T>(g.bin[2], 0, 1));
    if (zsep) {
      const T rz = rotated ? A::add(z, g.centre[2]) : z;
      S3ZTap<T> e;
      e.inside = !axis_outside<T>(rz, p.D);
      AxisTap<T> t;
      axis_tap<T>(rz, p.D, t);
      if (p.order == 0) nearest_axis<T>(t.l, t.h);
      e.o0 = t.i0 * HW;
      e.o1 = t.i1 * HW;
      e.z0 = t.i0;
      e.z1 = t.i1;
      e.l = t.l;
      e.h = t.h;
      sh.zt[i] = e;
    } else {
      S3ZProd<T> e;
      e.p[0] = A::mul(g.rot[2], z);
      e.p[1] = A::mul(g.rot[5], z);
      e.p[2] = A::mul(g.rot[8], z);
      sh.zp[i] = e;
    }
  }
  __syncthreads();

}

// Everything after the prologue, gathering through L1/L2 with plain loads.
template <typename T>
__device__ void s3_body_l1(const Params& p, const S3Launch& L, const S3Cta& k, S3Shared<T>& sh) {
  typedef Ar<T> A;
  typedef P2<T> Q;
  typedef typename Q::V V;
  const int tw = k.tw, th = k.th, ck = k.ck, c = k.c, pd0 = k.pd0, npd = k.npd;
  const long long nc = k.nc;
  const int fm = kS3FloatPattern;
  const RoiGeom<T>& g = sh.g;
  const bool zsep = sh.zsep != 0;
  const bool rotated = (p.kind == KIND_ROTATED);
  const bool bad_batch = (g.batch < 0 || g.batch >= p.N);
  // ---- this thread's two output columns
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pw0 = tw * kS3TileW + (warp & 1) * 16 + (lane & 7) * 2;
  const int ph = th * kS3TileH + (warp >> 1) * 4 + (lane >> 3);
  if (ph >= p.oh || pw0 >= p.ow) return;
  const bool has_b = (pw0 + 1 < p.ow);
  const long long plane_o = (long long)p.oh * p.ow;
  T* out = (T*)p.out + nc * p.ovol + (long long)pd0 * plane_o + (long long)ph * p.ow + pw0;
  const bool vec = L.vec_store && has_b;

  if (bad_batch) {
    if (p.status && threadIdx.x == 0 && tw == 0 && th == 0 && ck == 0) atomicOr(p.status, STATUS_BAD_BATCH_INDEX);
    for (int i = 0; i < npd; ++i) {
      out[i * plane_o] = A::fi(0);
      if (has_b) out[i * plane_o + 1] = A::fi(0);
    }
    return;
  }
  const T* vol = (const T*)p.in + ((long long)g.batch * p.C + c) * p.vol;
  const V zero2 = Q::dup(A::fi(0));

  // lattice coordinates of the two voxels in the roi frame
  const T sub_x = lattice_sub<T>(g.bin[0], 0, 1), sub_y = lattice_sub<T>(g.bin[1], 0, 1);
  const T xa = A::add(lattice_base<T>(g.start[0], pw0, g.bin[0], fm), sub_x);
  const T xb = A::add(lattice_base<T>(g.start[0], has_b ? pw0 + 1 : pw0, g.bin[0], fm), sub_x);
  const T y = A::add(lattice_base<T>(g.start[1], ph, g.bin[1], fm), sub_y);
  const V x2 = Q::make(xa, xb);

  if (zsep) {
    // ---- in-plane position, taps and weights: once per thread
    V rx2, ry2;
    if (rotated) {
      rx2 = Q::add(Q::row_xy(Q::dup(g.rot[0]), x2, Q::dup(A::mul(g.rot[1], y))), Q::dup(g.centre[0]));
      ry2 = Q::add(Q::row_xy(Q::dup(g.rot[3]), x2, Q::dup(A::mul(g.rot[4], y))), Q::dup(g.centre[1]));
    } else {
      rx2 = x2;
      ry2 = Q::dup(y);
    }
    const T rx[2] = {Q::lo(rx2), Q::hi(rx2)}, ry[2] = {Q::lo(ry2), Q::hi(ry2)};
    int o00[2], o01[2], o10[2], o11[2];
    T lx[2], hx[2], ly[2], hy[2];
    bool in[2];
#pragma unroll
    for (int v = 0; v < 2; ++v) {
      in[v] = !(axis_outside<T>(ry[v], p.H) || axis_outside<T>(rx[v], p.W));
      AxisTap<T> tx, ty;
      axis_tap<T>(rx[v], p.W, tx);
      axis_tap<T>(ry[v], p.H, ty);
      if (p.order == 0) { nearest_axis<T>(tx.l, tx.h); nearest_axis<T>(ty.l, ty.h); }
      o00[v] = ty.i0 * p.W + tx.i0;
      o01[v] = ty.i0 * p.W + tx.i1;
      o10[v] = ty.i1 * p.W + tx.i0;
      o11[v] = ty.i1 * p.W + tx.i1;
      lx[v] = tx.l; hx[v] = tx.h; ly[v] = ty.l; hy[v] = ty.h;
    }
    in[1] = in[1] && has_b;
    const V lx2 = Q::make(lx[0], lx[1]), hx2 = Q::make(hx[0], hx[1]);
    const V ly2 = Q::make(ly[0], ly[1]), hy2 = Q::make(hy[0], hy[1]);

    V q0[4], q1[4];          // tap values of the two source planes, lanes = the two voxels
    long long have1 = -1;    // plane offset whose values sit in q1
    for (int i = 0; i < npd; ++i) {
      const S3ZTap<T> e = sh.zt[i];
      V val = zero2;
      if (e.inside) {
        if (e.o0 == have1) {
#pragma unroll
          for (int k = 0; k < 4; ++k) q0[k] = q1[k];
        } else {
          const T* pl = vol + e.o0;
          q0[0] = Q::make(__ldg(pl + o00[0]), __ldg(pl + o00[1]));
          q0[1] = Q::make(__ldg(pl + o01[0]), __ldg(pl + o01[1]));
          q0[2] = Q::make(__ldg(pl + o10[0]), __ldg(pl + o10[1]));
          q0[3] = Q::make(__ldg(pl + o11[0]), __ldg(pl + o11[1]));
        }
        if (e.o1 == e.o0) {
#pragma unroll
          for (int k = 0; k < 4; ++k) q1[k] = q0[k];
        } else {
          const T* pl = vol + e.o1;
          q1[0] = Q::make(__ldg(pl + o00[0]), __ldg(pl + o00[1]));
          q1[1] = Q::make(__ldg(pl + o01[0]), __ldg(pl + o01[1]));
          q1[2] = Q::make(__ldg(pl + o10[0]), __ldg(pl + o10[1]));
          q1[3] = Q::make(__ldg(pl + o11[0]), __ldg(pl + o11[1]));
        }
        have1 = e.o1;
        const V hz2 = Q::dup(e.h), lz2 = Q::dup(e.l);
        const V hzhy = Q::mul(hz2, hy2), hzly = Q::mul(hz2, ly2);
        const V lzhy = Q::mul(lz2, hy2), lzly = Q::mul(lz2, ly2);
        V acc = Q::tap_first(Q::mul(hzhy, hx2), q0[0], Q::mul(hzhy, lx2), q0[1]);
        acc = Q::tap_next(acc, Q::mul(hzly, hx2), q0[2]);
        acc = Q::tap_next(acc, Q::mul(hzly, lx2), q0[3]);
        acc = Q::tap_next(acc, Q::mul(lzhy, hx2), q1[0]);
        acc = Q::tap_next(acc, Q::mul(lzhy, lx2), q1[1]);
        acc = Q::tap_next(acc, Q::mul(lzly, hx2), q1[2]);
        acc = Q::tap_next(acc, Q::mul(lzly, lx2), q1[3]);
        // output_val = 0 + val (normalises -0), then /count with count == 1
        val = Q::select(Q::add(zero2, acc), in[0], in[1]);
      }
      T* o = out + i * plane_o;
      if (vec) {
        Q::store2(o, val);
      } else {
        o[0] = Q::lo(val);
        if (has_b) o[1] = Q::hi(val);
      }
    }
    return;
  }

  // ---- general rotation: positions change with depth
  s3_full_depth_loop<T, 1>(p, sh, npd, c, pw0, ph, kS3TileH, L.vec_store != 0, out);
}

template <typename T>
__global__ void __launch_bounds__(kS3Threads)
resample_fwd_stream3d(const Params p, const S3Launch L) {
  __shared__ S3Shared<T> sh;
  const S3Cta k = s3_cta(p, L);
  if (s3_filtered_out<T>(p, L, k)) return;
  s3_prologue<T>(p, k, sh);
  s3_body_l1<T>(p, L, k, sh);
}

// The second launch of a rotated forward: the rois under a general rotation, which the
// plane-streaming launch left out.  A fixed grid of CTAs (a few per SM) first marks those rois
// in a shared bit mask -- when there is none, which is the usual case for the augmentations, the
// whole grid is gone after a few loads -- and then strides over the (roi, channel, tile, chunk)
// work items of the marked rois.
constexpr int kS3RestMaxRois = 16384;
template <typename T>
__global__ void __launch_bounds__(kS3Threads)
resample_fwd_stream3d_rest(const Params p, const S3Launch L, long long items) {
  __shared__ S3Shared<T> sh;
  __shared__ unsigned general[kS3RestMaxRois / 32];
  // the launch that follows in the stream (the plane-streaming kernel) depends on nothing this
  // kernel writes: let it start as soon as every CTA of this grid has got here
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  int mine = 0;
  for (int n0 = 0; n0 < p.R; n0 += kS3Threads) {
    const int n = n0 + threadIdx.x;
    const bool g = n < p.R && !s3_roi_is_planar<T>(p, n);
    const unsigned m = __ballot_sync(0xffffffffu, g);
    if ((threadIdx.x & 31) == 0 && n < kS3RestMaxRois) general[n >> 5] = m;
    mine |= g;
  }
  if (!__syncthreads_or(mine)) return;
  for (long long item = blockIdx.x; item < items; item += gridDim.x) {
    const S3Cta k = s3_cta(p, L, item);
    if (!((general[k.n >> 5] >> (k.n & 31)) & 1u)) continue;  // CTA-uniform
    s3_prologue<T>(p, k, sh);
    s3_body_l1<T>(p, L, k, sh);
    __syncthreads();  // the next item's prologue overwrites the tables
  }
}

}  // namespace mvr
