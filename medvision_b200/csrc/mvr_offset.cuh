// Dense displacement-field warp ("elastic deformation"): out[b,c,p] = interp(img[b,c], p + offset[b,:,p]).
//
// The reference routes this through its deformable-convolution machinery
// (medvision/ops/cuda_fun_tools.py:94-167): a 1x1(x1) deformable im2col
// (medvision/csrc/cuda_aug/deform_{2d,3d}_cuda_kernel.cuh) into a column buffer, then an addmm
// with an identity weight and a zero bias (cuda_aug/deform_3d_cuda.cu:118-146), then a permute.
// With a 1x1(x1) kernel, stride 1, no padding and one deformable group the column of a voxel is
// the interpolated value itself and the identity GEMM returns it unchanged, so the whole chain is
// one gather.  Arithmetic, as the reference: sample position = (element type)(integer voxel
// index) + offset, one rounded addition per axis; the sample counts only if every coordinate
// lies strictly inside (-1, size); interpolation helpers as in the roi kernels (orders 0, 1, 3).
//
// Layout of the work: a thread owns two w-adjacent voxels of one sample, forms their taps and
// weights once and applies them to every channel (the field is shared by the channels); offsets
// and results move as 2-element vectors, coalesced along w.
#pragma once
#include "mvr_stream3d.cuh"

namespace mvr {

struct OffsetParams {
  const void* img;   // (B, C, [D,] H, W)
  const void* off;   // (B, NDIM, [D,] H, W): displacement along d, h, w (3D) or h, w (2D), in voxels
  void* out;         // (B, C, [D,] H, W)
  int B, C, D, H, W, order, fm, vec_ok;
  int off_f32;       // the field is float32 although the image is half: rounded to half on load (= offset.half())
};

constexpr int kOffsetThreads = 256;

// two w-adjacent displacements of one axis, as the image's element type
template <typename T>
__device__ __forceinline__ typename P2<T>::V load_offset_pair(const OffsetParams& p, long long q, bool has_b) {
  typedef P2<T> Q;
  const T* f = (const T*)p.off + q;
  if (p.vec_ok) return *reinterpret_cast<const typename Q::V*>(f);
  return Q::make(f[0], has_b ? f[1] : Ar<T>::fi(0));
}
template <>
__device__ __forceinline__ __half2 load_offset_pair<__half>(const OffsetParams& p, long long q, bool has_b) {
  if (p.off_f32) {
    const float* f = (const float*)p.off + q;
    if (p.vec_ok) return __float22half2_rn(*reinterpret_cast<const float2*>(f));
    return __floats2half2_rn(f[0], has_b ? f[1] : 0.0f);
  }
  const __half* f = (const __half*)p.off + q;
  if (p.vec_ok) return *reinterpret_cast<const __half2*>(f);
  return __halves2half2(f[0], has_b ? f[1] : __float2half_rn(0.0f));
}

template <typename T, int NDIM, bool CUBIC>
__device__ __forceinline__ void apply_offset_pair(const OffsetParams& p, int b, int d, int h, int wp) {
  typedef Ar<T> A;
  typedef P2<T> Q;
  typedef typename Q::V V;
  const int w0 = wp * 2;
  const bool has_b = w0 + 1 < p.W;
  const long long vol = (long long)p.D * p.H * p.W;
  const long long s0 = ((long long)d * p.H + h) * p.W + w0;
  const long long off0 = (long long)b * NDIM * vol + s0;
  const T zero = A::fi(0);

  // displacement of the two voxels per axis (index 0 = w, 1 = h, 2 = d)
  V o2[3];
#pragma unroll
  for (int a = 0; a < NDIM; ++a) {
    const long long q = off0 + (long long)(NDIM - 1 - a) * vol;  // channel order of the field: d, h, w
    o2[a] = load_offset_pair<T>(p, q, has_b);
  }
  // sample positions: (T)index + offset
  const V cx = Q::add(Q::make(A::fi(w0), A::fi(w0 + 1)), o2[0]);
  const V cy = Q::add(Q::dup(A::fi(h)), o2[1]);
  const V cz = (NDIM == 3) ? Q::add(Q::dup(A::fi(d)), o2[2]) : Q::dup(zero);
  // strictly inside (-1, size) on every axis, else the result is 0
  bool ina = A::tof(Q::lo(cx)) > -1.0f && A::tof(Q::lo(cx)) < (float)p.W && A::tof(Q::lo(cy)) > -1.0f &&
             A::tof(Q::lo(cy)) < (float)p.H;
  bool inb = has_b && A::tof(Q::hi(cx)) > -1.0f && A::tof(Q::hi(cx)) < (float)p.W && A::tof(Q::hi(cy)) > -1.0f &&
             A::tof(Q::hi(cy)) < (float)p.H;
  if (NDIM == 3) {
    ina = ina && A::tof(Q::lo(cz)) > -1.0f && A::tof(Q::lo(cz)) < (float)p.D;
    inb = inb && A::tof(Q::hi(cz)) > -1.0f && A::tof(Q::hi(cz)) < (float)p.D;
  }
  const T* img = (const T*)p.img + (long long)b * p.C * vol;
  T* out = (T*)p.out + (long long)b * p.C * vol + s0;
  const V zero2 = Q::dup(zero);

  if (CUBIC) {  // Catmull-Rom: per voxel
    for (int c = 0; c < p.C; ++c, img += vol, out += vol) {
      T va = zero, vb = zero;
      if (NDIM == 3) {
        if (ina) va = hermite_3d<T>(img, p.D, p.H, p.W, Q::lo(cz), Q::lo(cy), Q::lo(cx), p.fm);
        if (inb) vb = hermite_3d<T>(img, p.D, p.H, p.W, Q::hi(cz), Q::hi(cy), Q::hi(cx), p.fm);
      } else {
        if (ina) va = hermite_2d<T>(img, p.H, p.W, Q::lo(cy), Q::lo(cx), p.fm);
        if (inb) vb = hermite_2d<T>(img, p.H, p.W, Q::hi(cy), Q::hi(cx), p.fm);
      }
      out[0] = va;
      if (has_b) out[1] = vb;
    }
    return;
  }

  AxisTap2<T> tx, ty, tz;
  axis_tap2<T>(cx, p.W, p.order, tx);
  axis_tap2<T>(cy, p.H, p.order, ty);
  if (NDIM == 3) axis_tap2<T>(cz, p.D, p.order, tz);
  const int W = p.W, HW = p.H * p.W;
  const int ba = ina ? (((NDIM == 3 ? tz.i0a * p.H : 0) + ty.i0a) * W + tx.i0a) : 0;
  const int bb = inb ? (((NDIM == 3 ? tz.i0b * p.H : 0) + ty.i0b) * W + tx.i0b) : 0;
  const int xa1 = ina ? tx.da : 0, xb1 = inb ? tx.db : 0;
  const int ya1 = (ina && ty.da) ? W : 0, yb1 = (inb && ty.db) ? W : 0;
  const int za1 = (NDIM == 3 && ina && tz.da) ? HW : 0, zb1 = (NDIM == 3 && inb && tz.db) ? HW : 0;
  const typename Q::M mask = Q::make_mask(ina, inb);
  V w[1 << NDIM];
  if (NDIM == 3) {
    const V hzhy = Q::mul(tz.h, ty.h), hzly = Q::mul(tz.h, ty.l);
    const V lzhy = Q::mul(tz.l, ty.h), lzly = Q::mul(tz.l, ty.l);
    w[0] = Q::mul(hzhy, tx.h); w[1] = Q::mul(hzhy, tx.l); w[2] = Q::mul(hzly, tx.h); w[3] = Q::mul(hzly, tx.l);
    w[4] = Q::mul(lzhy, tx.h); w[5] = Q::mul(lzhy, tx.l); w[6] = Q::mul(lzly, tx.h); w[7] = Q::mul(lzly, tx.l);
  } else {
    w[0] = Q::mul(ty.h, tx.h); w[1] = Q::mul(ty.h, tx.l); w[2] = Q::mul(ty.l, tx.h); w[3] = Q::mul(ty.l, tx.l);
  }
#pragma unroll 1
  for (int c = 0; c < p.C; ++c, img += vol, out += vol) {
    const T* pa = img + ba;
    const T* pb = img + bb;
    V v[1 << NDIM];
    v[0] = Q::make(__ldg(pa), __ldg(pb));
    v[1] = Q::make(__ldg(pa + xa1), __ldg(pb + xb1));
    v[2] = Q::make(__ldg(pa + ya1), __ldg(pb + yb1));
    v[3] = Q::make(__ldg(pa + ya1 + xa1), __ldg(pb + yb1 + xb1));
    if (NDIM == 3) {
      v[4] = Q::make(__ldg(pa + za1), __ldg(pb + zb1));
      v[5] = Q::make(__ldg(pa + za1 + xa1), __ldg(pb + zb1 + xb1));
      v[6] = Q::make(__ldg(pa + za1 + ya1), __ldg(pb + zb1 + yb1));
      v[7] = Q::make(__ldg(pa + za1 + ya1 + xa1), __ldg(pb + zb1 + yb1 + xb1));
    }
    V acc = Q::tap_first(w[0], v[0], w[1], v[1]);
#pragma unroll
    for (int k = 2; k < (1 << NDIM); ++k) acc = Q::tap_next(acc, w[k], v[k]);
    // a sample outside the image gives the literal 0; inside, the reference returns the sum as it is
    const V val = Q::apply(acc, mask);
    if (p.vec_ok) {
      Q::store2(out, val);
    } else {
      out[0] = Q::lo(val);
      if (has_b) out[1] = Q::hi(val);
    }
  }
  (void)zero2;
}

template <typename T, int NDIM, bool CUBIC>
__global__ void __launch_bounds__(kOffsetThreads, CUBIC ? 1 : 4)
apply_offset_kernel(const OffsetParams p) {
  typedef Ar<T> A;
  typedef P2<T> Q;
  typedef typename Q::V V;
  // grid.x covers the voxel pairs of one sample (fewer than 2^30), grid.y strides over the batch
  const unsigned pairs_w = (unsigned)(p.W + 1) >> 1;
  const unsigned per_sample = (unsigned)p.D * (unsigned)p.H * pairs_w;
  const unsigned idx = blockIdx.x * (unsigned)kOffsetThreads + threadIdx.x;
  if (idx >= per_sample) return;
  const int wp = (int)(idx % pairs_w);
  const unsigned row = idx / pairs_w;
  const int h = (int)(row % (unsigned)p.H);
  const int d = (int)(row / (unsigned)p.H);
  for (int b = blockIdx.y; b < p.B; b += gridDim.y) apply_offset_pair<T, NDIM, CUBIC>(p, b, d, h, wp);
}

template <int NDIM>
inline int launch_apply_offset(const OffsetParams& p, int dtype, cudaStream_t st) {
  const long long per_sample = (long long)p.D * p.H * ((p.W + 1) / 2);
  if (per_sample == 0 || p.B == 0 || p.C == 0) return 0;
  const dim3 grid((unsigned)((per_sample + kOffsetThreads - 1) / kOffsetThreads), (unsigned)min(p.B, 65535));
  const bool cubic = p.order == 3;
  if (dtype == 0) {
    if (cubic) apply_offset_kernel<float, NDIM, true><<<grid, kOffsetThreads, 0, st>>>(p);
    else apply_offset_kernel<float, NDIM, false><<<grid, kOffsetThreads, 0, st>>>(p);
  } else {
    if (cubic) apply_offset_kernel<__half, NDIM, true><<<grid, kOffsetThreads, 0, st>>>(p);
    else apply_offset_kernel<__half, NDIM, false><<<grid, kOffsetThreads, 0, st>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

}  // namespace mvr
