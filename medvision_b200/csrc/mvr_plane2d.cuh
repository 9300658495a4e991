// Dense 2D forward (one sample per output pixel: every 2D augmentation call): the 2D counterpart
// of the 3D gather path.  A thread owns two w-adjacent pixels (the two lanes of half2
// arithmetic), walks down a column of row blocks of its 32 x (16 * kP2Blocks) tile and applies
// the taps and weights of a pixel pair to every channel; the roi is decoded once per CTA; stores
// are 2-element vectors, consecutive along w within a warp row.  The arithmetic is the
// reference's (medvision/csrc/cuda/roi_align_rotated_2d_cuda_kernel.cuh:15-90,
// roi_align_2d_cuda_kernel.cuh:11-74, interpolation_helpers_2d.h), one rounded operation at a
// time: only the x products of the rotation, which do not change down a column, are hoisted.
#pragma once
#include "mvr_stream3d.cuh"

namespace mvr {

constexpr int kP2Blocks = 8;  // row blocks of kS3TileH rows per CTA

template <typename T, int ORDER>
__global__ void __launch_bounds__(kS3Threads)
resample_fwd_plane2d(const Params p, int tiles_w, int tiles_h, int vec_store) {
  typedef Ar<T> A;
  typedef P2<T> Q;
  typedef typename Q::V V;
  __shared__ RoiGeom<T> g_sh;
  const int fm = kS3FloatPattern;
  long long cta = blockIdx.x;
  const int tw = (int)(cta % tiles_w); cta /= tiles_w;
  const int th = (int)(cta % tiles_h); cta /= tiles_h;
  const long long n = cta;
  if (threadIdx.x == 0) {
    const int osz[3] = {p.ow, p.oh, 1};
    decode_roi<T>((const T*)p.rois, n, 2, p.kind, osz, p.spatial_scale, 1, p.aligned, fm, g_sh);
  }
  __syncthreads();
  const RoiGeom<T>& g = g_sh;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pw0 = tw * kS3TileW + (warp & 1) * 16 + (lane & 7) * 2;
  const int row0 = th * (kS3TileH * kP2Blocks) + (warp >> 1) * 4 + (lane >> 3);
  if (pw0 >= p.ow || row0 >= p.oh) return;
  const bool has_b = (pw0 + 1 < p.ow);
  const bool vec = vec_store && has_b;
  const long long ovol = p.ovol, vol_e = p.vol;
  T* out = (T*)p.out + n * p.C * ovol + pw0;
  const T zero = A::fi(0);
  const V zero2 = Q::dup(zero);

  if (g.batch < 0 || g.batch >= p.N) {
    if (p.status && threadIdx.x == 0 && tw == 0 && th == 0) atomicOr(p.status, STATUS_BAD_BATCH_INDEX);
    for (int b = 0; b < kP2Blocks; ++b) {
      const int ph = row0 + b * kS3TileH;
      if (ph >= p.oh) break;
      for (int c = 0; c < p.C; ++c) {
        T* o = out + c * ovol + (long long)ph * p.ow;
        o[0] = zero;
        if (has_b) o[1] = zero;
      }
    }
    return;
  }
  const T* vol = (const T*)p.in + (long long)g.batch * p.C * vol_e;
  const bool rotated = (p.kind == KIND_ROTATED);
  const T sub_x = lattice_sub<T>(g.bin[0], 0, 1), sub_y = lattice_sub<T>(g.bin[1], 0, 1);
  const T xa = A::add(lattice_base<T>(g.start[0], pw0, g.bin[0], fm), sub_x);
  const T xb = A::add(lattice_base<T>(g.start[0], has_b ? pw0 + 1 : pw0, g.bin[0], fm), sub_x);
  const V x2 = Q::make(xa, xb);
  const V cos2 = Q::dup(g.rot[0]), sin2 = Q::dup(g.rot[1]);
  const V cx2 = Q::dup(g.centre[0]), cy2 = Q::dup(g.centre[1]);
  const int W = p.W, H = p.H, C = p.C, oh = p.oh;
  const long long row_step = (long long)kS3TileH * p.ow;
  T* orow = out + (long long)row0 * p.ow;

#pragma unroll 1
  for (int b = 0, ph = row0; b < kP2Blocks && ph < oh; ++b, ph += kS3TileH, orow += row_step) {
    const T y = A::add(lattice_base<T>(g.start[1], ph, g.bin[1], fm), sub_y);
    V rx2, ry2;
    if (rotated) {
      // rx = (x*cos - y*sin) + cx ; ry = (x*sin + y*cos) + cy
      rx2 = Q::add(Q::row_xy(cos2, x2, Q::dup(A::neg(A::mul(y, g.rot[1])))), cx2);
      ry2 = Q::add(Q::row_xy(sin2, x2, Q::dup(A::mul(y, g.rot[0]))), cy2);
    } else {
      rx2 = x2;
      ry2 = Q::dup(y);
    }
    AxisTap2<T> tx, ty;
    axis_tap2<T>(rx2, W, ORDER, tx);
    axis_tap2<T>(ry2, H, ORDER, ty);
    const bool ina = !(tx.outa || ty.outa), inb = has_b && !(tx.outb || ty.outb);
    // 32-bit offsets of the four taps of either pixel inside a channel's plane
    const int a0 = ty.i0a * W + tx.i0a, b0 = ty.i0b * W + tx.i0b;
    const int a1 = a0 + tx.da, b1 = b0 + tx.db;
    const int a2 = a0 + (ty.da ? W : 0), b2 = b0 + (ty.db ? W : 0);
    const int a3 = a2 + tx.da, b3 = b2 + tx.db;
    const V w0 = Q::mul(ty.h, tx.h), w1 = Q::mul(ty.h, tx.l), w2 = Q::mul(ty.l, tx.h), w3 = Q::mul(ty.l, tx.l);
    const typename Q::M mask = Q::make_mask(ina, inb);
    const T* plane = vol;
    T* o = orow;
#pragma unroll 1
    for (int c = 0; c < C; ++c, plane += vol_e, o += ovol) {
      const V v0 = Q::make(__ldg(plane + a0), __ldg(plane + b0));
      const V v1 = Q::make(__ldg(plane + a1), __ldg(plane + b1));
      const V v2 = Q::make(__ldg(plane + a2), __ldg(plane + b2));
      const V v3 = Q::make(__ldg(plane + a3), __ldg(plane + b3));
      V acc = Q::tap_first(w0, v0, w1, v1);
      acc = Q::tap_next(acc, w2, v2);
      acc = Q::tap_next(acc, w3, v3);
      // output_val = 0 + val (normalises -0), then / count with count == 1
      const V val = Q::apply(Q::add(zero2, acc), mask);
      if (vec) {
        Q::store2(o, val);
      } else {
        o[0] = Q::lo(val);
        if (has_b) o[1] = Q::hi(val);
      }
    }
  }
}

// 0 launched, 1 not applicable
inline int try_launch_plane2d(const Params& p, int dtype, cudaStream_t st) {
  if (p.ndim != 2 || p.sampling_ratio != 1 || p.order > 1) return 1;
  if (dtype != 0 && dtype != 1) return 1;
  if (dtype == 0 && p.fm != kS3FloatPattern) return 1;
  if (p.ovol < 4096 || p.ow < 8) return 1;
  if (p.vol >= 0x7fffffffLL) return 1;                       // 32-bit offsets inside a plane
  if (dtype == 1 && (p.H > 2048 || p.W > 2048)) return 1;    // sizes as half values
  const int tiles_w = (p.ow + kS3TileW - 1) / kS3TileW;
  const int tiles_h = (p.oh + kS3TileH * kP2Blocks - 1) / (kS3TileH * kP2Blocks);
  const long long ctas = (long long)p.R * tiles_w * tiles_h;
  if (ctas > 0x7fffffffLL) return 1;
  const size_t esz = dtype == 0 ? 4 : 2;
  const int vec_store = ((p.ow & 1) == 0) && (((uintptr_t)p.out) % (2 * esz) == 0);
  const unsigned grid = (unsigned)ctas;
  if (dtype == 0) {
    if (p.order == 0) resample_fwd_plane2d<float, 0><<<grid, kS3Threads, 0, st>>>(p, tiles_w, tiles_h, vec_store);
    else resample_fwd_plane2d<float, 1><<<grid, kS3Threads, 0, st>>>(p, tiles_w, tiles_h, vec_store);
  } else {
    if (p.order == 0) resample_fwd_plane2d<__half, 0><<<grid, kS3Threads, 0, st>>>(p, tiles_w, tiles_h, vec_store);
    else resample_fwd_plane2d<__half, 1><<<grid, kS3Threads, 0, st>>>(p, tiles_w, tiles_h, vec_store);
  }
  return 0;
}

}  // namespace mvr
