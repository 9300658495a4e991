// Catmull-Rom (order 3) forward for 3D volumes -- the dense-field blow-up of the elastic
// deformation and the order-3 Resize / Affine calls.
//
// Same arithmetic as hermite_3d() in mvr_geom.cuh (the restatement of
// medvision/csrc/cuda_aug/interpolation_helpers_3d.h:572-792), reorganised around the fact
// that the 64 weights of a sample depend on the roi and the output voxel but NOT on the
// channel: a thread owns one output voxel of one roi, forms the per-axis cubics and the 64
// weights once and applies them to up to four channels at a time, with 32-bit tap offsets (the general kernel redoes
// all of it per channel and keeps its weight tables in local memory).  Per (z, y) tap pair the
// four x weights are the doubles (wx*wy)*wz rounded to the element type, the four products are
// summed left to right and the group is added to the running value -- the reference's order.
#pragma once
#include "mvr_generic.cuh"

namespace mvr {

constexpr int kCubicTiles = 4;  // runs of kGenericThreads output voxels per CTA (amortises the roi decode)

// NC = channels carried per pass (C % NC == 0).  Requires D*H*W < 2^31 (32-bit tap offsets inside
// one channel's volume; the channel bases are 64-bit pointers).
template <typename T, int NC>
__global__ void __launch_bounds__(kGenericThreads)
resample_fwd_cubic3d(const Params p, int ctas_per_roi) {
  typedef Ar<T> A;
  constexpr int fm = kReferenceContraction;  // the launcher sends other patterns to the general kernel
  __shared__ GenericShared<T> sh;
  const long long n = blockIdx.x / ctas_per_roi;
  const int first_tile = (int)(blockIdx.x % ctas_per_roi) * kCubicTiles;
  generic_prologue<T>(p, n, sh);
  const RoiGeom<T>& g = sh.g;
  const bool bad = g.batch < 0 || g.batch >= p.N;
  if (bad && p.status && first_tile == 0 && threadIdx.x == 0) atomicOr(p.status, STATUS_BAD_BATCH_INDEX);
  const T* vol0 = (const T*)p.in + (long long)(bad ? 0 : g.batch) * p.C * p.vol;
  const T zero = A::fi(0);
  const int HW = p.H * p.W;

#pragma unroll 1
  for (int t = 0; t < kCubicTiles; ++t) {
    const long long e = (long long)(first_tile + t) * kGenericThreads + threadIdx.x;
    if (e >= p.ovol) return;
    T* out = (T*)p.out + n * p.C * p.ovol + e;
    if (bad) {
      for (int c = 0; c < p.C; ++c) out[c * p.ovol] = zero;
      continue;
    }
    const int pw = (int)(e % p.ow);
    const int ph = (int)((e / p.ow) % p.oh);
    const int pd = (int)(e / ((long long)p.ow * p.oh));
    const T bx = lattice_base<T>(g.start[0], pw, g.bin[0], fm);
    const T by = lattice_base<T>(g.start[1], ph, g.bin[1], fm);
    const T bz = lattice_base<T>(g.start[2], pd, g.bin[2], fm);

#pragma unroll 1
    for (int c0 = 0; c0 < p.C; c0 += NC) {
      const T* vc[NC];
#pragma unroll
      for (int cc = 0; cc < NC; ++cc) vc[cc] = vol0 + (long long)(c0 + cc) * p.vol;
      T acc[NC];
#pragma unroll
      for (int cc = 0; cc < NC; ++cc) acc[cc] = zero;
      for (int iz = 0; iz < g.grid[2]; ++iz) {
        const T z = A::add(bz, sub_offset<T>(sh, 2, iz));
        for (int iy = 0; iy < g.grid[1]; ++iy) {
          const T y = A::add(by, sub_offset<T>(sh, 1, iy));
          for (int ix = 0; ix < g.grid[0]; ++ix) {
            const T x = A::add(bx, sub_offset<T>(sh, 0, ix));
            T sx, sy, sz;
            to_volume<T, 3>(g, p.kind, fm, x, y, z, sx, sy, sz);
            T val[NC];
#pragma unroll
            for (int cc = 0; cc < NC; ++cc) val[cc] = zero;
            if (!(axis_outside<T>(sy, p.H) || axis_outside<T>(sx, p.W) || axis_outside<T>(sz, p.D))) {
              int jx[4], jy[4], jz[4];
              double wx[4], wy[4], wz[4];
              hermite_axis<T, true>(sx, p.W, jx, wx);
              hermite_axis<T, true>(sy, p.H, jy, wy);
              hermite_axis<T, true>(sz, p.D, jz, wz);
#pragma unroll
              for (int k = 0; k < 4; ++k) { jz[k] *= HW; jy[k] *= p.W; }
#pragma unroll
              for (int k = 0; k < 4; ++k) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  T w[4];
                  int o[4];
                  const int base = jz[k] + jy[j];
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    w[i] = from_double<T>(__dmul_rn(__dmul_rn(wx[i], wy[j]), wz[k]));
                    o[i] = base + jx[i];
                  }
#pragma unroll
                  for (int cc = 0; cc < NC; ++cc) {
                    T v[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) v[i] = __ldg(vc[cc] + o[i]);
                    val[cc] = A::add(val[cc], hermite_group4<T>(w, v, fm));
                  }
                }
              }
            }
#pragma unroll
            for (int cc = 0; cc < NC; ++cc) acc[cc] = A::add(acc[cc], val[cc]);
          }
        }
      }
#pragma unroll
      for (int cc = 0; cc < NC; ++cc) out[(long long)(c0 + cc) * p.ovol] = A::div(acc[cc], g.count_fwd);
    }
  }
}

// 2D counterpart (hermite_2d() of mvr_geom.cuh, interpolation_helpers_2d.h:335-424): u^2 and u^3
// stay float, the sixteen weights are the doubles wx*wy rounded to the element type, and the
// sixteen products are ONE left-to-right sum (x fastest) per channel.
template <typename T, int NC>
__global__ void __launch_bounds__(kGenericThreads)
resample_fwd_cubic2d(const Params p, int ctas_per_roi) {
  typedef Ar<T> A;
  constexpr int fm = kReferenceContraction;
  __shared__ GenericShared<T> sh;
  const long long n = blockIdx.x / ctas_per_roi;
  const int first_tile = (int)(blockIdx.x % ctas_per_roi) * kCubicTiles;
  generic_prologue<T>(p, n, sh);
  const RoiGeom<T>& g = sh.g;
  const bool bad = g.batch < 0 || g.batch >= p.N;
  if (bad && p.status && first_tile == 0 && threadIdx.x == 0) atomicOr(p.status, STATUS_BAD_BATCH_INDEX);
  const T* vol0 = (const T*)p.in + (long long)(bad ? 0 : g.batch) * p.C * p.vol;
  const T zero = A::fi(0);

#pragma unroll 1
  for (int t = 0; t < kCubicTiles; ++t) {
    const long long e = (long long)(first_tile + t) * kGenericThreads + threadIdx.x;
    if (e >= p.ovol) return;
    T* out = (T*)p.out + n * p.C * p.ovol + e;
    if (bad) {
      for (int c = 0; c < p.C; ++c) out[c * p.ovol] = zero;
      continue;
    }
    const int pw = (int)(e % p.ow), ph = (int)(e / p.ow);
    const T bx = lattice_base<T>(g.start[0], pw, g.bin[0], fm);
    const T by = lattice_base<T>(g.start[1], ph, g.bin[1], fm);
#pragma unroll 1
    for (int c0 = 0; c0 < p.C; c0 += NC) {
      const T* vc[NC];
#pragma unroll
      for (int cc = 0; cc < NC; ++cc) vc[cc] = vol0 + (long long)(c0 + cc) * p.vol;
      T acc[NC];
#pragma unroll
      for (int cc = 0; cc < NC; ++cc) acc[cc] = zero;
      for (int iy = 0; iy < g.grid[1]; ++iy) {
        const T y = A::add(by, sub_offset<T>(sh, 1, iy));
        for (int ix = 0; ix < g.grid[0]; ++ix) {
          const T x = A::add(bx, sub_offset<T>(sh, 0, ix));
          T sx, sy, sz;
          to_volume<T, 2>(g, p.kind, fm, x, y, zero, sx, sy, sz);
          T val[NC];
#pragma unroll
          for (int cc = 0; cc < NC; ++cc) val[cc] = zero;
          if (!(axis_outside<T>(sy, p.H) || axis_outside<T>(sx, p.W))) {
            int jx[4], jy[4];
            double wx[4], wy[4];
            hermite_axis<T, false>(sx, p.W, jx, wx);
            hermite_axis<T, false>(sy, p.H, jy, wy);
            T w[16];
            int o[16];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int row = jy[j] * p.W;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                w[j * 4 + i] = from_double<T>(__dmul_rn(wx[i], wy[j]));
                o[j * 4 + i] = row + jx[i];
              }
            }
#pragma unroll
            for (int cc = 0; cc < NC; ++cc) {
              T v[16];
#pragma unroll
              for (int k = 0; k < 16; ++k) v[k] = __ldg(vc[cc] + o[k]);
              val[cc] = tap_sum<T, 16>(w, v, fm);
            }
          }
#pragma unroll
          for (int cc = 0; cc < NC; ++cc) acc[cc] = A::add(acc[cc], val[cc]);
        }
      }
#pragma unroll
      for (int cc = 0; cc < NC; ++cc) out[(long long)(c0 + cc) * p.ovol] = A::div(acc[cc], g.count_fwd);
    }
  }
}

inline int fm_of(const Params& p) { return p.fm; }

// 0 launched, 1 not applicable (volume too large for 32-bit tap offsets, or a float contraction pattern other
// than the reference build's, which only the debugging switch selects), -1 too many CTAs
template <typename T>
inline int launch_cubic3d(const Params& p, cudaStream_t st) {
  if (p.vol >= 0x7fffffffLL || fm_of(p) != kReferenceContraction) return 1;
  const int ctas_per_roi = (p.tiles_per_vol + kCubicTiles - 1) / kCubicTiles;
  const long long ctas = (long long)p.R * ctas_per_roi;
  if (ctas > 0x7fffffffLL) return -1;
  const unsigned grid = (unsigned)ctas;
  if (p.ndim == 2) {
    if (p.C % 4 == 0) resample_fwd_cubic2d<T, 4><<<grid, kGenericThreads, 0, st>>>(p, ctas_per_roi);
    else if (p.C % 3 == 0) resample_fwd_cubic2d<T, 3><<<grid, kGenericThreads, 0, st>>>(p, ctas_per_roi);
    else if (p.C % 2 == 0) resample_fwd_cubic2d<T, 2><<<grid, kGenericThreads, 0, st>>>(p, ctas_per_roi);
    else resample_fwd_cubic2d<T, 1><<<grid, kGenericThreads, 0, st>>>(p, ctas_per_roi);
    return 0;
  }
  if (p.C % 4 == 0) resample_fwd_cubic3d<T, 4><<<grid, kGenericThreads, 0, st>>>(p, ctas_per_roi);
  else if (p.C % 3 == 0) resample_fwd_cubic3d<T, 3><<<grid, kGenericThreads, 0, st>>>(p, ctas_per_roi);
  else if (p.C % 2 == 0) resample_fwd_cubic3d<T, 2><<<grid, kGenericThreads, 0, st>>>(p, ctas_per_roi);
  else resample_fwd_cubic3d<T, 1><<<grid, kGenericThreads, 0, st>>>(p, ctas_per_roi);
  return 0;
}

}  // namespace mvr
