// Forward and backward for the calls the streaming kernels do not take (detection heads: many
// small rois, a few output bins each, several samples per bin; 2D; double; sampling_ratio != 1),
// orders 0 and 1.
//
// Work is laid out flat, as in the reference (one thread per output element in (roi, channel,
// [d,] h, w) order), so every thread of a CTA has work whatever the size of a roi's output.  What
// differs from the reference (medvision/csrc/cuda/roi_align_rotated_3d_cuda_kernel.cuh:15-120 and
// siblings): the rois a CTA's 128 outputs belong to (at most kFlatMaxRois) are decoded once each,
// by different threads at the same time, into shared memory -- the reference decodes the roi and
// evaluates up to six sin/cos in every thread, and rebuilds the rotation matrix for every sample;
// the sample loops of the common fixed sampling ratios (1, 2) are unrolled so that all tap loads
// of an output are in flight together; the flat index is taken apart with multiply-shift constants
// from the host instead of divisions; at a fixed sampling ratio the divisions by the sample count
// and the grid (powers of two) are exact scalings.  Calls with 2^31 outputs or more, or under another
// float contraction pattern than the reference build's, go to the general kernels.  The arithmetic
// of every sample is the reference's, operation by operation.
#pragma once
#include "mvr_generic.cuh"
#include "mvr_stream3d.cuh"

namespace mvr {

constexpr int kFlatThreads = 128;
constexpr int kFlatMinPerRoi = 32;                                     // outputs per roi (C * ovol) at least
constexpr int kFlatMaxRois = kFlatThreads / kFlatMinPerRoi + 2;        // rois a CTA can span
constexpr int kFlatFm = kS3FloatPattern;                               // float contraction pattern these kernels are built for

// n / d for 0 <= n < 2^31 by one multiplication: m = floor(2^32 (2^s - d) / d) + 1 with s = ceil(log2 d), then
// q = (hi32(n * m) + n) >> s (the sum cannot carry out of 32 bits because hi32(n * m) <= n < 2^31).
struct FlatDiv {
  unsigned d, m, s;
};
inline FlatDiv make_flat_div(unsigned d) {
  FlatDiv f;
  f.d = d;
  unsigned s = 0;
  while ((1ull << s) < d) ++s;
  f.s = s;
  f.m = (unsigned)((((1ull << s) - d) << 32) / d + 1);
  return f;
}
__device__ __forceinline__ int flat_div(int n, const FlatDiv& f) {
  return (int)((__umulhi((unsigned)n, f.m) + (unsigned)n) >> f.s);
}
// the four divisors of the flat index: outputs per roi, per channel, per output row and rows per plane
struct FlatDivs {
  FlatDiv per_roi, ovol, ow, oh;
};

// These kernels run for 10-30 us, of which the boundary between two launches on a stream is 2 us: they are launched
// as programmatic dependents, so that the CTAs of a call can become resident while the last CTAs of the call before
// it are still running.  Every kernel waits (griddepcontrol.wait) for the complete end of whatever precedes it in the
// stream before it touches memory, and lets its own dependents be scheduled from then on.  After a kernel that
// never signals (any kernel that is not one of these) the launch behaves like a plain one.
__device__ __forceinline__ void flat_grid_dependency() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// type in which the contributions to one cell are summed before they leave (see the backward of resample_flat)
template <typename T> struct FlatWide;
template <> struct FlatWide<float> {
  typedef float type;
  __device__ __forceinline__ static float narrow(float v) { return v; }
};
template <> struct FlatWide<__half> {
  typedef float type;
  __device__ __forceinline__ static __half narrow(float v) { return __float2half_rn(v); }
};
template <> struct FlatWide<double> {
  typedef double type;
  __device__ __forceinline__ static double narrow(double v) { return v; }
};

// SR: compile-time sampling ratio per axis (1 or 2), or 0 = taken from the roi at run time
// (any fixed ratio, or the adaptive ceil(bin) grid).
// OFF: type of the tap offsets inside one channel's volume (int when D*H*W < 2^31).
template <typename T, int NDIM, int SR, bool BWD, typename OFF>
// (the 2D half backward is the one instantiation that gains from a full single wave of 16 CTAs per SM: 22.6 against
// 26.7 us on the rotated 2D head; the float kernels lose more to the 32-register limit than the wave gives)
__global__ void __launch_bounds__(kFlatThreads, (NDIM == 2 && BWD && sizeof(T) == 2 && SR != 0) ? 16 : 1)
resample_flat(const Params p, const FlatDivs fd, int total) {
  typedef Ar<T> A;
  constexpr int fm = kFlatFm;
  flat_grid_dependency();
  __shared__ RoiGeom<T> geo[kFlatMaxRois];
  const int per_roi = (int)fd.per_roi.d;
  const int e0 = (int)blockIdx.x * kFlatThreads;
  const int n0 = flat_div(e0, fd.per_roi);
  const int rem0 = e0 - n0 * per_roi;
  const int e_last = min(e0 + kFlatThreads, total) - 1;
  const int n_rois = flat_div(e_last, fd.per_roi) - n0 + 1;
  if ((int)threadIdx.x < n_rois) {
    const int osz[3] = {p.ow, p.oh, p.od};
    decode_roi<T>((const T*)p.rois, n0 + threadIdx.x, NDIM, p.kind, osz, p.spatial_scale, p.sampling_ratio, p.aligned,
                  fm, geo[threadIdx.x]);
  }
  __syncthreads();
  const int e = e0 + (int)threadIdx.x;
  if (e >= total) return;
  const int t = rem0 + (int)threadIdx.x;
  const int r = flat_div(t, fd.per_roi);
  const int rem = t - r * per_roi;
  const RoiGeom<T>& g = geo[r];
  const int c = flat_div(rem, fd.ovol);
  const int v = rem - c * (int)fd.ovol.d;
  const int row = flat_div(v, fd.ow);                    // (pd * oh + ph)
  const int pw = v - row * p.ow;
  const int pd = (NDIM == 3) ? flat_div(row, fd.oh) : 0;
  const int ph = (NDIM == 3) ? row - pd * p.oh : row;
  const T zero = A::fi(0);
  // count of samples per output when the sampling ratio is fixed at compile time: a power of two
  constexpr float inv_count = 1.0f / (float)((SR ? SR : 1) * (SR ? SR : 1) * ((NDIM == 3 && SR) ? SR : 1));

  if (g.batch < 0 || g.batch >= p.N) {
    if (p.status && rem == 0) atomicOr(p.status, STATUS_BAD_BATCH_INDEX);
    if (!BWD) ((T*)p.out)[e] = zero;
    return;
  }
  // fwd: the volume read; bwd: the gradient volume accumulated into
  const T* vol = (const T*)(BWD ? p.out : p.in) + ((long long)g.batch * p.C + c) * p.vol;
  T* gvol = (T*)p.out + ((long long)g.batch * p.C + c) * p.vol;
  const T* const glo = (const T*)p.out;                                // the whole gradient tensor
  const T* const ghi = glo + (long long)p.N * p.C * p.vol;
  const T go = BWD ? ((const T*)p.in)[e] : zero;

  const T bx = lattice_base<T>(g.start[0], pw, g.bin[0], fm);
  const T by = lattice_base<T>(g.start[1], ph, g.bin[1], fm);
  const T bz = (NDIM == 3) ? lattice_base<T>(g.start[2], pd, g.bin[2], fm) : zero;
  const int gx = SR ? SR : g.grid[0], gy = SR ? SR : g.grid[1], gz = (NDIM == 3) ? (SR ? SR : g.grid[2]) : 1;

  T acc = zero;
  // backward: the cell of the volume whose contributions are being summed.  Always for half gradients (the sums are
  // what keeps the small addends of an up-sampling roi); for float and double only with a run-time sample grid, where
  // consecutive samples share cells often enough for the saved reductions to pay for the bookkeeping (on the
  // down-sampling detection heads at ratio 2 it costs 15 % and saves nothing).
  constexpr bool kCellSums = BWD && (SR == 0 || sizeof(T) == 2);
  typedef typename FlatWide<T>::type Wide;
  OFF cell_off[1 << NDIM];
  Wide cell_sum[1 << NDIM];
  bool cell_held = false;
  auto flush_cell = [&]() {
    if (!cell_held) return;
#pragma unroll
    for (int k = 0; k < (1 << NDIM); k += 2)
      atomic_add_pair(gvol + cell_off[k], gvol + cell_off[k + 1], FlatWide<T>::narrow(cell_sum[k]),
                      FlatWide<T>::narrow(cell_sum[k + 1]), glo, ghi);
  };
  auto sample = [&](T x, T y, T z) {
    T sx, sy, sz;
    to_volume<T, NDIM>(g, p.kind, fm, x, y, z, sx, sy, sz);
    T w[1 << NDIM];
    OFF off[1 << NDIM];
    const bool in = make_taps<T, NDIM, OFF>(p.D, p.H, p.W, sz, sy, sx, p.order, w, off);
    if (BWD) {
      if (!in) return;
      if (kCellSums) {
        // Consecutive samples of an output often fall into the same cell of the volume (adaptive sampling spaces
        // them at most a voxel apart; an up-sampling roi puts all of them there): their contributions -- each
        // rounded to the element type as the reference forms it -- are summed in a wider type per cell and leave
        // once, when the walk leaves the cell.  Fewer reductions, and the many small addends of an up-sampling roi
        // are no longer lost one by one against a large half accumulator.
        if (!cell_held || off[0] != cell_off[0]) {
          flush_cell();
#pragma unroll
          for (int k = 0; k < (1 << NDIM); ++k) { cell_off[k] = off[k]; cell_sum[k] = 0; }
          cell_held = true;
        }
#pragma unroll
        for (int k = 0; k < (1 << NDIM); ++k)
          cell_sum[k] += (Wide)A::tof(SR ? A::scale_pow2(A::mul(go, w[k]), inv_count) : A::div(A::mul(go, w[k]), g.count_bwd));
      } else {
#pragma unroll
        for (int k = 0; k < (1 << NDIM); k += 2) {
          // a fixed ratio makes the sample count a power of two: the division is an exact scaling
          const T g0 = A::scale_pow2(A::mul(go, w[k]), inv_count);
          const T g1 = A::scale_pow2(A::mul(go, w[k + 1]), inv_count);
          atomic_add_pair(gvol + off[k], gvol + off[k + 1], g0, g1, glo, ghi);
        }
      }
    } else {
      T val = zero;
      if (in) {
        T tap[1 << NDIM];
#pragma unroll
        for (int k = 0; k < (1 << NDIM); ++k) tap[k] = __ldg(vol + off[k]);
        val = tap_sum<T, (1 << NDIM)>(w, tap, fm);
      }
      acc = A::add(acc, val);
    }
  };

  if (SR) {
    constexpr int S = SR ? SR : 1;
    T subx[S], suby[S], subz[S];
#pragma unroll
    for (int i = 0; i < S; ++i) {
      subx[i] = lattice_sub_pow2<T, S>(g.bin[0], i);
      suby[i] = lattice_sub_pow2<T, S>(g.bin[1], i);
      subz[i] = (NDIM == 3) ? lattice_sub_pow2<T, S>(g.bin[2], i) : zero;
    }
#pragma unroll
    for (int iz = 0; iz < ((NDIM == 3) ? S : 1); ++iz) {
      const T z = (NDIM == 3) ? A::add(bz, subz[iz]) : zero;
#pragma unroll
      for (int iy = 0; iy < S; ++iy) {
        const T y = A::add(by, suby[iy]);
#pragma unroll
        for (int ix = 0; ix < S; ++ix) sample(A::add(bx, subx[ix]), y, z);
      }
    }
  } else {
    for (int iz = 0; iz < gz; ++iz) {
      const T z = (NDIM == 3) ? A::add(bz, lattice_sub<T>(g.bin[2], iz, gz)) : zero;
      for (int iy = 0; iy < gy; ++iy) {
        const T y = A::add(by, lattice_sub<T>(g.bin[1], iy, gy));
        for (int ix = 0; ix < gx; ++ix) sample(A::add(bx, lattice_sub<T>(g.bin[0], ix, gx)), y, z);
      }
    }
  }
  if (BWD && kCellSums) flush_cell();
  if (!BWD) ((T*)p.out)[e] = SR ? A::scale_pow2(acc, inv_count) : A::div(acc, g.count_fwd);
}

// Forward for axis-aligned boxes (RoIAlign) with a fixed sampling ratio of 1 or 2.  Without a
// rotation the sample lattice is a product of three per-axis lattices: the taps and weights of
// an axis are formed once per axis sample (SR per axis) instead of once per sample (SR^NDIM),
// and the z*y weight products once per (z, y) sample pair.  Every product and sum is the one the
// reference forms (w = (hz*hy)*hx, left-to-right tap sum); nearest picks per axis, which selects
// the same tap as the reference's joint first-match rule.
template <typename T, int NDIM, int SR, typename OFF>
__global__ void __launch_bounds__(kFlatThreads, 10)
resample_flat_box_fwd(const Params p, const FlatDivs fd, int total) {
  typedef Ar<T> A;
  constexpr int fm = kFlatFm;
  flat_grid_dependency();
  __shared__ RoiGeom<T> geo[kFlatMaxRois];
  const int per_roi = (int)fd.per_roi.d;
  const int e0 = (int)blockIdx.x * kFlatThreads;
  const int n0 = flat_div(e0, fd.per_roi);
  const int rem0 = e0 - n0 * per_roi;
  const int e_last = min(e0 + kFlatThreads, total) - 1;
  const int n_rois = flat_div(e_last, fd.per_roi) - n0 + 1;
  if ((int)threadIdx.x < n_rois) {
    const int osz[3] = {p.ow, p.oh, p.od};
    decode_roi<T>((const T*)p.rois, n0 + threadIdx.x, NDIM, KIND_BOX, osz, p.spatial_scale, SR, p.aligned, fm,
                  geo[threadIdx.x]);
  }
  __syncthreads();
  const int e = e0 + (int)threadIdx.x;
  if (e >= total) return;
  const int t = rem0 + (int)threadIdx.x;
  const int r = flat_div(t, fd.per_roi);
  const int rem = t - r * per_roi;
  const RoiGeom<T>& g = geo[r];
  const int c = flat_div(rem, fd.ovol);
  const int v = rem - c * (int)fd.ovol.d;
  const int row = flat_div(v, fd.ow);
  const int pdv = (NDIM == 3) ? flat_div(row, fd.oh) : 0;
  const int pos[3] = {v - row * p.ow, (NDIM == 3) ? row - pdv * p.oh : row, pdv};
  const T zero = A::fi(0);
  constexpr float inv_count = 1.0f / (float)(SR * SR * (NDIM == 3 ? SR : 1));
  if (g.batch < 0 || g.batch >= p.N) {
    if (p.status && rem == 0) atomicOr(p.status, STATUS_BAD_BATCH_INDEX);
    ((T*)p.out)[e] = zero;
    return;
  }
  const T* vol = (const T*)p.in + ((long long)g.batch * p.C + c) * p.vol;
  const int size[3] = {p.W, p.H, p.D};
  const OFF stride[3] = {(OFF)1, (OFF)p.W, (OFF)p.H * p.W};

  // per axis and axis sample: the two tap offsets, the two weights, and whether the sample counts
  OFF o0[NDIM][SR], o1[NDIM][SR];
  T wl[NDIM][SR], wh[NDIM][SR];
  bool in[NDIM][SR];
#pragma unroll
  for (int a = 0; a < NDIM; ++a) {
    const T base = lattice_base<T>(g.start[a], pos[a], g.bin[a], fm);
#pragma unroll
    for (int i = 0; i < SR; ++i) {
      const T cc = A::add(base, lattice_sub_pow2<T, SR>(g.bin[a], i));
      in[a][i] = !axis_outside<T>(cc, size[a]);
      AxisTap<T> tp;
      axis_tap<T>(cc, size[a], tp);
      if (p.order == 0) nearest_axis<T>(tp.l, tp.h);
      o0[a][i] = tp.i0 * stride[a];
      o1[a][i] = tp.i1 * stride[a];
      wl[a][i] = tp.l;
      wh[a][i] = tp.h;
    }
  }

  T acc = zero;
  if (NDIM == 3) {
#pragma unroll
    for (int iz = 0; iz < SR; ++iz) {
#pragma unroll
      for (int iy = 0; iy < SR; ++iy) {
        const T hzhy = A::mul(wh[2][iz], wh[1][iy]), hzly = A::mul(wh[2][iz], wl[1][iy]);
        const T lzhy = A::mul(wl[2][iz], wh[1][iy]), lzly = A::mul(wl[2][iz], wl[1][iy]);
        const OFF b00 = o0[2][iz] + o0[1][iy], b01 = o0[2][iz] + o1[1][iy];
        const OFF b10 = o1[2][iz] + o0[1][iy], b11 = o1[2][iz] + o1[1][iy];
        const bool in_zy = in[2][iz] && in[1][iy];
#pragma unroll
        for (int ix = 0; ix < SR; ++ix) {
          // the taps of a sample outside the band are still valid addresses (clamped): load and
          // compute without a branch, then drop the value
          const OFF x0 = o0[0][ix], x1 = o1[0][ix];
          const T hx = wh[0][ix], lx = wl[0][ix];
          const T w[8] = {A::mul(hzhy, hx), A::mul(hzhy, lx), A::mul(hzly, hx), A::mul(hzly, lx),
                          A::mul(lzhy, hx), A::mul(lzhy, lx), A::mul(lzly, hx), A::mul(lzly, lx)};
          const T tap[8] = {__ldg(vol + (b00 + x0)), __ldg(vol + (b00 + x1)), __ldg(vol + (b01 + x0)),
                            __ldg(vol + (b01 + x1)), __ldg(vol + (b10 + x0)), __ldg(vol + (b10 + x1)),
                            __ldg(vol + (b11 + x0)), __ldg(vol + (b11 + x1))};
          const T sum = tap_sum<T, 8>(w, tap, fm);
          const T val = (in_zy && in[0][ix]) ? sum : zero;
          acc = A::add(acc, val);
        }
      }
    }
  } else {
#pragma unroll
    for (int iy = 0; iy < SR; ++iy) {
#pragma unroll
      for (int ix = 0; ix < SR; ++ix) {
        const OFF x0 = o0[0][ix], x1 = o1[0][ix], y0 = o0[1][iy], y1 = o1[1][iy];
        const T w[4] = {A::mul(wh[1][iy], wh[0][ix]), A::mul(wh[1][iy], wl[0][ix]),
                        A::mul(wl[1][iy], wh[0][ix]), A::mul(wl[1][iy], wl[0][ix])};
        const T tap[4] = {__ldg(vol + (y0 + x0)), __ldg(vol + (y0 + x1)), __ldg(vol + (y1 + x0)),
                          __ldg(vol + (y1 + x1))};
        const T sum = tap_sum<T, 4>(w, tap, fm);
        const T val = (in[1][iy] && in[0][ix]) ? sum : zero;
        acc = A::add(acc, val);
      }
    }
  }
  ((T*)p.out)[e] = A::scale_pow2(acc, inv_count);
}

template <typename K>
inline void flat_launch(K kernel, unsigned grid, cudaStream_t st, const Params& p, const FlatDivs& fd, int total) {
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kFlatThreads);
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, p, fd, total);
}

// 0 launched, 1 not applicable
template <typename T>
inline int launch_flat(const Params& p, bool fwd, cudaStream_t st) {
  if (p.order > 1 || p.fm != kFlatFm) return 1;
  const long long per_roi = (long long)p.C * p.ovol;
  if (per_roi < kFlatMinPerRoi) return 1;
  const long long total = (long long)p.R * per_roi;
  if (total + kFlatThreads > 0x7fffffffLL) return 1;  // flat indices (and one CTA beyond) stay below 2^31
  const unsigned grid = (unsigned)((total + kFlatThreads - 1) / kFlatThreads);
  FlatDivs fd;
  fd.per_roi = make_flat_div((unsigned)per_roi);
  fd.ovol = make_flat_div((unsigned)p.ovol);
  fd.ow = make_flat_div((unsigned)p.ow);
  fd.oh = make_flat_div((unsigned)p.oh);
  const int tot = (int)total;
  const int sr = (p.sampling_ratio == 1 || p.sampling_ratio == 2) ? p.sampling_ratio : 0;
  const bool small = p.vol < 0x7fffffffLL;
  if (fwd && p.kind == KIND_BOX && sr > 0) {
#define MVR_BOX(ND, SRV)                                                                             \
  {                                                                                                  \
    if (small) flat_launch(resample_flat_box_fwd<T, ND, SRV, int>, grid, st, p, fd, tot);         \
    else flat_launch(resample_flat_box_fwd<T, ND, SRV, long long>, grid, st, p, fd, tot);         \
  }
    if (p.ndim == 2) {
      if (sr == 1) MVR_BOX(2, 1) else MVR_BOX(2, 2)
    } else {
      if (sr == 1) MVR_BOX(3, 1) else MVR_BOX(3, 2)
    }
#undef MVR_BOX
    return 0;
  }
#define MVR_FLAT(ND, SRV)                                                                            \
  {                                                                                                  \
    if (small) {                                                                                     \
      if (fwd) flat_launch(resample_flat<T, ND, SRV, false, int>, grid, st, p, fd, tot);          \
      else flat_launch(resample_flat<T, ND, SRV, true, int>, grid, st, p, fd, tot);               \
    } else {                                                                                         \
      if (fwd) flat_launch(resample_flat<T, ND, SRV, false, long long>, grid, st, p, fd, tot);    \
      else flat_launch(resample_flat<T, ND, SRV, true, long long>, grid, st, p, fd, tot);         \
    }                                                                                                \
  }
  if (p.ndim == 2) {
    if (sr == 1) MVR_FLAT(2, 1) else if (sr == 2) MVR_FLAT(2, 2) else MVR_FLAT(2, 0)
  } else {
    if (sr == 1) MVR_FLAT(3, 1) else if (sr == 2) MVR_FLAT(3, 2) else MVR_FLAT(3, 0)
  }
#undef MVR_FLAT
  return 0;
}

}  // namespace mvr
