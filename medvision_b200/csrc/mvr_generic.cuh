// General resampling kernels: every dimensionality (2D / 3D), roi kind (axis-aligned box /
// rotated), interpolation order (0, 1), sampling_ratio (fixed or adaptive) and element type.
// They serve the detection-style calls (many small rois, a handful of output bins each,
// several sub-samples per bin), which are latency-bound, and are the fall-back of the
// streaming kernels in mvr_stream3d.cuh.
//
// One CTA owns a run of output elements of ONE (roi, channel) pair, so the roi is decoded and
// its sin/cos evaluated once per CTA instead of once per output element
// (medvision/csrc/cuda/roi_align_rotated_3d_cuda_kernel.cuh:32-73 does it per element), and
// the in-bin sub-sample offsets ((i+.5)*bin)/g -- the only divisions of the sample lattice --
// are tabulated per axis in shared memory.  All flat offsets are 64-bit (the reference's int
// index overflows beyond 2^31 elements, medvision/csrc/cuda/cuda_helpers.h:10-12).
#pragma once
#include "mvr_geom.cuh"

namespace mvr {

struct Params {
  const void* in;    // fwd: features (N,C,[D,]H,W) ; bwd: grad_out (R,C,[od,]oh,ow)
  const void* rois;  // (R, 5|7|6|10), same element type
  void* out;         // fwd: output (R,C,[od,]oh,ow) ; bwd: grad_in (N,C,[D,]H,W), accumulated into
  int* status;       // device word, OR-ed with STATUS_* bits; may be null
  int ndim, kind, order, aligned, sampling_ratio, fm;
  int N, C, D, H, W, R, od, oh, ow;
  float spatial_scale;
  long long vol, ovol;  // D*H*W, od*oh*ow
  int tiles_per_vol;    // CTAs per (roi, channel)
};

enum { STATUS_BAD_BATCH_INDEX = 1 };

constexpr int kGenericThreads = 256;
constexpr int kMaxGridTab = 32;  // sub-sample table entries per axis kept in shared memory

template <typename T>
struct GenericShared {
  RoiGeom<T> g;
  T sub[3][kMaxGridTab];
};

template <typename T>
__device__ __forceinline__ void generic_prologue(const Params& p, long long n, GenericShared<T>& sh) {
  if (threadIdx.x == 0) {
    const int osz[3] = {p.ow, p.oh, p.od};
    decode_roi<T>((const T*)p.rois, n, p.ndim, p.kind, osz, p.spatial_scale, p.sampling_ratio, p.aligned, p.fm, sh.g);
  }
  __syncthreads();
  if (threadIdx.x < 3 * kMaxGridTab) {
    const int a = threadIdx.x / kMaxGridTab, i = threadIdx.x % kMaxGridTab;
    if (a < p.ndim && i < sh.g.grid[a]) sh.sub[a][i] = lattice_sub<T>(sh.g.bin[a], i, sh.g.grid[a]);
  }
  __syncthreads();
}

template <typename T>
__device__ __forceinline__ T sub_offset(const GenericShared<T>& sh, int a, int i) {
  return (i < kMaxGridTab) ? sh.sub[a][i] : lattice_sub<T>(sh.g.bin[a], i, sh.g.grid[a]);
}

// sample position in the volume for local lattice coordinates (x, y, z)
template <typename T, int NDIM>
__device__ __forceinline__ void to_volume(const RoiGeom<T>& g, int kind, int fm, T x, T y, T z, T& sx, T& sy, T& sz) {
  if (kind == KIND_ROTATED) {
    if (NDIM == 2) {
      sx = rot_row2<T>(x, g.rot[0], y, g.rot[1], true, g.centre[0], fm);
      sy = rot_row2<T>(x, g.rot[1], y, g.rot[0], false, g.centre[1], fm);
      sz = z;
    } else {
      sx = rot_row3<T>(g.rot[0], x, g.rot[1], y, g.rot[2], z, g.centre[0], Fm::row(fm, 0));
      sy = rot_row3<T>(g.rot[3], x, g.rot[4], y, g.rot[5], z, g.centre[1], Fm::row(fm, 1));
      sz = rot_row3<T>(g.rot[6], x, g.rot[7], y, g.rot[8], z, g.centre[2], Fm::row(fm, 2));
    }
  } else {
    sx = x; sy = y; sz = z;
  }
}

template <typename T, int NDIM>
__global__ void __launch_bounds__(kGenericThreads)
resample_fwd_generic(const Params p) {
  typedef Ar<T> A;
  __shared__ GenericShared<T> sh;
  const long long cta = blockIdx.x;
  const long long nc = cta / p.tiles_per_vol;
  const int tile = (int)(cta % p.tiles_per_vol);
  const long long n = nc / p.C;
  const int c = (int)(nc % p.C);
  generic_prologue<T>(p, n, sh);
  const RoiGeom<T>& g = sh.g;

  const long long e = (long long)tile * kGenericThreads + threadIdx.x;
  if (e >= p.ovol) return;
  T* out = (T*)p.out + nc * p.ovol + e;
  if (g.batch < 0 || g.batch >= p.N) {
    if (p.status && e == 0) atomicOr(p.status, STATUS_BAD_BATCH_INDEX);
    *out = A::fi(0);
    return;
  }
  const int pw = (int)(e % p.ow);
  const int ph = (int)((e / p.ow) % p.oh);
  const int pd = (int)(e / ((long long)p.ow * p.oh));
  const T* vol = (const T*)p.in + ((long long)g.batch * p.C + c) * p.vol;

  const T bx = lattice_base<T>(g.start[0], pw, g.bin[0], p.fm);
  const T by = lattice_base<T>(g.start[1], ph, g.bin[1], p.fm);
  const T bz = (NDIM == 3) ? lattice_base<T>(g.start[2], pd, g.bin[2], p.fm) : A::fi(0);
  const int gd = (NDIM == 3) ? g.grid[2] : 1;

  T acc = A::fi(0);
  for (int iz = 0; iz < gd; ++iz) {
    const T z = (NDIM == 3) ? A::add(bz, sub_offset<T>(sh, 2, iz)) : A::fi(0);
    for (int iy = 0; iy < g.grid[1]; ++iy) {
      const T y = A::add(by, sub_offset<T>(sh, 1, iy));
      for (int ix = 0; ix < g.grid[0]; ++ix) {
        const T x = A::add(bx, sub_offset<T>(sh, 0, ix));
        T sx, sy, sz;
        to_volume<T, NDIM>(g, p.kind, p.fm, x, y, z, sx, sy, sz);
        T w[1 << NDIM], v[1 << NDIM];
        long long off[1 << NDIM];
        T val = A::fi(0);
        if (p.order == 3) {
          val = (NDIM == 2) ? hermite_2d<T>(vol, p.H, p.W, sy, sx, p.fm) : hermite_3d<T>(vol, p.D, p.H, p.W, sz, sy, sx, p.fm);
        } else if (make_taps<T, NDIM>(p.D, p.H, p.W, sz, sy, sx, p.order, w, off)) {
#pragma unroll
          for (int k = 0; k < (1 << NDIM); ++k) v[k] = __ldg(vol + off[k]);
          val = tap_sum<T, (1 << NDIM)>(w, v, p.fm);
        }
        acc = A::add(acc, val);
      }
    }
  }
  *out = A::div(acc, g.count_fwd);
}

// element-type atomic add, as the reference's atomicAdd(scalar_t*, scalar_t)
__device__ __forceinline__ void atomic_add_T(float* p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void atomic_add_T(double* p, double v) { atomicAdd(p, v); }
// half: a plain reduction (`atomicAdd(__half*)` asks for the old value back and is several times slower);
// .noftz keeps subnormals, as the reference's half atomicAdd does
__device__ __forceinline__ void atomic_add_T(__half* p, __half v) {
  asm volatile("red.global.add.noftz.f16 [%0], %1;" ::"l"(p), "h"(__half_as_ushort(v)) : "memory");
}

// The two x-neighbours of a tap row (p1 == p0 + 1, or p1 == p0 where the upper tap is clamped onto the last
// column), added to a gradient volume that spans [lo, hi).  Each lane is still an element-type add in whatever
// order the hardware serves it, as with the reference's scalar atomics.
//
// float: the reduction path costs one slot per lane and 16-byte chunk, whatever the width of the operation (and
// lanes that hit the SAME address do not merge), so a lane sends ONE four-element reduction to the 16-byte window
// of its lower tap, with the two values in their slots and zeros elsewhere (x + 0 = x); only a lane whose lower tap
// sits in the window's last slot sends its upper tap separately -- 1.25 operations per row on average.  A window
// that would reach outside the volume (its first or last elements, when its ends are not 16-byte aligned) is not
// used: those lanes send two scalar reductions.
__device__ __forceinline__ void atomic_add_pair(float* p0, float* p1, float v0, float v1, const float* lo,
                                                const float* hi) {
  const unsigned k0 = (unsigned)(reinterpret_cast<unsigned long long>(p0) >> 2) & 3u;
  const unsigned k1 = k0 + (unsigned)(p1 - p0);
  float* base = p0 - k0;
  if (base < lo || base + 4 > hi) {
    atomicAdd(p0, v0);
    atomicAdd(p1, v1);
    return;
  }
  const float a = (k0 == 0 ? v0 : 0.0f) + (k1 == 0 ? v1 : 0.0f);
  const float b = (k0 == 1 ? v0 : 0.0f) + (k1 == 1 ? v1 : 0.0f);
  const float c = (k0 == 2 ? v0 : 0.0f) + (k1 == 2 ? v1 : 0.0f);
  const float d = (k0 == 3 ? v0 : 0.0f) + (k1 == 3 ? v1 : 0.0f);
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(base), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
  if (k1 == 4) atomicAdd(p1, v1);
}
// half: the same with the 16-byte window of eight halves (the upper tap falls outside it one time in eight)
__device__ __forceinline__ void atomic_add_pair(__half* p0, __half* p1, __half v0, __half v1, const __half* lo,
                                                const __half* hi) {
  const unsigned k0 = (unsigned)(reinterpret_cast<unsigned long long>(p0) >> 1) & 7u;
  __half* base = p0 - k0;
  if (base < lo || base + 8 > hi) {
    atomic_add_T(p0, v0);
    atomic_add_T(p1, v1);
    return;
  }
  if (p1 == p0) {  // clamped upper tap: its weight is zero
    v0 = __hadd_rn(v0, v1);
    v1 = __ushort_as_half((unsigned short)0);
  }
  const unsigned k1 = k0 + 1u;
  // the two values at halves k0 and k0 + 1 of a 128-bit word
  const unsigned long long u0 = (unsigned long long)__half_as_ushort(v0) << (16u * (k0 & 3u));
  const unsigned long long u1 = (k1 < 8u) ? (unsigned long long)__half_as_ushort(v1) << (16u * (k1 & 3u)) : 0ull;
  const unsigned long long w_lo = (k0 < 4u ? u0 : 0ull) | (k1 < 4u ? u1 : 0ull);
  const unsigned long long w_hi = (k0 >= 4u ? u0 : 0ull) | (k1 >= 4u ? u1 : 0ull);
  asm volatile("red.global.add.noftz.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(base), "r"((unsigned)w_lo),
               "r"((unsigned)(w_lo >> 32)), "r"((unsigned)w_hi), "r"((unsigned)(w_hi >> 32))
               : "memory");
  if (k1 == 8u && p1 != p0) atomic_add_T(p1, v1);
}
__device__ __forceinline__ void atomic_add_pair(double* p0, double* p1, double v0, double v1, const double*,
                                                const double*) {
  atomicAdd(p0, v0);
  atomicAdd(p1, v1);
}

template <typename T, int NDIM>
__global__ void __launch_bounds__(kGenericThreads)
resample_bwd_generic(const Params p) {
  typedef Ar<T> A;
  __shared__ GenericShared<T> sh;
  const long long cta = blockIdx.x;
  const long long nc = cta / p.tiles_per_vol;
  const int tile = (int)(cta % p.tiles_per_vol);
  const long long n = nc / p.C;
  const int c = (int)(nc % p.C);
  generic_prologue<T>(p, n, sh);
  const RoiGeom<T>& g = sh.g;

  const long long e = (long long)tile * kGenericThreads + threadIdx.x;
  if (e >= p.ovol) return;
  if (g.batch < 0 || g.batch >= p.N) {
    if (p.status && e == 0) atomicOr(p.status, STATUS_BAD_BATCH_INDEX);
    return;
  }
  const int pw = (int)(e % p.ow);
  const int ph = (int)((e / p.ow) % p.oh);
  const int pd = (int)(e / ((long long)p.ow * p.oh));
  T* gvol = (T*)p.out + ((long long)g.batch * p.C + c) * p.vol;
  const T go = ((const T*)p.in)[nc * p.ovol + e];

  const T bx = lattice_base<T>(g.start[0], pw, g.bin[0], p.fm);
  const T by = lattice_base<T>(g.start[1], ph, g.bin[1], p.fm);
  const T bz = (NDIM == 3) ? lattice_base<T>(g.start[2], pd, g.bin[2], p.fm) : A::fi(0);
  const int gd = (NDIM == 3) ? g.grid[2] : 1;

  for (int iz = 0; iz < gd; ++iz) {
    const T z = (NDIM == 3) ? A::add(bz, sub_offset<T>(sh, 2, iz)) : A::fi(0);
    for (int iy = 0; iy < g.grid[1]; ++iy) {
      const T y = A::add(by, sub_offset<T>(sh, 1, iy));
      for (int ix = 0; ix < g.grid[0]; ++ix) {
        const T x = A::add(bx, sub_offset<T>(sh, 0, ix));
        T sx, sy, sz;
        to_volume<T, NDIM>(g, p.kind, p.fm, x, y, z, sx, sy, sz);
        T w[1 << NDIM];
        long long off[1 << NDIM];
        if (!make_taps<T, NDIM>(p.D, p.H, p.W, sz, sy, sx, p.order, w, off)) continue;
#pragma unroll
        for (int k = 0; k < (1 << NDIM); ++k) {
          const T gk = A::div(A::mul(go, w[k]), g.count_bwd);
          atomic_add_T(gvol + off[k], gk);
        }
      }
    }
  }
}

// Measurement utility (no counterpart in the reference): sets mask[b, c, voxel] = 1 for every
// input element that some tap of the forward call reads, whatever its weight.  The number of
// set bytes is the "distinct input elements touched" term of the forward's algorithmic bytes.
template <typename T, int NDIM>
__global__ void __launch_bounds__(kGenericThreads)
resample_mark_generic(const Params p) {
  typedef Ar<T> A;
  __shared__ GenericShared<T> sh;
  const long long cta = blockIdx.x;
  const long long nc = cta / p.tiles_per_vol;
  const int tile = (int)(cta % p.tiles_per_vol);
  const long long n = nc / p.C;
  const int c = (int)(nc % p.C);
  generic_prologue<T>(p, n, sh);
  const RoiGeom<T>& g = sh.g;
  const long long e = (long long)tile * kGenericThreads + threadIdx.x;
  if (e >= p.ovol || g.batch < 0 || g.batch >= p.N) return;
  const int pw = (int)(e % p.ow);
  const int ph = (int)((e / p.ow) % p.oh);
  const int pd = (int)(e / ((long long)p.ow * p.oh));
  unsigned char* mask = (unsigned char*)p.out + ((long long)g.batch * p.C + c) * p.vol;
  const T bx = lattice_base<T>(g.start[0], pw, g.bin[0], p.fm);
  const T by = lattice_base<T>(g.start[1], ph, g.bin[1], p.fm);
  const T bz = (NDIM == 3) ? lattice_base<T>(g.start[2], pd, g.bin[2], p.fm) : A::fi(0);
  const int gd = (NDIM == 3) ? g.grid[2] : 1;
  for (int iz = 0; iz < gd; ++iz) {
    const T z = (NDIM == 3) ? A::add(bz, sub_offset<T>(sh, 2, iz)) : A::fi(0);
    for (int iy = 0; iy < g.grid[1]; ++iy) {
      const T y = A::add(by, sub_offset<T>(sh, 1, iy));
      for (int ix = 0; ix < g.grid[0]; ++ix) {
        const T x = A::add(bx, sub_offset<T>(sh, 0, ix));
        T sx, sy, sz;
        to_volume<T, NDIM>(g, p.kind, p.fm, x, y, z, sx, sy, sz);
        T w[1 << NDIM];
        long long off[1 << NDIM];
        if (!make_taps<T, NDIM>(p.D, p.H, p.W, sz, sy, sx, p.order, w, off)) continue;
#pragma unroll
        for (int k = 0; k < (1 << NDIM); ++k) mask[off[k]] = 1;
      }
    }
  }
}

}  // namespace mvr
