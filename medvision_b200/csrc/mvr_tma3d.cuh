// TMA-staged variant of the streaming 3D forward kernel (z-separable rois only; every other
// CTA runs the plain-load body of mvr_stream3d.cuh).
//
// What changes with respect to the plain-load body
//   * The source planes a CTA needs are copied into shared memory by the TMA unit, one
//     rectangular box per plane -- the bounding box of the tile's in-plane taps -- through a ring
//     of buffers (as many as fit the ring for the chosen box size), several planes ahead of their use.  The copy costs no issue slots, and
//     the 2^2 in-plane taps of a voxel become four shared-memory loads at FIXED offsets from one
//     per-thread address (+0, +1 element, +1 row, +1 row +1 element):
//       - when the reference clamps a neighbour index (x1 = x0 at the last column, y1 = y0 at
//         the last row) the corresponding weight is exactly 0, and the box element read instead
//         lies outside the tensor, where the TMA unit fills zeros: 0 * 0 = 0 = 0 * v for finite v;
//       - the box x-origin is rounded down to a 16-byte boundary, as the TMA unit requires.
//   * Which planes to copy and in which order is decided once per CTA (plane schedule).  A
//     ninth warp is the producer: one of its lanes waits for a free ring slot and starts the
//     next copy.  The eight consumer warps never meet at a CTA-wide barrier inside the depth
//     loop: a warp waits for a plane ("full" mbarrier), moves its eight tap values into
//     registers and immediately hands the slot back ("empty" mbarrier, one arrival per warp);
//     the values of the newest plane and the one before stay in registers, which is all a depth
//     needs, so every plane is read from shared memory once per warp.
// Waits on mbarriers are bounded: on expiry the waiting thread raises STATUS_TMA_TIMEOUT and an
// abort flag that ends the other waits; the producer leaves only after its own copies in flight
// have landed (bounded again).
//
// No cluster launch, no multicast: every CTA fetches its own boxes from this GPU's memory.
#pragma once
#include <cuda.h>

#include "mvr_stream3d.cuh"

namespace mvr {

enum { STATUS_TMA_TIMEOUT = 2 };

constexpr int kT3RingBytes = 40960;   // shared-memory ring of plane boxes
constexpr int kT3MaxStages = 12;
constexpr int kT3MaxBoxBytes = 12800; // largest box; leaves three ring slots
constexpr int kT3MaxBoxes = 6;
constexpr int kT3MaxPlanes = 2 * kS3MaxChunk;
constexpr unsigned kT3SpinLimit = 1u << 22;
constexpr int kT3Threads = kS3Threads + 32;  // 8 consumer warps + 1 producer warp

struct T3Maps {
  CUtensorMap map[kT3MaxBoxes];  // same tensor (W, H, N*C*D), different box sizes, ascending
  int bw[kT3MaxBoxes], bh[kT3MaxBoxes];
  int n;
};

// per output depth, for the consumers
template <typename T>
struct __align__(8) T3Ent {
  T h, l;               // z weights
  unsigned short adv;   // new planes to take from the ring before this depth (0, 1 or 2)
  unsigned short flags; // T3_INSIDE, T3_SAME
};
enum { T3_INSIDE = 1, T3_SAME = 2 };  // SAME: both z taps are the newest plane

template <typename T>
struct T3Shared {
  S3Shared<T> s3;
  unsigned long long full[kT3MaxStages];   // producer -> consumers: the plane has landed
  unsigned long long empty[kT3MaxStages];  // consumers -> producer: every warp has read the plane
  int plane[kT3MaxPlanes];                 // plane schedule: source plane index, in order of use
  T3Ent<T> ent[kS3MaxChunk];
  int warp_tot[4];
  int starts;                              // depths that start a run of inside depths (must be <= 1)
  int ok;                                  // 0: the plane order is not of the expected form -> plain loads
  int box[4];                              // xmin, xmax, ymin, ymax over the tile's inside voxels
  volatile int abort_flag;
};

__device__ __forceinline__ unsigned t3_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void t3_mbar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(t3_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void t3_mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(t3_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void t3_mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(t3_smem(bar)) : "memory");
}
__device__ __forceinline__ bool t3_mbar_try_wait(unsigned long long* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n"
      "  .reg .pred p;\n"
      "  mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "  selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(t3_smem(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when the limit is reached or another thread of the CTA gave up.
__device__ __forceinline__ bool t3_mbar_wait(unsigned long long* bar, unsigned parity, volatile int* abort_flag) {
  if (t3_mbar_try_wait(bar, parity)) return true;
  for (unsigned spin = 0; spin < kT3SpinLimit; ++spin) {
    if (t3_mbar_try_wait(bar, parity)) return true;
    if ((spin & 255u) == 255u && abort_flag && *abort_flag) return false;
    if (spin > 16) __nanosleep(40);
  }
  return false;
}
__device__ __forceinline__ void t3_tma_load_3d(unsigned dst, const CUtensorMap* map, unsigned long long* bar, int x,
                                               int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(t3_smem(bar))
      : "memory");
}

// the four in-plane taps of this thread's two voxels, out of one ring slot
template <typename T>
__device__ __forceinline__ void t3_read_plane(const unsigned char* sa, const unsigned char* sb, unsigned row,
                                              typename P2<T>::V* q) {
  typedef P2<T> Q;
  const T* a0 = reinterpret_cast<const T*>(sa);
  const T* b0 = reinterpret_cast<const T*>(sb);
  const T* a1 = reinterpret_cast<const T*>(sa + row);
  const T* b1 = reinterpret_cast<const T*>(sb + row);
  q[0] = Q::make(a0[0], b0[0]);
  q[1] = Q::make(a0[1], b0[1]);
  q[2] = Q::make(a1[0], b1[0]);
  q[3] = Q::make(a1[1], b1[1]);
}

// the reference's tap sum for two voxels at once: older plane first (w1..w4), newer plane last
template <typename T>
__device__ __forceinline__ typename P2<T>::V t3_interp(T h, T l, typename P2<T>::V hy2, typename P2<T>::V ly2,
                                                       typename P2<T>::V hx2, typename P2<T>::V lx2,
                                                       const typename P2<T>::V* p0, const typename P2<T>::V* p1) {
  typedef P2<T> Q;
  typedef typename Q::V V;
  const V hz2 = Q::dup(h), lz2 = Q::dup(l);
  const V hzhy = Q::mul(hz2, hy2), hzly = Q::mul(hz2, ly2);
  const V lzhy = Q::mul(lz2, hy2), lzly = Q::mul(lz2, ly2);
  V acc = Q::tap_first(Q::mul(hzhy, hx2), p0[0], Q::mul(hzhy, lx2), p0[1]);
  acc = Q::tap_next(acc, Q::mul(hzly, hx2), p0[2]);
  acc = Q::tap_next(acc, Q::mul(hzly, lx2), p0[3]);
  acc = Q::tap_next(acc, Q::mul(lzhy, hx2), p1[0]);
  acc = Q::tap_next(acc, Q::mul(lzhy, lx2), p1[1]);
  acc = Q::tap_next(acc, Q::mul(lzly, hx2), p1[2]);
  acc = Q::tap_next(acc, Q::mul(lzly, lx2), p1[3]);
  return acc;
}

template <typename T>
__global__ void __launch_bounds__(kT3Threads)
resample_fwd_stream3d_tma(const Params p, const S3Launch L, const __grid_constant__ T3Maps maps) {
  typedef Ar<T> A;
  typedef P2<T> Q;
  typedef typename Q::V V;
  extern __shared__ __align__(128) unsigned char t3_dyn[];
  unsigned char* ring = t3_dyn;  // kT3RingBytes, 128-byte aligned
  T3Shared<T>& sh = *reinterpret_cast<T3Shared<T>*>(t3_dyn + kT3RingBytes);

  const S3Cta k = s3_cta(p, L);
  if (threadIdx.x == 0) {
    sh.box[0] = 0x7fffffff; sh.box[1] = -0x7fffffff; sh.box[2] = 0x7fffffff; sh.box[3] = -0x7fffffff;
    sh.abort_flag = 0;
    sh.starts = 0;
    sh.ok = 1;
  }
  s3_prologue<T>(p, k, sh.s3);  // ends with __syncthreads()
  const RoiGeom<T>& g = sh.s3.g;
  const bool bad_batch = (g.batch < 0 || g.batch >= p.N);
  if (!sh.s3.zsep || bad_batch) {  // CTA-uniform
    if (threadIdx.x < kS3Threads) s3_body_l1<T>(p, L, k, sh.s3);
    return;
  }

  const int fm = kS3FloatPattern;
  const bool rotated = (p.kind == KIND_ROTATED);
  const int npd = k.npd;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool consumer = warp < kS3Threads / 32;
  const int pw0 = k.tw * kS3TileW + (warp & 1) * 16 + (lane & 7) * 2;
  const int ph = k.th * kS3TileH + (warp >> 1) * 4 + (lane >> 3);
  const bool active = consumer && (ph < p.oh && pw0 < p.ow);
  const bool has_b = active && (pw0 + 1 < p.ow);

  // ---- in-plane position, taps and weights of the two voxels: once per thread
  int x0a = 0, x0b = 0, y0a = 0, y0b = 0;
  bool ina = false, inb = false;
  V lx2, hx2, ly2, hy2;
  {
    const int pwa = active ? pw0 : 0, pwb = has_b ? pw0 + 1 : pwa, phc = active ? ph : 0;
    const T sub_x = lattice_sub<T>(g.bin[0], 0, 1), sub_y = lattice_sub<T>(g.bin[1], 0, 1);
    const T xa = A::add(lattice_base<T>(g.start[0], pwa, g.bin[0], fm), sub_x);
    const T xb = A::add(lattice_base<T>(g.start[0], pwb, g.bin[0], fm), sub_x);
    const T y = A::add(lattice_base<T>(g.start[1], phc, g.bin[1], fm), sub_y);
    const V x2 = Q::make(xa, xb);
    V rx2, ry2;
    if (rotated) {
      rx2 = Q::add(Q::row_xy(Q::dup(g.rot[0]), x2, Q::dup(A::mul(g.rot[1], y))), Q::dup(g.centre[0]));
      ry2 = Q::add(Q::row_xy(Q::dup(g.rot[3]), x2, Q::dup(A::mul(g.rot[4], y))), Q::dup(g.centre[1]));
    } else {
      rx2 = x2;
      ry2 = Q::dup(y);
    }
    AxisTap<T> txa, txb, tya, tyb;
    ina = active && !(axis_outside<T>(Q::lo(ry2), p.H) || axis_outside<T>(Q::lo(rx2), p.W));
    inb = has_b && !(axis_outside<T>(Q::hi(ry2), p.H) || axis_outside<T>(Q::hi(rx2), p.W));
    axis_tap<T>(Q::lo(rx2), p.W, txa);
    axis_tap<T>(Q::hi(rx2), p.W, txb);
    axis_tap<T>(Q::lo(ry2), p.H, tya);
    axis_tap<T>(Q::hi(ry2), p.H, tyb);
    if (p.order == 0) {
      nearest_axis<T>(txa.l, txa.h); nearest_axis<T>(txb.l, txb.h);
      nearest_axis<T>(tya.l, tya.h); nearest_axis<T>(tyb.l, tyb.h);
    }
    x0a = txa.i0; x0b = txb.i0; y0a = tya.i0; y0b = tyb.i0;
    lx2 = Q::make(txa.l, txb.l); hx2 = Q::make(txa.h, txb.h);
    ly2 = Q::make(tya.l, tyb.l); hy2 = Q::make(tya.h, tyb.h);
  }

  // ---- bounding box of the tile's base taps (inside voxels only)
  {
    int xmin = 0x7fffffff, xmax = -0x7fffffff, ymin = 0x7fffffff, ymax = -0x7fffffff;
    if (ina) { xmin = xmax = x0a; ymin = ymax = y0a; }
    if (inb) { xmin = min(xmin, x0b); xmax = max(xmax, x0b); ymin = min(ymin, y0b); ymax = max(ymax, y0b); }
    xmin = __reduce_min_sync(0xffffffffu, xmin); xmax = __reduce_max_sync(0xffffffffu, xmax);
    ymin = __reduce_min_sync(0xffffffffu, ymin); ymax = __reduce_max_sync(0xffffffffu, ymax);
    if (lane == 0 && xmin <= xmax) {
      atomicMin(&sh.box[0], xmin); atomicMax(&sh.box[1], xmax);
      atomicMin(&sh.box[2], ymin); atomicMax(&sh.box[3], ymax);
    }
  }

  // ---- plane schedule, in parallel over the depths of the chunk.
  // The distinct source planes are used in a fixed order; a depth needs the newest plane (its z1)
  // and either the same plane again or the one fetched just before it (its z0).  Thread i compares
  // depth i with depth i-1, decides how many planes are new (0, 1 or 2), and a prefix sum of
  // those counts gives each new plane its position in the schedule.
  {
    const int i = threadIdx.x;
    int adv = 0, z_first = 0, z_second = 0;
    if (i < npd) {
      const S3ZTap<T> e = sh.s3.zt[i];
      T3Ent<T> t;
      t.h = e.h; t.l = e.l; t.flags = 0;
      if (e.inside) {
        const bool same = (e.z0 == e.z1);
        bool ok = true;
        bool prev_in = false;
        int pz0 = 0, pz1 = 0;
        if (i > 0) { prev_in = sh.s3.zt[i - 1].inside != 0; pz0 = sh.s3.zt[i - 1].z0; pz1 = sh.s3.zt[i - 1].z1; }
        if (!prev_in) {
          adv = same ? 1 : 2;
          atomicAdd(&sh.starts, 1);
          z_first = e.z0; z_second = e.z1;
        } else {
          const bool n0 = (e.z0 != pz0 && e.z0 != pz1);
          const bool n1 = !same && (e.z1 != pz0 && e.z1 != pz1);
          adv = (n0 ? 1 : 0) + (n1 ? 1 : 0);
          if (same) ok = n0 || (e.z1 == pz1);
          else if (adv == 1) ok = n1 && (e.z0 == pz1);
          else if (adv == 0) ok = (e.z1 == pz1) && (e.z0 == pz0) && (pz0 != pz1);
          z_first = (adv == 2 || same) ? e.z0 : e.z1;
          z_second = e.z1;
        }
        if (!ok) sh.ok = 0;
        t.flags = (unsigned short)(T3_INSIDE | (same ? T3_SAME : 0));
      }
      t.adv = (unsigned short)adv;
      sh.ent[i] = t;
    }
    int v = adv;  // inclusive prefix sum within the warp
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, v, d);
      if (lane >= d) v += u;
    }
    if (lane == 31 && warp < 4) sh.warp_tot[warp] = v;
    if (threadIdx.x == 0) {
      for (int s = 0; s < kT3MaxStages; ++s) {
        t3_mbar_init(&sh.full[s], 1);
        t3_mbar_init(&sh.empty[s], kS3Threads / 32);
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    if (adv > 0) {
      int pos = v - adv;
      for (int w = 0; w < warp; ++w) pos += sh.warp_tot[w];
      sh.plane[pos] = z_first;
      if (adv == 2) sh.plane[pos + 1] = z_second;
    }
  }
  __syncthreads();  // the last CTA-wide barrier: from here on warps run independently

  // ---- choose the smallest box that holds the tile's taps (+1 neighbour column and row)
  const int esz = (int)sizeof(T);
  const int xalign = 16 / esz;
  const bool any_inside = sh.box[0] <= sh.box[1];
  int bx0 = 0, by0 = 0, bsel = -1;
  if (any_inside) {
    bx0 = sh.box[0] - (sh.box[0] % xalign);
    by0 = sh.box[2];
    const int need_w = sh.box[1] + 2 - bx0, need_h = sh.box[3] + 2 - by0;
    for (int j = 0; j < maps.n; ++j)
      if (bsel < 0 && need_w <= maps.bw[j] && need_h <= maps.bh[j]) bsel = j;
    if (bsel < 0 || !sh.ok || sh.starts > 1) {  // footprint exceeds every box, or unusual plane order
      if (threadIdx.x < kS3Threads) s3_body_l1<T>(p, L, k, sh.s3);
      return;
    }
  }
  const int bw = any_inside ? maps.bw[bsel] : 0, bh = any_inside ? maps.bh[bsel] : 0;
  const int n_planes = any_inside ? sh.warp_tot[0] + sh.warp_tot[1] + sh.warp_tot[2] + sh.warp_tot[3] : 0;
  const unsigned box_bytes = (unsigned)(bw * bh * esz);
  const unsigned stride = (box_bytes + 127u) & ~127u;
  const int nst = any_inside ? min(kT3MaxStages, (int)(kT3RingBytes / stride)) : 1;

  if (!consumer) {
    // ================= producer warp: one lane feeds the ring =================
    if (lane != 0) return;
    const int zbase = (g.batch * p.C + k.c) * p.D;  // index of the volume's first plane in (N*C*D)
    const unsigned ring_s = t3_smem(ring);
    int s = 0;
    unsigned par = 1;  // a fresh "empty" barrier lets the first nst waits through
    int issued = 0;
    bool ok = true;
    for (; issued < n_planes; ++issued) {
      ok = t3_mbar_wait(&sh.empty[s], par, &sh.abort_flag);
      if (!ok) break;
      t3_mbar_expect_tx(&sh.full[s], box_bytes);
      t3_tma_load_3d(ring_s + s * stride, &maps.map[bsel], &sh.full[s], bx0, by0, zbase + sh.plane[issued]);
      if (++s == nst) { s = 0; par ^= 1u; }
    }
    if (!ok) {
      sh.abort_flag = 1;
      if (p.status) atomicOr(p.status, STATUS_TMA_TIMEOUT);
      // stay until this CTA's copies in flight have landed (bounded), so that none writes into
      // shared memory that already belongs to another CTA
      for (int j = max(0, issued - nst); j < issued; ++j)
        t3_mbar_wait(&sh.full[j % nst], (unsigned)((j / nst) & 1), nullptr);
    }
    return;
  }

  // ================= consumer warps =================
  const unsigned row = (unsigned)(bw * esz);
  const unsigned char* pa = ring + (ina ? ((y0a - by0) * bw + (x0a - bx0)) * esz : 0);
  const unsigned char* pb = ring + (inb ? ((y0b - by0) * bw + (x0b - bx0)) * esz : 0);
  const typename Q::M mask = Q::make_mask(ina, inb);

  const long long plane_o = (long long)p.oh * p.ow;
  T* o = (T*)p.out + k.nc * p.ovol + (long long)k.pd0 * plane_o + (long long)(active ? ph : 0) * p.ow + (active ? pw0 : 0);
  const bool vec = L.vec_store && has_b;
  const V zero2 = Q::dup(A::fi(0));

  int s = 0;
  unsigned par = 0;
  unsigned soff = 0;      // s * stride
  unsigned newest = 1;    // parity of the schedule position of the newest plane read (starts "odd")
  V qe[4], qo[4];         // tap values of the planes at even / odd schedule positions
#pragma unroll
  for (int t = 0; t < 4; ++t) qe[t] = qo[t] = zero2;

  for (int i = 0; i < npd; ++i, o += plane_o) {
    const T3Ent<T> e = sh.ent[i];
    V val = zero2;
    if ((e.flags & T3_INSIDE) && any_inside) {  // uniform
      for (int a = 0; a < (int)e.adv; ++a) {
        if (!t3_mbar_wait(&sh.full[s], par, &sh.abort_flag)) {
          sh.abort_flag = 1;
          if (p.status && lane == 0) atomicOr(p.status, STATUS_TMA_TIMEOUT);
          return;  // no barrier follows: leaving is safe, the producer drains its copies
        }
        newest ^= 1u;
        if (newest) t3_read_plane<T>(pa + soff, pb + soff, row, qo);
        else t3_read_plane<T>(pa + soff, pb + soff, row, qe);
        __syncwarp();
        if (lane == 0) t3_mbar_arrive(&sh.empty[s]);  // this warp is done with the slot
        soff += stride;
        if (++s == nst) { s = 0; soff = 0; par ^= 1u; }
      }
      const bool same = (e.flags & T3_SAME) != 0;
      V acc;
      if (newest) {
        V older[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) older[t] = same ? qo[t] : qe[t];
        acc = t3_interp<T>(e.h, e.l, hy2, ly2, hx2, lx2, older, qo);
      } else {
        V older[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) older[t] = same ? qe[t] : qo[t];
        acc = t3_interp<T>(e.h, e.l, hy2, ly2, hx2, lx2, older, qe);
      }
      // output_val = 0 + val (normalises -0), then /count with count == 1
      val = Q::apply(Q::add(zero2, acc), mask);
    }
    if (vec) {
      Q::store2(o, val);
    } else if (active) {
      o[0] = Q::lo(val);
      if (has_b) o[1] = Q::hi(val);
    }
  }
}

// ---- host side ---------------------------------------------------------------------------

typedef CUresult (*T3EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point query (no link against libcuda)
inline T3EncodeTiled t3_encode_fn() {
  static T3EncodeTiled fn = []() -> T3EncodeTiled {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return (T3EncodeTiled)ptr;
  }();
  return fn;
}

// Tensor maps over the feature tensor viewed as (W, H, N*C*D), one per box size.
// Returns false when the tensor cannot be described (row pitch or base not 16-byte aligned, ...).
inline bool t3_make_maps(const Params& p, int dtype, T3Maps& m) {
  T3EncodeTiled enc = t3_encode_fn();
  if (!enc) return false;
  const size_t esz = dtype == 0 ? 4 : 2;
  const unsigned long long planes = (unsigned long long)p.N * p.C * p.D;
  if (((uintptr_t)p.in) % 16 != 0 || ((size_t)p.W * esz) % 16 != 0 || planes > 0x7fffffffULL) return false;
  // boxes in elements, ascending in area; every one fits kT3MaxBoxBytes
  // Box widths keep the row pitch at 8 or 24 (mod 32) four-byte words: the four rows a warp
  // reads then fall into different shared-memory banks.
  static const int half_boxes[][2] = {{48, 24}, {48, 32}, {48, 40}, {80, 40}, {80, 48}, {112, 48}};
  static const int float_boxes[][2] = {{40, 24}, {40, 32}, {56, 32}, {56, 40}, {72, 40}};
  const int (*boxes)[2] = dtype == 0 ? float_boxes : half_boxes;
  const int nb = dtype == 0 ? 5 : 6;
  const cuuint64_t gdim[3] = {(cuuint64_t)p.W, (cuuint64_t)p.H, (cuuint64_t)planes};
  const cuuint64_t gstride[2] = {(cuuint64_t)p.W * esz, (cuuint64_t)p.W * p.H * esz};
  const cuuint32_t estride[3] = {1, 1, 1};
  m.n = 0;
  for (int j = 0; j < nb; ++j) {
    const cuuint32_t box[3] = {(cuuint32_t)boxes[j][0], (cuuint32_t)boxes[j][1], 1};
    if ((size_t)box[0] * box[1] * esz > (size_t)kT3MaxBoxBytes) continue;
    CUresult r = enc(&m.map[m.n], dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                     const_cast<void*>(p.in), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    m.bw[m.n] = boxes[j][0];
    m.bh[m.n] = boxes[j][1];
    ++m.n;
  }
  return m.n > 0;
}

template <typename T>
inline size_t t3_dynamic_smem() { return (size_t)kT3RingBytes + sizeof(T3Shared<T>); }

// Picks the streaming kernel when the call has its shape; returns MVR_STREAM3D_NOT_APPLICABLE
// otherwise (the caller then uses the general kernel).
inline int try_launch_stream3d(const Params& p, int dtype, cudaStream_t st) {
  if (p.ndim != 3 || p.sampling_ratio != 1) return MVR_STREAM3D_NOT_APPLICABLE;
  if (dtype != 0 /*f32*/ && dtype != 1 /*f16*/) return MVR_STREAM3D_NOT_APPLICABLE;
  if (dtype == 0 && p.fm != kS3FloatPattern) return MVR_STREAM3D_NOT_APPLICABLE;
  // small outputs (detection heads) are better served one element per thread
  if (p.ovol < 4096 || p.ow < 8) return MVR_STREAM3D_NOT_APPLICABLE;
  if ((long long)p.H * p.W >= 0x7fffffffLL) return MVR_STREAM3D_NOT_APPLICABLE;

  S3Launch L;
  L.tiles_w = (p.ow + kS3TileW - 1) / kS3TileW;
  L.tiles_h = (p.oh + kS3TileH - 1) / kS3TileH;
  // depth chunk: long enough to amortise the per-thread set-up and to reuse planes, short
  // enough to give every SM several CTAs
  const long long per_depth_ctas = (long long)p.R * p.C * L.tiles_w * L.tiles_h;
  int chunk = kS3MaxChunk;
  while (chunk > 8 && per_depth_ctas * ((p.od + chunk - 1) / chunk) < 148LL * 12) chunk >>= 1;
  if (chunk > p.od) chunk = p.od;
  L.chunk = chunk;
  L.chunks = (p.od + chunk - 1) / chunk;
  const size_t esz = dtype == 0 ? 4 : 2;
  L.vec_store = ((p.ow & 1) == 0) && (((uintptr_t)p.out) % (2 * esz) == 0);
  const long long ctas = per_depth_ctas * L.chunks;
  if (ctas > 0x7fffffffLL) return MVR_STREAM3D_NOT_APPLICABLE;
  static const bool use_tma = getenv("MVR_NO_TMA") == nullptr;
  T3Maps maps;
  if (use_tma && t3_make_maps(p, dtype, maps)) {
    // more dynamic shared memory than the default limit: opt in (per function and device)
    if (dtype == 0) {
      cudaFuncSetAttribute(resample_fwd_stream3d_tma<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)t3_dynamic_smem<float>());
      resample_fwd_stream3d_tma<float><<<(unsigned)ctas, kT3Threads, t3_dynamic_smem<float>(), st>>>(p, L, maps);
    } else {
      cudaFuncSetAttribute(resample_fwd_stream3d_tma<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)t3_dynamic_smem<__half>());
      resample_fwd_stream3d_tma<__half><<<(unsigned)ctas, kT3Threads, t3_dynamic_smem<__half>(), st>>>(p, L, maps);
    }
  } else {
    if (dtype == 0) resample_fwd_stream3d<float><<<(unsigned)ctas, kS3Threads, 0, st>>>(p, L);
    else resample_fwd_stream3d<__half><<<(unsigned)ctas, kS3Threads, 0, st>>>(p, L);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

}  // namespace mvr
