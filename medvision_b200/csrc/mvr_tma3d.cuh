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
// Every CTA fetches its own boxes from this GPU's memory; no copy is shared between CTAs and
// there is no cluster launch.
#pragma once
#include <cuda.h>
#include <atomic>

#include "mvr_label.cuh"

namespace mvr {

enum { STATUS_TMA_TIMEOUT = 2 };

constexpr int kT3MaxStages = 16;      // ring slots (the ring itself is sized at launch)
constexpr int kT3MaxBoxBytes = 12800; // largest box; leaves three ring slots
constexpr int kT3MaxBoxes = 6;
constexpr int kT3MaxPlanes = 2 * kS3MaxChunk;
constexpr int kT3Threads = kS3Threads + 32;  // 8 consumer warps + 1 producer warp
constexpr int kT3Pairs = 2;                   // voxel pairs per consumer thread
constexpr int kT3RingBytes = 60 * 1024;       // plane ring of one CTA: what three resident CTAs per SM can share
static_assert(kT3RingBytes >= 3 * ((kT3MaxBoxBytes + 127) & ~127), "the ring must hold three of the largest boxes");

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
  unsigned short flags; // T3_INSIDE
};
enum { T3_INSIDE = 1 };

template <typename T>
struct T3Shared {
  S3Shared<T> s3;
  unsigned long long full[kT3MaxStages];   // producer -> consumers: the plane has landed
  unsigned long long empty[kT3MaxStages];  // consumers -> producer: every warp has read the plane
  int plane[kT3MaxPlanes];                 // plane schedule: source plane index, in order of use
  T3Ent<T> ent[kS3MaxChunk];
  int warp_tot[4];
  int box[4];                              // xmin, xmax, ymin, ymax over the tile's inside voxels
  volatile int abort_flag;
};

__device__ __forceinline__ unsigned t3_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void t3_mbar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(t3_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void t3_mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void t3_mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One try: the hardware suspends the thread until the phase completes or a system-dependent time limit
// passes (no issue slots are spent while suspended; in the common case the first try succeeds).
__device__ __forceinline__ bool t3_mbar_try_wait(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n"
      "  .reg .pred p;\n"
      "  mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "  selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait (producer side): false when `tries` tries did not see the phase complete or another
// thread of the CTA gave up.
__device__ __forceinline__ bool t3_mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag, unsigned tries) {
  if (t3_mbar_try_wait(bar, parity)) return true;
  for (unsigned t = 1; t < tries; ++t) {
    if (t3_mbar_try_wait(bar, parity)) return true;
    if ((t & 63u) == 0 && abort_flag && *abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ void t3_tma_load_3d(unsigned dst, const CUtensorMap* map, unsigned bar, int x, int y,
                                               int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}

// Two elements from two 32-bit shared-memory addresses, as the two lanes of a pair.
template <typename T>
__device__ __forceinline__ typename P2<T>::V t3_lds_pair(unsigned addr_a, unsigned addr_b);
template <>
__device__ __forceinline__ __half2 t3_lds_pair<__half>(unsigned addr_a, unsigned addr_b) {
  unsigned va, vb;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(va) : "r"(addr_a) : "memory");
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(vb) : "r"(addr_b) : "memory");
  const unsigned packed = __byte_perm(va, vb, 0x5410);
  return *reinterpret_cast<const __half2*>(&packed);
}
template <>
__device__ __forceinline__ Float2Lanes t3_lds_pair<float>(unsigned addr_a, unsigned addr_b) {
  Float2Lanes v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v.a) : "r"(addr_a) : "memory");
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v.b) : "r"(addr_b) : "memory");
  return v;
}

// Bounded wait written as one PTX loop (no divergence bookkeeping around it): up to `tries` tries, each
// of which the hardware may suspend.
__device__ __forceinline__ bool t3_mbar_wait_ptx(unsigned bar, unsigned parity, unsigned tries) {
  unsigned ok;
  asm volatile(
      "{\n"
      "  .reg .pred p, q;\n"
      "  .reg .u32 c;\n"
      "  mov.u32 c, 0;\n"
      "T3_WAIT_LOOP:\n"
      "  mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "  @p bra T3_WAIT_DONE;\n"
      "  add.u32 c, c, 1;\n"
      "  setp.lt.u32 q, c, %3;\n"
      "  @q bra T3_WAIT_LOOP;\n"
      "T3_WAIT_DONE:\n"
      "  selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(tries)
      : "memory");
  return ok != 0;
}
// lane 0 of the warp arrives; the others fall through (predicated, no branch)
__device__ __forceinline__ void t3_mbar_arrive_lane0(unsigned bar, int lane) {
  asm volatile(
      "{\n"
      "  .reg .pred p;\n"
      "  setp.eq.s32 p, %1, 0;\n"
      "  @p mbarrier.arrive.shared::cta.b64 _, [%0];\n"
      "}\n" ::"r"(bar), "r"(lane)
      : "memory");
}

// The rare ways out of the plane-streaming kernel (batch index outside the batch, coordinates that
// are not finite, a tile whose footprint exceeds every box): the CTA's tile, 16 rows at a time,
// through the gather path.
template <typename T>
__device__ __forceinline__ void t3_fallback(const Params& p, const S3Launch& L, const S3Cta& k, S3Shared<T>& sh, int np) {
  if (threadIdx.x >= kS3Threads) return;
  for (int q = 0; q < np; ++q) {
    S3Cta k2 = k;
    k2.th = k.th * np + q;
    if (k2.th * kS3TileH < p.oh) s3_body_l1<T>(p, L, k2, sh);
  }
}

// NP = voxel pairs per thread: pair q sits 16*q output rows below pair 0, so a CTA covers a
// 32 (w) x 16*NP (h) tile.  More work per thread spreads the per-depth control (table read, ring
// hand-shake, loop) over more voxels.
// VEC: even output width and aligned pointer, every stored pair is one vector store.
template <typename T, int NP, bool VEC>
__device__ __forceinline__ void t3_body(const Params& p, const S3Launch& L, const T3Maps& maps) {
  typedef Ar<T> A;
  typedef P2<T> Q;
  typedef typename Q::V V;
  extern __shared__ __align__(128) unsigned char t3_dyn[];
  unsigned char* ring = t3_dyn;  // kT3RingBytes, 128-byte aligned
  T3Shared<T>& sh = *reinterpret_cast<T3Shared<T>*>(t3_dyn + kT3RingBytes);

  const S3Cta k = s3_cta(p, L);  // k.th counts tiles of 16*NP rows here
  if (s3_filtered_out<T>(p, L, k)) return;
  if (threadIdx.x == 0) {
    sh.box[0] = 0x7fffffff; sh.box[1] = -0x7fffffff; sh.box[2] = 0x7fffffff; sh.box[3] = -0x7fffffff;
    sh.abort_flag = 0;
  }
  s3_prologue<T>(p, k, sh.s3);  // ends with __syncthreads()
  const RoiGeom<T>& g = sh.s3.g;
  const bool bad_batch = (g.batch < 0 || g.batch >= p.N);
  if (bad_batch || !sh.s3.zsep) {  // CTA-uniform: zeros and the status bit / coordinates that are not finite
    t3_fallback<T>(p, L, k, sh.s3, NP);
    return;
  }

  const int fm = kS3FloatPattern;
  const bool rotated = (p.kind == KIND_ROTATED);
  const int npd = k.npd;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool consumer = warp < kS3Threads / 32;
  const int pw0 = k.tw * kS3TileW + (warp & 1) * 16 + (lane & 7) * 2;
  const int ph0 = k.th * (kS3TileH * NP) + (warp >> 1) * 4 + (lane >> 3);
  const bool col_ok = consumer && pw0 < p.ow;
  const bool has_b = col_ok && (pw0 + 1 < p.ow);

  // ---- in-plane position, taps and weights of the 2*NP voxels: once per thread
  int x0a[NP], x0b[NP], y0a[NP], y0b[NP];
  bool ina[NP], inb[NP], act[NP];
  V lx2[NP], hx2[NP], ly2[NP], hy2[NP];
  {
    const T sub_x = lattice_sub<T>(g.bin[0], 0, 1), sub_y = lattice_sub<T>(g.bin[1], 0, 1);
    const int pwa = col_ok ? pw0 : 0, pwb = has_b ? pw0 + 1 : pwa;
    const T xa = A::add(lattice_base<T>(g.start[0], pwa, g.bin[0], fm), sub_x);
    const T xb = A::add(lattice_base<T>(g.start[0], pwb, g.bin[0], fm), sub_x);
    const V x2 = Q::make(xa, xb);
#pragma unroll
    for (int q = 0; q < NP; ++q) {
      const int ph = ph0 + q * kS3TileH;
      act[q] = col_ok && ph < p.oh;
      const T y = A::add(lattice_base<T>(g.start[1], act[q] ? ph : 0, g.bin[1], fm), sub_y);
      V rx2, ry2;
      if (rotated) {
        rx2 = Q::add(Q::row_xy(Q::dup(g.rot[0]), x2, Q::dup(A::mul(g.rot[1], y))), Q::dup(g.centre[0]));
        ry2 = Q::add(Q::row_xy(Q::dup(g.rot[3]), x2, Q::dup(A::mul(g.rot[4], y))), Q::dup(g.centre[1]));
      } else {
        rx2 = x2;
        ry2 = Q::dup(y);
      }
      AxisTap<T> txa, txb, tya, tyb;
      ina[q] = act[q] && !(axis_outside<T>(Q::lo(ry2), p.H) || axis_outside<T>(Q::lo(rx2), p.W));
      inb[q] = act[q] && has_b && !(axis_outside<T>(Q::hi(ry2), p.H) || axis_outside<T>(Q::hi(rx2), p.W));
      axis_tap<T>(Q::lo(rx2), p.W, txa);
      axis_tap<T>(Q::hi(rx2), p.W, txb);
      axis_tap<T>(Q::lo(ry2), p.H, tya);
      axis_tap<T>(Q::hi(ry2), p.H, tyb);
      if (p.order == 0) {
        nearest_axis<T>(txa.l, txa.h); nearest_axis<T>(txb.l, txb.h);
        nearest_axis<T>(tya.l, tya.h); nearest_axis<T>(tyb.l, tyb.h);
      }
      x0a[q] = txa.i0; x0b[q] = txb.i0; y0a[q] = tya.i0; y0b[q] = tyb.i0;
      lx2[q] = Q::make(txa.l, txb.l); hx2[q] = Q::make(txa.h, txb.h);
      ly2[q] = Q::make(tya.l, tyb.l); hy2[q] = Q::make(tya.h, tyb.h);
    }
  }

  // ---- bounding box of the tile's base taps (inside voxels only)
  {
    int xmin = 0x7fffffff, xmax = -0x7fffffff, ymin = 0x7fffffff, ymax = -0x7fffffff;
#pragma unroll
    for (int q = 0; q < NP; ++q) {
      if (ina[q]) { xmin = min(xmin, x0a[q]); xmax = max(xmax, x0a[q]); ymin = min(ymin, y0a[q]); ymax = max(ymax, y0a[q]); }
      if (inb[q]) { xmin = min(xmin, x0b[q]); xmax = max(xmax, x0b[q]); ymin = min(ymin, y0b[q]); ymax = max(ymax, y0b[q]); }
    }
    xmin = __reduce_min_sync(0xffffffffu, xmin); xmax = __reduce_max_sync(0xffffffffu, xmax);
    ymin = __reduce_min_sync(0xffffffffu, ymin); ymax = __reduce_max_sync(0xffffffffu, ymax);
    if (lane == 0 && xmin <= xmax) {
      atomicMin(&sh.box[0], xmin); atomicMax(&sh.box[1], xmax);
      atomicMin(&sh.box[2], ymin); atomicMax(&sh.box[3], ymax);
    }
  }

  // ---- plane schedule, in parallel over the depths of the chunk.
  // A warp keeps the tap values of two planes in registers: "older" and "newest".  After depth
  // i-1 they are (z0, z1) of that depth.  Depth i then needs, with (z0, z1) its own planes:
  //   nothing new          if (z0, z1) equals what is held;
  //   one new plane (z1)   if z0 is the newest held plane (the usual step along z);
  //   two new planes       otherwise (first depth, a jump, or any unusual order).
  // Thread i decides this from depths i-1 and i alone; a prefix sum over the counts gives every
  // new plane its position in the schedule that the producer follows.
  {
    const int i = threadIdx.x;
    int adv = 0, z_first = 0, z_second = 0;
    if (i < npd) {
      const S3ZTap<T> e = sh.s3.zt[i];
      T3Ent<T> t;
      t.h = e.h; t.l = e.l; t.flags = 0;
      if (e.inside) {
        adv = 2;
        if (i > 0 && sh.s3.zt[i - 1].inside) {
          const int pz0 = sh.s3.zt[i - 1].z0, pz1 = sh.s3.zt[i - 1].z1;
          if (e.z0 == pz0 && e.z1 == pz1) adv = 0;
          else if (e.z0 == pz1) adv = 1;
        }
        z_first = (adv == 2) ? e.z0 : e.z1;
        z_second = e.z1;
        t.flags = T3_INSIDE;
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
    if (bsel < 0) {  // the tile's footprint exceeds every box: plain loads
      t3_fallback<T>(p, L, k, sh.s3, NP);
      return;
    }
  }
  const int bw = any_inside ? maps.bw[bsel] : 0, bh = any_inside ? maps.bh[bsel] : 0;
  const int n_planes = any_inside ? sh.warp_tot[0] + sh.warp_tot[1] + sh.warp_tot[2] + sh.warp_tot[3] : 0;
  const unsigned box_bytes = (unsigned)(bw * bh * esz);
  // (passed through a warp reduction: the compiler then knows the value is the same in every lane and can keep
  // slot offsets in uniform registers)
  const unsigned stride = __reduce_max_sync(0xffffffffu, (box_bytes + 127u) & ~127u);
  const int nst = any_inside ? min(kT3MaxStages, (int)((unsigned)kT3RingBytes / stride)) : 1;  // >= 4
  const unsigned ring_s = t3_smem(ring);
  const unsigned full_s = t3_smem(&sh.full[0]), empty_s = t3_smem(&sh.empty[0]);

  if (!consumer) {
    // ================= producer warp: one lane feeds the ring =================
    if (lane != 0) return;
    const int zbase = (g.batch * p.C + k.c) * p.D;  // index of the volume's first plane in (N*C*D)
    int s = 0;
    unsigned par = 1;  // a fresh "empty" barrier lets the first nst waits through
    int issued = 0;
    bool ok = true;
    for (; issued < n_planes; ++issued) {
      ok = t3_mbar_wait(empty_s + 8u * s, par, &sh.abort_flag, L.wait_tries);
      if (!ok) break;
      if (issued != L.skip_plane) {  // self-test of the bounded waits: the left-out plane never arrives
        t3_mbar_expect_tx(full_s + 8u * s, box_bytes);
        t3_tma_load_3d(ring_s + s * stride, &maps.map[bsel], full_s + 8u * s, bx0, by0, zbase + sh.plane[issued]);
      }
      if (++s == nst) { s = 0; par ^= 1u; }
    }
    if (!ok) {
      sh.abort_flag = 1;
      if (p.status) atomicOr(p.status, STATUS_TMA_TIMEOUT);
      // stay until this CTA's copies in flight have landed (bounded), so that none writes into
      // shared memory that already belongs to another CTA
      for (int j = max(0, issued - nst); j < issued; ++j)
        if (j != L.skip_plane) t3_mbar_wait(full_s + 8u * (j % nst), (unsigned)((j / nst) & 1), nullptr, L.wait_tries);
    }
    return;
  }

  // ================= consumer warps =================
  const unsigned row = (unsigned)(bw * esz);
  unsigned oa[NP], ob[NP];  // shared-memory addresses of the base taps in ring slot 0
  typename Q::M mask[NP];
#pragma unroll
  for (int q = 0; q < NP; ++q) {
    oa[q] = ring_s + (ina[q] ? (unsigned)(((y0a[q] - by0) * bw + (x0a[q] - bx0)) * esz) : 0u);
    ob[q] = ring_s + (inb[q] ? (unsigned)(((y0b[q] - by0) * bw + (x0b[q] - bx0)) * esz) : 0u);
    mask[q] = Q::make_mask(ina[q], inb[q]);
  }

  const long long plane_o = (long long)p.oh * p.ow;
  const long long sub_o = (long long)kS3TileH * p.ow;  // output offset between a thread's pairs
  T* o = (T*)p.out + k.nc * p.ovol + (long long)k.pd0 * plane_o +
         (long long)(act[0] ? ph0 : 0) * p.ow + (col_ok ? pw0 : 0);
  const V zero2 = Q::dup(A::fi(0));

  unsigned soff = 0;                      // byte offset of the current ring slot
  unsigned fa = full_s, ea = empty_s;     // its two mbarriers
  const unsigned ring_end = stride * nst;
  unsigned par = 0;
  // Tap values of the two planes held in registers (lanes = the two voxels): x0y0, x1y0, x0y1,
  // x1y1.  Which of the two sets is the newest plane alternates with every fetch; `b_newest`
  // tracks it, and the code below exists once per role assignment, so no register is ever moved.
  V ra[NP][4], rb[NP][4];
#pragma unroll
  for (int q = 0; q < NP; ++q)
#pragma unroll
    for (int t = 0; t < 4; ++t) ra[q][t] = rb[q][t] = zero2;
  bool b_newest = true;
  const unsigned tries = L.wait_tries;

// take the next plane of the schedule out of the ring into register set R
#define T3_FETCH(R)                                                                       \
  {                                                                                       \
    if (!t3_mbar_wait_ptx(fa, par, tries)) {                                              \
      sh.abort_flag = 1;                                                                  \
      if (p.status && lane == 0) atomicOr(p.status, STATUS_TMA_TIMEOUT);                  \
      return; /* no barrier follows: leaving is safe, the producer drains its copies */   \
    }                                                                                     \
    _Pragma("unroll") for (int q = 0; q < NP; ++q) {                                      \
      const unsigned ua = oa[q] + soff, ub = ob[q] + soff;                                \
      R[q][0] = t3_lds_pair<T>(ua, ub);                                                   \
      R[q][1] = t3_lds_pair<T>(ua + esz, ub + esz);                                       \
      R[q][2] = t3_lds_pair<T>(ua + row, ub + row);                                       \
      R[q][3] = t3_lds_pair<T>(ua + row + esz, ub + row + esz);                           \
    }                                                                                     \
    __syncwarp();                                                                         \
    t3_mbar_arrive_lane0(ea, lane); /* this warp is done with the slot */                 \
    soff += stride; fa += 8u; ea += 8u;                                                   \
    if (soff == ring_end) { soff = 0; fa = full_s; ea = empty_s; par ^= 1u; }             \
  }

// the reference's tap sum: older plane OLD supplies taps 1-4, newest plane NEW taps 5-8
#define T3_COMPUTE(OLD, NEW)                                                              \
  {                                                                                       \
    const V hz2 = Q::dup(e.h), lz2 = Q::dup(e.l);                                         \
    _Pragma("unroll") for (int q = 0; q < NP; ++q) {                                      \
      const V hzhy = Q::mul(hz2, hy2[q]), hzly = Q::mul(hz2, ly2[q]);                     \
      const V lzhy = Q::mul(lz2, hy2[q]), lzly = Q::mul(lz2, ly2[q]);                     \
      V acc = Q::tap_first(Q::mul(hzhy, hx2[q]), OLD[q][0], Q::mul(hzhy, lx2[q]), OLD[q][1]); \
      acc = Q::tap_next(acc, Q::mul(hzly, hx2[q]), OLD[q][2]);                            \
      acc = Q::tap_next(acc, Q::mul(hzly, lx2[q]), OLD[q][3]);                            \
      acc = Q::tap_next(acc, Q::mul(lzhy, hx2[q]), NEW[q][0]);                            \
      acc = Q::tap_next(acc, Q::mul(lzhy, lx2[q]), NEW[q][1]);                            \
      acc = Q::tap_next(acc, Q::mul(lzly, hx2[q]), NEW[q][2]);                            \
      acc = Q::tap_next(acc, Q::mul(lzly, lx2[q]), NEW[q][3]);                            \
      /* output_val = 0 + val (normalises -0), then /count with count == 1 */             \
      val[q] = Q::apply(Q::add(zero2, acc), mask[q]);                                     \
    }                                                                                     \
  }

#define T3_DEPTH_LOOP(STORE)                                                              \
  for (int i = 0; i < npd; ++i, o += plane_o) {                                           \
    const T3Ent<T> e = sh.ent[i];                                                         \
    V val[NP];                                                                            \
    _Pragma("unroll") for (int q = 0; q < NP; ++q) val[q] = zero2;                        \
    if (e.flags && any_inside) { /* uniform */                                            \
      if (b_newest) {                                                                     \
        if (e.adv == 1) { T3_FETCH(ra); b_newest = false; T3_COMPUTE(rb, ra); }           \
        else { if (e.adv == 2) { T3_FETCH(ra); T3_FETCH(rb); } T3_COMPUTE(ra, rb); }      \
      } else {                                                                            \
        if (e.adv == 1) { T3_FETCH(rb); b_newest = true; T3_COMPUTE(ra, rb); }            \
        else { if (e.adv == 2) { T3_FETCH(rb); T3_FETCH(ra); } T3_COMPUTE(rb, ra); }      \
      }                                                                                   \
    }                                                                                     \
    _Pragma("unroll") for (int q = 0; q < NP; ++q) { STORE }                              \
  }

  if (VEC) {
    T3_DEPTH_LOOP(if (act[q]) Q::store2(o + q * sub_o, val[q]);)
  } else {
    T3_DEPTH_LOOP(if (act[q]) { T* oq = o + q * sub_o; oq[0] = Q::lo(val[q]); if (has_b) oq[1] = Q::hi(val[q]); })
  }
#undef T3_DEPTH_LOOP
#undef T3_COMPUTE
#undef T3_FETCH
}

template <typename T, int NP, bool VEC>
__global__ void __launch_bounds__(kT3Threads, 3)
resample_fwd_stream3d_tma(const Params p, const S3Launch L, const __grid_constant__ T3Maps maps) {
  t3_body<T, NP, VEC>(p, L, maps);
  // This grid may have been started before the gather launch ahead of it in the stream has finished
  // (programmatic dependent launch).  One thread waits for that launch before the grid ends, so that
  // the completion of this grid implies the completion of both, whatever follows in the stream.
  if (blockIdx.x == 0 && threadIdx.x == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
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
  static const int half_boxes[][2] = {{48, 40}, {48, 48}, {80, 40}, {80, 56}, {80, 72}, {112, 56}};
  static const int float_boxes[][2] = {{40, 40}, {56, 40}, {56, 56}, {72, 40}};
  const int (*boxes)[2] = dtype == 0 ? float_boxes : half_boxes;
  const int nb = dtype == 0 ? 4 : 6;
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

// Self-test hook (mvr_selftest_tma_skip_plane): schedule index of a plane that the producers of the next
// plane-streaming launches leave out, so that the consumers' bounded waits run out; -1 = off.
inline std::atomic<int> g_t3_selftest_skip_plane{-1};

// A label field to be resampled along with an image (same rois, given in float32; see mvr_label.cuh).
struct T3LabelJob {
  Params p;        // in = labels, rois = float32 rois, out = int32 result, order 0, sampling_ratio 1
  int label_dtype; // LABEL_*
  bool done;       // set when the label items rode along with the image's gather launch
};

// Picks the streaming kernel when the call has its shape; returns MVR_STREAM3D_NOT_APPLICABLE
// otherwise (the caller then uses the general kernel).  `label`: optional label job of the same call.
inline int try_launch_stream3d(const Params& p, int dtype, cudaStream_t st, T3LabelJob* label = nullptr) {
  if (p.ndim != 3 || p.sampling_ratio != 1 || p.order > 1) return MVR_STREAM3D_NOT_APPLICABLE;
  if (dtype != 0 /*f32*/ && dtype != 1 /*f16*/) return MVR_STREAM3D_NOT_APPLICABLE;
  if (dtype == 0 && p.fm != kS3FloatPattern) return MVR_STREAM3D_NOT_APPLICABLE;
  // small outputs (detection heads) are better served one element per thread
  if (p.ovol < 4096 || p.ow < 8) return MVR_STREAM3D_NOT_APPLICABLE;
  if (p.vol >= 0x7fffffffLL) return MVR_STREAM3D_NOT_APPLICABLE;           // 32-bit offsets inside a volume
  if (dtype == 1 && (p.D > 2048 || p.H > 2048 || p.W > 2048)) return MVR_STREAM3D_NOT_APPLICABLE;  // sizes as half values

  T3Maps maps;
  const bool tma = t3_make_maps(p, dtype, maps);
  const int pairs = kT3Pairs;
  const size_t esz = dtype == 0 ? 4 : 2;

  // ---- geometry of the gather kernel (plain loads through L1): 32 x 16 tiles, short depth chunks.
  // Rois under a general rotation are bound by load latency and want many CTAs.  Measured on
  // RandomAffine 16 x 128^3 with three-axis rotations: 8 depths per CTA 329 us, 16: 365, 32: 430,
  // 64: 725.
  S3Launch G;
  G.tiles_w = (p.ow + kS3TileW - 1) / kS3TileW;
  G.tiles_h = (p.oh + kS3TileH - 1) / kS3TileH;
  const long long g_per_depth = (long long)p.R * p.C * G.tiles_w * G.tiles_h;
  {
    int chunk = kS3MaxChunk;
    while (chunk > 8 && g_per_depth * ((p.od + chunk - 1) / chunk) < 148LL * 16) chunk >>= 1;
    G.chunk = min(chunk, p.od);
  }
  G.chunks = (p.od + G.chunk - 1) / G.chunk;
  G.vec_store = ((p.ow & 1) == 0) && (((uintptr_t)p.out) % (2 * esz) == 0);
  G.filter = 0;
  const long long g_ctas = g_per_depth * G.chunks;
  if (g_ctas > 0x7fffffffLL) return MVR_STREAM3D_NOT_APPLICABLE;
  if (!tma) {
    if (dtype == 0) resample_fwd_stream3d<float><<<(unsigned)g_ctas, kS3Threads, 0, st>>>(p, G);
    else resample_fwd_stream3d<__half><<<(unsigned)g_ctas, kS3Threads, 0, st>>>(p, G);
    return cudaGetLastError() == cudaSuccess ? 0 : -8;
  }

  // ---- geometry of the plane-streaming kernel: 32 x 16*pairs tiles, long depth chunks.
  // The set-up of a CTA costs about as much as five depths, so: the fewest chunks that still give
  // every SM about five CTAs.  Measured on Resize 4 x (160,512,512) -> (128,256,256): 43 depths
  // per CTA 83 us, 26: 84, 64: 87, 16: 91; on 96^3 crops one chunk of 96 beats two of 48 by 9 %.
  S3Launch L;
  L.tiles_w = G.tiles_w;
  L.tiles_h = (p.oh + kS3TileH * pairs - 1) / (kS3TileH * pairs);
  const long long per_depth_ctas = (long long)p.R * p.C * L.tiles_w * L.tiles_h;
  {
    long long want = (148LL * 5 + per_depth_ctas - 1) / per_depth_ctas;
    want = std::max<long long>(want, (p.od + kS3MaxChunk - 1) / kS3MaxChunk);
    want = std::min<long long>(want, std::max(1, p.od / 8));
    int chunk = (int)((p.od + want - 1) / want);
    L.chunk = chunk;
  }
  L.chunks = (p.od + L.chunk - 1) / L.chunk;
  L.vec_store = G.vec_store;
  const long long ctas = per_depth_ctas * L.chunks;
  if (ctas > 0x7fffffffLL) return MVR_STREAM3D_NOT_APPLICABLE;
  L.skip_plane = g_t3_selftest_skip_plane.load();
  if (L.skip_plane >= 0) L.wait_tries = 32;  // self-test of the bounded waits: short limits
  // axis-aligned boxes have no rotation: one launch; rotated rois: this launch takes those that turn
  // about z at most, the gather launch below takes the rest
  const bool two = (p.kind == KIND_ROTATED);
  L.filter = two ? 1 : 0;
  G.filter = 2;
  // The gather launch goes first and lets its dependents start as soon as its CTAs are resident
  // (programmatic dependent launch); the plane-streaming launch is that dependent and waits for
  // nothing, since the two write disjoint rois.  When no roi is under a general rotation the
  // gather CTAs are gone after a few loads and the two launches cost one kernel boundary, not two.
  bool overlap = false;
  if (two) {
    if (p.R <= kS3RestMaxRois) {
      static int occ[2] = {0, 0};  // resident CTAs per SM of the two instantiations
      if (occ[dtype] == 0) {
        int n = 0;
        if (dtype == 0) cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, resample_fwd_stream3d_rest<float>, kS3Threads, 0);
        else cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, resample_fwd_stream3d_rest<__half>, kS3Threads, 0);
        occ[dtype] = n > 0 ? n : 1;
      }
      G.filter = 0;
      S3Launch Ll;
      long long items_l = 0;
      if (label && label_stream3d_geometry(label->p, Ll, items_l)) {
        const unsigned grid = (unsigned)std::min<long long>(std::max(g_ctas, items_l), 148LL * occ[dtype]);
#define T3_REST_LABEL(TYPE, IT) \
  resample_fwd_stream3d_rest_label<TYPE, IT><<<grid, kS3Threads, 0, st>>>(p, G, g_ctas, label->p, Ll, items_l)
#define T3_REST_LABEL_T(TYPE)                                              \
  switch (label->label_dtype) {                                            \
    case LABEL_U8: T3_REST_LABEL(TYPE, unsigned char); break;              \
    case LABEL_I16: T3_REST_LABEL(TYPE, short); break;                     \
    case LABEL_I32: T3_REST_LABEL(TYPE, int); break;                       \
    default: T3_REST_LABEL(TYPE, long long); break;                        \
  }
        if (dtype == 0) T3_REST_LABEL_T(float) else T3_REST_LABEL_T(__half)
#undef T3_REST_LABEL_T
#undef T3_REST_LABEL
        label->done = true;
      } else {
        const unsigned grid = (unsigned)std::min<long long>(g_ctas, 148LL * occ[dtype]);
        if (dtype == 0) resample_fwd_stream3d_rest<float><<<grid, kS3Threads, 0, st>>>(p, G, g_ctas);
        else resample_fwd_stream3d_rest<__half><<<grid, kS3Threads, 0, st>>>(p, G, g_ctas);
      }
      overlap = true;
    } else {
      if (dtype == 0) resample_fwd_stream3d<float><<<(unsigned)g_ctas, kS3Threads, 0, st>>>(p, G);
      else resample_fwd_stream3d<__half><<<(unsigned)g_ctas, kS3Threads, 0, st>>>(p, G);
    }
    if (cudaGetLastError() != cudaSuccess) return -8;
  }
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ctas);
  cfg.blockDim = dim3(kT3Threads);
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = overlap ? 1 : 0;
  cudaError_t err = cudaSuccess;
  // more dynamic shared memory than the default limit: opt in (per function and device)
#define T3_LAUNCH_V(TYPE, NP, VEC)                                                                           \
  {                                                                                                          \
    cfg.dynamicSmemBytes = t3_dynamic_smem<TYPE>();                                              \
    cudaFuncSetAttribute(resample_fwd_stream3d_tma<TYPE, NP, VEC>,                                           \
                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cfg.dynamicSmemBytes);            \
    err = cudaLaunchKernelEx(&cfg, resample_fwd_stream3d_tma<TYPE, NP, VEC>, p, L, maps);                    \
  }
#define T3_LAUNCH(TYPE, NP)                                                                                  \
  {                                                                                                          \
    if (L.vec_store) T3_LAUNCH_V(TYPE, NP, true) else T3_LAUNCH_V(TYPE, NP, false)                           \
  }
  if (dtype == 0) {
    if (pairs == 2) T3_LAUNCH(float, 2) else T3_LAUNCH(float, 1)
  } else {
    if (pairs == 2) T3_LAUNCH(__half, 2) else T3_LAUNCH(__half, 1)
  }
#undef T3_LAUNCH
#undef T3_LAUNCH_V
  if (err != cudaSuccess) return -8;
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

}  // namespace mvr
