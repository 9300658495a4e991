// Streaming backward kernel for dense 3D resampling (sampling_ratio == 1): the transpose of
// mvr_stream3d.cuh.  Same tiling (CTA = 32 x 16 output positions x a depth chunk of one
// (roi, channel), two w-adjacent voxels per thread), same coordinate arithmetic, and for every
// output voxel the eight products grad_out * w_k -- rounded to the element type exactly as the
// reference forms them (medvision/csrc/cuda/roi_align_rotated_3d_cuda_kernel.cuh:242-260; the
// division by count is a division by one here) -- are scattered with reductions.
//
// Accumulation: the reference adds into grad_in with atomics in the ELEMENT type, in whatever
// order the hardware serves them.  Float gradients are accumulated the same way (fp32
// reductions straight into grad_in).  Half gradients are accumulated in FLOAT in a scratch
// volume of the same shape and rounded to half once at the end: half atomics are slow, and a
// half running sum loses the small contributions that up-sampling produces by the dozen per
// voxel.  The result differs from any one run of the reference by less than two runs of the
// reference differ from each other.
#pragma once
#include <mutex>

#include "mvr_stream3d.cuh"

namespace mvr {

template <typename T> struct BwdAcc;
template <> struct BwdAcc<float> { typedef float type; };
template <> struct BwdAcc<__half> { typedef float type; };

// a tap row's two x-neighbours into the float accumulator volume [lo, hi): see atomic_add_pair
__device__ __forceinline__ void bwd_red_row(float* p0, float* p1, float v0, float v1, const float* lo, const float* hi) {
  atomic_add_pair(p0, p1, v0, v1, lo, hi);
}

template <typename T>
__global__ void __launch_bounds__(kS3Threads)
resample_bwd_stream3d(const Params p, const S3Launch L, typename BwdAcc<T>::type* __restrict__ acc_base) {
  typedef Ar<T> A;
  typedef P2<T> Q;
  typedef typename Q::V V;
  typedef typename BwdAcc<T>::type Acc;
  __shared__ S3Shared<T> sh;
  const S3Cta k = s3_cta(p, L);
  s3_prologue<T>(p, k, sh);
  const RoiGeom<T>& g = sh.g;
  const int fm = kS3FloatPattern;
  const bool zsep = sh.zsep != 0;
  const bool rotated = (p.kind == KIND_ROTATED);
  if (g.batch < 0 || g.batch >= p.N) {
    if (p.status && threadIdx.x == 0 && k.tw == 0 && k.th == 0 && k.ck == 0) atomicOr(p.status, STATUS_BAD_BATCH_INDEX);
    return;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pw0 = k.tw * kS3TileW + (warp & 1) * 16 + (lane & 7) * 2;
  const int ph = k.th * kS3TileH + (warp >> 1) * 4 + (lane >> 3);
  if (ph >= p.oh || pw0 >= p.ow) return;
  const bool has_b = (pw0 + 1 < p.ow);
  const long long plane_o = (long long)p.oh * p.ow;
  const T* go = (const T*)p.in + k.nc * p.ovol + (long long)k.pd0 * plane_o + (long long)ph * p.ow + pw0;
  Acc* acc = acc_base + ((long long)g.batch * p.C + k.c) * p.vol;
  const Acc* const acc_lo = acc_base;
  const Acc* const acc_hi = acc_base + (long long)p.N * p.C * p.vol;
  const long long HW = (long long)p.H * p.W;

  const T sub_x = lattice_sub<T>(g.bin[0], 0, 1), sub_y = lattice_sub<T>(g.bin[1], 0, 1);
  const T xa = A::add(lattice_base<T>(g.start[0], pw0, g.bin[0], fm), sub_x);
  const T xb = A::add(lattice_base<T>(g.start[0], has_b ? pw0 + 1 : pw0, g.bin[0], fm), sub_x);
  const T y = A::add(lattice_base<T>(g.start[1], ph, g.bin[1], fm), sub_y);
  const V x2 = Q::make(xa, xb);

  if (zsep) {
    // in-plane taps and weights: once per thread
    V rx2, ry2;
    if (rotated) {
      rx2 = Q::add(Q::row_xy(Q::dup(g.rot[0]), x2, Q::dup(A::mul(g.rot[1], y))), Q::dup(g.centre[0]));
      ry2 = Q::add(Q::row_xy(Q::dup(g.rot[3]), x2, Q::dup(A::mul(g.rot[4], y))), Q::dup(g.centre[1]));
    } else {
      rx2 = x2;
      ry2 = Q::dup(y);
    }
    AxisTap<T> txa, txb, tya, tyb;
    const bool ina = !(axis_outside<T>(Q::lo(ry2), p.H) || axis_outside<T>(Q::lo(rx2), p.W));
    const bool inb = has_b && !(axis_outside<T>(Q::hi(ry2), p.H) || axis_outside<T>(Q::hi(rx2), p.W));
    axis_tap<T>(Q::lo(rx2), p.W, txa);
    axis_tap<T>(Q::hi(rx2), p.W, txb);
    axis_tap<T>(Q::lo(ry2), p.H, tya);
    axis_tap<T>(Q::hi(ry2), p.H, tyb);
    if (p.order == 0) {
      nearest_axis<T>(txa.l, txa.h); nearest_axis<T>(txb.l, txb.h);
      nearest_axis<T>(tya.l, tya.h); nearest_axis<T>(tyb.l, tyb.h);
    }
    const int oa[4] = {tya.i0 * p.W + txa.i0, tya.i0 * p.W + txa.i1, tya.i1 * p.W + txa.i0, tya.i1 * p.W + txa.i1};
    const int ob[4] = {tyb.i0 * p.W + txb.i0, tyb.i0 * p.W + txb.i1, tyb.i1 * p.W + txb.i0, tyb.i1 * p.W + txb.i1};
    const V lx2 = Q::make(txa.l, txb.l), hx2 = Q::make(txa.h, txb.h);
    const V ly2 = Q::make(tya.l, tyb.l), hy2 = Q::make(tya.h, tyb.h);
    // Along the depth walk consecutive outputs mostly share a source plane (the upper plane of one
    // depth is the lower plane of the next, or both planes repeat when up-sampling): the
    // contributions to the two planes in hand are summed in float registers and go to memory
    // once, when the walk leaves the plane.
    float acc0[8], acc1[8];  // [0..3] voxel a, [4..7] voxel b; taps x0y0, x1y0, x0y1, x1y1
#pragma unroll
    for (int t = 0; t < 8; ++t) acc0[t] = acc1[t] = 0.0f;
    long long held0 = -1, held1 = -1;  // plane offsets of acc0 / acc1, -1: nothing held
    auto flush = [&](const float* a, long long plane) {
      if (plane < 0) return;
      Acc* pl = acc + plane;
      if (ina) {
        bwd_red_row(pl + oa[0], pl + oa[1], a[0], a[1], acc_lo, acc_hi);
        bwd_red_row(pl + oa[2], pl + oa[3], a[2], a[3], acc_lo, acc_hi);
      }
      if (inb) {
        bwd_red_row(pl + ob[0], pl + ob[1], a[4], a[5], acc_lo, acc_hi);
        bwd_red_row(pl + ob[2], pl + ob[3], a[6], a[7], acc_lo, acc_hi);
      }
    };
    for (int i = 0; i < k.npd; ++i) {
      const S3ZTap<T> e = sh.zt[i];
      if (!e.inside) continue;
      const T ga = go[i * plane_o];
      const T gb = has_b ? go[i * plane_o + 1] : A::fi(0);
      const V g2 = Q::make(ga, gb);
      const V hz2 = Q::dup(e.h), lz2 = Q::dup(e.l);
      const V hzhy = Q::mul(hz2, hy2), hzly = Q::mul(hz2, ly2);
      const V lzhy = Q::mul(lz2, hy2), lzly = Q::mul(lz2, ly2);
      // g_k = grad * w_k, each product rounded
      const V w[8] = {Q::mul(hzhy, hx2), Q::mul(hzhy, lx2), Q::mul(hzly, hx2), Q::mul(hzly, lx2),
                      Q::mul(lzhy, hx2), Q::mul(lzhy, lx2), Q::mul(lzly, hx2), Q::mul(lzly, lx2)};
      float c0[8], c1[8];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const V lo = Q::mul(g2, w[t]), hi = Q::mul(g2, w[4 + t]);
        c0[t] = A::tof(Q::lo(lo)); c0[4 + t] = A::tof(Q::hi(lo));
        c1[t] = A::tof(Q::lo(hi)); c1[4 + t] = A::tof(Q::hi(hi));
      }
      if (e.o0 == held0 && e.o1 == held1) {  // CTA-uniform
#pragma unroll
        for (int t = 0; t < 8; ++t) { acc0[t] += c0[t]; acc1[t] += c1[t]; }
      } else if (e.o0 == held1) {
        flush(acc0, held0);
#pragma unroll
        for (int t = 0; t < 8; ++t) { acc0[t] = acc1[t] + c0[t]; acc1[t] = c1[t]; }
        held0 = held1;
        held1 = e.o1;
      } else {
        flush(acc0, held0);
        flush(acc1, held1);
#pragma unroll
        for (int t = 0; t < 8; ++t) { acc0[t] = c0[t]; acc1[t] = c1[t]; }
        held0 = e.o0;
        held1 = e.o1;
      }
    }
    flush(acc0, held0);
    flush(acc1, held1);
    return;
  }

  // general rotation
  V sxy[3];
#pragma unroll
  for (int r = 0; r < 3; ++r)
    sxy[r] = Q::row_xy(Q::dup(g.rot[3 * r]), x2, Q::dup(A::mul(g.rot[3 * r + 1], y)));
  const V c2[3] = {Q::dup(g.centre[0]), Q::dup(g.centre[1]), Q::dup(g.centre[2])};
  for (int i = 0; i < k.npd; ++i) {
    const S3ZProd<T> e = sh.zp[i];
    const V rx2 = Q::add(Q::add(sxy[0], Q::dup(e.p[0])), c2[0]);
    const V ry2 = Q::add(Q::add(sxy[1], Q::dup(e.p[1])), c2[1]);
    const V rz2 = Q::add(Q::add(sxy[2], Q::dup(e.p[2])), c2[2]);
    const T rx[2] = {Q::lo(rx2), Q::hi(rx2)}, ry[2] = {Q::lo(ry2), Q::hi(ry2)}, rz[2] = {Q::lo(rz2), Q::hi(rz2)};
    const T gv[2] = {go[i * plane_o], has_b ? go[i * plane_o + 1] : A::fi(0)};
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      if (s == 1 && !has_b) continue;
      T w[8];
      long long off[8];
      if (!make_taps<T, 3>(p.D, p.H, p.W, rz[s], ry[s], rx[s], p.order, w, off)) continue;
#pragma unroll
      for (int t = 0; t < 8; t += 2)
        bwd_red_row(acc + off[t], acc + off[t + 1], A::tof(A::mul(gv[s], w[t])), A::tof(A::mul(gv[s], w[t + 1])), acc_lo,
                    acc_hi);
    }
  }
  (void)HW;
}

// grad_in (half) += scratch (float), rounded once
__global__ void bwd_fold_half(__half* __restrict__ grad_in, const float* __restrict__ scratch, long long n) {
  const long long i0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i0 + 8 <= n && ((uintptr_t)(grad_in + i0) % 16 == 0)) {
    const float4 s0 = *reinterpret_cast<const float4*>(scratch + i0);
    const float4 s1 = *reinterpret_cast<const float4*>(scratch + i0 + 4);
    uint4 gv = *reinterpret_cast<const uint4*>(grad_in + i0);
    __half2* h = reinterpret_cast<__half2*>(&gv);
    const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(h[j]);
      h[j] = __floats2half2_rn(f.x + s[2 * j], f.y + s[2 * j + 1]);
    }
    *reinterpret_cast<uint4*>(grad_in + i0) = gv;
  } else {
    for (long long i = i0; i < n && i < i0 + 8; ++i)
      grad_in[i] = __float2half_rn(__half2float(grad_in[i]) + scratch[i]);
  }
}

// Shape test and launch geometry of the streaming backward.
inline bool bwd_stream3d_applicable(const Params& p, int dtype, S3Launch& L, long long& ctas) {
  if (p.ndim != 3 || p.sampling_ratio != 1) return false;
  if (dtype != 0 && dtype != 1) return false;
  if (dtype == 0 && p.fm != kS3FloatPattern) return false;
  if (p.ovol < 4096 || p.ow < 8) return false;
  if ((long long)p.H * p.W >= 0x7fffffffLL) return false;
  L.tiles_w = (p.ow + kS3TileW - 1) / kS3TileW;
  L.tiles_h = (p.oh + kS3TileH - 1) / kS3TileH;
  const long long per_depth_ctas = (long long)p.R * p.C * L.tiles_w * L.tiles_h;
  int chunk = kS3MaxChunk;
  while (chunk > 8 && per_depth_ctas * ((p.od + chunk - 1) / chunk) < 148LL * 16) chunk >>= 1;
  if (chunk > p.od) chunk = p.od;
  L.chunk = chunk;
  L.chunks = (p.od + chunk - 1) / chunk;
  L.vec_store = 0;
  L.filter = 0;
  ctas = per_depth_ctas * L.chunks;
  return ctas <= 0x7fffffffLL;
}

// Half backward through a float scratch volume of n = N*C*D*H*W elements that the caller of this
// function owns: clear it, scatter into it, fold it into grad_in.  Allocates nothing.
inline int launch_bwd_stream3d_half(const Params& p, const S3Launch& L, long long ctas, float* scratch,
                                    cudaStream_t st) {
  const long long n = (long long)p.N * p.C * p.vol;
  cudaMemsetAsync(scratch, 0, (size_t)n * sizeof(float), st);
  resample_bwd_stream3d<__half><<<(unsigned)ctas, kS3Threads, 0, st>>>(p, L, scratch);
  const long long blocks = (n + 8 * 256 - 1) / (8 * 256);
  bwd_fold_half<<<(unsigned)blocks, 256, 0, st>>>((__half*)p.out, scratch, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

// The memory pool the float accumulator volumes come from: one per device, the library's own.  The device's
// default pool hands unused memory back to the driver at every synchronisation, so a host that synchronises
// between steps would pay for mapping the volume again on every call (measured: 0.95 ms became 1.1-1.6 ms); this
// pool keeps up to kBwdPoolKeepBytes of what it has been given and never touches the settings of the host's pools.
constexpr unsigned long long kBwdPoolKeepBytes = 1ull << 30;
constexpr int kBwdPoolMaxDevices = 64;
struct BwdPools {
  std::mutex mutex;
  cudaMemPool_t pool[kBwdPoolMaxDevices] = {};
};
inline BwdPools& bwd_pools() {
  static BwdPools pools;
  return pools;
}
// pool of the current device (created on first use), or nullptr
inline cudaMemPool_t bwd_pool_of_current_device(bool create) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kBwdPoolMaxDevices) return nullptr;
  BwdPools& ps = bwd_pools();
  std::lock_guard<std::mutex> lock(ps.mutex);
  if (!ps.pool[dev] && create) {
    cudaMemPoolProps props = {};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = dev;
    cudaMemPool_t pool = nullptr;
    if (cudaMemPoolCreate(&pool, &props) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    unsigned long long keep = kBwdPoolKeepBytes;
    cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    ps.pool[dev] = pool;
  }
  return ps.pool[dev];
}

// Launches the streaming backward when the call has its shape (3D, one sample per voxel, half or
// float in the reference's contraction pattern); MVR_STREAM3D_NOT_APPLICABLE otherwise.
// Half needs a float scratch volume: it is taken from the library's memory pool on the call's stream and
// returned to it on the same stream.
inline int try_launch_bwd_stream3d(const Params& p, int dtype, cudaStream_t st) {
  S3Launch L;
  long long ctas = 0;
  if (!bwd_stream3d_applicable(p, dtype, L, ctas)) return MVR_STREAM3D_NOT_APPLICABLE;
  if (dtype == 0) {
    resample_bwd_stream3d<float><<<(unsigned)ctas, kS3Threads, 0, st>>>(p, L, (float*)p.out);
    return cudaGetLastError() == cudaSuccess ? 0 : -8;
  }
  const long long n = (long long)p.N * p.C * p.vol;
  float* scratch = nullptr;
  cudaMemPool_t pool = bwd_pool_of_current_device(true);
  if (!pool || cudaMallocFromPoolAsync((void**)&scratch, (size_t)n * sizeof(float), pool, st) != cudaSuccess) {
    cudaGetLastError();
    return MVR_STREAM3D_NOT_APPLICABLE;  // no memory for the scratch volume: element-type atomics instead
  }
  const int rc = launch_bwd_stream3d_half(p, L, ctas, scratch, st);
  cudaFreeAsync(scratch, st);
  return rc;
}

}  // namespace mvr
