// Label (segmentation map) resampling: what the reference's augmentations do to a `seg` field,
//     affine_3d(seg.float(), rois, out_size, 1, 1, aligned, order=0).int()
// (medvision/aug_cuda_batch/aug_spatial.py:158-194 and the seg twins of the other transforms),
// in one kernel on the integer tensor: no float copy of the input, no float result, no cast pass.
//
// The geometry is the float32 path of the affine kernels, operation by operation (rois are
// float32, as the reference builds them; the float contraction pattern of the reference build).
// With order 0 the eight weights are one-hot, so the reference's tap sum is the value of one tap
// (or 0 when no weight qualifies or the sample lies outside the band): that tap is picked per
// axis and is the only element read.  The value goes through float, as in the reference:
// (int32)(float)label.
//
// Layout of the work as in the gather path of the forward: a thread owns two w-adjacent voxels
// of a 32 x 16 tile and walks a depth chunk; for rois that turn about z at most the in-plane tap
// is fixed along the walk and the plane comes from the per-depth table.
#pragma once
#include "mvr_stream3d.cuh"

namespace mvr {

template <typename IT>
__device__ __forceinline__ int label_value(const IT* p) { return __float2int_rz((float)__ldg(p)); }

// one-hot choice of an axis: offset index (i0 or i1), or -1 when neither weight qualifies
__device__ __forceinline__ int label_axis_pick(float c, int size, bool& outside) {
  outside = axis_outside<float>(c, size);
  AxisTap<float> t;
  axis_tap<float>(c, size, t);
  nearest_axis<float>(t.l, t.h);
  return t.h == 1.0f ? t.i0 : (t.l == 1.0f ? t.i1 : -1);
}

// One work item (32 x 16 tile x depth chunk of one (roi, channel)) of the dense 3D label path.
template <typename IT>
__device__ __forceinline__ void label_item_stream3d(const Params& p, const S3Launch& L, const S3Cta& k, S3Shared<float>& sh) {
  typedef Ar<float> A;
  s3_prologue<float>(p, k, sh);  // p.order == 0: the per-depth weights in the table are one-hot
  const RoiGeom<float>& g = sh.g;
  const int fm = kS3FloatPattern;
  const bool rotated = (p.kind == KIND_ROTATED);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pw0 = k.tw * kS3TileW + (warp & 1) * 16 + (lane & 7) * 2;
  const int ph = k.th * kS3TileH + (warp >> 1) * 4 + (lane >> 3);
  if (ph >= p.oh || pw0 >= p.ow) return;
  const bool has_b = (pw0 + 1 < p.ow);
  const long long plane_o = (long long)p.oh * p.ow;
  int* out = (int*)p.out + k.nc * p.ovol + (long long)k.pd0 * plane_o + (long long)ph * p.ow + pw0;
  const bool vec = L.vec_store && has_b;
  const int npd = k.npd;

  if (g.batch < 0 || g.batch >= p.N) {
    if (p.status && threadIdx.x == 0 && k.tw == 0 && k.th == 0 && k.ck == 0) atomicOr(p.status, STATUS_BAD_BATCH_INDEX);
    for (int i = 0; i < npd; ++i) {
      out[i * plane_o] = 0;
      if (has_b) out[i * plane_o + 1] = 0;
    }
    return;
  }
  const IT* vol = (const IT*)p.in + ((long long)g.batch * p.C + k.c) * p.vol;
  const float sub_x = lattice_sub<float>(g.bin[0], 0, 1), sub_y = lattice_sub<float>(g.bin[1], 0, 1);
  const float x[2] = {A::add(lattice_base<float>(g.start[0], pw0, g.bin[0], fm), sub_x),
                      A::add(lattice_base<float>(g.start[0], has_b ? pw0 + 1 : pw0, g.bin[0], fm), sub_x)};
  const float y = A::add(lattice_base<float>(g.start[1], ph, g.bin[1], fm), sub_y);

  if (sh.zsep) {
    int off[2];  // in-plane offset of the picked tap, -1: the voxel is 0 at every depth
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      float rx = x[s], ry = y;
      if (rotated) {
        rx = A::add(__fmaf_rn(g.rot[0], x[s], A::mul(g.rot[1], y)), g.centre[0]);
        ry = A::add(__fmaf_rn(g.rot[3], x[s], A::mul(g.rot[4], y)), g.centre[1]);
      }
      bool ox, oy;
      const int ix = label_axis_pick(rx, p.W, ox), iy = label_axis_pick(ry, p.H, oy);
      off[s] = (ox || oy || ix < 0 || iy < 0 || (s == 1 && !has_b)) ? -1 : iy * p.W + ix;
    }
#pragma unroll 4
    for (int i = 0; i < npd; ++i, out += plane_o) {  // unrolled: several depths' loads in flight
      const S3ZTap<float> e = sh.zt[i];
      int va = 0, vb = 0;
      const bool take0 = e.h == 1.0f, take1 = e.l == 1.0f;
      if (e.inside && (take0 || take1)) {
        const IT* pl = vol + (take0 ? e.o0 : e.o1);
        if (off[0] >= 0) va = label_value<IT>(pl + off[0]);
        if (off[1] >= 0) vb = label_value<IT>(pl + off[1]);
      }
      if (vec) {
        *reinterpret_cast<int2*>(out) = make_int2(va, vb);
      } else {
        out[0] = va;
        if (has_b) out[1] = vb;
      }
    }
    return;
  }

  // general rotation: the three coordinates change with depth
  float sxy[2][3];
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int r = 0; r < 3; ++r) sxy[s][r] = __fmaf_rn(g.rot[3 * r], x[s], A::mul(g.rot[3 * r + 1], y));
  const long long HW = (long long)p.H * p.W;
  for (int i = 0; i < npd; ++i, out += plane_o) {
    const S3ZProd<float> e = sh.zp[i];
    int val[2] = {0, 0};
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      if (s == 1 && !has_b) continue;
      const float rx = A::add(A::add(sxy[s][0], e.p[0]), g.centre[0]);
      const float ry = A::add(A::add(sxy[s][1], e.p[1]), g.centre[1]);
      const float rz = A::add(A::add(sxy[s][2], e.p[2]), g.centre[2]);
      bool ox, oy, oz;
      const int ix = label_axis_pick(rx, p.W, ox), iy = label_axis_pick(ry, p.H, oy), iz = label_axis_pick(rz, p.D, oz);
      if (!(ox || oy || oz || ix < 0 || iy < 0 || iz < 0)) val[s] = label_value<IT>(vol + iz * HW + (long long)iy * p.W + ix);
    }
    if (vec) {
      *reinterpret_cast<int2*>(out) = make_int2(val[0], val[1]);
    } else {
      out[0] = val[0];
      if (has_b) out[1] = val[1];
    }
  }
}

template <typename IT>
__global__ void __launch_bounds__(kS3Threads)
resample_label_stream3d(const Params p, const S3Launch L) {
  __shared__ S3Shared<float> sh;
  label_item_stream3d<IT>(p, L, s3_cta(p, L), sh);
}

// The gather launch of a rotated forward (resample_fwd_stream3d_rest) with the label field of the same
// augmentation call riding along: the persistent CTAs first take the image's work items under a general
// rotation (none for the augmentations, which turn about z only), then stride over the label items.  An
// image field and its label field thus cost the two overlapped launches of the image alone.
// p / L / items: the image (element type T); pl / Ll / items_l: the label job (float32 rois, int32 result).
template <typename T, typename IT>
__global__ void __launch_bounds__(kS3Threads)
resample_fwd_stream3d_rest_label(const Params p, const S3Launch L, long long items, const Params pl, const S3Launch Ll,
                                 long long items_l) {
  __shared__ union Tables {
    S3Shared<T> img;
    S3Shared<float> lab;
  } sh;
  __shared__ unsigned general[kS3RestMaxRois / 32];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  int mine = 0;
  for (int n0 = 0; n0 < p.R; n0 += kS3Threads) {
    const int n = n0 + threadIdx.x;
    const bool g = n < p.R && !s3_roi_is_planar<T>(p, n);
    const unsigned m = __ballot_sync(0xffffffffu, g);
    if ((threadIdx.x & 31) == 0 && n < kS3RestMaxRois) general[n >> 5] = m;
    mine |= g;
  }
  if (__syncthreads_or(mine))
    for (long long item = blockIdx.x; item < items; item += gridDim.x) {
      const S3Cta k = s3_cta(p, L, item);
      if (!((general[k.n >> 5] >> (k.n & 31)) & 1u)) continue;  // CTA-uniform
      s3_prologue<T>(p, k, sh.img);
      s3_body_l1<T>(p, L, k, sh.img);
      __syncthreads();  // the next item's prologue overwrites the tables
    }
  for (long long item = blockIdx.x; item < items_l; item += gridDim.x) {
    label_item_stream3d<IT>(pl, Ll, s3_cta(pl, Ll, item), sh.lab);
    __syncthreads();
  }
}

// 2D labels and small 3D outputs: one thread per output element, every roi decoded per CTA as in
// the flat kernels.
template <typename IT, int NDIM>
__global__ void __launch_bounds__(256)
resample_label_flat(const Params p, int per_roi) {
  typedef Ar<float> A;
  constexpr int kMaxRois = 256 / 32 + 2;
  __shared__ RoiGeom<float> geo[kMaxRois];
  const long long total = (long long)p.R * per_roi;
  const long long e0 = (long long)blockIdx.x * 256;
  const long long n0 = e0 / per_roi;
  const int rem0 = (int)(e0 - n0 * per_roi);
  const long long e_last = min(e0 + 256, total) - 1;
  const int n_rois = (int)(e_last / per_roi - n0) + 1;
  if ((int)threadIdx.x < n_rois) {
    const int osz[3] = {p.ow, p.oh, p.od};
    decode_roi<float>((const float*)p.rois, n0 + threadIdx.x, NDIM, p.kind, osz, p.spatial_scale, 1, p.aligned, p.fm,
                      geo[threadIdx.x]);
  }
  __syncthreads();
  const long long e = e0 + threadIdx.x;
  if (e >= total) return;
  const int t = rem0 + (int)threadIdx.x;
  const int r = t / per_roi;
  const int rem = t - r * per_roi;
  const RoiGeom<float>& g = geo[r];
  const int ovol = (int)p.ovol;
  const int c = rem / ovol;
  const int v = rem - c * ovol;
  const int pw = v % p.ow, ph = (v / p.ow) % p.oh, pd = (NDIM == 3) ? v / (p.ow * p.oh) : 0;
  int* out = (int*)p.out + e;
  if (g.batch < 0 || g.batch >= p.N) {
    if (p.status && rem == 0) atomicOr(p.status, STATUS_BAD_BATCH_INDEX);
    *out = 0;
    return;
  }
  const IT* vol = (const IT*)p.in + ((long long)g.batch * p.C + c) * p.vol;
  const float x = A::add(lattice_base<float>(g.start[0], pw, g.bin[0], p.fm), lattice_sub<float>(g.bin[0], 0, 1));
  const float y = A::add(lattice_base<float>(g.start[1], ph, g.bin[1], p.fm), lattice_sub<float>(g.bin[1], 0, 1));
  const float z = (NDIM == 3)
      ? A::add(lattice_base<float>(g.start[2], pd, g.bin[2], p.fm), lattice_sub<float>(g.bin[2], 0, 1)) : 0.0f;
  float sx, sy, sz;
  to_volume<float, NDIM>(g, p.kind, p.fm, x, y, z, sx, sy, sz);
  bool ox, oy, oz = false;
  const int ix = label_axis_pick(sx, p.W, ox), iy = label_axis_pick(sy, p.H, oy);
  const int iz = (NDIM == 3) ? label_axis_pick(sz, p.D, oz) : 0;
  int val = 0;
  if (!(ox || oy || oz || ix < 0 || iy < 0 || iz < 0))
    val = label_value<IT>(vol + ((long long)iz * p.H + iy) * p.W + ix);
  *out = val;
}

enum { LABEL_U8 = 0, LABEL_I16 = 1, LABEL_I32 = 2, LABEL_I64 = 3 };

// Work items of the dense 3D label path; false: the call has not its shape.
inline bool label_stream3d_geometry(const Params& p, S3Launch& L, long long& items) {
  if (!(p.ndim == 3 && p.ovol >= 4096 && p.ow >= 8 && p.vol < 0x7fffffffLL && p.fm == kS3FloatPattern)) return false;
  L.tiles_w = (p.ow + kS3TileW - 1) / kS3TileW;
  L.tiles_h = (p.oh + kS3TileH - 1) / kS3TileH;
  const long long per_depth = (long long)p.R * p.C * L.tiles_w * L.tiles_h;
  int chunk = kS3MaxChunk;
  while (chunk > 8 && per_depth * ((p.od + chunk - 1) / chunk) < 148LL * 16) chunk >>= 1;
  L.chunk = min(chunk, p.od);
  L.chunks = (p.od + L.chunk - 1) / L.chunk;
  L.vec_store = ((p.ow & 1) == 0) && (((uintptr_t)p.out) % 8 == 0);
  L.filter = 0;
  items = per_depth * L.chunks;
  return items <= 0x7fffffffLL;
}

// p: in = labels, rois = float32 rois, out = int32 result, order = 0, sampling_ratio = 1
inline int launch_label(const Params& p, int label_dtype, cudaStream_t st) {
  if (p.R == 0 || p.C == 0) return 0;
  S3Launch L;
  long long items = 0;
  if (label_stream3d_geometry(p, L, items)) {
    {
      const long long ctas = items;
      const unsigned grid = (unsigned)ctas;
      switch (label_dtype) {
        case LABEL_U8: resample_label_stream3d<unsigned char><<<grid, kS3Threads, 0, st>>>(p, L); break;
        case LABEL_I16: resample_label_stream3d<short><<<grid, kS3Threads, 0, st>>>(p, L); break;
        case LABEL_I32: resample_label_stream3d<int><<<grid, kS3Threads, 0, st>>>(p, L); break;
        default: resample_label_stream3d<long long><<<grid, kS3Threads, 0, st>>>(p, L); break;
      }
      return cudaGetLastError() == cudaSuccess ? 0 : -8;
    }
  }
  const long long per_roi = (long long)p.C * p.ovol;
  if (per_roi < 32 || per_roi > (1LL << 30)) return -9;
  const long long ctas = ((long long)p.R * per_roi + 255) / 256;
  if (ctas > 0x7fffffffLL) return -9;
  const unsigned grid = (unsigned)ctas;
  const int pr = (int)per_roi;
#define MVR_LABEL(IT)                                                              \
  {                                                                                \
    if (p.ndim == 2) resample_label_flat<IT, 2><<<grid, 256, 0, st>>>(p, pr);      \
    else resample_label_flat<IT, 3><<<grid, 256, 0, st>>>(p, pr);                  \
  }
  switch (label_dtype) {
    case LABEL_U8: MVR_LABEL(unsigned char) break;
    case LABEL_I16: MVR_LABEL(short) break;
    case LABEL_I32: MVR_LABEL(int) break;
    default: MVR_LABEL(long long) break;
  }
#undef MVR_LABEL
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

}  // namespace mvr
