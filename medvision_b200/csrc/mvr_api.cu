// C ABI of the resampling library (declared in include/mvr.h): argument checks, kernel
// selection and launch.  No torch types; device pointers and sizes only.
#include <cuda_runtime.h>
#include <atomic>
#include <cstdlib>
#include <mutex>

#include "../../include/mvr.h"
#include "mvr_generic.cuh"
#include "mvr_tma3d.cuh"
#include "mvr_bwd3d.cuh"
#include "mvr_offset.cuh"
#include "mvr_cubic3d.cuh"
#include "mvr_flat.cuh"
#include "mvr_label.cuh"
#include "mvr_plane2d.cuh"

// ---- scratch of the entry point that allocates nothing ------------------------------------
// Lives in the library image: every GPU that loads the library holds these 16 MiB until the
// process exits.  In host code the name below is only a stand-in for the device array; the
// device address is asked for once per device (noalloc_scratch_of_current_device).
static __device__ __align__(256) float g_noalloc_scratch[MVR_NOALLOC_MAX_ELEMENTS];

namespace {

using namespace mvr;

constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mutex;
float* g_noalloc_addr[kMaxDevices] = {};

// Device address of g_noalloc_scratch on the CURRENT device, looked up on the first call for that
// device and remembered.
int noalloc_scratch_of_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return MVR_ERR_NO_DEVICE;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_addr[dev]) {
    float* addr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress((void**)&addr, g_noalloc_scratch);
    if (e != cudaSuccess || !addr) {
      cudaGetLastError();
      return MVR_ERR_SCRATCH_ADDRESS;
    }
    g_noalloc_addr[dev] = addr;
  }
  *out = g_noalloc_addr[dev];
  return MVR_OK;
}

// Float contraction pattern of the reference build (see mvr_arith.cuh).
// Found by matching the reference's own kernels bit for bit on a B200 (float32, all roi
// kinds): every family fuses its first product, the 3D rotation adds the hoisted R_i3*z
// with a plain add, and R22 = sa*sb*sg + ca*cg fuses its SECOND product.
std::atomic<int> g_contraction(kReferenceContraction);

int roi_width_of(int ndim, int kind) { return kind == KIND_BOX ? (ndim == 2 ? 5 : 7) : (ndim == 2 ? 6 : 10); }

int check_common(const void* a, const void* rois, void* b, int dtype, int ndim, int kind, int64_t N, int64_t C,
                 int64_t D, int64_t H, int64_t W, int64_t R, int roi_width, int od, int oh, int ow, int order,
                 bool allow_cubic = false) {
  if (dtype != MVR_F32 && dtype != MVR_F16 && dtype != MVR_F64) return MVR_ERR_DTYPE;
  if (ndim != 2 && ndim != 3) return MVR_ERR_NDIM;
  if (kind != MVR_ROI_BOX && kind != MVR_ROI_ROTATED) return MVR_ERR_ROI_KIND;
  if (order != 0 && order != 1 && !(allow_cubic && order == 3)) return MVR_ERR_ORDER;
  if (roi_width != roi_width_of(ndim, kind)) return MVR_ERR_ROI_WIDTH;
  if (N < 0 || C < 0 || R < 0 || D < 1 || H < 1 || W < 1 || od < 1 || oh < 1 || ow < 1) return MVR_ERR_SHAPE;
  if (ndim == 2 && (D != 1 || od != 1)) return MVR_ERR_SHAPE;
  if (D > INT32_MAX || H > INT32_MAX || W > INT32_MAX || N > INT32_MAX || C > INT32_MAX || R > INT32_MAX)
    return MVR_ERR_TOO_LARGE;
  if (R > 0 && C > 0 && (!a || !rois || !b)) return MVR_ERR_NULL;
  return MVR_OK;
}

Params make_params(const void* in, const void* rois, void* out, int ndim, int kind, int64_t N, int64_t C, int64_t D,
                   int64_t H, int64_t W, int64_t R, int od, int oh, int ow, float spatial_scale, int sampling_ratio,
                   int aligned, int order, int* status) {
  Params p;
  p.in = in; p.rois = rois; p.out = out; p.status = status;
  p.ndim = ndim; p.kind = kind; p.order = order; p.aligned = aligned ? 1 : 0; p.sampling_ratio = sampling_ratio;
  p.fm = g_contraction.load();
  p.N = (int)N; p.C = (int)C; p.D = (int)D; p.H = (int)H; p.W = (int)W; p.R = (int)R;
  p.od = od; p.oh = oh; p.ow = ow;
  p.spatial_scale = spatial_scale;
  p.vol = (long long)D * H * W;
  p.ovol = (long long)od * oh * ow;
  p.tiles_per_vol = (int)((p.ovol + kGenericThreads - 1) / kGenericThreads);
  return p;
}

template <typename T>
int launch_generic(const Params& p, bool fwd, cudaStream_t st) {
  const long long ctas = (long long)p.R * p.C * p.tiles_per_vol;
  if (ctas > 0x7fffffffLL) return MVR_ERR_TOO_LARGE;
  const dim3 grid((unsigned)ctas), block(kGenericThreads);
  if (fwd) {
    if (p.ndim == 2) resample_fwd_generic<T, 2><<<grid, block, 0, st>>>(p);
    else resample_fwd_generic<T, 3><<<grid, block, 0, st>>>(p);
  } else {
    if (p.ndim == 2) resample_bwd_generic<T, 2><<<grid, block, 0, st>>>(p);
    else resample_bwd_generic<T, 3><<<grid, block, 0, st>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? MVR_OK : MVR_ERR_LAUNCH;
}

template <typename T>
int launch_mark(const Params& p, cudaStream_t st) {
  const long long ctas = (long long)p.R * p.C * p.tiles_per_vol;
  if (ctas > 0x7fffffffLL) return MVR_ERR_TOO_LARGE;
  if (p.ndim == 2) resample_mark_generic<T, 2><<<(unsigned)ctas, kGenericThreads, 0, st>>>(p);
  else resample_mark_generic<T, 3><<<(unsigned)ctas, kGenericThreads, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? MVR_OK : MVR_ERR_LAUNCH;
}

// The kernels that need neither the streaming shape nor any memory beyond inputs and outputs:
// the flat kernel where it applies, else the one-CTA-per-tile kernel.
int dispatch_flat_or_generic(const Params& p, int dtype, bool fwd, cudaStream_t st) {
  {
    int rc;
    switch (dtype) {
      case MVR_F32: rc = launch_flat<float>(p, fwd, st); break;
      case MVR_F16: rc = launch_flat<__half>(p, fwd, st); break;
      default: rc = launch_flat<double>(p, fwd, st); break;
    }
    if (rc == 0) return cudaGetLastError() == cudaSuccess ? MVR_OK : MVR_ERR_LAUNCH;
  }
  switch (dtype) {
    case MVR_F32: return launch_generic<float>(p, fwd, st);
    case MVR_F16: return launch_generic<__half>(p, fwd, st);
    default: return launch_generic<double>(p, fwd, st);
  }
}

int dispatch(const Params& p, int dtype, bool fwd, cudaStream_t st) {
  if (p.R == 0 || p.C == 0) return MVR_OK;
  {
    const int rc = fwd ? try_launch_stream3d(p, dtype, st) : try_launch_bwd_stream3d(p, dtype, st);
    if (rc != MVR_STREAM3D_NOT_APPLICABLE) return rc;
  }
  if (fwd && try_launch_plane2d(p, dtype, st) == 0)
    return cudaGetLastError() == cudaSuccess ? MVR_OK : MVR_ERR_LAUNCH;
  if (fwd && p.order == 3) {  // Catmull-Rom, 2D and 3D
    int rc;
    switch (dtype) {
      case MVR_F32: rc = launch_cubic3d<float>(p, st); break;
      case MVR_F16: rc = launch_cubic3d<__half>(p, st); break;
      default: rc = launch_cubic3d<double>(p, st); break;
    }
    if (rc < 0) return MVR_ERR_TOO_LARGE;
    if (rc == 0) return cudaGetLastError() == cudaSuccess ? MVR_OK : MVR_ERR_LAUNCH;
  }
  return dispatch_flat_or_generic(p, dtype, fwd, st);
}

}  // namespace

extern "C" {

const char* mvr_strerror(int code) {
  switch (code) {
    case MVR_OK: return "ok";
    case MVR_ERR_DTYPE: return "unsupported element type (float32, float16, float64 only)";
    case MVR_ERR_NDIM: return "ndim must be 2 or 3";
    case MVR_ERR_ROI_KIND: return "roi kind must be box or rotated";
    case MVR_ERR_ORDER: return "only support order = 0 (nearest) or 1 (linear)";
    case MVR_ERR_SHAPE: return "bad tensor shape";
    case MVR_ERR_NULL: return "null data pointer";
    case MVR_ERR_ROI_WIDTH: return "wrong roi size!";
    case MVR_ERR_LAUNCH: return "CUDA kernel launch failed";
    case MVR_ERR_TOO_LARGE: return "problem too large for one launch";
    case MVR_ERR_NO_DEVICE: return "no CUDA device";
    case MVR_ERR_SCRATCH_LIMIT:
      return "gradient volume larger than the built-in scratch of mvr_roi_resample_bwd_noalloc "
             "(4194304 elements): use mvr_roi_resample_bwd, or split the batch";
    case MVR_ERR_SCRATCH_ADDRESS: return "the device address of the built-in scratch could not be obtained";
    case MVR_ERR_UNSUPPORTED: return "this entry point has no kernel for the given shape";
    default: return "unknown error";
  }
}

int mvr_version(void) { return 1; }

long long mvr_cached_memory_bytes(void) {
  cudaMemPool_t pool = bwd_pool_of_current_device(false);
  if (!pool) return 0;
  unsigned long long bytes = 0;
  if (cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReservedMemCurrent, &bytes) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return (long long)bytes;
}

int mvr_release_cached_memory(void) {
  cudaMemPool_t pool = bwd_pool_of_current_device(false);
  if (!pool) return MVR_OK;
  if (cudaMemPoolTrimTo(pool, 0) != cudaSuccess) {
    cudaGetLastError();
    return MVR_ERR_LAUNCH;
  }
  return MVR_OK;
}

int mvr_selftest_tma_skip_plane(int plane) { return g_t3_selftest_skip_plane.exchange(plane < 0 ? -1 : plane); }

int mvr_set_float_contraction(int bits) { return g_contraction.exchange(bits & 0x00ffffff); }
int mvr_get_float_contraction(void) { return g_contraction.load(); }

static int resample_fwd_impl(const void* features, const void* rois, void* output, int dtype, int ndim, int roi_kind,
                             int64_t N, int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width, int od,
                             int oh, int ow, float spatial_scale, int sampling_ratio, int aligned, int order,
                             int* status, void* stream, bool allow_cubic) {
  int rc = check_common(features, rois, output, dtype, ndim, roi_kind, N, C, D, H, W, R, roi_width, od, oh, ow, order,
                        allow_cubic);
  if (rc != MVR_OK) return rc;
  Params p = make_params(features, rois, output, ndim, roi_kind, N, C, D, H, W, R, od, oh, ow, spatial_scale,
                         sampling_ratio, aligned, order, status);
  return dispatch(p, dtype, true, (cudaStream_t)stream);
}

int mvr_roi_resample_fwd(const void* features, const void* rois, void* output, int dtype, int ndim, int roi_kind,
                         int64_t N, int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width,
                         int od, int oh, int ow, float spatial_scale, int sampling_ratio, int aligned, int order,
                         int* status, void* stream) {
  return resample_fwd_impl(features, rois, output, dtype, ndim, roi_kind, N, C, D, H, W, R, roi_width, od, oh, ow,
                           spatial_scale, sampling_ratio, aligned, order, status, stream, false);
}

int mvr_roi_resample_bwd(const void* grad_out, const void* rois, void* grad_in, int dtype, int ndim, int roi_kind,
                         int64_t N, int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width,
                         int od, int oh, int ow, float spatial_scale, int sampling_ratio, int aligned, int order,
                         int* status, void* stream) {
  int rc = check_common(grad_out, rois, grad_in, dtype, ndim, roi_kind, N, C, D, H, W, R, roi_width, od, oh, ow, order);
  if (rc != MVR_OK) return rc;
  Params p = make_params(grad_out, rois, grad_in, ndim, roi_kind, N, C, D, H, W, R, od, oh, ow, spatial_scale,
                         sampling_ratio, aligned, order, status);
  return dispatch(p, dtype, false, (cudaStream_t)stream);
}

int mvr_roi_resample_touched(const void* rois, unsigned char* mask, int dtype, int ndim, int roi_kind, int64_t N,
                             int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width, int od, int oh,
                             int ow, float spatial_scale, int sampling_ratio, int aligned, int order, void* stream) {
  int rc = check_common(rois, rois, mask, dtype, ndim, roi_kind, N, C, D, H, W, R, roi_width, od, oh, ow, order);
  if (rc != MVR_OK) return rc;
  Params p = make_params(nullptr, rois, mask, ndim, roi_kind, N, C, D, H, W, R, od, oh, ow, spatial_scale,
                         sampling_ratio, aligned, order, nullptr);
  if (p.R == 0 || p.C == 0) return MVR_OK;
  switch (dtype) {
    case MVR_F32: return launch_mark<float>(p, (cudaStream_t)stream);
    case MVR_F16: return launch_mark<__half>(p, (cudaStream_t)stream);
    default: return launch_mark<double>(p, (cudaStream_t)stream);
  }
}

int mvr_roi_resample_bwd_noalloc(const void* grad_out, const void* rois, void* grad_in, int dtype, int ndim,
                                 int roi_kind, int64_t N, int64_t C, int64_t D, int64_t H, int64_t W, int64_t R,
                                 int roi_width, int od, int oh, int ow, float spatial_scale, int sampling_ratio,
                                 int aligned, int order, int* status, void* stream) {
  int rc = check_common(grad_out, rois, grad_in, dtype, ndim, roi_kind, N, C, D, H, W, R, roi_width, od, oh, ow, order);
  if (rc != MVR_OK) return rc;
  Params p = make_params(grad_out, rois, grad_in, ndim, roi_kind, N, C, D, H, W, R, od, oh, ow, spatial_scale,
                         sampling_ratio, aligned, order, status);
  if (p.R == 0 || p.C == 0) return MVR_OK;
  cudaStream_t st = (cudaStream_t)stream;
  S3Launch L;
  long long ctas = 0;
  if (bwd_stream3d_applicable(p, dtype, L, ctas)) {
    if (dtype == MVR_F32) {  // float gradients are reduced straight into grad_in: no scratch at all
      resample_bwd_stream3d<float><<<(unsigned)ctas, kS3Threads, 0, st>>>(p, L, (float*)p.out);
      return cudaGetLastError() == cudaSuccess ? MVR_OK : MVR_ERR_LAUNCH;
    }
    // half: the float accumulator volume is the library's own static array
    if ((long long)p.N * p.C * p.vol > (long long)MVR_NOALLOC_MAX_ELEMENTS) return MVR_ERR_SCRATCH_LIMIT;
    float* scratch = nullptr;
    rc = noalloc_scratch_of_current_device(&scratch);
    if (rc != MVR_OK) return rc;
    return launch_bwd_stream3d_half(p, L, ctas, scratch, st) == 0 ? MVR_OK : MVR_ERR_LAUNCH;
  }
  // every other shape goes where the regular entry point sends it: kernels that accumulate with
  // element-type atomics straight into grad_in and use no scratch
  return dispatch_flat_or_generic(p, dtype, false, st);
}

static int affine_label_impl(const void* labels, int label_dtype, const float* rois, int32_t* output, int ndim,
                             int64_t N, int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width, int od,
                             int oh, int ow, float spatial_scale, int aligned, int* status, void* stream) {
  if (label_dtype < MVR_LABEL_U8 || label_dtype > MVR_LABEL_I64) return MVR_ERR_DTYPE;
  int rc = check_common(labels, rois, output, MVR_F32, ndim, MVR_ROI_ROTATED, N, C, D, H, W, R, roi_width, od, oh, ow, 0);
  if (rc != MVR_OK) return rc;
  Params p = make_params(labels, rois, output, ndim, MVR_ROI_ROTATED, N, C, D, H, W, R, od, oh, ow, spatial_scale, 1,
                         aligned, 0, status);
  rc = launch_label(p, label_dtype, (cudaStream_t)stream);
  return rc == 0 ? MVR_OK : (rc == -9 ? MVR_ERR_UNSUPPORTED : MVR_ERR_LAUNCH);
}

int mvr_affine_label_2d(const void* labels, int label_dtype, const float* rois, int32_t* output, int64_t N, int64_t C,
                        int64_t H, int64_t W, int64_t R, int roi_width, int oh, int ow, float spatial_scale,
                        int aligned, int* status, void* stream) {
  return affine_label_impl(labels, label_dtype, rois, output, 2, N, C, 1, H, W, R, roi_width, 1, oh, ow,
                           spatial_scale, aligned, status, stream);
}
int mvr_affine_label_3d(const void* labels, int label_dtype, const float* rois, int32_t* output, int64_t N, int64_t C,
                        int64_t D, int64_t H, int64_t W, int64_t R, int roi_width, int od, int oh, int ow,
                        float spatial_scale, int aligned, int* status, void* stream) {
  return affine_label_impl(labels, label_dtype, rois, output, 3, N, C, D, H, W, R, roi_width, od, oh, ow,
                           spatial_scale, aligned, status, stream);
}

int mvr_affine_fields_3d(const void* image, int dtype, const void* image_rois, void* image_out, int64_t C_image,
                         const void* labels, int label_dtype, const float* label_rois, int32_t* label_out,
                         int64_t C_label, int64_t N, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width, int od,
                         int oh, int ow, float spatial_scale, int aligned, int order, int* status, void* stream) {
  if (label_dtype < MVR_LABEL_U8 || label_dtype > MVR_LABEL_I64) return MVR_ERR_DTYPE;
  int rc = check_common(image, image_rois, image_out, dtype, 3, MVR_ROI_ROTATED, N, C_image, D, H, W, R, roi_width, od, oh,
                        ow, order);
  if (rc != MVR_OK) return rc;
  rc = check_common(labels, label_rois, label_out, MVR_F32, 3, MVR_ROI_ROTATED, N, C_label, D, H, W, R, roi_width, od, oh,
                    ow, 0);
  if (rc != MVR_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  Params pi = make_params(image, image_rois, image_out, 3, MVR_ROI_ROTATED, N, C_image, D, H, W, R, od, oh, ow,
                          spatial_scale, 1, aligned, order, status);
  T3LabelJob job;
  job.p = make_params(labels, label_rois, label_out, 3, MVR_ROI_ROTATED, N, C_label, D, H, W, R, od, oh, ow, spatial_scale,
                      1, aligned, 0, status);
  job.label_dtype = label_dtype;
  job.done = false;
  if (pi.R > 0 && pi.C > 0) {
    int ri = try_launch_stream3d(pi, dtype, st, job.p.C > 0 ? &job : nullptr);
    if (ri == MVR_STREAM3D_NOT_APPLICABLE) ri = dispatch(pi, dtype, true, st);  // small outputs and the like
    if (ri != MVR_OK) return ri < 0 && ri != -8 ? ri : MVR_ERR_LAUNCH;
  }
  if (!job.done && job.p.R > 0 && job.p.C > 0) {  // the label could not ride along: a launch of its own
    rc = launch_label(job.p, label_dtype, st);
    if (rc != 0) return rc == -9 ? MVR_ERR_UNSUPPORTED : MVR_ERR_LAUNCH;
  }
  return MVR_OK;
}

static int apply_offset_impl(const void* img, const void* offset, void* out, int dtype, int offset_dtype, int ndim,
                             int64_t B, int64_t C, int64_t D, int64_t H, int64_t W, int order, void* stream) {
  if (dtype != MVR_F32 && dtype != MVR_F16) return MVR_ERR_DTYPE;
  if (offset_dtype != dtype && !(dtype == MVR_F16 && offset_dtype == MVR_F32)) return MVR_ERR_DTYPE;
  if (order != 0 && order != 1 && order != 3) return MVR_ERR_ORDER;
  if (B < 0 || C < 0 || D < 1 || H < 1 || W < 1) return MVR_ERR_SHAPE;
  if (D * H * W >= 0x7fffffffLL || B > INT32_MAX || C > INT32_MAX) return MVR_ERR_TOO_LARGE;
  if (B > 0 && C > 0 && (!img || !offset || !out)) return MVR_ERR_NULL;
  OffsetParams p;
  p.img = img; p.off = offset; p.out = out;
  p.B = (int)B; p.C = (int)C; p.D = (int)D; p.H = (int)H; p.W = (int)W;
  p.order = order;
  p.fm = kReferenceContraction;
  p.off_f32 = (dtype == MVR_F16 && offset_dtype == MVR_F32) ? 1 : 0;
  const size_t pair = (dtype == MVR_F32 ? 4 : 2) * 2, off_pair = (offset_dtype == MVR_F32 ? 4 : 2) * 2;
  p.vec_ok = ((W & 1) == 0) && ((uintptr_t)offset % off_pair == 0) && ((uintptr_t)out % pair == 0);
  const int rc = ndim == 2 ? launch_apply_offset<2>(p, dtype, (cudaStream_t)stream)
                           : launch_apply_offset<3>(p, dtype, (cudaStream_t)stream);
  return rc == 0 ? MVR_OK : (rc == -9 ? MVR_ERR_TOO_LARGE : MVR_ERR_LAUNCH);
}

int mvr_apply_offset_2d(const void* img, const void* offset, void* out, int dtype, int offset_dtype, int64_t B,
                        int64_t C, int64_t H, int64_t W, int order, void* stream) {
  return apply_offset_impl(img, offset, out, dtype, offset_dtype, 2, B, C, 1, H, W, order, stream);
}
int mvr_apply_offset_3d(const void* img, const void* offset, void* out, int dtype, int offset_dtype, int64_t B,
                        int64_t C, int64_t D, int64_t H, int64_t W, int order, void* stream) {
  return apply_offset_impl(img, offset, out, dtype, offset_dtype, 3, B, C, D, H, W, order, stream);
}

// ---- the reference's extension surface --------------------------------------------------
// Axis-aligned RoIAlign has no `aligned` argument: the box kernels never shift by half a pixel.

int mvr_roi_align_2d_forward(const void* input, const void* rois, void* output, int dtype, int64_t N, int64_t C,
                             int64_t H, int64_t W, int64_t R, int roi_width, int oh, int ow, float spatial_scale,
                             int sampling_ratio, int order, int* status, void* stream) {
  return mvr_roi_resample_fwd(input, rois, output, dtype, 2, MVR_ROI_BOX, N, C, 1, H, W, R, roi_width, 1, oh, ow,
                              spatial_scale, sampling_ratio, 0, order, status, stream);
}
int mvr_roi_align_2d_backward(const void* top_grad, const void* rois, void* bottom_grad, int dtype, int64_t N,
                              int64_t C, int64_t H, int64_t W, int64_t R, int roi_width, int oh, int ow,
                              float spatial_scale, int sampling_ratio, int order, int* status, void* stream) {
  return mvr_roi_resample_bwd(top_grad, rois, bottom_grad, dtype, 2, MVR_ROI_BOX, N, C, 1, H, W, R, roi_width, 1, oh,
                              ow, spatial_scale, sampling_ratio, 0, order, status, stream);
}
int mvr_roi_align_3d_forward(const void* input, const void* rois, void* output, int dtype, int64_t N, int64_t C,
                             int64_t D, int64_t H, int64_t W, int64_t R, int roi_width, int od, int oh, int ow,
                             float spatial_scale, int sampling_ratio, int order, int* status, void* stream) {
  return mvr_roi_resample_fwd(input, rois, output, dtype, 3, MVR_ROI_BOX, N, C, D, H, W, R, roi_width, od, oh, ow,
                              spatial_scale, sampling_ratio, 0, order, status, stream);
}
int mvr_roi_align_3d_backward(const void* top_grad, const void* rois, void* bottom_grad, int dtype, int64_t N,
                              int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width, int od, int oh,
                              int ow, float spatial_scale, int sampling_ratio, int order, int* status, void* stream) {
  return mvr_roi_resample_bwd(top_grad, rois, bottom_grad, dtype, 3, MVR_ROI_BOX, N, C, D, H, W, R, roi_width, od, oh,
                              ow, spatial_scale, sampling_ratio, 0, order, status, stream);
}
int mvr_roi_align_rotated_2d_forward(const void* input, const void* rois, void* output, int dtype, int64_t N,
                                     int64_t C, int64_t H, int64_t W, int64_t R, int roi_width, int oh, int ow,
                                     float spatial_scale, int sampling_ratio, int aligned, int order, int* status,
                                     void* stream) {
  return mvr_roi_resample_fwd(input, rois, output, dtype, 2, MVR_ROI_ROTATED, N, C, 1, H, W, R, roi_width, 1, oh, ow,
                              spatial_scale, sampling_ratio, aligned, order, status, stream);
}
int mvr_roi_align_rotated_2d_backward(const void* top_grad, const void* rois, void* bottom_grad, int dtype, int64_t N,
                                      int64_t C, int64_t H, int64_t W, int64_t R, int roi_width, int oh, int ow,
                                      float spatial_scale, int sampling_ratio, int aligned, int order, int* status,
                                      void* stream) {
  return mvr_roi_resample_bwd(top_grad, rois, bottom_grad, dtype, 2, MVR_ROI_ROTATED, N, C, 1, H, W, R, roi_width, 1,
                              oh, ow, spatial_scale, sampling_ratio, aligned, order, status, stream);
}
int mvr_roi_align_rotated_3d_forward(const void* input, const void* rois, void* output, int dtype, int64_t N,
                                     int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width, int od,
                                     int oh, int ow, float spatial_scale, int sampling_ratio, int aligned, int order,
                                     int* status, void* stream) {
  return mvr_roi_resample_fwd(input, rois, output, dtype, 3, MVR_ROI_ROTATED, N, C, D, H, W, R, roi_width, od, oh, ow,
                              spatial_scale, sampling_ratio, aligned, order, status, stream);
}
int mvr_roi_align_rotated_3d_backward(const void* top_grad, const void* rois, void* bottom_grad, int dtype, int64_t N,
                                      int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width, int od,
                                      int oh, int ow, float spatial_scale, int sampling_ratio, int aligned, int order,
                                      int* status, void* stream) {
  return mvr_roi_resample_bwd(top_grad, rois, bottom_grad, dtype, 3, MVR_ROI_ROTATED, N, C, D, H, W, R, roi_width, od,
                              oh, ow, spatial_scale, sampling_ratio, aligned, order, status, stream);
}
int mvr_affine_2d(const void* input, const void* rois, void* output, int dtype, int64_t N, int64_t C, int64_t H,
                  int64_t W, int64_t R, int roi_width, int oh, int ow, float spatial_scale, int sampling_ratio,
                  int aligned, int order, int* status, void* stream) {
  // the only entry points with order 3 (Catmull-Rom), as in the reference
  return resample_fwd_impl(input, rois, output, dtype, 2, MVR_ROI_ROTATED, N, C, 1, H, W, R, roi_width, 1, oh, ow,
                           spatial_scale, sampling_ratio, aligned, order, status, stream, true);
}
int mvr_affine_3d(const void* input, const void* rois, void* output, int dtype, int64_t N, int64_t C, int64_t D,
                  int64_t H, int64_t W, int64_t R, int roi_width, int od, int oh, int ow, float spatial_scale,
                  int sampling_ratio, int aligned, int order, int* status, void* stream) {
  return resample_fwd_impl(input, rois, output, dtype, 3, MVR_ROI_ROTATED, N, C, D, H, W, R, roi_width, od, oh, ow,
                           spatial_scale, sampling_ratio, aligned, order, status, stream, true);
}

}  // extern "C"
