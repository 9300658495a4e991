/* medvision-b200 resampling library: C ABI.
 *
 * B200 (sm_100a) implementation of the RoI Align / RoI Align Rotated / affine_{2d,3d}
 * gather-interpolate path of MedVision.  The ten `mvr_<name>` entry points at the end are
 * what the reference's Python layer binds as `medvision._C.<name>`
 * (medvision/csrc/vision.cpp:34-48,74-75); each one takes the same arguments in the same
 * order, with every tensor replaced by a device pointer plus its sizes, and a stream.
 *
 * Conventions
 *  - All data pointers are DEVICE pointers on the current device; tensors are contiguous
 *    NC[D]HW, rois are (R, roi_width) in the SAME element type as the features
 *    (medvision/ops/cuda_fun_tools.py:37,82 casts them before the call).
 *      box 2D      (R,5)  [batch, x1, y1, x2, y2]              medvision/ops/roi_align_nd.py:162-165
 *      box 3D      (R,7)  [batch, x1, y1, z1, x2, y2, z2]
 *      rotated 2D  (R,6)  [batch, cx, cy, w, h, angle]         medvision/ops/roi_align_rotated_nd.py:171-175
 *      rotated 3D  (R,10) [batch, cx, cy, cz, w, h, d, angle_x, angle_y, angle_z]   (radians)
 *  - Calls are asynchronous on `stream` (a cudaStream_t passed as void*; NULL = the legacy
 *    default stream) and never synchronise.  The forward entry points allocate nothing.  The
 *    dense 3D half-precision backward takes a float scratch volume of the gradient's shape from a
 *    stream-ordered memory pool of the library's own (cudaMallocFromPoolAsync / cudaFreeAsync on
 *    `stream`), which keeps up to 1 GiB of what it was given between calls: see
 *    mvr_cached_memory_bytes / mvr_release_cached_memory.  The pool is created by the first such
 *    call on a device; make that call before any stream capture begins.
 *  - Return value: MVR_OK or a negative MVR_ERR_* code; nothing is launched on error.
 *    `mvr_strerror` gives the message, worded as the reference's AT_ERROR text where one
 *    exists ("wrong roi size! size_rois should be 10", medvision/csrc/roi_align_rotated_3d.h:34-36).
 *  - `status` is an optional device int (may be NULL).  A roi whose batch index is outside
 *    [0, N) is not sampled (the reference would read out of bounds): its outputs are zero,
 *    its gradient is dropped, and bit MVR_STATUS_BAD_BATCH_INDEX is OR-ed into *status.
 *  - There is no CPU implementation: a missing GPU or library is an error, as in the
 *    reference ("RoIAlignRotated is not implemented on CPU", roi_align_rotated_3d.h:93-95).
 */
#ifndef MVR_H_
#define MVR_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types (the reference dispatches float, double and half:
 * AT_DISPATCH_FLOATING_TYPES_AND_HALF, medvision/csrc/cuda/roi_align_rotated_3d_cuda.cu:14) */
#define MVR_F32 0
#define MVR_F16 1
#define MVR_F64 2

#define MVR_ROI_BOX 0
#define MVR_ROI_ROTATED 1

#define MVR_OK 0
#define MVR_ERR_DTYPE (-1)
#define MVR_ERR_NDIM (-2)
#define MVR_ERR_ROI_KIND (-3)
#define MVR_ERR_ORDER (-4)
#define MVR_ERR_SHAPE (-5)
#define MVR_ERR_NULL (-6)
#define MVR_ERR_ROI_WIDTH (-7)
#define MVR_ERR_LAUNCH (-8)
#define MVR_ERR_TOO_LARGE (-9)
#define MVR_ERR_NO_DEVICE (-10)
#define MVR_ERR_SCRATCH_LIMIT (-11)
#define MVR_ERR_SCRATCH_ADDRESS (-12)
#define MVR_ERR_UNSUPPORTED (-13)     /* the entry point has no kernel for this shape: use the general one */

/* element types of label volumes (mvr_affine_label_*) */
#define MVR_LABEL_U8 0
#define MVR_LABEL_I16 1
#define MVR_LABEL_I32 2
#define MVR_LABEL_I64 3

#define MVR_STATUS_BAD_BATCH_INDEX 1

const char* mvr_strerror(int code);
int mvr_version(void);

/* The memory pool behind the dense 3D half backward (current device).  Bytes the pool holds at
 * the moment (0 before the first such call), and: give all of it that is not in use back to the
 * driver.  Neither has a counterpart in the reference, which allocates nothing. */
long long mvr_cached_memory_bytes(void);
int mvr_release_cached_memory(void);

/* Which float products are fused into the following addition (bit set of the contraction
 * pattern; half arithmetic never fuses).  The default reproduces the reference build
 * (nvcc -fmad=true).  Returns the previous value.  Process-wide; not a per-call option. */
int mvr_set_float_contraction(int bits);
int mvr_get_float_contraction(void);

/* Self-test of the bounded waits in the plane-streaming forward kernel; has no counterpart in the
 * reference.  While `plane` >= 0, the producer of every CTA of that kernel leaves out the plane with
 * this index of its schedule and all waits get a limit of about a millisecond: the consumers'
 * wait for that plane runs out, every thread RETURNS (no trap, no endless loop), status bit
 * MVR_STATUS_TMA_TIMEOUT is set and the output of the call is incomplete.  -1 switches it off.
 * Process-wide; returns the previous value.  For tests only: it proves that a copy that never
 * arrives ends in an error status with the context intact. */
#define MVR_STATUS_TMA_TIMEOUT 2
int mvr_selftest_tma_skip_plane(int plane);

/* General forward: output[r, c, p] = mean over the roi bin's sub-samples of
 * interp(features[batch(r), c], sample position).
 * Replaces the six forward launchers (medvision/csrc/cuda/roi_align_{2d,3d}_cuda.cu:5-30,
 * roi_align_rotated_{2d,3d}_cuda.cu:5-30, medvision/csrc/cuda_aug/affine_{2d,3d}_cuda.cu:5-30).
 * ndim 2: D and od must be 1.  roi_width is rois.size(1) and is checked against (ndim, roi_kind).
 * order 0 = nearest, 1 = linear.  R == 0 is a no-op. */
int mvr_roi_resample_fwd(const void* features, const void* rois, void* output, int dtype, int ndim, int roi_kind,
                         int64_t N, int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width,
                         int od, int oh, int ow, float spatial_scale, int sampling_ratio, int aligned, int order,
                         int* status, void* stream);

/* General backward: grad_in += scatter of grad_out * tap weight / sample count.  grad_in has
 * the feature shape, must be zero-filled by the caller (as the reference's Python does,
 * medvision/ops/roi_align_rotated_nd.py:148) and is accumulated into, like the reference
 * (medvision/csrc/cuda/roi_align_rotated_3d_cuda_kernel.cuh:251-260): with atomics in the element
 * type, except that half gradients of dense 3D calls are summed in float and rounded once.
 * The two x-neighbours of a tap row are added by one 16-byte reduction that carries zeros in its
 * other slots, so elements of grad_in next to a tap may have +0 added to them (a -0 becomes +0);
 * nothing outside the N*C*D*H*W elements of grad_in is touched.
 * Replaces the four backward launchers (medvision/csrc/cuda/roi_align*_cuda.cu:32-55). */
int mvr_roi_resample_bwd(const void* grad_out, const void* rois, void* grad_in, int dtype, int ndim, int roi_kind,
                         int64_t N, int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width,
                         int od, int oh, int ow, float spatial_scale, int sampling_ratio, int aligned, int order,
                         int* status, void* stream);

/* Backward for callers that must not allocate device memory.  It has no counterpart in the
 * reference.
 *
 * Same arguments, same result and same error codes as mvr_roi_resample_bwd.  The difference is
 * where the float accumulator of the dense 3D half-precision backward lives: the regular entry
 * point borrows it from the library's stream-ordered memory pool for the duration of the call; this one uses
 * a fixed array inside the library image and calls no cudaMalloc / cudaFree / pool routine at all
 * (shapes and element types that need no accumulator volume go to the very same kernels as with
 * the regular entry point, which never allocated for them either).
 *
 * It is meant for hosts where an allocation at call time is not an option: a plug-in whose
 * run-time hook is forbidden to allocate once initialisation is over, a worker that shares the GPU
 * with a framework which has already reserved the whole device for its own caching allocator (so
 * that a foreign allocation fails or fragments it), or a loop with a latency budget that cannot
 * absorb the implicit synchronisation an allocation may bring.
 *
 * Limits and rules
 *  - The accumulator holds MVR_NOALLOC_MAX_ELEMENTS = 4 194 304 floats (16 MiB).  Every GPU on
 *    which the library is loaded keeps that memory until the process ends.  A half call whose
 *    gradient volume N*C*D*H*W exceeds it returns MVR_ERR_SCRATCH_LIMIT and launches nothing.
 *  - The first call on a device asks the runtime for the array's device address (once per device,
 *    with that device current); make that first call before any stream capture begins.
 *  - All calls on a device share the one array.  Each call clears the part it uses on `stream`
 *    before scattering into it, so earlier contents never leak into a result; but two calls that
 *    can overlap on the GPU (different streams, no dependency between them) race on it and both
 *    results are garbage.  Serialise such calls. */
#define MVR_NOALLOC_MAX_ELEMENTS 4194304
int mvr_roi_resample_bwd_noalloc(const void* grad_out, const void* rois, void* grad_in, int dtype, int ndim,
                                 int roi_kind, int64_t N, int64_t C, int64_t D, int64_t H, int64_t W, int64_t R,
                                 int roi_width, int od, int oh, int ow, float spatial_scale, int sampling_ratio,
                                 int aligned, int order, int* status, void* stream);

/* Measurement utility; has no counterpart in the reference.  Sets mask[b, c, voxel] = 1 (bytes,
 * feature shape, zero-filled by the caller) for every input element that a tap of the
 * corresponding forward call reads.  The count of set bytes is the "distinct input elements
 * touched" term of the forward's algorithmic byte count. */
int mvr_roi_resample_touched(const void* rois, unsigned char* mask, int dtype, int ndim, int roi_kind,
                             int64_t N, int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width,
                             int od, int oh, int ow, float spatial_scale, int sampling_ratio, int aligned, int order,
                             void* stream);

/* ---- the reference's extension surface, one entry per `m.def` ------------------------- */

/* medvision/csrc/vision.cpp:34  roi_align_2d_forward(input, rois, output, oh, ow, spatial_scale, sampling_ratio, order)
 * (medvision/csrc/roi_align_2d.h) */
int mvr_roi_align_2d_forward(const void* input, const void* rois, void* output, int dtype,
                             int64_t N, int64_t C, int64_t H, int64_t W, int64_t R, int roi_width,
                             int oh, int ow, float spatial_scale, int sampling_ratio, int order,
                             int* status, void* stream);
/* medvision/csrc/vision.cpp:35  roi_align_2d_backward(top_grad, rois, bottom_grad, oh, ow, spatial_scale, sampling_ratio, order) */
int mvr_roi_align_2d_backward(const void* top_grad, const void* rois, void* bottom_grad, int dtype,
                              int64_t N, int64_t C, int64_t H, int64_t W, int64_t R, int roi_width,
                              int oh, int ow, float spatial_scale, int sampling_ratio, int order,
                              int* status, void* stream);
/* medvision/csrc/vision.cpp:37  roi_align_3d_forward(input, rois, output, od, oh, ow, spatial_scale, sampling_ratio, order)
 * (medvision/csrc/roi_align_3d.h) */
int mvr_roi_align_3d_forward(const void* input, const void* rois, void* output, int dtype,
                             int64_t N, int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width,
                             int od, int oh, int ow, float spatial_scale, int sampling_ratio, int order,
                             int* status, void* stream);
/* medvision/csrc/vision.cpp:38  roi_align_3d_backward */
int mvr_roi_align_3d_backward(const void* top_grad, const void* rois, void* bottom_grad, int dtype,
                              int64_t N, int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width,
                              int od, int oh, int ow, float spatial_scale, int sampling_ratio, int order,
                              int* status, void* stream);
/* medvision/csrc/vision.cpp:40-41  roi_align_rotated_2d_forward(input, rois, output, oh, ow, spatial_scale,
 * sampling_ratio, aligned, order)  (medvision/csrc/roi_align_rotated_2d.h) */
int mvr_roi_align_rotated_2d_forward(const void* input, const void* rois, void* output, int dtype,
                                     int64_t N, int64_t C, int64_t H, int64_t W, int64_t R, int roi_width,
                                     int oh, int ow, float spatial_scale, int sampling_ratio, int aligned, int order,
                                     int* status, void* stream);
/* medvision/csrc/vision.cpp:42-43  roi_align_rotated_2d_backward */
int mvr_roi_align_rotated_2d_backward(const void* top_grad, const void* rois, void* bottom_grad, int dtype,
                                      int64_t N, int64_t C, int64_t H, int64_t W, int64_t R, int roi_width,
                                      int oh, int ow, float spatial_scale, int sampling_ratio, int aligned, int order,
                                      int* status, void* stream);
/* medvision/csrc/vision.cpp:45-46  roi_align_rotated_3d_forward(input, rois, output, od, oh, ow, spatial_scale,
 * sampling_ratio, aligned, order)  (medvision/csrc/roi_align_rotated_3d.h:71-96) */
int mvr_roi_align_rotated_3d_forward(const void* input, const void* rois, void* output, int dtype,
                                     int64_t N, int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width,
                                     int od, int oh, int ow, float spatial_scale, int sampling_ratio, int aligned,
                                     int order, int* status, void* stream);
/* medvision/csrc/vision.cpp:47-48  roi_align_rotated_3d_backward  (medvision/csrc/roi_align_rotated_3d.h:98-117) */
int mvr_roi_align_rotated_3d_backward(const void* top_grad, const void* rois, void* bottom_grad, int dtype,
                                      int64_t N, int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width,
                                      int od, int oh, int ow, float spatial_scale, int sampling_ratio, int aligned,
                                      int order, int* status, void* stream);
/* medvision/csrc/vision.cpp:74  affine_2d(input, rois, output, oh, ow, spatial_scale, sampling_ratio, aligned, order)
 * (medvision/csrc/affine_2d.h) -- forward only; order may also be 3 (Catmull-Rom) */
int mvr_affine_2d(const void* input, const void* rois, void* output, int dtype,
                  int64_t N, int64_t C, int64_t H, int64_t W, int64_t R, int roi_width,
                  int oh, int ow, float spatial_scale, int sampling_ratio, int aligned, int order,
                  int* status, void* stream);
/* medvision/csrc/vision.cpp:75  affine_3d(input, rois, output, od, oh, ow, spatial_scale, sampling_ratio, aligned, order)
 * (medvision/csrc/affine_3d.h:40-65) -- forward only; order may also be 3 (Catmull-Rom) */
int mvr_affine_3d(const void* input, const void* rois, void* output, int dtype,
                  int64_t N, int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width,
                  int od, int oh, int ow, float spatial_scale, int sampling_ratio, int aligned, int order,
                  int* status, void* stream);

/* ---- label volumes -------------------------------------------------------------------- */

/* What the reference's augmentations do to a segmentation field,
 *     affine_3d(seg.float(), rois, out_size, spatial_scale, 1, aligned, order = 0).int()
 * (medvision/aug_cuda_batch/aug_spatial.py:158-194 and the `apply_to_seg` twins of the other
 * transforms), on the integer tensor itself: labels is (N, C, [D,] H, W) of label_dtype, rois is
 * FLOAT32 (R, 6 | 10) as the reference builds it, output is int32 (R, C, [od,] oh, ow).  Same
 * float32 geometry and nearest rule as mvr_affine_*; the value is (int32)(float)label.  Replaces
 * two cast passes and a float resample; has no single counterpart in the reference's extension.
 * Returns MVR_ERR_UNSUPPORTED for rois with fewer than 32 output elements (use the cast path). */
int mvr_affine_label_2d(const void* labels, int label_dtype, const float* rois, int32_t* output,
                        int64_t N, int64_t C, int64_t H, int64_t W, int64_t R, int roi_width,
                        int oh, int ow, float spatial_scale, int aligned, int* status, void* stream);
int mvr_affine_label_3d(const void* labels, int label_dtype, const float* rois, int32_t* output,
                        int64_t N, int64_t C, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width,
                        int od, int oh, int ow, float spatial_scale, int aligned, int* status, void* stream);

/* An image field and its label field of one augmentation call in one go; has no counterpart in the
 * reference, whose transforms call affine_3d twice (medvision/aug_cuda_batch/aug_spatial.py:404-446 for the
 * image, :451-493 for the label: seg.float() -> affine_3d(order 0) -> .int()).
 * image / image_rois / image_out: as mvr_affine_3d with sampling_ratio 1 (orders 0, 1); labels / label_rois /
 * label_out: as mvr_affine_label_3d (label_rois are the same rois in float32).  Results are those of the two
 * separate calls.  For dense outputs of rotated rois the label's work items ride along with the first of the
 * image's two overlapped launches, so the pair costs the launches of the image alone; other shapes fall back
 * to one launch each. */
int mvr_affine_fields_3d(const void* image, int dtype, const void* image_rois, void* image_out, int64_t C_image,
                         const void* labels, int label_dtype, const float* label_rois, int32_t* label_out,
                         int64_t C_label, int64_t N, int64_t D, int64_t H, int64_t W, int64_t R, int roi_width, int od,
                         int oh, int ow, float spatial_scale, int aligned, int order, int* status, void* stream);

/* ---- elastic warp ---------------------------------------------------------------------- */

/* out[b, c, p] = interp(img[b, c], p + offset[b, :, p]) for every voxel p; float32 / float16;
 * order 0, 1 or 3.  img and out are (B, C, H, W), offset is (B, 2, H, W) with the displacement
 * along h, then w, in pixels.  offset_dtype is the field's element type: the image's, or
 * MVR_F32 with a half image -- the field is then rounded to half as it is read, which is what
 * the reference's `offset = offset.half()` (cuda_fun_tools.py:116-119) does in a pass of its own.
 * Replaces, for the one way the reference uses it (medvision/ops/cuda_fun_tools.py:94-130
 * apply_offset_2d: 1x1 kernel, stride 1, no padding, identity weight, zero bias),
 * medvision/csrc/vision.cpp:76 deform_2d(input, weight, bias, offset, ...) -> deform_2d.h ->
 * cuda_aug/deform_2d_cuda.cu (deformable im2col + addmm + permute). */
int mvr_apply_offset_2d(const void* img, const void* offset, void* out, int dtype, int offset_dtype, int64_t B,
                        int64_t C, int64_t H, int64_t W, int order, void* stream);
/* 3D: img / out (B, C, D, H, W), offset (B, 3, D, H, W) = displacement along d, h, w.
 * Replaces medvision/csrc/vision.cpp:77 deform_3d as used by apply_offset_3d
 * (medvision/ops/cuda_fun_tools.py:133-167, cuda_aug/deform_3d_cuda.cu:44-152). */
int mvr_apply_offset_3d(const void* img, const void* offset, void* out, int dtype, int offset_dtype, int64_t B,
                        int64_t C, int64_t D, int64_t H, int64_t W, int order, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MVR_H_ */
