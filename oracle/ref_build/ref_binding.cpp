// Test infrastructure, not product code.
//
// Python binding for the reference's OWN dispatch functions of the resampling path
// (medvision/csrc/roi_align_{2d,3d}.h, roi_align_rotated_{2d,3d}.h, affine_{2d,3d}.h) and of the
// elastic warp (deform_{2d,3d}.h), included from the reference checkout and bound under the
// names that medvision/csrc/vision.cpp:34-48,74-77 gives them.  Only these twelve functions
// are bound, so the unrelated NMS / deformable-conv sources are not compiled.
#ifndef WITH_CUDA
#define WITH_CUDA
#endif
#include <torch/extension.h>

#include "roi_align_2d.h"
#include "roi_align_3d.h"
#include "roi_align_rotated_2d.h"
#include "roi_align_rotated_3d.h"
#include "affine_2d.h"
#include "affine_3d.h"
#include "deform_2d.h"
#include "deform_3d.h"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("roi_align_2d_forward", &roi_align_2d_forward, "roi_align_2d_forward");
  m.def("roi_align_2d_backward", &roi_align_2d_backward, "roi_align_2d_backward");
  m.def("roi_align_3d_forward", &roi_align_3d_forward, "roi_align_3d_forward");
  m.def("roi_align_3d_backward", &roi_align_3d_backward, "roi_align_3d_backward");
  m.def("roi_align_rotated_2d_forward", &roi_align_rotated_2d_forward, "roi_align_rotated_2d_forward");
  m.def("roi_align_rotated_2d_backward", &roi_align_rotated_2d_backward, "roi_align_rotated_2d_backward");
  m.def("roi_align_rotated_3d_forward", &roi_align_rotated_3d_forward, "roi_align_rotated_3d_forward");
  m.def("roi_align_rotated_3d_backward", &roi_align_rotated_3d_backward, "roi_align_rotated_3d_backward");
  m.def("affine_2d", &affine_2d, "affine_2d");
  m.def("affine_3d", &affine_3d, "affine_3d");
  m.def("deform_2d", &deform_2d, "deform_2d");
  m.def("deform_3d", &deform_3d, "deform_3d");
}
