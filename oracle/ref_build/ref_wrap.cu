// Test infrastructure, not product code.
//
// One translation unit per reference launcher file.  The reference source named by
// REF_SRC (e.g. "cuda/roi_align_rotated_3d_cuda.cu", relative to medvision/csrc of
// the reference checkout) is compiled unmodified, where it lies: it is pulled in by
// #include, never copied.  The only obstacle to building it against a current torch
// is that its launchers pass `tensor.type()` (an at::DeprecatedTypeProperties) as the
// dispatch key, which AT_DISPATCH_* no longer accepts; the overload below, declared in
// the namespace where the dispatch macros look their helper up, restores that form
// without touching a single token of the reference.
#include <torch/extension.h>
#include <cuda.h>
#include <float.h>
#include <stdio.h>
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <ATen/cuda/CUDAApplyUtils.cuh>
#include <THC/THCAtomics.cuh>

#ifndef REF_SRC
#error "compile with -DREF_SRC='\"cuda/<launcher>.cu\"'"
#endif

namespace detail {
inline at::ScalarType scalar_type(const at::DeprecatedTypeProperties& t) { return t.scalarType(); }
}  // namespace detail

#include REF_SRC
