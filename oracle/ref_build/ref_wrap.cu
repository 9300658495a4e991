// Test infrastructure, not product code.
//
// One translation unit per reference launcher file.  The reference source named by
// REF_SRC (e.g. "cuda/roi_align_rotated_3d_cuda.cu", relative to medvision/csrc of
// the reference checkout) is compiled unmodified, where it lies: it is pulled in by
// #include, never copied.  The only obstacle to building it against a current torch
// is that its launchers spell the dispatch key `tensor.type()`; all torch headers
// the reference needs are therefore included FIRST (their include guards keep them
// from being re-read), and the identifier `type` is then mapped to `scalar_type`
// for the reference's own tokens only.
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

#define type scalar_type
#include REF_SRC
#undef type
