#pragma once

// Operator boundary of the ring-attention forward for CUDA/C++ callers.
//
// The reference's include/attention_api.cuh (lines 1-30) declares no function: it holds the
// torch-extension style argument checks and a CUDA error macro.  Those macro names are kept here;
// the entry points themselves are the extern "C" functions of ring_attention_b200.h, and the
// argument block is Ring_fwd_params (csrc/ring.h:5-19 of the reference, extended in this repository).

#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>

#include "ring_attention_b200.h"
#include "../ringattention_b200/csrc/ring.h"

// The tensor checks need torch/extension.h; they are only defined for translation units that
// include it themselves (the pure C-ABI build does not depend on torch).
#if defined(TORCH_EXTENSION_NAME) || defined(TORCH_CHECK)
#define CHECK_CUDA(x) TORCH_CHECK(x.device().is_cuda(), #x " must be a CUDA tensor")
#define CHECK_CONTIGUOUS(x) TORCH_CHECK(x.is_contiguous(), #x " must be contiguous")
#define CHECK_INPUT(x) \
  CHECK_CUDA(x);       \
  CHECK_CONTIGUOUS(x)
#endif

// For application code (drivers, tests).  Library code returns RingStatus instead of exiting.
#ifndef CUDA_ERROR_CHECK
#define CUDA_ERROR_CHECK(condition)                                                          \
  do {                                                                                       \
    cudaError_t error_ = (condition);                                                        \
    if (error_ != cudaSuccess) {                                                             \
      std::printf("CUDA_CHECK error in line %d of file %s : %s \n", __LINE__, __FILE__,      \
                  cudaGetErrorString(error_));                                               \
      std::exit(EXIT_FAILURE);                                                               \
    }                                                                                        \
  } while (0)
#endif
