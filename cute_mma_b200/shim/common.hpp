// Error convention of the C++ shim: like the reference's GEMM_CHECK_CUDA (common.hpp:8-14) a failed
// call throws std::runtime_error; the text carries the library's own message.
#pragma once
#include <stdexcept>
#include <string>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/cute_mma_b200.h"

#define GEMM_LIKELY(x) __builtin_expect(!!(x), 1)
#define GEMM_UNLIKELY(x) __builtin_expect(!!(x), 0)

#define GEMM_CHECK_CUDA(call)                                                                              \
  do {                                                                                                     \
    cudaError_t status_ = (call);                                                                          \
    if (GEMM_UNLIKELY(status_ != cudaSuccess))                                                             \
      throw std::runtime_error("CUDA call failed with status " + std::to_string(static_cast<int>(status_))); \
  } while (0)

#define B200_CHECK(call)                                                                                   \
  do {                                                                                                     \
    int status_ = (call);                                                                                  \
    if (GEMM_UNLIKELY(status_ != B200_OK))                                                                 \
      throw std::runtime_error("cute_mma_b200 call failed with status " + std::to_string(status_) + ": " + \
                               b200_last_error());                                                         \
  } while (0)
