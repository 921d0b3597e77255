// Stands in for the host-side part of the reference's src/common.cuh that callers of the attention
// operators use: the standard headers it brings along and the CK() check of CUDA runtime calls
// (src/common.cuh:3-13: throws std::runtime_error with file, line, the call and the CUDA error text).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <utility>

#ifndef CK
#define CK(x)                                                                                            \
  do {                                                                                                   \
    cudaError_t ck_e_ = (x);                                                                             \
    if (ck_e_ != cudaSuccess)                                                                            \
      throw std::runtime_error(std::string(__FILE__) + ":" + std::to_string(__LINE__) + " " + #x + " -> " + \
                               cudaGetErrorString(ck_e_));                                               \
  } while (0)
#endif
