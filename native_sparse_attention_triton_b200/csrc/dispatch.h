// dtype / head-dim dispatch for the extern "C" entry points.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

// dtype codes of the C interface
#define NSA_DTYPE_BF16 0
#define NSA_DTYPE_FP16 1

// Calls FN<T, D>(...) for the supported (dtype, head_dim) pairs; evaluates to kUnsupported otherwise.
#define NSA_DISPATCH_T_D(dtype, head_dim, FN, ...)                                      \
  ((dtype) == NSA_DTYPE_BF16                                                            \
       ? ((head_dim) == 128 ? FN<__nv_bfloat16, 128>(__VA_ARGS__)                       \
                            : ((head_dim) == 64 ? FN<__nv_bfloat16, 64>(__VA_ARGS__)    \
                                                : (int)nsa::kUnsupported))              \
       : ((dtype) == NSA_DTYPE_FP16                                                     \
              ? ((head_dim) == 128 ? FN<__half, 128>(__VA_ARGS__)                       \
                                   : ((head_dim) == 64 ? FN<__half, 64>(__VA_ARGS__)    \
                                                       : (int)nsa::kUnsupported))       \
              : (int)nsa::kUnsupported))
