// Linear compression forward on the 5th-generation tensor cores (linear_fwd_tc.cu).
#pragma once
#include <cuda_runtime.h>

namespace nsa {

// true when the tcgen05 kernel handles this problem (head_dim 128, tiles of 128 windows worth filling, enough tokens for
// the two tensor maps that cover x); otherwise the caller runs linear_fwd_kernel
bool linear_fwd_tc_eligible(int head_dim, int max_y_len, int total_len, int kernel_size, int kernel_stride);

// y[m, h, :] = sum_tap x[cu[b] + m * stride + tap, h, :] @ w[h, tap * d:(tap + 1) * d, :], rounded to the storage type,
// then + bias[h, :] (or nothing) in the storage type.  x [total_len, H, 128] with strides (x_sn, x_sh), w [H, ks * 128, 128]
// and y [total_y, H, 128] contiguous.
int linear_fwd_tc(const void* x, const void* w, const void* bias, void* y, const int* cu, const int* ycu, int batch,
                  int max_y_len, int total_len, int num_heads, int kernel_size, int kernel_stride, long long x_sn,
                  long long x_sh, int dtype, cudaStream_t stream);

}  // namespace nsa
