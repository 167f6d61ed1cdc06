// Pooling compression forward as a stream of TMA chunks through shared memory (pool_fwd_stream.cu).
#pragma once
#include <cuda_runtime.h>

namespace nsa {

// true when the streaming kernel handles this problem (enough windows to fill the device, a ring that holds a group of
// windows plus chunks in flight); otherwise the caller runs pool_fwd_kernel
bool pool_fwd_stream_eligible(int num_heads, int head_dim, int total_y, int kernel_size, int kernel_stride);

// y[m, h, :] = sum_t w[h, t] * x[cu[b] + m * stride + t, h, :]  (w == nullptr: the mean), rounded to the storage type, then
// + bias[h, :] (or nothing) in the storage type.  x [total_len, H, d] with strides (x_sn, x_sh), y [total_y, H, d] contiguous.
int pool_fwd_stream(const void* x, const void* w, const void* bias, void* y, const int* cu, const int* ycu, int batch,
                    int total_len, int total_y, int max_y_len, int num_heads, int head_dim, int kernel_size, int kernel_stride,
                    long long x_sn, long long x_sh, int dtype, cudaStream_t stream);

}  // namespace nsa
