// Pooling compression backward as chunk streams (pool_bwd_stream.cu): dx and the per-tap partial sums of dw in one pass.
#pragma once
#include <cuda_runtime.h>

namespace nsa {

bool pool_bwd_stream_eligible(int num_heads, int head_dim, int total_len, int kernel_size, int kernel_stride);

// fp32 words of workspace the streaming pass needs for the partial sums of dw (0 when it does not run)
long long pool_bwd_stream_partial_floats(int num_heads, int head_dim, int total_len, int batch, int max_seqlen,
                                         int kernel_size, int kernel_stride);

// dx [total_len, H, 128] contiguous <- dy, w;  when w != nullptr also partial[slot][H][ks] (fp32, `slots` of them, zeroed
// here) <- x, dy, to be summed in slot order by the caller.  Returns the number of slots through *slots.
int pool_bwd_stream(const void* x, const void* w, const void* dy, void* dx, float* partial, int* slots, const int* cu,
                    const int* ycu, int batch, int total_len, int max_seqlen, int num_heads, int head_dim, int kernel_size,
                    int kernel_stride, long long x_sn, long long x_sh, int dtype, cudaStream_t stream);

}  // namespace nsa
