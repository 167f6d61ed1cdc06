// Parameter block shared by the two implementations of the dK/dV pass (mma.sync and tcgen05).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace nsa {

struct DkdvParams {
  const float2* ld;    // [Nq, Hq]
  float* dk32;         // [Nk, Hkv, D] fp32 accumulators (zeroed)
  float* dv32;
  float* dq32 = nullptr;  // sparse tcgen05 pass only: [Nq, Hq, D] fp32 accumulator (zeroed); non-null = also produce dQ
  const int* cu_q;
  const int* cu_k;      // dense: compressed cu; sparse: same as cu_q
  // sparse
  const int* cu_blocks;
  const int* offsets;
  const int* item_base;
  const int* item_bin;   // [items] bin of every work item
  int* item_counter;     // zero at launch: the persistent tcgen05 pass hands out items from it
  const int* list;
  int B, Hq, Hkv, G, TB, chunk, block_size;
  int NW;  // sparse: token windows per KV head; bin x = (head * NW + window) * TB + block

  int window, stride, causal;
  int left;  // dense pass only; >= 0: sliding window (key >= t - left, plain causal mask), < 0: none
  float scale2, sm_scale;
  Status st;
};


// dQ pass of dense strided-causal attention
struct DenseBwdParams {
  const void* q;
  const void* o;
  const void* dout;
  const float* lse;
  float2* ld;  // [Nq, Hq] (lse, delta) written by the dQ pass
  void* dq;
  const int* cu_q;
  const int* cu_k;
  long long q_sn, q_sh, o_sn, o_sh, do_sn, do_sh, dq_sn, dq_sh;
  int B, Hq, Hkv, G, logG;
  int window, stride, causal;
  int left;  // >= 0: sliding window (key >= t - left, plain causal mask), < 0: none
  float scale2, sm_scale;
  Status st;
};

// tcgen05 implementation of the dense dQ pass (dense_dq_tc.cu).  k/v strides in elements.
int dense_dq_tc(const void* k, const void* v, long long k_sn, long long k_sh, long long v_sn, long long v_sh, int total_q,
                int total_k, int max_seqlen_q, int head_dim, int dtype, DenseBwdParams p, cudaStream_t stream);

// tcgen05 dK/dV pass of the top-k sparse attention (sparse_dkdv_tc.cu); head_dim 128, group size a power of two.
// strides: q_n q_h k_n k_h v_n v_h do_n do_h (elements); grid = (work items, 64-key tiles per block).
template <typename T>
int launch_sparse_dkdv_tc(const void* q, const void* dout, const void* k, const void* v, const long long* strides, int Nk, dim3 grid,
                          DkdvParams p, cudaStream_t stream);

// tcgen05 dK/dV pass of the dense attention with the keys as the M dimension (dense_dkdv_tc.cu); head_dim 128,
// group size a power of two <= 16.  p.chunk = tokens per CTA (a multiple of 128).
template <typename T>
int launch_dense_dkdv_tc(const void* q, const void* dout, const void* k, const void* v, const long long* strides, int Nq, int Nk,
                         int max_q, int max_k, int batch, DkdvParams p, cudaStream_t stream);

}  // namespace nsa
