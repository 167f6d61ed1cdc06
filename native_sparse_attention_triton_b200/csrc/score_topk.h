// Parameter block shared by the two implementations of the score / top-k kernel (mma.sync and tcgen05).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace nsa {

struct ScoreParams {
  const void* q;
  const float* lse;  // [Nq, Hq] base-2
  int* topk_idx;
  const int* cu_q;
  const int* cu_k;
  long long q_sn, q_sh;
  long long t_sh, t_sn, t_sk;
  int B, Hq, Hkv, G, logG;
  int window, stride, block_size;
  int topk_out, init_blocks, local_blocks, nb_pad;
  int nwarps;
  float scale2;
  Status st;
};

// tcgen05 implementation (score_topk_tc.cu).  Returns kUnsupported when the per-token block scores of one CTA
// do not fit in shared memory, in which case the caller uses the mma.sync kernel.
int score_topk_tc(const void* q, const void* k, long long k_sn, long long k_sh, int Nq, int Nk, int max_seqlen_q, int head_dim,
                  int dtype, ScoreParams p, cudaStream_t stream);

// tcgen05 implementation with two row tiles per CTA (score_topk_pp_tc.cu); same contract, tighter shared-memory limit.
int score_topk_pp_tc(const void* q, const void* k, long long k_sn, long long k_sh, int Nq, int Nk, int max_seqlen_q, int head_dim,
                     int dtype, ScoreParams p, cudaStream_t stream);

}  // namespace nsa
