// Warp-cooperative top-k block selection shared by the prefill and decode score kernels.
#pragma once
#include "common.cuh"

namespace nsa {

__device__ __forceinline__ bool better_pick(float v1, int b1, float v2, int b2) {  // is (v1,b1) a better pick than (v2,b2)?
  if (b1 < 0) return false;
  if (b2 < 0) return true;
  return v1 > v2 || (v1 == v2 && b1 < b2);
}

// sc[0..bq] : finite, non-negative block scores of one token in shared memory (modified in place:
// taken blocks are overwritten with +inf).  Writes `Tout` ids to out[j*out_stride]: the taken
// blocks in ascending order, then -1.  Forced blocks: b < init_blocks and b > bq - local_blocks.
// Ties go to the lower block id.  Must be called by all 32 lanes of a warp.
__device__ __forceinline__ void warp_select_topk(float* sc, int bq, int Tout, int init_blocks, int local_blocks, int* out,
                                                 long long out_stride) {
  const int lane = lane_id();
  const unsigned lt_mask = (1u << lane) - 1u;
  const int ncand = bq + 1;
  if (ncand <= Tout) {
    for (int j = lane; j < Tout; j += 32) out[j * out_stride] = j < ncand ? j : -1;
    return;
  }
  for (int bb = lane; bb < ncand; bb += 32)
    if (bb < init_blocks || bb > bq - local_blocks) sc[bb] = INFINITY;
  const int lo = max(init_blocks, bq - local_blocks + 1);
  const int nforced = min(init_blocks, ncand) + max(0, bq - lo + 1);
  const int need = max(0, Tout - nforced);
  __syncwarp();
  float best_v = -1.f;
  int best_b = -1;
  for (int bb = lane; bb < ncand; bb += 32) {
    const float v = sc[bb];
    if (v != INFINITY && v > best_v) { best_v = v; best_b = bb; }
  }
  for (int r = 0; r < need; ++r) {
    float v = best_v;
    int bb = best_b;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, off);
      const int ob = __shfl_xor_sync(0xffffffffu, bb, off);
      if (better_pick(ov, ob, v, bb)) { v = ov; bb = ob; }
    }
    if (bb < 0) break;
    if ((bb & 31) == lane) {
      sc[bb] = INFINITY;
      best_v = -1.f;
      best_b = -1;
      for (int x = lane; x < ncand; x += 32) {
        const float xv = sc[x];
        if (xv != INFINITY && xv > best_v) { best_v = xv; best_b = x; }
      }
    }
  }
  __syncwarp();
  int base = 0;
  for (int b0 = 0; b0 < ncand; b0 += 32) {
    const int bb = b0 + lane;
    const bool sel = bb < ncand && sc[bb] == INFINITY;
    const unsigned mk = __ballot_sync(0xffffffffu, sel);
    const int pos = base + __popc(mk & lt_mask);
    if (sel && pos < Tout) out[pos * out_stride] = bb;
    base += __popc(mk);
  }
  for (int j = base + lane; j < Tout; j += 32) out[j * out_stride] = -1;
  __syncwarp();
}

// weight of offset o in the key-score -> block-score fold (a = window/stride, c = block/stride)
__device__ __forceinline__ int fold_weight(int o, int a, int c) { return min(min(o, a + c - 2 - o), min(a - 1, c - 1)) + 1; }

}  // namespace nsa
