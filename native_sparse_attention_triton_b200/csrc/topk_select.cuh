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
__device__ __forceinline__ void warp_select_topk_smem(float* sc, int bq, int Tout, int init_blocks, int local_blocks, int* out,
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

// Same contract as warp_select_topk_smem for bq < 1024: every lane keeps its 32 candidates (block ids lane, lane+32, ...)
// in registers, so a selection round is 32 register compares plus a 5-step warp argmax instead of a shared-memory rescan.
template <int NJ>
__device__ __forceinline__ void warp_select_topk_reg(float* sc, int bq, int Tout, int init_blocks, int local_blocks, int* out,
                                                     long long out_stride);

__device__ __forceinline__ void warp_select_topk(float* sc, int bq, int Tout, int init_blocks, int local_blocks, int* out,
                                                 long long out_stride) {
  const int ncand = bq + 1;
  if (ncand > 1024) warp_select_topk_smem(sc, bq, Tout, init_blocks, local_blocks, out, out_stride);
  else if (ncand > 512) warp_select_topk_reg<32>(sc, bq, Tout, init_blocks, local_blocks, out, out_stride);
  else if (ncand > 256) warp_select_topk_reg<16>(sc, bq, Tout, init_blocks, local_blocks, out, out_stride);
  else warp_select_topk_reg<8>(sc, bq, Tout, init_blocks, local_blocks, out, out_stride);
}

// NJ = candidates per lane (block ids lane, lane + 32, ..., lane + 32*(NJ-1)); requires bq < 32*NJ.
template <int NJ>
__device__ __forceinline__ void warp_select_topk_reg(float* sc, int bq, int Tout, int init_blocks, int local_blocks, int* out,
                                                     long long out_stride) {
  const int ncand = bq + 1;
  const int lane = lane_id();
  const unsigned lt_mask = (1u << lane) - 1u;
  if (ncand <= Tout) {
    for (int j = lane; j < Tout; j += 32) out[j * out_stride] = j < ncand ? j : -1;
    return;
  }
  // scores are non-negative, so their bit patterns order like unsigned integers; -1 marks "not a candidate"
  int v[NJ];
  unsigned taken = 0u;  // bit j: candidate j*32 + lane is selected
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int bb = j * 32 + lane;
    int x = -1;
    if (bb < ncand) {
      if (bb < init_blocks || bb > bq - local_blocks) taken |= 1u << j; else x = __float_as_int(fmaxf(sc[bb], 0.f));
    }
    v[j] = x;
  }
  const int nforced = __reduce_add_sync(0xffffffffu, __popc(taken));
  const int need = max(0, Tout - nforced);
  for (int r = 0; r < need; ++r) {
    // local (max, lowest index holding it) by a tree: on ties the lower j wins
    int tv[NJ], tj[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) { tv[j] = v[j]; tj[j] = j; }
#pragma unroll
    for (int w = NJ / 2; w >= 1; w >>= 1)
#pragma unroll
      for (int j = 0; j < w; ++j) {
        const bool hi = tv[j + w] > tv[j];   // strict: equal values keep the lower index (j < j + w)
        tv[j] = hi ? tv[j + w] : tv[j];
        tj[j] = hi ? tj[j + w] : tj[j];
      }
    const int wmx = __reduce_max_sync(0xffffffffu, tv[0]);
    if (wmx < 0) break;  // no candidate left
    const int mine = tv[0] == wmx ? tj[0] * 32 + lane : 0x7fffffff;
    const int wb = __reduce_min_sync(0xffffffffu, mine);
    if ((wb & 31) == lane) {
      const int jw = wb >> 5;
      taken |= 1u << jw;
#pragma unroll
      for (int j = 0; j < NJ; ++j)
        if (j == jw) v[j] = -1;
    }
  }
  // emit ascending: only the 32-id groups that hold a selected block are visited
  int base = 0;
  unsigned groups = __reduce_or_sync(0xffffffffu, taken);
  while (groups) {
    const int j = __ffs(groups) - 1;
    groups &= groups - 1;
    const bool sel = (taken >> j) & 1u;
    const unsigned mk = __ballot_sync(0xffffffffu, sel);
    const int pos = base + __popc(mk & lt_mask);
    if (sel && pos < Tout) out[pos * out_stride] = j * 32 + lane;
    base += __popc(mk);
  }
  for (int j = base + lane; j < Tout; j += 32) out[j * out_stride] = -1;
  __syncwarp();
}

// weight of offset o in the key-score -> block-score fold (a = window/stride, c = block/stride)
__device__ __forceinline__ int fold_weight(int o, int a, int c) { return min(min(o, a + c - 2 - o), min(a - 1, c - 1)) + 1; }

}  // namespace nsa
