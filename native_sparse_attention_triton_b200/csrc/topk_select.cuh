// Warp-cooperative top-k block selection shared by the prefill and decode score kernels.
#pragma once
#include "common.cuh"

namespace nsa {

// sc[0..bq] : finite, non-negative block scores of one token in shared memory (modified in place: taken blocks are
// overwritten with +inf, candidates a lane has pulled into its cache with -1).  Writes `Tout` ids to out[j*out_stride]:
// the taken blocks in ascending order, then -1.  Forced blocks: b < init_blocks and b > bq - local_blocks.
// Ties go to the lower block id.  Must be called by all 32 lanes of a warp.
//
// Lane l owns the candidates l, l+32, ...  It keeps its C best remaining ones in a small sorted cache (filled by one
// rolled scan of its candidates), so a selection round is two warp reductions and a cache pop; a lane rescans only
// after it has won C rounds.  The code is deliberately compact (rolled loops, candidates left in shared memory): the
// selection runs once per CTA, and a fully unrolled register version spent its time fetching instructions.
__device__ __forceinline__ void warp_select_topk(float* sc, int bq, int Tout, int init_blocks, int local_blocks, int* out,
                                                 long long out_stride) {
  constexpr int C = 4;
  const int lane = lane_id();
  const unsigned lt_mask = (1u << lane) - 1u;
  const int ncand = bq + 1;
  if (ncand <= Tout) {
    for (int j = lane; j < Tout; j += 32) out[j * out_stride] = j < ncand ? j : -1;
    return;
  }
  // forced blocks: [0, n_init) and [lo, bq]
  const int n_init = min(init_blocks, ncand);
  const int lo = max(n_init, bq - local_blocks + 1);
  const int nforced = n_init + (bq - lo + 1);
  for (int bb = lane; bb < n_init; bb += 32) sc[bb] = INFINITY;
  for (int bb = lo + lane; bb <= bq; bb += 32) sc[bb] = INFINITY;
  const int need = max(0, Tout - nforced);
  // scores are non-negative, so their bit patterns order like integers; -1 marks an empty cache slot
  int cv[C], cb[C];
  bool exhausted = false;  // nothing left to scan for this lane
  auto refill = [&](bool active) {
    if (active) {
#pragma unroll
      for (int c = 0; c < C; ++c) { cv[c] = -1; cb[c] = 0; }
      auto offer = [&](int val, int x) {
        if (val == static_cast<int>(0x80000000u)) val = 0;  // -0.0 is a score of zero, not a marker
        if (val >= 0 && val < 0x7f800000 && val > cv[C - 1]) {  // a live candidate that beats the cache's last entry
          cv[C - 1] = val;
          cb[C - 1] = x;
#pragma unroll
          for (int c = C - 1; c >= 1; --c)
            if (cv[c] > cv[c - 1]) {  // strict: on ties the earlier (lower) id stays ahead
              const int tv = cv[c], tb = cb[c];
              cv[c] = cv[c - 1]; cb[c] = cb[c - 1];
              cv[c - 1] = tv; cb[c - 1] = tb;
            }
        }
      };
      // four loads in flight per step: the scan is bound by shared-memory latency, not by the compares
#pragma unroll 1
      for (int x = lane; x < ncand; x += 128) {
        int vals[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) vals[u] = (x + 32 * u < ncand) ? __float_as_int(sc[x + 32 * u]) : -1;
#pragma unroll
        for (int u = 0; u < 4; ++u) offer(vals[u], x + 32 * u);
      }
#pragma unroll
      for (int c = 0; c < C; ++c)
        if (cv[c] >= 0) sc[cb[c]] = -1.f;  // now lives in the cache
      exhausted = cv[C - 1] < 0;
    }
  };
  __syncwarp();
  refill(true);
  int my_id = -1;  // lane i < nforced + (rounds won so far) holds the i-th taken block (forced ones first)
  if (lane < n_init) my_id = lane; else if (lane < nforced) my_id = lo + (lane - n_init);
  int ntaken = nforced;
  for (int r = 0; r < need; ++r) {
    const bool empty = cv[0] < 0 && !exhausted;
    if (__any_sync(0xffffffffu, empty)) refill(empty);
    const int wmx = __reduce_max_sync(0xffffffffu, cv[0]);
    if (wmx < 0) break;  // no candidate left
    const int wb = __reduce_min_sync(0xffffffffu, cv[0] == wmx ? cb[0] : 0x7fffffff);
    if (lane == ntaken) my_id = wb;
    ++ntaken;
    if ((wb & 31) == lane) {
      sc[wb] = INFINITY;
#pragma unroll
      for (int c = 0; c + 1 < C; ++c) { cv[c] = cv[c + 1]; cb[c] = cb[c + 1]; }
      cv[C - 1] = -1;
    }
  }
  __syncwarp();
  if (nforced <= Tout && Tout <= 32) {
    // emit ascending: at most 32 taken blocks, one per lane; a block's output position is the number of smaller ids
    int rank = 0;
#pragma unroll 1
    for (int j = 0; j < ntaken; ++j) rank += __shfl_sync(0xffffffffu, my_id, j) < my_id ? 1 : 0;
    if (lane < ntaken) out[rank * out_stride] = my_id;
    for (int j = ntaken + lane; j < Tout; j += 32) out[j * out_stride] = -1;
  } else {
    // general case: scan the marks in ascending order
    int base = 0;
#pragma unroll 1
    for (int b0 = 0; b0 < ncand && base < Tout; b0 += 32) {
      const int bb = b0 + lane;
      const bool sel = bb < ncand && sc[bb] == INFINITY;
      const unsigned mk = __ballot_sync(0xffffffffu, sel);
      const int pos = base + __popc(mk & lt_mask);
      if (sel && pos < Tout) out[pos * out_stride] = bb;
      base += __popc(mk);
    }
    for (int j = base + lane; j < Tout; j += 32) out[j * out_stride] = -1;
  }
  __syncwarp();
}

// weight of offset o in the key-score -> block-score fold (a = window/stride, c = block/stride)
__device__ __forceinline__ int fold_weight(int o, int a, int c) { return min(min(o, a + c - 2 - o), min(a - 1, c - 1)) + 1; }

}  // namespace nsa
