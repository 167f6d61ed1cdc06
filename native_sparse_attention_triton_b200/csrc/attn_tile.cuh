// Warp-level tile arithmetic shared by all attention kernels.
//
// One warp owns a 16-row tile (the query heads of one KV group, for one or a few
// query tokens).  Operand tiles live in 128B-swizzled shared memory exactly as TMA
// wrote them: [rows][64*panels] 16-bit elements, see swz_addr in common.cuh.
#pragma once
#include "common.cuh"

namespace nsa {

constexpr int kKeyTile = 64;  // keys per shared-memory tile
constexpr float kLog2e = 1.4426950408889634f;

// C[16 x 8*NT] += A[16 x 16*KS] * B^T ; the tile stores B as [n][k] (k contiguous).
// n0: first tile row used, kchunk0: first 16-byte chunk (8 elements) of the k range.
template <typename T, int NT, int KS, int ROWS>
__device__ __forceinline__ void mma_nk(float (&c)[NT][4], const uint32_t (&a)[KS][4], uint32_t tile, int n0, int kchunk0) {
  const int l = lane_id();
  const int row_in = (l & 7) + ((l >> 4) << 3);
  const int ch_in = (l >> 3) & 1;
#pragma unroll
  for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
    for (int jp = 0; jp < NT / 2; ++jp) {
      uint32_t b[4];
      ldmatrix_x4(b, swz_addr<ROWS>(tile, n0 + jp * 16 + row_in, kchunk0 + 2 * kk + ch_in));
      DT<T>::mma(c[2 * jp], a[kk], b[0], b[1]);
      DT<T>::mma(c[2 * jp + 1], a[kk], b[2], b[3]);
    }
  }
}

// C[16 x 8*NT] += A[16 x 16*KS] * B ; the tile stores B as [k][n] (n contiguous).
// k0: first tile row used, nchunk0: first 16-byte chunk of the n range.
template <typename T, int NT, int KS, int ROWS>
__device__ __forceinline__ void mma_kn(float (&c)[NT][4], const uint32_t (&a)[KS][4], uint32_t tile, int k0, int nchunk0) {
  const int l = lane_id();
  const int row_in = (l & 7) + (((l >> 3) & 1) << 3);
  const int ch_in = l >> 4;
#pragma unroll
  for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
    for (int jp = 0; jp < NT / 2; ++jp) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, swz_addr<ROWS>(tile, k0 + kk * 16 + row_in, nchunk0 + 2 * jp + ch_in));
      DT<T>::mma(c[2 * jp], a[kk], b[0], b[1]);
      DT<T>::mma(c[2 * jp + 1], a[kk], b[2], b[3]);
    }
  }
}

// A-operand fragments of a [16 x 16*KS] row-major tile in swizzled shared memory.
template <int KS, int ROWS>
__device__ __forceinline__ void load_a_frags(uint32_t (&a)[KS][4], uint32_t tile, int m0, int kchunk0) {
  const int l = lane_id();
  const int row_in = (l & 7) + (((l >> 3) & 1) << 3);
  const int ch_in = l >> 4;
#pragma unroll
  for (int kk = 0; kk < KS; ++kk) ldmatrix_x4(a[kk], swz_addr<ROWS>(tile, m0 + row_in, kchunk0 + 2 * kk + ch_in));
}

// A-operand fragments of a 16-row tile read straight from global memory.
// rowptr(r) returns the address of row r (r in 0..15) or nullptr for a padding row.
template <typename T, int KS, typename RowPtr>
__device__ __forceinline__ void load_a_frags_global(uint32_t (&a)[KS][4], RowPtr rowptr) {
  const int l = lane_id();
  const T* r0 = rowptr(l >> 2);
  const T* r1 = rowptr((l >> 2) + 8);
  const int c = (l & 3) * 2;
#pragma unroll
  for (int kk = 0; kk < KS; ++kk) {
    a[kk][0] = r0 ? __ldg(reinterpret_cast<const uint32_t*>(r0 + kk * 16 + c)) : 0u;
    a[kk][1] = r1 ? __ldg(reinterpret_cast<const uint32_t*>(r1 + kk * 16 + c)) : 0u;
    a[kk][2] = r0 ? __ldg(reinterpret_cast<const uint32_t*>(r0 + kk * 16 + c + 8)) : 0u;
    a[kk][3] = r1 ? __ldg(reinterpret_cast<const uint32_t*>(r1 + kk * 16 + c + 8)) : 0u;
  }
}

// accumulator fragments [16 x 16*KS] (fp32) -> A-operand fragments (16-bit)
template <typename T, int KS>
__device__ __forceinline__ void acc_to_a_frags(uint32_t (&a)[KS][4], const float (&s)[2 * KS][4]) {
#pragma unroll
  for (int kk = 0; kk < KS; ++kk) {
    a[kk][0] = DT<T>::pack(s[2 * kk][0], s[2 * kk][1]);
    a[kk][1] = DT<T>::pack(s[2 * kk][2], s[2 * kk][3]);
    a[kk][2] = DT<T>::pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[kk][3] = DT<T>::pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
  }
}

// One online-softmax step over a [16 x 64] logit tile (base-2 domain).
//   s    : raw dot products; on return the probabilities relative to the new running max
//   lim  : per fragment row (lane/4 and lane/4+8), number of leading visible keys of this tile
//   m, l : running max (already scaled) and running sum
//   o    : output accumulator, rescaled in place
template <int NT_O>
__device__ __forceinline__ void online_softmax_step(float (&s)[8][4], const int (&lim)[2], float scale2, float (&m)[2],
                                                    float (&l)[2], float (&o)[NT_O][4]) {
  const int c0 = (lane_id() & 3) * 2;
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = e >> 1;
      const int col = j * 8 + c0 + (e & 1);
      float v = (col < lim[r]) ? s[j][e] * scale2 : -INFINITY;
      s[j][e] = v;
      mx[r] = fmaxf(mx[r], v);
    }
  }
  float corr[2], mnew[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = quad_max(mx[r]);
    mnew[r] = fmaxf(m[r], mx[r]);
    const float msafe = (mnew[r] == -INFINITY) ? 0.f : mnew[r];
    corr[r] = fast_exp2(m[r] - msafe);  // m = -inf -> 0
    m[r] = mnew[r];
    mnew[r] = msafe;
  }
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = e >> 1;
      float p = fast_exp2(s[j][e] - mnew[r]);
      s[j][e] = p;
      sum[r] += p;
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) l[r] = l[r] * corr[r] + quad_sum(sum[r]);
#pragma unroll
  for (int j = 0; j < NT_O; ++j) {
    o[j][0] *= corr[0];
    o[j][1] *= corr[0];
    o[j][2] *= corr[1];
    o[j][3] *= corr[1];
  }
}

// One warp attends over a private list of 64-key tiles with a private two-buffer TMA pipeline
// (K tile and V tile, the next one of each kind in flight while the current one is used).
//   tile_at(i, kpos, lim) : position token of tile i and its number of leading visible keys
//   issue(is_v, kpos)     : lane 0 starts the TMA load of that tile into kbuf / vbuf (with expect_tx)
// barK / barV are single-arrival mbarriers owned by the warp; `phase` carries their parity.
// on_scores(kpos, limv, s) sees every tile's raw logits (mma accumulator layout, before scaling and masking).
struct NoScoreHook {
  __device__ __forceinline__ void operator()(int, int, const float (&)[8][4]) const {}
};
template <typename T, int D, typename TileAt, typename Issue, typename OnScores = NoScoreHook>
__device__ __forceinline__ void warp_attend_tiles(const uint32_t (&qf)[D / 16][4], float (&o)[D / 8][4], float (&m)[2],
                                                  float (&l)[2], int ntiles, uint32_t kbuf, uint32_t vbuf, uint64_t* barK,
                                                  uint64_t* barV, uint32_t& phase, float scale2, const Status& st,
                                                  TileAt tile_at, Issue issue, OnScores on_scores = OnScores(),
                                                  bool first_tile_issued = false) {
  const int lane = lane_id();
  if (ntiles > 0 && lane == 0 && !first_tile_issued) {
    int kpos, limv;
    tile_at(0, kpos, limv);
    issue(false, kpos);
    issue(true, kpos);
  }
  for (int i = 0; i < ntiles; ++i) {
    int kpos, limv, knext = 0, ldummy;
    tile_at(i, kpos, limv);
    if (i + 1 < ntiles) tile_at(i + 1, knext, ldummy);
    mbar_wait(barK, phase, st);
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    mma_nk<T, 8, D / 16, kKeyTile>(s, qf, kbuf, 0, 0);
    __syncwarp();
    if (i + 1 < ntiles && lane == 0) issue(false, knext);
    on_scores(kpos, limv, s);
    const int lim[2] = {limv, limv};
    online_softmax_step<D / 8>(s, lim, scale2, m, l, o);
    uint32_t pf[4][4];
    acc_to_a_frags<T, 4>(pf, s);
    mbar_wait(barV, phase, st);
    mma_kn<T, D / 8, 4, kKeyTile>(o, pf, vbuf, 0, 0);
    __syncwarp();
    if (i + 1 < ntiles && lane == 0) issue(true, knext);
    phase ^= 1;
  }
}

// Write a warp's [16 x D] fp32 accumulator as 16-bit rows through a shared staging area
// (>= 16*(D+8)*2 bytes, private to the warp), 16 bytes per lane per store.
// rowptr(r) gives the destination of row r or nullptr to skip it.
template <typename T, int D, typename RowPtr>
__device__ __forceinline__ void store_rows_staged(const float (&o)[D / 8][4], const float (&rscale)[2], T* stage, RowPtr rowptr) {
  constexpr int LD = D + 8;  // padding keeps the 4-byte fragment stores conflict-free
  const int l = lane_id();
  const int r0 = l >> 2, c0 = (l & 3) * 2;
  __syncwarp();
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    *reinterpret_cast<uint32_t*>(stage + r0 * LD + j * 8 + c0) = DT<T>::pack(o[j][0] * rscale[0], o[j][1] * rscale[0]);
    *reinterpret_cast<uint32_t*>(stage + (r0 + 8) * LD + j * 8 + c0) = DT<T>::pack(o[j][2] * rscale[1], o[j][3] * rscale[1]);
  }
  __syncwarp();
  constexpr int CH = D / 8;  // 16-byte chunks per row
#pragma unroll
  for (int it = 0; it < 16 * CH / 32; ++it) {
    const int idx = it * 32 + l;
    const int r = idx / CH, ch = idx % CH;
    T* dst = rowptr(r);
    if (dst) *reinterpret_cast<uint4*>(dst + ch * 8) = *reinterpret_cast<const uint4*>(stage + r * LD + ch * 8);
  }
  __syncwarp();
}

}  // namespace nsa
