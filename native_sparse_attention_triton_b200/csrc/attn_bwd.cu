// Backward of the two trainable attention operators.
//
//   dQ pass   : query-stationary, same tiling as the forward kernels (dense: CTA-shared TMA ring,
//               sparse: per-warp TMA pipeline over the selected blocks).  Recomputes
//               P = exp2(S*scale - lse), dP = dO V^T, dS = P (dP - delta) scale, dQ += dS K.
//               It also produces delta[n, hq] = sum_d O * dO and stores (lse, delta) pairs for
//               the second pass.
//   dK/dV pass: key-tile-stationary.  A CTA owns 64 keys (one warp per 16 keys, K/V tile resident
//               in shared memory) and streams query "slots" -- the G query heads of one token,
//               fetched as one TMA box from q and dO -- through a multi-stage ring fed by a
//               producer warp.  Dense attention walks a contiguous token range; sparse attention
//               walks the list of tokens that selected the block (an inverted index built on the
//               device by histogram -> scan -> scatter).  The G heads are reduced on the mma K
//               dimension, so no per-head dK/dV copies exist.  Partial results of the CTAs that
//               share a key tile are added with fp32 red.global into a zeroed accumulator and
//               converted to the storage type at the end.
#include <cstdlib>
#include <utility>

#include "attn_tile.cuh"
#include "dispatch.h"
#include "host_util.h"
#include "nsa_b200.h"
#include "attn_bwd.h"

namespace nsa {

constexpr int kMaxTilesBwd = 64;

// ------------------------------------------------------------------------------------------------
// shared tile arithmetic of the dQ pass
// ------------------------------------------------------------------------------------------------
template <typename T, int D>
__device__ __forceinline__ void dq_tile(const uint32_t (&qf)[D / 16][4], const uint32_t (&dof)[D / 16][4],
                                        float (&dq)[D / 8][4], uint32_t kbuf, uint32_t vbuf, const int (&lim)[2],
                                        const float (&lse2)[2], const float (&delta)[2], float scale2, float sm_scale) {
  const int c0 = (lane_id() & 3) * 2;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    float s[4][4], dp[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      dp[j][0] = dp[j][1] = dp[j][2] = dp[j][3] = 0.f;
    }
    mma_nk<T, 4, D / 16, kKeyTile>(s, qf, kbuf, 32 * half, 0);
    mma_nk<T, 4, D / 16, kKeyTile>(dp, dof, vbuf, 32 * half, 0);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const int col = 32 * half + j * 8 + c0 + (e & 1);
        const float pr = masked_exp2(col < lim[r], s[j][e] * scale2 - lse2[r]);
        s[j][e] = pr * (dp[j][e] - delta[r]) * sm_scale;
      }
    }
    uint32_t dsf[2][4];
    acc_to_a_frags<T, 2>(dsf, s);
    mma_kn<T, D / 8, 2, kKeyTile>(dq, dsf, kbuf, 32 * half, 0);
  }
}

// delta of the two fragment rows of this lane from O and dO rows in global memory
template <typename T, int D>
__device__ __forceinline__ void row_delta(const T* o0, const T* o1, const uint32_t (&dof)[D / 16][4], float (&delta)[2]) {
  const int c = (lane_id() & 3) * 2;
  float a0 = 0.f, a1 = 0.f;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
    for (int hi = 0; hi < 2; ++hi) {
      if (o0) {
        const float2 ov = DT<T>::unpack(__ldg(reinterpret_cast<const uint32_t*>(o0 + kk * 16 + c + 8 * hi)));
        const float2 dv = DT<T>::unpack(dof[kk][2 * hi]);
        a0 += ov.x * dv.x + ov.y * dv.y;
      }
      if (o1) {
        const float2 ov = DT<T>::unpack(__ldg(reinterpret_cast<const uint32_t*>(o1 + kk * 16 + c + 8 * hi)));
        const float2 dv = DT<T>::unpack(dof[kk][2 * hi + 1]);
        a1 += ov.x * dv.x + ov.y * dv.y;
      }
    }
  }
  delta[0] = quad_sum(a0);
  delta[1] = quad_sum(a1);
}

// ------------------------------------------------------------------------------------------------
// sparse dQ
// ------------------------------------------------------------------------------------------------
struct SparseBwdParams {
  const void* q;
  const void* o;
  const void* dout;
  const float* lse;
  float2* ld;
  void* dq;
  const int* topk_idx;
  const int* cu_seqlens;
  long long q_sn, q_sh, o_sn, o_sh, do_sn, do_sh, dq_sn, dq_sh;
  long long t_sh, t_sn, t_sk;
  int N, B, Hq, Hkv, G, T, block_size;
  float scale2, sm_scale;
  Status st;
};

template <typename T, int D, int WARPS, int KBUFS>
__global__ void __launch_bounds__(WARPS * 32, 1)
sparse_dq_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, SparseBwdParams p) {
  constexpr int TILE_BYTES = kKeyTile * D * 2;
  constexpr int PANELS = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* kbuf = smem + warp * (KBUFS + 1) * TILE_BYTES;  // KBUFS K tiles, then one V tile
  uint8_t* vbuf = kbuf + KBUFS * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + WARPS * (KBUFS + 1) * TILE_BYTES);
  uint64_t* barK = bars + (KBUFS + 1) * warp;  // [KBUFS]
  uint64_t* barV = barK + KBUFS;
  int* tiles = reinterpret_cast<int*>(bars + (KBUFS + 1) * WARPS) + warp * kMaxTilesBwd;
  const int n = blockIdx.x * WARPS + warp;
  if (n >= p.N) return;
  const int h = blockIdx.y;
  if (lane == 0) {
    for (int kb = 0; kb < KBUFS; ++kb) mbar_init(barK + kb, 1);
    mbar_init(barV, 1);
    fence_barrier_init();
  }
  __syncwarp();
  const int b = find_sequence(p.cu_seqlens, p.B, n);
  const int s0 = __ldg(p.cu_seqlens + b);
  const int t = n - s0;
  const int BS = p.block_size, bq = t / BS, nsub = BS / kKeyTile;
  int ntiles = 0;
  const int* tptr = p.topk_idx + h * p.t_sh + (long long)n * p.t_sn;
  for (int base = 0; base < p.T; base += 32) {
    const int j = base + lane;
    const int idx = (j < p.T) ? __ldg(tptr + j * p.t_sk) : -1;
    const bool valid = idx >= 0 && idx <= bq;
    const int cnt = valid ? min(nsub, (t - idx * BS) / kKeyTile + 1) : 0;
    int incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    const int excl = incl - cnt;
    for (int s = 0; s < cnt; ++s) {
      const int pos = ntiles + excl + s;
      if (pos < kMaxTilesBwd) tiles[pos] = idx * BS + s * kKeyTile;
    }
    ntiles += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (ntiles > kMaxTilesBwd) {
    p.st.raise(kErrBadIndex);
    ntiles = kMaxTilesBwd;
  }
  __syncwarp();
  // K and V tiles have a barrier each: dP = dO V^T comes first, so the next V tile is requested as soon as dP is done
  // and travels under the S, dS and dQ products.  With one K buffer the next K tile is requested at the end of a tile
  // and travels under the next dP; with two it is requested a whole tile ahead.
  auto issue_k = [&](int i) {
    uint8_t* dst = kbuf + (i % KBUFS) * TILE_BYTES;
    mbar_expect_tx(barK + (i % KBUFS), TILE_BYTES);
#pragma unroll
    for (int pn = 0; pn < PANELS; ++pn) tma_load_3d(dst + pn * (kKeyTile * 128), &tmK, barK + (i % KBUFS), pn * 64, h, s0 + tiles[i]);
  };
  auto issue_v = [&](int kpos) {
    mbar_expect_tx(barV, TILE_BYTES);
#pragma unroll
    for (int pn = 0; pn < PANELS; ++pn) tma_load_3d(vbuf + pn * (kKeyTile * 128), &tmV, barV, pn * 64, h, s0 + kpos);
  };
  if (ntiles > 0 && lane == 0) {
    issue_v(tiles[0]);
    issue_k(0);
    if (KBUFS > 1 && ntiles > 1) issue_k(1);
  }

  const int r_lo = lane >> 2;
  const bool rok[2] = {r_lo < p.G, r_lo + 8 < p.G};
  const long long rowoff[2] = {(long long)n * p.Hq + h * p.G + r_lo, (long long)n * p.Hq + h * p.G + r_lo + 8};
  float lse2[2], delta[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) lse2[r] = rok[r] ? __ldg(p.lse + rowoff[r]) : 0.f;
  auto rowptr = [&](const void* base, long long sn, long long sh) {
    const T* bptr = static_cast<const T*>(base) + (long long)n * sn + (long long)h * p.G * sh;
    return [=](int r) -> const T* { return r < p.G ? bptr + r * sh : nullptr; };
  };
  uint32_t qf[D / 16][4], dof[D / 16][4];
  load_a_frags_global<T, D / 16>(qf, rowptr(p.q, p.q_sn, p.q_sh));
  load_a_frags_global<T, D / 16>(dof, rowptr(p.dout, p.do_sn, p.do_sh));
  {
    auto orow = rowptr(p.o, p.o_sn, p.o_sh);
    row_delta<T, D>(orow(r_lo), orow(r_lo + 8), dof, delta);
  }
  if ((lane & 3) == 0) {
#pragma unroll
    for (int r = 0; r < 2; ++r)
      if (rok[r]) p.ld[rowoff[r]] = make_float2(lse2[r], delta[r]);
  }
  float dq[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) dq[j][0] = dq[j][1] = dq[j][2] = dq[j][3] = 0.f;
  uint32_t phase = 0;
  for (int i = 0; i < ntiles; ++i) {
    const int kpos = tiles[i];
    const int limv = min(kKeyTile, t - kpos + 1);
    const int c0 = (lane & 3) * 2;
    float dp[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) dp[j][0] = dp[j][1] = dp[j][2] = dp[j][3] = 0.f;
    mbar_wait(barV, phase, p.st);
    mma_nk<T, 8, D / 16, kKeyTile>(dp, dof, smem_u32(vbuf), 0, 0);
    __syncwarp();
    if (i + 1 < ntiles && lane == 0) issue_v(tiles[i + 1]);
    const uint32_t kb_addr = smem_u32(kbuf + (i % KBUFS) * TILE_BYTES);
    mbar_wait(barK + (i % KBUFS), (i / KBUFS) & 1, p.st);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float sacc[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f;
      mma_nk<T, 4, D / 16, kKeyTile>(sacc, qf, kb_addr, 32 * half, 0);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          const int col = 32 * half + j * 8 + c0 + (e & 1);
          const float pr = masked_exp2(col < limv, sacc[j][e] * p.scale2 - lse2[r]);
          sacc[j][e] = pr * (dp[half * 4 + j][e] - delta[r]) * p.sm_scale;
        }
      }
      uint32_t dsf[2][4];
      acc_to_a_frags<T, 2>(dsf, sacc);
      mma_kn<T, D / 8, 2, kKeyTile>(dq, dsf, kb_addr, 32 * half, 0);
    }
    __syncwarp();
    if (i + KBUFS < ntiles && lane == 0) issue_k(i + KBUFS);
    phase ^= 1;
  }
  T* dbase = static_cast<T*>(p.dq) + (long long)n * p.dq_sn + (long long)h * p.G * p.dq_sh;
  const float one[2] = {1.f, 1.f};
  store_rows_staged<T, D>(dq, one, reinterpret_cast<T*>(kbuf), [&](int r) -> T* { return r < p.G ? dbase + r * p.dq_sh : nullptr; });
}

// ------------------------------------------------------------------------------------------------
// inverted index: for every (kv head, global block) the list of tokens that selected it
// ------------------------------------------------------------------------------------------------
struct IndexParams {
  const int* topk_idx;
  const int* cu_seqlens;
  const int* cu_blocks;  // [B+1] prefix sum of ceil(len / block_size)
  // A bin is (kv head, token window, global block): bin = (head * NW + window) * TB + block.  Binning the tokens of a
  // block's list by window, with the window as the slower index, makes CTAs that run at the same time gather Q/dO rows
  // of the same few thousand tokens, so the rows are read from DRAM once and then served by L2.
  int* count;            // [bins]
  int* cursor;           // [bins]
  int* offsets;          // [bins + 1] exclusive scan of count
  int* item_base;        // [bins + 1] exclusive scan of ceil(count / chunk)
  int* item_bin;         // [items] the bin of every work item (so that a CTA finds its bin with one load, not a search)
  int* list;             // [capacity] global token ids
  long long t_sh, t_sn, t_sk;
  int N, B, Hkv, T, block_size, TB, chunk;
  int W, NW;             // tokens per window, windows
  long long capacity;
  Status st;
};

template <bool FILL>
__global__ void index_scatter_kernel(IndexParams p) {
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)p.Hkv * p.N;
  if (gid >= total) return;
  const int h = gid / p.N, n = gid % p.N;
  const int b = find_sequence(p.cu_seqlens, p.B, n);
  const int t = n - __ldg(p.cu_seqlens + b);
  const int bq = t / p.block_size;
  const int blk0 = __ldg(p.cu_blocks + b);
  const int* tptr = p.topk_idx + h * p.t_sh + (long long)n * p.t_sn;
  for (int j = 0; j < p.T; ++j) {
    const int idx = __ldg(tptr + j * p.t_sk);
    if (idx < 0 || idx > bq) continue;
    const int x = (h * p.NW + n / p.W) * p.TB + blk0 + idx;
    if (blk0 + idx >= p.TB) { p.st.raise(kErrBadIndex); continue; }
    if (!FILL) {
      atomicAdd(p.count + x, 1);
    } else {
      const int pos = atomicAdd(p.cursor + x, 1);
      const long long dst = (long long)p.offsets[x] + pos;
      if (dst < p.capacity) p.list[dst] = n; else p.st.raise(kErrBadIndex);
    }
  }
}

// single CTA: exclusive scans of count and of the per-bin item count, 1024 bins per round (warp shuffles, then the 32 warp
// totals); also writes the bin of every work item
__global__ void __launch_bounds__(1024) index_scan_kernel(IndexParams p) {
  __shared__ int w_cnt[32], w_itm[32];
  __shared__ int carry_cnt, carry_itm;
  const int total = p.Hkv * p.NW * p.TB;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) { carry_cnt = 0; carry_itm = 0; }
  __syncthreads();
  for (int base = 0; base < total; base += 1024) {
    const int i = base + threadIdx.x;
    const int c = i < total ? p.count[i] : 0;
    const int it = (c + p.chunk - 1) / p.chunk;
    int vc = c, vi = it;  // inclusive scans within the warp
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int tc = __shfl_up_sync(0xffffffffu, vc, off), ti = __shfl_up_sync(0xffffffffu, vi, off);
      if (lane >= off) { vc += tc; vi += ti; }
    }
    if (lane == 31) { w_cnt[warp] = vc; w_itm[warp] = vi; }
    __syncthreads();
    if (warp == 0) {  // exclusive scan of the 32 warp totals
      const int tc0 = w_cnt[lane], ti0 = w_itm[lane];
      int sc = tc0, si = ti0;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int tc = __shfl_up_sync(0xffffffffu, sc, off), ti = __shfl_up_sync(0xffffffffu, si, off);
        if (lane >= off) { sc += tc; si += ti; }
      }
      w_cnt[lane] = sc - tc0;
      w_itm[lane] = si - ti0;
    }
    __syncthreads();
    const int incl_c = carry_cnt + w_cnt[warp] + vc, incl_i = carry_itm + w_itm[warp] + vi;
    if (i < total) {
      p.offsets[i] = incl_c - c;
      const int first = incl_i - it;
      p.item_base[i] = first;
      for (int k2 = 0; k2 < it; ++k2) p.item_bin[first + k2] = i;
    }
    __syncthreads();
    if (threadIdx.x == 1023) { carry_cnt = incl_c; carry_itm = incl_i; }
    __syncthreads();
  }
  if (threadIdx.x == 0) { p.offsets[total] = carry_cnt; p.item_base[total] = carry_itm; }
}

// ------------------------------------------------------------------------------------------------
// dK / dV pass
// ------------------------------------------------------------------------------------------------
constexpr int kSlots = 2;        // tokens per pipeline stage
constexpr int kBwdStages = 4;

template <typename T, int D, bool SPARSE>
__global__ void __launch_bounds__(160, 1)
dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
            const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, DkdvParams p) {
  constexpr int TILE_BYTES = kKeyTile * D * 2;     // K or V tile
  constexpr int SLOT_BYTES = 16 * D * 2;           // Q or dO rows of one token
  constexpr int PANELS = D / 64;
  constexpr int STAGE_BYTES = kSlots * 2 * SLOT_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ktile = smem;
  uint8_t* vtile = smem + TILE_BYTES;
  uint8_t* ring = smem + 2 * TILE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + kBwdStages * STAGE_BYTES);
  uint64_t* empty = full + kBwdStages;
  uint64_t* kvbar = empty + kBwdStages;
  float2* ld_sh = reinterpret_cast<float2*>(kvbar + 1);                 // [stages][slots][16]
  int* tok_sh = reinterpret_cast<int*>(ld_sh + kBwdStages * kSlots * 16);  // [stages][slots] in-sequence position or -1
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- which key tile and which tokens ----
  int h, qs, Lq, krow0, kpos, kvalid;   // krow0: global K row of the tile's first key; kpos: its in-sequence index
  int tok_begin, tok_count;             // dense: first token position and count; sparse: list offset and count
  if (SPARSE) {
    const int item = blockIdx.x;
    const int total_x = p.Hkv * p.NW * p.TB;
    if (item >= __ldg(p.item_base + total_x)) return;
    const int x = __ldg(p.item_bin + item);  // item_base[x] <= item < item_base[x + 1]
    h = x / (p.NW * p.TB);
    const int gb = x % p.TB;
    const int b = find_sequence(p.cu_blocks, p.B, gb);
    qs = __ldg(p.cu_q + b);
    Lq = __ldg(p.cu_q + b + 1) - qs;
    const int blk = gb - __ldg(p.cu_blocks + b);
    kpos = blk * p.block_size + blockIdx.y * kKeyTile;
    krow0 = qs + kpos;
    kvalid = min(kKeyTile, Lq - kpos);
    const int c = item - __ldg(p.item_base + x);
    const int cnt = __ldg(p.offsets + x + 1) - __ldg(p.offsets + x);
    tok_begin = __ldg(p.offsets + x) + c * p.chunk;
    tok_count = min(p.chunk, cnt - c * p.chunk);
  } else {
    const int b = blockIdx.z / p.Hkv;
    h = blockIdx.z % p.Hkv;
    qs = __ldg(p.cu_q + b);
    Lq = __ldg(p.cu_q + b + 1) - qs;
    const int ks0 = __ldg(p.cu_k + b), Lk = __ldg(p.cu_k + b + 1) - ks0;
    kpos = blockIdx.x * kKeyTile;  // key tiles vary fastest: CTAs that run together share a token chunk in L2
    if (kpos >= Lk) return;
    krow0 = ks0 + kpos;
    kvalid = min(kKeyTile, Lk - kpos);
    const int t_first = p.causal ? kpos * p.stride + p.window - 1 : 0;
    const int c_lo = blockIdx.y * p.chunk;
    tok_begin = max(c_lo, t_first);
    tok_count = min(c_lo + p.chunk, Lq) - tok_begin;
  }
  if (kvalid <= 0 || tok_count <= 0) return;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kBwdStages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 4);
    }
    mbar_init(kvbar, 1);
    fence_barrier_init();
  }
  // Rows the TMA boxes never write (heads >= G, the unused slot of an odd tail) are multiplied by
  // exact zeros later; clear the ring once so that they cannot hold NaN bit patterns.
  for (int i = threadIdx.x; i < kBwdStages * STAGE_BYTES / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(ring)[i] = make_uint4(0u, 0u, 0u, 0u);
  fence_proxy_async();
  __syncthreads();
  const int ngroups = (tok_count + kSlots - 1) / kSlots;

  if (warp == 4) {
    // ================= producer warp =================
    if (lane == 0) {
      mbar_expect_tx(kvbar, 2 * TILE_BYTES);
#pragma unroll
      for (int pn = 0; pn < PANELS; ++pn) {
        tma_load_3d(ktile + pn * (kKeyTile * 128), &tmK, kvbar, pn * 64, h, krow0);
        tma_load_3d(vtile + pn * (kKeyTile * 128), &tmV, kvbar, pn * 64, h, krow0);
      }
    }
    for (int g = 0; g < ngroups; ++g) {
      const int s = g % kBwdStages;
      if (g >= kBwdStages) mbar_wait(empty + s, ((g / kBwdStages) - 1) & 1, p.st);
      // lanes 0..15 serve slot 0, lanes 16..31 slot 1: each fetches the (lse, delta) pair of one head
      const int slot = lane >> 4, head = lane & 15;
      const int ti = g * kSlots + slot;
      int n = -1, tpos = -1;
      if (ti < tok_count) {
        if (SPARSE) { n = __ldg(p.list + tok_begin + ti); tpos = n - qs; }
        else { tpos = tok_begin + ti; n = qs + tpos; }
      }
      float2 ldv = make_float2(INFINITY, 0.f);
      if (n >= 0 && head < p.G) ldv = __ldg(p.ld + (long long)n * p.Hq + h * p.G + head);
      ld_sh[(s * kSlots + slot) * 16 + head] = ldv;
      if (head == 0) tok_sh[s * kSlots + slot] = tpos;
      const int n0 = __shfl_sync(0xffffffffu, n, 0), n1 = __shfl_sync(0xffffffffu, n, 16);
      __syncwarp();
      if (lane == 0) {
        const int nvalid = (n0 >= 0) + (n1 >= 0);
        mbar_expect_tx(full + s, nvalid * 2 * p.G * D * 2);
        uint8_t* st = ring + s * STAGE_BYTES;
#pragma unroll
        for (int sl = 0; sl < kSlots; ++sl) {
          const int nn = sl == 0 ? n0 : n1;
          if (nn < 0) continue;
#pragma unroll
          for (int pn = 0; pn < PANELS; ++pn) {
            tma_load_3d(st + sl * 2 * SLOT_BYTES + pn * (16 * 128), &tmQ, full + s, pn * 64, h * p.G, nn);
            tma_load_3d(st + sl * 2 * SLOT_BYTES + SLOT_BYTES + pn * (16 * 128), &tmDO, full + s, pn * 64, h * p.G, nn);
          }
        }
      }
    }
    return;
  }

  // ================= consumer warps: 16 keys each =================
  float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    dk[j][0] = dk[j][1] = dk[j][2] = dk[j][3] = 0.f;
    dv[j][0] = dv[j][1] = dv[j][2] = dv[j][3] = 0.f;
  }
  const int r_lo = lane >> 2, c0 = (lane & 3) * 2;
  // a token at position t sees key (kpos + row) iff t >= need[row]
  int need[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + r_lo + 8 * r;
    const int kidx = kpos + row;
    need[r] = (row < kvalid) ? (p.causal ? kidx * p.stride + p.window - 1 : 0) : 0x7fffffff;
  }
  const uint32_t kt = smem_u32(ktile), vt = smem_u32(vtile);
  const int a_row = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), a_ch = lane >> 4;   // A-fragment addressing
  const int b_row = (lane & 7) + ((lane >> 4) << 3), b_ch = (lane >> 3) & 1;              // B (n,k) addressing
  mbar_wait(kvbar, 0, p.st);

  for (int g = 0; g < ngroups; ++g) {
    const int s = g % kBwdStages;
    mbar_wait(full + s, (g / kBwdStages) & 1, p.st);
    const uint32_t stg = smem_u32(ring + s * STAGE_BYTES);
    float st_[kSlots * 2][4], dp_[kSlots * 2][4];
#pragma unroll
    for (int j = 0; j < kSlots * 2; ++j) {
      st_[j][0] = st_[j][1] = st_[j][2] = st_[j][3] = 0.f;
      dp_[j][0] = dp_[j][1] = dp_[j][2] = dp_[j][3] = 0.f;
    }
    // S^T = K Q^T and dP^T = V dO^T for both slots
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t ka[4], va[4];
      ldmatrix_x4(ka, swz_addr<kKeyTile>(kt, a_row, 2 * kk + a_ch));
      ldmatrix_x4(va, swz_addr<kKeyTile>(vt, a_row, 2 * kk + a_ch));
#pragma unroll
      for (int sl = 0; sl < kSlots; ++sl) {
        uint32_t bq[4], bo[4];
        ldmatrix_x4(bq, swz_addr<16>(stg + sl * 2 * SLOT_BYTES, b_row, 2 * kk + b_ch));
        ldmatrix_x4(bo, swz_addr<16>(stg + sl * 2 * SLOT_BYTES + SLOT_BYTES, b_row, 2 * kk + b_ch));
        DT<T>::mma(st_[2 * sl], ka, bq[0], bq[1]);
        DT<T>::mma(st_[2 * sl + 1], ka, bq[2], bq[3]);
        DT<T>::mma(dp_[2 * sl], va, bo[0], bo[1]);
        DT<T>::mma(dp_[2 * sl + 1], va, bo[2], bo[3]);
      }
    }
    // P^T and dS^T
#pragma unroll
    for (int sl = 0; sl < kSlots; ++sl) {
      const int tpos = tok_sh[s * kSlots + sl];
      const float2* ldp = ld_sh + (s * kSlots + sl) * 16;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          const int head = j * 8 + c0 + (e & 1);
          const float2 ldv = ldp[head];
          const bool vis = tpos >= need[r] && head < p.G;   // tpos = -1 for an empty slot
          const float pr = masked_exp2(vis, st_[2 * sl + j][e] * p.scale2 - ldv.x);
          st_[2 * sl + j][e] = pr;
          dp_[2 * sl + j][e] = vis ? pr * (dp_[2 * sl + j][e] - ldv.y) * p.sm_scale : 0.f;
        }
      }
    }
    // dV += P^T dO ; dK += dS^T Q   (k dimension = the 16 head rows of each slot)
#pragma unroll
    for (int sl = 0; sl < kSlots; ++sl) {
      uint32_t pf[1][4], dsf[1][4];
      const float(&ps)[2][4] = *reinterpret_cast<const float(*)[2][4]>(&st_[2 * sl]);
      const float(&ds)[2][4] = *reinterpret_cast<const float(*)[2][4]>(&dp_[2 * sl]);
      acc_to_a_frags<T, 1>(pf, ps);
      acc_to_a_frags<T, 1>(dsf, ds);
      mma_kn<T, D / 8, 1, 16>(dv, pf, stg + sl * 2 * SLOT_BYTES + SLOT_BYTES, 0, 0);
      mma_kn<T, D / 8, 1, 16>(dk, dsf, stg + sl * 2 * SLOT_BYTES, 0, 0);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty + s);
  }

  // ---- add this CTA's partial dK / dV ----
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + r_lo + 8 * r;
    if (row >= kvalid) continue;
    float* dkr = p.dk32 + ((size_t)(krow0 + row) * p.Hkv + h) * D;
    float* dvr = p.dv32 + ((size_t)(krow0 + row) * p.Hkv + h) * D;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      atomicAdd(reinterpret_cast<float2*>(dkr + j * 8 + c0), make_float2(dk[j][2 * r], dk[j][2 * r + 1]));
      atomicAdd(reinterpret_cast<float2*>(dvr + j * 8 + c0), make_float2(dv[j][2 * r], dv[j][2 * r + 1]));
    }
  }
}

// fp32 accumulator -> storage type, rows of D contiguous elements with arbitrary row strides.  A thread converts
// kConvertUnroll float4 pieces, 256 pieces apart, and issues all of its loads before the first store: one 16-byte load in
// flight per thread left HBM two thirds busy.
constexpr int kConvertUnroll = 4;
template <typename T>
__global__ void __launch_bounds__(256) convert_rows_kernel(const float* __restrict__ src, void* dst, long long rows, int Hkv, int D,
                                                           long long d_sn, long long d_sh) {
  const int CH = D / 4;
  const long long total = rows * Hkv * CH;
  const long long base = (long long)blockIdx.x * (256 * kConvertUnroll) + threadIdx.x;
  float4 v[kConvertUnroll];
#pragma unroll
  for (int u = 0; u < kConvertUnroll; ++u) {
    const long long idx = base + u * 256;
    v[u] = idx < total ? __ldcs(reinterpret_cast<const float4*>(src) + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int u = 0; u < kConvertUnroll; ++u) {
    const long long idx = base + u * 256;
    if (idx >= total) continue;
    const int c = idx % CH;
    const int h = (idx / CH) % Hkv;
    const long long n = idx / ((long long)CH * Hkv);
    uint2 out;
    out.x = DT<T>::pack(v[u].x, v[u].y);
    out.y = DT<T>::pack(v[u].z, v[u].w);
    *reinterpret_cast<uint2*>(static_cast<T*>(dst) + n * d_sn + (long long)h * d_sh + c * 4) = out;
  }
}

// (lse, delta) per (token, query head) for the backward passes: delta = sum_d o * dO in fp32.  16 lanes per row of
// D 16-bit elements (16 bytes each for D = 128); one pass over o and dO.
template <typename T, int D>
__global__ void row_stats_kernel(const T* __restrict__ o, const T* __restrict__ dout, const float* __restrict__ lse,
                                 float2* __restrict__ ld, long long rows, int Hq, long long o_sn, long long o_sh, long long do_sn,
                                 long long do_sh) {
  constexpr int EPL = D / 16;  // elements per lane
  const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
  const int sub = threadIdx.x & 15;
  float acc = 0.f;
  if (row < rows) {
    const long long n = row / Hq;
    const int h = (int)(row % Hq);
    const T* po = o + n * o_sn + (long long)h * o_sh + sub * EPL;
    const T* pd = dout + n * do_sn + (long long)h * do_sh + sub * EPL;
    if constexpr (EPL == 8) {
      const uint4 a = *reinterpret_cast<const uint4*>(po), b = *reinterpret_cast<const uint4*>(pd);
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 x = DT<T>::unpack(aw[j]), y = DT<T>::unpack(bw[j]);
        acc = fmaf(x.x, y.x, acc);
        acc = fmaf(x.y, y.y, acc);
      }
    } else {
#pragma unroll
      for (int j = 0; j < EPL; ++j) acc = fmaf(DT<T>::to_float(po[j]), DT<T>::to_float(pd[j]), acc);
    }
  }
#pragma unroll
  for (int off = 8; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (row < rows && sub == 0) ld[row] = make_float2(__ldg(lse + row), acc);
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

template <typename T, int D, bool SPARSE>
static int launch_dkdv(const void* q, const void* dout, const void* k, const void* v, const long long* strides, int Nq, int Nk,
                       dim3 grid, DkdvParams p, cudaStream_t stream) {
  // strides: q_n q_h k_n k_h v_n v_h do_n do_h
  CUtensorMap tmQ, tmDO, tmK, tmV;
  int rc = make_tmap_3d(&tmQ, DT<T>::kTmapType, q, D, p.Hq, Nq, strides[1], strides[0], 64, p.G, 1);
  if (rc) return rc;
  rc = make_tmap_3d(&tmDO, DT<T>::kTmapType, dout, D, p.Hq, Nq, strides[7], strides[6], 64, p.G, 1);
  if (rc) return rc;
  rc = make_tmap_3d(&tmK, DT<T>::kTmapType, k, D, p.Hkv, Nk, strides[3], strides[2], 64, 1, kKeyTile);
  if (rc) return rc;
  rc = make_tmap_3d(&tmV, DT<T>::kTmapType, v, D, p.Hkv, Nk, strides[5], strides[4], 64, 1, kKeyTile);
  if (rc) return rc;
  constexpr int TILE_BYTES = kKeyTile * D * 2;
  constexpr int STAGE_BYTES = kSlots * 2 * 16 * D * 2;
  const size_t smem = 1024 + 2 * TILE_BYTES + kBwdStages * STAGE_BYTES + (2 * kBwdStages + 1) * sizeof(uint64_t) +
                      kBwdStages * kSlots * (16 * sizeof(float2) + sizeof(int)) + 64;
  auto kern = dkdv_kernel<T, D, SPARSE>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_rc(e);
  { LaunchScope ls_(SPARSE ? "sparse_dkdv" : "dense_dkdv", stream); kern<<<grid, 160, smem, stream>>>(tmQ, tmDO, tmK, tmV, p); }
  return cuda_rc(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------------
// host drivers
// ------------------------------------------------------------------------------------------------
struct DenseBwdWs { float2* ld; float* dk32; float* dv32; };

static size_t dense_ws_bytes(int total_q, int total_k, int Hq, int Hkv, int D) {
  return align_up((size_t)total_q * Hq * sizeof(float2), 256) + 2 * align_up((size_t)total_k * Hkv * D * sizeof(float), 256);
}

template <typename T, int D>
static int run_dense_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                         const int* cu_q, const int* cu_k, void* dq, void* dk, void* dv, void* ws, int total_q, int total_k,
                         int batch, int max_q, int max_k, int Hq, int Hkv, int causal, int window, int stride, int left,
                         const long long* S, float sm_scale, cudaStream_t stream) {
  // S: q_n q_h k_n k_h v_n v_h o_n o_h do_n do_h dq_n dq_h dk_n dk_h dv_n dv_h
  const int G = Hq / Hkv;
  uint8_t* w = static_cast<uint8_t*>(ws);
  float2* ld = reinterpret_cast<float2*>(w);
  w += align_up((size_t)total_q * Hq * sizeof(float2), 256);
  float* dk32 = reinterpret_cast<float*>(w);
  w += align_up((size_t)total_k * Hkv * D * sizeof(float), 256);
  float* dv32 = reinterpret_cast<float*>(w);
  cudaError_t e = cudaMemsetAsync(dk32, 0, 2 * align_up((size_t)total_k * Hkv * D * sizeof(float), 256), stream);
  if (e != cudaSuccess) return cuda_rc(e);

  DenseBwdParams p;
  p.q = q; p.o = o; p.dout = dout; p.lse = lse; p.ld = ld; p.dq = dq; p.cu_q = cu_q; p.cu_k = cu_k;
  p.q_sn = S[0]; p.q_sh = S[1]; p.o_sn = S[6]; p.o_sh = S[7]; p.do_sn = S[8]; p.do_sh = S[9]; p.dq_sn = S[10]; p.dq_sh = S[11];
  p.B = batch; p.Hq = Hq; p.Hkv = Hkv; p.G = G;
  p.logG = 0;
  while ((1 << p.logG) < G) ++p.logG;
  p.window = window; p.stride = stride; p.causal = causal; p.left = left;
  p.scale2 = sm_scale * kLog2e; p.sm_scale = sm_scale;
  p.st.word = status_word();
  if (left >= 0 && D != 128) return kUnsupported;  // the sliding window needs the tcgen05 dK/dV pass (head_dim 128)
  {
    const int dt = DT<T>::kTmapType == CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 ? NSA_DTYPE_BF16 : NSA_DTYPE_FP16;
    const int rc = dense_dq_tc(k, v, S[2], S[3], S[4], S[5], total_q, total_k, max_q, D, dt, p, stream);
    if (rc) return rc;
  }
  DkdvParams d;
  d.ld = ld; d.dk32 = dk32; d.dv32 = dv32; d.cu_q = cu_q; d.cu_k = cu_k;
  d.cu_blocks = nullptr; d.offsets = nullptr; d.item_base = nullptr; d.item_bin = nullptr; d.item_counter = nullptr; d.list = nullptr;
  d.B = batch; d.Hq = Hq; d.Hkv = Hkv; d.G = G; d.TB = 0; d.NW = 1; d.block_size = kKeyTile;
  int chunk = 256;
  while (chunk < 1024 && chunk * 16 < max_q) chunk <<= 1;
  d.chunk = chunk;
  d.window = window; d.stride = stride; d.causal = causal; d.left = left;
  d.scale2 = p.scale2; d.sm_scale = sm_scale; d.st = p.st;
  const long long ds[8] = {S[0], S[1], S[2], S[3], S[4], S[5], S[8], S[9]};
  dim3 grid((max_k + kKeyTile - 1) / kKeyTile, (max_q + chunk - 1) / chunk, batch * Hkv);
  int rc;
  if constexpr (D == 128) {
    rc = launch_dense_dkdv_tc<T>(q, dout, k, v, ds, total_q, total_k, max_q, max_k, batch, d, stream);
  } else {
    rc = launch_dkdv<T, D, false>(q, dout, k, v, ds, total_q, total_k, grid, d, stream);
  }
  if (rc) return rc;
  const long long n4 = (long long)total_k * Hkv * (D / 4);
  { LaunchScope ls_("convert_dk", stream); convert_rows_kernel<T><<<(unsigned)((n4 + 256 * kConvertUnroll - 1) / (256 * kConvertUnroll)), 256, 0, stream>>>(dk32, dk, total_k, Hkv, D, S[12], S[13]); }
  { LaunchScope ls_("convert_dv", stream); convert_rows_kernel<T><<<(unsigned)((n4 + 256 * kConvertUnroll - 1) / (256 * kConvertUnroll)), 256, 0, stream>>>(dv32, dv, total_k, Hkv, D, S[14], S[15]); }
  return cuda_rc(cudaGetLastError());
}

constexpr int kSparseChunk = 512;  // tokens of one block's list handled by one CTA

// Token windows of the inverted index: as many tokens as keep the Q and dO rows of one KV-head group (G heads) within
// about half of the L2 cache, a power of two, at least 1024.  Returns (tokens per window, windows).
static bool sparse_fused_dq(int G, int D) { return D == 128 && G >= 4 && (G & (G - 1)) == 0; }

static std::pair<int, int> sparse_windows(int N, int G, int D) {
  // Q and dO rows (16-bit) and, where the tcgen05 pass also produces dQ, the fp32 dQ accumulator rows it reduces into
  const long long bytes_per_token = 2ll * G * D * 2 + (sparse_fused_dq(G, D) ? 4ll * G * D : 0);
  int W = 1024;
  while (2ll * W * bytes_per_token <= (64ll << 20)) W <<= 1;
  return {W, (N + W - 1) / W};
}

static size_t sparse_ws_bytes(int N, int batch, int Hq, int Hkv, int D, int topk, int block_size) {
  const size_t TB = (size_t)N / block_size + batch;
  const size_t x = (size_t)Hkv * sparse_windows(N, Hq / Hkv, D).second * TB + 1;
  return align_up((size_t)N * Hq * sizeof(float2), 256) + 2 * align_up((size_t)N * Hkv * D * sizeof(float), 256) +
         4 * align_up(x * sizeof(int), 256) + align_up((size_t)Hkv * N * topk * sizeof(int), 256) +
         align_up(((size_t)Hkv * N * topk / kSparseChunk + x) * sizeof(int), 256) +
         (sparse_fused_dq(Hq / Hkv, D) ? align_up((size_t)N * Hq * D * sizeof(float), 256) : 0);
}

template <typename T, int D>
static int run_sparse_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                          const int* topk_idx, const int* cu, const int* cu_blocks, void* dq, void* dk, void* dv, void* ws,
                          int N, int batch, int Hq, int Hkv, int topk, int block_size, const long long* S, float sm_scale,
                          cudaStream_t stream) {
  // S: q_n q_h k_n k_h v_n v_h o_n o_h do_n do_h dq_n dq_h dk_n dk_h dv_n dv_h idx_h idx_n idx_k
  const int G = Hq / Hkv;
  const int TB = N / block_size + batch;
  const auto [W, NW] = sparse_windows(N, G, D);
  const size_t X = (size_t)Hkv * NW * TB + 1;
  uint8_t* w = static_cast<uint8_t*>(ws);
  float2* ld = reinterpret_cast<float2*>(w);
  w += align_up((size_t)N * Hq * sizeof(float2), 256);
  float* dk32 = reinterpret_cast<float*>(w);
  w += align_up((size_t)N * Hkv * D * sizeof(float), 256);
  float* dv32 = reinterpret_cast<float*>(w);
  w += align_up((size_t)N * Hkv * D * sizeof(float), 256);
  int* count = reinterpret_cast<int*>(w);
  w += align_up(X * sizeof(int), 256);
  int* cursor = reinterpret_cast<int*>(w);
  w += align_up(X * sizeof(int), 256);
  int* offsets = reinterpret_cast<int*>(w);
  w += align_up(X * sizeof(int), 256);
  int* item_base = reinterpret_cast<int*>(w);
  w += align_up(X * sizeof(int), 256);
  int* list = reinterpret_cast<int*>(w);
  w += align_up((size_t)Hkv * N * topk * sizeof(int), 256);
  int* item_bin = reinterpret_cast<int*>(w);   // one entry per possible work item (the grid's upper bound below)
  w += align_up(((size_t)Hkv * N * topk / kSparseChunk + X) * sizeof(int), 256);
  const bool fused = sparse_fused_dq(G, D);  // dQ comes out of the tcgen05 dK/dV pass; otherwise the per-token dQ kernel runs
  float* dq32 = fused ? reinterpret_cast<float*>(w) : nullptr;
  // dk32, dv32, count, cursor are contiguous: one memset
  cudaError_t e = cudaMemsetAsync(dk32, 0, reinterpret_cast<uint8_t*>(offsets) - reinterpret_cast<uint8_t*>(dk32), stream);
  if (e != cudaSuccess) return cuda_rc(e);
  if (fused) {
    e = cudaMemsetAsync(dq32, 0, (size_t)N * Hq * D * sizeof(float), stream);
    if (e != cudaSuccess) return cuda_rc(e);
  }

  SparseBwdParams p;
  p.q = q; p.o = o; p.dout = dout; p.lse = lse; p.ld = ld; p.dq = dq; p.topk_idx = topk_idx; p.cu_seqlens = cu;
  p.q_sn = S[0]; p.q_sh = S[1]; p.o_sn = S[6]; p.o_sh = S[7]; p.do_sn = S[8]; p.do_sh = S[9]; p.dq_sn = S[10]; p.dq_sh = S[11];
  p.t_sh = S[16]; p.t_sn = S[17]; p.t_sk = S[18];
  p.N = N; p.B = batch; p.Hq = Hq; p.Hkv = Hkv; p.G = G; p.T = topk; p.block_size = block_size;
  p.scale2 = sm_scale * kLog2e; p.sm_scale = sm_scale;
  p.st.word = status_word();

  IndexParams ip;
  ip.topk_idx = topk_idx; ip.cu_seqlens = cu; ip.cu_blocks = cu_blocks; ip.count = count; ip.cursor = cursor;
  ip.offsets = offsets; ip.item_base = item_base; ip.item_bin = item_bin; ip.list = list;
  ip.t_sh = S[16]; ip.t_sn = S[17]; ip.t_sk = S[18];
  ip.N = N; ip.B = batch; ip.Hkv = Hkv; ip.T = topk; ip.block_size = block_size; ip.TB = TB; ip.chunk = kSparseChunk; ip.W = W; ip.NW = NW;
  ip.capacity = (long long)Hkv * N * topk;
  ip.st = p.st;
  const long long hn = (long long)Hkv * N;
  { LaunchScope ls_("index_count", stream); index_scatter_kernel<false><<<(unsigned)((hn + 255) / 256), 256, 0, stream>>>(ip); }
  { LaunchScope ls_("index_scan", stream); index_scan_kernel<<<1, 1024, 0, stream>>>(ip); }
  { LaunchScope ls_("index_fill", stream); index_scatter_kernel<true><<<(unsigned)((hn + 255) / 256), 256, 0, stream>>>(ip); }
  if ((e = cudaGetLastError()) != cudaSuccess) return cuda_rc(e);
  if (fused) {
    const long long rows = (long long)N * Hq;
    LaunchScope ls_("row_stats", stream);
    row_stats_kernel<T, D><<<(unsigned)((rows * 16 + 255) / 256), 256, 0, stream>>>(
        static_cast<const T*>(o), static_cast<const T*>(dout), lse, ld, rows, Hq, S[6], S[7], S[8], S[9]);
    if ((e = cudaGetLastError()) != cudaSuccess) return cuda_rc(e);
  } else
  {
    // one K buffer and as many warps as shared memory holds: measured 11.7 ms with 6 warps, 10.2 ms with 7, 12.0 ms with
    // 4 warps and two K buffers (64 K tokens) -- the kernel is bound by latency, and warps are what hides it
    constexpr int KBUFS = 1;
    constexpr int WARPS = (D == 128) ? 7 : 8;
    constexpr int TILE_BYTES = kKeyTile * D * 2;
    CUtensorMap tmK, tmV;
    int rc = make_tmap_3d(&tmK, DT<T>::kTmapType, k, D, Hkv, N, S[3], S[2], 64, 1, kKeyTile);
    if (rc) return rc;
    rc = make_tmap_3d(&tmV, DT<T>::kTmapType, v, D, Hkv, N, S[5], S[4], 64, 1, kKeyTile);
    if (rc) return rc;
    const size_t smem = 1024 + WARPS * (KBUFS + 1) * TILE_BYTES + (KBUFS + 1) * WARPS * sizeof(uint64_t) + WARPS * kMaxTilesBwd * sizeof(int);
    auto kern = sparse_dq_kernel<T, D, WARPS, KBUFS>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_rc(e);
    dim3 grid((N + WARPS - 1) / WARPS, Hkv);
    { LaunchScope ls_("sparse_dq", stream); kern<<<grid, WARPS * 32, smem, stream>>>(tmK, tmV, p); }
    if ((e = cudaGetLastError()) != cudaSuccess) return cuda_rc(e);
  }
  DkdvParams d;
  d.ld = ld; d.dk32 = dk32; d.dv32 = dv32; d.dq32 = dq32; d.cu_q = cu; d.cu_k = cu;
  d.cu_blocks = cu_blocks; d.offsets = offsets; d.item_base = item_base; d.item_bin = item_bin; d.list = list;
  d.item_counter = cursor + (X - 1);   // the spare last word of the zeroed cursor array
  d.B = batch; d.Hq = Hq; d.Hkv = Hkv; d.G = G; d.TB = TB; d.NW = NW; d.chunk = kSparseChunk; d.block_size = block_size;
  d.window = 1; d.stride = 1; d.causal = 1; d.left = -1;
  d.scale2 = p.scale2; d.sm_scale = sm_scale; d.st = p.st;
  const long long ds[8] = {S[0], S[1], S[2], S[3], S[4], S[5], S[8], S[9]};
  // upper bound on work items: every selection in a full chunk, plus one partial chunk per (head, block)
  const long long max_items = ((long long)Hkv * N * topk) / kSparseChunk + (long long)Hkv * NW * TB;
  dim3 grid((unsigned)max_items, block_size / kKeyTile, 1);
  int rc;
  if constexpr (D == 128) {
    rc = (G >= 4 && (G & (G - 1)) == 0) ? launch_sparse_dkdv_tc<T>(q, dout, k, v, ds, N, grid, d, stream)
                                                         : launch_dkdv<T, D, true>(q, dout, k, v, ds, N, N, grid, d, stream);
  } else {
    rc = launch_dkdv<T, D, true>(q, dout, k, v, ds, N, N, grid, d, stream);
  }
  if (rc) return rc;
  if (fused) {
    const long long q4 = (long long)N * Hq * (D / 4);
    LaunchScope ls_("convert_dq", stream);
    convert_rows_kernel<T><<<(unsigned)((q4 + 256 * kConvertUnroll - 1) / (256 * kConvertUnroll)), 256, 0, stream>>>(dq32, dq, N, Hq, D, S[10], S[11]);
  }
  const long long n4 = (long long)N * Hkv * (D / 4);
  { LaunchScope ls_("convert_dk", stream); convert_rows_kernel<T><<<(unsigned)((n4 + 256 * kConvertUnroll - 1) / (256 * kConvertUnroll)), 256, 0, stream>>>(dk32, dk, N, Hkv, D, S[12], S[13]); }
  { LaunchScope ls_("convert_dv", stream); convert_rows_kernel<T><<<(unsigned)((n4 + 256 * kConvertUnroll - 1) / (256 * kConvertUnroll)), 256, 0, stream>>>(dv32, dv, N, Hkv, D, S[14], S[15]); }
  return cuda_rc(cudaGetLastError());
}

}  // namespace nsa

extern "C" long long nsa_varlen_attn_bwd_workspace(int total_q, int total_k, int num_q_heads, int num_kv_heads, int head_dim) {
  return (long long)nsa::dense_ws_bytes(total_q, total_k, num_q_heads, num_kv_heads, head_dim);
}

static int varlen_attn_bwd_common(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                  const float* lse, const int* cu_seqlens_q, const int* cu_seqlens_k, void* dq, void* dk,
                                  void* dv, void* workspace, long long workspace_bytes, int total_q, int total_k, int batch,
                                  int max_seqlen_q, int max_seqlen_k, int num_q_heads, int num_kv_heads, int head_dim,
                                  int causal, int window, int stride, int left, const long long* strides, float sm_scale,
                                  int dtype, void* stream) {
  using namespace nsa;
  if (!q || !k || !v || !o || !dout || !lse || !cu_seqlens_q || !cu_seqlens_k || !dq || !dk || !dv || !workspace || !strides)
    return kInvalid;
  if (total_q <= 0 || total_k <= 0 || batch <= 0 || max_seqlen_q <= 0 || max_seqlen_k <= 0) return kInvalid;
  if (num_kv_heads <= 0 || num_q_heads % num_kv_heads) return kInvalid;
  const int G = num_q_heads / num_kv_heads;
  if (G > 16 || (G & (G - 1))) return kUnsupported;
  if (left >= 0 && (!causal || window != 1 || stride != 1)) return kUnsupported;
  for (int i = 0; i < 16; ++i)
    if (strides[i] % 8) return kInvalid;
  if (workspace_bytes < (long long)dense_ws_bytes(total_q, total_k, num_q_heads, num_kv_heads, head_dim)) return kWorkspace;
  return NSA_DISPATCH_T_D(dtype, head_dim, run_dense_bwd, q, k, v, o, dout, lse, cu_seqlens_q, cu_seqlens_k, dq, dk, dv,
                          workspace, total_q, total_k, batch, max_seqlen_q, max_seqlen_k, num_q_heads, num_kv_heads, causal,
                          window, stride, left, strides, sm_scale, static_cast<cudaStream_t>(stream));
}

extern "C" int nsa_varlen_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                   const float* lse, const int* cu_seqlens_q, const int* cu_seqlens_k, void* dq, void* dk,
                                   void* dv, void* workspace, long long workspace_bytes, int total_q, int total_k, int batch,
                                   int max_seqlen_q, int max_seqlen_k, int num_q_heads, int num_kv_heads, int head_dim,
                                   int causal, int window, int stride, const long long* strides, float sm_scale, int dtype,
                                   void* stream) {
  return varlen_attn_bwd_common(q, k, v, o, dout, lse, cu_seqlens_q, cu_seqlens_k, dq, dk, dv, workspace, workspace_bytes,
                                total_q, total_k, batch, max_seqlen_q, max_seqlen_k, num_q_heads, num_kv_heads, head_dim,
                                causal, window, stride, -1, strides, sm_scale, dtype, stream);
}

extern "C" int nsa_window_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                   const float* lse, const int* cu_seqlens, void* dq, void* dk, void* dv, void* workspace,
                                   long long workspace_bytes, int total_len, int batch, int max_seqlen, int num_q_heads,
                                   int num_kv_heads, int head_dim, int window_left, const long long* strides, float sm_scale,
                                   int dtype, void* stream) {
  if (window_left < 0) return nsa::kInvalid;
  return varlen_attn_bwd_common(q, k, v, o, dout, lse, cu_seqlens, cu_seqlens, dq, dk, dv, workspace, workspace_bytes, total_len,
                                total_len, batch, max_seqlen, max_seqlen, num_q_heads, num_kv_heads, head_dim, 1, 1, 1,
                                window_left, strides, sm_scale, dtype, stream);
}

extern "C" long long nsa_topk_sparse_attn_bwd_workspace(int total_len, int batch, int num_q_heads, int num_kv_heads,
                                                        int head_dim, int topk, int block_size) {
  return (long long)nsa::sparse_ws_bytes(total_len, batch, num_q_heads, num_kv_heads, head_dim, topk, block_size);
}

extern "C" int nsa_topk_sparse_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                        const float* lse, const int* topk_idx, const int* cu_seqlens,
                                        const int* cu_seqblocks, void* dq, void* dk, void* dv, void* workspace,
                                        long long workspace_bytes, int total_len, int batch, int num_q_heads,
                                        int num_kv_heads, int head_dim, int topk, int block_size, const long long* strides,
                                        float sm_scale, int dtype, void* stream) {
  using namespace nsa;
  if (!q || !k || !v || !o || !dout || !lse || !topk_idx || !cu_seqlens || !cu_seqblocks || !dq || !dk || !dv || !workspace ||
      !strides)
    return kInvalid;
  if (total_len <= 0 || batch <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads) return kInvalid;
  const int G = num_q_heads / num_kv_heads;
  if (G > 16) return kUnsupported;
  if (block_size < kKeyTile || block_size % kKeyTile) return kUnsupported;
  if (topk <= 0 || (long long)topk * (block_size / kKeyTile) > kMaxTilesBwd) return kUnsupported;
  for (int i = 0; i < 16; ++i)
    if (strides[i] % 8) return kInvalid;
  if (workspace_bytes < (long long)sparse_ws_bytes(total_len, batch, num_q_heads, num_kv_heads, head_dim, topk, block_size))
    return kWorkspace;
  return NSA_DISPATCH_T_D(dtype, head_dim, run_sparse_bwd, q, k, v, o, dout, lse, topk_idx, cu_seqlens, cu_seqblocks, dq, dk, dv,
                          workspace, total_len, batch, num_q_heads, num_kv_heads, topk, block_size, strides, sm_scale,
                          static_cast<cudaStream_t>(stream));
}
