// Block-importance scores and top-k block selection on the 5th-generation tensor cores, two row tiles per CTA.
//
// Same arithmetic as score_topk_tc.cu (logits produced TRANSPOSED, S^T = K Q^T, a thread owns one key and sums the G
// heads of a token inside its own columns; key scores -> shared memory -> block scores -> warp top-k), but a CTA
// works on TWO row tiles A and B of 128 rows = (128/G consecutive tokens) x (G heads) each, B right after A:
//   warps 0..3 : tile A, one thread per key of the current 128-key tile, all 128 (token, head) columns of the tile
//   warps 4..7 : tile B
//   warp 8     : TMA producer (both Q tiles once, K tiles through a ring shared by the two row tiles)
//   warp 9     : TMEM allocation and MMA issue, alternating between the row tiles
// While one group exponentiates, the tensor pipe produces the other group's logits, and the two groups' barriers and
// fold steps interleave instead of stalling all eight warps at once; each K tile is fetched once for 256 rows.
// TMEM columns: tile g, buffer b at g*256 + b*128 (S^T is double-buffered per row tile).
#include "attn_tile.cuh"
#include "dispatch.h"
#include "host_util.h"
#include "score_topk.h"
#include "tc5.cuh"
#include "topk_select.cuh"

namespace nsa {

#ifndef NSA_SCORE_POLY_EVERY
#define NSA_SCORE_POLY_EVERY 2
#endif
constexpr int kScorePolyEvery = NSA_SCORE_POLY_EVERY;  // one pair of exponentials in kScorePolyEvery is evaluated as a polynomial

namespace {
constexpr int kPpKeyTile = 128;
constexpr int kPpStages = 2;

__device__ __forceinline__ void bar_sync_group(int g) { asm volatile("bar.sync %0, 128;\n" ::"r"(1 + g) : "memory"); }
}  // namespace

template <typename T, int D, int LOGG>
__global__ void __launch_bounds__(320, 1)
score_topk_pp_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, ScoreParams p) {
  constexpr int PANELS = D / 64;
  constexpr int PANEL_BYTES = 128 * 128;
  constexpr int Q_BYTES = 128 * D * 2;
  constexpr int K_BYTES = kPpKeyTile * D * 2;
  constexpr int GG = 1 << LOGG;
  constexpr int TPT = 128 >> LOGG;  // tokens per row tile
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* q_sm = smem;                              // [2] row tiles
  uint8_t* k_sm = q_sm + 2 * Q_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(k_sm + kPpStages * K_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = k_full + kPpStages;
  uint64_t* s_full = k_empty + kPpStages;            // [2 tiles][2 buffers]
  uint64_t* s_empty = s_full + 4;                    // [2 tiles][2 buffers]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_empty + 4);
  float* lse_sh = reinterpret_cast<float*>(tmem_slot + 2);       // [2][128] per column (token, head)
  float* keysc = lse_sh + 2 * 128;                                // [2 tiles][2 buffers][TPT][128]
  float* bsc = keysc + 2 * 2 * TPT * kPpKeyTile;                  // [2 tiles][TPT][nb_pad]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (smem_u32(smem) & 1023u) {  // the swizzled operand tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) p.st.raise(kErrSmemLayout);
    return;
  }
  const int b = blockIdx.y, h = blockIdx.z;
  const int qs = __ldg(p.cu_q + b), Lq = __ldg(p.cu_q + b + 1) - qs;
  const int ksq = __ldg(p.cu_k + b), Lk = __ldg(p.cu_k + b + 1) - ksq;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int q0 = qt * 2 * TPT;
  if (q0 >= Lq) return;
  auto visible = [&](int t) { return t < p.window - 1 ? 0 : min(Lk, (t - p.window + 1) / p.stride + 1); };
  const int t_hi = min(q0 + 2 * TPT, Lq) - 1;
  const int ntiles = (visible(t_hi) + kPpKeyTile - 1) / kPpKeyTile;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kPpStages; ++s) {
      mbar_init(k_full + s, 1);
      mbar_init(k_empty + s, 1);
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(s_full + s, 1);
      mbar_init(s_empty + s, 4);
    }
    fence_barrier_init();
  }
  // per-column log-sum-exp of both tiles, zeroed block scores
  if (threadIdx.x < 256) {
    const int col = threadIdx.x;  // tile = col / 128
    const int t = q0 + (col >> LOGG);
    lse_sh[col] = t < Lq ? __ldg(p.lse + (long long)(qs + t) * p.Hq + h * p.G + (col & (GG - 1))) : INFINITY;
  }
  for (int i = threadIdx.x; i < 2 * TPT * p.nb_pad; i += blockDim.x) bsc[i] = 0.f;
  if (warp == 9) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 8) {
    // ===================== TMA producer =====================
    if (lane == 0 && ntiles > 0) {
      mbar_expect_tx(q_full, 2 * Q_BYTES);
#pragma unroll
      for (int g = 0; g < 2; ++g)
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn)
          tma_load_3d(q_sm + g * Q_BYTES + pn * PANEL_BYTES, &tmQ, q_full, pn * 64, h * p.G, qs + q0 + g * TPT);
      for (int i = 0; i < ntiles; ++i) {
        const int s = i % kPpStages;
        if (i >= kPpStages) mbar_wait(k_empty + s, ((i / kPpStages) - 1) & 1, p.st);
        mbar_expect_tx(k_full + s, K_BYTES);
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn)
          tma_load_3d(k_sm + s * K_BYTES + pn * PANEL_BYTES, &tmK, k_full + s, pn * 64, h, ksq + i * kPpKeyTile);
      }
    }
  } else if (warp == 9) {
    // ===================== MMA issuer: converged warp, one elected lane issues (see tc5.cuh) =====================
    if (ntiles > 0) {
      const uint32_t idesc = umma_idesc<T>(128, 128, false, false);
      const uint32_t q_addr = smem_u32(q_sm);
      mbar_wait(q_full, 0, p.st);
      for (int i = 0; i < ntiles; ++i) {
        const int s = i % kPpStages;
        mbar_wait(k_full + s, (i / kPpStages) & 1, p.st);
        const uint32_t k_addr = smem_u32(k_sm + s * K_BYTES);
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          const int sb = g * 2 + (i & 1);
          if (i >= 2) mbar_wait(s_empty + sb, ((i >> 1) - 1) & 1, p.st);
          tc_fence_after_sync();
          if (elect_one()) {
            umma_block_ss<D / 16, PANEL_BYTES>(tmem + (uint32_t)(g * 256 + (i & 1) * 128), k_addr, q_addr + g * Q_BYTES, idesc);
            if (g == 1) umma_commit(k_empty + s);
            umma_commit(s_full + sb);
          }
          __syncwarp();
        }
      }
    }
  } else {
    // ===================== key-score threads: group g (tile A: warps 0..3, tile B: warps 4..7), one thread per key ==========
    const int g = warp >> 2;
    const int key_l = threadIdx.x & 127;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(g * 256);
    const int a = p.window / p.stride, c = p.block_size / p.stride;
    const int tq0 = q0 + g * TPT;  // first token of the group's row tile
    float* ks_g = keysc + g * 2 * TPT * kPpKeyTile;
    float* bsc_g = bsc + (size_t)g * TPT * p.nb_pad;
    const float4* lse4 = reinterpret_cast<const float4*>(lse_sh + g * 128);
    // this thread's (token, relative block) pairs of the fold step; the same for every tile
    const int nblk = kPpKeyTile / c + (a - 1 + c - 1) / c;  // blocks touched by one key tile
    int ftok[3], fbrel[3], fk0[3];
#pragma unroll
    for (int r = 0; r < 3; ++r) {
      const int idx = key_l + 128 * r;
      ftok[r] = idx < TPT * nblk ? idx / nblk : -1;
      fbrel[r] = idx - (idx / nblk) * nblk;
      fk0[r] = fbrel[r] * c - (a - 1);
    }
    for (int i = 0; i < ntiles; ++i) {
      const int bsel = i & 1;
      const int key = i * kPpKeyTile + key_l;  // compressed-key index inside the sequence
      // tokens are consecutive, so the tokens that see this key are a suffix of the tile's tokens:
      // token tq0 + j sees key  iff  tq0 + j >= key*stride + window - 1  (and key < Lk)
      const int tok_min = key < Lk ? min(TPT, max(0, key * p.stride + p.window - 1 - tq0)) : TPT;
      float* ks_t = ks_g + bsel * TPT * kPpKeyTile;
      mbar_wait(s_full + g * 2 + bsel, (i >> 1) & 1, p.st);
      tc_fence_after_sync();
#pragma unroll
      for (int hc = 0; hc < 2; ++hc) {  // 64 columns at a time
        uint32_t su[2][32];
        tmem_ld32(lane_base + bsel * 128 + hc * 64, su[0]);
        tmem_ld32(lane_base + bsel * 128 + hc * 64 + 32, su[1]);
        tmem_ld_wait();
        if (hc == 1) {  // the logits of this buffer are in registers: the next product may overwrite it
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(s_empty + g * 2 + bsel);
        }
        // sums over the G heads of each token; a token's sum is kept or dropped as a whole (visible tokens are a suffix)
#pragma unroll
        for (int tk = 0; tk < 64 / GG; ++tk) {
          float e[GG];
#pragma unroll
          for (int q4 = 0; q4 < GG / 4; ++q4) {
            const int col = tk * GG + q4 * 4;  // within the 64
            const float4 l4 = lse4[(hc * 64 + col) >> 2];
            const float2 sc2 = make_float2(p.scale2, p.scale2);
            const float2 x01 = ffma2(make_float2(__uint_as_float(su[col >> 5][(col + 0) & 31]), __uint_as_float(su[col >> 5][(col + 1) & 31])),
                                     sc2, make_float2(-l4.x, -l4.y));
            const float2 x23 = ffma2(make_float2(__uint_as_float(su[col >> 5][(col + 2) & 31]), __uint_as_float(su[col >> 5][(col + 3) & 31])),
                                     sc2, make_float2(-l4.z, -l4.w));
            // a share of the exponentials runs as a polynomial on the FMA pipe (the other unit bounds this pass)
            const int pair0 = (tk * (GG / 4) + q4) * 2;
            const float2 e01 = (pair0 % kScorePolyEvery == kScorePolyEvery - 1) ? exp2_poly2(x01) : make_float2(fast_exp2(x01.x), fast_exp2(x01.y));
            const float2 e23 = ((pair0 + 1) % kScorePolyEvery == kScorePolyEvery - 1) ? exp2_poly2(x23) : make_float2(fast_exp2(x23.x), fast_exp2(x23.y));
            e[q4 * 4 + 0] = e01.x;
            e[q4 * 4 + 1] = e01.y;
            e[q4 * 4 + 2] = e23.x;
            e[q4 * 4 + 3] = e23.y;
          }
#pragma unroll
          for (int w = GG / 2; w >= 1; w >>= 1)
#pragma unroll
            for (int gg = 0; gg < w; ++gg) e[gg] += e[gg + w];
          const int tok = hc * (64 / GG) + tk;
          ks_t[tok * kPpKeyTile + key_l] = tok >= tok_min ? e[0] : 0.f;
        }
      }
      bar_sync_group(g);  // key scores of this tile are complete
      // fold: block b_lo + brel reads tile-local keys fk0 .. fk0 + a + c - 2 (the layout repeats every tile: c divides 128)
      const int b_lo = i * (kPpKeyTile / c);
#pragma unroll
      for (int r = 0; r < 3; ++r) {
        const int bb = b_lo + fbrel[r];
        if (ftok[r] < 0 || bb >= p.nb_pad) continue;
        const float* src = ks_t + ftok[r] * kPpKeyTile + fk0[r];
        float part[8];
#pragma unroll
        for (int o = 0; o < 8; ++o) {   // a + c - 1 <= 8 offsets (checked on the host); loads are independent
          const bool ok = o <= a + c - 2 && fk0[r] + o >= 0 && fk0[r] + o < kPpKeyTile;
          part[o] = ok ? (float)fold_weight(o, a, c) * src[o] : 0.f;
        }
        const float accb = ((part[0] + part[1]) + (part[2] + part[3])) + ((part[4] + part[5]) + (part[6] + part[7]));
        bsc_g[(size_t)ftok[r] * p.nb_pad + bb] += accb;
      }
    }
    bar_sync_group(g);  // every block score of the group is final before its warps start selecting
    // ---- selection: the tokens of the row tile are dealt to the group's four warps ----
    for (int tok = warp & 3; tok < TPT; tok += 4) {
      const int t = tq0 + tok;
      if (t >= Lq) break;
      warp_select_topk(bsc_g + (size_t)tok * p.nb_pad, t / p.block_size, p.topk_out, p.init_blocks, p.local_blocks,
                       p.topk_idx + h * p.t_sh + (long long)(qs + t) * p.t_sn, p.t_sk);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, 512);
}

template <typename T, int D>
static int launch_score_topk_pp_tc(const void* q, const void* k, long long k_sn, long long k_sh, int Nq, int Nk, int max_seqlen_q,
                                   ScoreParams p, cudaStream_t stream) {
  const int TPT = 128 / p.G;
  const size_t smem = 2 * 128 * D * 2 + kPpStages * kPpKeyTile * D * 2 + 16 * sizeof(uint64_t) + 16 + 256 * sizeof(float) +
                      (size_t)2 * TPT * (2 * kPpKeyTile + p.nb_pad) * sizeof(float);
  if (smem > 226 * 1024) return kUnsupported;
  CUtensorMap tmQ, tmK;
  int rc = make_tmap_3d(&tmQ, DT<T>::kTmapType, q, D, p.Hq, Nq, p.q_sh, p.q_sn, 64, p.G, TPT);
  if (rc) return rc;
  rc = make_tmap_3d(&tmK, DT<T>::kTmapType, k, D, p.Hkv, Nk, k_sh, k_sn, 64, 1, kPpKeyTile);
  if (rc) return rc;
  auto kern = p.logG == 4 ? score_topk_pp_tc_kernel<T, D, 4> : (p.logG == 3 ? score_topk_pp_tc_kernel<T, D, 3> : score_topk_pp_tc_kernel<T, D, 2>);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_rc(e);
  dim3 grid((max_seqlen_q + 2 * TPT - 1) / (2 * TPT), p.B, p.Hkv);
  { LaunchScope ls_("score_topk_tc", stream); kern<<<grid, 320, smem, stream>>>(tmQ, tmK, p); }
  return cuda_rc(cudaGetLastError());
}

// Returns kUnsupported when the block scores of two row tiles do not fit in shared memory (very long sequences) or the
// fold geometry needs more than 3 (token, block) pairs per thread; the caller then uses the one-tile kernel.
int score_topk_pp_tc(const void* q, const void* k, long long k_sn, long long k_sh, int Nq, int Nk, int max_seqlen_q, int head_dim,
                     int dtype, ScoreParams p, cudaStream_t stream) {
  if (p.G < 4 || p.G > 16) return kUnsupported;
  const int a = p.window / p.stride, c = p.block_size / p.stride;
  if (c <= 0 || kPpKeyTile % c || a + c - 1 > 8 || (128 / p.G) * (kPpKeyTile / c + (a - 1 + c - 1) / c) > 3 * 128) return kUnsupported;
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_score_topk_pp_tc, q, k, k_sn, k_sh, Nq, Nk, max_seqlen_q, p, stream);
}

}  // namespace nsa
