// Block-importance scores and top-k block selection on the 5th-generation tensor cores.
//
// Per CTA: 128 query rows = (128/G tokens) x (G heads of one KV head).  The logits are produced TRANSPOSED,
//     S^T = K Q^T   [128 keys x 128 rows]   A = K tile (K-major), B = Q tile (K-major), accumulator in TMEM,
// so that a thread owns one KEY (one TMEM lane) and the columns it reads are (token, head) pairs: the sum over
// the G heads of a group -- which the selection score needs -- is a sum over G adjacent columns inside one
// thread, with every head normalised by its own final log-sum-exp (read from shared memory).
//   key_score[token][key] -> shared memory -> folded into block_score[token][block] (weights = overlap counts of
//   compression windows and selection blocks) -> warp-level top-k with forced initial / local blocks.
//   warps 0..7: two threads per key (64 columns each);  warp 8: TMA producer (Q once, K tiles in a 3-stage ring);
//   warp 9: TMEM allocation and MMA issue.  S^T is double-buffered in TMEM ([0,128) and [128,256)).
#include "attn_tile.cuh"
#include "dispatch.h"
#include "host_util.h"
#include "score_topk.h"
#include "tc5.cuh"
#include "topk_select.cuh"

namespace nsa {

constexpr int kScKeyTile = 128;
constexpr int kScStages = 3;

__device__ __forceinline__ void bar_sync_softmax() { asm volatile("bar.sync 1, 256;\n" ::: "memory"); }

template <typename T, int D, int LOGG>
__global__ void __launch_bounds__(320, 1)
score_topk_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, ScoreParams p) {
  constexpr int PANELS = D / 64;
  constexpr int PANEL_BYTES = 128 * 128;
  constexpr int Q_BYTES = 128 * D * 2;
  constexpr int K_BYTES = kScKeyTile * D * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_sm = smem;
  uint8_t* k_sm = q_sm + Q_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(k_sm + kScStages * K_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = k_full + kScStages;
  uint64_t* s_full = k_empty + kScStages;
  uint64_t* s_empty = s_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_empty + 2);
  float* lse_sh = reinterpret_cast<float*>(tmem_slot + 2);      // [128] per column (token, head)
  int* nvis_sh = reinterpret_cast<int*>(lse_sh + 128);           // [TPT] visible keys per token
  const int TPT = 128 >> p.logG;                                 // tokens per CTA
  float* keysc = reinterpret_cast<float*>(nvis_sh + 32);         // [TPT][128]
  float* bsc = keysc + 2 * TPT * kScKeyTile;                     // [TPT][nb_pad]   (key scores are double-buffered)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.y, h = blockIdx.z;
  const int qs = __ldg(p.cu_q + b), Lq = __ldg(p.cu_q + b + 1) - qs;
  const int ksq = __ldg(p.cu_k + b), Lk = __ldg(p.cu_k + b + 1) - ksq;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int q0 = qt * TPT;
  if (q0 >= Lq) return;
  auto visible = [&](int t) { return t < p.window - 1 ? 0 : min(Lk, (t - p.window + 1) / p.stride + 1); };
  const int t_hi = min(q0 + TPT, Lq) - 1;
  const int ntiles = (visible(t_hi) + kScKeyTile - 1) / kScKeyTile;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kScStages; ++s) {
      mbar_init(k_full + s, 1);
      mbar_init(k_empty + s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(s_full + s, 1);
      mbar_init(s_empty + s, 8);
    }
    fence_barrier_init();
  }
  // per-column log-sum-exp, per-token visibility, zeroed block scores
  if (threadIdx.x < 128) {
    const int col = threadIdx.x;
    const int t = q0 + (col >> p.logG);
    lse_sh[col] = t < Lq ? __ldg(p.lse + (long long)(qs + t) * p.Hq + h * p.G + (col & (p.G - 1))) : INFINITY;
    if (col < TPT) nvis_sh[col] = (q0 + col < Lq) ? visible(q0 + col) : 0;
  }
  for (int i = threadIdx.x; i < TPT * p.nb_pad; i += blockDim.x) bsc[i] = 0.f;
  if (warp == 9) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 8) {
    if (lane == 0 && ntiles > 0) {
      mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int pn = 0; pn < PANELS; ++pn) tma_load_3d(q_sm + pn * PANEL_BYTES, &tmQ, q_full, pn * 64, h * p.G, qs + q0);
      for (int i = 0; i < ntiles; ++i) {
        const int s = i % kScStages;
        if (i >= kScStages) mbar_wait(k_empty + s, ((i / kScStages) - 1) & 1, p.st);
        mbar_expect_tx(k_full + s, K_BYTES);
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn)
          tma_load_3d(k_sm + s * K_BYTES + pn * PANEL_BYTES, &tmK, k_full + s, pn * 64, h, ksq + i * kScKeyTile);
      }
    }
  } else if (warp == 9) {
    // The whole warp runs the control flow converged; one elected lane issues (see tc5.cuh on why).
    if (ntiles > 0) {
      const uint32_t idesc = umma_idesc<T>(128, 128, false, false);
      const uint32_t q_addr = smem_u32(q_sm);
      mbar_wait(q_full, 0, p.st);
      for (int i = 0; i < ntiles; ++i) {
        const int s = i % kScStages;
        mbar_wait(k_full + s, (i / kScStages) & 1, p.st);
        if (i >= 2) mbar_wait(s_empty + (i & 1), ((i >> 1) - 1) & 1, p.st);
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(k_sm + s * K_BYTES);
        if (elect_one()) {
          umma_block_ss<D / 16, PANEL_BYTES>(tmem + (uint32_t)((i & 1) * 128), k_addr, q_addr, idesc);
          umma_commit(k_empty + s);
          umma_commit(s_full + (i & 1));
        }
        __syncwarp();
      }
    }
  } else {
    // ===================== two threads per key: warps 0..3 take columns 0..63, warps 4..7 columns 64..127 =====================
    const int half = warp >> 2;
    const int key_l = (warp & 3) * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(half * 64);
    const int a = p.window / p.stride, c = p.block_size / p.stride;
    // this thread's (token, relative block) pairs of the fold step; the same for every tile
    const int nblk = kScKeyTile / c + (a - 1 + c - 1) / c;  // blocks touched by one key tile
    int ftok[2], fbrel[2], fk0[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int idx = threadIdx.x + 256 * r;
      ftok[r] = idx < TPT * nblk ? idx / nblk : -1;
      fbrel[r] = idx - (idx / nblk) * nblk;
      fk0[r] = fbrel[r] * c - (a - 1);
    }
    // log-sum-exp of this thread's 64 columns in registers (read once)
    float lse_r[64];
#pragma unroll
    for (int col = 0; col < 64; ++col) lse_r[col] = lse_sh[half * 64 + col];
    for (int i = 0; i < ntiles; ++i) {
      const int bsel = i & 1;
      const int key = i * kScKeyTile + key_l;  // compressed-key index inside the sequence
      // tokens are consecutive, so the tokens that see this key are a suffix of the CTA's tokens:
      // token q0 + j sees key  iff  q0 + j >= key*stride + window - 1  (and key < Lk)
      const int tok_min = key < Lk ? min(TPT, max(0, key * p.stride + p.window - 1 - q0)) : TPT;
      mbar_wait(s_full + bsel, (i >> 1) & 1, p.st);
      tc_fence_after_sync();
      uint32_t su[2][32];
      tmem_ld32(lane_base + bsel * 128, su[0]);
      tmem_ld32(lane_base + bsel * 128 + 32, su[1]);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty + bsel);
      // sums over the G heads of each token; a token's sum is kept or dropped as a whole (visible tokens are a suffix)
      constexpr int GG = 1 << LOGG;
#pragma unroll
      for (int tk = 0; tk < 64 / GG; ++tk) {
        float e[GG];
#pragma unroll
        for (int g = 0; g < GG; ++g) {
          const int col = tk * GG + g;
          e[g] = fast_exp2(fmaf(__uint_as_float(su[col >> 5][col & 31]), p.scale2, -lse_r[col]));
        }
#pragma unroll
        for (int w = GG / 2; w >= 1; w >>= 1)
#pragma unroll
          for (int g = 0; g < w; ++g) e[g] += e[g + w];
        const int tok = half * (64 / GG) + tk;
        keysc[((i & 1) * TPT + tok) * kScKeyTile + key_l] = tok >= tok_min ? e[0] : 0.f;
      }
      bar_sync_softmax();  // key scores of this tile are complete
      // fold: block b_lo + brel reads tile-local keys fk0 .. fk0 + a + c - 2 (the layout repeats every tile: c divides 128)
      const int b_lo = i * (kScKeyTile / c);
      const float* ks_t = keysc + (i & 1) * TPT * kScKeyTile;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int bb = b_lo + fbrel[r];
        if (ftok[r] < 0 || bb >= p.nb_pad) continue;
        const float* src = ks_t + ftok[r] * kScKeyTile + fk0[r];
        float part[8];
#pragma unroll
        for (int o = 0; o < 8; ++o) {   // a + c - 1 <= 8 offsets (checked on the host); loads are independent
          const bool ok = o <= a + c - 2 && fk0[r] + o >= 0 && fk0[r] + o < kScKeyTile;
          part[o] = ok ? (float)fold_weight(o, a, c) * src[o] : 0.f;
        }
        const float accb = ((part[0] + part[1]) + (part[2] + part[3])) + ((part[4] + part[5]) + (part[6] + part[7]));
        bsc[(size_t)ftok[r] * p.nb_pad + bb] += accb;
      }
    }
    bar_sync_softmax();  // every block score is final before any warp starts selecting
    // ---- selection: the tokens of the CTA are dealt to the four warps ----
    for (int tok = warp; tok < TPT; tok += 8) {
      const int t = q0 + tok;
      if (t >= Lq) break;
      warp_select_topk(bsc + (size_t)tok * p.nb_pad, t / p.block_size, p.topk_out, p.init_blocks, p.local_blocks,
                       p.topk_idx + h * p.t_sh + (long long)(qs + t) * p.t_sn, p.t_sk);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, 256);
}

template <typename T, int D>
static int launch_score_topk_tc(const void* q, const void* k, long long k_sn, long long k_sh, int Nq, int Nk, int max_seqlen_q,
                                ScoreParams p, cudaStream_t stream) {
  const int TPT = 128 / p.G;
  const size_t smem = 1024 + 128 * D * 2 + kScStages * kScKeyTile * D * 2 + 16 * sizeof(uint64_t) + 16 + 128 * sizeof(float) +
                      32 * sizeof(int) + (size_t)TPT * (2 * kScKeyTile + p.nb_pad) * sizeof(float);
  if (smem > 220 * 1024) return kUnsupported;
  CUtensorMap tmQ, tmK;
  int rc = make_tmap_3d(&tmQ, DT<T>::kTmapType, q, D, p.Hq, Nq, p.q_sh, p.q_sn, 64, p.G, TPT);
  if (rc) return rc;
  rc = make_tmap_3d(&tmK, DT<T>::kTmapType, k, D, p.Hkv, Nk, k_sh, k_sn, 64, 1, kScKeyTile);
  if (rc) return rc;
  auto kern = p.logG == 4 ? score_topk_tc_kernel<T, D, 4> : (p.logG == 3 ? score_topk_tc_kernel<T, D, 3> : score_topk_tc_kernel<T, D, 2>);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_rc(e);
  dim3 grid((max_seqlen_q + TPT - 1) / TPT, p.B, p.Hkv);
  { LaunchScope ls_("score_topk_tc", stream); kern<<<grid, 320, smem, stream>>>(tmQ, tmK, p); }
  return cuda_rc(cudaGetLastError());
}

int score_topk_tc(const void* q, const void* k, long long k_sn, long long k_sh, int Nq, int Nk, int max_seqlen_q, int head_dim,
                  int dtype, ScoreParams p, cudaStream_t stream) {
  if (p.G < 4 || p.G > 16) return kUnsupported;  // 8 to 32 tokens per CTA
  const int a = p.window / p.stride, c = p.block_size / p.stride;
  // the fold step assumes that the block layout repeats every 128-key tile and that 3 (token, block) pairs per thread suffice
  if (c <= 0 || kScKeyTile % c || a + c - 1 > 8 || (128 / p.G) * (kScKeyTile / c + (a - 1 + c - 1) / c) > 2 * 256) return kUnsupported;
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_score_topk_tc, q, k, k_sn, k_sh, Nq, Nk, max_seqlen_q, p, stream);
}

}  // namespace nsa
