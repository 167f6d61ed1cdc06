// Block-importance scores and top-k block selection for attention over compressed keys.
//
// For every query token t and KV head, with p = softmax probability of compressed key i
// (already normalised by the row's final log-sum-exp from the forward pass):
//     key_score[i]   = sum over the G query heads of the group of p
//     block_score[b] = sum_o w[o] * key_score[b*c - (a-1) + o],  a = window/stride, c = block/stride,
//                      w[o] = #{(x, y): x < a, y < c, x + y = o}
// blocks b < init_blocks and b in (bq - local_blocks, bq] (bq = t / block) are always taken; the
// remaining picks are the highest scores among blocks <= bq.  Output: ascending ids, -1 padding.
//
// The [kv_heads, tokens, keys] score matrix of the reference is never materialised: a warp owns
// 16 rows = (16/G tokens) x (G heads), sums over heads with lane shuffles inside the mma
// accumulator layout, folds key scores into per-token block scores held in shared memory, and
// selects with warp-level argmax rounds.
#include <cstdlib>

#include "attn_tile.cuh"
#include "dispatch.h"
#include "host_util.h"
#include "nsa_b200.h"
#include "topk_select.cuh"
#include "score_topk.h"

namespace nsa {

__device__ __forceinline__ int visible_keys_c(int t, int Lk, int window, int stride) {
  if (t < window - 1) return 0;
  return min(Lk, (t - window + 1) / stride + 1);
}

template <typename T, int D, int STAGES>
__global__ void __launch_bounds__(256)
score_topk_kernel(const __grid_constant__ CUtensorMap tmK, ScoreParams p) {
  constexpr int TILE_BYTES = kKeyTile * D * 2;
  constexpr int PANELS = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * TILE_BYTES);
  uint64_t* empty = full + STAGES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int WARPS = p.nwarps;
  const int QPW = 16 >> p.logG;
  const int QT = WARPS * QPW;
  float* bsc_all = reinterpret_cast<float*>(empty + STAGES);           // [QT][nb_pad]
  float* ks_all = bsc_all + (size_t)QT * p.nb_pad;                     // [QT][64]
  float* bsc = bsc_all + (size_t)warp * QPW * p.nb_pad;
  float* kst = ks_all + warp * QPW * kKeyTile;

  const int b = blockIdx.y, h = blockIdx.z;
  const int qs = __ldg(p.cu_q + b), Lq = __ldg(p.cu_q + b + 1) - qs;
  const int ksq = __ldg(p.cu_k + b), Lk = __ldg(p.cu_k + b + 1) - ksq;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int q0 = qt * QT;
  if (q0 >= Lq) return;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, WARPS);
    }
    fence_barrier_init();
  }
  for (int i = threadIdx.x; i < QT * p.nb_pad; i += blockDim.x) bsc_all[i] = 0.f;
  __syncthreads();

  const int t_hi = min(q0 + QT, Lq) - 1;
  const int ntiles = (visible_keys_c(t_hi, Lk, p.window, p.stride) + kKeyTile - 1) / kKeyTile;
  const int tw_hi = min(q0 + (warp + 1) * QPW, Lq) - 1;
  const int my_tiles = (tw_hi >= q0 + warp * QPW) ? (visible_keys_c(tw_hi, Lk, p.window, p.stride) + kKeyTile - 1) / kKeyTile : 0;

  auto issue = [&](int tile) {
    const int s = tile % STAGES;
    uint8_t* kb = smem + s * TILE_BYTES;
    mbar_expect_tx(full + s, TILE_BYTES);
#pragma unroll
    for (int pn = 0; pn < PANELS; ++pn) tma_load_3d(kb + pn * (kKeyTile * 128), &tmK, full + s, pn * 64, h, ksq + tile * kKeyTile);
  };
  if (threadIdx.x == 0)
    for (int i = 0; i < STAGES - 1 && i < ntiles; ++i) issue(i);

  const int r_lo = lane >> 2;
  int tq[2], nvis[2];
  float lse2[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r_lo + 8 * r;
    tq[r] = q0 + warp * QPW + (row >> p.logG);
    const bool ok = tq[r] < Lq;
    nvis[r] = ok ? visible_keys_c(tq[r], Lk, p.window, p.stride) : 0;
    lse2[r] = ok ? __ldg(p.lse + (long long)(qs + tq[r]) * p.Hq + h * p.G + (row & (p.G - 1))) : 0.f;
  }
  const T* qbase = static_cast<const T*>(p.q) + (long long)(qs + q0 + warp * QPW) * p.q_sn + (long long)h * p.G * p.q_sh;
  uint32_t qf[D / 16][4];
  load_a_frags_global<T, D / 16>(qf, [&](int r) -> const T* {
    const int qi = r >> p.logG;
    return (q0 + warp * QPW + qi < Lq) ? qbase + qi * p.q_sn + (r & (p.G - 1)) * p.q_sh : nullptr;
  });

  const int a = p.window / p.stride, c = p.block_size / p.stride;
  const int nshuf = min(p.logG, 3);
  const int gc = min(p.G, 8);
  const bool writer = ((r_lo & (gc - 1)) == 0);
  const int qi_w0 = r_lo >> p.logG;                  // token slot written from fragment row r_lo
  const int qi_w1 = (r_lo + 8) >> p.logG;            // token slot written from fragment row r_lo + 8 (G < 16)

  for (int i = 0; i < ntiles; ++i) {
    const int s = i % STAGES;
    if (threadIdx.x == 0) {
      const int j = i + STAGES - 1;
      if (j < ntiles) {
        if (j >= STAGES) mbar_wait(empty + (j % STAGES), ((j / STAGES) - 1) & 1, p.st);
        issue(j);
      }
    }
    __syncwarp();
    mbar_wait(full + s, (i / STAGES) & 1, p.st);
    if (i < my_tiles) {
      float sc[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
      mma_nk<T, 8, D / 16, kKeyTile>(sc, qf, smem_u32(smem + s * TILE_BYTES), 0, 0);
      const int i0 = i * kKeyTile;
      const int lim0 = nvis[0] - i0, lim1 = nvis[1] - i0;
      const int c0 = (lane & 3) * 2;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int col = j * 8 + c0 + e;
          float v0 = masked_exp2(col < lim0, sc[j][e] * p.scale2 - lse2[0]);
          float v1 = masked_exp2(col < lim1, sc[j][e + 2] * p.scale2 - lse2[1]);
          if (p.logG == 4) v0 += v1;
          for (int sh = 0; sh < nshuf; ++sh) {
            v0 += __shfl_xor_sync(0xffffffffu, v0, 4 << sh);
            if (p.logG < 4) v1 += __shfl_xor_sync(0xffffffffu, v1, 4 << sh);
          }
          if (writer) {
            kst[qi_w0 * kKeyTile + col] = v0;
            if (p.logG < 4) kst[qi_w1 * kKeyTile + col] = v1;
          }
        }
      }
      __syncwarp();
      // fold the 64 key scores of each token into its block scores
      const int b_lo = i0 / c;
      const int b_hi = min((i0 + kKeyTile - 1 + a - 1) / c, p.nb_pad - 1);
      const int nblk = b_hi - b_lo + 1;
      for (int idx = lane; idx < QPW * nblk; idx += 32) {
        const int qi = idx / nblk, bb = b_lo + idx % nblk;
        float acc = 0.f;
        for (int o = 0; o <= a + c - 2; ++o) {
          const int key = bb * c - (a - 1) + o - i0;
          if (key >= 0 && key < kKeyTile) {
            acc += (float)fold_weight(o, a, c) * kst[qi * kKeyTile + key];
          }
        }
        bsc[(size_t)qi * p.nb_pad + bb] += acc;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty + s);
  }
  __syncwarp();

  // ---- selection, one token at a time ----
  for (int qi = 0; qi < QPW; ++qi) {
    const int t = q0 + warp * QPW + qi;
    if (t >= Lq) break;
    warp_select_topk(bsc + (size_t)qi * p.nb_pad, t / p.block_size, p.topk_out, p.init_blocks, p.local_blocks,
                     p.topk_idx + h * p.t_sh + (long long)(qs + t) * p.t_sn, p.t_sk);
  }
}

template <typename T, int D>
static int launch_score_topk(const void* k, long long k_sn, long long k_sh, int Nk, int max_seqlen_q, ScoreParams p,
                             cudaStream_t stream) {
  constexpr int STAGES = 4;
  constexpr int TILE_BYTES = kKeyTile * D * 2;
  CUtensorMap tmK;
  int rc = make_tmap_3d(&tmK, DT<T>::kTmapType, k, D, p.Hkv, Nk, k_sh, k_sn, 64, 1, kKeyTile);
  if (rc) return rc;
  const int QPW = 16 / p.G;
  int nwarps = 8;
  auto smem_for = [&](int w) {
    return (size_t)1024 + STAGES * TILE_BYTES + 2 * STAGES * sizeof(uint64_t) +
           (size_t)w * QPW * (p.nb_pad + kKeyTile) * sizeof(float);
  };
  while (nwarps > 1 && smem_for(nwarps) > 200 * 1024) nwarps >>= 1;
  if (smem_for(nwarps) > 220 * 1024) return kUnsupported;  // too many candidate blocks per token for one CTA
  p.nwarps = nwarps;
  const size_t smem = smem_for(nwarps);
  auto kern = score_topk_kernel<T, D, STAGES>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_rc(e);
  const int QT = nwarps * QPW;
  dim3 grid((max_seqlen_q + QT - 1) / QT, p.B, p.Hkv);
  { LaunchScope ls_("score_topk", stream); kern<<<grid, nwarps * 32, smem, stream>>>(tmK, p); }
  return cuda_rc(cudaGetLastError());
}

}  // namespace nsa

extern "C" int nsa_compressed_attn_topk(const void* q, const void* k, const float* lse, const int* cu_seqlens_q,
                                        const int* cu_seqlens_k, int* topk_idx, int total_q, int total_k, int batch,
                                        int max_seqlen_q, int num_q_heads, int num_kv_heads, int head_dim,
                                        int kernel_size, int kernel_stride, int block_size, int topk, int init_blocks,
                                        int local_blocks, const long long* strides, float sm_scale, int dtype,
                                        void* stream) {
  using namespace nsa;
  if (!q || !k || !lse || !cu_seqlens_q || !cu_seqlens_k || !topk_idx || !strides) return kInvalid;
  if (total_q <= 0 || total_k <= 0 || batch <= 0 || max_seqlen_q <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads)
    return kInvalid;
  if (kernel_size % kernel_stride || block_size % kernel_stride || kernel_stride < 1 || topk < 1) return kInvalid;
  if (init_blocks < 0 || local_blocks < 0 || topk < init_blocks + local_blocks) return kInvalid;
  const int G = num_q_heads / num_kv_heads;
  if (G > 16 || (G & (G - 1))) return kUnsupported;
  ScoreParams p;
  p.q = q; p.lse = lse; p.topk_idx = topk_idx; p.cu_q = cu_seqlens_q; p.cu_k = cu_seqlens_k;
  // strides: q_n q_h k_n k_h idx_h idx_n idx_k
  p.q_sn = strides[0]; p.q_sh = strides[1];
  p.t_sh = strides[4]; p.t_sn = strides[5]; p.t_sk = strides[6];
  p.B = batch; p.Hq = num_q_heads; p.Hkv = num_kv_heads; p.G = G;
  p.logG = 0;
  while ((1 << p.logG) < G) ++p.logG;
  p.window = kernel_size; p.stride = kernel_stride; p.block_size = block_size;
  const int max_blocks = (max_seqlen_q + block_size - 1) / block_size;
  p.topk_out = topk < max_blocks ? topk : max_blocks;
  p.init_blocks = init_blocks; p.local_blocks = local_blocks;
  p.nb_pad = (max_blocks + 31) & ~31;
  p.scale2 = sm_scale * kLog2e;
  p.st.word = status_word();
  if ((p.q_sn | p.q_sh) % 8 || !aligned16(q)) return kInvalid;
  {
    // two row tiles per CTA when their block scores fit in shared memory, else one, else the mma.sync kernel (G < 4)
    int rc = score_topk_pp_tc(q, k, strides[2], strides[3], total_q, total_k, max_seqlen_q, head_dim, dtype, p,
                              static_cast<cudaStream_t>(stream));
    if (rc == kUnsupported)
      rc = score_topk_tc(q, k, strides[2], strides[3], total_q, total_k, max_seqlen_q, head_dim, dtype, p,
                         static_cast<cudaStream_t>(stream));
    if (rc != kUnsupported) return rc;
  }
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_score_topk, k, strides[2], strides[3], total_k, max_seqlen_q, p,
                          static_cast<cudaStream_t>(stream));
}
