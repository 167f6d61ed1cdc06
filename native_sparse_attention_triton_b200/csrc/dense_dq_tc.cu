// dQ pass of dense strided-causal attention on the 5th-generation tensor cores.
//
// CTA = 128 rows = (128/G tokens) x (G heads of one KV head), key tiles of 128:
//     S  = Q  K^T   [128 x 128]  A = Q  (K-major), B = K tile (K-major)       TMEM [0,128)
//     dP = dO V^T   [128 x 128]  A = dO (K-major), B = V tile (K-major)       TMEM [128,256)
//     dQ += dS K    [128 x D]    A = dS (SMEM, K-major), B = K tile (MN-major) TMEM [256,256+D)
// Q and dO stay in SMEM for the whole CTA; K tiles alternate between two buffers (a K tile is needed from its
// S product until its dQ product), V has one buffer (free as soon as dP is done).  The issuing thread keeps two
// independent streams going -- S/dP of the next tile and dQ of the current one -- whichever is ready.
//   warps 0..7 : two threads per row (64 key columns each): P = exp2(S*scale - lse), dS = P (dP - delta) scale
//                as 16-bit into the SMEM tile the dQ product reads; they also compute delta = sum(O * dO) of their
//                row up front and publish (lse, delta) for the dK/dV pass; at the end they store dQ
//   warp 8     : TMA producer;   warp 9 : TMEM allocation and MMA issue (one thread)
#include "attn_bwd.h"
#include "attn_tile.cuh"
#include "dispatch.h"
#include "host_util.h"
#include "tc5.cuh"

namespace nsa {

template <typename T, int D>
__global__ void __launch_bounds__(320, 1)
dense_dq_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                   const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, DenseBwdParams p) {
  constexpr int KT = 128;
  constexpr int PANELS = D / 64;
  constexpr int PANEL_BYTES = 128 * 128;
  constexpr int ROW_BYTES = 128 * D * 2;   // Q, dO, K tile, V tile: all [128][D]
  constexpr int DS_BYTES = 128 * KT * 2;   // dS tile [128 rows][128 keys]: 2 panels
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_sm = smem;
  uint8_t* do_sm = q_sm + ROW_BYTES;
  uint8_t* k_sm = do_sm + ROW_BYTES;        // two buffers
  uint8_t* v_sm = k_sm + 2 * ROW_BYTES;
  uint8_t* ds_sm = v_sm + ROW_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ds_sm + DS_BYTES);
  uint64_t* qdo_full = bars;
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* k_empty = k_full + 2;   // [2]
  uint64_t* v_full = k_empty + 2;
  uint64_t* v_empty = v_full + 1;
  uint64_t* sdp_full = v_empty + 1;
  uint64_t* sdp_empty = sdp_full + 1;
  uint64_t* ds_full = sdp_empty + 1;
  uint64_t* ds_empty = ds_full + 1;
  uint64_t* all_done = ds_empty + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(all_done + 1);
  float* delta_sh = reinterpret_cast<float*>(tmem_slot + 2);  // [2][128] partial row sums of O*dO

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.y, h = blockIdx.z;
  const int qs = __ldg(p.cu_q + b), Lq = __ldg(p.cu_q + b + 1) - qs;
  const int ksq = __ldg(p.cu_k + b), Lk = __ldg(p.cu_k + b + 1) - ksq;
  const int QT = 128 >> p.logG;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int q0 = qt * QT;
  if (q0 >= Lq) return;
  auto visible = [&](int t) {
    if (!p.causal) return Lk;
    return t < p.window - 1 ? 0 : min(Lk, (t - p.window + 1) / p.stride + 1);
  };
  const int t_hi = min(q0 + QT, Lq) - 1;
  const int ntiles = (visible(t_hi) + KT - 1) / KT;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full + s, 1);
      mbar_init(k_empty + s, 1);
    }
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(sdp_empty, 8);
    mbar_init(ds_full, 8);
    mbar_init(ds_empty, 1);
    mbar_init(all_done, 1);
    fence_barrier_init();
  }
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
      mbar_expect_tx(qdo_full, 2 * ROW_BYTES);
#pragma unroll
      for (int pn = 0; pn < PANELS; ++pn) {
        tma_load_3d(q_sm + pn * PANEL_BYTES, &tmQ, qdo_full, pn * 64, h * p.G, qs + q0);
        tma_load_3d(do_sm + pn * PANEL_BYTES, &tmDO, qdo_full, pn * 64, h * p.G, qs + q0);
      }
      for (int i = 0; i < ntiles; ++i) {
        const int s = i & 1;
        if (i >= 2) mbar_wait(k_empty + s, ((i >> 1) - 1) & 1, p.st);
        mbar_expect_tx(k_full + s, ROW_BYTES);
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn)
          tma_load_3d(k_sm + s * ROW_BYTES + pn * PANEL_BYTES, &tmK, k_full + s, pn * 64, h, ksq + i * KT);
        if (i >= 1) mbar_wait(v_empty, (i - 1) & 1, p.st);
        mbar_expect_tx(v_full, ROW_BYTES);
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn) tma_load_3d(v_sm + pn * PANEL_BYTES, &tmV, v_full, pn * 64, h, ksq + i * KT);
      }
    }
  } else if (warp == 9) {
    // ===================== MMA issuer =====================
    if (lane == 0 && ntiles > 0) {
      const uint32_t idesc_s = umma_idesc<T>(128, KT, false, false);
      const uint32_t idesc_q = umma_idesc<T>(128, D, false, true);
      const uint32_t q_addr = smem_u32(q_sm), do_addr = smem_u32(do_sm), v_addr = smem_u32(v_sm), ds_addr = smem_u32(ds_sm);
      auto issue_sdp = [&](int i) {
        const uint32_t k_addr = smem_u32(k_sm + (i & 1) * ROW_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * PANEL_BYTES + (kk & 3) * 32;
          umma_ss(tmem, umma_desc_kmajor(q_addr + off), umma_desc_kmajor(k_addr + off), idesc_s, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * PANEL_BYTES + (kk & 3) * 32;
          umma_ss(tmem + 128, umma_desc_kmajor(do_addr + off), umma_desc_kmajor(v_addr + off), idesc_s, kk > 0);
        }
        umma_commit(v_empty);
        umma_commit(sdp_full);
      };
      auto issue_dq = [&](int i) {
        const uint32_t k_addr = smem_u32(k_sm + (i & 1) * ROW_BYTES);
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
          const uint32_t a_off = (kk >> 2) * PANEL_BYTES + (kk & 3) * 32;
          umma_ss(tmem + 256, umma_desc_kmajor(ds_addr + a_off), umma_desc_mnmajor(k_addr + kk * 2048, PANEL_BYTES), idesc_q,
                  i > 0 || kk > 0);
        }
        umma_commit(k_empty + (i & 1));
        umma_commit(ds_empty);
      };
      mbar_wait(qdo_full, 0, p.st);
      int ns = 0, nd = 0;
      long long t0 = clock64();
      while (nd < ntiles) {
        bool progressed = false;
        if (ns < ntiles && ns - nd < 2 && mbar_try_wait(k_full + (ns & 1), (ns >> 1) & 1) && mbar_try_wait(v_full, ns & 1) &&
            (ns < 1 || mbar_try_wait(sdp_empty, (ns - 1) & 1))) {
          tc_fence_after_sync();
          issue_sdp(ns);
          ++ns;
          progressed = true;
        }
        if (nd < ns && mbar_try_wait(ds_full, nd & 1)) {
          tc_fence_after_sync();
          issue_dq(nd);
          ++nd;
          progressed = true;
        }
        if (progressed) {
          t0 = clock64();
        } else if (clock64() - t0 > (1ll << 30) || (p.st.word && (*reinterpret_cast<volatile int*>(p.st.word) & kErrWaitTimeout))) {
          p.st.raise(kErrWaitTimeout);
          break;
        }
      }
      umma_commit(all_done);
    }
  } else {
    // ===================== softmax / dS: two threads per row =====================
    const int half = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const int tpos = q0 + (row >> p.logG);
    const int head = h * p.G + (row & (p.G - 1));
    const bool valid = tpos < Lq;
    const int nvis = valid ? visible(tpos) : 0;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    // ---- delta = sum_d O * dO of this row (each of the two threads sums half of the row) ----
    float part = 0.f;
    if (valid) {
      const T* orow = static_cast<const T*>(p.o) + (long long)(qs + tpos) * p.o_sn + (long long)head * p.o_sh + half * (D / 2);
      const T* drow = static_cast<const T*>(p.dout) + (long long)(qs + tpos) * p.do_sn + (long long)head * p.do_sh + half * (D / 2);
#pragma unroll
      for (int c = 0; c < D / 16; ++c) {
        const uint4 ov = __ldg(reinterpret_cast<const uint4*>(orow) + c), dv = __ldg(reinterpret_cast<const uint4*>(drow) + c);
        const uint32_t ou[4] = {ov.x, ov.y, ov.z, ov.w}, du[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 a = DT<T>::unpack(ou[e]), bb = DT<T>::unpack(du[e]);
          part += a.x * bb.x + a.y * bb.y;
        }
      }
    }
    delta_sh[half * 128 + row] = part;
    asm volatile("bar.sync 1, 256;\n" ::: "memory");
    const float delta = delta_sh[row] + delta_sh[128 + row];
    const float lse2 = valid ? __ldg(p.lse + (long long)(qs + tpos) * p.Hq + head) : INFINITY;
    if (valid && half == 0) p.ld[(long long)(qs + tpos) * p.Hq + head] = make_float2(lse2, delta);
    const float nlse = -lse2;

    for (int i = 0; i < ntiles; ++i) {
      mbar_wait(sdp_full, i & 1, p.st);
      tc_fence_after_sync();
      uint32_t su[2][32], du[2][32];
      tmem_ld32(lane_base + half * 64, su[0]);
      tmem_ld32(lane_base + half * 64 + 32, su[1]);
      tmem_ld32(lane_base + 128 + half * 64, du[0]);
      tmem_ld32(lane_base + 128 + half * 64 + 32, du[1]);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(sdp_empty);
      const int lim = nvis - i * KT - half * 64;
      uint32_t dw[32];
#pragma unroll
      for (int j = 0; j < 64; j += 2) {
        const float p0 = masked_exp2(j < lim, fmaf(__uint_as_float(su[j >> 5][j & 31]), p.scale2, nlse));
        const float p1 = masked_exp2(j + 1 < lim, fmaf(__uint_as_float(su[(j + 1) >> 5][(j + 1) & 31]), p.scale2, nlse));
        const float d0 = p0 * (__uint_as_float(du[j >> 5][j & 31]) - delta) * p.sm_scale;
        const float d1 = p1 * (__uint_as_float(du[(j + 1) >> 5][(j + 1) & 31]) - delta) * p.sm_scale;
        dw[j >> 1] = DT<T>::pack(d0, d1);
      }
      if (i > 0) mbar_wait(ds_empty, (i - 1) & 1, p.st);  // dQ of the previous tile has read the dS tile
      const uint32_t dsrow = smem_u32(ds_sm) + half * PANEL_BYTES + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(dsrow + ((c ^ (row & 7)) << 4)), "r"(dw[c * 4]),
                     "r"(dw[c * 4 + 1]), "r"(dw[c * 4 + 2]), "r"(dw[c * 4 + 3]) : "memory");
      fence_proxy_async();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    // ---- epilogue: dQ row (this thread stores D/2 of its D values) ----
    if (ntiles > 0) {
      mbar_wait(all_done, 0, p.st);
      tc_fence_after_sync();
    }
    T* dqrow = static_cast<T*>(p.dq) + (long long)(qs + tpos) * p.dq_sn + (long long)head * p.dq_sh + half * (D / 2);
#pragma unroll
    for (int c = 0; c < D / 64; ++c) {
      uint32_t r[32];
      if (ntiles > 0) {
        tmem_ld32(lane_base + 256 + half * (D / 2) + c * 32, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = 0u;
      }
      if (valid) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 out;
          out.x = DT<T>::pack(__uint_as_float(r[q4 * 8 + 0]), __uint_as_float(r[q4 * 8 + 1]));
          out.y = DT<T>::pack(__uint_as_float(r[q4 * 8 + 2]), __uint_as_float(r[q4 * 8 + 3]));
          out.z = DT<T>::pack(__uint_as_float(r[q4 * 8 + 4]), __uint_as_float(r[q4 * 8 + 5]));
          out.w = DT<T>::pack(__uint_as_float(r[q4 * 8 + 6]), __uint_as_float(r[q4 * 8 + 7]));
          *reinterpret_cast<uint4*>(dqrow + c * 32 + q4 * 8) = out;
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, 512);
}

template <typename T, int D>
static int launch_dense_dq_tc(const void* k, const void* v, long long k_sn, long long k_sh, long long v_sn, long long v_sh,
                              int total_q, int total_k, int max_seqlen_q, DenseBwdParams p, cudaStream_t stream) {
  CUtensorMap tmQ, tmDO, tmK, tmV;
  const int QT = 128 / p.G;
  int rc = make_tmap_3d(&tmQ, DT<T>::kTmapType, p.q, D, p.Hq, total_q, p.q_sh, p.q_sn, 64, p.G, QT);
  if (rc) return rc;
  rc = make_tmap_3d(&tmDO, DT<T>::kTmapType, p.dout, D, p.Hq, total_q, p.do_sh, p.do_sn, 64, p.G, QT);
  if (rc) return rc;
  rc = make_tmap_3d(&tmK, DT<T>::kTmapType, k, D, p.Hkv, total_k, k_sh, k_sn, 64, 1, 128);
  if (rc) return rc;
  rc = make_tmap_3d(&tmV, DT<T>::kTmapType, v, D, p.Hkv, total_k, v_sh, v_sn, 64, 1, 128);
  if (rc) return rc;
  const size_t smem = 1024 + 5 * (128 * D * 2) + 128 * 128 * 2 + 16 * sizeof(uint64_t) + 16 + 256 * sizeof(float);
  auto kern = dense_dq_tc_kernel<T, D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_rc(e);
  dim3 grid((max_seqlen_q + QT - 1) / QT, p.B, p.Hkv);
  { LaunchScope ls_("dense_dq_tc", stream); kern<<<grid, 320, smem, stream>>>(tmQ, tmDO, tmK, tmV, p); }
  return cuda_rc(cudaGetLastError());
}

int dense_dq_tc(const void* k, const void* v, long long k_sn, long long k_sh, long long v_sn, long long v_sh, int total_q,
                int total_k, int max_seqlen_q, int head_dim, int dtype, DenseBwdParams p, cudaStream_t stream) {
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_dense_dq_tc, k, v, k_sn, k_sh, v_sn, v_sh, total_q, total_k, max_seqlen_q, p,
                          stream);
}

}  // namespace nsa
