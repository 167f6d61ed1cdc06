// dQ pass of dense strided-causal attention on the 5th-generation tensor cores.
//
// CTA = 128 rows = (128/G tokens) x (G heads of one KV head), key tiles of 128:
//     S  = Q  K^T   [128 x 128]  A = Q  (SMEM, K-major), B = K tile (SMEM, K-major)       TMEM [0,128)
//     dP = dO V^T   [128 x 128]  A = dO (SMEM, K-major), B = V tile (SMEM, K-major)       TMEM [128,256)
//     dQ += dS K    [128 x D]    A = dS (TMEM, 16-bit),  B = K tile (SMEM, MN-major)      TMEM [256,256+D)
// Q and dO stay in SMEM for the whole CTA; K tiles go through a ring of three (a K tile lives from its S product
// to its dQ product), V tiles through a ring of two.  dS is written by the softmax threads over the dP logits it
// was computed from, so the dQ product reads its A operand from tensor memory.  The issuing thread polls three
// queues; the pipe order in steady state is S(i+1), dQ(i), dP(i+1): the S product of the next tile covers the
// dS phase of the current one and dQ/dP cover the P phase of the next.
//   warps 0..7 : two threads per row (64 key columns each).  P phase (after S): P = exp2(S*scale - lse) kept in
//                registers; dS phase (after dP): dS = P (dP - delta) scale -> TMEM.  They also compute
//                delta = sum(O * dO) of their row up front and publish (lse, delta) for the dK/dV pass; at the end
//                they store dQ
//                through shared memory and one TMA store per panel (row by row in the last CTA of a sequence)
//   warp 8     : TMA producer (Q and the first K tile first, so that the first S product starts before dO, V and O have
//                arrived);   warp 9 : TMEM allocation and MMA issue (one thread)
#include "attn_bwd.h"
#include "attn_tile.cuh"
#include "dispatch.h"
#include "host_util.h"
#include "tc5.cuh"

namespace nsa {

namespace {
constexpr int kDqKStages = 3;
constexpr int kDqVStages = 2;
}

template <typename T, int D>
__global__ void __launch_bounds__(320, 1)
dense_dq_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                   const __grid_constant__ CUtensorMap tmO, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const __grid_constant__ CUtensorMap tmDQ, DenseBwdParams p) {
  constexpr int KT = 128;
  constexpr int PANELS = D / 64;
  constexpr int PANEL_BYTES = 128 * 128;
  constexpr int ROW_BYTES = 128 * D * 2;   // Q, dO, K tile, V tile: all [128][D]
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* q_sm = smem;
  uint8_t* do_sm = q_sm + ROW_BYTES;
  uint8_t* k_sm = do_sm + ROW_BYTES;                 // ring of kDqKStages
  uint8_t* v_sm = k_sm + kDqKStages * ROW_BYTES;     // ring of kDqVStages
  float* delta_sh = reinterpret_cast<float*>(v_sm + kDqVStages * ROW_BYTES);  // [2][128] partial row sums of O*dO
  uint64_t* bars = reinterpret_cast<uint64_t*>(delta_sh + 256);
  uint64_t* qdo_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = k_full + kDqKStages;
  uint64_t* v_full = k_empty + kDqKStages;
  uint64_t* v_empty = v_full + kDqVStages;
  uint64_t* s_full = v_empty + kDqVStages;
  uint64_t* s_empty = s_full + 1;
  uint64_t* dp_full = s_empty + 1;
  uint64_t* ds_full = dp_full + 1;
  uint64_t* all_done = ds_full + 1;
  uint64_t* o_full = all_done + 1;   // the O rows, staged in the last K stage for the delta computation
  uint64_t* o_done = o_full + 1;     // ... and read by all softmax warps
  uint64_t* q_full = o_done + 1;     // the Q rows alone (the first S product needs only them and the first K tile)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (smem_u32(smem) & 1023u) {  // the swizzled operand tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) p.st.raise(kErrSmemLayout);
    return;
  }
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
  // with a sliding window the first key tiles are invisible to every row of the CTA: start at tile kt0
  const int kt0 = p.left >= 0 ? max(0, q0 - p.left) / KT : 0;
  const int ntiles = max(0, (visible(t_hi) + KT - 1) / KT - kt0);

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int s = 0; s < kDqKStages; ++s) {
      mbar_init(k_full + s, 1);
      mbar_init(k_empty + s, 1);
    }
    for (int s = 0; s < kDqVStages; ++s) {
      mbar_init(v_full + s, 1);
      mbar_init(v_empty + s, 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_empty, 8);
    mbar_init(dp_full, 1);
    mbar_init(ds_full, 8);
    mbar_init(all_done, 1);
    mbar_init(o_full, 1);
    mbar_init(o_done, 8);
    mbar_init(q_full, 1);
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
      // Order of arrival: Q and the first K tile (the first S product can start), then dO and the first V tile (dP), then O
      // (delta), then the remaining key tiles.
      uint8_t* o_sm = k_sm + (kDqKStages - 1) * ROW_BYTES;  // the O rows borrow the last K stage, which the ring needs only
                                                            // for its third tile
      mbar_expect_tx(q_full, ROW_BYTES);
#pragma unroll
      for (int pn = 0; pn < PANELS; ++pn) tma_load_3d(q_sm + pn * PANEL_BYTES, &tmQ, q_full, pn * 64, h * p.G, qs + q0);
      for (int i = 0; i < ntiles; ++i) {
        const int sk = i % kDqKStages, sv = i % kDqVStages;
        if (i >= kDqKStages) mbar_wait(k_empty + sk, ((i / kDqKStages) - 1) & 1, p.st);
        if (i == kDqKStages - 1) mbar_wait(o_done, 0, p.st);
        mbar_expect_tx(k_full + sk, ROW_BYTES);
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn)
          tma_load_3d(k_sm + sk * ROW_BYTES + pn * PANEL_BYTES, &tmK, k_full + sk, pn * 64, h, ksq + (kt0 + i) * KT);
        if (i == 0) {
          mbar_expect_tx(qdo_full, ROW_BYTES);
#pragma unroll
          for (int pn = 0; pn < PANELS; ++pn) tma_load_3d(do_sm + pn * PANEL_BYTES, &tmDO, qdo_full, pn * 64, h * p.G, qs + q0);
        }
        if (i >= kDqVStages) mbar_wait(v_empty + sv, ((i / kDqVStages) - 1) & 1, p.st);
        mbar_expect_tx(v_full + sv, ROW_BYTES);
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn)
          tma_load_3d(v_sm + sv * ROW_BYTES + pn * PANEL_BYTES, &tmV, v_full + sv, pn * 64, h, ksq + (kt0 + i) * KT);
        if (i == 0) {
          mbar_expect_tx(o_full, ROW_BYTES);
#pragma unroll
          for (int pn = 0; pn < PANELS; ++pn) tma_load_3d(o_sm + pn * PANEL_BYTES, &tmO, o_full, pn * 64, h * p.G, qs + q0);
        }
      }
    }
  } else if (warp == 9) {
    // ===================== MMA issuer =====================
    // The whole warp runs the control flow converged; one elected lane issues (see tc5.cuh on why).
    if (ntiles > 0) {
      const uint32_t idesc_s = umma_idesc<T>(128, KT, false, false);
      const uint32_t idesc_q = umma_idesc<T>(128, D, false, true);
      const uint32_t q_addr = smem_u32(q_sm), do_addr = smem_u32(do_sm), k_base = smem_u32(k_sm), v_base = smem_u32(v_sm);
      mbar_wait(q_full, 0, p.st);
      // S(i) may start once the softmax threads have read S(i-1); dP(i) once dQ(i-1) has been issued (it overwrites
      // dS(i-1); the pipe executes in issue order); dQ(i) needs dS(i).
      int ns = 0, np = 0, nq = 0;
      long long t0 = 0;
      int idle = 0;
      while (nq < ntiles) {
        bool progressed = false;
        if (ns < ntiles && mbar_test(k_full + (ns % kDqKStages), (ns / kDqKStages) & 1) &&
            (ns < 1 || mbar_test(s_empty, (ns - 1) & 1))) {
          tc_fence_after_sync();
          if (elect_one()) {
            umma_block_ss<D / 16, PANEL_BYTES>(tmem, q_addr, k_base + (ns % kDqKStages) * ROW_BYTES, idesc_s);
            umma_commit(s_full);
          }
          __syncwarp();
          ++ns;
          progressed = true;
        }
        if (nq < np && mbar_test(ds_full, nq & 1)) {
          tc_fence_after_sync();
          const int sk = nq % kDqKStages;
          if (elect_one()) {
            umma_block_ts<KT / 16, PANEL_BYTES>(tmem + 256, tmem + 128, k_base + sk * ROW_BYTES, idesc_q, nq > 0);
            umma_commit(k_empty + sk);
          }
          __syncwarp();
          ++nq;
          progressed = true;
        }
        if (np < ntiles && np == nq && np < ns && mbar_test(v_full + (np % kDqVStages), (np / kDqVStages) & 1) &&
            (np > 0 || mbar_test(qdo_full, 0))) {  // the first dP also needs the dO rows
          tc_fence_after_sync();
          const int sv = np % kDqVStages;
          if (elect_one()) {
            umma_block_ss<D / 16, PANEL_BYTES>(tmem + 128, do_addr, v_base + sv * ROW_BYTES, idesc_s);
            umma_commit(v_empty + sv);
            umma_commit(dp_full);
          }
          __syncwarp();
          ++np;
          progressed = true;
        }
        if (progressed) {
          idle = 0;
        } else if (((++idle) & 1023) == 0) {
          // bounded: every 1024 idle polls look at the clock and at the grid-wide abort flag (a global-memory read,
          // far too slow to sit in the polling path itself)
          if (idle == 1024) t0 = clock64();
          if (clock64() - t0 > (1ll << 30) || (p.st.word && (*reinterpret_cast<volatile int*>(p.st.word) & kErrWaitTimeout))) {
            p.st.raise(kErrWaitTimeout);
            break;
          }
        }
      }
      if (elect_one()) umma_commit(all_done);
      __syncwarp();
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
    // ---- delta = sum_d O * dO of this row, from the SMEM copies (each of the two threads sums half of the row) ----
    const float lse2 = valid ? __ldg(p.lse + (long long)(qs + tpos) * p.Hq + head) : INFINITY;
    float part = 0.f;
    if (ntiles > 0) {
      mbar_wait(qdo_full, 0, p.st);
      mbar_wait(o_full, 0, p.st);
      const uint32_t o_addr = smem_u32(k_sm + (kDqKStages - 1) * ROW_BYTES), d_addr = smem_u32(do_sm);
#pragma unroll
      for (int c = 0; c < D / 16; ++c) {
        const int ci = half * (D / 16) + c;  // 16-byte chunk of the row
        const uint32_t off = (ci >> 3) * PANEL_BYTES + row * 128 + (((ci & 7) ^ (row & 7)) << 4);
        uint32_t ou[4], du[4];
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];\n" : "=r"(ou[0]), "=r"(ou[1]), "=r"(ou[2]), "=r"(ou[3]) : "r"(o_addr + off));
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];\n" : "=r"(du[0]), "=r"(du[1]), "=r"(du[2]), "=r"(du[3]) : "r"(d_addr + off));
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 a = DT<T>::unpack(ou[e]), bb = DT<T>::unpack(du[e]);
          part += a.x * bb.x + a.y * bb.y;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(o_done);
    }
    if (!valid) part = 0.f;
    delta_sh[half * 128 + row] = part;
    asm volatile("bar.sync 1, 256;\n" ::: "memory");
    const float delta = delta_sh[row] + delta_sh[128 + row];
    if (valid && half == 0) p.ld[(long long)(qs + tpos) * p.Hq + head] = make_float2(lse2, delta);
    const float nlse = -lse2;
    const float ndsc = -delta * p.sm_scale;

    for (int i = 0; i < ntiles; ++i) {
      // ---- P phase ----
      mbar_wait(s_full, i & 1, p.st);
      tc_fence_after_sync();
      float pf[64];
      {
        uint32_t su[2][32];
        tmem_ld32(lane_base + half * 64, su[0]);
        tmem_ld32(lane_base + half * 64 + 32, su[1]);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_empty);
        const int lim = nvis - (kt0 + i) * KT - half * 64;  // columns below lim are visible ...
        const int lo = p.left >= 0 ? tpos - p.left - (kt0 + i) * KT - half * 64 : 0;  // ... from column lo on
        // tiles every row of the warp sees in full (all but those on the mask's edges) skip the mask instructions
        if (__all_sync(0xffffffffu, lim >= 64 && lo <= 0)) {
#pragma unroll
          for (int j = 0; j < 64; j += 2) {
            const float2 x = ffma2(make_float2(__uint_as_float(su[j >> 5][j & 31]), __uint_as_float(su[j >> 5][(j & 31) + 1])),
                                   make_float2(p.scale2, p.scale2), make_float2(nlse, nlse));
            pf[j] = fast_exp2(x.x);
            pf[j + 1] = fast_exp2(x.y);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 64; ++j)
            pf[j] = masked_exp2(j < lim && j >= lo, fmaf(__uint_as_float(su[j >> 5][j & 31]), p.scale2, nlse));
        }
      }
      // ---- dS phase ----
      mbar_wait(dp_full, i & 1, p.st);
      tc_fence_after_sync();
      {
        uint32_t du[2][32];
        tmem_ld32(lane_base + 128 + half * 64, du[0]);
        tmem_ld32(lane_base + 128 + half * 64 + 32, du[1]);
        tmem_ld_wait();
        uint32_t dw[32];
#pragma unroll
        for (int j = 0; j < 64; j += 2) {
          const float2 t2 = ffma2(make_float2(__uint_as_float(du[j >> 5][j & 31]), __uint_as_float(du[j >> 5][(j & 31) + 1])),
                                  make_float2(p.sm_scale, p.sm_scale), make_float2(ndsc, ndsc));
          const float2 d2 = fmul2(make_float2(pf[j], pf[j + 1]), t2);
          dw[j >> 1] = DT<T>::pack(d2.x, d2.y);
        }
        tmem_st32(lane_base + 128 + half * 64, dw);  // over this thread's own dP logits
        tmem_st_wait();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    // ---- epilogue: dQ row (this thread stores D/2 of its D values) ----
    if (ntiles > 0) {
      mbar_wait(all_done, 0, p.st);
      tc_fence_after_sync();
    }
    // A CTA whose rows all belong to its sequence stages the tile in shared memory (the first K stage, free by now, in the
    // swizzled panel layout the loads use) and writes it with one TMA store per panel: 16-byte stores of one row per lane
    // cost several thousand clocks of the store path per CTA.  Other CTAs (the last of a sequence) store row by row.
    const bool staged = ntiles > 0 && q0 + QT <= Lq;
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
      if (staged) {
        const uint32_t stage = smem_u32(k_sm);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int ci = (half * (D / 2) + c * 32) / 8 + q4;  // 16-byte chunk of the row
          const uint32_t off = (ci >> 3) * PANEL_BYTES + row * 128 + (((ci & 7) ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(stage + off),
                       "r"(DT<T>::pack(__uint_as_float(r[q4 * 8 + 0]), __uint_as_float(r[q4 * 8 + 1]))),
                       "r"(DT<T>::pack(__uint_as_float(r[q4 * 8 + 2]), __uint_as_float(r[q4 * 8 + 3]))),
                       "r"(DT<T>::pack(__uint_as_float(r[q4 * 8 + 4]), __uint_as_float(r[q4 * 8 + 5]))),
                       "r"(DT<T>::pack(__uint_as_float(r[q4 * 8 + 6]), __uint_as_float(r[q4 * 8 + 7]))) : "memory");
        }
      } else if (valid) {
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
    if (staged) {
      fence_proxy_async();  // the TMA engine reads the tile through the async proxy
      asm volatile("bar.sync 1, 256;\n" ::: "memory");
      if (threadIdx.x == 0) {
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn) tma_store_3d(&tmDQ, k_sm + pn * PANEL_BYTES, pn * 64, h * p.G, qs + q0);
        tma_store_commit();
        tma_store_wait_read();
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
  CUtensorMap tmQ, tmDO, tmO, tmK, tmV;
  const int QT = 128 / p.G;
  int rc = make_tmap_3d(&tmQ, DT<T>::kTmapType, p.q, D, p.Hq, total_q, p.q_sh, p.q_sn, 64, p.G, QT);
  if (rc) return rc;
  rc = make_tmap_3d(&tmDO, DT<T>::kTmapType, p.dout, D, p.Hq, total_q, p.do_sh, p.do_sn, 64, p.G, QT);
  if (rc) return rc;
  rc = make_tmap_3d(&tmO, DT<T>::kTmapType, p.o, D, p.Hq, total_q, p.o_sh, p.o_sn, 64, p.G, QT);
  if (rc) return rc;
  rc = make_tmap_3d(&tmK, DT<T>::kTmapType, k, D, p.Hkv, total_k, k_sh, k_sn, 64, 1, 128);
  if (rc) return rc;
  rc = make_tmap_3d(&tmV, DT<T>::kTmapType, v, D, p.Hkv, total_k, v_sh, v_sn, 64, 1, 128);
  if (rc) return rc;
  CUtensorMap tmDQ;
  rc = make_tmap_3d(&tmDQ, DT<T>::kTmapType, p.dq, D, p.Hq, total_q, p.dq_sh, p.dq_sn, 64, p.G, QT);
  if (rc) return rc;
  const size_t smem = (size_t)(2 + kDqKStages + kDqVStages) * (128 * D * 2) + 256 * sizeof(float) + 24 * sizeof(uint64_t) + 16;
  auto kern = dense_dq_tc_kernel<T, D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_rc(e);
  dim3 grid((max_seqlen_q + QT - 1) / QT, p.B, p.Hkv);
  { LaunchScope ls_("dense_dq_tc", stream); kern<<<grid, 320, smem, stream>>>(tmQ, tmDO, tmO, tmK, tmV, tmDQ, p); }
  return cuda_rc(cudaGetLastError());
}

int dense_dq_tc(const void* k, const void* v, long long k_sn, long long k_sh, long long v_sn, long long v_sh, int total_q,
                int total_k, int max_seqlen_q, int head_dim, int dtype, DenseBwdParams p, cudaStream_t stream) {
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_dense_dq_tc, k, v, k_sn, k_sh, v_sn, v_sh, total_q, total_k, max_seqlen_q, p,
                          stream);
}

}  // namespace nsa
