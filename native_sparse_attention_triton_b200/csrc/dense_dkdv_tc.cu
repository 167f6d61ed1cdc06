// dK/dV pass of dense strided-causal attention on the 5th-generation tensor cores (head_dim 128),
// transposed formulation: the KEYS are the M dimension of every product.
//
// CTA = one tile of 128 keys (K and V tiles resident in SMEM) x a stream of row tiles; a row tile is
// 128 rows = (128/G consecutive tokens) x (G query heads of the KV group).
//     S^T  = K  Q^T          [128 keys x 128 rows]   A = K tile (SMEM, K-major),  B = Q  rows (SMEM, K-major)
//     dP^T = V  dO^T         [128 keys x 128 rows]   A = V tile (SMEM, K-major),  B = dO rows (SMEM, K-major)
//     dV  += P^T  dO         [128 keys x 128 d]      A = P^T  (TMEM, 16-bit),     B = dO rows (SMEM, MN-major)
//     dK  += dS^T Q          [128 keys x 128 d]      A = dS^T (TMEM, 16-bit),     B = Q  rows (SMEM, MN-major)
// P^T and dS^T are written by the softmax threads over the logits they were computed from, so the two
// accumulating products read their A operand from tensor memory and the only shared-memory traffic of the
// tensor pipe is one 128 x 128 operand per product.  A thread owns one key (TMEM lane); the per-row
// statistics (lse, delta) are broadcast reads from a small SMEM table the producer warp fills.
//   warps 0..7 : two threads per key (64 of the 128 row columns each)
//   warp 8     : TMA producer (Q ring of 3 tiles, dO ring of 2) and the per-row table
//   warp 9     : TMEM allocation, MMA issue (one thread polls four queues: S, dP, dV, dK)
// TMEM columns: dV [0,128)  dK [128,256)  S^T / P^T [256,384)  dP^T / dS^T [384,512).
#include "attn_bwd.h"
#include "host_util.h"
#include "tc5.cuh"

namespace nsa {
namespace {
constexpr int kQStages = 3;
constexpr int kDoStages = 2;
constexpr int kTileBytes = 128 * 128 * 2;  // any 128 x 128 operand tile of 16-bit elements: two panels of [128][64]
constexpr int kPanelBytes = 128 * 128;

__device__ __forceinline__ void red_add_v4(float* dst, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(dst), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
}  // namespace

template <typename T>
__global__ void __launch_bounds__(320, 1)
dense_dkdv_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                     const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, DkdvParams p, int logG) {
  constexpr int D = 128;
  constexpr int KT = 128;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* k_sm = smem;
  uint8_t* v_sm = k_sm + kTileBytes;
  uint8_t* q_ring = v_sm + kTileBytes;
  uint8_t* do_ring = q_ring + kQStages * kTileBytes;
  float* nlse_sh = reinterpret_cast<float*>(do_ring + kDoStages * kTileBytes);  // [2][128]  -lse (base 2)
  float* dsc_sh = nlse_sh + 2 * 128;                                              // [2][128]  delta * sm_scale
  uint64_t* bars = reinterpret_cast<uint64_t*>(dsc_sh + 2 * 128);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;
  uint64_t* q_empty = q_full + kQStages;
  uint64_t* do_full = q_empty + kQStages;
  uint64_t* do_empty = do_full + kDoStages;
  uint64_t* meta_full = do_empty + kDoStages;  // [2]
  uint64_t* meta_empty = meta_full + 2;        // [2]
  uint64_t* s_full = meta_empty + 2;
  uint64_t* dp_full = s_full + 1;
  uint64_t* p_full = dp_full + 1;
  uint64_t* ds_full = p_full + 1;
  uint64_t* all_done = ds_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(all_done + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int TPT = 128 >> logG;  // tokens per row tile

  // the swizzled operand tiles need a 1024-byte aligned base
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) p.st.raise(kErrSmemLayout);
    return;
  }

  // ---- which key tile, which tokens ----
  const int b = blockIdx.z / p.Hkv;
  const int h = blockIdx.z % p.Hkv;
  const int qs = __ldg(p.cu_q + b);
  const int Lq = __ldg(p.cu_q + b + 1) - qs;
  const int ks0 = __ldg(p.cu_k + b), Lk = __ldg(p.cu_k + b + 1) - ks0;
  const int kpos = blockIdx.x * KT;  // key tiles vary fastest: CTAs that run together share a token chunk in L2
  if (kpos >= Lk) return;
  const int krow0 = ks0 + kpos;
  const int kvalid = min(KT, Lk - kpos);
  const int t_first = p.causal ? kpos * p.stride + p.window - 1 : 0;
  const int c_lo = blockIdx.y * p.chunk;
  const int tok_begin = max(c_lo, t_first);
  // sliding window: key j is seen by tokens up to j + left only
  const int tok_end = p.left >= 0 ? min(min(c_lo + p.chunk, Lq), kpos + kvalid + p.left) : min(c_lo + p.chunk, Lq);
  if (tok_end <= tok_begin) return;
  const int ntiles = (tok_end - tok_begin + TPT - 1) / TPT;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < kQStages; ++s) {
      mbar_init(q_full + s, 1);
      mbar_init(q_empty + s, 1);
    }
    for (int s = 0; s < kDoStages; ++s) {
      mbar_init(do_full + s, 1);
      mbar_init(do_empty + s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(meta_full + s, 1);
      mbar_init(meta_empty + s, 8);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_full, 8);
    mbar_init(ds_full, 8);
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
    // ===================== producer =====================
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * kTileBytes);
#pragma unroll
      for (int pn = 0; pn < 2; ++pn) {
        tma_load_3d(k_sm + pn * kPanelBytes, &tmK, kv_full, pn * 64, h, krow0);
        tma_load_3d(v_sm + pn * kPanelBytes, &tmV, kv_full, pn * 64, h, krow0);
      }
    }
    for (int i = 0; i < ntiles; ++i) {
      const int tok0 = tok_begin + i * TPT;  // in-sequence position of the tile's first token
      if (lane == 0) {
        const int s = i % kQStages;
        if (i >= kQStages) mbar_wait(q_empty + s, ((i / kQStages) - 1) & 1, p.st);
        mbar_expect_tx(q_full + s, kTileBytes);
#pragma unroll
        for (int pn = 0; pn < 2; ++pn)
          tma_load_3d(q_ring + s * kTileBytes + pn * kPanelBytes, &tmQ, q_full + s, pn * 64, h * p.G, qs + tok0);
      }
      {
        const int s = i & 1;
        if (i >= 2) mbar_wait(meta_empty + s, ((i >> 1) - 1) & 1, p.st);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = lane + 32 * j;
          const int tok = tok0 + (r >> logG);
          float2 ldv = make_float2(INFINITY, 0.f);
          if (tok < tok_end) ldv = __ldg(p.ld + (long long)(qs + tok) * p.Hq + h * p.G + (r & (p.G - 1)));
          nlse_sh[s * 128 + r] = -ldv.x;
          dsc_sh[s * 128 + r] = ldv.y * p.sm_scale;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(meta_full + s);
      }
      if (lane == 0) {
        const int s = i % kDoStages;
        if (i >= kDoStages) mbar_wait(do_empty + s, ((i / kDoStages) - 1) & 1, p.st);
        mbar_expect_tx(do_full + s, kTileBytes);
#pragma unroll
        for (int pn = 0; pn < 2; ++pn)
          tma_load_3d(do_ring + s * kTileBytes + pn * kPanelBytes, &tmDO, do_full + s, pn * 64, h * p.G, qs + tok0);
      }
      __syncwarp();
    }
  } else if (warp == 9) {
    // ===================== MMA issuer =====================
    // The whole warp runs the control flow (so that it stays warp-uniform and cheap); one elected lane issues.
    {
      const uint32_t idesc_s = umma_idesc<T>(128, 128, false, false);
      const uint32_t idesc_t = umma_idesc<T>(128, 128, false, true);
      const uint32_t k_addr = smem_u32(k_sm), v_addr = smem_u32(v_sm), q_base = smem_u32(q_ring), do_base = smem_u32(do_ring);
      auto issue_logits = [&](uint32_t a_addr, uint32_t b_addr, uint32_t d_tmem, uint64_t* bar) {
        if (elect_one()) {
          umma_block_ss<D / 16, kPanelBytes>(d_tmem, a_addr, b_addr, idesc_s);
          umma_commit(bar);
        }
        __syncwarp();
      };
      auto issue_grad = [&](uint32_t a_tmem, uint32_t b_addr, uint32_t d_tmem, bool first, uint64_t* bar) {
        if (elect_one()) {
          umma_block_ts<128 / 16, kPanelBytes>(d_tmem, a_tmem, b_addr, idesc_t, !first);
          umma_commit(bar);
        }
        __syncwarp();
      };
      mbar_wait(kv_full, 0, p.st);
      // Four queues share the tensor pipe.  S(i) may start once dV(i-1) has been issued (it overwrites P^T(i-1);
      // the pipe executes in issue order), dP(i) once dK(i-1) has been issued; dV(i) needs P^T(i), dK(i) needs dS^T(i).
      int ns = 0, np = 0, nv = 0, nk = 0;
      long long t0 = 0;
      int idle = 0;
      while (nk < ntiles) {
        bool progressed = false;
        if (nv < ns && nv < np && mbar_test(p_full, nv & 1)) {
          tc_fence_after_sync();
          issue_grad(tmem + 256, do_base + (nv % kDoStages) * kTileBytes, tmem, nv == 0, do_empty + (nv % kDoStages));
          ++nv;
          progressed = true;
        }
        if (ns < ntiles && ns == nv && mbar_test(q_full + (ns % kQStages), (ns / kQStages) & 1)) {
          tc_fence_after_sync();
          issue_logits(k_addr, q_base + (ns % kQStages) * kTileBytes, tmem + 256, s_full);
          ++ns;
          progressed = true;
        }
        if (nk < np && mbar_test(ds_full, nk & 1)) {
          tc_fence_after_sync();
          issue_grad(tmem + 384, q_base + (nk % kQStages) * kTileBytes, tmem + 128, nk == 0, q_empty + (nk % kQStages));
          ++nk;
          progressed = true;
        }
        if (np < ntiles && np == nk && mbar_test(do_full + (np % kDoStages), (np / kDoStages) & 1)) {
          tc_fence_after_sync();
          issue_logits(v_addr, do_base + (np % kDoStages) * kTileBytes, tmem + 384, dp_full);
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
    // ===================== softmax / dS threads: thread = (key, half of the row columns) =====================
    const int half = warp >> 2;
    const int key = (warp & 3) * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    // first in-sequence token position that sees this key
    const int thr = p.causal ? (kpos + key) * p.stride + p.window - 1 : 0;
    const bool key_ok = key < kvalid;
    for (int i = 0; i < ntiles; ++i) {
      const int ms = i & 1;
      const int tok0 = tok_begin + i * TPT;
      // visible columns of this thread: [clo, chi) in tile columns, shifted to the thread's own 64
      const int clo = max(0, thr - tok0) << logG;
      int chi = key_ok ? (min(TPT, tok_end - tok0) << logG) : 0;
      if (p.left >= 0) chi = min(chi, max(0, kpos + key + p.left - tok0 + 1) << logG);
      const int clo_rel = clo - half * 64;
      const unsigned span = chi > clo ? (unsigned)(chi - clo) : 0u;

      mbar_wait(meta_full + ms, (i >> 1) & 1, p.st);
      mbar_wait(s_full, i & 1, p.st);
      tc_fence_after_sync();
      float pf[64];
      {
        uint32_t su[2][32];
        tmem_ld32(lane_base + 256 + half * 64, su[0]);
        tmem_ld32(lane_base + 256 + half * 64 + 32, su[1]);
        tmem_ld_wait();
        const float4* nl4 = reinterpret_cast<const float4*>(nlse_sh + ms * 128 + half * 64);
        // tiles every key of the warp sees in full (all but those on the mask's edge) skip the mask instructions
        if (__all_sync(0xffffffffu, clo == 0 && chi == 128)) {
#pragma unroll
          for (int j4 = 0; j4 < 16; ++j4) {
            const float4 nl = nl4[j4];
            const int j = 4 * j4;
            const float2 sc2 = make_float2(p.scale2, p.scale2);
            const float2 x01 = ffma2(make_float2(__uint_as_float(su[j >> 5][(j + 0) & 31]), __uint_as_float(su[j >> 5][(j + 1) & 31])), sc2,
                                     make_float2(nl.x, nl.y));
            const float2 x23 = ffma2(make_float2(__uint_as_float(su[j >> 5][(j + 2) & 31]), __uint_as_float(su[j >> 5][(j + 3) & 31])), sc2,
                                     make_float2(nl.z, nl.w));
            pf[j + 0] = fast_exp2(x01.x);
            pf[j + 1] = fast_exp2(x01.y);
            pf[j + 2] = fast_exp2(x23.x);
            pf[j + 3] = fast_exp2(x23.y);
          }
        } else {
#pragma unroll
          for (int j4 = 0; j4 < 16; ++j4) {
            const float4 nl = nl4[j4];
            const int j = 4 * j4;
            pf[j + 0] = masked_exp2((unsigned)(j + 0 - clo_rel) < span, fmaf(__uint_as_float(su[j >> 5][(j + 0) & 31]), p.scale2, nl.x));
            pf[j + 1] = masked_exp2((unsigned)(j + 1 - clo_rel) < span, fmaf(__uint_as_float(su[j >> 5][(j + 1) & 31]), p.scale2, nl.y));
            pf[j + 2] = masked_exp2((unsigned)(j + 2 - clo_rel) < span, fmaf(__uint_as_float(su[j >> 5][(j + 2) & 31]), p.scale2, nl.z));
            pf[j + 3] = masked_exp2((unsigned)(j + 3 - clo_rel) < span, fmaf(__uint_as_float(su[j >> 5][(j + 3) & 31]), p.scale2, nl.w));
          }
        }
        uint32_t pk[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) pk[j] = DT<T>::pack(pf[2 * j], pf[2 * j + 1]);
        tmem_st32(lane_base + 256 + half * 64, pk);  // over this thread's own logits
        tmem_st_wait();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);

      mbar_wait(dp_full, i & 1, p.st);
      tc_fence_after_sync();
      {
        uint32_t du[2][32];
        tmem_ld32(lane_base + 384 + half * 64, du[0]);
        tmem_ld32(lane_base + 384 + half * 64 + 32, du[1]);
        tmem_ld_wait();
        const float4* dl4 = reinterpret_cast<const float4*>(dsc_sh + ms * 128 + half * 64);
        uint32_t pk[32];
#pragma unroll
        for (int j4 = 0; j4 < 16; ++j4) {
          const float4 dl = dl4[j4];
          const int j = 4 * j4;
          const float2 sm2 = make_float2(p.sm_scale, p.sm_scale);
          const float2 t01 = ffma2(make_float2(__uint_as_float(du[j >> 5][(j + 0) & 31]), __uint_as_float(du[j >> 5][(j + 1) & 31])), sm2,
                                   make_float2(-dl.x, -dl.y));
          const float2 t23 = ffma2(make_float2(__uint_as_float(du[j >> 5][(j + 2) & 31]), __uint_as_float(du[j >> 5][(j + 3) & 31])), sm2,
                                   make_float2(-dl.z, -dl.w));
          const float2 d01 = fmul2(make_float2(pf[j + 0], pf[j + 1]), t01);
          const float2 d23 = fmul2(make_float2(pf[j + 2], pf[j + 3]), t23);
          pk[2 * j4] = DT<T>::pack(d01.x, d01.y);
          pk[2 * j4 + 1] = DT<T>::pack(d23.x, d23.y);
        }
        tmem_st32(lane_base + 384 + half * 64, pk);
        tmem_st_wait();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(ds_full);
        mbar_arrive(meta_empty + ms);
      }
    }
    // ---- drain: thread (key, half) adds 64 of the 128 d columns of its key's dV and dK rows ----
    mbar_wait(all_done, 0, p.st);
    tc_fence_after_sync();
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      float* dst = (which == 0 ? p.dv32 : p.dk32) + ((size_t)(krow0 + key) * p.Hkv + h) * D + half * 64;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32(lane_base + which * 128 + half * 64 + c * 32, r);
        tmem_ld_wait();
        if (key_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            red_add_v4(dst + c * 32 + j, __uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                       __uint_as_float(r[j + 3]));
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, 512);
}

template <typename T>
int launch_dense_dkdv_tc(const void* q, const void* dout, const void* k, const void* v, const long long* strides, int Nq, int Nk,
                         int max_q, int max_k, int batch, DkdvParams p, cudaStream_t stream) {
  constexpr int D = 128;
  int logG = 0;
  while ((1 << logG) < p.G) ++logG;
  const int TPT = 128 >> logG;
  CUtensorMap tmQ, tmDO, tmK, tmV;
  int rc = make_tmap_3d(&tmQ, DT<T>::kTmapType, q, D, p.Hq, Nq, strides[1], strides[0], 64, p.G, TPT);
  if (rc) return rc;
  rc = make_tmap_3d(&tmDO, DT<T>::kTmapType, dout, D, p.Hq, Nq, strides[7], strides[6], 64, p.G, TPT);
  if (rc) return rc;
  rc = make_tmap_3d(&tmK, DT<T>::kTmapType, k, D, p.Hkv, Nk, strides[3], strides[2], 64, 1, 128);
  if (rc) return rc;
  rc = make_tmap_3d(&tmV, DT<T>::kTmapType, v, D, p.Hkv, Nk, strides[5], strides[4], 64, 1, 128);
  if (rc) return rc;
  const size_t smem = (size_t)(2 + kQStages + kDoStages) * kTileBytes + 4 * 128 * sizeof(float) + 24 * sizeof(uint64_t) + 16;
  auto kern = dense_dkdv_tc_kernel<T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_rc(e);
  dim3 grid((max_k + 127) / 128, (max_q + p.chunk - 1) / p.chunk, batch * p.Hkv);
  { LaunchScope ls_("dense_dkdv_tc", stream); kern<<<grid, 320, smem, stream>>>(tmQ, tmDO, tmK, tmV, p, logG); }
  return cuda_rc(cudaGetLastError());
}

template int launch_dense_dkdv_tc<__nv_bfloat16>(const void*, const void*, const void*, const void*, const long long*, int, int, int,
                                                 int, int, DkdvParams, cudaStream_t);
template int launch_dense_dkdv_tc<__half>(const void*, const void*, const void*, const void*, const long long*, int, int, int, int,
                                          int, DkdvParams, cudaStream_t);

}  // namespace nsa
