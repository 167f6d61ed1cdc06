// dK/dV pass on the 5th-generation tensor cores (head_dim 128).
//
// CTA = one tile of 64 keys (K and V tile resident in SMEM) x a stream of row tiles; a row tile is
// 128 rows = (128/G tokens) x (G query heads).  All four products have M = 128:
//     S    = Q  K^T          [128 rows x 64 keys]   A = Q  (K-major),  B = K tile (K-major)
//     dP   = dO V^T          [128 rows x 64 keys]   A = dO (K-major),  B = V tile (K-major)
//     dV^T = dO^T P          [128 d    x 64 keys]   A = dO (MN-major), B = P  [rows][keys] (MN-major)
//     dK^T = Q^T  dS         [128 d    x 64 keys]   A = Q  (MN-major), B = dS [rows][keys] (MN-major)
// so the token/head rows are the reduction dimension of the last two and the G heads of a KV group are
// summed inside the MMA.  S and dP are double-buffered in TMEM (tile i+1 is computed while the softmax
// threads work on tile i); dV^T and dK^T stay in TMEM for the whole CTA and are added to the fp32
// accumulators in global memory at the end.
//   warps 0..7 : two threads per row (32 key columns each): P = exp2(S*scale - lse), dS = P (dP - delta) scale,
//                written as 16-bit [rows][keys] tiles; at the end they drain dV / dK from TMEM
//   warp 8     : TMA producer (Q and dO rows of the tile, one box per token for gathered tokens)
//   warp 9     : TMEM allocation, MMA issue (one thread)
// TMEM columns: S0 [0,64) S1 [64,128) dP0 [128,192) dP1 [192,256) dV^T [256,320) dK^T [320,384).
#include "attn_bwd.h"
#include "attn_tile.cuh"
#include "host_util.h"
#include "tc5.cuh"

namespace nsa {

constexpr int kRowStages = 2;

template <typename T, bool SPARSE>
__global__ void __launch_bounds__(320, 1)
dkdv_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
               const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, DkdvParams p) {
  constexpr int D = 128;
  constexpr int KT = 64;                       // keys per CTA
  constexpr int KV_BYTES = KT * D * 2;         // 16 KB, 2 panels of [64 keys][64 d]
  constexpr int KV_PANEL = KT * 128;
  constexpr int ROW_BYTES = 128 * D * 2;       // Q or dO rows of one tile: 32 KB, 2 panels of [128 rows][64 d]
  constexpr int ROW_PANEL = 128 * 128;
  constexpr int PD_BYTES = 128 * KT * 2;       // P or dS tile [128 rows][64 keys]: 16 KB, one panel
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_sm = smem;
  uint8_t* v_sm = k_sm + KV_BYTES;
  uint8_t* ring = v_sm + KV_BYTES;                       // [stages][Q rows | dO rows]
  uint8_t* p_sm = ring + kRowStages * 2 * ROW_BYTES;
  uint8_t* ds_sm = p_sm + PD_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ds_sm + PD_BYTES);
  uint64_t* kv_full = bars;                 // 1
  uint64_t* row_full = bars + 1;            // [stages]
  uint64_t* row_empty = row_full + kRowStages;
  uint64_t* sdp_full = row_empty + kRowStages;   // [2]
  uint64_t* sdp_empty = sdp_full + 2;            // [2]
  uint64_t* pds_full = sdp_empty + 2;            // 1
  uint64_t* pds_empty = pds_full + 1;            // 1
  uint64_t* all_done = pds_empty + 1;            // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(all_done + 1);
  float2* ld_sh = reinterpret_cast<float2*>(tmem_slot + 2);              // [stages][128]
  int* tok_sh = reinterpret_cast<int*>(ld_sh + kRowStages * 128);         // [stages][128] in-sequence position or -1

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int logG = 0;
  while ((1 << logG) < p.G) ++logG;
  const int TPT = 128 >> logG;  // tokens per row tile

  // ---- which key tile and which tokens (same decoding as the mma.sync kernel) ----
  int h, qs, Lq, krow0, kpos, kvalid, tok_begin, tok_count;
  if (SPARSE) {
    const int item = blockIdx.x;
    const int total_x = p.Hkv * p.TB;
    if (item >= __ldg(p.item_base + total_x)) return;
    int lo = 0, hi = total_x;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (__ldg(p.item_base + mid) <= item) lo = mid; else hi = mid;
    }
    const int x = lo;
    h = x / p.TB;
    const int gb = x % p.TB;
    const int b = find_sequence(p.cu_blocks, p.B, gb);
    qs = __ldg(p.cu_q + b);
    Lq = __ldg(p.cu_q + b + 1) - qs;
    const int blk = gb - __ldg(p.cu_blocks + b);
    kpos = blk * p.block_size + blockIdx.y * KT;
    krow0 = qs + kpos;
    kvalid = min(KT, Lq - kpos);
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
    kpos = blockIdx.x * KT;  // key tiles vary fastest: CTAs that run together share a token chunk in L2
    if (kpos >= Lk) return;
    krow0 = ks0 + kpos;
    kvalid = min(KT, Lk - kpos);
    const int t_first = p.causal ? kpos * p.stride + p.window - 1 : 0;
    const int c_lo = blockIdx.y * p.chunk;
    tok_begin = max(c_lo, t_first);
    tok_count = min(c_lo + p.chunk, Lq) - tok_begin;
  }
  if (kvalid <= 0 || tok_count <= 0) return;
  const int ntiles = (tok_count + TPT - 1) / TPT;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < kRowStages; ++s) {
      mbar_init(row_full + s, 1);
      mbar_init(row_empty + s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(sdp_full + s, 1);
      mbar_init(sdp_empty + s, 8);
    }
    mbar_init(pds_full, 8);
    mbar_init(pds_empty, 1);
    mbar_init(all_done, 1);
    fence_barrier_init();
  }
  // rows that no TMA box writes (tokens missing from a tail tile) are multiplied by exact zeros later:
  // clear the ring once so that they cannot hold NaN bit patterns
  for (int i = threadIdx.x; i < kRowStages * 2 * ROW_BYTES / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(ring)[i] = make_uint4(0u, 0u, 0u, 0u);
  fence_proxy_async();
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
      mbar_expect_tx(kv_full, 2 * KV_BYTES);
#pragma unroll
      for (int pn = 0; pn < 2; ++pn) {
        tma_load_3d(k_sm + pn * KV_PANEL, &tmK, kv_full, pn * 64, h, krow0);
        tma_load_3d(v_sm + pn * KV_PANEL, &tmV, kv_full, pn * 64, h, krow0);
      }
    }
    for (int i = 0; i < ntiles; ++i) {
      const int s = i % kRowStages;
      if (i >= kRowStages) mbar_wait(row_empty + s, ((i / kRowStages) - 1) & 1, p.st);
      // token of slot `lane` (TPT <= 32 slots)
      int n = -1;
      const int ti = i * TPT + lane;
      if (lane < TPT && ti < tok_count) n = SPARSE ? __ldg(p.list + tok_begin + ti) : qs + tok_begin + ti;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = lane + 32 * j;
        const int nn = __shfl_sync(0xffffffffu, n, r >> logG);
        float2 ldv = make_float2(INFINITY, 0.f);
        if (nn >= 0) ldv = __ldg(p.ld + (long long)nn * p.Hq + h * p.G + (r & (p.G - 1)));
        ld_sh[s * 128 + r] = ldv;
        tok_sh[s * 128 + r] = nn >= 0 ? nn - qs : -1;
      }
      __syncwarp();
      uint8_t* qd = ring + s * 2 * ROW_BYTES;
      if (SPARSE) {
        const unsigned vm = __ballot_sync(0xffffffffu, n >= 0);
        if (lane == 0) mbar_expect_tx(row_full + s, __popc(vm) * 2 * p.G * D * 2);
        __syncwarp();
        if (n >= 0) {
          const int roff = (lane << logG) * 128;  // this token's first row inside the tile
#pragma unroll
          for (int pn = 0; pn < 2; ++pn) {
            tma_load_3d(qd + pn * ROW_PANEL + roff, &tmQ, row_full + s, pn * 64, h * p.G, n);
            tma_load_3d(qd + ROW_BYTES + pn * ROW_PANEL + roff, &tmDO, row_full + s, pn * 64, h * p.G, n);
          }
        }
      } else if (lane == 0) {
        mbar_expect_tx(row_full + s, 2 * ROW_BYTES);
#pragma unroll
        for (int pn = 0; pn < 2; ++pn) {
          tma_load_3d(qd + pn * ROW_PANEL, &tmQ, row_full + s, pn * 64, h * p.G, qs + tok_begin + i * TPT);
          tma_load_3d(qd + ROW_BYTES + pn * ROW_PANEL, &tmDO, row_full + s, pn * 64, h * p.G, qs + tok_begin + i * TPT);
        }
      }
    }
  } else if (warp == 9) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc<T>(128, KT, false, false);
      const uint32_t idesc_t = umma_idesc<T>(128, KT, true, true);
      const uint32_t k_addr = smem_u32(k_sm), v_addr = smem_u32(v_sm), p_addr = smem_u32(p_sm), ds_addr = smem_u32(ds_sm);
      auto issue_sdp = [&](int i) {
        const uint32_t q_addr = smem_u32(ring + (i % kRowStages) * 2 * ROW_BYTES);
        const uint32_t do_addr = q_addr + ROW_BYTES;
        const uint32_t ts = tmem + (uint32_t)((i & 1) * KT), tdp = tmem + 128u + (uint32_t)((i & 1) * KT);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t a_off = (kk >> 2) * ROW_PANEL + (kk & 3) * 32, b_off = (kk >> 2) * KV_PANEL + (kk & 3) * 32;
          umma_ss(ts, umma_desc_kmajor(q_addr + a_off), umma_desc_kmajor(k_addr + b_off), idesc_s, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t a_off = (kk >> 2) * ROW_PANEL + (kk & 3) * 32, b_off = (kk >> 2) * KV_PANEL + (kk & 3) * 32;
          umma_ss(tdp, umma_desc_kmajor(do_addr + a_off), umma_desc_kmajor(v_addr + b_off), idesc_s, kk > 0);
        }
        umma_commit(sdp_full + (i & 1));
      };
      auto issue_dvdk = [&](int i) {
        const uint32_t q_addr = smem_u32(ring + (i % kRowStages) * 2 * ROW_BYTES);
        const uint32_t do_addr = q_addr + ROW_BYTES;
#pragma unroll
        for (int kk = 0; kk < 128 / 16; ++kk)   // reduction over the 128 rows, 16 at a time
          umma_ss(tmem + 256, umma_desc_mnmajor(do_addr + kk * 2048, ROW_PANEL), umma_desc_mnmajor(p_addr + kk * 2048, PD_BYTES),
                  idesc_t, i > 0 || kk > 0);
#pragma unroll
        for (int kk = 0; kk < 128 / 16; ++kk)
          umma_ss(tmem + 320, umma_desc_mnmajor(q_addr + kk * 2048, ROW_PANEL), umma_desc_mnmajor(ds_addr + kk * 2048, PD_BYTES),
                  idesc_t, i > 0 || kk > 0);
        umma_commit(row_empty + (i % kRowStages));
        umma_commit(pds_empty);
      };
      mbar_wait(kv_full, 0, p.st);
      // Two independent streams of work share the tensor pipe: S/dP of tile ns (needs the tile's rows and a free TMEM
      // buffer) and dV/dK of tile nd (needs P and dS of that tile).  Whichever is ready is issued; neither blocks the other.
      int ns = 0, nd = 0;
      long long t0 = 0;
      int idle = 0;
      while (nd < ntiles) {
        bool progressed = false;
        if (ns < ntiles && ns - nd < 2 && mbar_test(row_full + (ns % kRowStages), (ns / kRowStages) & 1) &&
            (ns < 2 || mbar_test(sdp_empty + (ns & 1), ((ns >> 1) - 1) & 1))) {
          tc_fence_after_sync();
          issue_sdp(ns);
          ++ns;
          progressed = true;
        }
        if (nd < ns && mbar_test(pds_full, nd & 1)) {
          tc_fence_after_sync();
          issue_dvdk(nd);
          ++nd;
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
      umma_commit(all_done);
    }
  } else {
    // ===================== softmax / dS threads: two threads per row (32 of the 64 key columns each) =====================
    const int half = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    for (int i = 0; i < ntiles; ++i) {
      const int bsel = i & 1, s = i % kRowStages;
      mbar_wait(row_full + s, (i / kRowStages) & 1, p.st);  // acquire the producer's per-row metadata of this stage
      mbar_wait(sdp_full + bsel, (i >> 1) & 1, p.st);
      tc_fence_after_sync();
      uint32_t su[32], du[32];
      tmem_ld32(lane_base + bsel * KT + half * 32, su);
      tmem_ld32(lane_base + 128 + bsel * KT + half * 32, du);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(sdp_empty + bsel);

      const int tpos = tok_sh[s * 128 + row];
      const float2 ldv = ld_sh[s * 128 + row];
      int lim = 0;
      if (tpos >= 0) {
        if (!p.causal) lim = kvalid;
        else if (tpos >= p.window - 1) lim = max(0, min(kvalid, (tpos - (p.window - 1)) / p.stride - kpos + 1));
      }
      lim -= half * 32;  // relative to this thread's first column
      const float nlse = -ldv.x, delta = ldv.y;
      uint32_t pw[16], dw[16];
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const float p0 = masked_exp2(j < lim, fmaf(__uint_as_float(su[j]), p.scale2, nlse));
        const float p1 = masked_exp2(j + 1 < lim, fmaf(__uint_as_float(su[j + 1]), p.scale2, nlse));
        const float d0 = p0 * (__uint_as_float(du[j]) - delta) * p.sm_scale;
        const float d1 = p1 * (__uint_as_float(du[j + 1]) - delta) * p.sm_scale;
        pw[j >> 1] = DT<T>::pack(p0, p1);
        dw[j >> 1] = DT<T>::pack(d0, d1);
      }
      if (i > 0) mbar_wait(pds_empty, (i - 1) & 1, p.st);  // the previous tile's dV/dK products have read P and dS
      const uint32_t prow = smem_u32(p_sm) + row * 128, dsrow = smem_u32(ds_sm) + row * 128;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        const uint32_t sw = (((half * 4 + c4) ^ (row & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(prow + sw), "r"(pw[c4 * 4]), "r"(pw[c4 * 4 + 1]),
                     "r"(pw[c4 * 4 + 2]), "r"(pw[c4 * 4 + 3]) : "memory");
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(dsrow + sw), "r"(dw[c4 * 4]), "r"(dw[c4 * 4 + 1]),
                     "r"(dw[c4 * 4 + 2]), "r"(dw[c4 * 4 + 3]) : "memory");
      }
      fence_proxy_async();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
    }
    // ---- drain: thread (d, half) holds column d of dV and dK for 32 of the 64 keys ----
    mbar_wait(all_done, 0, p.st);
    tc_fence_after_sync();
    const int d = row;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      float* dst = (which == 0 ? p.dv32 : p.dk32) + ((size_t)krow0 * p.Hkv + h) * D + d;
      uint32_t r[32];
      tmem_ld32(lane_base + 256 + which * 64 + half * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int key = half * 32 + j;
        if (key < kvalid) atomicAdd(dst + (size_t)key * p.Hkv * D, __uint_as_float(r[j]));
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, 512);
}

template <typename T, bool SPARSE>
int launch_dkdv_tc(const void* q, const void* dout, const void* k, const void* v, const long long* strides, int Nq, int Nk,
                   dim3 grid, DkdvParams p, cudaStream_t stream) {
  constexpr int D = 128;
  const int TPT = 128 / p.G;
  CUtensorMap tmQ, tmDO, tmK, tmV;
  const int tok_box = SPARSE ? 1 : TPT;
  int rc = make_tmap_3d(&tmQ, DT<T>::kTmapType, q, D, p.Hq, Nq, strides[1], strides[0], 64, p.G, tok_box);
  if (rc) return rc;
  rc = make_tmap_3d(&tmDO, DT<T>::kTmapType, dout, D, p.Hq, Nq, strides[7], strides[6], 64, p.G, tok_box);
  if (rc) return rc;
  rc = make_tmap_3d(&tmK, DT<T>::kTmapType, k, D, p.Hkv, Nk, strides[3], strides[2], 64, 1, 64);
  if (rc) return rc;
  rc = make_tmap_3d(&tmV, DT<T>::kTmapType, v, D, p.Hkv, Nk, strides[5], strides[4], 64, 1, 64);
  if (rc) return rc;
  const size_t smem = 1024 + 2 * (64 * D * 2) + kRowStages * 2 * (128 * D * 2) + 2 * (128 * 64 * 2) + 16 * sizeof(uint64_t) + 16 +
                      kRowStages * 128 * (sizeof(float2) + sizeof(int));
  auto kern = dkdv_tc_kernel<T, SPARSE>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_rc(e);
  { LaunchScope ls_(SPARSE ? "sparse_dkdv_tc" : "dense_dkdv_tc", stream); kern<<<grid, 320, smem, stream>>>(tmQ, tmDO, tmK, tmV, p); }
  return cuda_rc(cudaGetLastError());
}

template int launch_dkdv_tc<__nv_bfloat16, false>(const void*, const void*, const void*, const void*, const long long*, int, int,
                                                  dim3, DkdvParams, cudaStream_t);
template int launch_dkdv_tc<__nv_bfloat16, true>(const void*, const void*, const void*, const void*, const long long*, int, int,
                                                 dim3, DkdvParams, cudaStream_t);
template int launch_dkdv_tc<__half, false>(const void*, const void*, const void*, const void*, const long long*, int, int, dim3,
                                           DkdvParams, cudaStream_t);
template int launch_dkdv_tc<__half, true>(const void*, const void*, const void*, const void*, const long long*, int, int, dim3,
                                          DkdvParams, cudaStream_t);

}  // namespace nsa
