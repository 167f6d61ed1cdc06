// Forward of dense varlen GQA attention with a strided-causal mask:
//     query at in-sequence position t sees key i  iff  t >= i*stride + (window - 1).
// window = 32, stride = 16 gives attention over compressed keys (compressed_attention);
// window = stride = 1 gives ordinary causal attention; causal = 0 gives full attention.
//
// A CTA owns 128 rows = (128/G query tokens) x (G query heads of one KV head); K/V tiles of 64
// keys stream through a TMA ring shared by the 8 warps, each warp keeps its 16 rows' Q
// fragments, running max/sum and the fp32 output accumulator in registers.
#include <cstdlib>

#include "attn_tile.cuh"
#include "dispatch.h"
#include "host_util.h"
#include "nsa_b200.h"

namespace nsa {

struct DenseFwdParams {
  const void* q;
  void* o;
  float* lse;  // [Nq, Hq]
  const int* cu_q;
  const int* cu_k;
  long long q_sn, q_sh, o_sn, o_sh;
  int B, Hq, Hkv, G, logG;
  int window, stride, causal;
  float scale2;
  Status st;
};

// number of keys visible to in-sequence query position t
__device__ __forceinline__ int visible_keys(int t, int Lk, int window, int stride, int causal) {
  if (!causal) return Lk;
  if (t < window - 1) return 0;
  return min(Lk, (t - window + 1) / stride + 1);
}

template <typename T, int D, int WARPS, int STAGES>
__global__ void __launch_bounds__(WARPS * 32, 1)
dense_fwd_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, DenseFwdParams p) {
  constexpr int TILE_BYTES = kKeyTile * D * 2;
  constexpr int PANELS = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * 2 * TILE_BYTES);
  uint64_t* empty = full + STAGES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int b = blockIdx.y, h = blockIdx.z;
  const int qs = __ldg(p.cu_q + b), Lq = __ldg(p.cu_q + b + 1) - qs;
  const int ksq = __ldg(p.cu_k + b), Lk = __ldg(p.cu_k + b + 1) - ksq;
  const int QPW = 16 >> p.logG;  // queries per warp
  const int QT = WARPS * QPW;    // queries per CTA
  const int qt = gridDim.x - 1 - blockIdx.x;  // long rows first
  const int q0 = qt * QT;
  if (q0 >= Lq) return;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, WARPS);
    }
    fence_barrier_init();
  }
  __syncthreads();

  const int t_hi = min(q0 + QT, Lq) - 1;
  const int ntiles = (visible_keys(t_hi, Lk, p.window, p.stride, p.causal) + kKeyTile - 1) / kKeyTile;
  const int tw_hi = min(q0 + (warp + 1) * QPW, Lq) - 1;  // last query of this warp (may be < its first one)
  const int my_tiles =
      (tw_hi >= q0 + warp * QPW) ? (visible_keys(tw_hi, Lk, p.window, p.stride, p.causal) + kKeyTile - 1) / kKeyTile : 0;

  auto issue = [&](int tile) {
    const int s = tile % STAGES;
    uint8_t* kb = smem + s * 2 * TILE_BYTES;
    mbar_expect_tx(full + s, 2 * TILE_BYTES);
#pragma unroll
    for (int pn = 0; pn < PANELS; ++pn) {
      tma_load_3d(kb + pn * (kKeyTile * 128), &tmK, full + s, pn * 64, h, ksq + tile * kKeyTile);
      tma_load_3d(kb + TILE_BYTES + pn * (kKeyTile * 128), &tmV, full + s, pn * 64, h, ksq + tile * kKeyTile);
    }
  };
  if (threadIdx.x == 0)
    for (int i = 0; i < STAGES - 1 && i < ntiles; ++i) issue(i);

  // rows of this warp: r -> query q0 + warp*QPW + (r >> logG), head h*G + (r & (G-1))
  const int r_lo = lane >> 2;
  int tq[2];      // in-sequence position of the two fragment rows of this lane
  int nvis[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    tq[r] = q0 + warp * QPW + ((r_lo + 8 * r) >> p.logG);
    nvis[r] = tq[r] < Lq ? visible_keys(tq[r], Lk, p.window, p.stride, p.causal) : 0;
  }
  const T* qbase = static_cast<const T*>(p.q) + (long long)(qs + q0 + warp * QPW) * p.q_sn + (long long)h * p.G * p.q_sh;
  uint32_t qf[D / 16][4];
  load_a_frags_global<T, D / 16>(qf, [&](int r) -> const T* {
    const int qi = r >> p.logG;
    return (q0 + warp * QPW + qi < Lq) ? qbase + qi * p.q_sn + (r & (p.G - 1)) * p.q_sh : nullptr;
  });

  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

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
      const uint32_t kb = smem_u32(smem + s * 2 * TILE_BYTES);
      float sc[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
      mma_nk<T, 8, D / 16, kKeyTile>(sc, qf, kb, 0, 0);
      const int lim[2] = {nvis[0] - i * kKeyTile, nvis[1] - i * kKeyTile};
      online_softmax_step<D / 8>(sc, lim, p.scale2, m, l, o);
      uint32_t pf[4][4];
      acc_to_a_frags<T, 4>(pf, sc);
      mma_kn<T, D / 8, 4, kKeyTile>(o, pf, kb + TILE_BYTES, 0, 0);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty + s);
  }

  // ---- epilogue ----
  float rs[2], lse2[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    rs[r] = l[r] > 0.f ? 1.f / l[r] : 0.f;
    lse2[r] = l[r] > 0.f ? m[r] + log2f(l[r]) : -INFINITY;
  }
  if ((lane & 3) == 0) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = r_lo + 8 * r;
      if (tq[r] < Lq && row < 16 && (row & (p.G - 1)) < p.G)
        p.lse[(long long)(qs + tq[r]) * p.Hq + h * p.G + (row & (p.G - 1))] = lse2[r];
    }
  }
  // every warp is past its last read of the ring before the staging area (stage 0.. region) is reused
  __syncthreads();
  T* stage = reinterpret_cast<T*>(smem + warp * (16 * (D + 8) * 2));
  T* obase = static_cast<T*>(p.o) + (long long)(qs + q0 + warp * QPW) * p.o_sn + (long long)h * p.G * p.o_sh;
  store_rows_staged<T, D>(o, rs, stage, [&](int r) -> T* {
    const int qi = r >> p.logG;
    return (q0 + warp * QPW + qi < Lq) ? obase + qi * p.o_sn + (r & (p.G - 1)) * p.o_sh : nullptr;
  });
}

template <typename T, int D>
static int launch_dense_fwd(const void* k, const void* v, long long k_sn, long long k_sh, long long v_sn, long long v_sh,
                            int Nk, int max_seqlen_q, DenseFwdParams p, cudaStream_t stream) {
  constexpr int WARPS = 8;
  constexpr int STAGES = (D == 128) ? 4 : 6;
  constexpr int TILE_BYTES = kKeyTile * D * 2;
  CUtensorMap tmK, tmV;
  int rc = make_tmap_3d(&tmK, DT<T>::kTmapType, k, D, p.Hkv, Nk, k_sh, k_sn, 64, 1, kKeyTile);
  if (rc) return rc;
  rc = make_tmap_3d(&tmV, DT<T>::kTmapType, v, D, p.Hkv, Nk, v_sh, v_sn, 64, 1, kKeyTile);
  if (rc) return rc;
  const size_t smem = 1024 + STAGES * 2 * TILE_BYTES + 2 * STAGES * sizeof(uint64_t);
  auto kern = dense_fwd_kernel<T, D, WARPS, STAGES>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_rc(e);
  const int QT = WARPS * (16 / p.G);
  dim3 grid((max_seqlen_q + QT - 1) / QT, p.B, p.Hkv);
  { LaunchScope ls_("dense_fwd", stream); kern<<<grid, WARPS * 32, smem, stream>>>(tmK, tmV, p); }
  return cuda_rc(cudaGetLastError());
}

// tcgen05 implementation (dense_fwd_tc.cu)
int varlen_attn_fwd_tc(const void* q, const void* k, const void* v, const int* cu_q, const int* cu_k, void* o, float* lse,
                       int total_q, int total_k, int batch, int max_seqlen_q, int Hq, int Hkv, int head_dim, int causal,
                       int window, int stride, int left, const long long* strides, float sm_scale, int dtype, cudaStream_t stream);

// The mma.sync kernel of this file stays selectable (environment variable NSA_B200_LEGACY_MMA=1) for A/B measurements.
static bool use_legacy_mma() {
  static const bool v = [] { const char* e = getenv("NSA_B200_LEGACY_MMA"); return e && e[0] == '1'; }();
  return v;
}

}  // namespace nsa

// left >= 0 adds the lower bound key >= t - left (sliding window); only with the plain causal mask and on the tcgen05 kernel
static int varlen_attn_fwd_common(const void* q, const void* k, const void* v, const int* cu_seqlens_q,
                                  const int* cu_seqlens_k, void* o, float* lse, int total_q, int total_k, int batch,
                                  int max_seqlen_q, int num_q_heads, int num_kv_heads, int head_dim, int causal,
                                  int window, int stride, int left, const long long* strides, float sm_scale, int dtype,
                                  void* stream) {
  using namespace nsa;
  if (left >= 0 && (!causal || window != 1 || stride != 1 || use_legacy_mma())) return kUnsupported;
  if (!q || !cu_seqlens_q || !cu_seqlens_k || !o || !lse || !strides) return kInvalid;
  if (total_q <= 0 || batch <= 0 || max_seqlen_q <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads) return kInvalid;
  if (window < 1 || stride < 1) return kInvalid;
  const int G = num_q_heads / num_kv_heads;
  if (G > 16 || (G & (G - 1))) return kUnsupported;
  if (total_k <= 0) {  // no key anywhere: outputs are zero, lse = -inf (caller pre-fills); nothing to launch
    return kOk;
  }
  if (!k || !v) return kInvalid;
  DenseFwdParams p;
  p.q = q; p.o = o; p.lse = lse; p.cu_q = cu_seqlens_q; p.cu_k = cu_seqlens_k;
  p.q_sn = strides[0]; p.q_sh = strides[1]; p.o_sn = strides[6]; p.o_sh = strides[7];
  p.B = batch; p.Hq = num_q_heads; p.Hkv = num_kv_heads; p.G = G;
  p.logG = 0;
  while ((1 << p.logG) < G) ++p.logG;
  p.window = window; p.stride = stride; p.causal = causal;
  p.scale2 = sm_scale * kLog2e;
  p.st.word = status_word();
  if ((p.q_sn | p.q_sh | p.o_sn | p.o_sh) % 8 || !aligned16(q) || !aligned16(o)) return kInvalid;
  if (!use_legacy_mma())
    return varlen_attn_fwd_tc(q, k, v, cu_seqlens_q, cu_seqlens_k, o, lse, total_q, total_k, batch, max_seqlen_q, num_q_heads,
                              num_kv_heads, head_dim, causal, window, stride, left, strides, sm_scale, dtype,
                              static_cast<cudaStream_t>(stream));
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_dense_fwd, k, v, strides[2], strides[3], strides[4], strides[5],
                          total_k, max_seqlen_q, p, static_cast<cudaStream_t>(stream));
}

extern "C" int nsa_varlen_attn_fwd(const void* q, const void* k, const void* v, const int* cu_seqlens_q,
                                   const int* cu_seqlens_k, void* o, float* lse, int total_q, int total_k, int batch,
                                   int max_seqlen_q, int num_q_heads, int num_kv_heads, int head_dim, int causal,
                                   int window, int stride, const long long* strides, float sm_scale, int dtype,
                                   void* stream) {
  return varlen_attn_fwd_common(q, k, v, cu_seqlens_q, cu_seqlens_k, o, lse, total_q, total_k, batch, max_seqlen_q, num_q_heads,
                                num_kv_heads, head_dim, causal, window, stride, -1, strides, sm_scale, dtype, stream);
}

extern "C" int nsa_window_attn_fwd(const void* q, const void* k, const void* v, const int* cu_seqlens, void* o, float* lse,
                                   int total_len, int batch, int max_seqlen, int num_q_heads, int num_kv_heads, int head_dim,
                                   int window_left, const long long* strides, float sm_scale, int dtype, void* stream) {
  if (window_left < 0) return nsa::kInvalid;
  return varlen_attn_fwd_common(q, k, v, cu_seqlens, cu_seqlens, o, lse, total_len, total_len, batch, max_seqlen, num_q_heads,
                                num_kv_heads, head_dim, 1, 1, 1, window_left, strides, sm_scale, dtype, stream);
}
