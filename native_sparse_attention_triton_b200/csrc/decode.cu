// Single-token (decode) attention against dense KV caches [batch, cache_len, kv_heads, d].
//
//  * flash decode            : every cache row below seqlens[b]
//  * top-k sparse decode     : the rows of the selected blocks below seqlens[b]
//  * compressed decode       : every compressed row below compress_seqlens[b], plus block scores
//                              and top-k block selection for the current token
//
// All three are bound by HBM: the cache rows are read once, through TMA, into per-warp
// shared-memory tiles; the G query heads of a KV head form the rows of the mma tile so the rows
// are shared by the whole group.  Long rows are split across warps/CTAs (split-KV); partial
// (max, sum, output) triples go through a caller-provided scratch buffer and a combine kernel.
#include "attn_tile.cuh"
#include "dispatch.h"
#include "host_util.h"
#include "nsa_b200.h"
#include "topk_select.cuh"

#include <mutex>

namespace nsa {

constexpr int kMaxTilesPerDecodeQuery = 64;
constexpr int kMaxDecodeSplits = 64;  // the combine kernel handles at most 64 partial results per row

struct DecodeParams {
  const void* q;
  void* o;
  const int* seqlens;
  const int* topk_idx;  // nullptr -> dense range
  float* part_o;        // [B*Hkv*S][16][D]
  float* part_ml;       // [B*Hkv*S][16][2]
  long long q_sb, q_sh, o_sb, o_sh;
  long long t_sh, t_sb, t_sk;
  int B, Hq, Hkv, G, T, block_size;
  int S, tiles_per_split;
  float scale2;
  Status st;
};

template <typename T, int D, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1)
decode_attn_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, DecodeParams p) {
  constexpr int TILE_BYTES = kKeyTile * D * 2;
  constexpr int PANELS = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* kbuf = smem + warp * 2 * TILE_BYTES;
  uint8_t* vbuf = kbuf + TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + WARPS * 2 * TILE_BYTES);
  uint64_t* barK = bars + 2 * warp;
  uint64_t* barV = barK + 1;
  int* tiles = reinterpret_cast<int*>(bars + 2 * WARPS) + warp * kMaxTilesPerDecodeQuery;

  const int task = blockIdx.x * WARPS + warp;
  if (task >= p.B * p.Hkv * p.S) return;
  const int split = task % p.S;
  const int h = (task / p.S) % p.Hkv;
  const int b = task / (p.S * p.Hkv);
  if (lane == 0) {
    mbar_init(barK, 1);
    mbar_init(barV, 1);
    fence_barrier_init();
  }
  __syncwarp();

  const int len = __ldg(p.seqlens + b);
  int t_begin, t_end;  // tile range of this split
  if (p.topk_idx) {
    const int BS = p.block_size, nsub = BS / kKeyTile;
    const int bq = len > 0 ? (len - 1) / BS : -1;
    int ntiles = 0;
    const int* tptr = p.topk_idx + h * p.t_sh + (long long)b * p.t_sb;
    for (int base = 0; base < p.T; base += 32) {
      const int j = base + lane;
      const int idx = (j < p.T) ? __ldg(tptr + j * p.t_sk) : -1;
      const bool valid = idx >= 0 && idx <= bq;
      const int cnt = valid ? min(nsub, (len - 1 - idx * BS) / kKeyTile + 1) : 0;
      int incl = cnt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      const int excl = incl - cnt;
      for (int s = 0; s < cnt; ++s) {
        const int pos = ntiles + excl + s;
        if (pos < kMaxTilesPerDecodeQuery) tiles[pos] = idx * BS + s * kKeyTile;
      }
      ntiles += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (ntiles > kMaxTilesPerDecodeQuery) {
      p.st.raise(kErrBadIndex);
      ntiles = kMaxTilesPerDecodeQuery;
    }
    __syncwarp();
    t_begin = min(ntiles, split * p.tiles_per_split);
    t_end = min(ntiles, t_begin + p.tiles_per_split);
  } else {
    const int ntiles = (len + kKeyTile - 1) / kKeyTile;
    t_begin = min(ntiles, split * p.tiles_per_split);
    t_end = min(ntiles, t_begin + p.tiles_per_split);
  }

  auto issue = [&](bool is_v, int kpos) {
    uint8_t* buf = is_v ? vbuf : kbuf;
    uint64_t* bar = is_v ? barV : barK;
    const CUtensorMap* tm = is_v ? &tmV : &tmK;
    mbar_expect_tx(bar, TILE_BYTES);
#pragma unroll
    for (int pn = 0; pn < PANELS; ++pn) tma_load_4d(buf + pn * (kKeyTile * 128), tm, bar, pn * 64, h, kpos, b);
  };
  const bool sparse = p.topk_idx != nullptr;
  auto tile_at = [&](int i, int& kpos, int& limv) {
    kpos = sparse ? tiles[t_begin + i] : (t_begin + i) * kKeyTile;
    limv = min(kKeyTile, len - kpos);
  };

  const T* qbase = static_cast<const T*>(p.q) + (long long)b * p.q_sb + (long long)h * p.G * p.q_sh;
  uint32_t qf[D / 16][4];
  load_a_frags_global<T, D / 16>(qf, [&](int r) -> const T* { return r < p.G ? qbase + r * p.q_sh : nullptr; });
  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  uint32_t phase = 0;
  warp_attend_tiles<T, D>(qf, o, m, l, t_end - t_begin, smem_u32(kbuf), smem_u32(vbuf), barK, barV, phase, p.scale2, p.st,
                          tile_at, issue);

  if (p.S == 1) {
    float rs[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) rs[r] = l[r] > 0.f ? 1.f / l[r] : 0.f;
    T* obase = static_cast<T*>(p.o) + (long long)b * p.o_sb + (long long)h * p.G * p.o_sh;
    store_rows_staged<T, D>(o, rs, reinterpret_cast<T*>(kbuf), [&](int r) -> T* { return r < p.G ? obase + r * p.o_sh : nullptr; });
  } else {
    float* po = p.part_o + (size_t)task * 16 * D;
    float* pml = p.part_ml + (size_t)task * 16 * 2;
    const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      *reinterpret_cast<float2*>(po + r0 * D + j * 8 + c0) = make_float2(o[j][0], o[j][1]);
      *reinterpret_cast<float2*>(po + (r0 + 8) * D + j * 8 + c0) = make_float2(o[j][2], o[j][3]);
    }
    if ((lane & 3) == 0) {
      *reinterpret_cast<float2*>(pml + r0 * 2) = make_float2(m[0], l[0]);
      *reinterpret_cast<float2*>(pml + (r0 + 8) * 2) = make_float2(m[1], l[1]);
    }
  }
}

// out[b, h*G + g, :] = sum_s o_s * 2^(m_s - m*) / sum_s l_s * 2^(m_s - m*)
// One CTA per (sequence, KV head, query head of the group), one thread per output column; the split weights are
// computed once by the first warp and shared.
template <typename T>
__global__ void decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, void* o,
                                      long long o_sb, long long o_sh, int Hkv, int G, int S, int D) {
  __shared__ float w_sh[64];
  __shared__ float inv_den;
  const int g = blockIdx.x % G;
  const int bh = blockIdx.x / G, b = bh / Hkv, h = bh % Hkv;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    if (lane < S) { const float* ml = part_ml + ((size_t)(bh * S + lane) * 16 + g) * 2; m0 = ml[0]; l0 = ml[1]; }
    if (lane + 32 < S) { const float* ml = part_ml + ((size_t)(bh * S + lane + 32) * 16 + g) * 2; m1 = ml[0]; l1 = ml[1]; }
    float mstar = fmaxf(m0, m1);
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) mstar = fmaxf(mstar, __shfl_xor_sync(0xffffffffu, mstar, off));
    const float w0 = (m0 == -INFINITY) ? 0.f : fast_exp2(m0 - mstar), w1 = (m1 == -INFINITY) ? 0.f : fast_exp2(m1 - mstar);
    float den = l0 * w0 + l1 * w1;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) den += __shfl_xor_sync(0xffffffffu, den, off);
    w_sh[lane] = w0;
    w_sh[lane + 32] = w1;
    if (lane == 0) inv_den = den > 0.f ? 1.f / den : 0.f;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float num = 0.f;
    for (int s = 0; s < S; ++s) num += part_o[((size_t)(bh * S + s) * 16 + g) * D + c] * w_sh[s];
    static_cast<T*>(o)[(long long)b * o_sb + (long long)(h * G + g) * o_sh + c] = DT<T>::from_float(num * inv_den);
  }
}

template <typename T, int D>
static int launch_decode(const void* k, const void* v, const long long* kv_strides, int cache_len, DecodeParams p,
                         cudaStream_t stream) {
  constexpr int WARPS = (D == 128) ? 6 : 8;
  constexpr int TILE_BYTES = kKeyTile * D * 2;
  CUtensorMap tmK, tmV;
  int rc = make_tmap_4d(&tmK, DT<T>::kTmapType, k, D, p.Hkv, cache_len, p.B, kv_strides[2], kv_strides[1], kv_strides[0], 64,
                        kKeyTile);
  if (rc) return rc;
  rc = make_tmap_4d(&tmV, DT<T>::kTmapType, v, D, p.Hkv, cache_len, p.B, kv_strides[5], kv_strides[4], kv_strides[3], 64,
                    kKeyTile);
  if (rc) return rc;
  const size_t smem = 1024 + WARPS * 2 * TILE_BYTES + WARPS * 2 * sizeof(uint64_t) + WARPS * kMaxTilesPerDecodeQuery * sizeof(int);
  auto kern = decode_attn_kernel<T, D, WARPS>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_rc(e);
  const int tasks = p.B * p.Hkv * p.S;
  { LaunchScope ls_("decode_attn", stream); kern<<<(tasks + WARPS - 1) / WARPS, WARPS * 32, smem, stream>>>(tmK, tmV, p); }
  if (p.S > 1)
    { LaunchScope ls_("decode_combine", stream); decode_combine_kernel<T><<<p.B * p.Hkv * p.G, 128, 0, stream>>>(p.part_o, p.part_ml, p.o, p.o_sb, p.o_sh, p.Hkv, p.G, p.S, D); }
  return cuda_rc(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------------
// compressed decode: one CTA of 4 warps per (sequence, KV head); output, block scores, selection
// ------------------------------------------------------------------------------------------------
struct CmpDecodeParams {
  const void* q;
  void* o;
  int* topk_idx;  // [Hkv, B, Tout] or nullptr
  const int* seqlens;
  const int* cmp_seqlens;
  long long q_sb, q_sh, o_sb, o_sh, t_sh, t_sb, t_sk;
  int B, Hq, Hkv, G;
  int window, stride, block_size, topk_out, init_blocks, local_blocks;
  int lc_pad, nb_pad;
  float scale2;
  Status st;
};

template <typename T, int D>
__global__ void __launch_bounds__(128, 1)
cmp_decode_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, CmpDecodeParams p) {
  constexpr int WARPS = 4;
  constexpr int TILE_BYTES = kKeyTile * D * 2;
  constexpr int PANELS = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* kbuf = smem + warp * 2 * TILE_BYTES;
  uint8_t* vbuf = kbuf + TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + WARPS * 2 * TILE_BYTES);
  uint64_t* barK = bars + 2 * warp;
  uint64_t* barV = barK + 1;
  float* lse_sh = reinterpret_cast<float*>(bars + 2 * WARPS);  // [16]
  float* ml_sh = lse_sh + 16;                                  // [WARPS][16][2]
  float* keysc = ml_sh + WARPS * 32;                           // [lc_pad]
  float* bsc = keysc + p.lc_pad;                               // [nb_pad]
  float* osum = reinterpret_cast<float*>(smem);                // [WARPS][16][D] overlays the tile buffers after pass 1

  const int b = blockIdx.x, h = blockIdx.y;
  const int len = __ldg(p.seqlens + b);
  const int Lc = __ldg(p.cmp_seqlens + b);
  const int ntiles = (Lc + kKeyTile - 1) / kKeyTile;
  if (lane == 0) {
    mbar_init(barK, 1);
    mbar_init(barV, 1);
    fence_barrier_init();
  }
  __syncthreads();

  const int my_tiles = (ntiles > warp) ? (ntiles - warp + WARPS - 1) / WARPS : 0;
  auto issue = [&](bool is_v, int kpos) {
    uint8_t* buf = is_v ? vbuf : kbuf;
    uint64_t* bar = is_v ? barV : barK;
    const CUtensorMap* tm = is_v ? &tmV : &tmK;
    mbar_expect_tx(bar, TILE_BYTES);
#pragma unroll
    for (int pn = 0; pn < PANELS; ++pn) tma_load_4d(buf + pn * (kKeyTile * 128), tm, bar, pn * 64, h, kpos, b);
  };
  auto tile_at = [&](int i, int& kpos, int& limv) {
    kpos = (warp + i * WARPS) * kKeyTile;
    limv = min(kKeyTile, Lc - kpos);
  };
  const T* qbase = static_cast<const T*>(p.q) + (long long)b * p.q_sb + (long long)h * p.G * p.q_sh;
  uint32_t qf[D / 16][4];
  load_a_frags_global<T, D / 16>(qf, [&](int r) -> const T* { return r < p.G ? qbase + r * p.q_sh : nullptr; });
  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  uint32_t phase = 0;
  warp_attend_tiles<T, D>(qf, o, m, l, my_tiles, smem_u32(kbuf), smem_u32(vbuf), barK, barV, phase, p.scale2, p.st, tile_at,
                          issue);

  // ---- combine the warps' partial results ----
  const int r0 = lane >> 2, c0 = (lane & 3) * 2;
  if ((lane & 3) == 0) {
    ml_sh[(warp * 16 + r0) * 2] = m[0];
    ml_sh[(warp * 16 + r0) * 2 + 1] = l[0];
    ml_sh[(warp * 16 + r0 + 8) * 2] = m[1];
    ml_sh[(warp * 16 + r0 + 8) * 2 + 1] = l[1];
  }
  __syncthreads();  // all tile reads done: the tile buffers may be overlaid
  float mstar[2], den[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r0 + 8 * r;
    mstar[r] = -INFINITY;
    for (int w = 0; w < WARPS; ++w) mstar[r] = fmaxf(mstar[r], ml_sh[(w * 16 + row) * 2]);
    den[r] = 0.f;
    for (int w = 0; w < WARPS; ++w)
      den[r] += ml_sh[(w * 16 + row) * 2 + 1] * (mstar[r] == -INFINITY ? 0.f : fast_exp2(ml_sh[(w * 16 + row) * 2] - mstar[r]));
  }
  {
    const float w0 = (m[0] == -INFINITY) ? 0.f : fast_exp2(m[0] - mstar[0]);
    const float w1 = (m[1] == -INFINITY) ? 0.f : fast_exp2(m[1] - mstar[1]);
    float* dst = osum + (size_t)warp * 16 * D;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      *reinterpret_cast<float2*>(dst + r0 * D + j * 8 + c0) = make_float2(o[j][0] * w0, o[j][1] * w0);
      *reinterpret_cast<float2*>(dst + (r0 + 8) * D + j * 8 + c0) = make_float2(o[j][2] * w1, o[j][3] * w1);
    }
  }
  if (warp == 0 && (lane & 3) == 0) {
    lse_sh[r0] = den[0] > 0.f ? mstar[0] + log2f(den[0]) : INFINITY;       // +inf -> probabilities 0
    lse_sh[r0 + 8] = den[1] > 0.f ? mstar[1] + log2f(den[1]) : INFINITY;
  }
  __syncthreads();
  T* obase = static_cast<T*>(p.o) + (long long)b * p.o_sb + (long long)h * p.G * p.o_sh;
  for (int idx = threadIdx.x; idx < p.G * D; idx += blockDim.x) {
    const int g = idx / D, c = idx % D;
    float num = 0.f, dn = 0.f;
    for (int w = 0; w < WARPS; ++w) {
      num += osum[((size_t)w * 16 + g) * D + c];
      const float mw = ml_sh[(w * 16 + g) * 2];
      float ms = -INFINITY;
      for (int w2 = 0; w2 < WARPS; ++w2) ms = fmaxf(ms, ml_sh[(w2 * 16 + g) * 2]);
      dn += ml_sh[(w * 16 + g) * 2 + 1] * (mw == -INFINITY ? 0.f : fast_exp2(mw - ms));
    }
    obase[(long long)g * p.o_sh + c] = DT<T>::from_float(dn > 0.f ? num / dn : 0.f);
  }
  if (!p.topk_idx) return;
  fence_proxy_async();  // the tile buffers were overlaid with ordinary stores (osum): every warp orders its own accesses
  __syncthreads();      // before the barrier, so that all of them precede the TMA refills issued after it

  // ---- pass 2: key scores = sum over heads of exp2(s - lse) ----
  float lse2[2] = {lse_sh[r0], lse_sh[r0 + 8]};
  const bool rv0 = r0 < p.G, rv1 = (r0 + 8) < p.G;
  if (my_tiles > 0 && lane == 0) issue(false, warp * kKeyTile);
  for (int i = 0; i < my_tiles; ++i) {
    const int kpos = (warp + i * WARPS) * kKeyTile;
    mbar_wait(barK, phase, p.st);
    float sc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
    mma_nk<T, 8, D / 16, kKeyTile>(sc, qf, smem_u32(kbuf), 0, 0);
    __syncwarp();
    if (i + 1 < my_tiles && lane == 0) issue(false, kpos + WARPS * kKeyTile);
    phase ^= 1;
    const int limv = Lc - kpos;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int col = j * 8 + c0 + e;
        float v = 0.f;
        if (col < limv) {
          if (rv0) v += fast_exp2(sc[j][e] * p.scale2 - lse2[0]);
          if (rv1) v += fast_exp2(sc[j][e + 2] * p.scale2 - lse2[1]);
        }
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        if (lane < 4 && kpos + col < p.lc_pad) keysc[kpos + col] = v;
      }
    }
  }
  __syncthreads();
  // ---- block scores and selection ----
  const int a = p.window / p.stride, c = p.block_size / p.stride;
  const int bq = (len - 1) / p.block_size;
  for (int bb = threadIdx.x; bb <= bq && bb < p.nb_pad; bb += blockDim.x) {
    float acc = 0.f;
    for (int o2 = 0; o2 <= a + c - 2; ++o2) {
      const int key = bb * c - (a - 1) + o2;
      if (key >= 0 && key < Lc) acc += (float)fold_weight(o2, a, c) * keysc[key];
    }
    bsc[bb] = acc;
  }
  __syncthreads();
  if (warp == 0)
    warp_select_topk(bsc, min(bq, p.nb_pad - 1), p.topk_out, p.init_blocks, p.local_blocks,
                     p.topk_idx + h * p.t_sh + (long long)b * p.t_sb, p.t_sk);
}

template <typename T, int D>
static int launch_cmp_decode(const void* k, const void* v, const long long* kv_strides, int cache_len, CmpDecodeParams p,
                             cudaStream_t stream) {
  constexpr int WARPS = 4;
  constexpr int TILE_BYTES = kKeyTile * D * 2;
  CUtensorMap tmK, tmV;
  int rc = make_tmap_4d(&tmK, DT<T>::kTmapType, k, D, p.Hkv, cache_len, p.B, kv_strides[2], kv_strides[1], kv_strides[0], 64,
                        kKeyTile);
  if (rc) return rc;
  rc = make_tmap_4d(&tmV, DT<T>::kTmapType, v, D, p.Hkv, cache_len, p.B, kv_strides[5], kv_strides[4], kv_strides[3], 64,
                    kKeyTile);
  if (rc) return rc;
  const size_t smem = 1024 + WARPS * 2 * TILE_BYTES + WARPS * 2 * sizeof(uint64_t) + (16 + WARPS * 32) * sizeof(float) +
                      (size_t)(p.lc_pad + p.nb_pad) * sizeof(float);
  if (smem > 220 * 1024) return kUnsupported;
  auto kern = cmp_decode_kernel<T, D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_rc(e);
  { LaunchScope ls_("cmp_decode", stream); kern<<<dim3(p.B, p.Hkv), WARPS * 32, smem, stream>>>(tmK, tmV, p); }
  return cuda_rc(cudaGetLastError());
}

static int decode_common_checks(const void* q, const void* k, const void* v, const void* o, const long long* strides,
                                int batch, int cache_len, int num_q_heads, int num_kv_heads) {
  if (!q || !k || !v || !o || !strides) return kInvalid;
  if (batch <= 0 || cache_len <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads) return kInvalid;
  if (num_q_heads / num_kv_heads > 16) return kUnsupported;
  for (int i = 0; i < 10; ++i)
    if (strides[i] % 8) return kInvalid;
  if (!aligned16(q) || !aligned16(o)) return kInvalid;
  return kOk;
}

}  // namespace nsa

extern "C" int nsa_decode_num_splits(int batch, int num_kv_heads, int max_tiles) {
  // aim at ~6 warps on each of the 148 SMs, never more splits than tiles
  const int pairs = batch * num_kv_heads;
  if (pairs <= 0 || max_tiles <= 1) return 1;
  int s = (148 * 6 + pairs - 1) / pairs;
  if (s > max_tiles) s = max_tiles;
  if (s > nsa::kMaxDecodeSplits) s = nsa::kMaxDecodeSplits;
  return s < 1 ? 1 : s;
}

// strides: q_b q_h | k_b k_n k_h | v_b v_n v_h | o_b o_h | idx_h idx_b idx_k   (13 entries, elements)
extern "C" int nsa_flash_attn_decode(const void* q, const void* k, const void* v, const int* seqlens, void* o,
                                     float* scratch, long long scratch_floats, int num_splits, int batch, int cache_len,
                                     int num_q_heads, int num_kv_heads, int head_dim, const long long* strides,
                                     float sm_scale, int dtype, void* stream) {
  using namespace nsa;
  if (!seqlens) return kInvalid;
  // reorder for the shared check: q_b q_h k_b k_n k_h v_b v_n v_h o_b o_h
  int rc = decode_common_checks(q, k, v, o, strides, batch, cache_len, num_q_heads, num_kv_heads);
  if (rc) return rc;
  DecodeParams p;
  p.q = q; p.o = o; p.seqlens = seqlens; p.topk_idx = nullptr;
  p.q_sb = strides[0]; p.q_sh = strides[1]; p.o_sb = strides[8]; p.o_sh = strides[9];
  p.t_sh = p.t_sb = p.t_sk = 0;
  p.B = batch; p.Hq = num_q_heads; p.Hkv = num_kv_heads; p.G = num_q_heads / num_kv_heads; p.T = 0; p.block_size = kKeyTile;
  const int max_tiles = (cache_len + kKeyTile - 1) / kKeyTile;
  p.S = num_splits < 1 ? 1 : (num_splits > max_tiles ? max_tiles : num_splits);
  if (p.S > kMaxDecodeSplits) p.S = kMaxDecodeSplits;
  p.tiles_per_split = (max_tiles + p.S - 1) / p.S;
  const long long need = p.S > 1 ? (long long)batch * num_kv_heads * p.S * 16 * (head_dim + 2) : 0;
  if (need > 0 && (!scratch || scratch_floats < need)) return kWorkspace;
  p.part_o = scratch;
  p.part_ml = scratch ? scratch + (size_t)batch * num_kv_heads * p.S * 16 * head_dim : nullptr;
  p.scale2 = sm_scale * kLog2e;
  p.st.word = status_word();
  const long long kvs[6] = {strides[2], strides[3], strides[4], strides[5], strides[6], strides[7]};
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_decode, k, v, kvs, cache_len, p, static_cast<cudaStream_t>(stream));
}

extern "C" int nsa_topk_sparse_attn_decode(const void* q, const void* k, const void* v, const int* topk_idx,
                                           const int* seqlens, void* o, float* scratch, long long scratch_floats,
                                           int num_splits, int batch, int cache_len, int num_q_heads, int num_kv_heads,
                                           int head_dim, int topk, int block_size, const long long* strides,
                                           float sm_scale, int dtype, void* stream) {
  using namespace nsa;
  if (!seqlens || !topk_idx) return kInvalid;
  int rc = decode_common_checks(q, k, v, o, strides, batch, cache_len, num_q_heads, num_kv_heads);
  if (rc) return rc;
  if (block_size < kKeyTile || block_size % kKeyTile) return kUnsupported;
  if (topk <= 0 || (long long)topk * (block_size / kKeyTile) > kMaxTilesPerDecodeQuery) return kUnsupported;
  DecodeParams p;
  p.q = q; p.o = o; p.seqlens = seqlens; p.topk_idx = topk_idx;
  p.q_sb = strides[0]; p.q_sh = strides[1]; p.o_sb = strides[8]; p.o_sh = strides[9];
  p.t_sh = strides[10]; p.t_sb = strides[11]; p.t_sk = strides[12];
  p.B = batch; p.Hq = num_q_heads; p.Hkv = num_kv_heads; p.G = num_q_heads / num_kv_heads; p.T = topk; p.block_size = block_size;
  const int max_tiles = topk * (block_size / kKeyTile);
  p.S = num_splits < 1 ? 1 : (num_splits > max_tiles ? max_tiles : num_splits);
  if (p.S > kMaxDecodeSplits) p.S = kMaxDecodeSplits;
  p.tiles_per_split = (max_tiles + p.S - 1) / p.S;
  const long long need = p.S > 1 ? (long long)batch * num_kv_heads * p.S * 16 * (head_dim + 2) : 0;
  if (need > 0 && (!scratch || scratch_floats < need)) return kWorkspace;
  p.part_o = scratch;
  p.part_ml = scratch ? scratch + (size_t)batch * num_kv_heads * p.S * 16 * head_dim : nullptr;
  p.scale2 = sm_scale * kLog2e;
  p.st.word = status_word();
  const long long kvs[6] = {strides[2], strides[3], strides[4], strides[5], strides[6], strides[7]};
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_decode, k, v, kvs, cache_len, p, static_cast<cudaStream_t>(stream));
}

extern "C" int nsa_compressed_attn_decode(const void* q, const void* k, const void* v, const int* seqlens,
                                          const int* compress_seqlens, void* o, int* topk_idx, int batch, int cache_len,
                                          int max_seqlen, int num_q_heads, int num_kv_heads, int head_dim,
                                          int kernel_size, int kernel_stride, int block_size, int topk, int init_blocks,
                                          int local_blocks, const long long* strides, float sm_scale, int dtype,
                                          void* stream) {
  using namespace nsa;
  if (!seqlens || !compress_seqlens) return kInvalid;
  int rc = decode_common_checks(q, k, v, o, strides, batch, cache_len, num_q_heads, num_kv_heads);
  if (rc) return rc;
  if (kernel_size % kernel_stride || block_size % kernel_stride || kernel_stride < 1) return kInvalid;
  if (topk_idx && (topk < 1 || topk < init_blocks + local_blocks || max_seqlen < 1)) return kInvalid;
  CmpDecodeParams p;
  p.q = q; p.o = o; p.topk_idx = topk_idx; p.seqlens = seqlens; p.cmp_seqlens = compress_seqlens;
  p.q_sb = strides[0]; p.q_sh = strides[1]; p.o_sb = strides[8]; p.o_sh = strides[9];
  p.t_sh = strides[10]; p.t_sb = strides[11]; p.t_sk = strides[12];
  p.B = batch; p.Hq = num_q_heads; p.Hkv = num_kv_heads; p.G = num_q_heads / num_kv_heads;
  p.window = kernel_size; p.stride = kernel_stride; p.block_size = block_size;
  const int max_blocks = topk_idx ? (max_seqlen + block_size - 1) / block_size : 1;
  p.topk_out = topk < max_blocks ? topk : max_blocks;
  p.init_blocks = init_blocks; p.local_blocks = local_blocks;
  p.lc_pad = ((cache_len + kKeyTile - 1) / kKeyTile) * kKeyTile;
  p.nb_pad = (max_blocks + 31) & ~31;
  p.scale2 = sm_scale * kLog2e;
  p.st.word = status_word();
  const long long kvs[6] = {strides[2], strides[3], strides[4], strides[5], strides[6], strides[7]};
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_cmp_decode, k, v, kvs, cache_len, p, static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------------------------------------
// Flash decode for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at all once they are running: a serving
// process that handed its whole memory budget to its own pool at start-up (any later allocation
// fails or fragments it), or a control loop that must not hit the implicit device synchronisation
// an allocation can cause.  The regular entry point makes such a caller provide the split-KV
// scratch; this variant keeps that scratch in the array below, which lives in the library's device
// image: every GPU that loads the library holds these 8 MiB until the process exits.
// ------------------------------------------------------------------------------------------------
namespace nsa {

constexpr long long kStaticScratchFloats = 2ll * 1024 * 1024;  // 8 MiB
static __device__ __align__(256) float g_decode_scratch[kStaticScratchFloats];

// Device address of g_decode_scratch on the current device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel can use; the address comes from cudaGetSymbolAddress,
// asked once per device with that device current.
static float* g_decode_scratch_ptr[64] = {};
static std::mutex g_decode_scratch_mutex;  // two host threads may make the first call on a device at the same time

static int static_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_rc(e);
  if (dev < 0 || dev >= 64) return kUnsupported;
  std::lock_guard<std::mutex> lock(g_decode_scratch_mutex);
  if (!g_decode_scratch_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_decode_scratch);
    if (e != cudaSuccess) return cuda_rc(e);
    g_decode_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_decode_scratch_ptr[dev];
  return kOk;
}

}  // namespace nsa

extern "C" long long nsa_flash_attn_decode_static_capacity(void) { return nsa::kStaticScratchFloats; }

extern "C" int nsa_flash_attn_decode_static(const void* q, const void* k, const void* v, const int* seqlens, void* o,
                                            int num_splits, int batch, int cache_len, int num_q_heads, int num_kv_heads,
                                            int head_dim, const long long* strides, float sm_scale, int dtype,
                                            void* stream) {
  using namespace nsa;
  if (batch <= 0 || cache_len <= 0 || num_kv_heads <= 0 || head_dim <= 0) return kInvalid;
  const int max_tiles = (cache_len + kKeyTile - 1) / kKeyTile;
  int splits = num_splits > 0 ? num_splits : nsa_decode_num_splits(batch, num_kv_heads, max_tiles);
  // the same clamps nsa_flash_attn_decode applies, so that the capacity check sees the split count that will run
  if (splits > max_tiles) splits = max_tiles;
  if (splits > kMaxDecodeSplits) splits = kMaxDecodeSplits;
  const long long per_split = (long long)batch * num_kv_heads * 16 * (head_dim + 2);
  if (num_splits <= 0)  // the library's own choice: take the largest split count whose partials fit (1 needs none)
    while (splits > 1 && per_split * splits > kStaticScratchFloats) --splits;
  const long long need = splits > 1 ? per_split * splits : 0;
  if (need > kStaticScratchFloats) return kWorkspace;  // an explicit split count that does not fit: ask for fewer
  float* scratch = nullptr;
  const int rc = static_scratch(&scratch);
  if (rc) return rc;
  // Every partial slot the combine step reads is written by this same call, so nothing has to be cleared.
  return nsa_flash_attn_decode(q, k, v, seqlens, o, scratch, kStaticScratchFloats, splits, batch, cache_len, num_q_heads,
                               num_kv_heads, head_dim, strides, sm_scale, dtype, stream);
}
