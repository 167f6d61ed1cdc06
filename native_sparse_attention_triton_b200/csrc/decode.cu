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
constexpr int kMaxDecodeSplits = 64;  // upper bound on the partial results combined per row
constexpr int kDecodeWarps = 6;       // warps (= concurrent tasks) per CTA; each owns one K and one V tile buffer

enum DecodeMode { kDecodeDense = 0, kDecodeSparse = 1, kDecodeCompressed = 2 };

struct DecodeParams {
  const void* q;
  void* o;
  const int* seqlens;      // dense / sparse: valid cache rows; compressed: sequence length including the current token
  const int* cmp_seqlens;  // compressed: valid compressed rows
  const int* topk_idx;     // sparse: selected blocks (input)
  int* topk_out_idx;       // compressed: selected blocks (output) or nullptr
  // scratch (caller memory): ctrl[0] = next task, ctrl[1 + b*Hkv + h] = splits of that pair finished so far
  int* ctrl;
  float* part_o;           // [pairs*S][16][D]
  float* part_ml;          // [pairs*S][16][2]
  float* logits;           // compressed: [pairs][16][lc_pad] scaled base-2 logits (-inf where masked)
  long long q_sb, q_sh, o_sb, o_sh;
  long long t_sh, t_sb, t_sk;
  int B, Hq, Hkv, G, T, block_size;
  int S, tiles_per_split, total_tasks;
  int window, stride, topk_out, init_blocks, local_blocks, lc_pad, nb_pad;
  float scale2;
  Status st;
};

__device__ __forceinline__ float4 ldcg4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }

// Split-KV single-token attention.  A TASK is (sequence, KV head, split): one warp streams the task's 64-key tiles through
// its own K and V buffers (TMA), the G query heads of the KV head being the rows of the mma tile.  Tasks are handed out
// dynamically (an atomic counter in the caller's scratch) so that ragged batches and task counts that are not a multiple
// of the machine still finish together; with no scratch (one split, nothing to combine) task = global warp index.
// The counters are incremented with wrap-around (atomicInc) so that a completed launch leaves every one of them at zero:
// the scratch has to be zero in its control words once, before its first use, and never again.
// A pair whose keys were split ends in the warp that finishes its LAST split (a per-pair counter): it merges the partial
// (max, sum, output) triples and writes the output, so there is no second launch.  In compressed mode the tasks also store
// the scaled logits; the finishing warp turns them into block scores (probabilities summed over the G heads, folded over
// the compression windows a block overlaps) and selects the top-k blocks.
template <typename T, int D, int MODE>
__global__ void __launch_bounds__(kDecodeWarps * 32, 1)
decode_attn_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, DecodeParams p) {
  constexpr int WARPS = kDecodeWarps;
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
  if (lane == 0) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tmK)) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&tmV)) : "memory");
    mbar_init(barK, 1);
    mbar_init(barV, 1);
    fence_barrier_init();
  }
  __syncwarp();
  uint32_t phase = 0;
  const int r0 = lane >> 2, c0 = (lane & 3) * 2;

  // tasks are fetched from the counter only when there are more of them than warps in the grid
  const bool dynamic = p.ctrl != nullptr && p.total_tasks > (int)gridDim.x * WARPS;
  for (int round = 0;; ++round) {
    int task;
    if (dynamic) {
      task = 0;
      // wraps to 0 after the last fetch of the launch (every task once, plus the one fetch that tells each warp to stop)
      if (lane == 0) task = (int)atomicInc(reinterpret_cast<unsigned*>(p.ctrl), (unsigned)(p.total_tasks + gridDim.x * WARPS - 1));
      task = __shfl_sync(0xffffffffu, task, 0);
    } else {
      task = blockIdx.x * WARPS + warp;
      if (round > 0) break;
    }
    if (task >= p.total_tasks) break;
    const int split = task % p.S;
    const int pair = task / p.S;
    const int h = pair % p.Hkv;
    const int b = pair / p.Hkv;

    // ---- the pair's tiles and this split's share ----
    const int len = __ldg(p.seqlens + b);
    int ntiles, rows;  // rows: valid cache rows of this pair
    if constexpr (MODE == kDecodeSparse) {
      const int BS = p.block_size, nsub = BS / kKeyTile;
      const int bq = len > 0 ? (len - 1) / BS : -1;
      rows = len;
      ntiles = 0;
      const int* tptr = p.topk_idx + h * p.t_sh + (long long)b * p.t_sb;
      __syncwarp();
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
    } else {
      rows = (MODE == kDecodeCompressed) ? __ldg(p.cmp_seqlens + b) : len;
      ntiles = (rows + kKeyTile - 1) / kKeyTile;
    }
    const int s_eff = max(1, min(p.S, (ntiles + p.tiles_per_split - 1) / p.tiles_per_split));  // splits of this pair that have tiles
    if (split >= s_eff) continue;
    const int t_begin = min(ntiles, split * p.tiles_per_split);
    const int t_end = min(ntiles, t_begin + p.tiles_per_split);

    auto issue = [&](bool is_v, int kpos) {
      uint8_t* buf = is_v ? vbuf : kbuf;
      uint64_t* bar = is_v ? barV : barK;
      const CUtensorMap* tm = is_v ? &tmV : &tmK;
      mbar_expect_tx(bar, TILE_BYTES);
#pragma unroll
      for (int pn = 0; pn < PANELS; ++pn) tma_load_4d(buf + pn * (kKeyTile * 128), tm, bar, pn * 64, h, kpos, b);
    };
    auto tile_at = [&](int i, int& kpos, int& limv) {
      kpos = (MODE == kDecodeSparse) ? tiles[t_begin + i] : (t_begin + i) * kKeyTile;
      limv = min(kKeyTile, rows - kpos);
    };
    float* lrow = (MODE == kDecodeCompressed) ? p.logits + (size_t)pair * 16 * p.lc_pad : nullptr;
    auto on_scores = [&](int kpos, int limv, const float (&sc)[8][4]) {
      if constexpr (MODE == kDecodeCompressed) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int col = j * 8 + c0;
          const float a0 = col < limv ? sc[j][0] * p.scale2 : -INFINITY, a1 = col + 1 < limv ? sc[j][1] * p.scale2 : -INFINITY;
          const float b0 = col < limv ? sc[j][2] * p.scale2 : -INFINITY, b1 = col + 1 < limv ? sc[j][3] * p.scale2 : -INFINITY;
          if (r0 < p.G) *reinterpret_cast<float2*>(lrow + (size_t)r0 * p.lc_pad + kpos + col) = make_float2(a0, a1);
          if (r0 + 8 < p.G) *reinterpret_cast<float2*>(lrow + (size_t)(r0 + 8) * p.lc_pad + kpos + col) = make_float2(b0, b1);
        }
      }
    };

    // the first tile is requested before anything else is fetched: the query rows arrive under its latency
    if (t_end > t_begin && lane == 0) {
      int kpos0, lim0;
      tile_at(0, kpos0, lim0);
      issue(false, kpos0);
      issue(true, kpos0);
    }
    const T* qbase = static_cast<const T*>(p.q) + (long long)b * p.q_sb + (long long)h * p.G * p.q_sh;
    uint32_t qf[D / 16][4];
    load_a_frags_global<T, D / 16>(qf, [&](int r) -> const T* { return r < p.G ? qbase + r * p.q_sh : nullptr; });
    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    warp_attend_tiles<T, D>(qf, o, m, l, t_end - t_begin, smem_u32(kbuf), smem_u32(vbuf), barK, barV, phase, p.scale2, p.st,
                            tile_at, issue, on_scores, true);

    T* obase = static_cast<T*>(p.o) + (long long)b * p.o_sb + (long long)h * p.G * p.o_sh;
    float lse_r[2];  // base-2 log-sum-exp of rows r0, r0 + 8 (compressed mode), +inf for rows without a key
    bool finisher = true;
    if (s_eff == 1) {
      float rs[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        rs[r] = l[r] > 0.f ? 1.f / l[r] : 0.f;
        lse_r[r] = l[r] > 0.f ? m[r] + log2f(l[r]) : INFINITY;
      }
      store_rows_staged<T, D>(o, rs, reinterpret_cast<T*>(kbuf), [&](int r) -> T* { return r < p.G ? obase + r * p.o_sh : nullptr; });
    } else {
      float* po = p.part_o + (size_t)task * 16 * D;
      float* pml = p.part_ml + (size_t)task * 16 * 2;
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        *reinterpret_cast<float2*>(po + r0 * D + j * 8 + c0) = make_float2(o[j][0], o[j][1]);
        *reinterpret_cast<float2*>(po + (r0 + 8) * D + j * 8 + c0) = make_float2(o[j][2], o[j][3]);
      }
      if ((lane & 3) == 0) {
        *reinterpret_cast<float2*>(pml + r0 * 2) = make_float2(m[0], l[0]);
        *reinterpret_cast<float2*>(pml + (r0 + 8) * 2) = make_float2(m[1], l[1]);
      }
      __threadfence();  // the partial result is visible device-wide before this split is counted
      __syncwarp();
      int done = 0;
      if (lane == 0) done = (int)atomicInc(reinterpret_cast<unsigned*>(p.ctrl + 1 + pair), (unsigned)(s_eff - 1));  // wraps to 0 at the last split
      done = __shfl_sync(0xffffffffu, done, 0);
      finisher = done == s_eff - 1;
      if (finisher) {
        __threadfence();
        // ---- merge the pair's partial results (they sit in L2) ----
        // lanes 0..15 own one row each: running maximum, then the weight 2^(m_s - m*) of every split and the denominator;
        // the weights go to shared memory (this warp's K buffer is idle), the loads are batched four at a time
        const size_t first = (size_t)pair * p.S;
        float* wbuf = reinterpret_cast<float*>(kbuf);  // [s_eff][16] weights, then [16] 1/denominator
        float my_lse = INFINITY;
        if (lane < 16) {
          // one round trip: every split's (max, sum) of this row goes to shared memory first, eight loads at a time
          const float* mlp = p.part_ml + (first * 16 + lane) * 2;
          float2* mls = reinterpret_cast<float2*>(vbuf) + lane;  // [s_eff][16] in the (idle) V buffer
#pragma unroll 8
          for (int s2 = 0; s2 < s_eff; ++s2) mls[s2 * 16] = __ldcg(reinterpret_cast<const float2*>(mlp + (size_t)s2 * 32));
          float mstar = -INFINITY;
          for (int s2 = 0; s2 < s_eff; ++s2) mstar = fmaxf(mstar, mls[s2 * 16].x);
          float den = 0.f;
          for (int s2 = 0; s2 < s_eff; ++s2) {
            const float2 ml = mls[s2 * 16];
            const float w = ml.x == -INFINITY ? 0.f : fast_exp2(ml.x - mstar);
            den += ml.y * w;
            wbuf[s2 * 16 + lane] = w;
          }
          wbuf[s_eff * 16 + lane] = den > 0.f ? 1.f / den : 0.f;
          my_lse = den > 0.f ? mstar + log2f(den) : INFINITY;
        }
        lse_r[0] = __shfl_sync(0xffffffffu, my_lse, r0);
        lse_r[1] = __shfl_sync(0xffffffffu, my_lse, r0 + 8);
        __syncwarp();
        // every lane owns D/32 columns of all rows: for each split, one independent load per row
        constexpr int CPL = D / 32;
        float acc[16][CPL];
#pragma unroll
        for (int g = 0; g < 16; ++g)
#pragma unroll
          for (int c = 0; c < CPL; ++c) acc[g][c] = 0.f;
        for (int s2 = 0; s2 < s_eff; ++s2) {
          const float* src = p.part_o + (first + s2) * 16 * D + lane * CPL;
#pragma unroll
          for (int g = 0; g < 16; ++g) {
            if (g < p.G) {
              const float w = wbuf[s2 * 16 + g];
              if constexpr (CPL == 4) {
                const float4 x = ldcg4(src + g * D);
                acc[g][0] += x.x * w; acc[g][1] += x.y * w; acc[g][2] += x.z * w; acc[g][3] += x.w * w;
              } else {
                const float2 x = __ldcg(reinterpret_cast<const float2*>(src + g * D));
                acc[g][0] += x.x * w; acc[g][1] += x.y * w;
              }
            }
          }
        }
#pragma unroll
        for (int g = 0; g < 16; ++g) {
          if (g < p.G) {
            const float inv = wbuf[s_eff * 16 + g];
            T* dst = obase + (long long)g * p.o_sh + lane * CPL;
            if constexpr (CPL == 4) {
              uint2 out;
              out.x = DT<T>::pack(acc[g][0] * inv, acc[g][1] * inv);
              out.y = DT<T>::pack(acc[g][2] * inv, acc[g][3] * inv);
              *reinterpret_cast<uint2*>(dst) = out;
            } else {
              *reinterpret_cast<uint32_t*>(dst) = DT<T>::pack(acc[g][0] * inv, acc[g][1] * inv);
            }
          }
        }
        __syncwarp();
      }
    }

    if constexpr (MODE == kDecodeCompressed) {
      if (finisher && p.topk_out_idx) {
        // ---- key scores -> block scores -> selection, by this warp, in its own (now idle) tile buffers ----
        __syncwarp();
        float* keysc = reinterpret_cast<float*>(kbuf);  // [lc_pad], then bsc [nb_pad]: fits the warp's 32 KB (checked by the host)
        float* bsc = keysc + p.lc_pad;
        // every lane needs the lse of all G rows: rows r0 / r0 + 8 live in lanes with (lane & 3) == 0
        float lse_all[16];
#pragma unroll
        for (int g = 0; g < 16; ++g) lse_all[g] = __shfl_sync(0xffffffffu, g < 8 ? lse_r[0] : lse_r[1], (g & 7) * 4);
        // four keys per lane and step: 4 x G independent loads (the logits sit in L2) before the first exponential
        for (int key0 = lane; key0 < rows; key0 += 128) {
          float x[4][16];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int key = key0 + 32 * u;
#pragma unroll
            for (int g = 0; g < 16; ++g) x[u][g] = (g < p.G && key < rows) ? __ldcg(lrow + (size_t)g * p.lc_pad + key) : -INFINITY;
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float v = 0.f;
#pragma unroll
            for (int g = 0; g < 16; ++g)
              if (g < p.G) v += fast_exp2(x[u][g] - lse_all[g]);
            if (key0 + 32 * u < rows) keysc[key0 + 32 * u] = v;
          }
        }
        __syncwarp();
        const int a = p.window / p.stride, c = p.block_size / p.stride;
        const int bq = (len - 1) / p.block_size;
        for (int bb = lane; bb <= bq && bb < p.nb_pad; bb += 32) {
          float acc = 0.f;
          for (int o2 = 0; o2 <= a + c - 2; ++o2) {
            const int key = bb * c - (a - 1) + o2;
            if (key >= 0 && key < rows) acc += (float)fold_weight(o2, a, c) * keysc[key];
          }
          bsc[bb] = acc;
        }
        __syncwarp();
        warp_select_topk(bsc, min(bq, p.nb_pad - 1), p.topk_out, p.init_blocks, p.local_blocks,
                         p.topk_out_idx + h * p.t_sh + (long long)b * p.t_sb, p.t_sk);
        __syncwarp();
      }
    }
    // the tile buffers were also written with ordinary stores (output staging, selection scratch): order them before
    // the TMA refills of the next task
    fence_proxy_async();
    __syncwarp();
  }
}

static long long align64(long long x) { return (x + 63) / 64 * 64; }

// floats of caller scratch: control words, partial results of the splits, logits (compressed mode only)
static long long decode_scratch_floats(long long pairs, int S, int D, int lc_pad) {
  if (S <= 1 && lc_pad == 0) return 0;
  return align64(pairs + 1) + (S > 1 ? pairs * S * 16 * (D + 2) : 0) + pairs * 16 * lc_pad;
}

template <typename T, int D>
static int launch_decode(const void* k, const void* v, const long long* kv_strides, int cache_len, DecodeParams p, int mode,
                         float* scratch, cudaStream_t stream) {
  constexpr int WARPS = kDecodeWarps;
  constexpr int TILE_BYTES = kKeyTile * D * 2;
  CUtensorMap tmK, tmV;
  int rc = make_tmap_4d(&tmK, DT<T>::kTmapType, k, D, p.Hkv, cache_len, p.B, kv_strides[2], kv_strides[1], kv_strides[0], 64,
                        kKeyTile);
  if (rc) return rc;
  rc = make_tmap_4d(&tmV, DT<T>::kTmapType, v, D, p.Hkv, cache_len, p.B, kv_strides[5], kv_strides[4], kv_strides[3], 64,
                    kKeyTile);
  if (rc) return rc;
  const long long pairs = (long long)p.B * p.Hkv;
  p.total_tasks = (int)(pairs * p.S);
  p.ctrl = nullptr; p.part_o = p.part_ml = p.logits = nullptr;
  if (scratch) {
    p.ctrl = reinterpret_cast<int*>(scratch);
    float* f = scratch + align64(pairs + 1);
    if (p.S > 1) {
      p.part_o = f;
      p.part_ml = f + pairs * p.S * 16 * D;
      f += pairs * p.S * 16 * (D + 2);
    }
    if (mode == kDecodeCompressed) p.logits = f;
  }
  const size_t smem = 1024 + WARPS * 2 * TILE_BYTES + WARPS * 2 * sizeof(uint64_t) + WARPS * kMaxTilesPerDecodeQuery * sizeof(int);
  int sms = 148;
  {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int ctas_all = (p.total_tasks + WARPS - 1) / WARPS;
  const int grid = p.ctrl ? (ctas_all < sms ? ctas_all : sms) : ctas_all;  // persistent when tasks are handed out dynamically
  auto launch = [&](auto kern, const char* name) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_rc(e);
    LaunchScope ls_(name, stream);
    kern<<<grid, WARPS * 32, smem, stream>>>(tmK, tmV, p);
    return cuda_rc(cudaGetLastError());
  };
  switch (mode) {
    case kDecodeDense: return launch(decode_attn_kernel<T, D, kDecodeDense>, "decode_attn");
    case kDecodeSparse: return launch(decode_attn_kernel<T, D, kDecodeSparse>, "decode_attn_sparse");
    default: return launch(decode_attn_kernel<T, D, kDecodeCompressed>, "decode_attn_compressed");
  }
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
  const long long pairs = (long long)batch * num_kv_heads;
  if (pairs <= 0 || max_tiles <= 1) return 1;
  const long long slots = 148ll * nsa::kDecodeWarps;  // tasks that run at the same time
  long long s;
  if (pairs * max_tiles <= slots) {
    s = max_tiles;  // everything fits in one wave: one tile per task is the shortest chain of dependent loads
  } else {
    // about one task per slot (handed out dynamically), at least two tiles per task so that the partial results stay a
    // small fraction of the bytes read; measured on the 76-sequence case, more and shorter tasks only added their
    // fixed cost (index parsing, query fetch, partial write) to a kernel whose floor is the first access' latency
    s = (slots + pairs - 1) / pairs;
    if (s > max_tiles / 2) s = max_tiles / 2;
    // long rows are cut into tasks of at most 64 tiles even when there are more pairs than slots: with ragged lengths the
    // longest rows otherwise finish alone (1216 pairs of up to 128 tiles: 5.4 TB/s unsplit, 6.3 TB/s in two or more pieces)
    const long long by_length = (max_tiles + 63) / 64;
    if (s < by_length) s = by_length;
  }
  if (s > 32) s = 32;  // one warp merges a pair's partial results: keep that short
  return s < 1 ? 1 : (int)s;
}

extern "C" long long nsa_decode_scratch_floats(int batch, int num_kv_heads, int head_dim, int num_splits) {
  return nsa::decode_scratch_floats((long long)batch * num_kv_heads, num_splits, head_dim, 0);
}

extern "C" long long nsa_compressed_decode_scratch_floats(int batch, int num_kv_heads, int head_dim, int num_splits,
                                                          int cache_len) {
  const int lc_pad = ((cache_len + nsa::kKeyTile - 1) / nsa::kKeyTile) * nsa::kKeyTile;
  return nsa::decode_scratch_floats((long long)batch * num_kv_heads, num_splits, head_dim, lc_pad);
}

namespace nsa {
static void set_splits(DecodeParams& p, int num_splits, int max_tiles) {
  p.S = num_splits < 1 ? 1 : (num_splits > max_tiles ? max_tiles : num_splits);
  if (p.S > kMaxDecodeSplits) p.S = kMaxDecodeSplits;
  if (p.S < 1) p.S = 1;
  p.tiles_per_split = (max_tiles + p.S - 1) / p.S;
}
}  // namespace nsa

// strides: q_b q_h | k_b k_n k_h | v_b v_n v_h | o_b o_h | idx_h idx_b idx_k   (13 entries, elements)
extern "C" int nsa_flash_attn_decode(const void* q, const void* k, const void* v, const int* seqlens, void* o,
                                     float* scratch, long long scratch_floats, int num_splits, int batch, int cache_len,
                                     int num_q_heads, int num_kv_heads, int head_dim, const long long* strides,
                                     float sm_scale, int dtype, void* stream) {
  using namespace nsa;
  if (!seqlens) return kInvalid;
  int rc = decode_common_checks(q, k, v, o, strides, batch, cache_len, num_q_heads, num_kv_heads);
  if (rc) return rc;
  DecodeParams p{};
  p.q = q; p.o = o; p.seqlens = seqlens;
  p.q_sb = strides[0]; p.q_sh = strides[1]; p.o_sb = strides[8]; p.o_sh = strides[9];
  p.B = batch; p.Hq = num_q_heads; p.Hkv = num_kv_heads; p.G = num_q_heads / num_kv_heads; p.T = 0; p.block_size = kKeyTile;
  set_splits(p, num_splits, (cache_len + kKeyTile - 1) / kKeyTile);
  const long long need = decode_scratch_floats((long long)batch * num_kv_heads, p.S, head_dim, 0);
  if (need > 0 && (!scratch || scratch_floats < need)) return kWorkspace;
  p.scale2 = sm_scale * kLog2e;
  p.st.word = status_word();
  const long long kvs[6] = {strides[2], strides[3], strides[4], strides[5], strides[6], strides[7]};
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_decode, k, v, kvs, cache_len, p, kDecodeDense, need > 0 ? scratch : nullptr,
                          static_cast<cudaStream_t>(stream));
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
  DecodeParams p{};
  p.q = q; p.o = o; p.seqlens = seqlens; p.topk_idx = topk_idx;
  p.q_sb = strides[0]; p.q_sh = strides[1]; p.o_sb = strides[8]; p.o_sh = strides[9];
  p.t_sh = strides[10]; p.t_sb = strides[11]; p.t_sk = strides[12];
  p.B = batch; p.Hq = num_q_heads; p.Hkv = num_kv_heads; p.G = num_q_heads / num_kv_heads; p.T = topk; p.block_size = block_size;
  set_splits(p, num_splits, topk * (block_size / kKeyTile));
  const long long need = decode_scratch_floats((long long)batch * num_kv_heads, p.S, head_dim, 0);
  if (need > 0 && (!scratch || scratch_floats < need)) return kWorkspace;
  p.scale2 = sm_scale * kLog2e;
  p.st.word = status_word();
  const long long kvs[6] = {strides[2], strides[3], strides[4], strides[5], strides[6], strides[7]};
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_decode, k, v, kvs, cache_len, p, kDecodeSparse, need > 0 ? scratch : nullptr,
                          static_cast<cudaStream_t>(stream));
}

extern "C" int nsa_compressed_attn_decode(const void* q, const void* k, const void* v, const int* seqlens,
                                          const int* compress_seqlens, void* o, int* topk_idx, float* scratch,
                                          long long scratch_floats, int num_splits, int batch, int cache_len, int max_seqlen,
                                          int num_q_heads, int num_kv_heads, int head_dim, int kernel_size, int kernel_stride,
                                          int block_size, int topk, int init_blocks, int local_blocks,
                                          const long long* strides, float sm_scale, int dtype, void* stream) {
  using namespace nsa;
  if (!seqlens || !compress_seqlens) return kInvalid;
  int rc = decode_common_checks(q, k, v, o, strides, batch, cache_len, num_q_heads, num_kv_heads);
  if (rc) return rc;
  if (kernel_size % kernel_stride || block_size % kernel_stride || kernel_stride < 1) return kInvalid;
  if (topk_idx && (topk < 1 || topk < init_blocks + local_blocks || max_seqlen < 1)) return kInvalid;
  DecodeParams p{};
  p.q = q; p.o = o; p.topk_out_idx = topk_idx; p.seqlens = seqlens; p.cmp_seqlens = compress_seqlens;
  p.q_sb = strides[0]; p.q_sh = strides[1]; p.o_sb = strides[8]; p.o_sh = strides[9];
  p.t_sh = strides[10]; p.t_sb = strides[11]; p.t_sk = strides[12];
  p.B = batch; p.Hq = num_q_heads; p.Hkv = num_kv_heads; p.G = num_q_heads / num_kv_heads; p.T = 0; p.block_size = block_size;
  p.window = kernel_size; p.stride = kernel_stride;
  const int max_blocks = topk_idx ? (max_seqlen + block_size - 1) / block_size : 1;
  p.topk_out = topk < max_blocks ? topk : max_blocks;
  p.init_blocks = init_blocks; p.local_blocks = local_blocks;
  p.lc_pad = ((cache_len + kKeyTile - 1) / kKeyTile) * kKeyTile;
  p.nb_pad = (max_blocks + 31) & ~31;
  // the warp that finishes a pair computes key scores and block scores in its own two tile buffers
  if ((long long)(p.lc_pad + p.nb_pad) * (long long)sizeof(float) > 2ll * kKeyTile * head_dim * 2) return kUnsupported;
  set_splits(p, num_splits, (cache_len + kKeyTile - 1) / kKeyTile);
  const long long need = decode_scratch_floats((long long)batch * num_kv_heads, p.S, head_dim, p.lc_pad);
  if (!scratch || scratch_floats < need) return kWorkspace;
  p.scale2 = sm_scale * kLog2e;
  p.st.word = status_word();
  const long long kvs[6] = {strides[2], strides[3], strides[4], strides[5], strides[6], strides[7]};
  return NSA_DISPATCH_T_D(dtype, head_dim, launch_decode, k, v, kvs, cache_len, p, kDecodeCompressed, scratch,
                          static_cast<cudaStream_t>(stream));
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
static long long g_decode_scratch_ctrl[64] = {};  // control words (ints) the previous call on the device counted in
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
  const long long pairs = (long long)batch * num_kv_heads;
  if (num_splits <= 0)  // the library's own choice: take the largest split count whose scratch fits (1 needs none)
    while (splits > 1 && decode_scratch_floats(pairs, splits, head_dim, 0) > kStaticScratchFloats) --splits;
  const long long need = decode_scratch_floats(pairs, splits, head_dim, 0);
  if (need > kStaticScratchFloats) return kWorkspace;  // an explicit split count that does not fit: ask for fewer
  float* scratch = nullptr;
  const int rc = static_scratch(&scratch);
  if (rc) return rc;
  if (need > 0) {
    // The control words at the front (one per (sequence, KV head) pair, plus one) are zero after every call, but what
    // lies behind them holds the previous call's partial results: a call with more pairs than the one before it clears
    // its longer control region first (a memset on `stream`; no allocation).
    int dev = 0;
    cudaGetDevice(&dev);
    const long long ctrl = align64(pairs + 1);
    std::lock_guard<std::mutex> lock(g_decode_scratch_mutex);
    if (ctrl > g_decode_scratch_ctrl[dev]) {
      cudaError_t e = cudaMemsetAsync(scratch, 0, (size_t)ctrl * sizeof(int), static_cast<cudaStream_t>(stream));
      if (e != cudaSuccess) return cuda_rc(e);
    }
    g_decode_scratch_ctrl[dev] = ctrl;
  }
  // The task and per-pair counters at the front of the array start at zero (the array is zero-initialised when the library
  // is loaded) and every completed call leaves them at zero; every partial slot that is read is written by this same call.
  return nsa_flash_attn_decode(q, k, v, seqlens, o, scratch, kStaticScratchFloats, splits, batch, cache_len, num_q_heads,
                               num_kv_heads, head_dim, strides, sm_scale, dtype, stream);
}
